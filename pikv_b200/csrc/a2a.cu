// Expert-sharded exchange helpers: quantise-and-pack routed K/V rows into fixed-size
// records ordered by destination rank, and store received records into the local paged
// cache.  The exchange itself (NCCL all-to-all over NVLink) runs between the two calls;
// both kernels only touch local memory.
//
// Record (int8 symmetric), 16-byte aligned:
//   int32 seq, int32 slot, 8 bytes pad | K codes [n_kv*128] | V codes [n_kv*128]
//   | K scales [n_kv] bf16 | V scales [n_kv] bf16 | pad to 16
#include "quant_group.cuh"

namespace pikv {

constexpr int PT = PIKV_PAGE_TOKENS;

__host__ __device__ inline size_t a2a_record_bytes(int n_kv) {
    size_t b = 16 + (size_t)2 * n_kv * 128 + (size_t)4 * n_kv;
    return (b + 15) / 16 * 16;
}

// one 8-lane group per (token, K|V, head); codes are written once per destination record
template <typename TIn>
__global__ void __launch_bounds__(256) a2a_pack_kernel(const TIn* k, const TIn* v, int T, int n_kv, int top_k,
                                                      const int* dst_seq, const int* slot, const int* seq_prefix,
                                                      const int* send_pos, uint8_t* send_buf) {
    const int sub = threadIdx.x & 7;
    const long long group = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;
    const int per_tok = 2 * n_kv;
    const bool active = group < (long long)T * per_tok;
    const int t = active ? (int)(group / per_tok) : 0;
    const int rr = active ? (int)(group % per_tok) : 0;
    const int which = rr / n_kv, head = rr % n_kv;
    QParams qp;
    uint32_t w[4];
    typename GroupQuant<TIn, 8, true>::Raw raw;
    GroupQuant<TIn, 8, true>::load((which ? v : k) + ((size_t)t * n_kv + head) * 128 + sub * 16, raw);
    GroupQuant<TIn, 8, true>::quant(raw, qp, w);
    if (!active) return;
    const size_t rec = a2a_record_bytes(n_kv);
    for (int j = 0; j < top_k; ++j) {
        const int sl = slot[(size_t)t * top_k + j];
        const int sp = send_pos ? send_pos[(size_t)t * top_k + j]
                                : (sl < 0 ? -1 : seq_prefix[dst_seq[(size_t)t * top_k + j]] + sl);
        if (sp < 0) continue;
        uint8_t* r = send_buf + (size_t)sp * rec;
        if (which == 0 && head == 0 && sub == 0) {
            reinterpret_cast<int*>(r)[0] = dst_seq[(size_t)t * top_k + j];
            reinterpret_cast<int*>(r)[1] = sl;
        }
        *reinterpret_cast<uint4*>(r + 16 + ((size_t)which * n_kv + head) * 128 + sub * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        if (sub == 0)
            reinterpret_cast<uint16_t*>(r + 16 + (size_t)2 * n_kv * 128)[which * n_kv + head] = f32_to_bf16_bits(qp.scale);
    }
}

__global__ void __launch_bounds__(256) a2a_unpack_kernel(const uint8_t* recv_buf, int n_records, int n_kv,
                                                        const int* page_table, int num_seqs, int max_pages,
                                                        int num_pages, int seq_offset, int capacity,
                                                        const int* seg_start, const int* seg_base, int n_seg,
                                                        uint8_t* k_codes, uint8_t* v_codes,
                                                        uint16_t* k_scale, uint16_t* v_scale, unsigned* status) {
    const int sub = threadIdx.x & 7;
    const long long group = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;
    const int per = 2 * n_kv;
    if (group >= (long long)n_records * per) return;
    const int i = (int)(group / per), rr = (int)(group % per);
    const int which = rr / n_kv, head = rr % n_kv;
    const size_t rec = a2a_record_bytes(n_kv);
    const uint8_t* r = recv_buf + (size_t)i * rec;
    const int seq = reinterpret_cast<const int*>(r)[0] - seq_offset;
    int s = reinterpret_cast<const int*>(r)[1];
    if (s < 0) return;
    if (seq < 0 || seq >= num_seqs) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_SEQ);
        return;
    }
    if (seg_start) {
        int sg = 0;
        while (sg + 1 < n_seg && i >= seg_start[sg + 1]) ++sg;
        s += seg_base[(size_t)sg * num_seqs + seq];
    }
    if (capacity > 0 && s >= capacity) return;
    if (s / PT >= max_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_SEQ);
        return;
    }
    const int page = page_table[(size_t)seq * max_pages + s / PT];
    if (page < 0 || page >= num_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_PAGE);
        return;
    }
    const int row = s % PT;
    const size_t prow = ((size_t)page * n_kv + head) * PT + row;
    const uint4 w = *reinterpret_cast<const uint4*>(r + 16 + ((size_t)which * n_kv + head) * 128 + sub * 16);
    uint8_t* dst = (which ? v_codes : k_codes) + prow * 128;
    *reinterpret_cast<uint4*>(dst + 16 * swz8_chunk(row, sub)) = w;
    if (sub == 0)
        (which ? v_scale : k_scale)[prow] = reinterpret_cast<const uint16_t*>(r + 16 + (size_t)2 * n_kv * 128)[which * n_kv + head];
}

}  // namespace pikv

using namespace pikv;

extern "C" size_t pikv_a2a_record_bytes(int32_t n_kv) { return n_kv > 0 ? a2a_record_bytes(n_kv) : 0; }

extern "C" int pikv_a2a_pack(const void* k, const void* v, int32_t dtype, int32_t T, int32_t n_kv, int32_t top_k,
                             const int32_t* dst_seq, const int32_t* slot, const int32_t* seq_prefix,
                             const int32_t* send_pos, void* send_buf, pikv_stream_t stream) {
    PIKV_REQUIRE(T >= 0 && n_kv > 0 && top_k > 0, PIKV_EINVAL, "a2a_pack: bad sizes");
    if (T == 0) return PIKV_OK;
    PIKV_REQUIRE(k && v && dst_seq && slot && send_buf, PIKV_EINVAL, "a2a_pack: null pointer");
    PIKV_REQUIRE(send_pos || seq_prefix, PIKV_EINVAL, "a2a_pack: give send_pos or seq_prefix");
    PIKV_REQUIRE(dtype == PIKV_BF16 || dtype == PIKV_F32, PIKV_EINVAL, "a2a_pack: bad dtype %d", dtype);
    const long long lanes = (long long)T * 2 * n_kv * 8;
    const int grid = (int)ceil_div64(lanes, 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == PIKV_BF16)
        a2a_pack_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k),
                                                             static_cast<const __nv_bfloat16*>(v), T, n_kv, top_k, dst_seq,
                                                             slot, seq_prefix, send_pos, static_cast<uint8_t*>(send_buf));
    else
        a2a_pack_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(v), T, n_kv,
                                                     top_k, dst_seq, slot, seq_prefix, send_pos, static_cast<uint8_t*>(send_buf));
    count_launch(1);
    return check_launch("a2a_pack_kernel");
}

extern "C" int pikv_a2a_unpack(const void* recv_buf, int32_t n_records, int32_t n_kv, const int32_t* page_table,
                               int32_t num_seqs, int32_t max_pages, int32_t num_pages, int32_t seq_offset,
                               int32_t capacity, const int32_t* seg_start, const int32_t* seg_base, int32_t n_seg,
                               void* k_codes, void* v_codes, void* k_scale, void* v_scale, uint32_t* status,
                               pikv_stream_t stream) {
    PIKV_REQUIRE(n_records >= 0 && n_kv > 0, PIKV_EINVAL, "a2a_unpack: bad sizes");
    if (n_records == 0) return PIKV_OK;
    PIKV_REQUIRE(recv_buf && page_table && k_codes && v_codes && k_scale && v_scale, PIKV_EINVAL, "a2a_unpack: null pointer");
    PIKV_REQUIRE((seg_start == nullptr) == (seg_base == nullptr) && (seg_start == nullptr || n_seg > 0), PIKV_EINVAL,
                 "a2a_unpack: seg_start and seg_base go together");
    const long long lanes = (long long)n_records * 2 * n_kv * 8;
    a2a_unpack_kernel<<<(int)ceil_div64(lanes, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(recv_buf), n_records, n_kv, page_table, num_seqs, max_pages, num_pages, seq_offset,
        capacity, seg_start, seg_base, n_seg, static_cast<uint8_t*>(k_codes), static_cast<uint8_t*>(v_codes), static_cast<uint16_t*>(k_scale),
        static_cast<uint16_t*>(v_scale), status);
    count_launch(1);
    return check_launch("a2a_unpack_kernel");
}
