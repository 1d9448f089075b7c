// Routed KV append fused with per-(token, head) quantisation, and the logical read-back.
//
// Work unit = one (token, K|V, head) group of 128 channels, handled by 8 lanes that each
// own 16 consecutive channels: two 16-byte loads of bf16 in, one 16-byte (int8) or 8-byte
// (int4) store of codes out per destination.  The 8 lanes of a group write one full
// 128-byte row of the destination page, so stores are whole lines even though the
// destinations are scattered.  The group statistics are a 3-step xor shuffle.
#include "common.cuh"

namespace pikv {

constexpr int APPEND_THREADS = 256;
constexpr int D = PIKV_HEAD_DIM;        // 128 channels per group
constexpr int PT = PIKV_PAGE_TOKENS;    // 16 tokens per page

struct AppendDev {
    const void* k;
    const void* v;
    int T, n_kv, top_k;
    const int* dst_seq;
    const int* slot;
    const int* page_table;
    int num_seqs, max_pages, num_pages;
    uint8_t* codes[2];
    uint16_t* scale[2];
    float* zp[2];
    unsigned* status;
};

template <typename TIn>
__device__ __forceinline__ void load16(const TIn* p, float (&x)[16]);
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[16]) {
    uint4 a = ld_stream_16(p);
    uint4 b = ld_stream_16(p + 8);
    bf16x2_to_f32(a.x, x[0], x[1]);   bf16x2_to_f32(a.y, x[2], x[3]);
    bf16x2_to_f32(a.z, x[4], x[5]);   bf16x2_to_f32(a.w, x[6], x[7]);
    bf16x2_to_f32(b.x, x[8], x[9]);   bf16x2_to_f32(b.y, x[10], x[11]);
    bf16x2_to_f32(b.z, x[12], x[13]); bf16x2_to_f32(b.w, x[14], x[15]);
}
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&x)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 a = ld_stream_16(p + 4 * i);
        x[4 * i + 0] = __uint_as_float(a.x); x[4 * i + 1] = __uint_as_float(a.y);
        x[4 * i + 2] = __uint_as_float(a.z); x[4 * i + 3] = __uint_as_float(a.w);
    }
}

template <typename TIn, int BITS, bool SYM>
__global__ void __launch_bounds__(APPEND_THREADS) kv_append_quant_kernel(AppendDev a) {
    constexpr int QMIN = SYM ? -(1 << (BITS - 1)) : 0;
    constexpr int QMAX = SYM ? (1 << (BITS - 1)) - 1 : (1 << BITS) - 1;
    constexpr int ROW_BYTES = D * BITS / 8;
    const int sub = threadIdx.x & 7;                       // lane within the group
    const long long group = ((long long)blockIdx.x * APPEND_THREADS + threadIdx.x) >> 3;
    const int per_tok = 2 * a.n_kv;
    const long long total = (long long)a.T * per_tok;
    const bool active = group < total;
    const int t = active ? (int)(group / per_tok) : 0;
    const int r = active ? (int)(group % per_tok) : 0;
    const int which = r / a.n_kv;                          // 0 = K, 1 = V
    const int head = r % a.n_kv;

    float x[16];
    if (active) {
        const TIn* src = static_cast<const TIn*>(which ? a.v : a.k) + ((size_t)t * a.n_kv + head) * D + sub * 16;
        load16<TIn>(src, x);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = 0.f;
    }
    float mn = x[0], mx = x[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (!active) return;
    const QParams qp = quant_params(mn, mx, QMIN, QMAX, SYM);
    const float inv = __frcp_rn(qp.scale);
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = (int)quant_code_fast(x[i], qp, inv, (float)QMIN, (float)QMAX);

    // pack
    uint32_t w[4];
    if (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = (uint32_t)(q[4 * i] & 0xff) | ((uint32_t)(q[4 * i + 1] & 0xff) << 8) |
                   ((uint32_t)(q[4 * i + 2] & 0xff) << 16) | ((uint32_t)(q[4 * i + 3] & 0xff) << 24);
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) v |= (uint32_t)(q[8 * i + j] & 0xf) << (4 * j);
            w[i] = v;
        }
    }
    const uint16_t scale_bits = f32_to_bf16_bits(qp.scale);

    for (int j = 0; j < a.top_k; ++j) {
        const int s = a.slot[(size_t)t * a.top_k + j];
        if (s < 0) continue;
        const int seq = a.dst_seq[(size_t)t * a.top_k + j];
        if (seq < 0 || seq >= a.num_seqs || (s / PT) >= a.max_pages) {
            if (a.status && sub == 0) atomicOr(a.status, PIKV_ST_BAD_SEQ);
            continue;
        }
        const int page = a.page_table[(size_t)seq * a.max_pages + s / PT];
        if (page < 0 || page >= a.num_pages) {
            if (a.status && sub == 0) atomicOr(a.status, PIKV_ST_BAD_PAGE);
            continue;
        }
        const int row = s % PT;
        const size_t prow = ((size_t)page * a.n_kv + head) * PT + row;
        uint8_t* dst = a.codes[which] + prow * ROW_BYTES;
        if (BITS == 8) {
            *reinterpret_cast<uint4*>(dst + 16 * swz8_chunk(row, sub)) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            *reinterpret_cast<uint2*>(dst + 8 * swz4_unit(row, sub)) = make_uint2(w[0], w[1]);
        }
        if (sub == 0) {
            a.scale[which][prow] = scale_bits;
            if (!SYM) a.zp[which][prow] = qp.zp;
        }
    }
}

// ---- logical read-back ----------------------------------------------------------------
// One 8-lane group per (row i, head): un-swizzle, unpack, dequantise with the stored
// bf16 scale / fp32 zero point.
__global__ void cache_gather_kernel(const int* seq, const int* pos, int n, const int* page_table, int num_seqs,
                                    int max_pages, int num_pages, int n_kv, int bits, const uint8_t* codes,
                                    const uint16_t* scale, const float* zp, float* out, int8_t* codes_out,
                                    unsigned* status) {
    const int sub = threadIdx.x & 7;
    const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    if (group >= (long long)n * n_kv) return;
    const int i = (int)(group / n_kv), head = (int)(group % n_kv);
    const int s = seq[i], p = pos[i];
    if (s < 0 || s >= num_seqs || p < 0 || p / PT >= max_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_SEQ);
        return;
    }
    const int page = page_table[(size_t)s * max_pages + p / PT];
    if (page < 0 || page >= num_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_PAGE);
        return;
    }
    const int row = p % PT;
    const size_t prow = ((size_t)page * n_kv + head) * PT + row;
    const float sc = bf16_bits_to_f32(scale[prow]);
    const float z = zp ? zp[prow] : 0.f;
    int q[16];
    if (bits == 8) {
        uint4 w = *reinterpret_cast<const uint4*>(codes + prow * D + 16 * swz8_chunk(row, sub));
        uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            int b = (ww[c >> 2] >> (8 * (c & 3))) & 0xff;
            q[c] = zp ? b : (int)(int8_t)b;
        }
    } else {
        uint2 w = *reinterpret_cast<const uint2*>(codes + prow * (D / 2) + 8 * swz4_unit(row, sub));
        uint32_t ww[2] = {w.x, w.y};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            int b = (ww[c >> 3] >> (4 * (c & 7))) & 0xf;
            q[c] = zp ? b : ((b ^ 8) - 8);
        }
    }
    const size_t o = ((size_t)i * n_kv + head) * D + sub * 16;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        if (out) out[o + c] = __fmul_rn(__fsub_rn((float)q[c], z), sc);
        if (codes_out) codes_out[o + c] = (int8_t)q[c];
    }
}

template <typename TIn>
static int launch_append(const AppendDev& a, int bits, int symmetric, cudaStream_t st) {
    const long long lanes = (long long)a.T * 2 * a.n_kv * 8;
    const int grid = (int)ceil_div64(lanes, APPEND_THREADS);
    if (bits == 8 && symmetric) kv_append_quant_kernel<TIn, 8, true><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (bits == 8) kv_append_quant_kernel<TIn, 8, false><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (symmetric) kv_append_quant_kernel<TIn, 4, true><<<grid, APPEND_THREADS, 0, st>>>(a);
    else kv_append_quant_kernel<TIn, 4, false><<<grid, APPEND_THREADS, 0, st>>>(a);
    count_launch(1);
    return check_launch("kv_append_quant_kernel");
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_kv_append_quant(const pikv_append_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "append: null params");
    PIKV_REQUIRE(p->T >= 0 && p->n_kv > 0 && p->top_k > 0, PIKV_EINVAL, "append: bad sizes");
    if (p->T == 0) return PIKV_OK;
    PIKV_REQUIRE(p->k && p->v && p->dst_seq && p->slot && p->page_table, PIKV_EINVAL, "append: null input pointer");
    PIKV_REQUIRE(p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL, "append: null cache pointer");
    PIKV_REQUIRE(p->bits == 8 || p->bits == 4, PIKV_EUNSUPPORTED, "append: bits=%d (8 or 4)", p->bits);
    PIKV_REQUIRE(p->symmetric || (p->k_zp && p->v_zp), PIKV_EINVAL, "append: asymmetric needs zero-point pools");
    PIKV_REQUIRE(p->dtype == PIKV_BF16 || p->dtype == PIKV_F32, PIKV_EINVAL, "append: bad dtype %d", p->dtype);
    PIKV_REQUIRE(p->num_seqs > 0 && p->max_pages > 0 && p->num_pages > 0, PIKV_EINVAL, "append: bad cache geometry");
    AppendDev a;
    a.k = p->k; a.v = p->v; a.T = p->T; a.n_kv = p->n_kv; a.top_k = p->top_k;
    a.dst_seq = p->dst_seq; a.slot = p->slot; a.page_table = p->page_table;
    a.num_seqs = p->num_seqs; a.max_pages = p->max_pages; a.num_pages = p->num_pages;
    a.codes[0] = static_cast<uint8_t*>(p->k_codes); a.codes[1] = static_cast<uint8_t*>(p->v_codes);
    a.scale[0] = static_cast<uint16_t*>(p->k_scale); a.scale[1] = static_cast<uint16_t*>(p->v_scale);
    a.zp[0] = static_cast<float*>(p->k_zp); a.zp[1] = static_cast<float*>(p->v_zp);
    a.status = p->status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->dtype == PIKV_BF16) return launch_append<__nv_bfloat16>(a, p->bits, p->symmetric, st);
    return launch_append<float>(a, p->bits, p->symmetric, st);
}

extern "C" int pikv_cache_gather(const int32_t* seq, const int32_t* pos, int32_t n, const int32_t* page_table,
                                 int32_t num_seqs, int32_t max_pages, int32_t num_pages, int32_t n_kv, int32_t bits,
                                 const void* codes, const void* scale, const void* zp, float* out, int8_t* codes_out,
                                 uint32_t* status, pikv_stream_t stream) {
    PIKV_REQUIRE(n >= 0 && n_kv > 0, PIKV_EINVAL, "cache_gather: bad sizes");
    if (n == 0) return PIKV_OK;
    PIKV_REQUIRE(seq && pos && page_table && codes && scale, PIKV_EINVAL, "cache_gather: null pointer");
    PIKV_REQUIRE(out || codes_out, PIKV_EINVAL, "cache_gather: no output given");
    PIKV_REQUIRE(bits == 8 || bits == 4, PIKV_EUNSUPPORTED, "cache_gather: bits=%d", bits);
    const long long lanes = (long long)n * n_kv * 8;
    cache_gather_kernel<<<(int)ceil_div64(lanes, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        seq, pos, n, page_table, num_seqs, max_pages, num_pages, n_kv, bits, static_cast<const uint8_t*>(codes),
        static_cast<const uint16_t*>(scale), static_cast<const float*>(zp), out, codes_out, status);
    count_launch(1);
    return check_launch("cache_gather_kernel");
}
