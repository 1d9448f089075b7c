// H2O scoring and eviction: score accumulate, segmented top-k select, page compaction.
//
// Select: one CTA per segment.  The segment's scores are staged once in shared memory as
// order-preserving 32-bit keys; the m-th largest key is found by an 8-bit radix select over
// the bits in which the segment's keys differ; elements above it are kept, and of the elements equal to it the ones with the
// lowest indices are kept until m are taken (an in-order ballot scan).  The same routine
// runs on the timestamps; both results are OR-ed into one keep bitmap from which the
// evict mask and the ascending kept-index list are written.
#include "common.cuh"

namespace pikv {

constexpr int SEL_THREADS = 1024;          // keys staged in shared memory: one CTA per SM
constexpr int SEL_THREADS_STREAM = 512;    // keys re-read from memory: small CTAs, several per SM
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_SMEM_KEYS = 49152;   // keys staged in shared memory up to this length

__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct SelShared {
    int hist[256];
    int warp_tot[SEL_WARPS];
    uint32_t warp_or[SEL_WARPS], warp_and[SEL_WARPS];
    int width;            // number of low key bits in which the segment's keys differ
    uint32_t prefix;      // key bits fixed so far
    int remaining;        // how many still to take among keys matching the prefix
    int eq_total;         // size of the bin chosen by the last pass (after the last digit: keys equal to the threshold)
    int cand_n;           // entries in the candidate list
    int total;
};

constexpr int SEL_CAND_CAP = 4096;     // candidate list (keys that matched the first digit), shared memory

// One pass of the radix select finished: warp 0 finds the bin holding the rem-th largest key among the
// keys that matched so far and narrows prefix / remaining; eq_total = size of that bin.
__device__ __forceinline__ void select_pick_bin(SelShared& sh, uint32_t prefix, int shift, int lane) {
    // lane handles bins [lane*8, lane*8+8); scan from the top bin down
    int local[8], sum = 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        local[b] = sh.hist[lane * 8 + b];
        sum += local[b];
    }
    // suffix sum over lanes: above = number of keys in bins owned by higher lanes
    int suffix = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_down_sync(0xffffffffu, suffix, o);
        if (lane + o < 32) suffix += v;
    }
    const int above = suffix - sum;
    const int rem = sh.remaining;
    // the target bin is the highest bin d with count(bins > d) < rem <= count(bins >= d)
    int cum = above;
    int found = -1, found_above = 0, found_cnt = 0;
#pragma unroll
    for (int b = 7; b >= 0; --b) {
        if (found < 0 && cum < rem && rem <= cum + local[b]) {
            found = lane * 8 + b;
            found_above = cum;
            found_cnt = local[b];
        }
        cum += local[b];
    }
    if (found >= 0) {
        sh.prefix = prefix | ((uint32_t)found << shift);
        sh.remaining = rem - found_above;
        sh.eq_total = found_cnt;
    }
}

// Marks in keepw (one bit per element) the m largest of src[0..n), ties to the lowest index.
// STAGED: the keys are copied to shared memory once and read from there; otherwise every scan reads the
// scores again (from L2 after the first one), which needs almost no shared memory and lets two CTAs share
// an SM.  Either way four keys are read at a time, and after the first digit only the keys of the chosen
// bin (a short list in shared memory) are looked at again.
template <bool STAGED, int NT>
__device__ void select_top_m(const float* __restrict__ src, int n, int m, uint32_t* keys, uint32_t* cand, uint32_t* keepw,
                             SelShared& sh) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (m <= 0) return;
    if (m >= n) {
        for (int w = tid; w < (n + 31) / 32; w += NT) {
            int rem = n - w * 32;
            keepw[w] |= rem >= 32 ? 0xffffffffu : ((1u << rem) - 1u);
        }
        __syncthreads();
        return;
    }
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    const float4* src4 = reinterpret_cast<const float4*>(src);
    const uint4* keys4 = reinterpret_cast<const uint4*>(keys);
    const int n4 = (STAGED || aligned) ? n / 4 : 0;          // whole groups of four keys
    auto global4 = [&](int i) {
        const float4 f = __ldg(src4 + i);
        return make_uint4(order_key(f.x), order_key(f.y), order_key(f.z), order_key(f.w));
    };
    auto key4 = [&](int i) { return STAGED ? keys4[i] : global4(i); };
    auto key1 = [&](int i) { return STAGED ? keys[i] : order_key(__ldg(src + i)); };
    // first scan: find the bits in which the keys differ at all (and stage them).  The scores of one segment
    // share their leading (sign / exponent) bits, and a radix digit taken from those would send most keys to
    // one or two bins.  The digits start at the first differing bit.
    uint32_t any = 0u, all = 0xffffffffu;
    if (aligned) {
        for (int i = tid; i < n / 4; i += NT) {
            const uint4 u = global4(i);
            if (STAGED) reinterpret_cast<uint4*>(keys)[i] = u;
            any |= u.x | u.y | u.z | u.w;
            all &= u.x & u.y & u.z & u.w;
        }
    }
    for (int i = (aligned ? 4 * (n / 4) : 0) + tid; i < n; i += NT) {
        const uint32_t u = order_key(src[i]);
        if (STAGED) keys[i] = u;
        any |= u;
        all &= u;
    }
    any = __reduce_or_sync(0xffffffffu, any);
    all = __reduce_and_sync(0xffffffffu, all);
    if (lane == 0) {
        sh.warp_or[warp] = any;
        sh.warp_and[warp] = all;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t o = 0u, a = 0xffffffffu;
        for (int w = 0; w < (NT / 32); ++w) {
            o |= sh.warp_or[w];
            a &= sh.warp_and[w];
        }
        const int width = 32 - __clz(o ^ a);                 // bits [width-1 .. 0] vary; 0: all keys equal
        sh.width = width;
        sh.prefix = width >= 32 ? 0u : (a & (0xffffffffu << width));
        sh.remaining = m;
        sh.eq_total = n;
        sh.cand_n = 0;
    }
    __syncthreads();
    // radix select over the varying bits, most significant digit first, 8 bits at a time
    bool use_list = false;
    int pass = 0;
    for (int top = sh.width; top > 0; ++pass) {
        const int bits = min(8, top);
        const int shift = top - bits;
        for (int i = tid; i < 256; i += NT) sh.hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        const uint32_t himask = top >= 32 ? 0u : (0xffffffffu << top);
        const uint32_t dmask = (1u << bits) - 1u;
        if (use_list) {
            const int cn = sh.cand_n;
            for (int i = tid; i < cn; i += NT) {
                const uint32_t u = cand[i];
                if ((u & himask) == prefix) atomicAdd(&sh.hist[(u >> shift) & dmask], 1);
            }
        } else {
            // second pass with a short chosen bin: the matching keys also go to the candidate list
            const bool fill = pass == 1 && sh.eq_total <= SEL_CAND_CAP;
            auto one = [&](uint32_t u) {
                if ((u & himask) == prefix) {
                    atomicAdd(&sh.hist[(u >> shift) & dmask], 1);
                    if (fill) cand[atomicAdd(&sh.cand_n, 1)] = u;
                }
            };
            for (int i = tid; i < n4; i += NT) {
                const uint4 u = key4(i);
                one(u.x); one(u.y); one(u.z); one(u.w);
            }
            for (int i = 4 * n4 + tid; i < n; i += NT) one(key1(i));
            use_list = fill;
        }
        __syncthreads();
        if (warp == 0) select_pick_bin(sh, prefix, shift, lane);
        __syncthreads();
        top = shift;
    }
    const uint32_t kth = sh.prefix;      // the m-th largest key
    const int need_eq = sh.remaining;    // how many keys equal to kth to keep (lowest indices)
    if (need_eq == sh.eq_total && (n4 == n / 4)) {
        // every key equal to the threshold is kept: one pass, four keys per thread, eight lanes per keep word
        const int n4r = (n + 3) / 4;
        for (int i0 = 0; i0 < n4r; i0 += NT) {
            const int i = i0 + tid;
            uint32_t nib = 0u;
            if (i < n4) {
                const uint4 u = key4(i);
                nib = (u.x >= kth ? 1u : 0u) | (u.y >= kth ? 2u : 0u) | (u.z >= kth ? 4u : 0u) | (u.w >= kth ? 8u : 0u);
            } else if (i < n4r) {
                for (int e = 0; e < 4; ++e)
                    if (4 * i + e < n && key1(4 * i + e) >= kth) nib |= 1u << e;
            }
            uint32_t word = nib << (4 * (lane & 7));
            word |= __shfl_xor_sync(0xffffffffu, word, 1);
            word |= __shfl_xor_sync(0xffffffffu, word, 2);
            word |= __shfl_xor_sync(0xffffffffu, word, 4);
            if ((lane & 7) == 0 && word && i < n4r) keepw[i >> 3] |= word;
        }
        __syncthreads();
        return;
    }
    // ties at the threshold of which only some are kept: in-order count of equal keys; warp w owns the
    // contiguous range [w*per, (w+1)*per)
    const int tiles = (n + 31) / 32;
    const int tiles_per = (tiles + (NT / 32) - 1) / (NT / 32);
    const int t0 = warp * tiles_per, t1 = min(tiles, t0 + tiles_per);
    int eq_cnt = 0;
    for (int t = t0; t < t1; ++t) {
        const int i = t * 32 + lane;
        uint32_t u = 0;
        bool in = i < n;
        if (in) u = key1(i);
        eq_cnt += __popc(__ballot_sync(0xffffffffu, in && u == kth));
    }
    if (lane == 0) sh.warp_tot[warp] = eq_cnt;
    __syncthreads();
    int eq_before = 0;
    for (int w = 0; w < warp; ++w) eq_before += sh.warp_tot[w];
    for (int t = t0; t < t1; ++t) {
        const int i = t * 32 + lane;
        uint32_t u = 0;
        bool in = i < n;
        if (in) u = key1(i);
        const bool gt = in && u > kth;
        const bool eq = in && u == kth;
        const unsigned eqb = __ballot_sync(0xffffffffu, eq);
        const int my_rank = eq_before + __popc(eqb & ((1u << lane) - 1u));
        const bool keep = gt || (eq && my_rank < need_eq);
        const unsigned kb = __ballot_sync(0xffffffffu, keep);
        if (lane == 0 && kb) keepw[t] |= kb;
        eq_before += __popc(eqb);
    }
    __syncthreads();
}

template <bool STAGED, int NT>
__global__ void __launch_bounds__(NT) h2o_select_kernel(const float* acc, const float* ts, int stride,
                                                                 const int* seg_len, int n_all, int num_heavy,
                                                                 int num_recent, uint8_t* evict_mask, int* keep_idx,
                                                                 int keep_stride, int* kept_count) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ SelShared sh;
    const int seg = blockIdx.x;
    int n = seg_len ? seg_len[seg] : n_all;
    n = max(0, min(n, stride));
    const int words_cap = (stride + 31) / 32;
    uint32_t* keepw = reinterpret_cast<uint32_t*>(smem_raw);
    // keys start on a 16-byte boundary (they are read four at a time); the candidate list follows them
    uint32_t* keys = keepw + ((words_cap + 3) & ~3);
    uint32_t* cand = keys + (STAGED ? ((stride + 3) & ~3) : 0);   // unstaged: the list follows the bitmap
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int w = tid; w < words_cap; w += NT) keepw[w] = 0u;
    __syncthreads();
    const float* a = acc + (size_t)seg * stride;
    const float* t = ts + (size_t)seg * stride;
    if (n > 0) {
        select_top_m<STAGED, NT>(a, n, min(num_heavy, n), keys, cand, keepw, sh);
        select_top_m<STAGED, NT>(t, n, min(num_recent, n), keys, cand, keepw, sh);
    }
    // outputs: evict mask bytes and ascending kept indices
    const int tiles = (stride + 31) / 32;
    const int tiles_per = (tiles + (NT / 32) - 1) / (NT / 32);
    const int t0 = warp * tiles_per, t1 = min(tiles, t0 + tiles_per);
    int cnt = 0;
    for (int tt = t0; tt < t1; ++tt) cnt += __popc(keepw[tt]);
    if (lane == 0) sh.warp_tot[warp] = cnt;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += sh.warp_tot[w];
    for (int tt = t0; tt < t1; ++tt) {
        const uint32_t kb = keepw[tt];
        const int i = tt * 32 + lane;
        const bool keep = (kb >> lane) & 1u;
        if (i < stride && evict_mask) evict_mask[(size_t)seg * stride + i] = keep ? 0 : 1;
        if (keep && keep_idx) {
            const int r = before + __popc(kb & ((1u << lane) - 1u));
            if (r < keep_stride) keep_idx[(size_t)seg * keep_stride + r] = i;
        }
        before += __popc(kb);
    }
    if (tid == 0 && kept_count) {
        int tot = 0;
        for (int w = 0; w < (NT / 32); ++w) tot += sh.warp_tot[w];
        kept_count[seg] = tot;
    }
}

__global__ void h2o_accumulate_kernel(float* acc, float* ts, int n, const int* idx, const float* w, int m, float now,
                                      unsigned* status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int j = idx ? idx[i] : i;
    if (j < 0 || j >= n) {
        if (status) atomicOr(status, PIKV_ST_BAD_INDEX);
        return;
    }
    acc[j] = __fadd_rn(acc[j], w[i]);
    ts[j] = now;
}
__global__ void h2o_decay_kernel(float* acc, int n, float decay) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] = __fmul_rn(acc[i], decay);
}

// ---- compaction ---------------------------------------------------------------------
struct CompactDev {
    pikv_compact_params p;
    int heads_per;   // heads moved per segment
};

__global__ void __launch_bounds__(256) h2o_compact_kernel(CompactDev c) {
    const pikv_compact_params& p = c.p;
    const int seg = blockIdx.x;
    const int sub = threadIdx.x & 7;
    const int item = (blockIdx.y * blockDim.x + threadIdx.x) >> 3;   // (row j, head slot)
    const int kept = min(p.kept_count[seg], p.keep_stride);
    const int j = item / c.heads_per, hs = item % c.heads_per;
    if (j >= kept) return;
    const int seq = p.per_head ? seg / p.n_kv : seg;
    const int head = p.per_head ? seg % p.n_kv : hs;
    const int spos = p.keep_idx[(size_t)seg * p.keep_stride + j];
    const int dpos = j;
    constexpr int PTK = PIKV_PAGE_TOKENS;
    if (seq >= p.num_seqs || spos < 0 || spos / PTK >= p.max_pages) {
        if (p.status && sub == 0) atomicOr(p.status, PIKV_ST_BAD_INDEX);
        return;
    }
    const int spage = p.src_page_table[(size_t)seq * p.max_pages + spos / PTK];
    const int dpage = p.dst_page_table[(size_t)seq * p.max_pages + dpos / PTK];
    if (spage < 0 || spage >= p.num_pages || dpage < 0 || dpage >= p.num_pages) {
        if (p.status && sub == 0) atomicOr(p.status, PIKV_ST_BAD_PAGE);
        return;
    }
    const int srow = spos % PTK, drow = dpos % PTK;
    const size_t sprow = ((size_t)spage * p.n_kv + head) * PTK + srow;
    const size_t dprow = ((size_t)dpage * p.n_kv + head) * PTK + drow;
    if (p.bits == 8) {
        const size_t so = sprow * 128 + 16 * swz8_chunk(srow, sub), dofs = dprow * 128 + 16 * swz8_chunk(drow, sub);
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.dst_k_codes) + dofs) =
            *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.src_k_codes) + so);
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.dst_v_codes) + dofs) =
            *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.src_v_codes) + so);
    } else {
        const size_t so = sprow * 64 + 8 * swz4_unit(srow, sub), dofs = dprow * 64 + 8 * swz4_unit(drow, sub);
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.dst_k_codes) + dofs) =
            *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.src_k_codes) + so);
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.dst_v_codes) + dofs) =
            *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.src_v_codes) + so);
    }
    if (sub == 0) {
        static_cast<uint16_t*>(p.dst_k_scale)[dprow] = static_cast<const uint16_t*>(p.src_k_scale)[sprow];
        static_cast<uint16_t*>(p.dst_v_scale)[dprow] = static_cast<const uint16_t*>(p.src_v_scale)[sprow];
        if (p.src_k_zp && p.dst_k_zp) {
            static_cast<float*>(p.dst_k_zp)[dprow] = static_cast<const float*>(p.src_k_zp)[sprow];
            static_cast<float*>(p.dst_v_zp)[dprow] = static_cast<const float*>(p.src_v_zp)[sprow];
        }
        if (hs == 0) {
            if (p.src_acc && p.dst_acc)
                p.dst_acc[(size_t)seg * p.score_stride + dpos] = p.src_acc[(size_t)seg * p.score_stride + spos];
            if (p.src_ts && p.dst_ts)
                p.dst_ts[(size_t)seg * p.score_stride + dpos] = p.src_ts[(size_t)seg * p.score_stride + spos];
        }
    }
}

// acc[b, kvh, pos] += sum over the group's query heads of exp(score - lse)
__global__ void h2o_accumulate_attn_kernel(const float* scores, int score_stride, const float* lse, const int* seq_len,
                                           int B, int n_q, int n_kv, float* acc, int acc_stride) {
    const int pos = blockIdx.x * blockDim.x + threadIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / n_kv, h = bh % n_kv;
    const int len = seq_len ? seq_len[b] : score_stride;
    if (pos >= len || pos >= acc_stride) return;
    const int g = n_q / n_kv;
    float s = 0.f;
    for (int i = 0; i < g; ++i) {
        const int qh = h * g + i;
        s += expf(scores[((size_t)b * n_q + qh) * score_stride + pos] - lse[(size_t)b * n_q + qh]);
    }
    acc[(size_t)bh * acc_stride + pos] += s;
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_h2o_accumulate(float* acc, float* ts, int32_t n, const int32_t* idx, const float* w, int32_t m,
                                   float now, float decay, uint32_t* status, pikv_stream_t stream) {
    PIKV_REQUIRE(acc && ts && w, PIKV_EINVAL, "h2o_accumulate: null pointer");
    PIKV_REQUIRE(n > 0 && m >= 0 && (idx != nullptr || m <= n), PIKV_EINVAL, "h2o_accumulate: bad sizes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int launches = 0;
    if (decay != 1.0f) {
        h2o_decay_kernel<<<ceil_div(n, 256), 256, 0, st>>>(acc, n, decay);
        ++launches;
    }
    if (m > 0) {
        h2o_accumulate_kernel<<<ceil_div(m, 256), 256, 0, st>>>(acc, ts, n, idx, w, m, now, status);
        ++launches;
    }
    count_launch(launches);
    return check_launch("h2o_accumulate");
}

extern "C" int pikv_h2o_select(const float* acc, const float* ts, int32_t segments, int32_t stride,
                               const int32_t* seg_len, int32_t n, int32_t num_heavy, int32_t num_recent,
                               uint8_t* evict_mask, int32_t* keep_idx, int32_t keep_stride, int32_t* kept_count,
                               pikv_stream_t stream) {
    PIKV_REQUIRE(acc && ts, PIKV_EINVAL, "h2o_select: null scores");
    PIKV_REQUIRE(segments > 0 && stride > 0 && n >= 0 && n <= stride, PIKV_EINVAL, "h2o_select: bad sizes");
    PIKV_REQUIRE(num_heavy >= 0 && num_recent >= 0, PIKV_EINVAL, "h2o_select: negative counts");
    PIKV_REQUIRE(keep_idx == nullptr || keep_stride > 0, PIKV_EINVAL, "h2o_select: keep_stride");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t words = (size_t)(stride + 31) / 32 * 4;
    // keys staged in shared memory whenever the segment fits (183 us against 191 us for 512 segments of 32768
    // with the re-reading variant, which serves longer segments); PIKV_H2O_STAGED=0 forces the latter (testing aid)
    const char* force = getenv("PIKV_H2O_STAGED");
    const bool staged = stride <= SEL_SMEM_KEYS && !(force && force[0] == '0');
    if (staged) {
        size_t smem = ((words + 15) & ~(size_t)15) + (size_t)((stride + 3) & ~3) * 4 + (size_t)SEL_CAND_CAP * 4;
        auto kern = h2o_select_kernel<true, SEL_THREADS>;
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("h2o_select smem attribute");
        kern<<<segments, SEL_THREADS, smem, st>>>(acc, ts, stride, seg_len, n, num_heavy, num_recent, evict_mask,
                                                  keep_idx, keep_stride, kept_count);
    } else {
        PIKV_REQUIRE(words <= 200 * 1024, PIKV_ELIMIT, "h2o_select: stride=%d too long", stride);
        const size_t smem = ((words + 15) & ~(size_t)15) + (size_t)SEL_CAND_CAP * 4;
        auto kern = h2o_select_kernel<false, SEL_THREADS_STREAM>;
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("h2o_select smem attribute");
        kern<<<segments, SEL_THREADS_STREAM, smem, st>>>(acc, ts, stride, seg_len, n, num_heavy, num_recent, evict_mask,
                                                   keep_idx, keep_stride, kept_count);
    }
    count_launch(1);
    return check_launch("h2o_select_kernel");
}

extern "C" int pikv_h2o_compact(const pikv_compact_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "h2o_compact: null params");
    PIKV_REQUIRE(p->keep_idx && p->kept_count && p->src_page_table && p->dst_page_table, PIKV_EINVAL,
                 "h2o_compact: null index pointer");
    PIKV_REQUIRE(p->src_k_codes && p->src_v_codes && p->src_k_scale && p->src_v_scale && p->dst_k_codes &&
                     p->dst_v_codes && p->dst_k_scale && p->dst_v_scale,
                 PIKV_EINVAL, "h2o_compact: null cache pointer");
    PIKV_REQUIRE(p->num_seqs > 0 && p->n_kv > 0 && p->keep_stride > 0 && p->max_pages > 0, PIKV_EINVAL,
                 "h2o_compact: bad sizes");
    PIKV_REQUIRE(p->bits == 8 || p->bits == 4, PIKV_EUNSUPPORTED, "h2o_compact: bits=%d", p->bits);
    CompactDev c;
    c.p = *p;
    c.heads_per = p->per_head ? 1 : p->n_kv;
    const int segments = p->per_head ? p->num_seqs * p->n_kv : p->num_seqs;
    const long long lanes = (long long)p->keep_stride * c.heads_per * 8;
    dim3 grid(segments, (unsigned)ceil_div64(lanes, 256));
    h2o_compact_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(c);
    count_launch(1);
    return check_launch("h2o_compact_kernel");
}

extern "C" int pikv_h2o_accumulate_attn(const float* scores, int32_t score_stride, const float* lse,
                                        const int32_t* seq_len, int32_t B, int32_t n_q, int32_t n_kv, float* acc,
                                        int32_t acc_stride, pikv_stream_t stream) {
    PIKV_REQUIRE(scores && lse && acc, PIKV_EINVAL, "h2o_accumulate_attn: null pointer");
    PIKV_REQUIRE(B > 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && score_stride > 0 && acc_stride > 0, PIKV_EINVAL,
                 "h2o_accumulate_attn: bad sizes");
    dim3 grid(ceil_div(min(score_stride, acc_stride), 256), B * n_kv);
    h2o_accumulate_attn_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(scores, score_stride, lse, seq_len, B,
                                                                                  n_q, n_kv, acc, acc_stride);
    count_launch(1);
    return check_launch("h2o_accumulate_attn_kernel");
}
