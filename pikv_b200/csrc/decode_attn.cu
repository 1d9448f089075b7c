// Decode attention over the quantised paged cache (8-bit symmetric or 4-bit asymmetric codes),
// dequantised in registers.
//
// Grid (split, kv head, stream); 4 warps per CTA, each warp streams whole pages (16 tokens x 128
// channels of K and of V plus their scales and, for 4 bits, zero points) of its split through a
// private ring in shared memory filled by bulk async copies (cp.async.bulk + mbarrier transaction
// counts), so the bytes in flight do not depend on registers.  Per page a warp runs 8 + 8
// mma.m16n8k16 (f16 x f16 -> f32) and an online softmax in the log2 domain; see decode_attn_kernel.
// Codes become f16 exactly with one byte-permute (bytes: 0x6400 | (code ^ 0x80) is 1024 + code + 128)
// or one AND-OR (nibbles: 0x6400 | n is 1024 + n).  Q is scaled by a power of two so that it is exact
// in f16.  The cache's swizzle makes the 16-byte shared-memory reads of a fragment conflict-free.
// Partial (O, m, l) of the 4 warps are merged in shared memory; with more than one split a second
// kernel merges the splits.
#include "common.cuh"

#include <mutex>

namespace pikv {

constexpr int DA_WARPS = 4;
constexpr int DA_THREADS = DA_WARPS * 32;
constexpr int DA_MAX_GROUP = 8;
constexpr unsigned DA_WAIT_LIMIT = 1u << 24;            // mbarrier polls before giving up

struct DecodeDev {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    int B, n_q, n_kv, G;
    const int* seq_ids;
    const int* seq_len;
    const int* page_table;
    int num_seqs, max_pages, num_pages;
    const uint8_t* k_codes;
    const uint8_t* v_codes;
    const uint16_t* k_scale;
    const uint16_t* v_scale;
    const float* k_zp;   // 4-bit asymmetric cache only
    const float* v_zp;
    int splits;
    float* lse;
    float* scores;
    int score_stride;
    float* part_o;    // [B*n_q][splits][128]
    float* part_ml;   // [B*n_q][splits][2]
    unsigned* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: returns false when the limit is hit
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned i = 0; i < DA_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two biased bytes (code ^ 0x80) of w selected by SEL -> two exact f16 codes
template <uint32_t SEL>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w_biased) {
    uint32_t x = __byte_perm(w_biased, 0x64646464u, SEL);          // 0x64bb64bb = (1024 + b, 1024 + b)
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&x), __half2half2(__ushort_as_half(0x6480)));  // - 1152
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Geometry of one stage of a warp's ring: a page of one head.
//   8 bit: 16 rows x 128 B of K, of V, 16 + 16 bf16 scales
//   4 bit: 16 rows x 64 B (two codes per byte, low nibble = even channel, 8-byte units swizzled by
//          row & 4), scales, 16 + 16 fp32 zero points
template <int BITS> struct DAGeom;
template <> struct DAGeom<8> { static constexpr int STAGES = 4, ROW = 128, PAGE = 16 * 128, STAGE = 2 * PAGE + 64; };
template <> struct DAGeom<4> { static constexpr int STAGES = 6, ROW = 64, PAGE = 16 * 64, STAGE = 2 * PAGE + 64 + 128; };
constexpr int DA_PBUF_BYTES = DA_MAX_GROUP * 32 * 2;    // per warp: P of two pages, [head][32 positions] f16

template <int BITS>
constexpr size_t da_smem_bytes() {
    return (size_t)DA_WARPS * DAGeom<BITS>::STAGES * DAGeom<BITS>::STAGE + DA_WARPS * DAGeom<BITS>::STAGES * sizeof(uint64_t) +
           DA_WARPS * DA_PBUF_BYTES;
}

// nibbles at bits SHIFT and SHIFT + 16 of w -> (1024 + n, 1024 + n') as two f16: one shift and one AND-OR
template <int SHIFT>
__device__ __forceinline__ uint32_t nib_pair_biased(uint32_t w) {
    return ((w >> SHIFT) & 0x000f000fu) | 0x64006400u;
}
// ... and with the 1024 taken off again (exact)
template <int SHIFT>
__device__ __forceinline__ uint32_t nib_pair(uint32_t w) {
    const uint32_t x = nib_pair_biased<SHIFT>(w);
    __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&x), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<uint32_t*>(&h);
}
// two bytes of w selected by SEL -> (1024 + b, 1024 + b') as two f16
template <uint32_t SEL>
__device__ __forceinline__ uint32_t bytes_to_h2_biased(uint32_t w) { return __byte_perm(w, 0x64646464u, SEL); }

// The legacy mma.sync path is what bounds this kernel on this GPU (one m16n8k16 holds a sub-core's tensor
// pipe for about 32 cycles), so the shapes are chosen to waste as few of its rows as possible:
//   S^T[pos, head] = Kcode[pos, :] . Q[head, :]    A = the page's 16 positions (all rows used), B = Q^T:
//                                                  8 mma per page
//   O^T[ch, head] += Vcode^T[ch, pos] . P'^T[pos, head]   A = 16 channels x 16 positions, 8 mma per page
// The softmax runs on S^T (a thread owns positions r, r+8 of heads 2j, 2j+1) and, for 8-bit codes, takes two
// pages (32 positions) per step; P goes through 512 bytes of shared memory to become the B operand of the
// second product.  Nothing but exact integers enters the
// tensor cores on the cache side:
//   q . x   = kscale * (q . code - zp * sum(q))                        (zp = 0 for the 8-bit cache)
//   P . x_c = sum_pos P' * (bias + code_c) - sum_pos P' * (bias + zp),  P' = P * vscale
// where bias is what the byte/nibble -> f16 trick leaves on (1152 = 1024 + 128 for bytes, 1024 for
// nibbles).  The second sum is the same for every channel: it is carried like the softmax denominator
// (corr) and subtracted at the end.
template <int BITS>
__global__ void __launch_bounds__(DA_THREADS, 3) decode_attn_kernel(DecodeDev d) {
    using GEO = DAGeom<BITS>;
    constexpr int STAGES = GEO::STAGES, STAGE_BYTES = GEO::STAGE, PAGE_BYTES = GEO::PAGE, ROW = GEO::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    // [warp][stage] rings, the barriers, the P buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)DA_WARPS * STAGES * STAGE_BYTES);
    __shared__ float ml_s[DA_WARPS][DA_MAX_GROUP][2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, j = lane & 3;
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int G = d.G;
    const int seq = d.seq_ids ? d.seq_ids[b] : b;
    const bool seq_ok = seq >= 0 && seq < d.num_seqs;
    int len = seq_ok ? d.seq_len[b] : 0;
    len = max(0, min(len, d.max_pages * PIKV_PAGE_TOKENS));
    if (!seq_ok && tid == 0 && d.status) atomicOr(d.status, PIKV_ST_BAD_SEQ);
    const int pages_total = (len + PIKV_PAGE_TOKENS - 1) / PIKV_PAGE_TOKENS;
    const int pps = (pages_total + d.splits - 1) / d.splits;
    const int p_begin = min(pages_total, split * pps), p_end = min(pages_total, p_begin + pps);
    // this warp's pages: p_begin + warp + DA_WARPS * i
    const int my_pages = (p_end - p_begin - warp + DA_WARPS - 1) / DA_WARPS;

    unsigned char* ring = smem + (size_t)warp * STAGES * STAGE_BYTES;
    __half* pbuf = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(bars + DA_WARPS * STAGES) + warp * DA_PBUF_BYTES);
    const uint32_t bar0 = smem_u32(bars + warp * STAGES);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int* pt_row = d.page_table + (size_t)(seq_ok ? seq : 0) * d.max_pages;
    auto issue = [&](int i) {   // lane 0 only: load this warp's i-th page into stage i % STAGES
        const int s = i % STAGES;
        int page = pt_row[p_begin + warp + DA_WARPS * i];
        if (page < 0 || page >= d.num_pages) {
            if (d.status) atomicOr(d.status, PIKV_ST_BAD_PAGE);
            page = 0;
        }
        const size_t prow = ((size_t)page * d.n_kv + h) * PIKV_PAGE_TOKENS;
        const uint32_t dst = smem_u32(ring + (size_t)s * STAGE_BYTES);
        const uint32_t bar = bar0 + 8 * s;
        mbar_expect_tx(bar, STAGE_BYTES);
        bulk_g2s(dst, d.k_codes + prow * ROW, PAGE_BYTES, bar);
        bulk_g2s(dst + PAGE_BYTES, d.v_codes + prow * ROW, PAGE_BYTES, bar);
        bulk_g2s(dst + 2 * PAGE_BYTES, d.k_scale + prow, 32, bar);
        bulk_g2s(dst + 2 * PAGE_BYTES + 32, d.v_scale + prow, 32, bar);
        if (BITS == 4) {
            bulk_g2s(dst + 2 * PAGE_BYTES + 64, d.k_zp + prow, 64, bar);
            bulk_g2s(dst + 2 * PAGE_BYTES + 128, d.v_zp + prow, 64, bar);
        }
    };
    if (lane == 0)
        for (int i = 0; i < min(my_pages, STAGES); ++i) issue(i);

    // ---- Q as the B operand: thread (r, j) holds Q[head r][32j .. 32j+32) as 16 f16 pairs ----
    uint32_t qf[16];
    float qm0, qm1;           // per head 2j, 2j+1: 2^e / sqrt(d) * log2(e), integer dot product -> log2-domain score
    float qs0 = 0.f, qs1 = 0.f;   // 4 bit: sum of the query over its 128 channels
    {
        float qv[32];
        if (r < G) {
            const __nv_bfloat16* qp = d.q + ((size_t)b * d.n_q + (size_t)h * G + r) * 128 + 32 * j;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 w = __ldg(reinterpret_cast<const uint4*>(qp) + i);
                bf16x2_to_f32(w.x, qv[8 * i + 0], qv[8 * i + 1]);
                bf16x2_to_f32(w.y, qv[8 * i + 2], qv[8 * i + 3]);
                bf16x2_to_f32(w.z, qv[8 * i + 4], qv[8 * i + 5]);
                bf16x2_to_f32(w.w, qv[8 * i + 6], qv[8 * i + 7]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) qv[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(qv[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = 0;
        if (amax > 32768.f) e = ilogbf(amax) - 14;     // a power of two keeps the bf16 query exact in f16
        const float down = ldexpf(1.0f, -e);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            // 8 bit: consecutive channel pairs; 4 bit: pairs (c, c + 4) inside each group of 8, the order in
            // which nib_pair() takes nibbles out of a word
            const int c = BITS == 8 ? 2 * i : 8 * (i >> 2) + (i & 3);
            const int c2 = BITS == 8 ? c + 1 : c + 4;
            qf[i] = pack_h2(qv[c] * down, qv[c2] * down);
        }
        const float qmul = ldexpf(1.0f, e) * 0.08838834764831845f * 1.4426950408889634f;
        qm0 = __shfl_sync(0xffffffffu, qmul, 8 * j);          // lane of (head 2j, j = 0)
        qm1 = __shfl_sync(0xffffffffu, qmul, 8 * j + 4);
        if (BITS == 4) {
            float qs = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) qs += qv[i] * down;
            qs += __shfl_xor_sync(0xffffffffu, qs, 1);
            qs += __shfl_xor_sync(0xffffffffu, qs, 2);
            qs0 = __shfl_sync(0xffffffffu, qs, 8 * j);
            qs1 = __shfl_sync(0xffffffffu, qs, 8 * j + 4);
        }
    }

    float o[8][4];
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[m][c] = 0.f;
    // running max, denominator and carried bias term of heads 2j and 2j+1 (this thread's share of the positions)
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f, corr0 = 0.f, corr1 = 0.f;
    bool timed_out = false;
    int i = 0;

    // raw S^T of one page: this thread gets positions r (t[0], t[1]) and r+8 (t[2], t[3]) of heads 2j, 2j+1,
    // scaled to the log2 domain; vw = bias + zero point of V at those positions (4 bit)
    auto page_scores = [&](const unsigned char* st, float (&t)[4], float& vw_lo, float& vw_hi) {
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};      // two accumulator chains
        if (BITS == 8) {
            const unsigned char* klo = st + r * 128;
            const unsigned char* khi = st + (r + 8) * 128;           // same swizzle key: (r + 8) & 7 = r
            const uint4 la = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j) ^ r));
            const uint4 lb = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j + 1) ^ r));
            const uint4 ha = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j) ^ r));
            const uint4 hb = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j + 1) ^ r));
            const uint32_t wl[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
            const uint32_t wh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t a = wl[kk] ^ 0x80808080u, c = wh[kk] ^ 0x80808080u;
                mma_f16((kk & 1) ? sb : sa, bytes_to_h2<0x4140>(a), bytes_to_h2<0x4140>(c), bytes_to_h2<0x4342>(a),
                        bytes_to_h2<0x4342>(c), qf[2 * kk], qf[2 * kk + 1]);
            }
        } else {
            const unsigned char* klo = st + r * 64;
            const unsigned char* khi = st + (r + 8) * 64;            // (r + 8) & 4 = r & 4
            const uint4 lq = *reinterpret_cast<const uint4*>(klo + 8 * ((2 * j) ^ (r & 4)));
            const uint4 hq = *reinterpret_cast<const uint4*>(khi + 8 * ((2 * j) ^ (r & 4)));
            const uint32_t wl[4] = {lq.x, lq.y, lq.z, lq.w};
            const uint32_t wh[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
            for (int wq = 0; wq < 4; ++wq) {
                mma_f16(sa, nib_pair<0>(wl[wq]), nib_pair<0>(wh[wq]), nib_pair<4>(wl[wq]), nib_pair<4>(wh[wq]), qf[4 * wq],
                        qf[4 * wq + 1]);
                mma_f16(sb, nib_pair<8>(wl[wq]), nib_pair<8>(wh[wq]), nib_pair<12>(wl[wq]), nib_pair<12>(wh[wq]),
                        qf[4 * wq + 2], qf[4 * wq + 3]);
            }
        }
        const uint16_t* ksc = reinterpret_cast<const uint16_t*>(st + 2 * PAGE_BYTES);
        const float ks_lo = __uint_as_float((uint32_t)ksc[r] << 16), ks_hi = __uint_as_float((uint32_t)ksc[r + 8] << 16);
        t[0] = sa[0] + sb[0]; t[1] = sa[1] + sb[1]; t[2] = sa[2] + sb[2]; t[3] = sa[3] + sb[3];
        if (BITS == 4) {
            const float* kzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 64);
            const float* vzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 128);
            const float z_lo = kzp[r], z_hi = kzp[r + 8];
            t[0] -= z_lo * qs0; t[1] -= z_lo * qs1; t[2] -= z_hi * qs0; t[3] -= z_hi * qs1;
            vw_lo = 1024.f + vzp[r];
            vw_hi = 1024.f + vzp[r + 8];
        }
        t[0] *= ks_lo * qm0; t[1] *= ks_lo * qm1; t[2] *= ks_hi * qm0; t[3] *= ks_hi * qm1;
    };
    // masks the positions past the sequence end and writes the raw scores out when asked
    auto page_mask_scores = [&](int pos0, float (&t)[4]) {
        if (pos0 + PIKV_PAGE_TOKENS > len) {
            if (pos0 + r >= len) t[0] = t[1] = -INFINITY;
            if (pos0 + r + 8 >= len) t[2] = t[3] = -INFINITY;
        }
        if (d.scores) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int hh = 2 * j + (c & 1), pp = r + 8 * (c >> 1);
                if (hh < G && pos0 + pp < len && pos0 + pp < d.score_stride)
                    d.scores[((size_t)b * d.n_q + (size_t)h * G + hh) * d.score_stride + pos0 + pp] = t[c] * 0.6931471805599453f;
            }
        }
    };
    // O^T += (bias + Vcode)^T . P'^T for one page; pb0 / pb1 = P'[head r][positions 2j, 2j+1] / [2j+8, 2j+9]
    auto page_pv = [&](const unsigned char* st, uint32_t pb0, uint32_t pb1) {
        const unsigned char* vbase = st + PAGE_BYTES;
        const int pp[4] = {2 * j, 2 * j + 1, 8 + 2 * j, 9 + 2 * j};
        if (BITS == 8) {
            const uint4 v0 = *reinterpret_cast<const uint4*>(vbase + pp[0] * 128 + 16 * (r ^ (pp[0] & 7)));
            const uint4 v1 = *reinterpret_cast<const uint4*>(vbase + pp[1] * 128 + 16 * (r ^ (pp[1] & 7)));
            const uint4 v2 = *reinterpret_cast<const uint4*>(vbase + pp[2] * 128 + 16 * (r ^ (pp[2] & 7)));
            const uint4 v3 = *reinterpret_cast<const uint4*>(vbase + pp[3] * 128 + 16 * (r ^ (pp[3] & 7)));
            const uint32_t vw0[4] = {v0.x, v0.y, v0.z, v0.w}, vw1[4] = {v1.x, v1.y, v1.z, v1.w};
            const uint32_t vw2[4] = {v2.x, v2.y, v2.z, v2.w}, vw3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const int wi = m >> 1;
                // bytes (2*(m&1)) and (2*(m&1)+1) of the two positions of a pair, interleaved, then code + 128
                const uint32_t ta = ((m & 1) ? __byte_perm(vw0[wi], vw1[wi], 0x7362) : __byte_perm(vw0[wi], vw1[wi], 0x5140)) ^ 0x80808080u;
                const uint32_t tb = ((m & 1) ? __byte_perm(vw2[wi], vw3[wi], 0x7362) : __byte_perm(vw2[wi], vw3[wi], 0x5140)) ^ 0x80808080u;
                // channel 16r+2m (a0, a2) and 16r+2m+1 (a1, a3); positions 2j, 2j+1 (a0, a1) and 8+2j, 9+2j (a2, a3)
                mma_f16(o[m], bytes_to_h2_biased<0x4140>(ta), bytes_to_h2_biased<0x4342>(ta), bytes_to_h2_biased<0x4140>(tb),
                        bytes_to_h2_biased<0x4342>(tb), pb0, pb1);
            }
        } else {
            // channels 16r .. 16r+15 of the four positions: one 8-byte unit each
            const uint2 v0 = *reinterpret_cast<const uint2*>(vbase + pp[0] * 64 + 8 * (r ^ (pp[0] & 4)));
            const uint2 v1 = *reinterpret_cast<const uint2*>(vbase + pp[1] * 64 + 8 * (r ^ (pp[1] & 4)));
            const uint2 v2 = *reinterpret_cast<const uint2*>(vbase + pp[2] * 64 + 8 * (r ^ (pp[2] & 4)));
            const uint2 v3 = *reinterpret_cast<const uint2*>(vbase + pp[3] * 64 + 8 * (r ^ (pp[3] & 4)));
#pragma unroll
            for (int hb = 0; hb < 4; ++hb) {
                // bytes 2hb', 2hb'+1 of word wq of both positions of a pair: (p.b, p.b', p'.b, p'.b')
                const int wq = hb >> 1;
                const uint32_t sel = (hb & 1) ? 0x7632u : 0x5410u;
                const uint32_t ga = __byte_perm(wq ? v0.y : v0.x, wq ? v1.y : v1.x, sel);
                const uint32_t gb = __byte_perm(wq ? v2.y : v2.x, wq ? v3.y : v3.x, sel);
                const int m = 2 * hb;   // byte m of the unit: channels 16r+2m (low nibble), 16r+2m+1 (high nibble)
                mma_f16(o[m], nib_pair_biased<0>(ga), nib_pair_biased<4>(ga), nib_pair_biased<0>(gb), nib_pair_biased<4>(gb), pb0, pb1);
                mma_f16(o[m + 1], nib_pair_biased<8>(ga), nib_pair_biased<12>(ga), nib_pair_biased<8>(gb), nib_pair_biased<12>(gb), pb0,
                        pb1);
            }
        }
    };

    // 8 bit: two pages (32 positions) per step of the online softmax, i.e. one max reduction and one rescale of
    // O for both (measured 0.794 -> 0.772 ms at 64 x 8 x 32768); the 4-bit kernel is faster with one (0.893
    // against 0.945 ms)
    constexpr int PPS = BITS == 8 ? 2 : 1;
    for (; i < my_pages; i += PPS) {
        const bool two = PPS == 2 && i + 1 < my_pages;           // warp-uniform
        const int sA = i % STAGES, sB = (i + 1) % STAGES;
        if (!mbar_wait(bar0 + 8 * sA, (uint32_t)(i / STAGES) & 1u) ||
            (two && !mbar_wait(bar0 + 8 * sB, (uint32_t)((i + 1) / STAGES) & 1u))) {
            timed_out = true;
            break;
        }
        const unsigned char* stA = ring + (size_t)sA * STAGE_BYTES;
        const unsigned char* stB = ring + (size_t)sB * STAGE_BYTES;
        const int posA = (p_begin + warp + DA_WARPS * i) * PIKV_PAGE_TOKENS;
        const int posB = (p_begin + warp + DA_WARPS * (i + 1)) * PIKV_PAGE_TOKENS;
        float tA[4], tB[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        float vwA_lo = 0.f, vwA_hi = 0.f, vwB_lo = 0.f, vwB_hi = 0.f;
        page_scores(stA, tA, vwA_lo, vwA_hi);
        page_mask_scores(posA, tA);
        if (two) {
            page_scores(stB, tB, vwB_lo, vwB_hi);
            page_mask_scores(posB, tB);
        }
        // ---- online softmax (log2 domain); the 8 lanes with the same j hold the positions of a head pair ----
        float mx0 = fmaxf(fmaxf(tA[0], tA[2]), fmaxf(tB[0], tB[2])), mx1 = fmaxf(fmaxf(tA[1], tA[3]), fmaxf(tB[1], tB[3]));
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0, mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float al0 = exp2f(m0 - mu0), al1 = exp2f(m1 - mu1);
        m0 = mn0;
        m1 = mn1;
        float la = 0.f, lb = 0.f, ca = 0.f, cb = 0.f;
        // P' = P * vscale, rounded to f16 as the tensor cores will see it; pbuf is [head][32 positions]
        auto page_probs = [&](const unsigned char* st, const float (&t)[4], float vw_lo, float vw_hi, int base) {
            const uint16_t* vsc = reinterpret_cast<const uint16_t*>(st + 2 * PAGE_BYTES + 32);
            const float vs_lo = __uint_as_float((uint32_t)vsc[r] << 16), vs_hi = __uint_as_float((uint32_t)vsc[r + 8] << 16);
            const float p0 = exp2f(t[0] - mu0), p1 = exp2f(t[1] - mu1), p2 = exp2f(t[2] - mu0), p3 = exp2f(t[3] - mu1);
            la += p0 + p2;
            lb += p1 + p3;
            const __half h0 = __float2half_rn(p0 * vs_lo), h1 = __float2half_rn(p1 * vs_lo);
            const __half h2 = __float2half_rn(p2 * vs_hi), h3 = __float2half_rn(p3 * vs_hi);
            if (BITS == 8) {
                ca += __half2float(h0) + __half2float(h2);           // x 1152 at the end
                cb += __half2float(h1) + __half2float(h3);
            } else {
                ca += __half2float(h0) * vw_lo + __half2float(h2) * vw_hi;
                cb += __half2float(h1) * vw_lo + __half2float(h3) * vw_hi;
            }
            pbuf[(2 * j) * 32 + base + r] = h0;
            pbuf[(2 * j + 1) * 32 + base + r] = h1;
            pbuf[(2 * j) * 32 + base + r + 8] = h2;
            pbuf[(2 * j + 1) * 32 + base + r + 8] = h3;
        };
        page_probs(stA, tA, vwA_lo, vwA_hi, 0);
        if (two) page_probs(stB, tB, vwB_lo, vwB_hi, 16);
        l0 = l0 * al0 + la;
        l1 = l1 * al1 + lb;
        corr0 = corr0 * al0 + ca;
        corr1 = corr1 * al1 + cb;
        // rescale O: this thread's columns are query heads 2j and 2j+1
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            o[m][0] *= al0; o[m][1] *= al1; o[m][2] *= al0; o[m][3] *= al1;
        }
        __syncwarp();
        page_pv(stA, *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 2 * j),
                *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 2 * j + 8));
        if (two)
            page_pv(stB, *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 16 + 2 * j),
                    *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 24 + 2 * j));
        __syncwarp();
        if (lane == 0) {
            if (i + STAGES < my_pages) issue(i + STAGES);
            if (PPS == 2 && i + 1 + STAGES < my_pages) issue(i + 1 + STAGES);
        }
    }
    if (timed_out) {
        // give the copies already issued one more bounded chance to land before the ring is reused
        if (lane == 0 && d.status) atomicOr(d.status, PIKV_ST_WAIT_TIMEOUT);
        for (int ii = i; ii < min(my_pages, i + STAGES); ++ii)
            (void)mbar_wait(bar0 + 8 * (ii % STAGES), (uint32_t)(ii / STAGES) & 1u);
    }

    // ---- denominators and the carried bias term: sum over the 8 lanes of a head pair ----
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        corr0 += __shfl_xor_sync(0xffffffffu, corr0, sh);
        corr1 += __shfl_xor_sync(0xffffffffu, corr1, sh);
    }
    if (BITS == 8) {
        corr0 *= 1152.f;
        corr1 *= 1152.f;
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        o[m][0] -= corr0; o[m][1] -= corr1; o[m][2] -= corr0; o[m][3] -= corr1;
    }
    // ---- merge the 4 warps ----
    __syncthreads();   // every warp is done with its ring; reuse it as the merge buffer
    float* mo = reinterpret_cast<float*>(smem);   // [warp][q][128]
    if (r == 0) {
        ml_s[warp][2 * j][0] = m0;
        ml_s[warp][2 * j][1] = l0;
        ml_s[warp][2 * j + 1][0] = m1;
        ml_s[warp][2 * j + 1][1] = l1;
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int ch = 16 * r + 2 * m;
        float* base = mo + (size_t)warp * DA_MAX_GROUP * 128;
        base[(2 * j) * 128 + ch] = o[m][0];
        base[(2 * j + 1) * 128 + ch] = o[m][1];
        base[(2 * j) * 128 + ch + 1] = o[m][2];
        base[(2 * j + 1) * 128 + ch + 1] = o[m][3];
    }
    __syncthreads();
    const int ch = tid;   // 128 threads = 128 channels
    for (int qh = 0; qh < G; ++qh) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) M = fmaxf(M, ml_s[w][qh][0]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) {
            const float mw = ml_s[w][qh][0];
            const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            acc += mo[((size_t)w * DA_MAX_GROUP + qh) * 128 + ch] * sc;
            l += ml_s[w][qh][1] * sc;
        }
        const size_t bq = (size_t)b * d.n_q + (size_t)h * G + qh;
        if (d.splits == 1) {
            d.out[bq * 128 + ch] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            if (ch == 0 && d.lse) d.lse[bq] = (l > 0.f) ? M * 0.6931471805599453f + logf(l) : -INFINITY;
        } else {
            d.part_o[(bq * d.splits + split) * 128 + ch] = acc;
            if (ch == 0) {
                d.part_ml[(bq * d.splits + split) * 2 + 0] = M;
                d.part_ml[(bq * d.splits + split) * 2 + 1] = l;
            }
        }
    }
}

__global__ void __launch_bounds__(128) decode_merge_kernel(DecodeDev d) {
    const size_t bq = blockIdx.x;
    const int ch = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < d.splits; ++s) M = fmaxf(M, d.part_ml[(bq * d.splits + s) * 2]);
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < d.splits; ++s) {
        const float ms = d.part_ml[(bq * d.splits + s) * 2];
        const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        acc += d.part_o[(bq * d.splits + s) * 128 + ch] * sc;
        l += d.part_ml[(bq * d.splits + s) * 2 + 1] * sc;
    }
    d.out[bq * 128 + ch] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    if (ch == 0 && d.lse) d.lse[bq] = (l > 0.f) ? M * 0.6931471805599453f + logf(l) : -INFINITY;
}

static int pick_splits(int B, int n_kv, int max_ctx) {
    const int pages = ceil_div(max(max_ctx, 1), PIKV_PAGE_TOKENS);
    const int resident = sm_count() * 3;
    int s = ceil_div(8 * resident, max(1, B * n_kv));
    s = min(s, max(1, pages / 64));   // at least 16 pages per warp (64 streams x 8 heads x 2048 tokens: 2 splits
                                      // 73 us, 4 splits 80 us, 8 splits 99 us)
    return max(1, min(s, 64));
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_decode_attn_default_splits(int32_t B, int32_t n_kv, int32_t max_ctx) {
    if (B <= 0 || n_kv <= 0) return 1;
    return pick_splits(B, n_kv, max_ctx);
}

extern "C" size_t pikv_decode_attn_workspace_bytes(int32_t B, int32_t n_q, int32_t n_kv, int32_t max_ctx,
                                                   int32_t splits) {
    if (B <= 0 || n_q <= 0 || n_kv <= 0) return 0;
    if (splits <= 0) splits = pick_splits(B, n_kv, max_ctx);
    return (size_t)B * n_q * splits * (128 + 2) * sizeof(float);
}

static int decode_attn_launch(const pikv_decode_params* p, pikv_stream_t stream, int bits) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "decode_attn: null params");
    PIKV_REQUIRE(p->q && p->out && p->seq_len && p->page_table, PIKV_EINVAL, "decode_attn: null pointer");
    PIKV_REQUIRE(p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL, "decode_attn: null cache pointer");
    PIKV_REQUIRE(p->B > 0 && p->n_q > 0 && p->n_kv > 0 && p->n_q % p->n_kv == 0, PIKV_EINVAL, "decode_attn: bad head counts");
    PIKV_REQUIRE(p->n_q / p->n_kv <= DA_MAX_GROUP, PIKV_EUNSUPPORTED, "decode_attn: %d query heads per KV head (max %d)",
                 p->n_q / p->n_kv, DA_MAX_GROUP);
    PIKV_REQUIRE(p->num_seqs > 0 && p->max_pages > 0 && p->num_pages > 0, PIKV_EINVAL, "decode_attn: bad cache geometry");
    PIKV_REQUIRE(p->n_kv <= 65535 && p->B <= 65535, PIKV_ELIMIT, "decode_attn: B and n_kv must be <= 65535");
    DecodeDev d;
    d.q = static_cast<const __nv_bfloat16*>(p->q);
    d.out = static_cast<__nv_bfloat16*>(p->out);
    d.B = p->B; d.n_q = p->n_q; d.n_kv = p->n_kv; d.G = p->n_q / p->n_kv;
    d.seq_ids = p->seq_ids; d.seq_len = p->seq_len; d.page_table = p->page_table;
    d.num_seqs = p->num_seqs; d.max_pages = p->max_pages; d.num_pages = p->num_pages;
    d.k_codes = static_cast<const uint8_t*>(p->k_codes); d.v_codes = static_cast<const uint8_t*>(p->v_codes);
    d.k_scale = static_cast<const uint16_t*>(p->k_scale); d.v_scale = static_cast<const uint16_t*>(p->v_scale);
    d.k_zp = static_cast<const float*>(p->k_zp); d.v_zp = static_cast<const float*>(p->v_zp);
    PIKV_REQUIRE(bits == 8 || (d.k_zp && d.v_zp), PIKV_EINVAL, "decode_attn_q4: the 4-bit cache needs k_zp and v_zp");
    d.splits = p->splits > 0 ? p->splits : pick_splits(p->B, p->n_kv, p->max_pages * PIKV_PAGE_TOKENS);
    d.lse = p->lse; d.scores = p->scores; d.score_stride = p->score_stride; d.status = p->status;
    PIKV_REQUIRE(d.scores == nullptr || d.score_stride > 0, PIKV_EINVAL, "decode_attn: score_stride");
    d.part_o = nullptr; d.part_ml = nullptr;
    if (d.splits > 1) {
        const size_t need = (size_t)p->B * p->n_q * d.splits * (128 + 2) * sizeof(float);
        PIKV_REQUIRE(p->workspace && p->workspace_bytes >= need, PIKV_EINVAL, "decode_attn: workspace too small (%zu needed)", need);
        d.part_o = static_cast<float*>(p->workspace);
        d.part_ml = d.part_o + (size_t)p->B * p->n_q * d.splits * 128;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(d.splits, p->n_kv, p->B);
    if (bits == 8) {
        const size_t smem = da_smem_bytes<8>();
        if (cudaFuncSetAttribute(decode_attn_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_attn smem attribute");
        decode_attn_kernel<8><<<grid, DA_THREADS, smem, st>>>(d);
    } else {
        const size_t smem = da_smem_bytes<4>();
        if (cudaFuncSetAttribute(decode_attn_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_attn smem attribute");
        decode_attn_kernel<4><<<grid, DA_THREADS, smem, st>>>(d);
    }
    int launches = 1;
    int rc = check_launch(bits == 8 ? "decode_attn_kernel<8>" : "decode_attn_kernel<4>");
    if (rc != PIKV_OK) return rc;
    if (d.splits > 1) {
        decode_merge_kernel<<<p->B * p->n_q, 128, 0, st>>>(d);
        ++launches;
        rc = check_launch("decode_merge_kernel");
    }
    count_launch(launches);
    return rc;
}

extern "C" int pikv_decode_attn_q8(const pikv_decode_params* p, pikv_stream_t stream) {
    return decode_attn_launch(p, stream, 8);
}

extern "C" int pikv_decode_attn_q4(const pikv_decode_params* p, pikv_stream_t stream) {
    return decode_attn_launch(p, stream, 4);
}

// ---- decode attention for callers that must not allocate --------------------------------------------
// Some hosts of this library cannot call cudaMalloc when they need attention: a serving process that
// handed all of HBM to its own page pool at start-up, a plug-in that runs inside someone else's
// allocator-free region, code between cudaStreamBeginCapture and EndCapture.  For them the split-KV
// partials live in this fixed array inside the library image.  Every GPU that loads the library keeps
// these 8 MiB until the process exits, and every call on a device shares them.
constexpr size_t DA_STATIC_SCRATCH_BYTES = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[DA_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address comes from the runtime, once per
// device, with that device current.
static int decode_static_scratch_ptr(void** out) {
    static void* ptrs[64];
    static bool have[64];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("decode_attn_static: cannot identify the current device");
        return PIKV_ECUDA;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("decode_attn_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return PIKV_ECUDA;
        }
        ptrs[dev] = p;
        have[dev] = true;
    }
    *out = ptrs[dev];
    return PIKV_OK;
}

extern "C" size_t pikv_decode_attn_static_scratch_bytes(void) { return DA_STATIC_SCRATCH_BYTES; }

extern "C" int pikv_decode_attn_q8_static(const pikv_decode_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "decode_attn_static: null params");
    PIKV_REQUIRE(p->B > 0 && p->n_q > 0 && p->n_kv > 0 && p->max_pages > 0, PIKV_EINVAL, "decode_attn_static: bad sizes");
    pikv_decode_params q = *p;
    q.splits = p->splits > 0 ? p->splits : pick_splits(p->B, p->n_kv, p->max_pages * PIKV_PAGE_TOKENS);
    const size_t need = q.splits > 1 ? (size_t)p->B * p->n_q * q.splits * (128 + 2) * sizeof(float) : 0;
    PIKV_REQUIRE(need <= DA_STATIC_SCRATCH_BYTES, PIKV_ELIMIT,
                 "decode_attn_static: %d streams x %d query heads x %d splits need %zu bytes of split scratch, the built-in "
                 "array holds %zu; lower `splits` or use pikv_decode_attn_q8 with your own workspace",
                 p->B, p->n_q, q.splits, need, DA_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    const int rc = decode_static_scratch_ptr(&scratch);
    if (rc != PIKV_OK) return rc;
    q.workspace = scratch;
    q.workspace_bytes = DA_STATIC_SCRATCH_BYTES;
    return pikv_decode_attn_q8(&q, stream);
}

