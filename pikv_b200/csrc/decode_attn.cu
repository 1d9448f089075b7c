// Decode attention over the int8 paged cache, dequantised in registers.
//
// Grid (split, kv head, stream); 4 warps per CTA, each warp streams whole pages
// (16 tokens x 128 channels of K and of V = 2 x 2 KiB plus 2 x 32 B of scales) of its
// split through a private 4-stage ring in shared memory filled by bulk async copies
// (cp.async.bulk + mbarrier transaction counts), so the bytes in flight do not depend on
// registers.  Per page a warp does
//   S[q, pos]   = Q[q, :] . Kcode[pos, :]      8 + 8 mma.m16n8k16 (f16 x f16 -> f32)
//   s           = S * kscale[pos] * 2^e / sqrt(d)   (fp32, log2 domain for exp2f)
//   online softmax over the positions, P kept in registers as the B operand of
//   O^T[c, q]  += (Vcode[pos, c] * vscale[pos]) . P[q, pos]      8 mma.m16n8k16
// int8 codes become f16 exactly with one byte-permute and one subtract per pair
// (0x6400 | (code ^ 0x80) is 1024 + code + 128 in f16).  Q is scaled by a power of two so
// that it is exact in f16.  The cache's chunk swizzle makes every 16-byte shared-memory
// read of a fragment conflict-free.  Partial (O, m, l) of the 4 warps are merged in shared
// memory; with more than one split a second kernel merges the splits.
#include "common.cuh"

#include <mutex>

namespace pikv {

constexpr int DA_WARPS = 4;
constexpr int DA_THREADS = DA_WARPS * 32;
constexpr int DA_STAGES = 4;
constexpr int DA_PAGE_BYTES = 16 * 128;                 // one page of one head, K or V
constexpr int DA_STAGE_BYTES = 2 * DA_PAGE_BYTES + 64;  // K, V, 16 K scales, 16 V scales
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
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 h = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(DA_THREADS, 3) decode_attn_q8_kernel(DecodeDev d) {
    extern __shared__ __align__(128) unsigned char smem[];
    // [warp][stage] rings, then the barriers
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)DA_WARPS * DA_STAGES * DA_STAGE_BYTES);
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

    unsigned char* ring = smem + (size_t)warp * DA_STAGES * DA_STAGE_BYTES;
    const uint32_t bar0 = smem_u32(bars + warp * DA_STAGES);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < DA_STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int* pt_row = d.page_table + (size_t)(seq_ok ? seq : 0) * d.max_pages;
    auto issue = [&](int i) {   // lane 0 only: load this warp's i-th page into stage i % STAGES
        const int s = i % DA_STAGES;
        int page = pt_row[p_begin + warp + DA_WARPS * i];
        if (page < 0 || page >= d.num_pages) {
            if (d.status) atomicOr(d.status, PIKV_ST_BAD_PAGE);
            page = 0;
        }
        const size_t prow = ((size_t)page * d.n_kv + h) * PIKV_PAGE_TOKENS;
        const uint32_t dst = smem_u32(ring + (size_t)s * DA_STAGE_BYTES);
        const uint32_t bar = bar0 + 8 * s;
        mbar_expect_tx(bar, DA_STAGE_BYTES);
        bulk_g2s(dst, d.k_codes + prow * 128, DA_PAGE_BYTES, bar);
        bulk_g2s(dst + DA_PAGE_BYTES, d.v_codes + prow * 128, DA_PAGE_BYTES, bar);
        bulk_g2s(dst + 2 * DA_PAGE_BYTES, d.k_scale + prow, 32, bar);
        bulk_g2s(dst + 2 * DA_PAGE_BYTES + 32, d.v_scale + prow, 32, bar);
    };
    if (lane == 0)
        for (int i = 0; i < min(my_pages, DA_STAGES); ++i) issue(i);

    // ---- Q fragments: thread (r, j) holds Q[head r][32j .. 32j+32) as 16 f16 pairs ----
    uint32_t qf[16];
    float qmul = 0.f;   // 2^e / sqrt(d) * log2(e): turns the integer dot product into log2-domain scores
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
        if (amax > 32768.f) e = ilogbf(amax) - 14;
        const float down = ldexpf(1.0f, -e);
#pragma unroll
        for (int i = 0; i < 16; ++i) qf[i] = pack_h2(qv[2 * i] * down, qv[2 * i + 1] * down);
        qmul = ldexpf(1.0f, e) * 0.08838834764831845f * 1.4426950408889634f;
    }

    float o[8][4];
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[m][c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool timed_out = false;
    int i = 0;

    for (; i < my_pages; ++i) {
        const int s = i % DA_STAGES;
        const uint32_t parity = (uint32_t)(i / DA_STAGES) & 1u;
        if (!mbar_wait(bar0 + 8 * s, parity)) {
            timed_out = true;
            break;
        }
        const unsigned char* st = ring + (size_t)s * DA_STAGE_BYTES;
        const int page_idx = p_begin + warp + DA_WARPS * i;
        const int pos0 = page_idx * PIKV_PAGE_TOKENS;

        // ---- S = Q . K^T for the page's 16 positions (two blocks of 8) ----
        float sacc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
            const int row = 8 * nb + r;
            const unsigned char* krow = st + row * 128;
            uint4 ka = *reinterpret_cast<const uint4*>(krow + 16 * ((2 * j) ^ r));
            uint4 kb = *reinterpret_cast<const uint4*>(krow + 16 * ((2 * j + 1) ^ r));
            uint32_t kw[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t w = kw[ks] ^ 0x80808080u;
                mma_f16(sacc[nb], qf[2 * ks], 0u, qf[2 * ks + 1], 0u, bytes_to_h2<0x4140>(w), bytes_to_h2<0x4342>(w));
            }
        }
        // scales of positions {2j, 2j+1} and {8+2j, 9+2j}
        const uint32_t* ksc = reinterpret_cast<const uint32_t*>(st + 2 * DA_PAGE_BYTES);
        const uint32_t* vsc = reinterpret_cast<const uint32_t*>(st + 2 * DA_PAGE_BYTES + 32);
        float ks0, ks1, ks2, ks3;
        bf16x2_to_f32(ksc[j], ks0, ks1);
        bf16x2_to_f32(ksc[4 + j], ks2, ks3);
        float t[4];
        t[0] = sacc[0][0] * (ks0 * qmul);
        t[1] = sacc[0][1] * (ks1 * qmul);
        t[2] = sacc[1][0] * (ks2 * qmul);
        t[3] = sacc[1][1] * (ks3 * qmul);
        const int pp[4] = {2 * j, 2 * j + 1, 8 + 2 * j, 9 + 2 * j};
        if (pos0 + PIKV_PAGE_TOKENS > len) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (pos0 + pp[c] >= len) t[c] = -INFINITY;
        }
        if (d.scores && r < G) {
            float* srow = d.scores + ((size_t)b * d.n_q + (size_t)h * G + r) * d.score_stride + pos0;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (pos0 + pp[c] < len && pos0 + pp[c] < d.score_stride) srow[pp[c]] = t[c] * 0.6931471805599453f;
        }
        // ---- online softmax (log2 domain) ----
        float mx = fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run - m_use);
        float p[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) p[c] = exp2f(t[c] - m_use);
        l_run = l_run * alpha + ((p[0] + p[1]) + (p[2] + p[3]));
        m_run = m_new;
        const uint32_t pb0 = pack_h2(p[0], p[1]), pb1 = pack_h2(p[2], p[3]);
        // rescale O: this thread's columns are query heads 2j and 2j+1
        const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * j) * 4);
        const float al1 = __shfl_sync(0xffffffffu, alpha, (2 * j + 1) * 4);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            o[m][0] *= al0; o[m][1] *= al1; o[m][2] *= al0; o[m][3] *= al1;
        }
        // ---- O^T += (Vcode * vscale)^T . P^T ----
        const unsigned char* vbase = st + DA_PAGE_BYTES;
        uint4 v0 = *reinterpret_cast<const uint4*>(vbase + pp[0] * 128 + 16 * (r ^ (pp[0] & 7)));
        uint4 v1 = *reinterpret_cast<const uint4*>(vbase + pp[1] * 128 + 16 * (r ^ (pp[1] & 7)));
        uint4 v2 = *reinterpret_cast<const uint4*>(vbase + pp[2] * 128 + 16 * (r ^ (pp[2] & 7)));
        uint4 v3 = *reinterpret_cast<const uint4*>(vbase + pp[3] * 128 + 16 * (r ^ (pp[3] & 7)));
        const uint32_t vw0[4] = {v0.x ^ 0x80808080u, v0.y ^ 0x80808080u, v0.z ^ 0x80808080u, v0.w ^ 0x80808080u};
        const uint32_t vw1[4] = {v1.x ^ 0x80808080u, v1.y ^ 0x80808080u, v1.z ^ 0x80808080u, v1.w ^ 0x80808080u};
        const uint32_t vw2[4] = {v2.x ^ 0x80808080u, v2.y ^ 0x80808080u, v2.z ^ 0x80808080u, v2.w ^ 0x80808080u};
        const uint32_t vw3[4] = {v3.x ^ 0x80808080u, v3.y ^ 0x80808080u, v3.z ^ 0x80808080u, v3.w ^ 0x80808080u};
        float vs0, vs1, vs2, vs3;
        bf16x2_to_f32(vsc[j], vs0, vs1);
        bf16x2_to_f32(vsc[4 + j], vs2, vs3);
        const uint32_t vsa = pack_h2(vs0, vs1), vsb = pack_h2(vs2, vs3);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const int wi = m >> 1;
            // bytes (2*(m&1)) and (2*(m&1)+1) of the two positions of a pair, interleaved
            const uint32_t ta = (m & 1) ? __byte_perm(vw0[wi], vw1[wi], 0x7362) : __byte_perm(vw0[wi], vw1[wi], 0x5140);
            const uint32_t tb = (m & 1) ? __byte_perm(vw2[wi], vw3[wi], 0x7362) : __byte_perm(vw2[wi], vw3[wi], 0x5140);
            const uint32_t a0 = hmul2_u32(bytes_to_h2<0x4140>(ta), vsa);   // channel 16r+2m,   positions 2j, 2j+1
            const uint32_t a1 = hmul2_u32(bytes_to_h2<0x4342>(ta), vsa);   // channel 16r+2m+1
            const uint32_t a2 = hmul2_u32(bytes_to_h2<0x4140>(tb), vsb);   // channel 16r+2m,   positions 8+2j, 9+2j
            const uint32_t a3 = hmul2_u32(bytes_to_h2<0x4342>(tb), vsb);
            mma_f16(o[m], a0, a1, a2, a3, pb0, pb1);
        }
        __syncwarp();
        if (lane == 0 && i + DA_STAGES < my_pages) issue(i + DA_STAGES);
    }
    if (timed_out) {
        // give the copies already issued one more bounded chance to land before the ring is reused
        if (lane == 0 && d.status) atomicOr(d.status, PIKV_ST_WAIT_TIMEOUT);
        for (int ii = i; ii < min(my_pages, i + DA_STAGES); ++ii)
            (void)mbar_wait(bar0 + 8 * (ii % DA_STAGES), (uint32_t)(ii / DA_STAGES) & 1u);
    }

    // ---- merge the 4 warps ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();   // every warp is done with its ring; reuse it as the merge buffer
    float* mo = reinterpret_cast<float*>(smem);   // [warp][q][128]
    if (j == 0 && r < DA_MAX_GROUP) {
        ml_s[warp][r][0] = m_run;
        ml_s[warp][r][1] = l_run;
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

// ---- 4-bit asymmetric cache ---------------------------------------------------------------------------
// Same structure over half the bytes.  A page of one head is 16 rows of 64 bytes (two codes per byte,
// low nibble = even channel, 8-byte units swizzled by row & 4) plus bf16 scales and fp32 zero points.
// The zero point never enters the tensor-core operands: with x = (code - zp) * scale,
//   q . x   = scale * (q . code - zp * sum(q))            (sum(q) once per query head)
//   P . x_c = sum_pos P * scale * code_c - sum_pos P * scale * zp
// and the second sum does not depend on the channel: it is carried like the softmax denominator and
// subtracted from every channel at the end.  Nibbles become f16 exactly (0x6400 | n is 1024 + n).
constexpr int DA4_STAGES = 6;
constexpr int DA4_PAGE_BYTES = 16 * 64;
constexpr int DA4_STAGE_BYTES = 2 * DA4_PAGE_BYTES + 64 + 128;   // K, V, scales (2 x 32 B), zero points (2 x 64 B)

template <uint32_t SEL>
__device__ __forceinline__ uint32_t nibs_to_h2(uint32_t u) {
    uint32_t x = __byte_perm(u, 0x64646464u, SEL);                  // (1024 + n, 1024 + n')
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&x), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(DA_THREADS, 3) decode_attn_q4_kernel(DecodeDev d) {
    extern __shared__ __align__(128) unsigned char smem[];
    // [warp][stage] rings, then the barriers
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)DA_WARPS * DA4_STAGES * DA4_STAGE_BYTES);
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

    unsigned char* ring = smem + (size_t)warp * DA4_STAGES * DA4_STAGE_BYTES;
    const uint32_t bar0 = smem_u32(bars + warp * DA4_STAGES);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < DA4_STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int* pt_row = d.page_table + (size_t)(seq_ok ? seq : 0) * d.max_pages;
    auto issue = [&](int i) {   // lane 0 only: load this warp's i-th page into stage i % STAGES
        const int s = i % DA4_STAGES;
        int page = pt_row[p_begin + warp + DA_WARPS * i];
        if (page < 0 || page >= d.num_pages) {
            if (d.status) atomicOr(d.status, PIKV_ST_BAD_PAGE);
            page = 0;
        }
        const size_t prow = ((size_t)page * d.n_kv + h) * PIKV_PAGE_TOKENS;
        const uint32_t dst = smem_u32(ring + (size_t)s * DA4_STAGE_BYTES);
        const uint32_t bar = bar0 + 8 * s;
        mbar_expect_tx(bar, DA4_STAGE_BYTES);
        bulk_g2s(dst, d.k_codes + prow * 64, DA4_PAGE_BYTES, bar);
        bulk_g2s(dst + DA4_PAGE_BYTES, d.v_codes + prow * 64, DA4_PAGE_BYTES, bar);
        bulk_g2s(dst + 2 * DA4_PAGE_BYTES, d.k_scale + prow, 32, bar);
        bulk_g2s(dst + 2 * DA4_PAGE_BYTES + 32, d.v_scale + prow, 32, bar);
        bulk_g2s(dst + 2 * DA4_PAGE_BYTES + 64, d.k_zp + prow, 64, bar);
        bulk_g2s(dst + 2 * DA4_PAGE_BYTES + 128, d.v_zp + prow, 64, bar);
    };
    if (lane == 0)
        for (int i = 0; i < min(my_pages, DA4_STAGES); ++i) issue(i);

    // ---- Q fragments: thread (r, j) holds Q[head r][32j .. 32j+32) as 16 f16 pairs ----
    uint32_t qf[16];
    float qmul = 0.f;   // 2^e / sqrt(d) * log2(e): turns the integer dot product into log2-domain scores
    float qsum = 0.f;
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
        if (amax > 32768.f) e = ilogbf(amax) - 14;
        const float down = ldexpf(1.0f, -e);
#pragma unroll
        for (int i = 0; i < 16; ++i) qf[i] = pack_h2(qv[2 * i] * down, qv[2 * i + 1] * down);
        qmul = ldexpf(1.0f, e) * 0.08838834764831845f * 1.4426950408889634f;
        // sum of the (scaled, f16-exact) query over all 128 channels of head r
        float qs = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) qs += qv[i] * down;
        qs += __shfl_xor_sync(0xffffffffu, qs, 1);
        qs += __shfl_xor_sync(0xffffffffu, qs, 2);
        qsum = qs;
    }
    float corr = 0.f;    // sum over positions of P * vscale * vzp for head r (this thread's 4 positions per page)

    float o[8][4];
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[m][c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool timed_out = false;
    int i = 0;

    for (; i < my_pages; ++i) {
        const int s = i % DA4_STAGES;
        const uint32_t parity = (uint32_t)(i / DA4_STAGES) & 1u;
        if (!mbar_wait(bar0 + 8 * s, parity)) {
            timed_out = true;
            break;
        }
        const unsigned char* st = ring + (size_t)s * DA4_STAGE_BYTES;
        const int page_idx = p_begin + warp + DA_WARPS * i;
        const int pos0 = page_idx * PIKV_PAGE_TOKENS;

        // ---- S = Q . K^T for the page's 16 positions (two blocks of 8) ----
        float sacc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
            const int row = 8 * nb + r;
            const unsigned char* krow = st + row * 64;
            // channels 32j .. 32j+31 of this row: units 2j, 2j+1 (the swizzle keeps the pair together)
            uint4 kq = *reinterpret_cast<const uint4*>(krow + 8 * ((2 * j) ^ (row & 4)));
            const uint32_t kw[4] = {kq.x, kq.y, kq.z, kq.w};
#pragma unroll
            for (int wq = 0; wq < 4; ++wq) {
                const uint32_t lo = kw[wq] & 0x0f0f0f0fu, hi = (kw[wq] >> 4) & 0x0f0f0f0fu;
                const uint32_t u01 = __byte_perm(lo, hi, 0x5140);   // (ch0, ch1, ch2, ch3) of this word
                const uint32_t u23 = __byte_perm(lo, hi, 0x7362);   // (ch4, ch5, ch6, ch7)
                mma_f16(sacc[nb], qf[4 * wq], 0u, qf[4 * wq + 1], 0u, nibs_to_h2<0x4140>(u01), nibs_to_h2<0x4342>(u01));
                mma_f16(sacc[nb], qf[4 * wq + 2], 0u, qf[4 * wq + 3], 0u, nibs_to_h2<0x4140>(u23), nibs_to_h2<0x4342>(u23));
            }
        }
        // scales of positions {2j, 2j+1} and {8+2j, 9+2j}
        const uint32_t* ksc = reinterpret_cast<const uint32_t*>(st + 2 * DA4_PAGE_BYTES);
        const uint32_t* vsc = reinterpret_cast<const uint32_t*>(st + 2 * DA4_PAGE_BYTES + 32);
        const float* kzp = reinterpret_cast<const float*>(st + 2 * DA4_PAGE_BYTES + 64);
        const float* vzp = reinterpret_cast<const float*>(st + 2 * DA4_PAGE_BYTES + 128);
        float ks0, ks1, ks2, ks3;
        bf16x2_to_f32(ksc[j], ks0, ks1);
        bf16x2_to_f32(ksc[4 + j], ks2, ks3);
        float t[4];
        const int pp[4] = {2 * j, 2 * j + 1, 8 + 2 * j, 9 + 2 * j};
        t[0] = (sacc[0][0] - kzp[pp[0]] * qsum) * (ks0 * qmul);
        t[1] = (sacc[0][1] - kzp[pp[1]] * qsum) * (ks1 * qmul);
        t[2] = (sacc[1][0] - kzp[pp[2]] * qsum) * (ks2 * qmul);
        t[3] = (sacc[1][1] - kzp[pp[3]] * qsum) * (ks3 * qmul);
        if (pos0 + PIKV_PAGE_TOKENS > len) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (pos0 + pp[c] >= len) t[c] = -INFINITY;
        }
        if (d.scores && r < G) {
            float* srow = d.scores + ((size_t)b * d.n_q + (size_t)h * G + r) * d.score_stride + pos0;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (pos0 + pp[c] < len && pos0 + pp[c] < d.score_stride) srow[pp[c]] = t[c] * 0.6931471805599453f;
        }
        // ---- online softmax (log2 domain) ----
        float mx = fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run - m_use);
        float p[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) p[c] = exp2f(t[c] - m_use);
        l_run = l_run * alpha + ((p[0] + p[1]) + (p[2] + p[3]));
        m_run = m_new;
        const uint32_t pb0 = pack_h2(p[0], p[1]), pb1 = pack_h2(p[2], p[3]);
        // rescale O: this thread's columns are query heads 2j and 2j+1
        const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * j) * 4);
        const float al1 = __shfl_sync(0xffffffffu, alpha, (2 * j + 1) * 4);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            o[m][0] *= al0; o[m][1] *= al1; o[m][2] *= al0; o[m][3] *= al1;
        }
        // ---- O^T += (Vcode * vscale)^T . P^T ----
        const unsigned char* vbase = st + DA4_PAGE_BYTES;
        // channels 16r .. 16r+15 of this thread's four positions: one 8-byte unit each
        uint2 v0 = *reinterpret_cast<const uint2*>(vbase + pp[0] * 64 + 8 * (r ^ (pp[0] & 4)));
        uint2 v1 = *reinterpret_cast<const uint2*>(vbase + pp[1] * 64 + 8 * (r ^ (pp[1] & 4)));
        uint2 v2 = *reinterpret_cast<const uint2*>(vbase + pp[2] * 64 + 8 * (r ^ (pp[2] & 4)));
        uint2 v3 = *reinterpret_cast<const uint2*>(vbase + pp[3] * 64 + 8 * (r ^ (pp[3] & 4)));
        const uint32_t vw[4][2] = {{v0.x, v0.y}, {v1.x, v1.y}, {v2.x, v2.y}, {v3.x, v3.y}};
        uint32_t vlo[4][2], vhi[4][2];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int wq = 0; wq < 2; ++wq) {
                vlo[c][wq] = vw[c][wq] & 0x0f0f0f0fu;            // even channels
                vhi[c][wq] = (vw[c][wq] >> 4) & 0x0f0f0f0fu;     // odd channels
            }
        float vs0, vs1, vs2, vs3;
        bf16x2_to_f32(vsc[j], vs0, vs1);
        bf16x2_to_f32(vsc[4 + j], vs2, vs3);
        const uint32_t vsa = pack_h2(vs0, vs1), vsb = pack_h2(vs2, vs3);
        // the zero-point term, with the probabilities as the tensor cores see them (rounded to f16)
        {
            const __half2 pa = *reinterpret_cast<const __half2*>(&pb0), pbh = *reinterpret_cast<const __half2*>(&pb1);
            const __half2 sa = *reinterpret_cast<const __half2*>(&vsa), sb = *reinterpret_cast<const __half2*>(&vsb);
            const float c_page = __low2float(pa) * __low2float(sa) * vzp[pp[0]] + __high2float(pa) * __high2float(sa) * vzp[pp[1]] +
                                 __low2float(pbh) * __low2float(sb) * vzp[pp[2]] + __high2float(pbh) * __high2float(sb) * vzp[pp[3]];
            corr = corr * alpha + c_page;
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            // byte m of the unit holds channels 16r+2m (low nibble) and 16r+2m+1 (high nibble)
            const int wq = m >> 2;
            const uint32_t sel = (m & 2) ? ((m & 1) ? 0x7373u : 0x6262u) : ((m & 1) ? 0x5151u : 0x4040u);
            const uint32_t ea = __byte_perm(vlo[0][wq], vlo[1][wq], sel);   // (p0, p1, p0, p1) of the even channel
            const uint32_t oa = __byte_perm(vhi[0][wq], vhi[1][wq], sel);
            const uint32_t eb = __byte_perm(vlo[2][wq], vlo[3][wq], sel);
            const uint32_t ob = __byte_perm(vhi[2][wq], vhi[3][wq], sel);
            const uint32_t a0 = hmul2_u32(nibs_to_h2<0x4140>(ea), vsa);   // channel 16r+2m,   positions 2j, 2j+1
            const uint32_t a1 = hmul2_u32(nibs_to_h2<0x4140>(oa), vsa);   // channel 16r+2m+1
            const uint32_t a2 = hmul2_u32(nibs_to_h2<0x4140>(eb), vsb);   // channel 16r+2m,   positions 8+2j, 9+2j
            const uint32_t a3 = hmul2_u32(nibs_to_h2<0x4140>(ob), vsb);
            mma_f16(o[m], a0, a1, a2, a3, pb0, pb1);
        }
        __syncwarp();
        if (lane == 0 && i + DA4_STAGES < my_pages) issue(i + DA4_STAGES);
    }
    if (timed_out) {
        // give the copies already issued one more bounded chance to land before the ring is reused
        if (lane == 0 && d.status) atomicOr(d.status, PIKV_ST_WAIT_TIMEOUT);
        for (int ii = i; ii < min(my_pages, i + DA4_STAGES); ++ii)
            (void)mbar_wait(bar0 + 8 * (ii % DA4_STAGES), (uint32_t)(ii / DA4_STAGES) & 1u);
    }

    // ---- zero-point term of P.V: per query head, the same for every channel ----
    corr += __shfl_xor_sync(0xffffffffu, corr, 1);
    corr += __shfl_xor_sync(0xffffffffu, corr, 2);
    {
        const float c0 = __shfl_sync(0xffffffffu, corr, (2 * j) * 4);
        const float c1 = __shfl_sync(0xffffffffu, corr, (2 * j + 1) * 4);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            o[m][0] -= c0; o[m][1] -= c1; o[m][2] -= c0; o[m][3] -= c1;
        }
    }
    // ---- merge the 4 warps ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();   // every warp is done with its ring; reuse it as the merge buffer
    float* mo = reinterpret_cast<float*>(smem);   // [warp][q][128]
    if (j == 0 && r < DA_MAX_GROUP) {
        ml_s[warp][r][0] = m_run;
        ml_s[warp][r][1] = l_run;
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
    s = min(s, max(1, pages / 32));   // at least 8 pages per warp
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
        const size_t smem = (size_t)DA_WARPS * DA_STAGES * DA_STAGE_BYTES + DA_WARPS * DA_STAGES * sizeof(uint64_t);
        if (cudaFuncSetAttribute(decode_attn_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_attn smem attribute");
        decode_attn_q8_kernel<<<grid, DA_THREADS, smem, st>>>(d);
    } else {
        const size_t smem = (size_t)DA_WARPS * DA4_STAGES * DA4_STAGE_BYTES + DA_WARPS * DA4_STAGES * sizeof(uint64_t);
        if (cudaFuncSetAttribute(decode_attn_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_attn smem attribute");
        decode_attn_q4_kernel<<<grid, DA_THREADS, smem, st>>>(d);
    }
    int launches = 1;
    int rc = check_launch(bits == 8 ? "decode_attn_q8_kernel" : "decode_attn_q4_kernel");
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

