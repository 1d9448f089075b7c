// Router gate for bf16 activations on tcgen05 tensor cores.
//
// logits[128 tokens, E] = act tile . w2^T is a skinny GEMM whose cost is reading the
// activations once (8 KiB per token at hidden 4096): TMA streams [128 x 64] activation
// tiles and [EP x 64] weight tiles (EP = E padded to 16/32/64, rows past E are zero-filled
// by TMA) through a shared-memory ring, one thread issues tcgen05.mma into a
// double-buffered accumulator in tensor memory, and four epilogue warps read one token
// row each (tcgen05.ld: all E logits of a token land in one thread's registers), so the
// softmax, top-k and renormalisation need no cross-thread traffic at all (up to 16 experts;
// above that E/16 warps share a row group, 16 columns per thread, see token_tail_wide).  Warp shuffles
// reduce the per-expert probability sums; ballots/match rank the (token, k) pairs of the
// CTA's chunk per expert.  The epilogue of tile i overlaps the loads and MMAs of tile i+1.
// The slot scan across CTAs is finished by gate_finalize_kernel (see gate.cu).
#include "gate_common.cuh"
#include "tc_common.cuh"

namespace pikv {

constexpr int GT_LOAD_THREADS = 64;      // warp 0 TMA, warp 1 MMA; 4 * Q epilogue warps follow
constexpr int GT_COLS = 16;              // expert columns per thread when Q > 1 threads share a token row

__device__ unsigned g_gate_tc_error = 0;

template <int Q>
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(128 * Q) : "memory"); }
// the Q warps that share the token rows of tensor-memory lane group lg (barriers 2..5; the number is an immediate
// so that the kernel claims six barriers, not all sixteen)
template <int Q, int ID>
__device__ __forceinline__ bool row_barrier_id(bool flag) {
    uint32_t out;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, %2, %3, q;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(out) : "r"((uint32_t)flag), "n"(ID), "n"(32 * Q) : "memory");
    return out != 0;
}
// barrier over a row group with an OR over a flag: its warps leave the tile loop together
template <int Q>
__device__ __forceinline__ bool row_barrier_any(int lg, bool flag) {
    switch (lg) {
        case 0: return row_barrier_id<Q, 2>(flag);
        case 1: return row_barrier_id<Q, 3>(flag);
        case 2: return row_barrier_id<Q, 4>(flag);
        default: return row_barrier_id<Q, 5>(flag);
    }
}
template <int Q>
__device__ __forceinline__ void row_barrier(int lg) {
    switch (lg) {
        case 0: asm volatile("bar.sync 2, %0;" ::"n"(32 * Q) : "memory"); break;
        case 1: asm volatile("bar.sync 3, %0;" ::"n"(32 * Q) : "memory"); break;
        case 2: asm volatile("bar.sync 4, %0;" ::"n"(32 * Q) : "memory"); break;
        default: asm volatile("bar.sync 5, %0;" ::"n"(32 * Q) : "memory"); break;
    }
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Shared memory of the epilogue when Q > 1 threads share a token: partial maxima and sums, and each
// thread's k best (probability, expert) of its 16 columns.
struct WideXchg {
    float* red;      // [2][Q][128]
    float* cval;     // [128][Q][k]
    uint8_t* cidx;   // [128][Q][k]
};

// Per-token tail for expert counts above 16: Q threads in Q warps of one lane group hold 16 logits each of
// token row `row`; they exchange the row maximum, the softmax denominator (partial sums added in column
// order) and their k best candidates, and the thread of column group 0 merges those and writes the
// routing outputs.  Same arithmetic per element as token_tail; every thread of the row group must call
// it (it synchronises), rows past the end of the batch pass valid = false and store nothing.  Leaves the
// probabilities of the thread's columns in l[].
template <int Q>
__device__ __forceinline__ void token_tail_wide(float (&l)[GT_COLS], const GateDev& g, int t, bool valid, int cg,
                                                int lg, int row, const WideXchg& x, uint8_t* sel_row) {
    const int E = g.E, e0 = cg * GT_COLS, k = g.k;
#pragma unroll
    for (int i = 0; i < GT_COLS; ++i) {
        const int e = e0 + i;
        if (e < E) {
            float v = l[i];
            if (g.temperature != 1.0f) v = __fdiv_rn(v, g.temperature);
            if (g.corr) v = __fmul_rn(v, g.corr[e]);
            if (g.mask_mode == PIKV_MASK_SINGLE)
                v = __fadd_rn(v, __fmul_rn(__fsub_rn(1.0f, g.mask[e]), -1e9f));
            else if (g.mask_mode == PIKV_MASK_MODULE)
                v = __fadd_rn(v, __fmul_rn(__fsub_rn(1.0f, g.mask[e]), -3.402823466e+38f));
            else if (g.mask_mode == PIKV_MASK_BIAS)
                v = __fadd_rn(v, g.mask[e]);
            l[i] = v;
        } else {
            l[i] = -INFINITY;
        }
    }
    float m = l[0];
#pragma unroll
    for (int i = 1; i < GT_COLS; ++i) m = fmaxf(m, l[i]);
    x.red[cg * 128 + row] = m;
    row_barrier<Q>(lg);
    m = x.red[row];
#pragma unroll
    for (int q = 1; q < Q; ++q) m = fmaxf(m, x.red[q * 128 + row]);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < GT_COLS; ++i) {
        const float p = (e0 + i < E) ? expf(l[i] - m) : 0.f;
        l[i] = p;
        s += p;
    }
    x.red[(Q + cg) * 128 + row] = s;
    row_barrier<Q>(lg);
    s = x.red[Q * 128 + row];
#pragma unroll
    for (int q = 1; q < Q; ++q) s += x.red[(Q + q) * 128 + row];
#pragma unroll
    for (int i = 0; i < GT_COLS; ++i) l[i] = __fdiv_rn(l[i], s);
    if (valid && g.probs) {
        if (E == Q * GT_COLS && (reinterpret_cast<uintptr_t>(g.probs) & 15) == 0) {
            float4* dst = reinterpret_cast<float4*>(g.probs + (size_t)t * E + e0);
#pragma unroll
            for (int i = 0; i < GT_COLS; i += 4) dst[i / 4] = make_float4(l[i], l[i + 1], l[i + 2], l[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < GT_COLS; ++i)
                if (e0 + i < E) g.probs[(size_t)t * E + e0 + i] = l[i];
        }
    }
    // the k best of this thread's columns; strict '>' keeps the lowest index on ties.  A thread with fewer than
    // k real columns pads with probability -1, which the merge never prefers to a real one.
    {
        unsigned taken = 0u;
        float* cv = x.cval + (size_t)(row * Q + cg) * k;
        uint8_t* ci = x.cidx + (size_t)(row * Q + cg) * k;
#pragma unroll
        for (int j = 0; j < GATE_MAX_K; ++j) {
            if (j < k) {
                float best = -1.f;
                int bi = 0;
#pragma unroll
                for (int i = 0; i < GT_COLS; ++i) {
                    if (e0 + i < E && !((taken >> i) & 1u) && l[i] > best) {
                        best = l[i];
                        bi = i;
                    }
                }
                taken |= 1u << bi;
                cv[j] = best;
                ci[j] = (uint8_t)(e0 + bi);
            }
        }
    }
    row_barrier<Q>(lg);
    if (cg == 0 && valid) {
        // candidates in (column group, rank) order: among equal probabilities the first one met has the lowest index
        const float* cv = x.cval + (size_t)row * Q * k;
        const uint8_t* ci = x.cidx + (size_t)row * Q * k;
        const int nc = Q * k;
        unsigned used = 0u;
        int idx[GATE_MAX_K];
        float val[GATE_MAX_K];
        float wsum = 0.f;
#pragma unroll
        for (int j = 0; j < GATE_MAX_K; ++j) {
            if (j < k) {
                float best = -2.f;
                int bc = 0;
                for (int c = 0; c < nc; ++c) {
                    const float v = cv[c];
                    if (!((used >> c) & 1u) && v > best) {
                        best = v;
                        bc = c;
                    }
                }
                used |= 1u << bc;
                idx[j] = ci[bc];
                val[j] = best;
                wsum += best;
            }
        }
        const float denom = __fadd_rn(wsum, g.eps);
#pragma unroll
        for (int j = 0; j < GATE_MAX_K; ++j) {
            if (j < k) {
                g.topk_idx[(size_t)t * k + j] = idx[j];
                if (g.topk_w) g.topk_w[(size_t)t * k + j] = __fdiv_rn(val[j], denom);
                sel_row[j] = (uint8_t)idx[j];
            }
        }
    }
}

struct GateTcArgs {
    GateDev g;
    int stages, tmem_cols, tiles, tiles_per_cta;
};

// EP: expert columns of the MMA (multiple of 16); EL <= EP: columns the per-token tail looks at (8 when E <= 8,
// which halves the serial softmax / top-k work of the epilogue warps); Q: epilogue warps per tensor-memory lane
// group.  With Q == 1 a thread owns a token row; above 16 experts that serial tail (one warp per scheduler) took
// longer than streaming the tile in, so Q = EL / 16 threads share a row, 16 columns each (token_tail_wide).
// Registers: 128 with one row per thread (without the cap the compiler stopped at 56 / 80 and spilled; the step of the
// pipelined schedule is 1 % faster without the spills); 96 with shared rows: 18 warps put five on one SM sub-partition
// of 16384 registers, so 112 compiles but does not launch.
template <int EP, int EL, int Q>
__global__ void __launch_bounds__(GT_LOAD_THREADS + 128 * Q) __maxnreg__(Q == 1 ? 128 : 96) gate_tc_kernel(const __grid_constant__ CUtensorMap tm_act,
                                                             const __grid_constant__ CUtensorMap tm_w,
                                                             GateTcArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (lr_smem_u32(smem_raw) & 1023u)) & 1023u);
    const GateDev& g = a.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int STAGE_A = LR_BM * LR_BK * 2;
    constexpr int STAGE_B = EP * LR_BK * 2;
    constexpr int STAGE = STAGE_A + STAGE_B;
    unsigned char* after_ring = smem + (size_t)a.stages * STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(after_ring);
    const uint32_t full0 = lr_smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * a.stages;
    const uint32_t tfull0 = empty0 + 8 * a.stages;       // [2] accumulator ready
    const uint32_t tempty0 = tfull0 + 16;                // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * a.stages + 4);
    static_assert(Q == 1 || EL == Q * GT_COLS, "a thread of a shared row owns 16 columns");
    constexpr int EPI = 128 * Q, EPI_WARPS = 4 * Q;
    int* warp_cnt = reinterpret_cast<int*>(tmem_slot + 4);           // [EPI_WARPS][EP]
    int* run = warp_cnt + EPI_WARPS * EP;                            // [EP]
    int* cnt_k = run + EP;                                           // [K][EP]
    float* psum_w = reinterpret_cast<float*>(cnt_k + GATE_MAX_K * EP);   // [4 lane groups][EP]
    WideXchg xc;
    xc.red = psum_w + 4 * EP;                                        // Q > 1 only: [2][Q][128]
    xc.cval = xc.red + (Q > 1 ? 2 * Q * 128 : 0);                    // [128][Q][k]
    xc.cidx = reinterpret_cast<uint8_t*>(xc.cval + (Q > 1 ? 128 * Q * g.k : 0));
    uint8_t* sel = xc.cidx + (Q > 1 ? 128 * Q * g.k : 0);            // [chunk * k]
    const uint32_t ring = lr_smem_u32(smem);

    const int tile0 = blockIdx.x * a.tiles_per_cta;
    const int ntiles = max(0, min(a.tiles_per_cta, a.tiles - tile0));
    const int num_kb = (g.H + LR_BK - 1) / LR_BK;
    const int chunk_start = blockIdx.x * g.chunk;
    const int ntok = max(0, min(g.chunk, g.T - chunk_start));

    if (threadIdx.x == 0) {
        tmem_slot[1] = 0;   // set by any epilogue thread whose wait ran out
        for (int s = 0; s < a.stages; ++s) {
            lr_mbar_init(full0 + 8 * s, 1);
            lr_mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            lr_mbar_init(tfull0 + 8 * s, 1);
            lr_mbar_init(tempty0 + 8 * s, EPI);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        lr_prefetch_tmap(&tm_act);
        lr_prefetch_tmap(&tm_w);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(lr_smem_u32(tmem_slot)), "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;
    // a kernel launched as a programmatic dependent of this one (the fused append) may be scheduled from here on;
    // it waits for this grid's completion before it reads anything written here.  (This kernel itself is launched
    // the plain way: as a programmatic dependent of the previous batch's gate its waiting CTAs kept the SMs' registers
    // busy, the append kernel of the pipelined schedule then ran in two waves, and the step got 4 % slower.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int lt = 0; lt < ntiles && !failed; ++lt) {
                const int m0 = (tile0 + lt) * LR_BM;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % a.stages;
                    const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
                    if (!lr_mbar_wait(empty0 + 8 * s, ph ^ 1u)) { failed = true; break; }
                    lr_mbar_expect_tx(full0 + 8 * s, (uint32_t)STAGE);
                    const uint32_t dst = ring + (uint32_t)s * STAGE;
                    lr_tma_load_2d(dst, &tm_act, kb * LR_BK, m0, full0 + 8 * s);
                    lr_tma_load_2d(dst + STAGE_A, &tm_w, kb * LR_BK, 0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = lr_instr_desc(EP);
            int it = 0;
            for (int lt = 0; lt < ntiles && !failed; ++lt) {
                const int slot = lt & 1;
                if (!lr_mbar_wait(tempty0 + 8 * slot, (((uint32_t)lt >> 1) & 1u) ^ 1u)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(slot * EP);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % a.stages;
                    const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
                    if (!lr_mbar_wait(full0 + 8 * s, ph)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = ring + (uint32_t)s * STAGE;
                    const uint32_t sb = sa + STAGE_A;
#pragma unroll
                    for (int k = 0; k < LR_BK / 16; ++k)
                        lr_mma(d_tmem, lr_smem_desc(sa + 32 * k), lr_smem_desc(sb + 32 * k), idesc, (kb | k) ? 1u : 0u);
                    lr_commit(empty0 + 8 * s);
                }
                lr_commit(tfull0 + 8 * slot);
            }
        }
    } else {
        const int et = threadIdx.x - GT_LOAD_THREADS; // index among the epilogue threads
        const int ew = et >> 5;
        const int lg = warp & 3;                      // tensor-memory lane group of this warp
        const int cg = ew >> 2;                       // column group (Q > 1)
        const int row = lg * 32 + lane;               // token row inside a tile
        constexpr int CL = Q == 1 ? EL : GT_COLS;     // logits per thread
        for (int i = et; i < 4 * EP; i += EPI) psum_w[i] = 0.f;
        // the bias is needed the moment the first accumulator arrives: its loads go out now
        float bias[CL];
#pragma unroll
        for (int e = 0; e < CL; ++e) bias[e] = (g.b2 && cg * CL + e < g.E) ? __ldg(g.b2 + cg * CL + e) : 0.f;
        epi_barrier<Q>();
        for (int lt = 0; lt < ntiles; ++lt) {
            const int slot = lt & 1;
            if (!lr_mbar_wait(tfull0 + 8 * slot, ((uint32_t)lt >> 1) & 1u)) failed = true;
            if (Q > 1) failed = row_barrier_any<Q>(lg, failed);   // the warps of a row group go on, or give up, together
            if (failed) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float l[CL];
#pragma unroll
            for (int c = 0; c < CL; c += 16) {
                float v[16];
                lr_tmem_ld16(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(slot * EP + cg * CL + c), v);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (c + i < CL) l[c + i] = v[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(tempty0 + 8 * slot);          // this thread's part of the row is out of tensor memory
            const int lt_tok = lt * LR_BM + row;      // token index inside the chunk
            const bool valid = lt_tok < ntok;
#pragma unroll
            for (int e = 0; e < CL; ++e) l[e] += bias[e];
            if constexpr (Q == 1) {
                if (valid) token_tail<EL>(l, g, chunk_start + lt_tok, sel + (size_t)lt_tok * g.k);
            } else {
                token_tail_wide<Q>(l, g, chunk_start + lt_tok, valid, cg, lg, row, xc, sel + (size_t)lt_tok * g.k);
            }
#pragma unroll
            for (int e = 0; e < CL; ++e) {
                const float s = warp_sum(valid ? l[e] : 0.f);
                if (lane == 0) psum_w[lg * EP + cg * CL + e] += s;
            }
        }
        if (failed) atomicOr(tmem_slot + 1, 1u);
        epi_barrier<Q>();
        const bool any_failed = tmem_slot[1] != 0;   // identical in all 128 threads from here on
        if (et < g.E) {
            // fixed order: lane groups 0..3 hold token rows 0-31, 32-63, ... of every tile
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) s += psum_w[q * EP + et];
            g.cta_psum[(size_t)blockIdx.x * g.E + et] = s;
        }
        // ---- rank the chunk's (token, k) pairs per expert, in order (all epilogue threads) ----
        const int npairs = any_failed ? 0 : ntok * g.k;
        for (int i = et; i < EP; i += EPI) run[i] = 0;
        for (int i = et; i < GATE_MAX_K * EP; i += EPI) cnt_k[i] = 0;
        epi_barrier<Q>();
        for (int base = 0; base < npairs; base += EPI) {
            for (int i = et; i < EPI_WARPS * EP; i += EPI) warp_cnt[i] = 0;
            epi_barrier<Q>();
            const int p = base + et;
            const bool valid = p < npairs;
            const int e = valid ? (int)sel[p] : 255;
            const unsigned peers = __match_any_sync(0xffffffffu, e);
            const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
            if (valid && rank_in_warp == 0) warp_cnt[ew * EP + e] = __popc(peers);
            if (valid) atomicAdd(&cnt_k[(p % g.k) * EP + e], 1);
            epi_barrier<Q>();
            if (valid) {
                int r = run[e] + rank_in_warp;
                for (int w = 0; w < ew; ++w) r += warp_cnt[w * EP + e];
                if (g.slot) g.slot[(size_t)chunk_start * g.k + p] = r;
            }
            epi_barrier<Q>();
            if (et < EP) {
                int add = 0;
#pragma unroll
                for (int w = 0; w < EPI_WARPS; ++w) add += warp_cnt[w * EP + et];
                run[et] += add;
            }
            epi_barrier<Q>();
        }
        for (int e = et; e < g.E; e += EPI) g.cta_cnt[(size_t)blockIdx.x * g.E + e] = run[e];
        for (int i = et; i < g.k * g.E; i += EPI) {
            const int j = i / g.E, e = i % g.E;
            g.cta_cnt_k[((size_t)blockIdx.x * g.k + j) * g.E + e] = cnt_k[j * EP + e];
        }
    }
    if (failed) atomicOr(&g_gate_tc_error, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

// one CTA per 128-token tile until the grid limit, then whole tiles per CTA
void gate_tc_geometry(GateDev& g) {
    const int tiles = ceil_div(g.T, LR_BM);
    g.chunk = ceil_div(tiles, GATE_MAX_CTAS) * LR_BM;
    g.G = ceil_div(g.T, g.chunk);
}

template <int EP, int EL, int Q>
static int launch_gate_tc(GateDev& g, cudaStream_t st) {
    GateTcArgs a;
    gate_tc_geometry(g);
    a.tiles = ceil_div(g.T, LR_BM);
    a.tiles_per_cta = g.chunk / LR_BM;
    a.g = g;
    CUtensorMap tm_act, tm_w;
    int rc = make_tmap(&tm_act, g.act, g.T, g.H, LR_BM);
    if (rc != PIKV_OK) return rc;
    rc = make_tmap(&tm_w, g.w2, g.E, g.H, EP);
    if (rc != PIKV_OK) return rc;
    const int stage = LR_BM * LR_BK * 2 + EP * LR_BK * 2;
    // barriers, tensor-memory slot, rank counters, probability sums, (Q > 1) the row exchange, selections, alignment slack
    const size_t xchg = Q > 1 ? sizeof(float) * 2 * Q * 128 + (size_t)128 * Q * g.k * (sizeof(float) + 1) : 0;
    const size_t tail = (2 * 8 + 4) * sizeof(uint64_t) + 16 + sizeof(int) * (4 * Q * EP + EP + GATE_MAX_K * EP) +
                        sizeof(float) * 4 * EP + xchg + (size_t)g.chunk * g.k + 1024;
    // one CTA per SM when the grid fits in one wave (or the registers of 16 epilogue warps leave room for one only), two otherwise
    const size_t budget = ((g.G <= sm_count() || Q >= 4) ? 200 * 1024 : 100 * 1024) - tail;
    a.stages = (int)max((size_t)2, min((size_t)8, budget / stage));
    int cols = 32;
    while (cols < 2 * EP) cols <<= 1;
    a.tmem_cols = cols;
    const size_t smem = (size_t)a.stages * stage + tail;
    auto kern = gate_tc_kernel<EP, EL, Q>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("gate_tc smem attribute");
    kern<<<g.G, GT_LOAD_THREADS + 128 * Q, smem, st>>>(tm_act, tm_w, a);
    return check_launch("gate_tc_kernel");
}

// true when the tensor-core path can take this problem
bool gate_tc_supported(const GateDev& g, int dtype) {
    return g.act != nullptr && dtype == PIKV_BF16 && g.H % 8 == 0 && g.H >= 16 &&
           ((uintptr_t)g.act % 16) == 0 && ((uintptr_t)g.w2 % 16) == 0;
}

int gate_tc_launch(GateDev& g, cudaStream_t st) {
    if (g.E <= 8) return launch_gate_tc<16, 8, 1>(g, st);
    if (g.E <= 16) return launch_gate_tc<16, 16, 1>(g, st);
    if (g.E <= 32) return launch_gate_tc<32, 32, 2>(g, st);
    return launch_gate_tc<64, 64, 4>(g, st);
}

}  // namespace pikv

namespace pikv { int gate_mlp_error_fetch(); }

// reads and clears the sticky error words of the tensor-core gate kernels
extern "C" int pikv_gate_error_state(void) {
    unsigned v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, pikv::g_gate_tc_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(pikv::g_gate_tc_error, &zero, sizeof(zero));
    const int m = pikv::gate_mlp_error_fetch();
    if (m < 0) return -1;
    return (int)v | m;
}
