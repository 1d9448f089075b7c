// Router gate for bf16 activations on tcgen05 tensor cores.
//
// logits[128 tokens, E] = act tile . w2^T is a skinny GEMM whose cost is reading the
// activations once (8 KiB per token at hidden 4096): TMA streams [128 x 64] activation
// tiles and [EP x 64] weight tiles (EP = E padded to 16/32/64, rows past E are zero-filled
// by TMA) through a shared-memory ring, one thread issues tcgen05.mma into a
// double-buffered accumulator in tensor memory, and four epilogue warps read one token
// row each (tcgen05.ld: all E logits of a token land in one thread's registers), so the
// softmax, top-k and renormalisation need no cross-thread traffic at all.  Warp shuffles
// reduce the per-expert probability sums; ballots/match rank the (token, k) pairs of the
// CTA's chunk per expert.  The epilogue of tile i overlaps the loads and MMAs of tile i+1.
// The slot scan across CTAs is finished by gate_finalize_kernel (see gate.cu).
#include "gate_common.cuh"
#include "tc_common.cuh"

namespace pikv {

constexpr int GT_THREADS = 192;          // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int GT_EPI = 128;
constexpr int GT_EPI_WARPS = 4;

__device__ unsigned g_gate_tc_error = 0;

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

struct GateTcArgs {
    GateDev g;
    int stages, tmem_cols, tiles, tiles_per_cta;
};

// EP: expert columns of the MMA (multiple of 16); EL <= EP: columns the per-token tail looks at (8 when E <= 8,
// which halves the serial softmax / top-k work of the four epilogue warps)
template <int EP, int EL>
__global__ void __launch_bounds__(GT_THREADS) gate_tc_kernel(const __grid_constant__ CUtensorMap tm_act,
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
    int* warp_cnt = reinterpret_cast<int*>(tmem_slot + 4);           // [4][EP]
    int* run = warp_cnt + GT_EPI_WARPS * EP;                         // [EP]
    int* cnt_k = run + EP;                                           // [K][EP]
    float* psum_w = reinterpret_cast<float*>(cnt_k + GATE_MAX_K * EP);   // [4][EP]
    uint8_t* sel = reinterpret_cast<uint8_t*>(psum_w + GT_EPI_WARPS * EP);   // [chunk * k]
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
            lr_mbar_init(tempty0 + 8 * s, GT_EPI);
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
        const int et = threadIdx.x - 64;              // 0..127 among the epilogue threads
        const int ew = et >> 5;
        const int lg = warp & 3;                      // tensor-memory lane group of this warp
        const int row = lg * 32 + lane;               // token row inside a tile
        for (int i = et; i < GT_EPI_WARPS * EP; i += GT_EPI) psum_w[i] = 0.f;
        // the bias is needed the moment the first accumulator arrives: its loads go out now
        float bias[EL];
#pragma unroll
        for (int e = 0; e < EL; ++e) bias[e] = (g.b2 && e < g.E) ? __ldg(g.b2 + e) : 0.f;
        epi_barrier();
        for (int lt = 0; lt < ntiles; ++lt) {
            const int slot = lt & 1;
            if (!lr_mbar_wait(tfull0 + 8 * slot, ((uint32_t)lt >> 1) & 1u)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float l[EL];
#pragma unroll
            for (int c = 0; c < EL; c += 16) {
                float v[16];
                lr_tmem_ld16(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(slot * EP + c), v);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (c + i < EL) l[c + i] = v[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(tempty0 + 8 * slot);          // this thread's row is out of tensor memory
            const int lt_tok = lt * LR_BM + row;      // token index inside the chunk
            const bool valid = lt_tok < ntok;
            if (valid) {
#pragma unroll
                for (int e = 0; e < EL; ++e) l[e] += bias[e];
                token_tail<EL>(l, g, chunk_start + lt_tok, sel + (size_t)lt_tok * g.k);
            }
#pragma unroll
            for (int e = 0; e < EL; ++e) {
                const float s = warp_sum(valid ? l[e] : 0.f);
                if (lane == 0) psum_w[ew * EP + e] += s;
            }
        }
        if (failed) atomicOr(tmem_slot + 1, 1u);
        epi_barrier();
        const bool any_failed = tmem_slot[1] != 0;   // identical in all 128 threads from here on
        if (et < g.E) {
            // fixed order: lane groups 0..3 hold token rows 0-31, 32-63, ... of every tile
            float s = 0.f;
            const int order[4] = {2, 3, 0, 1};        // epilogue warp index holding lane group 0,1,2,3
#pragma unroll
            for (int q = 0; q < 4; ++q) s += psum_w[order[q] * EP + et];
            g.cta_psum[(size_t)blockIdx.x * g.E + et] = s;
        }
        // ---- rank the chunk's (token, k) pairs per expert, in order (128 threads) ----
        const int npairs = any_failed ? 0 : ntok * g.k;
        for (int i = et; i < EP; i += GT_EPI) run[i] = 0;
        for (int i = et; i < GATE_MAX_K * EP; i += GT_EPI) cnt_k[i] = 0;
        epi_barrier();
        for (int base = 0; base < npairs; base += GT_EPI) {
            for (int i = et; i < GT_EPI_WARPS * EP; i += GT_EPI) warp_cnt[i] = 0;
            epi_barrier();
            const int p = base + et;
            const bool valid = p < npairs;
            const int e = valid ? (int)sel[p] : 255;
            const unsigned peers = __match_any_sync(0xffffffffu, e);
            const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
            if (valid && rank_in_warp == 0) warp_cnt[ew * EP + e] = __popc(peers);
            if (valid) atomicAdd(&cnt_k[(p % g.k) * EP + e], 1);
            epi_barrier();
            if (valid) {
                int r = run[e] + rank_in_warp;
                for (int w = 0; w < ew; ++w) r += warp_cnt[w * EP + e];
                if (g.slot) g.slot[(size_t)chunk_start * g.k + p] = r;
            }
            epi_barrier();
            if (et < EP) {
                int add = 0;
#pragma unroll
                for (int w = 0; w < GT_EPI_WARPS; ++w) add += warp_cnt[w * EP + et];
                run[et] += add;
            }
            epi_barrier();
        }
        for (int e = et; e < g.E; e += GT_EPI) g.cta_cnt[(size_t)blockIdx.x * g.E + e] = run[e];
        for (int i = et; i < g.k * g.E; i += GT_EPI) {
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

template <int EP, int EL>
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
    const size_t tail = (2 * 8 + 4) * sizeof(uint64_t) + 16 + sizeof(int) * (GT_EPI_WARPS * EP + EP + GATE_MAX_K * EP) +
                        sizeof(float) * GT_EPI_WARPS * EP + (size_t)g.chunk * g.k + 1024;
    // one CTA per SM when the grid fits in one wave, two otherwise
    const size_t budget = (g.G <= sm_count() ? 200 * 1024 : 100 * 1024) - tail;
    a.stages = (int)max((size_t)2, min((size_t)8, budget / stage));
    int cols = 32;
    while (cols < 2 * EP) cols <<= 1;
    a.tmem_cols = cols;
    const size_t smem = (size_t)a.stages * stage + tail;
    auto kern = gate_tc_kernel<EP, EL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("gate_tc smem attribute");
    kern<<<g.G, GT_THREADS, smem, st>>>(tm_act, tm_w, a);
    return check_launch("gate_tc_kernel");
}

// true when the tensor-core path can take this problem
bool gate_tc_supported(const GateDev& g, int dtype) {
    return g.act != nullptr && dtype == PIKV_BF16 && g.H % 8 == 0 && g.H >= 16 &&
           ((uintptr_t)g.act % 16) == 0 && ((uintptr_t)g.w2 % 16) == 0;
}

int gate_tc_launch(GateDev& g, cudaStream_t st) {
    if (g.E <= 8) return launch_gate_tc<16, 8>(g, st);
    if (g.E <= 16) return launch_gate_tc<16, 16>(g, st);
    if (g.E <= 32) return launch_gate_tc<32, 32>(g, st);
    return launch_gate_tc<64, 64>(g, st);
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
