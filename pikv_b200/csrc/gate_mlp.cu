// The whole gate net of the router in one kernel, on tcgen05 tensor cores:
//   logits[T,E] = relu(x[T,K] . w1[H1,K]^T + b1) . w2[E,H1]^T + b2      (core/single/pikv_routing.py:34-38)
// followed by the per-token tail of the gate (softmax, top-k, renormalisation, ranks) exactly as gate_tc.cu
// does it.  The hidden activations [T,H1] never exist in HBM: a CTA owns 128 tokens and walks the hidden
// units in chunks of 256.  Per chunk
//   warp 0   TMA: [128 x 64] tiles of x and [256 x 64] tiles of w1 through a shared-memory ring, and the
//            [EP x 256] slice of w2 (double-buffered)
//   warp 1   one thread issues tcgen05.mma: GEMM1 (M=128, N=256, K=16 per instruction) into tensor-memory
//            columns 0..255, then - one chunk behind, so that it never waits for the epilogue - GEMM2
//            (M=128, N=EP) from the chunk's ReLU'd activations in shared memory into columns 256..
//   warps 2-5  drain GEMM1's accumulator (tcgen05.ld), add b1, ReLU, round to bf16 and store the chunk as
//            the K-major, 128-byte-swizzled A operand of GEMM2; after the last chunk read the 128 logit rows
//            and run the gate tail
// Reads x once from HBM (w1 is shared by all CTAs through L2).  Every mbarrier wait is bounded; on a timeout
// the CTA raises the gate's sticky error word and drains.
#include "gate_common.cuh"
#include "tc_common.cuh"

namespace pikv {

constexpr int GM_THREADS = 192;
constexpr int GM_EPI = 128;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_BN = 256;                 // hidden units per chunk
constexpr int GM_KB_PER_CHUNK = GM_BN / LR_BK;   // 4 k-blocks of GEMM2 per chunk

__device__ unsigned g_gate_mlp_error = 0;   // sticky: a bounded wait of gate_mlp_kernel ran out

__device__ __forceinline__ void gm_epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void gm_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

struct GateMlpArgs {
    GateDev g;              // g.H = H1 (inputs of the second layer), g.w2 / g.b2 = second layer
    const float* b1;        // [H1] or null
    int K;                  // inputs of the first layer
    int stages, chunks;
};

template <int EP, int EL>
__global__ void __launch_bounds__(GM_THREADS) gate_mlp_kernel(const __grid_constant__ CUtensorMap tm_x,
                                                              const __grid_constant__ CUtensorMap tm_w1,
                                                              const __grid_constant__ CUtensorMap tm_w2, GateMlpArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (lr_smem_u32(smem_raw) & 1023u)) & 1023u);
    const GateDev& g = a.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int STAGE_A = LR_BM * LR_BK * 2;            // 16 KB
    constexpr int STAGE_B = GM_BN * LR_BK * 2;            // 32 KB
    constexpr int STAGE = STAGE_A + STAGE_B;
    constexpr int H_TILE = LR_BM * LR_BK * 2;             // one k-block of the hidden chunk: 16 KB
    constexpr int W2_KB = EP * LR_BK * 2;                 // one k-block of the w2 slice
    constexpr int W2_BUF = GM_KB_PER_CHUNK * W2_KB;
    unsigned char* hbuf = smem + (size_t)a.stages * STAGE;            // [4][128 x 64] bf16, 1024-aligned
    unsigned char* w2buf = hbuf + GM_KB_PER_CHUNK * H_TILE;           // [2][4][EP x 64] bf16
    uint64_t* bars = reinterpret_cast<uint64_t*>(w2buf + 2 * W2_BUF);
    const uint32_t full0 = lr_smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * a.stages;
    const uint32_t d1_full = empty0 + 8 * a.stages, d1_empty = d1_full + 8;
    const uint32_t h_full = d1_empty + 8, h_empty = h_full + 8;
    const uint32_t w2_full0 = h_empty + 8, w2_empty0 = w2_full0 + 16;    // [2] each
    const uint32_t d2_full = w2_empty0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * a.stages + 9);
    int* warp_cnt = reinterpret_cast<int*>(tmem_slot + 4);               // [4][EP]
    int* run = warp_cnt + GM_EPI_WARPS * EP;                             // [EP]
    int* cnt_k = run + EP;                                               // [K][EP]
    float* psum_w = reinterpret_cast<float*>(cnt_k + GATE_MAX_K * EP);   // [4][EP]
    uint8_t* sel = reinterpret_cast<uint8_t*>(psum_w + GM_EPI_WARPS * EP);   // [128 * k]
    const uint32_t ring = lr_smem_u32(smem);
    const uint32_t hbuf_s = lr_smem_u32(hbuf), w2buf_s = lr_smem_u32(w2buf);

    const int m0 = blockIdx.x * LR_BM;
    const int ntok = max(0, min(LR_BM, g.T - m0));
    const int num_kb = (a.K + LR_BK - 1) / LR_BK;
    const int NC = a.chunks;

    if (threadIdx.x == 0) {
        tmem_slot[1] = 0;
        for (int s = 0; s < a.stages; ++s) {
            lr_mbar_init(full0 + 8 * s, 1);
            lr_mbar_init(empty0 + 8 * s, 1);
        }
        lr_mbar_init(d1_full, 1);
        lr_mbar_init(d1_empty, GM_EPI);
        lr_mbar_init(h_full, GM_EPI);
        lr_mbar_init(h_empty, 1);
        for (int b = 0; b < 2; ++b) {
            lr_mbar_init(w2_full0 + 8 * b, 1);
            lr_mbar_init(w2_empty0 + 8 * b, 1);
        }
        lr_mbar_init(d2_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        lr_prefetch_tmap(&tm_x);
        lr_prefetch_tmap(&tm_w1);
        lr_prefetch_tmap(&tm_w2);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(lr_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t d1_tmem = tmem_base, d2_tmem = tmem_base + GM_BN;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int n = 0; n < NC && !failed; ++n) {
                // this chunk's slice of w2 (buffer n & 1, last used by chunk n - 2)
                const int b = n & 1;
                if (!lr_mbar_wait(w2_empty0 + 8 * b, (((uint32_t)n >> 1) & 1u) ^ 1u)) { failed = true; break; }
                lr_mbar_expect_tx(w2_full0 + 8 * b, (uint32_t)W2_BUF);
                for (int q = 0; q < GM_KB_PER_CHUNK; ++q)
                    lr_tma_load_2d(w2buf_s + (uint32_t)(b * W2_BUF + q * W2_KB), &tm_w2, n * GM_BN + q * LR_BK, 0, w2_full0 + 8 * b);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % a.stages;
                    const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
                    if (!lr_mbar_wait(empty0 + 8 * s, ph ^ 1u)) { failed = true; break; }
                    lr_mbar_expect_tx(full0 + 8 * s, (uint32_t)STAGE);
                    const uint32_t dst = ring + (uint32_t)s * STAGE;
                    lr_tma_load_2d(dst, &tm_x, kb * LR_BK, m0, full0 + 8 * s);
                    lr_tma_load_2d(dst + STAGE_A, &tm_w1, kb * LR_BK, n * GM_BN, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc1 = lr_instr_desc(GM_BN), idesc2 = lr_instr_desc(EP);
            // second product of chunk n: its ReLU'd activations (shared memory) times its slice of w2
            auto gemm2 = [&](int n) -> bool {
                const int b = n & 1;
                if (!lr_mbar_wait(h_full, (uint32_t)n & 1u)) return false;
                if (!lr_mbar_wait(w2_full0 + 8 * b, ((uint32_t)n >> 1) & 1u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int q = 0; q < GM_KB_PER_CHUNK; ++q)
#pragma unroll
                    for (int k = 0; k < LR_BK / 16; ++k)
                        lr_mma(d2_tmem, lr_smem_desc(hbuf_s + (uint32_t)(q * H_TILE + 32 * k)),
                               lr_smem_desc(w2buf_s + (uint32_t)(b * W2_BUF + q * W2_KB + 32 * k)), idesc2, (n | q | k) ? 1u : 0u);
                lr_commit(h_empty);
                lr_commit(w2_empty0 + 8 * b);
                return true;
            };
            int it = 0;
            for (int n = 0; n < NC && !failed; ++n) {
                if (!lr_mbar_wait(d1_empty, ((uint32_t)n & 1u) ^ 1u)) { failed = true; break; }   // chunk n-1 is out of columns 0..255
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % a.stages;
                    const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
                    if (!lr_mbar_wait(full0 + 8 * s, ph)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = ring + (uint32_t)s * STAGE;
                    const uint32_t sb = sa + STAGE_A;
#pragma unroll
                    for (int k = 0; k < LR_BK / 16; ++k)
                        lr_mma(d1_tmem, lr_smem_desc(sa + 32 * k), lr_smem_desc(sb + 32 * k), idesc1, (kb | k) ? 1u : 0u);
                    lr_commit(empty0 + 8 * s);
                }
                if (failed) break;
                lr_commit(d1_full);
                if (n >= 1 && !gemm2(n - 1)) { failed = true; break; }
            }
            if (!failed && NC >= 1 && !gemm2(NC - 1)) failed = true;
            lr_commit(d2_full);                        // the logits are complete (or as far as they got)
        }
    } else {
        const int et = threadIdx.x - 64;              // 0..127 among the epilogue threads
        const int ew = et >> 5;
        const int lg = warp & 3;                      // tensor-memory lane group of this warp
        const int row = lg * 32 + lane;               // token row inside the tile
        for (int i = et; i < GM_EPI_WARPS * EP; i += GM_EPI) psum_w[i] = 0.f;
        gm_epi_barrier();
        for (int n = 0; n < NC && !failed; ++n) {
            if (!lr_mbar_wait(d1_full, (uint32_t)n & 1u)) { failed = true; break; }
            if (!lr_mbar_wait(h_empty, ((uint32_t)n & 1u) ^ 1u)) { failed = true; break; }     // GEMM2 of chunk n-1 has read the buffer
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int q = 0; q < GM_KB_PER_CHUNK; ++q) {
                uint32_t pk[32];                      // 64 hidden units of this token, bf16 pairs
#pragma unroll
                for (int c = 0; c < 64; c += 16) {
                    float v[16];
                    lr_tmem_ld16(d1_tmem + ((uint32_t)(lg * 32) << 16) + (uint32_t)(q * 64 + c), v);
                    const int h0 = n * GM_BN + q * 64 + c;
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        float x0 = v[i], x1 = v[i + 1];
                        if (a.b1) {
                            if (h0 + i < g.H) x0 += __ldg(a.b1 + h0 + i);
                            if (h0 + i + 1 < g.H) x1 += __ldg(a.b1 + h0 + i + 1);
                        }
                        x0 = fmaxf(x0, 0.f);
                        x1 = fmaxf(x1, 0.f);
                        pk[(c + i) >> 1] = (uint32_t)f32_to_bf16_bits(x0) | ((uint32_t)f32_to_bf16_bits(x1) << 16);
                    }
                }
                if (q == GM_KB_PER_CHUNK - 1) {
                    // every column of this row has left tensor memory: GEMM1 of the next chunk may start
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    gm_mbar_arrive(d1_empty);
                }
                // K-major tile with the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)
                unsigned char* hrow = hbuf + (size_t)q * H_TILE + (size_t)row * 128;
#pragma unroll
                for (int c16 = 0; c16 < 8; ++c16)
                    *reinterpret_cast<uint4*>(hrow + 16 * (c16 ^ (row & 7))) =
                        make_uint4(pk[4 * c16], pk[4 * c16 + 1], pk[4 * c16 + 2], pk[4 * c16 + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stores are for the tensor cores to read
            gm_mbar_arrive(h_full);
        }
        // ---- the logits of this thread's token, then the gate tail ----
        if (!failed && !lr_mbar_wait(d2_full, 0)) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float l[EL];
#pragma unroll
        for (int c = 0; c < EL; c += 16) {
            float v[16];
            lr_tmem_ld16(d2_tmem + ((uint32_t)(lg * 32) << 16) + (uint32_t)c, v);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (c + i < EL) l[c + i] = v[i];
        }
        const bool valid = row < ntok && !failed;
        if (valid) {
            if (g.b2) {
#pragma unroll
                for (int e = 0; e < EL; ++e)
                    if (e < g.E) l[e] += __ldg(g.b2 + e);
            }
            token_tail<EL>(l, g, m0 + row, sel + (size_t)row * g.k);
        }
#pragma unroll
        for (int e = 0; e < EL; ++e) {
            const float s = warp_sum(valid ? l[e] : 0.f);
            if (lane == 0) psum_w[ew * EP + e] += s;
        }
        if (failed) atomicOr(tmem_slot + 1, 1u);
        gm_epi_barrier();
        const bool any_failed = tmem_slot[1] != 0;
        if (et < g.E) {
            float s = 0.f;
            const int order[4] = {2, 3, 0, 1};        // epilogue warp index holding lane group 0,1,2,3
#pragma unroll
            for (int q = 0; q < 4; ++q) s += psum_w[order[q] * EP + et];
            g.cta_psum[(size_t)blockIdx.x * g.E + et] = s;
        }
        // ---- rank the tile's (token, k) pairs per expert, in order (128 threads) ----
        const int npairs = any_failed ? 0 : ntok * g.k;
        for (int i = et; i < EP; i += GM_EPI) run[i] = 0;
        for (int i = et; i < GATE_MAX_K * EP; i += GM_EPI) cnt_k[i] = 0;
        gm_epi_barrier();
        for (int base = 0; base < npairs; base += GM_EPI) {
            for (int i = et; i < GM_EPI_WARPS * EP; i += GM_EPI) warp_cnt[i] = 0;
            gm_epi_barrier();
            const int p = base + et;
            const bool pv = p < npairs;
            const int e = pv ? (int)sel[p] : 255;
            const unsigned peers = __match_any_sync(0xffffffffu, e);
            const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
            if (pv && rank_in_warp == 0) warp_cnt[ew * EP + e] = __popc(peers);
            if (pv) atomicAdd(&cnt_k[(p % g.k) * EP + e], 1);
            gm_epi_barrier();
            if (pv) {
                int rk = run[e] + rank_in_warp;
                for (int w = 0; w < ew; ++w) rk += warp_cnt[w * EP + e];
                if (g.slot) g.slot[(size_t)m0 * g.k + p] = rk;
            }
            gm_epi_barrier();
            if (et < EP) {
                int add = 0;
#pragma unroll
                for (int w = 0; w < GM_EPI_WARPS; ++w) add += warp_cnt[w * EP + et];
                run[et] += add;
            }
            gm_epi_barrier();
        }
        for (int e = et; e < g.E; e += GM_EPI) g.cta_cnt[(size_t)blockIdx.x * g.E + e] = run[e];
        for (int i = et; i < g.k * g.E; i += GM_EPI) {
            const int jj = i / g.E, e = i % g.E;
            g.cta_cnt_k[((size_t)blockIdx.x * g.k + jj) * g.E + e] = cnt_k[jj * EP + e];
        }
    }
    if (failed) atomicOr(&g_gate_mlp_error, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int EP, int EL>
static int launch_gate_mlp(GateDev& g, const void* x, int K, const void* w1, const float* b1, cudaStream_t st) {
    GateMlpArgs a;
    a.g = g;
    a.b1 = b1;
    a.K = K;
    a.chunks = ceil_div(g.H, GM_BN);
    CUtensorMap tm_x, tm_w1, tm_w2;
    int rc = make_tmap(&tm_x, x, g.T, K, LR_BM);
    if (rc != PIKV_OK) return rc;
    rc = make_tmap(&tm_w1, w1, g.H, K, GM_BN);
    if (rc != PIKV_OK) return rc;
    rc = make_tmap(&tm_w2, g.w2, g.E, g.H, EP);
    if (rc != PIKV_OK) return rc;
    constexpr int STAGE = LR_BM * LR_BK * 2 + GM_BN * LR_BK * 2;
    constexpr int FIXED = GM_KB_PER_CHUNK * LR_BM * LR_BK * 2 + 2 * GM_KB_PER_CHUNK * EP * LR_BK * 2;
    const size_t tail = (2 * 8 + 9) * sizeof(uint64_t) + 16 + sizeof(int) * (GM_EPI_WARPS * EP + EP + GATE_MAX_K * EP) +
                        sizeof(float) * GM_EPI_WARPS * EP + (size_t)LR_BM * g.k + 1024;
    a.stages = (int)min((size_t)8, ((size_t)227 * 1024 - FIXED - tail) / STAGE);
    PIKV_REQUIRE(a.stages >= 2, PIKV_EUNSUPPORTED, "gate_mlp: not enough shared memory for E=%d", g.E);
    const size_t smem = (size_t)a.stages * STAGE + FIXED + tail;
    auto kern = gate_mlp_kernel<EP, EL>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("gate_mlp smem attribute");
    kern<<<g.G, GM_THREADS, smem, st>>>(tm_x, tm_w1, tm_w2, a);
    return check_launch("gate_mlp_kernel");
}

// reads and clears this kernel's sticky error word (called by pikv_gate_error_state)
int gate_mlp_error_fetch() {
    unsigned v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gate_mlp_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gate_mlp_error, &zero, sizeof(zero));
    return (int)v;
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_gate_mlp_fused(const pikv_gate_params* p, const void* x, int32_t K, const void* w1, const float* b1,
                                   pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr && x != nullptr && w1 != nullptr, PIKV_EINVAL, "gate_mlp: null pointer");
    PIKV_REQUIRE(p->dtype == PIKV_BF16, PIKV_EUNSUPPORTED, "gate_mlp: bf16 inputs and weights only");
    PIKV_REQUIRE(p->w2 != nullptr && p->H > 0 && K > 0, PIKV_EINVAL, "gate_mlp: the second layer (w2, H) and K are required");
    PIKV_REQUIRE(K % 8 == 0 && p->H % 8 == 0, PIKV_EUNSUPPORTED, "gate_mlp: K=%d and H=%d must be multiples of 8", K, p->H);
    PIKV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w1 % 16) == 0 && ((uintptr_t)p->w2 % 16) == 0, PIKV_EINVAL,
                 "gate_mlp: x, w1 and w2 must be 16-byte aligned");
    PIKV_REQUIRE(p->phase == PIKV_GATE_WHOLE, PIKV_EINVAL, "gate_mlp: phase must be PIKV_GATE_WHOLE");
    PIKV_REQUIRE(p->T <= LR_BM * GATE_MAX_CTAS, PIKV_ELIMIT, "gate_mlp: at most %d tokens per call", LR_BM * GATE_MAX_CTAS);
    // validation, geometry and the workspace layout are the gate's own (one 128-token tile per CTA here)
    pikv_gate_params q = *p;
    q.act = x;                      // only so that the shared checks see an activation pointer
    GateDev g;
    int rc = gate_run(&q, nullptr, 0, &g);
    if (rc != PIKV_OK) return rc;
    PIKV_REQUIRE(g.chunk == LR_BM, PIKV_ELIMIT, "gate_mlp: unexpected chunking (%d tokens per CTA)", g.chunk);
    g.act = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g.E <= 8) rc = launch_gate_mlp<16, 8>(g, x, K, w1, b1, st);
    else if (g.E <= 16) rc = launch_gate_mlp<16, 16>(g, x, K, w1, b1, st);
    else if (g.E <= 32) rc = launch_gate_mlp<32, 32>(g, x, K, w1, b1, st);
    else rc = launch_gate_mlp<64, 64>(g, x, K, w1, b1, st);
    if (rc != PIKV_OK) return rc;
    count_launch(1);
    return gate_run(&q, st, GATE_DO_SLOTS, nullptr);
}
