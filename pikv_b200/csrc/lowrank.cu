// Low-rank projection GEMM on 5th-generation tensor cores:
//   out[M,N] = act(x[M,K] . w[N,K]^T + bias) (+ residual),  bf16 operands, fp32 accumulate.
//
// One CTA per (128-row tile of x, column block of <= 256 outputs), 6 warps:
//   warp 0   TMA producer: cp.async.bulk.tensor 2D loads of a [128 x 64] tile of x and a
//            [BN x 64] tile of w (128-byte swizzle) into a 4-stage shared-memory ring
//   warp 1   allocates tensor memory, one lane issues tcgen05.mma (M=128, N=BN, K=16; four
//            per 64-wide k block) straight from shared-memory descriptors and signals
//            stage release / accumulator completion with tcgen05.commit
//   warps 2-5 epilogue: tcgen05.ld their 32 accumulator rows out of tensor memory,
//            bias + ReLU (+ residual) in registers, vector stores
// Arithmetic intensity at rank 64 is ~60 FLOP/B, far below the B200 ridge, so the kernel
// is HBM-bound by design: what matters is that the ring keeps >= 64 KiB in flight per SM.
// Every mbarrier wait is bounded; on a timeout the CTA sets an error word and drains.
#include "tc_common.cuh"

namespace pikv {

constexpr int LR_THREADS = 192;
constexpr int LR_MAX_BN = 256;

__device__ unsigned g_lowrank_error = 0;   // sticky: set when a bounded wait ran out

struct LowrankArgs {
    const float* bias;
    const __nv_bfloat16* residual;
    void* out;
    int out_f32, M, N, K, relu, bn, stages, tmem_cols;
};

__global__ void __launch_bounds__(LR_THREADS) lowrank_gemm_kernel(const __grid_constant__ CUtensorMap tm_x,
                                                                  const __grid_constant__ CUtensorMap tm_w,
                                                                  LowrankArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // operand tiles with the 128-byte swizzle must start on a 1024-byte boundary
    unsigned char* smem = smem_raw + ((1024u - (lr_smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stage_a = LR_BM * LR_BK * 2;
    const int stage_b = a.bn * LR_BK * 2;
    const int stage_bytes = stage_a + stage_b;
    // ring first (1024-byte aligned tiles), then barriers and the tensor-memory address slot
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * stage_bytes);
    const uint32_t full0 = lr_smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * a.stages;
    const uint32_t accum_bar = empty0 + 8 * a.stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * a.stages + 1);
    const uint32_t ring = lr_smem_u32(smem);

    const int m0 = blockIdx.x * LR_BM;
    const int n0 = blockIdx.y * LR_MAX_BN;
    const int num_kb = (a.K + LR_BK - 1) / LR_BK;   // a ragged last block is zero-filled by TMA

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            lr_mbar_init(full0 + 8 * s, 1);
            lr_mbar_init(empty0 + 8 * s, 1);
        }
        lr_mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        lr_prefetch_tmap(&tm_x);
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

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % a.stages;
                const uint32_t ph = (uint32_t)(kb / a.stages) & 1u;
                if (!lr_mbar_wait(empty0 + 8 * s, ph ^ 1u)) { failed = true; break; }
                lr_mbar_expect_tx(full0 + 8 * s, (uint32_t)stage_bytes);
                const uint32_t dst = ring + (uint32_t)s * stage_bytes;
                lr_tma_load_2d(dst, &tm_x, kb * LR_BK, m0, full0 + 8 * s);
                lr_tma_load_2d(dst + stage_a, &tm_w, kb * LR_BK, n0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = lr_instr_desc(a.bn);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % a.stages;
                const uint32_t ph = (uint32_t)(kb / a.stages) & 1u;
                if (!lr_mbar_wait(full0 + 8 * s, ph)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = ring + (uint32_t)s * stage_bytes;
                const uint32_t sb = sa + stage_a;
#pragma unroll
                for (int k = 0; k < LR_BK / 16; ++k) {
                    // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
                    lr_mma(tmem_base, lr_smem_desc(sa + 32 * k), lr_smem_desc(sb + 32 * k), idesc, (kb | k) ? 1u : 0u);
                }
                lr_commit(empty0 + 8 * s);       // frees the stage once these MMAs have read it
            }
            lr_commit(accum_bar);                // accumulator complete (or as far as it got)
        }
    } else {
        // epilogue warps 2..5 -> tensor-memory lane groups (warp % 4)
        const int lg = warp & 3;
        const int row = lg * 32 + lane;
        const int m = m0 + row;
        if (!lr_mbar_wait(accum_bar, 0)) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!failed) {
            for (int c = 0; c < a.bn; c += 16) {
                float v[16];
                lr_tmem_ld16(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)c, v);
                const int n = n0 + c;
                if (m < a.M) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float x = v[i] + (a.bias ? __ldg(a.bias + n + i) : 0.f);
                        if (a.relu) x = fmaxf(x, 0.f);
                        v[i] = x;
                    }
                    if (a.residual) {
                        const uint4* rp = reinterpret_cast<const uint4*>(a.residual + (size_t)m * a.N + n);
                        uint4 r0 = __ldg(rp), r1 = __ldg(rp + 1);
                        const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float lo, hi;
                            bf16x2_to_f32(rw[i], lo, hi);
                            v[2 * i] += lo;
                            v[2 * i + 1] += hi;
                        }
                    }
                    if (a.out_f32) {
                        float4* op = reinterpret_cast<float4*>(static_cast<float*>(a.out) + (size_t)m * a.N + n);
#pragma unroll
                        for (int i = 0; i < 4; ++i) op[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    } else {
                        uint32_t pk[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            pk[i] = (uint32_t)f32_to_bf16_bits(v[2 * i]) | ((uint32_t)f32_to_bf16_bits(v[2 * i + 1]) << 16);
                        uint4* op = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + (size_t)m * a.N + n);
                        op[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        op[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                    }
                }
            }
        }
    }
    if (failed) atomicOr(&g_lowrank_error, 1u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols) : "memory");
    }
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_lowrank_project(const void* x, const void* w, const float* bias, const void* residual, void* out,
                                    int32_t out_dtype, int32_t M, int32_t N, int32_t K, int32_t relu,
                                    pikv_stream_t stream) {
    PIKV_REQUIRE(x && w && out, PIKV_EINVAL, "lowrank: null pointer");
    PIKV_REQUIRE(M > 0 && N > 0 && K > 0, PIKV_EINVAL, "lowrank: bad sizes");
    PIKV_REQUIRE(K % 16 == 0, PIKV_EUNSUPPORTED, "lowrank: K=%d must be a multiple of 16", K);
    PIKV_REQUIRE(N % 16 == 0, PIKV_EUNSUPPORTED, "lowrank: N=%d must be a multiple of 16", N);
    PIKV_REQUIRE(out_dtype == PIKV_BF16 || out_dtype == PIKV_F32, PIKV_EINVAL, "lowrank: bad out dtype");
    PIKV_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0, PIKV_EINVAL,
                 "lowrank: pointers must be 16-byte aligned");
    const int n_blocks = ceil_div(N, LR_MAX_BN);
    // all column blocks share one kernel shape: the widest block
    const int bn = N >= LR_MAX_BN ? LR_MAX_BN : N;
    PIKV_REQUIRE(N % bn == 0, PIKV_EUNSUPPORTED, "lowrank: N=%d above %d must be a multiple of %d", N, LR_MAX_BN, LR_MAX_BN);
    CUtensorMap tm_x, tm_w;
    int rc = make_tmap(&tm_x, x, M, K, LR_BM);
    if (rc != PIKV_OK) return rc;
    rc = make_tmap(&tm_w, w, N, K, bn);
    if (rc != PIKV_OK) return rc;
    LowrankArgs a;
    a.bias = bias;
    a.residual = static_cast<const __nv_bfloat16*>(residual);
    a.out = out;
    a.out_f32 = out_dtype == PIKV_F32;
    a.M = M; a.N = N; a.K = K; a.relu = relu; a.bn = bn;
    const int stage_bytes = LR_BM * LR_BK * 2 + bn * LR_BK * 2;
    a.stages = max(2, min(6, (bn <= 64 ? 96 * 1024 : 192 * 1024) / stage_bytes));
    int cols = 32;
    while (cols < bn) cols <<= 1;
    a.tmem_cols = cols;
    const size_t smem = (size_t)a.stages * stage_bytes + (2 * a.stages + 1) * sizeof(uint64_t) + 16 + 1024;
    if (cudaFuncSetAttribute(lowrank_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("lowrank smem attribute");
    dim3 grid(ceil_div(M, LR_BM), n_blocks);
    lowrank_gemm_kernel<<<grid, LR_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(tm_x, tm_w, a);
    count_launch(1);
    return check_launch("lowrank_gemm_kernel");
}

// reads and clears the sticky error word of the tcgen05 kernel (synchronises the stream's device)
extern "C" int pikv_lowrank_error_state(void) {
    unsigned v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_lowrank_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_lowrank_error, &zero, sizeof(zero));
    return (int)v;
}
