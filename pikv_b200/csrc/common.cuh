// Shared host/device helpers for the pikv_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/pikv_b200.h"

namespace pikv {

// ---- host-side error plumbing ------------------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int  sm_count();          // SMs of the current device (cached per device)
int  check_launch(const char* what);   // cudaGetLastError -> status

#define PIKV_REQUIRE(cond, code, ...)                      \
    do {                                                   \
        if (!(cond)) {                                     \
            ::pikv::set_error(__VA_ARGS__);                \
            return (code);                                 \
        }                                                  \
    } while (0)

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers ----------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }

// two bf16 packed in a 32-bit word -> two floats (exact)
__device__ __forceinline__ void bf16x2_to_f32(uint32_t w, float& a, float& b) {
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
}

// fp32 -> bf16 bits, round to nearest even (NaN-safe via the intrinsic)
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 16-byte global load that bypasses L1 allocation (streamed once)
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ld_stream_8(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// ---- the reference's quantisation arithmetic, one group ------------------------
// core/single/module/pikv_compression.py:965-1006.  Every operation is a separately
// rounded IEEE fp32 op (the intrinsics are never contracted into FMAs) so codes are
// bit-identical to the PyTorch path.
struct QParams {
    float scale, zp;
};
__device__ __forceinline__ QParams quant_params(float x_min, float x_max, int qmin, int qmax, bool symmetric) {
    if (x_max == x_min) x_max = __fadd_rn(x_min, 1e-5f);
    QParams p;
    float range = (float)(qmax - qmin);
    if (symmetric) {
        float abs_max = fmaxf(fabsf(x_min), fabsf(x_max));
        p.scale = __fdiv_rn(__fmul_rn(2.0f, abs_max), range);
        p.zp = 0.0f;
    } else {
        p.scale = __fdiv_rn(__fsub_rn(x_max, x_min), range);
        p.zp = __fsub_rn((float)qmin, rintf(__fdiv_rn(x_min, p.scale)));
    }
    return p;
}
__device__ __forceinline__ float quant_code(float x, QParams p, float qmin, float qmax) {
    return fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(x, p.scale), p.zp)), qmin), qmax);
}
// Same code as quant_code without a division per element: y ~ x * (1/scale) + zp is within a
// few ulp of the exactly rounded x / scale + zp, so rint(y) can only differ from the reference
// when y sits next to a .5 boundary; exactly those elements (and any non-finite y) take the
// IEEE-division path.  inv = __frcp_rn(scale).
__device__ __forceinline__ float quant_code_fast(float x, QParams p, float inv, float qmin, float qmax) {
    const float y = __fadd_rn(__fmul_rn(x, inv), p.zp);
    float q = rintf(y);
    const float d = fabsf(__fsub_rn(y, q));          // distance to the nearest integer, <= 0.5
    if (!(d < 0.499f) || !(fabsf(y) < 1.0e6f)) q = rintf(__fadd_rn(__fdiv_rn(x, p.scale), p.zp));
    return fminf(fmaxf(q, qmin), qmax);
}
__device__ __forceinline__ float dequant_code(float q, QParams p) {
    return __fmul_rn(__fsub_rn(q, p.zp), p.scale);
}

// physical byte offset of logical 16-byte chunk c (8-bit codes, 128-byte rows)
__device__ __forceinline__ int swz8_chunk(int row_in_page, int c) { return c ^ (row_in_page & 7); }
// physical 8-byte unit of logical unit u (4-bit codes, 64-byte rows)
__device__ __forceinline__ int swz4_unit(int row_in_page, int u) { return u ^ (row_in_page & 4); }

#endif  // __CUDACC__

}  // namespace pikv
