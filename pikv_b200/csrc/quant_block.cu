// Block-wide fake quantisation (the drop-in arithmetic of QuantizedCompressor.forward):
// every column group is one block whose min/max run over ALL rows.
//
//   stats   thread per column, CTA per (128 columns, row block): per-column min/max partials
//   params  thread per group: reduce partials over row blocks and the group's columns,
//           then scale / zero point with the reference's formulas
//   apply   same shape as stats: codes, dequantised values, per-column squared-error partials
//   err     thread per group: reduce the squared-error partials (fixed order)
// All reductions have a fixed order, so results are run-to-run identical.
#include "common.cuh"
#include <float.h>

namespace pikv {

constexpr int QB_COLS = 128;
constexpr int QB_MAX_RB = 128;

template <typename TIn> __device__ __forceinline__ float ldx(const TIn* p);
template <> __device__ __forceinline__ float ldx<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldx<__nv_bfloat16>(const __nv_bfloat16* p) {
    return bf16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(p)));
}

template <typename TIn>
__global__ void __launch_bounds__(QB_COLS) qb_stats_kernel(const TIn* x, int N, int H, int rows_per, float* ws_min,
                                                           float* ws_max) {
    const int col = blockIdx.x * QB_COLS + threadIdx.x;
    const int rb = blockIdx.y;
    if (col >= H) return;
    const int r0 = rb * rows_per, r1 = min(N, r0 + rows_per);
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (int r = r0; r < r1; ++r) {
        float v = ldx<TIn>(x + (size_t)r * H + col);
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
    }
    ws_min[(size_t)rb * H + col] = mn;
    ws_max[(size_t)rb * H + col] = mx;
}

__global__ void qb_params_kernel(const float* ws_min, const float* ws_max, int H, int RB, int group_size, int G,
                                 int qmin, int qmax, int symmetric, float* params, float* params_out) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= G) return;
    const int c0 = g * group_size, c1 = min(H, c0 + group_size);
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (int rb = 0; rb < RB; ++rb)
        for (int c = c0; c < c1; ++c) {
            mn = fminf(mn, ws_min[(size_t)rb * H + c]);
            mx = fmaxf(mx, ws_max[(size_t)rb * H + c]);
        }
    QParams p = quant_params(mn, mx, qmin, qmax, symmetric != 0);
    params[2 * g] = p.scale;
    params[2 * g + 1] = p.zp;
    if (params_out) {
        params_out[2 * g] = p.scale;
        params_out[2 * g + 1] = p.zp;
    }
}

template <typename TIn>
__global__ void __launch_bounds__(QB_COLS) qb_apply_kernel(const TIn* x, int N, int H, int rows_per, int group_size,
                                                           const float* params, float qmin, float qmax, float* dq_out,
                                                           float* q_out, float* ws_err) {
    const int col = blockIdx.x * QB_COLS + threadIdx.x;
    const int rb = blockIdx.y;
    if (col >= H) return;
    const int g = col / group_size;
    QParams p;
    p.scale = params[2 * g];
    p.zp = params[2 * g + 1];
    const int r0 = rb * rows_per, r1 = min(N, r0 + rows_per);
    float err = 0.f;
    const float inv = __frcp_rn(p.scale);
    for (int r = r0; r < r1; ++r) {
        const size_t o = (size_t)r * H + col;
        const float v = ldx<TIn>(x + o);
        const float q = quant_code_fast(v, p, inv, qmin, qmax);
        const float dq = dequant_code(q, p);
        if (dq_out) dq_out[o] = dq;
        if (q_out) q_out[o] = q;
        const float d = __fsub_rn(v, dq);
        err = __fadd_rn(err, __fmul_rn(d, d));
    }
    if (ws_err) ws_err[(size_t)rb * H + col] = err;
}

__global__ void qb_err_kernel(const float* ws_err, int H, int RB, int group_size, int G, float* sq_err) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= G) return;
    const int c0 = g * group_size, c1 = min(H, c0 + group_size);
    float s = 0.f;
    for (int rb = 0; rb < RB; ++rb)
        for (int c = c0; c < c1; ++c) s += ws_err[(size_t)rb * H + c];
    sq_err[g] = s;
}

}  // namespace pikv

using namespace pikv;

extern "C" size_t pikv_quant_block_workspace_bytes(int32_t N, int32_t H, int32_t group_size) {
    (void)N;
    if (H <= 0 || group_size <= 0) return 0;
    return ((size_t)3 * QB_MAX_RB * H + 2 * (size_t)H) * sizeof(float);
}

extern "C" int pikv_quant_block(const void* x, int32_t dtype, int32_t N, int32_t H, int32_t group_size, int32_t qmin,
                                int32_t qmax, int32_t symmetric, const float* params_in, float* params_out,
                                float* dq_out, float* q_out, float* sq_err, void* workspace, size_t workspace_bytes,
                                pikv_stream_t stream) {
    PIKV_REQUIRE(x != nullptr, PIKV_EINVAL, "quant_block: null input");
    PIKV_REQUIRE(N > 0 && H > 0 && group_size > 0, PIKV_EINVAL, "quant_block: bad sizes");
    PIKV_REQUIRE(qmax > qmin, PIKV_EINVAL, "quant_block: qmax must exceed qmin");
    PIKV_REQUIRE(dtype == PIKV_F32 || dtype == PIKV_BF16, PIKV_EINVAL, "quant_block: bad dtype %d", dtype);
    PIKV_REQUIRE(workspace && workspace_bytes >= pikv_quant_block_workspace_bytes(N, H, group_size), PIKV_EINVAL,
                 "quant_block: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int G = ceil_div(H, group_size);
    const int col_blocks = ceil_div(H, QB_COLS);
    int RB = ceil_div(4 * sm_count(), col_blocks);
    RB = max(1, min(min(RB, QB_MAX_RB), ceil_div(N, 8)));
    const int rows_per = ceil_div(N, RB);
    RB = ceil_div(N, rows_per);
    float* ws = static_cast<float*>(workspace);
    float* ws_min = ws;
    float* ws_max = ws + (size_t)QB_MAX_RB * H;
    float* ws_err = ws + (size_t)2 * QB_MAX_RB * H;
    float* params = ws + (size_t)3 * QB_MAX_RB * H;
    dim3 grid(col_blocks, RB);
    int launches = 0;
    if (params_in == nullptr) {
        if (dtype == PIKV_F32)
            qb_stats_kernel<float><<<grid, QB_COLS, 0, st>>>(static_cast<const float*>(x), N, H, rows_per, ws_min, ws_max);
        else
            qb_stats_kernel<__nv_bfloat16><<<grid, QB_COLS, 0, st>>>(static_cast<const __nv_bfloat16*>(x), N, H,
                                                                    rows_per, ws_min, ws_max);
        qb_params_kernel<<<ceil_div(G, 128), 128, 0, st>>>(ws_min, ws_max, H, RB, group_size, G, qmin, qmax, symmetric,
                                                           params, params_out);
        launches += 2;
    } else {
        if (cudaMemcpyAsync(params, params_in, sizeof(float) * 2 * G, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return check_launch("quant_block params copy");
        if (params_out &&
            cudaMemcpyAsync(params_out, params_in, sizeof(float) * 2 * G, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return check_launch("quant_block params copy");
    }
    if (dq_out || q_out || sq_err) {
        float* werr = sq_err ? ws_err : nullptr;
        if (dtype == PIKV_F32)
            qb_apply_kernel<float><<<grid, QB_COLS, 0, st>>>(static_cast<const float*>(x), N, H, rows_per, group_size,
                                                             params, (float)qmin, (float)qmax, dq_out, q_out, werr);
        else
            qb_apply_kernel<__nv_bfloat16><<<grid, QB_COLS, 0, st>>>(static_cast<const __nv_bfloat16*>(x), N, H,
                                                                     rows_per, group_size, params, (float)qmin,
                                                                     (float)qmax, dq_out, q_out, werr);
        ++launches;
        if (sq_err) {
            qb_err_kernel<<<ceil_div(G, 128), 128, 0, st>>>(ws_err, H, RB, group_size, G, sq_err);
            ++launches;
        }
    }
    count_launch(launches);
    return check_launch("quant_block");
}
