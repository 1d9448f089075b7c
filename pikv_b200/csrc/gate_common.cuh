// Shared between the SIMT and the tcgen05 gate kernels: launch geometry, the per-token tail
// (mask, softmax, top-k, renormalisation) and the argument block.
#pragma once
#include "common.cuh"

namespace pikv {

constexpr int GATE_THREADS = 256;
constexpr int GATE_WARPS = GATE_THREADS / 32;
constexpr int GATE_MAX_CTAS = 1024;
constexpr int GATE_MAX_CHUNK = 4096;   // tokens per CTA
constexpr int GATE_MAX_K = 8;
constexpr int GATE_MAX_E = 64;

struct GateDev {
    const void* act;
    const void* w2;
    const float* b2;
    const float* logits_in;
    int T, H, E, k;
    const float* mask;
    int mask_mode;
    const float* corr;
    float temperature, eps;
    int capacity;
    const int* slot_base;
    float* probs;
    int* topk_idx;
    float* topk_w;
    int* slot;
    int* counts_k;
    float* prob_sum;
    int* new_len;
    int chunk, G;
    int* cta_cnt;     // [G][E]
    int* cta_cnt_k;   // [G][k][E]
    float* cta_psum;  // [G][E]
};

// ---- per-token tail: everything after the logits ---------------------------------
// l[] holds the token's logits (entries >= E are ignored).  Writes the token's outputs
// and returns the probabilities in l[].
template <int EP>
__device__ __forceinline__ void token_tail(float (&l)[EP], const GateDev& g, int t, uint8_t* sel_row) {
    const int E = g.E;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        if (e < E) {
            float x = l[e];
            if (g.temperature != 1.0f) x = __fdiv_rn(x, g.temperature);
            if (g.corr) x = __fmul_rn(x, g.corr[e]);
            if (g.mask_mode == PIKV_MASK_SINGLE)
                x = __fadd_rn(x, __fmul_rn(__fsub_rn(1.0f, g.mask[e]), -1e9f));
            else if (g.mask_mode == PIKV_MASK_MODULE)
                x = __fadd_rn(x, __fmul_rn(__fsub_rn(1.0f, g.mask[e]), -3.402823466e+38f));
            else if (g.mask_mode == PIKV_MASK_BIAS)
                x = __fadd_rn(x, g.mask[e]);
            l[e] = x;
        } else {
            l[e] = -INFINITY;
        }
    }
    float m = l[0];
#pragma unroll
    for (int e = 1; e < EP; ++e) m = fmaxf(m, l[e]);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        float p = (e < E) ? expf(l[e] - m) : 0.f;
        l[e] = p;
        s += p;
    }
#pragma unroll
    for (int e = 0; e < EP; ++e) l[e] = __fdiv_rn(l[e], s);
    if (g.probs) {
        if (EP == 8 && E == 8 && (reinterpret_cast<uintptr_t>(g.probs) & 15) == 0) {     // one 32-byte row: two vector stores
            float4* row = reinterpret_cast<float4*>(g.probs + (size_t)t * 8);
            row[0] = make_float4(l[0], l[1], l[2], l[3]);
            row[1] = make_float4(l[4 % EP], l[5 % EP], l[6 % EP], l[7 % EP]);
        } else {
#pragma unroll
            for (int e = 0; e < EP; ++e)
                if (e < E) g.probs[(size_t)t * E + e] = l[e];
        }
    }
    // top-k on the probabilities; strict '>' keeps the lowest index on ties
    unsigned long long taken = 0ull;
    int idx[GATE_MAX_K];
    float val[GATE_MAX_K];
    float wsum = 0.f;
#pragma unroll
    for (int j = 0; j < GATE_MAX_K; ++j) {
        if (j < g.k) {
            float best = -1.f;
            int bi = 0;
#pragma unroll
            for (int e = 0; e < EP; ++e) {
                bool free_e = !((taken >> e) & 1ull);
                if (e < E && free_e && l[e] > best) {
                    best = l[e];
                    bi = e;
                }
            }
            taken |= 1ull << bi;
            idx[j] = bi;
            val[j] = best;
            wsum += best;
        }
    }
    const float denom = __fadd_rn(wsum, g.eps);
#pragma unroll
    for (int j = 0; j < GATE_MAX_K; ++j) {
        if (j < g.k) {
            g.topk_idx[(size_t)t * g.k + j] = idx[j];
            if (g.topk_w) g.topk_w[(size_t)t * g.k + j] = __fdiv_rn(val[j], denom);
            sel_row[j] = (uint8_t)idx[j];
        }
    }
}

// what gate_run does: launch the scoring kernel, launch the slot finalisation, and whether the chunk-local
// ranks go to the workspace instead of the caller's slot array (for a consumer that finishes the scan
// itself).  With neither launch flag it only validates and fills *out (geometry, workspace layout).
enum : int { GATE_DO_SCORE = 1, GATE_DO_SLOTS = 2, GATE_RANKS_TO_WS = 4 };
int gate_run(const pikv_gate_params* p, cudaStream_t st, int what, GateDev* out);

// tensor-core path (gate_tc.cu): bf16 activations through TMA + tcgen05
bool gate_tc_supported(const GateDev& g, int dtype);
void gate_tc_geometry(GateDev& g);                  // sets g.chunk and g.G
int gate_tc_launch(GateDev& g, cudaStream_t st);   // sets g.chunk and g.G for the finalize kernel

}  // namespace pikv
