// Router gate: last-layer logits + softmax + top-k + load-balance counts + slot scan.
//
// Two launches, no atomics on floats, no inter-CTA waiting:
//   gate_*_kernel   each CTA owns a contiguous chunk of tokens; per token it forms the
//                   logits, softmax, top-k and renormalised weights, then ranks its own
//                   (token, k) pairs per expert in order and publishes per-CTA counts;
//   gate_finalize   each CTA turns its local ranks into global slots from the exclusive
//                   prefix of the per-CTA counts; CTA 0 also reduces the totals.
// Results are therefore run-to-run bit-identical.
#include "gate_common.cuh"
#include <stdlib.h>

namespace pikv {

// ---- per-CTA ranking of its (token, k) pairs, in order ----------------------------
// sel[0..npairs) holds the expert of every pair of this CTA's chunk.  Writes the local
// rank (number of earlier pairs of the chunk with the same expert) to slot[] and the
// per-CTA counts to the workspace.
template <int EP>
__device__ __forceinline__ void cta_rank_tail(const GateDev& g, const uint8_t* sel, int chunk_start, int ntok,
                                              int* warp_cnt /*[WARPS][EP]*/, int* run /*[EP]*/,
                                              int* cnt_k /*[K][EP]*/) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int npairs = ntok * g.k;
    for (int i = tid; i < EP; i += GATE_THREADS) run[i] = 0;
    for (int i = tid; i < GATE_MAX_K * EP; i += GATE_THREADS) cnt_k[i] = 0;
    __syncthreads();
    for (int base = 0; base < npairs; base += GATE_THREADS) {
        for (int i = tid; i < GATE_WARPS * EP; i += GATE_THREADS) warp_cnt[i] = 0;
        __syncthreads();
        const int p = base + tid;
        const bool valid = p < npairs;
        const int e = valid ? (int)sel[p] : 255;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (valid && rank_in_warp == 0) warp_cnt[warp * EP + e] = __popc(peers);
        if (valid) atomicAdd(&cnt_k[(p % g.k) * EP + e], 1);   // integer: order-independent
        __syncthreads();
        if (valid) {
            int r = run[e] + rank_in_warp;
            for (int w = 0; w < warp; ++w) r += warp_cnt[w * EP + e];
            if (g.slot) g.slot[(size_t)chunk_start * g.k + p] = r;
        }
        __syncthreads();
        if (tid < EP) {
            int add = 0;
#pragma unroll
            for (int w = 0; w < GATE_WARPS; ++w) add += warp_cnt[w * EP + tid];
            run[tid] += add;
        }
        __syncthreads();
    }
    const int cta = blockIdx.x;
    for (int e = tid; e < g.E; e += GATE_THREADS) g.cta_cnt[(size_t)cta * g.E + e] = run[e];
    for (int i = tid; i < g.k * g.E; i += GATE_THREADS) {
        int j = i / g.E, e = i % g.E;
        g.cta_cnt_k[((size_t)cta * g.k + j) * g.E + e] = cnt_k[j * EP + e];
    }
}

// ---- gate from activations: SIMT fp32 dot products --------------------------------
// One warp forms the logits of TPW tokens at a time: lanes split the hidden dimension in
// 8-element vectors, every w2 vector is reused for the TPW tokens, partial sums meet in
// an xor butterfly (fixed order), then lane i < TPW runs the tail of token i.
template <typename TIn> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
        bf16x2_to_f32(r.x, v[0], v[1]);
        bf16x2_to_f32(r.y, v[2], v[3]);
        bf16x2_to_f32(r.z, v[4], v[5]);
        bf16x2_to_f32(r.w, v[6], v[7]);
    }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        float4 a = __ldg(reinterpret_cast<const float4*>(p));
        float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};

template <typename TIn, int EP, int TPW>
__global__ void __launch_bounds__(GATE_THREADS) gate_act_kernel(GateDev g) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int* warp_cnt = reinterpret_cast<int*>(smem_raw);                 // [WARPS][EP]
    int* run = warp_cnt + GATE_WARPS * EP;                            // [EP]
    int* cnt_k = run + EP;                                            // [K][EP]
    float* psum_rows = reinterpret_cast<float*>(cnt_k + GATE_MAX_K * EP);  // [WARPS][TPW][EP]
    uint8_t* sel = reinterpret_cast<uint8_t*>(psum_rows + GATE_WARPS * TPW * EP);  // [chunk*k]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk_start = blockIdx.x * g.chunk;
    const int ntok = min(g.chunk, g.T - chunk_start);
    const TIn* act = static_cast<const TIn*>(g.act);
    const TIn* w2 = static_cast<const TIn*>(g.w2);
    const int H = g.H, E = g.E;

    for (int i = tid; i < GATE_WARPS * TPW * EP; i += GATE_THREADS) psum_rows[i] = 0.f;
    __syncthreads();

    for (int tile = warp * TPW; tile < ntok; tile += GATE_WARPS * TPW) {
        float acc[TPW][EP];
#pragma unroll
        for (int i = 0; i < TPW; ++i)
#pragma unroll
            for (int e = 0; e < EP; ++e) acc[i][e] = 0.f;
        const TIn* rows[TPW];
        bool ok[TPW];
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
            ok[i] = (tile + i) < ntok;
            rows[i] = act + (size_t)(chunk_start + (ok[i] ? tile + i : tile)) * H;
        }
        for (int c = lane * 8; c < H; c += 32 * 8) {
            float a[TPW][8];
#pragma unroll
            for (int i = 0; i < TPW; ++i) Vec8<TIn>::load(rows[i] + c, a[i]);
#pragma unroll
            for (int e = 0; e < EP; ++e) {
                if (e < E) {
                    float w[8];
                    Vec8<TIn>::load(w2 + (size_t)e * H + c, w);
#pragma unroll
                    for (int i = 0; i < TPW; ++i)
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[i][e] = fmaf(a[i][j], w[j], acc[i][e]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TPW; ++i)
#pragma unroll
            for (int e = 0; e < EP; ++e) acc[i][e] = warp_sum(acc[i][e]);
        float l[EP];
#pragma unroll
        for (int e = 0; e < EP; ++e) {
            l[e] = 0.f;
#pragma unroll
            for (int i = 0; i < TPW; ++i)
                if (lane == i) l[e] = acc[i][e];
            if (g.b2 && e < E) l[e] += g.b2[e];
        }
        if (lane < TPW && (tile + lane) < ntok) {
            token_tail<EP>(l, g, chunk_start + tile + lane, sel + (size_t)(tile + lane) * g.k);
            float* row = psum_rows + (warp * TPW + lane) * EP;
#pragma unroll
            for (int e = 0; e < EP; ++e) row[e] += l[e];
        }
    }
    __syncthreads();
    if (tid < E) {
        float s = 0.f;
        for (int r = 0; r < GATE_WARPS * TPW; ++r) s += psum_rows[r * EP + tid];
        g.cta_psum[(size_t)blockIdx.x * E + tid] = s;
    }
    cta_rank_tail<EP>(g, sel, chunk_start, ntok, warp_cnt, run, cnt_k);
}

// ---- gate from precomputed logits: one thread per token ---------------------------
template <int EP>
__global__ void __launch_bounds__(GATE_THREADS) gate_logits_kernel(GateDev g) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int* warp_cnt = reinterpret_cast<int*>(smem_raw);
    int* run = warp_cnt + GATE_WARPS * EP;
    int* cnt_k = run + EP;
    float* psum_w = reinterpret_cast<float*>(cnt_k + GATE_MAX_K * EP);   // [WARPS][EP]
    uint8_t* sel = reinterpret_cast<uint8_t*>(psum_w + GATE_WARPS * EP);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk_start = blockIdx.x * g.chunk;
    const int ntok = min(g.chunk, g.T - chunk_start);
    const int E = g.E;
    for (int i = tid; i < GATE_WARPS * EP; i += GATE_THREADS) psum_w[i] = 0.f;
    __syncthreads();
    for (int base = 0; base < ntok; base += GATE_THREADS) {
        const int lt = base + tid;
        float l[EP];
        const bool valid = lt < ntok;
#pragma unroll
        for (int e = 0; e < EP; ++e)
            l[e] = (valid && e < E) ? g.logits_in[(size_t)(chunk_start + lt) * E + e] : 0.f;
        if (valid) token_tail<EP>(l, g, chunk_start + lt, sel + (size_t)lt * g.k);
#pragma unroll
        for (int e = 0; e < EP; ++e) {
            float s = warp_sum(valid ? l[e] : 0.f);
            if (lane == 0 && e < E) psum_w[warp * EP + e] += s;
        }
    }
    __syncthreads();
    if (tid < E) {
        float s = 0.f;
        for (int w = 0; w < GATE_WARPS; ++w) s += psum_w[w * EP + tid];
        g.cta_psum[(size_t)blockIdx.x * E + tid] = s;
    }
    cta_rank_tail<EP>(g, sel, chunk_start, ntok, warp_cnt, run, cnt_k);
}

// ---- finalize: local ranks -> global slots; totals --------------------------------
// Threads are laid out as (expert e, part): part p sums the per-CTA counters of CTAs p, p+parts, ...
// so the reads of one prefix are spread over 256/EP2 threads and overlap; parts are combined in a
// fixed order (the float sums stay run-to-run identical).
// sum of p[c * stride] for c = first, first + step, ... < end, eight loads in flight per round trip and
// added in index order (with 64 experts a thread walks a quarter of the CTAs)
template <typename V>
__device__ __forceinline__ V strided_sum(const V* p, size_t stride, int first, int end, int step) {
    V s = V(0);
    int c = first;
    for (; c + 7 * step < end; c += 8 * step) {
        V v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(p + (size_t)(c + u * step) * stride);
#pragma unroll
        for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; c < end; c += step) s += __ldg(p + (size_t)c * stride);
    return s;
}

__global__ void __launch_bounds__(GATE_THREADS) gate_finalize_kernel(GateDev g) {
    __shared__ int base_s[GATE_MAX_E];
    __shared__ int part_i[GATE_THREADS];
    __shared__ float part_f[GATE_THREADS];
    const int tid = threadIdx.x, cta = blockIdx.x, E = g.E;
    int ep2 = 8;
    while (ep2 < E) ep2 <<= 1;
    const int parts = GATE_THREADS / ep2;
    const int e = tid & (ep2 - 1), part = tid / ep2;
    {
        part_i[tid] = e < E ? strided_sum(g.cta_cnt + e, (size_t)E, part, cta, parts) : 0;
    }
    __syncthreads();
    if (tid < E) {
        int b = g.slot_base ? g.slot_base[tid] : 0;
        for (int p = 0; p < parts; ++p) b += part_i[p * ep2 + tid];
        base_s[tid] = b;
    }
    __syncthreads();
    const int chunk_start = cta * g.chunk;
    const int ntok = min(g.chunk, g.T - chunk_start);
    if (g.slot) {
        const size_t off = (size_t)chunk_start * g.k;
        for (int p = tid; p < ntok * g.k; p += GATE_THREADS) {
            int ee = g.topk_idx[off + p];
            int s = base_s[ee] + g.slot[off + p];
            g.slot[off + p] = (g.capacity <= 0 || s < g.capacity) ? s : -1;
        }
    }
    if (cta != 0) return;
    // totals over all CTAs: per-column counts, probability sums, new lengths
    int tot = 0;
    for (int j = 0; j < g.k; ++j) {
        const int s = e < E ? strided_sum(g.cta_cnt_k + (size_t)j * E + e, (size_t)g.k * E, part, g.G, parts) : 0;
        __syncthreads();
        part_i[tid] = s;
        __syncthreads();
        if (tid < E) {
            int cnt = 0;
            for (int p = 0; p < parts; ++p) cnt += part_i[p * ep2 + tid];
            if (g.counts_k) g.counts_k[j * E + tid] = cnt;
            tot += cnt;
        }
    }
    part_f[tid] = e < E ? strided_sum(g.cta_psum + e, (size_t)E, part, g.G, parts) : 0.f;
    __syncthreads();
    if (tid < E) {
        float sum = 0.f;
        for (int p = 0; p < parts; ++p) sum += part_f[p * ep2 + tid];
        if (g.prob_sum) g.prob_sum[tid] = sum;
        if (g.new_len) {
            int n = (g.slot_base ? g.slot_base[tid] : 0) + tot;
            g.new_len[tid] = (g.capacity > 0 && n > g.capacity) ? g.capacity : n;
        }
    }
}

// ---- dense dispatch / combine ------------------------------------------------------
__global__ void dispatch_scatter_kernel(const int* topk_idx, const float* topk_w, const int* slot,
                                        const int* counts_k, int T, int E, int k, int cap, int mode,
                                        float* dispatch, float* combine) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= T * k) return;
    const int t = p / k, j = p % k;
    const int e = topk_idx[p];
    int pos;
    if (mode == 0) {
        pos = slot[p];
    } else {
        // core/single/pikv_routing.py:107-128: the position in pass j is the number of
        // earlier passes in which this expert received at least one token.
        pos = 0;
        for (int i = 0; i < j; ++i) pos += counts_k[i * E + e] > 0 ? 1 : 0;
        if (pos >= cap) pos = -1;
    }
    if (pos < 0 || pos >= cap) return;
    const size_t o = ((size_t)t * E + e) * cap + pos;
    dispatch[o] = 1.0f;
    combine[o] = topk_w[p];
}

static int gate_geometry(int T, int* chunk_out, int* G_out) {
    int sms = sm_count();
    int G = min(GATE_MAX_CTAS, max(1, min(2 * sms, ceil_div(T, 32))));
    int chunk = ceil_div(T, G);
    if (chunk > GATE_MAX_CHUNK) chunk = GATE_MAX_CHUNK;
    G = ceil_div(T, chunk);
    if (G > GATE_MAX_CTAS) return -1;
    *chunk_out = chunk;
    *G_out = G;
    return 0;
}

template <typename TIn, int EP, int TPW>
static int launch_act(const GateDev& g, cudaStream_t st) {
    size_t smem = sizeof(int) * (GATE_WARPS * EP + EP + GATE_MAX_K * EP) + sizeof(float) * GATE_WARPS * TPW * EP +
                  (size_t)g.chunk * g.k;
    auto kern = gate_act_kernel<TIn, EP, TPW>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<g.G, GATE_THREADS, smem, st>>>(g);
    return check_launch("gate_act_kernel");
}
template <int EP>
static int launch_logits(const GateDev& g, cudaStream_t st) {
    size_t smem = sizeof(int) * (GATE_WARPS * EP + EP + GATE_MAX_K * EP) + sizeof(float) * GATE_WARPS * EP +
                  (size_t)g.chunk * g.k;
    auto kern = gate_logits_kernel<EP>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<g.G, GATE_THREADS, smem, st>>>(g);
    return check_launch("gate_logits_kernel");
}

}  // namespace pikv

using namespace pikv;

extern "C" size_t pikv_gate_workspace_bytes(int32_t T, int32_t E, int32_t top_k) {
    if (T <= 0 || E <= 0 || top_k <= 0) return 0;
    // per-CTA counters, then T*top_k chunk-local ranks (used when a consumer finishes the slot scan)
    return (size_t)GATE_MAX_CTAS * (size_t)E * (size_t)(top_k + 2) * 4 + (size_t)T * (size_t)top_k * 4;
}

namespace pikv {
int gate_run(const pikv_gate_params* p, cudaStream_t st, int what, GateDev* out) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "gate: null params");
    PIKV_REQUIRE(p->T > 0 && p->E > 0 && p->top_k > 0, PIKV_EINVAL, "gate: T, E, top_k must be positive");
    PIKV_REQUIRE(p->E <= GATE_MAX_E, PIKV_ELIMIT, "gate: E=%d exceeds %d", p->E, GATE_MAX_E);
    PIKV_REQUIRE(p->top_k <= GATE_MAX_K && p->top_k <= p->E, PIKV_ELIMIT, "gate: top_k=%d must be <= min(E, %d)",
                 p->top_k, GATE_MAX_K);
    PIKV_REQUIRE(p->topk_idx != nullptr, PIKV_EINVAL, "gate: topk_idx output is required");
    PIKV_REQUIRE(p->act != nullptr || p->logits_in != nullptr, PIKV_EINVAL, "gate: give act+w2 or logits_in");
    PIKV_REQUIRE(p->mask_mode == PIKV_MASK_NONE || p->expert_mask != nullptr, PIKV_EINVAL,
                 "gate: mask_mode set without expert_mask");
    PIKV_REQUIRE(p->mask_mode >= 0 && p->mask_mode <= 3, PIKV_EINVAL, "gate: bad mask_mode %d", p->mask_mode);
    PIKV_REQUIRE(p->workspace != nullptr && p->workspace_bytes >= pikv_gate_workspace_bytes(p->T, p->E, p->top_k),
                 PIKV_EINVAL, "gate: workspace too small");
    GateDev g;
    g.act = p->act; g.w2 = p->w2; g.b2 = p->b2; g.logits_in = p->logits_in;
    g.T = p->T; g.H = p->H; g.E = p->E; g.k = p->top_k;
    g.mask = p->expert_mask; g.mask_mode = p->expert_mask ? p->mask_mode : PIKV_MASK_NONE;
    g.corr = p->correction; g.temperature = p->temperature == 0.f ? 1.f : p->temperature; g.eps = p->renorm_eps;
    g.capacity = p->capacity; g.slot_base = p->slot_base;
    g.probs = p->probs; g.topk_idx = p->topk_idx; g.topk_w = p->topk_w; g.slot = p->slot;
    g.counts_k = p->counts_k; g.prob_sum = p->prob_sum; g.new_len = p->new_len;
    PIKV_REQUIRE(gate_geometry(p->T, &g.chunk, &g.G) == 0, PIKV_ELIMIT, "gate: T=%d too large for one call", p->T);
    int* ws = static_cast<int*>(p->workspace);
    g.cta_cnt = ws;
    g.cta_cnt_k = ws + (size_t)GATE_MAX_CTAS * g.E;
    g.cta_psum = reinterpret_cast<float*>(ws + (size_t)GATE_MAX_CTAS * g.E * (g.k + 1));
    if (what & GATE_RANKS_TO_WS) g.slot = ws + (size_t)GATE_MAX_CTAS * g.E * (g.k + 2);
    int rc;
    const int E = g.E;
    const bool use_tc = g.act != nullptr && g.w2 != nullptr && gate_tc_supported(g, p->dtype) && !(p->phase & PIKV_GATE_FORCE_SIMT);
    if (!(what & GATE_DO_SCORE)) {
        if (use_tc) gate_tc_geometry(g);
        if (out) *out = g;
        if (!(what & GATE_DO_SLOTS)) return PIKV_OK;
        gate_finalize_kernel<<<g.G, GATE_THREADS, 0, st>>>(g);
        count_launch(1);
        return check_launch("gate_finalize_kernel");
    }
    if (use_tc) {
        rc = gate_tc_launch(g, st);
    } else if (g.act != nullptr) {
        PIKV_REQUIRE(g.w2 != nullptr, PIKV_EINVAL, "gate: w2 is required with act");
        PIKV_REQUIRE(g.H > 0 && g.H % 8 == 0, PIKV_EUNSUPPORTED, "gate: H=%d must be a positive multiple of 8", g.H);
        PIKV_REQUIRE(p->dtype == PIKV_F32 || p->dtype == PIKV_BF16, PIKV_EINVAL, "gate: bad dtype %d", p->dtype);
#define PIKV_GATE_DISPATCH(TIn)                                                     \
        if (E <= 4) rc = launch_act<TIn, 4, 4>(g, st);                              \
        else if (E <= 8) rc = launch_act<TIn, 8, 4>(g, st);                         \
        else if (E <= 16) rc = launch_act<TIn, 16, 4>(g, st);                       \
        else if (E <= 32) rc = launch_act<TIn, 32, 2>(g, st);                       \
        else rc = launch_act<TIn, 64, 1>(g, st);
        if (p->dtype == PIKV_BF16) { PIKV_GATE_DISPATCH(__nv_bfloat16) } else { PIKV_GATE_DISPATCH(float) }
#undef PIKV_GATE_DISPATCH
    } else {
        if (E <= 4) rc = launch_logits<4>(g, st);
        else if (E <= 8) rc = launch_logits<8>(g, st);
        else if (E <= 16) rc = launch_logits<16>(g, st);
        else if (E <= 32) rc = launch_logits<32>(g, st);
        else rc = launch_logits<64>(g, st);
    }
    if (rc != PIKV_OK) return rc;
    if (out) *out = g;
    if (!(what & GATE_DO_SLOTS)) {
        count_launch(1);
        return PIKV_OK;
    }
    gate_finalize_kernel<<<g.G, GATE_THREADS, 0, st>>>(g);
    count_launch(2);
    return check_launch("gate_finalize_kernel");
}
}  // namespace pikv

extern "C" int pikv_gate_fused(const pikv_gate_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "gate: null params");
    const int phase = p->phase & ~PIKV_GATE_FORCE_SIMT;
    PIKV_REQUIRE(phase >= PIKV_GATE_WHOLE && phase <= PIKV_GATE_SLOTS, PIKV_EINVAL, "gate: bad phase %d", p->phase);
    const int what = phase == PIKV_GATE_SCORE ? GATE_DO_SCORE : phase == PIKV_GATE_SLOTS ? GATE_DO_SLOTS
                                                                                        : (GATE_DO_SCORE | GATE_DO_SLOTS);
    return gate_run(p, static_cast<cudaStream_t>(stream), what, nullptr);
}

extern "C" int pikv_dispatch_scatter(const int32_t* topk_idx, const float* topk_w, const int32_t* slot,
                                     const int32_t* counts_k, int32_t T, int32_t E, int32_t top_k,
                                     int32_t capacity, int32_t position_mode, float* dispatch, float* combine,
                                     pikv_stream_t stream) {
    PIKV_REQUIRE(topk_idx && topk_w && dispatch && combine, PIKV_EINVAL, "dispatch_scatter: null pointer");
    PIKV_REQUIRE(T > 0 && E > 0 && top_k > 0 && capacity > 0, PIKV_EINVAL, "dispatch_scatter: bad sizes");
    PIKV_REQUIRE(position_mode == 0 ? slot != nullptr : counts_k != nullptr, PIKV_EINVAL,
                 "dispatch_scatter: slot (mode 0) or counts_k (mode 1) required");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    size_t bytes = (size_t)T * E * capacity * sizeof(float);
    if (cudaMemsetAsync(dispatch, 0, bytes, st) != cudaSuccess || cudaMemsetAsync(combine, 0, bytes, st) != cudaSuccess)
        return check_launch("dispatch_scatter memset");
    int n = T * top_k;
    dispatch_scatter_kernel<<<ceil_div(n, 256), 256, 0, st>>>(topk_idx, topk_w, slot, counts_k, T, E, top_k, capacity,
                                                              position_mode, dispatch, combine);
    count_launch(1);
    return check_launch("dispatch_scatter_kernel");
}
