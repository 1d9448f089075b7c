// Decode step of the striped expert-sharded cache: every stream's query goes to the ranks that hold rows of
// the caches of its top-k experts, each rank attends over what it holds, the partial results go back to the
// stream's home rank, which merges them.  All exchanges are plain stores into peer-mapped buffers (NVLink)
// followed by per-rank flag words; every wait is bounded and reports through the status word.
//
//   home    shard_decode_post_kernel     q rows -> the ranks that need them, routing records -> every rank,
//                                        then this rank's "posted" flag on every rank
//   owner   decode_plan_kernel<true>     (decode_attn.cu) waits for every rank's flag, turns the S x k routing
//                                        records into the request list of the local decode call (sequence, local
//                                        length, q row), then plans that call as for any other request list
//   owner   decode_attn_kernel<8>        (decode_attn.cu) over the local request list
//   owner   decode_return_kernel         (decode_attn.cu) normalised partial + log-sum-exp -> the home rank,
//                                        then this rank's "done" flag on every rank
//   home    shard_decode_combine_kernel  waits for every rank's "done" flag, merges the ranks' partials of each
//                                        (stream, choice) by log-sum-exp, then combines the k choices
#include "shard_decode.cuh"

namespace pikv {

struct SDCtx {
    pikv_shard_decode_ctx c;
    int log2_stripe;
    unsigned limit_us;
};

// One warp per (local stream, destination rank): the stream's routing records go to that rank, and its query rows
// if the rank owns a stripe of either selected pair.  (One warp per stream, storing to every rank in turn, took
// 36 us for the 32 streams of a rank of eight: four CTAs, 64 KB of stores behind one another per warp.)  A CTA makes
// its units' stores visible with one system-scope fence, the last CTA raises the flags.
constexpr int SD_POST_THREADS = 256;

__global__ void __launch_bounds__(SD_POST_THREADS) shard_decode_post_kernel(SDCtx x, const uint4* q_local, const int* topk_idx,
                                                                            const float* topk_w, const int* pair_len) {
    const pikv_shard_decode_ctx& c = x.c;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (SD_POST_THREADS / 32) + (threadIdx.x >> 5);
    if (unit < c.streams_per_rank * c.world) {
        const int sl = unit / c.world, r = unit % c.world;
        const int s = c.rank * c.streams_per_rank + sl;
        // the query rows are needed almost always: their loads go out before the dependent loads of the routing
        // records (n_q <= 64: up to 32 words of 16 bytes per lane)
        const int row16 = c.n_q * 16;                         // 16-byte words of one stream's query rows
        uint4 qv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (lane + 32 * i < row16) qv[i] = q_local[(size_t)sl * row16 + lane + 32 * i];
        unsigned m = 0;
        if (lane < c.top_k) {
            const int e = topk_idx[sl * c.top_k + lane];
            const bool ok = e >= 0 && e < c.num_experts;
            const int len = ok ? max(0, pair_len[(size_t)sl * c.num_experts + e]) : 0;
            if (!ok && c.status && r == 0) atomicOr(c.status, PIKV_ST_BAD_SEQ);
            const int4 rec = make_int4(ok ? e : 0, len, __float_as_int(topk_w[sl * c.top_k + lane]), 0);
            static_cast<int4*>(c.peer_route[r])[(size_t)s * c.top_k + lane] = rec;
            if (len > 0) {
                const int rot = (c.expert_rot[e] + s) % c.world;
                const int stripes = (len + (1 << x.log2_stripe) - 1) >> x.log2_stripe;
                for (int cc = 0; cc < min(stripes, c.world); ++cc) m |= 1u << ((rot + cc) % c.world);
            }
        }
        const unsigned mask = __reduce_or_sync(0xffffffffu, m);
        if (mask >> r & 1u) {
            uint4* dst = static_cast<uint4*>(c.peer_q[r]) + (size_t)s * row16;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (lane + 32 * i < row16) dst[lane + 32 * i] = qv[i];
        }
    }
    // the last CTA to get here raises this rank's flag on every rank: one thread per destination, because a
    // system-scope release store takes about 2 us and eight of them in a row cost more than the rest of the kernel
    __shared__ unsigned raise_s;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(c.counters, 1u);
        raise_s = 0u;
        if (prev == gridDim.x - 1) {
            c.counters[0] = 0;
            const unsigned step = (*c.seq & ~SD_FAILED) + 1u;
            *c.seq = step;
            __threadfence_system();
            raise_s = step;              // never 0: steps count from 1
        }
    }
    __syncthreads();
    if (raise_s != 0u && threadIdx.x < c.world) sd_flag_store(c.peer_post_flags[threadIdx.x] + c.rank, raise_s);
}

// One warp per (local stream, query head), a lane owns four channels; a grid that is resident at once walks the units,
// so the wait for the ranks' "done" flags happens once per CTA (a system-scope poll per unit cost 38 us a step).
constexpr int SD_COMBINE_THREADS = 128;

__global__ void __launch_bounds__(SD_COMBINE_THREADS) shard_decode_combine_kernel(SDCtx x, const int* topk_idx, const float* topk_w,
                                                                                  const int* pair_len, __nv_bfloat16* out,
                                                                                  float* lse_out, int mode) {
    const pikv_shard_decode_ctx& c = x.c;
    __shared__ int ok_s;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    const unsigned step = *c.seq & ~SD_FAILED;
    if (threadIdx.x < c.world && !sd_flag_wait(c.peer_done_flags[c.rank] + threadIdx.x, step, x.limit_us)) {
        ok_s = 0;
        if (c.status) atomicOr(c.status, PIKV_ST_WAIT_TIMEOUT);
    }
    __syncthreads();
    if (!ok_s) return;
    const float* part_o = c.peer_part_o[c.rank];
    const float* part_lse = c.peer_part_lse[c.rank];
    const int units = c.streams_per_rank * c.n_q;
    for (int unit = blockIdx.x * (SD_COMBINE_THREADS / 32) + (threadIdx.x >> 5); unit < units;
         unit += gridDim.x * (SD_COMBINE_THREADS / 32)) {
        const int sl = unit / c.n_q, qg = unit % c.n_q;
        const int s = c.rank * c.streams_per_rank + sl;
        float4 res = make_float4(0.f, 0.f, 0.f, 0.f);
        float M_all = -INFINITY, den_all = 0.f;                 // mode 1: running merge over the choices
        for (int jsel = 0; jsel < c.top_k; ++jsel) {
            const int e = topk_idx[sl * c.top_k + jsel];
            if (e < 0 || e >= c.num_experts) continue;
            const int len = max(0, pair_len[(size_t)sl * c.num_experts + e]);
            const int rot = (c.expert_rot[e] + s) % c.world;
            const size_t base = ((size_t)sl * c.top_k + jsel) * c.world;
            float M = -INFINITY;
            float lse_r[8];
            float4 o_r[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                lse_r[r] = -INFINITY;
                o_r[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < c.world && striped_local_len(len, rot, r, c.world, x.log2_stripe) > 0) {
                    // written by a peer during this kernel's lifetime: read at L2
                    lse_r[r] = __ldcg(part_lse + (base + r) * c.n_q + qg);
                    o_r[r] = __ldcg(reinterpret_cast<const float4*>(part_o + ((base + r) * c.n_q + qg) * 128) + lane);
                }
                M = fmaxf(M, lse_r[r]);
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (lse_r[r] == -INFINITY) continue;
                const float wgt = expf(lse_r[r] - M);
                acc.x += wgt * o_r[r].x; acc.y += wgt * o_r[r].y; acc.z += wgt * o_r[r].z; acc.w += wgt * o_r[r].w;
                den += wgt;
            }
            const float4 o_j = den > 0.f ? make_float4(acc.x / den, acc.y / den, acc.z / den, acc.w / den)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
            const float lse_j = den > 0.f ? M + logf(den) : -INFINITY;
            if (mode == 0) {
                const float w = topk_w[sl * c.top_k + jsel];  // expert output times routing weight, summed
                res.x += w * o_j.x; res.y += w * o_j.y; res.z += w * o_j.z; res.w += w * o_j.w;
            } else if (lse_j != -INFINITY) {
                const float Mn = fmaxf(M_all, lse_j);
                const float a = M_all == -INFINITY ? 0.f : expf(M_all - Mn), b = expf(lse_j - Mn);
                res.x = res.x * a + o_j.x * b; res.y = res.y * a + o_j.y * b;
                res.z = res.z * a + o_j.z * b; res.w = res.w * a + o_j.w * b;
                den_all = den_all * a + b;
                M_all = Mn;
            }
            if (lse_out && lane == 0) lse_out[((size_t)sl * c.top_k + jsel) * c.n_q + qg] = lse_j;
        }
        if (mode != 0) {
            res = den_all > 0.f ? make_float4(res.x / den_all, res.y / den_all, res.z / den_all, res.w / den_all)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(res.x, res.y), hi = __floats2bfloat162_rn(res.z, res.w);
        reinterpret_cast<uint2*>(out + ((size_t)sl * c.n_q + qg) * 128)[lane] =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

static int sd_check(const pikv_shard_decode_ctx* c, SDCtx* x, const char* who) {
    PIKV_REQUIRE(c != nullptr, PIKV_EINVAL, "%s: null context", who);
    PIKV_REQUIRE(c->world >= 1 && c->world <= 8 && c->rank >= 0 && c->rank < c->world, PIKV_EINVAL, "%s: bad world / rank", who);
    PIKV_REQUIRE(c->num_experts > 0 && c->num_streams > 0 && c->top_k > 0 && c->top_k <= 8 && c->n_q > 0 && c->n_q <= 64, PIKV_EINVAL,
                 "%s: bad sizes (top_k <= 8, n_q <= 64)", who);
    PIKV_REQUIRE(c->streams_per_rank > 0 && c->streams_per_rank * c->world == c->num_streams, PIKV_EINVAL,
                 "%s: num_streams must be world * streams_per_rank", who);
    PIKV_REQUIRE(c->expert_rot && c->seq && c->counters, PIKV_EINVAL, "%s: null pointer", who);
    int log2 = -1;
    for (int b = 4; b < 27; ++b)
        if ((1 << b) == c->stripe) log2 = b;
    PIKV_REQUIRE(log2 > 0, PIKV_EINVAL, "%s: stripe=%d must be a power of two >= 16", who, c->stripe);
    for (int r = 0; r < c->world; ++r)
        PIKV_REQUIRE(c->peer_q[r] && c->peer_route[r] && c->peer_post_flags[r] && c->peer_part_o[r] && c->peer_part_lse[r] &&
                         c->peer_done_flags[r],
                     PIKV_EINVAL, "%s: null exchange buffer for rank %d", who, r);
    x->c = *c;
    x->log2_stripe = log2;
    x->limit_us = c->wait_limit_us > 0 ? (unsigned)c->wait_limit_us : PIKV_DEFAULT_WAIT_US;
    return PIKV_OK;
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_shard_decode_post(const pikv_shard_decode_ctx* c, const void* q_local, const int32_t* topk_idx,
                                      const float* topk_w, const int32_t* pair_len, pikv_stream_t stream) {
    SDCtx x;
    int rc = sd_check(c, &x, "shard_decode_post");
    if (rc != PIKV_OK) return rc;
    PIKV_REQUIRE(q_local && topk_idx && topk_w && pair_len, PIKV_EINVAL, "shard_decode_post: null pointer");
    const int post_ctas = (c->streams_per_rank * c->world + SD_POST_THREADS / 32 - 1) / (SD_POST_THREADS / 32);
    shard_decode_post_kernel<<<post_ctas, SD_POST_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        x, static_cast<const uint4*>(q_local), topk_idx, topk_w, pair_len);
    count_launch(1);
    return check_launch("shard_decode_post_kernel");
}

extern "C" int pikv_shard_decode_attn(const pikv_shard_decode_ctx* c, const pikv_decode_params* cache, int32_t* seq_ids,
                                      int32_t* seq_len, int32_t* q_rows, pikv_stream_t stream) {
    SDCtx x;
    int rc = sd_check(c, &x, "shard_decode_attn");
    if (rc != PIKV_OK) return rc;
    PIKV_REQUIRE(cache && seq_ids && seq_len && q_rows, PIKV_EINVAL, "shard_decode_attn: null pointer");
    PIKV_REQUIRE(cache->n_q == c->n_q, PIKV_EINVAL, "shard_decode_attn: the cache call and the context disagree on n_q");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the request list is built by the decode call's own plan kernel, after it has seen every rank's "posted" flag
    ShardPlan sp;
    sp.world = c->world; sp.rank = c->rank; sp.num_experts = c->num_experts; sp.num_streams = c->num_streams;
    sp.top_k = c->top_k; sp.log2_stripe = x.log2_stripe; sp.limit_us = x.limit_us;
    sp.post_flags = c->peer_post_flags[c->rank];
    sp.seq = c->seq;
    sp.route = static_cast<const int4*>(c->peer_route[c->rank]);
    sp.expert_rot = c->expert_rot;
    sp.status = c->status;
    sp.seq_ids = seq_ids; sp.seq_len = seq_len; sp.q_rows = q_rows;
    pikv_decode_params p = *cache;
    p.B = c->num_streams * c->top_k;
    p.q = c->peer_q[c->rank];
    p.out = nullptr;
    p.seq_ids = seq_ids;
    p.seq_len = seq_len;
    p.lse = nullptr;
    p.scores = nullptr;
    ShardReturn t;
    t.world = c->world; t.rank = c->rank; t.top_k = c->top_k; t.streams_per_rank = c->streams_per_rank;
    for (int r = 0; r < 8; ++r) {
        t.peer_part_o[r] = r < c->world ? c->peer_part_o[r] : nullptr;
        t.peer_part_lse[r] = r < c->world ? c->peer_part_lse[r] : nullptr;
        t.peer_done_flags[r] = r < c->world ? c->peer_done_flags[r] : nullptr;
    }
    t.counter = c->counters + 1;
    t.seq = c->seq;
    return decode_attn_run(&p, st, 8, q_rows, &t, &sp);
}

extern "C" int pikv_shard_decode_combine(const pikv_shard_decode_ctx* c, const int32_t* topk_idx, const float* topk_w,
                                         const int32_t* pair_len, void* out, float* lse_out, int32_t mode,
                                         pikv_stream_t stream) {
    SDCtx x;
    int rc = sd_check(c, &x, "shard_decode_combine");
    if (rc != PIKV_OK) return rc;
    PIKV_REQUIRE(topk_idx && topk_w && pair_len && out, PIKV_EINVAL, "shard_decode_combine: null pointer");
    PIKV_REQUIRE(mode == 0 || mode == 1, PIKV_EINVAL, "shard_decode_combine: mode must be 0 (weighted sum) or 1 (log-sum-exp merge)");
    const int units = c->streams_per_rank * c->n_q, per_cta = SD_COMBINE_THREADS / 32;
    const int ctas = min((units + per_cta - 1) / per_cta, sm_count() * 4);
    shard_decode_combine_kernel<<<ctas, SD_COMBINE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        x, topk_idx, topk_w, pair_len, static_cast<__nv_bfloat16*>(out), lse_out, mode);
    count_launch(1);
    return check_launch("shard_decode_combine_kernel");
}

extern "C" size_t pikv_shard_decode_buffer_bytes(int32_t what, int32_t world, int32_t num_streams, int32_t top_k, int32_t n_q) {
    if (world <= 0 || num_streams <= 0 || top_k <= 0 || n_q <= 0 || num_streams % world != 0) return 0;
    const size_t sl = (size_t)(num_streams / world);
    switch (what) {
        case 0: return (size_t)num_streams * n_q * 128 * 2;               // q
        case 1: return (size_t)num_streams * top_k * 16;                   // route
        case 2: return (size_t)world * 4;                                  // post flags
        case 3: return sl * top_k * world * n_q * 128 * sizeof(float);     // part_o
        case 4: return sl * top_k * world * n_q * sizeof(float);           // part_lse
        case 5: return (size_t)world * 4;                                  // done flags
        default: return 0;
    }
}
