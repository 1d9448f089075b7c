// Routed KV append fused with per-(token, head) quantisation, and the logical read-back.
//
// Work unit = the K and the V slice of one (token, head): two groups of 128 channels handled
// by 8 lanes that each own 16 consecutive channels of both: four 16-byte loads of bf16 in,
// one 16-byte (int8) or 8-byte (int4) store of codes per tensor and destination out.  The 8 lanes of a group write one full
// 128-byte row of the destination page, so stores are whole lines even though the
// destinations are scattered.  The group statistics are a 3-step xor shuffle.
#include "quant_group.cuh"
#include "gate_common.cuh"

namespace pikv {

constexpr int APPEND_THREADS = 256;
constexpr int D = PIKV_HEAD_DIM;        // 128 channels per group
constexpr int PT = PIKV_PAGE_TOKENS;    // 16 tokens per page
constexpr int APPEND_MAX_K = 8;          // destinations per token

struct AppendDev {
    const void* k;
    const void* v;
    int T, n_kv, top_k, log2_nkv;
    const int* dst_seq;
    const int* slot;
    const int* page_table;
    int num_seqs, max_pages, num_pages;
    uint8_t* codes[2];
    uint16_t* scale[2];
    float* zp[2];
    unsigned* status;
    // expert-sharded variant: destination pools live on the rank that owns the sequence
    int world, per, capacity;
    int rank, which;             // which: 0 every destination, 1 only this rank's sequences, 2 only the other ranks'
    const int* slot_base;        // [num_seqs] added to the slot
    uint8_t* pcodes[2][8];       // [K|V][rank] peer-mapped code pools
    uint16_t* pscale[2][8];
    uint16_t* mirror[2];         // local [world][pool] copies that take the scales of remote rows (or null)
    size_t mirror_stride;        // entries per rank in a mirror
    // striped variant (MODE 3): dst_seq holds the expert, slot the row's position in the (expert, stream) pair
    int st_experts, st_mul, st_add, st_log2;   // pair = expert * st_mul + stream; stream = token_stream[t] or st_add
    const int* st_rot;           // [experts] rotation of every expert
    const int* st_cap;           // [experts] rows a pair of that expert may hold, or null
    const int* st_stream;        // [T] stream of every token, or null
    // rotary variant (MODE 4): K is rotated before it is quantised
    const float* rope_cos;       // [max_pos][64]
    const float* rope_sin;
    const int* rope_pos;         // [T] position of every token, or null (position = token index)
    int rope_max_pos;
    // fused route + append: the gate left chunk-local ranks in `slot` and per-chunk counters behind
    const int* g_cta_cnt;        // [G][E]
    const int* g_cta_cnt_k;      // [G][k][E]
    const float* g_cta_psum;     // [G][E]
    const int* g_slot_base;      // [E] or null
    int gG, gchunk, gE, gcap;
    int* g_slot_out;             // [T][k] final slots
    int* g_counts_k;
    float* g_prob_sum;
    int* g_new_len;
};

// One 8-lane group per (token, head) item: both the K and the V slice of that head.  The grid is
// persistent (three CTAs per SM) and every group walks its items with a stride of the whole grid
// in a three-deep software pipeline, so that no load is consumed in the iteration that issued it:
//   item i+2   slot / destination-sequence loads
//   item i+1   page-table loads (addresses from the values fetched one iteration earlier) and the
//              four 16-byte K/V loads
//   item i     statistics, codes, stores
template <int TOPK>
struct AppendRoute {
    int s[TOPK];     // slot, -1 = dropped
    int q[TOPK];     // destination sequence
};

__device__ __forceinline__ void append_split(const AppendDev& a, unsigned pair, unsigned& t, unsigned& head) {
    if (a.log2_nkv >= 0) {
        t = pair >> a.log2_nkv;
        head = pair & ((1u << a.log2_nkv) - 1u);
    } else {
        t = pair / (unsigned)a.n_kv;
        head = pair % (unsigned)a.n_kv;
    }
}

template <int TOPK>
__device__ __forceinline__ void append_stage_route(const AppendDev& a, unsigned pair, unsigned total, AppendRoute<TOPK>& r) {
    unsigned t = 0, head = 0;
    const bool active = pair < total;
    if (active) append_split(a, pair, t, head);
#pragma unroll
    for (int j = 0; j < TOPK; ++j) {
        const bool on = active && j < a.top_k;
        r.s[j] = on ? __ldg(a.slot + (size_t)t * a.top_k + j) : -1;
        r.q[j] = on ? __ldg(a.dst_seq + (size_t)t * a.top_k + j) : 0;
    }
}

// K / V loads of an item: independent of the routing
template <typename TIn, int BITS, bool SYM>
__device__ __forceinline__ void append_stage_kv(const AppendDev& a, unsigned pair, unsigned total, int sub,
                                                typename GroupQuant<TIn, BITS, SYM>::Raw& k,
                                                typename GroupQuant<TIn, BITS, SYM>::Raw& v) {
    unsigned t = 0, head = 0;
    if (pair < total) append_split(a, pair, t, head);
    const size_t off = ((size_t)t * a.n_kv + head) * D + sub * 16;
    GroupQuant<TIn, BITS, SYM>::load(static_cast<const TIn*>(a.k) + off, k);
    GroupQuant<TIn, BITS, SYM>::load(static_cast<const TIn*>(a.v) + off, v);
}

// final slot (MODE 1: + this rank's base on the owner; MODE 2: + exclusive prefix of the gate's
// per-chunk counters, from shared memory) and the page-table load
template <int TOPK, int MODE>
__device__ __forceinline__ void append_stage_page(const AppendDev& a, unsigned pair, unsigned total, int sub,
                                                  AppendRoute<TOPK>& r, int (&page)[TOPK], const int* base_s) {
    unsigned t = 0, head = 0;
    if (pair < total) append_split(a, pair, t, head);
#pragma unroll
    for (int j = 0; j < TOPK; ++j) {
        page[j] = -1;
        if (MODE == 1 && r.s[j] >= 0 && r.q[j] >= 0 && r.q[j] < a.num_seqs) {
            const int sf = r.s[j] + __ldg(a.slot_base + r.q[j]);
            r.s[j] = (a.capacity > 0 && sf >= a.capacity) ? -1 : sf;
            const bool mine = r.q[j] / a.per == a.rank;
            if ((a.which == 1 && !mine) || (a.which == 2 && mine)) r.s[j] = -1;
        }
        if (MODE == 3 && r.s[j] >= 0) {
            // owner rank and slot on it of row r.s[j] of pair (expert r.q[j], stream): stripes of 2^st_log2 rows
            // rotate over the ranks from (rot[expert] + stream) mod world; the owner travels in bits 27..29
            const int e = r.q[j];
            if (e < 0 || e >= a.st_experts) {
                if (a.status && sub == 0 && head == 0) atomicOr(a.status, PIKV_ST_BAD_SEQ);
                r.s[j] = -1;
            } else {
                const int stream = a.st_stream ? __ldg(a.st_stream + t) : a.st_add;
                const int pos = r.s[j] + (a.slot_base ? __ldg(a.slot_base + e) : 0);
                const int c = pos >> a.st_log2;
                const int owner = (int)((unsigned)(__ldg(a.st_rot + e) + stream + c) % (unsigned)a.world);
                const int local = ((c / a.world) << a.st_log2) | (pos & ((1 << a.st_log2) - 1));
                const bool mine = owner == a.rank;
                const bool drop = (a.st_cap && pos >= __ldg(a.st_cap + e)) || local >= (1 << 27) ||
                                  (a.which == 1 && !mine) || (a.which == 2 && mine);
                r.s[j] = drop ? -1 : (local | (owner << 27));
                r.q[j] = e * a.st_mul + stream;
            }
        }
        if (MODE == 2 && r.s[j] >= 0 && r.q[j] >= 0 && r.q[j] < a.gE) {
            const int sf = r.s[j] + base_s[(t / (unsigned)a.gchunk) * a.gE + r.q[j]];
            r.s[j] = (a.gcap > 0 && sf >= a.gcap) ? -1 : sf;
            if (head == 0 && sub == 0 && a.g_slot_out) a.g_slot_out[(size_t)t * a.top_k + j] = r.s[j];
        }
        if (r.s[j] >= 0) {
            const int sl = MODE == 3 ? (r.s[j] & ((1 << 27) - 1)) : r.s[j];
            if (r.q[j] < 0 || r.q[j] >= a.num_seqs || (sl / PT) >= a.max_pages) {
                if (a.status && sub == 0 && head == 0) atomicOr(a.status, PIKV_ST_BAD_SEQ);
            } else {
                page[j] = __ldg(a.page_table + (size_t)r.q[j] * a.max_pages + sl / PT);
            }
        }
    }
}

// MODE 0: slots as given.  MODE 1: expert-sharded (peer pools, per-rank slot base).  MODE 2: fused with
// the gate (chunk-local ranks + per-chunk counters -> final slots, totals by CTA 0).
template <typename TIn, int BITS, bool SYM, int TOPK, int MODE>
__device__ __forceinline__ void kv_append_body(const AppendDev& a) {
    constexpr int ROW_BYTES = D * BITS / 8;
    constexpr bool SHARDED = MODE == 1 || MODE == 3;
    using GQ = GroupQuant<TIn, BITS, SYM>;
    extern __shared__ int base_s[];                        // MODE 2: [G][E] first slot of every chunk
    const int sub = threadIdx.x & 7;                       // lane within the group
    const unsigned stride = gridDim.x * (unsigned)(APPEND_THREADS / 8);
    const unsigned total = (unsigned)a.T * (unsigned)a.n_kv;
    unsigned pair = (blockIdx.x * (unsigned)APPEND_THREADS + threadIdx.x) >> 3;
    // the four groups of a warp hold consecutive items: the loop condition is warp-uniform
    unsigned warp_first = (blockIdx.x * (unsigned)APPEND_THREADS + (threadIdx.x & ~31u)) >> 3;
    const bool any = warp_first < total;

    AppendRoute<TOPK> r0, r1, r2;
    int pg0[TOPK], pg1[TOPK];
    typename GQ::Raw k0, v0, k1, v1;
    // prologue: the loads that need nothing from the gate go out first
    if (any) append_stage_kv<TIn, BITS, SYM>(a, pair, total, sub, k0, v0);
    // MODE 2 is launched as a programmatic dependent of the gate kernel: its CTAs may become resident, and their
    // first K/V loads go out, while the gate is still running; everything the gate writes is read after this wait
    // (which returns at once when the launch carried no such dependency)
    if (MODE == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (any) {
        append_stage_route<TOPK>(a, pair, total, r0);
        append_stage_route<TOPK>(a, pair + stride, total, r1);
    }
    if (MODE == 2) {
        // exclusive prefix over the gate's chunks, per expert: warp w scans experts w, w+8, ...
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
        const int G = a.gG, E = a.gE;
        for (int i = tid; i < G * E; i += APPEND_THREADS) base_s[i] = __ldg(a.g_cta_cnt + i);
        __syncthreads();
        for (int e = warp; e < E; e += APPEND_THREADS / 32) {
            int carry = a.g_slot_base ? __ldg(a.g_slot_base + e) : 0;
            for (int c0 = 0; c0 < G; c0 += 32) {
                const int c = c0 + lane;
                const int v = c < G ? base_s[c * E + e] : 0;
                int inc = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int n = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += n;
                }
                if (c < G) base_s[c * E + e] = carry + inc - v;
                carry += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (blockIdx.x == 0 && lane == 0 && a.g_new_len)
                a.g_new_len[e] = (a.gcap > 0 && carry > a.gcap) ? a.gcap : carry;
        }
        __syncthreads();
        // totals of the routing step: one (column, expert) count or one expert's probability sum per CTA,
        // every thread a fixed subset of the chunks and a fixed reduction tree (run-to-run identical bits)
        __shared__ float tot_f[APPEND_THREADS / 32];
        __shared__ int tot_i[APPEND_THREADS / 32];
        const int n_cnt = a.top_k * E;
        for (int item = blockIdx.x; item < n_cnt + E; item += gridDim.x) {
            int si = 0;
            float sf = 0.f;
            if (item < n_cnt) {
                const int j = item / E, e = item % E;
                for (int c = tid; c < G; c += APPEND_THREADS) si += __ldg(a.g_cta_cnt_k + ((size_t)c * a.top_k + j) * E + e);
            } else {
                for (int c = tid; c < G; c += APPEND_THREADS) sf += __ldg(a.g_cta_psum + (size_t)c * E + (item - n_cnt));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                si += __shfl_xor_sync(0xffffffffu, si, o);
                sf += __shfl_xor_sync(0xffffffffu, sf, o);
            }
            __syncthreads();
            if (lane == 0) tot_i[warp] = si, tot_f[warp] = sf;
            __syncthreads();
            if (tid == 0) {
                int ti = 0;
                float tf = 0.f;
                for (int w = 0; w < APPEND_THREADS / 32; ++w) ti += tot_i[w], tf += tot_f[w];
                if (item < n_cnt) {
                    if (a.g_counts_k) a.g_counts_k[item] = ti;
                } else if (a.g_prob_sum) {
                    a.g_prob_sum[item - n_cnt] = tf;
                }
            }
        }
    }
    if (!any) return;
    append_stage_page<TOPK, MODE>(a, pair, total, sub, r0, pg0, base_s);

    while (warp_first < total) {
        append_stage_route<TOPK>(a, pair + 2 * stride, total, r2);
        if (warp_first + stride < total) {
            append_stage_kv<TIn, BITS, SYM>(a, pair + stride, total, sub, k1, v1);
            append_stage_page<TOPK, MODE>(a, pair + stride, total, sub, r1, pg1, base_s);
        }

        QParams kq, vq;
        uint32_t kw[4], vw[4];
        if constexpr (MODE == 4) {
            // rotary position embedding on K (core/single/pikv_attention.py:329-390: halves split at 64, cos / sin
            // from the caller's tables, every product and sum a separately rounded fp32 operation), then the
            // fp32 quantisation path: the rotated K never exists in bf16
            const uint32_t ww[8] = {k0.a.x, k0.a.y, k0.a.z, k0.a.w, k0.b.x, k0.b.y, k0.b.z, k0.b.w};
            float x[16], out[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) bf16x2_to_f32(ww[i], x[2 * i], x[2 * i + 1]);
            unsigned t = 0, head = 0;
            if (pair < total) append_split(a, pair, t, head);
            int pos = a.rope_pos ? __ldg(a.rope_pos + t) : (int)t;
            pos = max(0, min(pos, a.rope_max_pos - 1));
            const float4* c4 = reinterpret_cast<const float4*>(a.rope_cos + (size_t)pos * 64 + 16 * (sub & 3));
            const float4* s4 = reinterpret_cast<const float4*>(a.rope_sin + (size_t)pos * 64 + 16 * (sub & 3));
            const float sign = sub < 4 ? -1.0f : 1.0f;           // top half: x cos - partner sin; bottom: x cos + partner sin
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 c = __ldg(c4 + i), sn = __ldg(s4 + i);
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float partner = __shfl_xor_sync(0xffffffffu, x[4 * i + e], 4);
                    out[4 * i + e] = __fadd_rn(__fmul_rn(x[4 * i + e], cc[e]), __fmul_rn(sign * partner, ss[e]));
                }
            }
            float mn, mx;
            qg_group_minmax(out, mn, mx);
            qg_quantize16<8, true>(out, mn, mx, kq, kw);
        } else {
            GQ::quant(k0, kq, kw);
        }
        GQ::quant(v0, vq, vw);
        const uint16_t ks_bits = qg_bf16_bits(kq.scale), vs_bits = qg_bf16_bits(vq.scale);
        if (pair < total) {
            unsigned t, head;
            append_split(a, pair, t, head);
#pragma unroll
            for (int j = 0; j < TOPK; ++j) {
                if (r0.s[j] < 0 || pg0[j] < 0) continue;
                if (pg0[j] >= a.num_pages) {
                    if (a.status && sub == 0 && head == 0) atomicOr(a.status, PIKV_ST_BAD_PAGE);
                    continue;
                }
                const int row = r0.s[j] % PT;
                const size_t prow = ((size_t)pg0[j] * a.n_kv + head) * PT + row;
                if (SHARDED) {
                    // the owner's pools, mapped into this GPU's address space: plain stores over NVLink
                    const int owner = MODE == 3 ? (r0.s[j] >> 27) : r0.q[j] / a.per;
                    const size_t o = prow * ROW_BYTES + 16 * swz8_chunk(row, sub);
                    *reinterpret_cast<uint4*>(a.pcodes[0][owner] + o) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
                    *reinterpret_cast<uint4*>(a.pcodes[1][owner] + o) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
                    if (sub == 0) {
                        // a 2-byte store costs the link as much as a 128-byte one: with mirrors the scales of
                        // remote rows stay here and shard_push_scales_kernel ships them 32 bytes at a time
                        if (a.mirror[0] != nullptr && owner != a.rank) {
                            a.mirror[0][(size_t)owner * a.mirror_stride + prow] = ks_bits;
                            a.mirror[1][(size_t)owner * a.mirror_stride + prow] = vs_bits;
                        } else {
                            a.pscale[0][owner][prow] = ks_bits;
                            a.pscale[1][owner][prow] = vs_bits;
                        }
                    }
                    continue;
                }
                if (BITS == 8) {
                    const size_t o = prow * ROW_BYTES + 16 * swz8_chunk(row, sub);
                    *reinterpret_cast<uint4*>(a.codes[0] + o) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
                    *reinterpret_cast<uint4*>(a.codes[1] + o) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
                } else {
                    const size_t o = prow * ROW_BYTES + 8 * swz4_unit(row, sub);
                    *reinterpret_cast<uint2*>(a.codes[0] + o) = make_uint2(kw[0], kw[1]);
                    *reinterpret_cast<uint2*>(a.codes[1] + o) = make_uint2(vw[0], vw[1]);
                }
                if (sub == 0) {
                    a.scale[0][prow] = ks_bits;
                    a.scale[1][prow] = vs_bits;
                    if (!SYM) {
                        a.zp[0][prow] = kq.zp;
                        a.zp[1][prow] = vq.zp;
                    }
                }
            }
        }
        // rotate the pipeline
        r0 = r1; r1 = r2;
        k0 = k1; v0 = v1;
#pragma unroll
        for (int j = 0; j < TOPK; ++j) pg0[j] = pg1[j];
        pair += stride;
        warp_first += stride;
    }
}

template <typename TIn, int BITS, bool SYM, int TOPK, int MODE>
__global__ void __launch_bounds__(APPEND_THREADS, 3) kv_append_quant_kernel(AppendDev a) {
    kv_append_body<TIn, BITS, SYM, TOPK, MODE>(a);
}

// ---- logical read-back ----------------------------------------------------------------
// One 8-lane group per (row i, head): un-swizzle, unpack, dequantise with the stored
// bf16 scale / fp32 zero point.
__global__ void cache_gather_kernel(const int* seq, const int* pos, int n, const int* page_table, int num_seqs,
                                    int max_pages, int num_pages, int n_kv, int bits, const uint8_t* codes,
                                    const uint16_t* scale, const float* zp, float* out, int8_t* codes_out,
                                    unsigned* status) {
    const int sub = threadIdx.x & 7;
    const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    if (group >= (long long)n * n_kv) return;
    const int i = (int)(group / n_kv), head = (int)(group % n_kv);
    const int s = seq[i], p = pos[i];
    if (s < 0 || s >= num_seqs || p < 0 || p / PT >= max_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_SEQ);
        return;
    }
    const int page = page_table[(size_t)s * max_pages + p / PT];
    if (page < 0 || page >= num_pages) {
        if (status && sub == 0) atomicOr(status, PIKV_ST_BAD_PAGE);
        return;
    }
    const int row = p % PT;
    const size_t prow = ((size_t)page * n_kv + head) * PT + row;
    const float sc = bf16_bits_to_f32(scale[prow]);
    const float z = zp ? zp[prow] : 0.f;
    int q[16];
    if (bits == 8) {
        uint4 w = *reinterpret_cast<const uint4*>(codes + prow * D + 16 * swz8_chunk(row, sub));
        uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            int b = (ww[c >> 2] >> (8 * (c & 3))) & 0xff;
            q[c] = zp ? b : (int)(int8_t)b;
        }
    } else {
        uint2 w = *reinterpret_cast<const uint2*>(codes + prow * (D / 2) + 8 * swz4_unit(row, sub));
        uint32_t ww[2] = {w.x, w.y};
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            int b = (ww[c >> 3] >> (4 * (c & 7))) & 0xf;
            q[c] = zp ? b : ((b ^ 8) - 8);
        }
    }
    const size_t o = ((size_t)i * n_kv + head) * D + sub * 16;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        if (out) out[o + c] = __fmul_rn(__fsub_rn((float)q[c], z), sc);
        if (codes_out) codes_out[o + c] = (int8_t)q[c];
    }
}

static void append_clear_gate(AppendDev& a) {
    a.g_cta_cnt = a.g_cta_cnt_k = a.g_slot_base = nullptr;
    a.g_cta_psum = nullptr;
    a.gG = a.gchunk = a.gE = a.gcap = 0;
    a.g_slot_out = a.g_counts_k = a.g_new_len = nullptr;
    a.g_prob_sum = nullptr;
}

// the part of the launch arguments every variant shares: inputs, geometry, local pools; no sharding, no gate
static void append_fill_common(const pikv_append_params* p, AppendDev& a) {
    a.k = p->k; a.v = p->v; a.T = p->T; a.n_kv = p->n_kv; a.top_k = p->top_k;
    a.log2_nkv = -1;
    for (int b = 0; b < 16; ++b)
        if ((1 << b) == p->n_kv) a.log2_nkv = b;
    a.dst_seq = p->dst_seq; a.slot = p->slot; a.page_table = p->page_table;
    a.num_seqs = p->num_seqs; a.max_pages = p->max_pages; a.num_pages = p->num_pages;
    a.codes[0] = static_cast<uint8_t*>(p->k_codes); a.codes[1] = static_cast<uint8_t*>(p->v_codes);
    a.scale[0] = static_cast<uint16_t*>(p->k_scale); a.scale[1] = static_cast<uint16_t*>(p->v_scale);
    a.zp[0] = static_cast<float*>(p->k_zp); a.zp[1] = static_cast<float*>(p->v_zp);
    a.status = p->status;
    a.world = 1; a.per = p->num_seqs; a.capacity = 0; a.slot_base = nullptr; a.rank = 0; a.which = 0;
    a.mirror[0] = a.mirror[1] = nullptr; a.mirror_stride = 0;
    for (int r = 0; r < 8; ++r) a.pcodes[0][r] = a.pcodes[1][r] = nullptr, a.pscale[0][r] = a.pscale[1][r] = nullptr;
    a.st_experts = a.st_mul = a.st_add = a.st_log2 = 0;
    a.st_rot = a.st_cap = a.st_stream = nullptr;
    a.rope_cos = a.rope_sin = nullptr; a.rope_pos = nullptr; a.rope_max_pos = 0;
    append_clear_gate(a);
}

template <typename TIn>
static int launch_append(const AppendDev& a, int bits, int symmetric, cudaStream_t st) {
    const long long lanes = (long long)a.T * a.n_kv * 8;
    // persistent: at most three resident CTAs per SM, each group strides over its items
    long long want = ceil_div64(lanes, APPEND_THREADS), cap_ctas = (long long)sm_count() * 3;
    const int grid = (int)(want < cap_ctas ? want : cap_ctas);
#define PIKV_APPEND_LAUNCH(BITS, SYM)                                                                   \
    do {                                                                                                \
        if (a.top_k <= 1) kv_append_quant_kernel<TIn, BITS, SYM, 1, 0><<<grid, APPEND_THREADS, 0, st>>>(a);      \
        else if (a.top_k <= 2) kv_append_quant_kernel<TIn, BITS, SYM, 2, 0><<<grid, APPEND_THREADS, 0, st>>>(a); \
        else if (a.top_k <= 4) kv_append_quant_kernel<TIn, BITS, SYM, 4, 0><<<grid, APPEND_THREADS, 0, st>>>(a); \
        else kv_append_quant_kernel<TIn, BITS, SYM, 8, 0><<<grid, APPEND_THREADS, 0, st>>>(a);                   \
    } while (0)
    if (bits == 8 && symmetric) PIKV_APPEND_LAUNCH(8, true);
    else if (bits == 8) PIKV_APPEND_LAUNCH(8, false);
    else if (symmetric) PIKV_APPEND_LAUNCH(4, true);
    else PIKV_APPEND_LAUNCH(4, false);
#undef PIKV_APPEND_LAUNCH
    count_launch(1);
    return check_launch("kv_append_quant_kernel");
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_kv_append_quant(const pikv_append_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "append: null params");
    PIKV_REQUIRE(p->T >= 0 && p->n_kv > 0 && p->top_k > 0, PIKV_EINVAL, "append: bad sizes");
    PIKV_REQUIRE(p->top_k <= APPEND_MAX_K, PIKV_ELIMIT, "append: top_k=%d exceeds %d", p->top_k, APPEND_MAX_K);
    if (p->T == 0) return PIKV_OK;
    PIKV_REQUIRE(p->k && p->v && p->dst_seq && p->slot && p->page_table, PIKV_EINVAL, "append: null input pointer");
    PIKV_REQUIRE(p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL, "append: null cache pointer");
    PIKV_REQUIRE(p->bits == 8 || p->bits == 4, PIKV_EUNSUPPORTED, "append: bits=%d (8 or 4)", p->bits);
    PIKV_REQUIRE(p->symmetric || (p->k_zp && p->v_zp), PIKV_EINVAL, "append: asymmetric needs zero-point pools");
    PIKV_REQUIRE(p->dtype == PIKV_BF16 || p->dtype == PIKV_F32, PIKV_EINVAL, "append: bad dtype %d", p->dtype);
    PIKV_REQUIRE(p->num_seqs > 0 && p->max_pages > 0 && p->num_pages > 0, PIKV_EINVAL, "append: bad cache geometry");
    PIKV_REQUIRE((long long)p->T * p->n_kv < (1ll << 28), PIKV_ELIMIT, "append: T * n_kv must stay below 2^28 per call");
    PIKV_REQUIRE((long long)p->num_pages * p->n_kv * PT < (1ll << 31), PIKV_ELIMIT, "append: page pool too large for 32-bit row indices");
    AppendDev a;
    append_fill_common(p, a);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->dtype == PIKV_BF16) return launch_append<__nv_bfloat16>(a, p->bits, p->symmetric, st);
    return launch_append<float>(a, p->bits, p->symmetric, st);
}

// ---- rotary embedding + quantise + append ---------------------------------------------------------------
extern "C" int pikv_kv_append_rope(const pikv_append_params* p, const float* rope_cos, const float* rope_sin,
                                   const int32_t* positions, int32_t max_pos, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "append_rope: null params");
    PIKV_REQUIRE(p->T >= 0 && p->n_kv > 0 && p->top_k > 0 && p->top_k <= APPEND_MAX_K, PIKV_EINVAL, "append_rope: bad sizes");
    if (p->T == 0) return PIKV_OK;
    PIKV_REQUIRE(p->k && p->v && p->dst_seq && p->slot && p->page_table && rope_cos && rope_sin, PIKV_EINVAL,
                 "append_rope: null input pointer");
    PIKV_REQUIRE(p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL, "append_rope: null cache pointer");
    PIKV_REQUIRE(p->dtype == PIKV_BF16 && p->bits == 8 && p->symmetric, PIKV_EUNSUPPORTED,
                 "append_rope: bf16 inputs, int8 symmetric codes only");
    PIKV_REQUIRE(max_pos > 0, PIKV_EINVAL, "append_rope: max_pos must be positive");
    PIKV_REQUIRE((reinterpret_cast<uintptr_t>(rope_cos) & 15) == 0 && (reinterpret_cast<uintptr_t>(rope_sin) & 15) == 0, PIKV_EINVAL,
                 "append_rope: the cos / sin tables must be 16-byte aligned");
    PIKV_REQUIRE(p->num_seqs > 0 && p->max_pages > 0 && p->num_pages > 0, PIKV_EINVAL, "append_rope: bad cache geometry");
    PIKV_REQUIRE((long long)p->T * p->n_kv < (1ll << 28) && (long long)p->num_pages * p->n_kv * PT < (1ll << 31), PIKV_ELIMIT,
                 "append_rope: problem too large for one call");
    AppendDev a;
    append_fill_common(p, a);
    a.rope_cos = rope_cos; a.rope_sin = rope_sin; a.rope_pos = positions; a.rope_max_pos = max_pos;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long lanes = (long long)a.T * a.n_kv * 8;
    long long want = ceil_div64(lanes, APPEND_THREADS), cap_ctas = (long long)sm_count() * 3;
    const int grid = (int)(want < cap_ctas ? want : cap_ctas);
    if (a.top_k <= 1) kv_append_quant_kernel<__nv_bfloat16, 8, true, 1, 4><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 2) kv_append_quant_kernel<__nv_bfloat16, 8, true, 2, 4><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 4) kv_append_quant_kernel<__nv_bfloat16, 8, true, 4, 4><<<grid, APPEND_THREADS, 0, st>>>(a);
    else kv_append_quant_kernel<__nv_bfloat16, 8, true, 8, 4><<<grid, APPEND_THREADS, 0, st>>>(a);
    count_launch(1);
    return check_launch("kv_append_quant_kernel (rotary)");
}

// ---- fused route + append ---------------------------------------------------------------------------
// Gate kernel, then the append kernel finishes the gate's slot scan itself: every append CTA rebuilds the
// exclusive prefix of the per-chunk counters in shared memory while its first K/V loads are in flight,
// adds it to the chunk-local ranks (kept in the gate's workspace), writes the final slots to the gate's slot
// output and stores the rows.  One launch and one dependent kernel boundary less than pikv_gate_fused +
// pikv_kv_append_quant, identical results.
static bool route_fusable(const pikv_gate_params* gp, const pikv_append_params* ap) {
    if (!(ap->dtype == PIKV_BF16 && ap->bits == 8 && ap->symmetric)) return false;
    GateDev g;
    if (gate_run(gp, nullptr, GATE_RANKS_TO_WS, &g) != PIKV_OK) return false;   // the gate launch reports the error
    return (size_t)g.G * g.E * sizeof(int) <= 40 * 1024;                                // prefix table in shared memory
}

static int route_check(const pikv_gate_params* gp, const pikv_append_params* ap, pikv_append_params* plain) {
    PIKV_REQUIRE(gp != nullptr && ap != nullptr, PIKV_EINVAL, "route_append: null params");
    PIKV_REQUIRE(gp->phase == PIKV_GATE_WHOLE, PIKV_EINVAL, "route_append: the gate's phase must be PIKV_GATE_WHOLE");
    PIKV_REQUIRE(gp->slot != nullptr && gp->topk_idx != nullptr, PIKV_EINVAL, "route_append: the gate's topk_idx and slot outputs are required");
    PIKV_REQUIRE(ap->T == gp->T && ap->top_k == gp->top_k && ap->num_seqs == gp->E, PIKV_EINVAL,
                 "route_append: gate and append disagree on T, top_k or the number of sequences");
    *plain = *ap;
    plain->dst_seq = gp->topk_idx;
    plain->slot = gp->slot;
    return PIKV_OK;
}

extern "C" int pikv_route_append(const pikv_gate_params* gp, const pikv_append_params* ap, pikv_stream_t stream) {
    pikv_append_params plain;
    int rc = route_check(gp, ap, &plain);
    if (rc != PIKV_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!route_fusable(gp, ap)) {
        rc = gate_run(gp, st, GATE_DO_SCORE | GATE_DO_SLOTS, nullptr);
        return rc != PIKV_OK ? rc : pikv_kv_append_quant(&plain, stream);
    }
    GateDev g;
    rc = gate_run(gp, st, GATE_DO_SCORE | GATE_RANKS_TO_WS, &g);
    if (rc != PIKV_OK) return rc;
    const size_t smem = (size_t)g.G * g.E * sizeof(int);
    const pikv_append_params* p = &plain;
    PIKV_REQUIRE(p->T > 0 && p->n_kv > 0 && p->top_k > 0 && p->top_k <= APPEND_MAX_K, PIKV_EINVAL, "route_append: bad sizes");
    PIKV_REQUIRE(p->k && p->v && p->page_table && p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL,
                 "route_append: null pointer");
    PIKV_REQUIRE((long long)p->T * p->n_kv < (1ll << 28) && (long long)p->num_pages * p->n_kv * PT < (1ll << 31), PIKV_ELIMIT,
                 "route_append: problem too large for one call");
    AppendDev a;
    append_fill_common(p, a);
    a.zp[0] = a.zp[1] = nullptr;
    a.g_cta_cnt = g.cta_cnt; a.g_cta_cnt_k = g.cta_cnt_k; a.g_cta_psum = g.cta_psum; a.g_slot_base = g.slot_base;
    a.gG = g.G; a.gchunk = g.chunk; a.gE = g.E; a.gcap = g.capacity;
    a.slot = g.slot;               // chunk-local ranks, in the gate's workspace
    a.g_slot_out = gp->slot; a.g_counts_k = g.counts_k; a.g_prob_sum = g.prob_sum; a.g_new_len = g.new_len;
    const long long lanes = (long long)a.T * a.n_kv * 8;
    long long want = ceil_div64(lanes, APPEND_THREADS), cap_ctas = (long long)sm_count() * 3;
    const int grid = (int)(want < cap_ctas ? want : cap_ctas);
    // programmatic dependent launch: the append CTAs are scheduled as soon as every gate CTA has started (the gate
    // kernel signals that at its top), so the launch latency and the first loads overlap the gate's tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(APPEND_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le;
    if (a.top_k <= 1) le = cudaLaunchKernelEx(&cfg, kv_append_quant_kernel<__nv_bfloat16, 8, true, 1, 2>, a);
    else if (a.top_k <= 2) le = cudaLaunchKernelEx(&cfg, kv_append_quant_kernel<__nv_bfloat16, 8, true, 2, 2>, a);
    else if (a.top_k <= 4) le = cudaLaunchKernelEx(&cfg, kv_append_quant_kernel<__nv_bfloat16, 8, true, 4, 2>, a);
    else le = cudaLaunchKernelEx(&cfg, kv_append_quant_kernel<__nv_bfloat16, 8, true, 8, 2>, a);
    (void)le;                      // reported by check_launch
    count_launch(1);
    return check_launch("kv_append_quant_kernel (fused with the gate)");
}

// ---- expert-sharded append: plan + launch -----------------------------------------------------------
// One CTA: from the all-gathered per-rank selection counts, the slot at which this rank's first row
// of every sequence lands on its owner (rows are ordered by source rank), and the new lengths.
__global__ void shard_plan_kernel(const int* gathered, int world, int E, int rank, int capacity, int* len_all,
                                  int* slot_base) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    int before = 0, total = 0;
    for (int s = 0; s < world; ++s) {
        const int c = gathered[s * E + e];
        if (s < rank) before += c;
        total += c;
    }
    const int len = len_all[e];
    slot_base[e] = len + before;
    const int n = len + total;
    len_all[e] = (capacity > 0 && n > capacity) ? capacity : n;
}

extern "C" int pikv_shard_plan(const int32_t* gathered, int32_t world, int32_t E, int32_t rank, int32_t capacity,
                               int32_t* len_all, int32_t* slot_base, pikv_stream_t stream) {
    PIKV_REQUIRE(gathered && len_all && slot_base, PIKV_EINVAL, "shard_plan: null pointer");
    PIKV_REQUIRE(world > 0 && E > 0 && rank >= 0 && rank < world, PIKV_EINVAL, "shard_plan: bad sizes");
    shard_plan_kernel<<<ceil_div(E, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(gathered, world, E, rank, capacity,
                                                                                       len_all, slot_base);
    count_launch(1);
    return check_launch("shard_plan_kernel");
}

// ---- count exchange + plan in one kernel, over peer memory ---------------------------------------------
// Each rank owns a ring of PIKV_XCHG_RING gather slots [world][E] and flags [world] in memory every peer
// has mapped.  One CTA per rank: sum this rank's selection counts over the k columns, store them into
// slot (step % ring) of EVERY rank's gather buffer (plain stores over NVLink), fence, raise the step
// number in every rank's flag word; then wait, with a limit, until all ranks' flags of that slot show
// this step, and compute slot_base / len_all from the local copy as shard_plan_kernel does.  A rank can
// be at most one step ahead of the slowest (its next plan needs that rank's next counts), so a ring of
// four never overwrites unread counts.
// Failure: if the wait runs out, every slot_base is set to the capacity (all rows of the step are
// dropped), PIKV_ST_WAIT_TIMEOUT is raised and the rank marks itself failed (top bit of *seq).  A failed
// rank keeps publishing, with the top bit of its flag set; a rank that sees that bit fails the same way
// at once.  So within one more step every rank's status word shows the failure, and from the failing step
// on the cache is invalid on all of them until a step with start_empty clears the marks.
constexpr unsigned XCHG_FAILED = 0x80000000u;

__device__ __forceinline__ void peer_flag_store(unsigned* flag, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned peer_flag_load(const unsigned* flag) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    return v;
}
// polls (1 us apart) until the low 31 bits of *flag reach `want`; returns the last value seen
__device__ __forceinline__ unsigned peer_flag_wait(const unsigned* flag, unsigned want, unsigned limit_us) {
    unsigned seen = 0;
    for (unsigned spins = 0;; ++spins) {
        seen = peer_flag_load(flag);
        if ((seen & ~XCHG_FAILED) == want || spins >= limit_us) break;
        __nanosleep(1000);
    }
    return seen;
}
static unsigned wait_limit(int32_t limit_us) { return limit_us > 0 ? (unsigned)limit_us : PIKV_DEFAULT_WAIT_US; }

__global__ void __launch_bounds__(256) shard_exchange_plan_kernel(pikv_shard_exchange_params p, unsigned limit_us) {
    __shared__ unsigned step_s, failed_s;
    const int tid = threadIdx.x;
    if (tid == 0) {
        const unsigned prev = *p.seq;
        step_s = (prev & ~XCHG_FAILED) + 1u;
        failed_s = p.start_empty ? 0u : (prev & XCHG_FAILED);
    }
    __syncthreads();
    const unsigned step = step_s & ~XCHG_FAILED;
    const unsigned was_failed = failed_s;
    const int ring = (int)(step % PIKV_XCHG_RING);
    const int E = p.E, W = p.world;
    for (int e = tid; e < E; e += blockDim.x) {
        int c = 0;
        for (int j = 0; j < p.top_k; ++j) c += p.counts_k[j * E + e];
        for (int r = 0; r < W; ++r) p.peer_gather[r][((size_t)ring * W + p.rank) * E + e] = c;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W) {
        peer_flag_store(p.peer_flags[tid] + ring * W + p.rank, step | was_failed);
        const unsigned seen = peer_flag_wait(p.peer_flags[p.rank] + ring * W + tid, step, limit_us);
        if ((seen & ~XCHG_FAILED) != step || (seen & XCHG_FAILED)) atomicOr(&failed_s, XCHG_FAILED);
    }
    __syncthreads();
    const bool ok = failed_s == 0;
    if (tid == 0) {
        *p.seq = step | failed_s;
        if (!ok && p.status) atomicOr(p.status, PIKV_ST_WAIT_TIMEOUT);
    }
    const int* gathered = p.peer_gather[p.rank] + (size_t)ring * W * E;
    for (int e = tid; e < E; e += blockDim.x) {
        int before = 0, total = 0;
        for (int s = 0; s < W; ++s) {
            const int c = __ldcg(gathered + s * E + e);   // written by peers: read at L2
            if (s < p.rank) before += c;
            total += c;
        }
        const int len = p.start_empty ? 0 : p.len_all[e];
        if (!ok) {
            p.slot_base[e] = p.capacity > 0 ? p.capacity : 0x3fffffff;
            if (p.start_empty) p.len_all[e] = 0;
            continue;
        }
        p.slot_base[e] = len + before;
        const int n = len + total;
        p.len_all[e] = (p.capacity > 0 && n > p.capacity) ? p.capacity : n;
    }
}

extern "C" int pikv_shard_exchange_plan(const pikv_shard_exchange_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "shard_exchange_plan: null params");
    PIKV_REQUIRE(p->counts_k && p->seq && p->len_all && p->slot_base, PIKV_EINVAL, "shard_exchange_plan: null pointer");
    PIKV_REQUIRE(p->world >= 1 && p->world <= 8 && p->rank >= 0 && p->rank < p->world && p->E > 0 && p->top_k > 0,
                 PIKV_EINVAL, "shard_exchange_plan: bad sizes");
    for (int r = 0; r < p->world; ++r)
        PIKV_REQUIRE(p->peer_gather[r] && p->peer_flags[r], PIKV_EINVAL, "shard_exchange_plan: null peer buffer for rank %d", r);
    shard_exchange_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(*p, wait_limit(p->wait_limit_us));
    count_launch(1);
    return check_launch("shard_exchange_plan_kernel");
}

// ---- barrier over peer memory --------------------------------------------------------------------------
// Every rank raises its step number in every rank's flag word and waits, with a limit, for all of them:
// the kernels queued before it on this stream on every rank (and their stores into peer memory) are complete
// when it returns.  A wait that runs out raises PIKV_ST_WAIT_TIMEOUT and returns; nothing spins for ever.
__global__ void __launch_bounds__(32) peer_barrier_kernel(pikv_peer_barrier_params p, unsigned limit_us) {
    const int tid = threadIdx.x;
    const unsigned step = (*p.seq & ~XCHG_FAILED) + 1u;
    __threadfence_system();
    __syncwarp();
    bool ok = true;
    if (tid < p.world) {
        peer_flag_store(p.peer_flags[tid] + p.rank, step);
        ok = (peer_flag_wait(p.peer_flags[p.rank] + tid, step, limit_us) & ~XCHG_FAILED) == step;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (tid == 0) {
        *p.seq = step;
        if (!ok && p.status) atomicOr(p.status, PIKV_ST_WAIT_TIMEOUT);
    }
}

extern "C" int pikv_peer_barrier(const pikv_peer_barrier_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr && p->seq != nullptr, PIKV_EINVAL, "peer_barrier: null params");
    PIKV_REQUIRE(p->world >= 1 && p->world <= 8 && p->rank >= 0 && p->rank < p->world, PIKV_EINVAL, "peer_barrier: bad sizes");
    for (int r = 0; r < p->world; ++r)
        PIKV_REQUIRE(p->peer_flags[r] != nullptr, PIKV_EINVAL, "peer_barrier: null flag buffer for rank %d", r);
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*p, wait_limit(p->wait_limit_us));
    count_launch(1);
    return check_launch("peer_barrier_kernel");
}

// ---- scales of the rows this rank stored on other GPUs --------------------------------------------------
// The append left them in the local mirrors, at the offsets they have in the owner's pools.  This rank's
// rows of sequence e occupy the slots [slot_base[e], slot_base[e] + count[e]) (cut at the capacity), i.e.
// whole pages except at the two ends, and one (page, head) holds its 16 scales in 32 contiguous bytes: one
// thread ships one (sequence, page, head) run, K and V, as two 16-byte stores when the page is whole and
// entry by entry at the ends (the neighbouring entries there belong to other ranks).
__global__ void __launch_bounds__(256) shard_push_scales_kernel(pikv_shard_push_params p) {
    const int e = blockIdx.x;
    const int owner = e / p.seqs_per_rank;
    if (owner == p.rank) return;
    int cnt = 0;
    for (int j = 0; j < p.top_k; ++j) cnt += p.counts_k[j * p.E + e];
    const int a = p.slot_base[e];
    int b = a + cnt;
    if (p.capacity > 0) b = min(b, p.capacity);
    if (b <= a) return;
    const int p0 = a / PT, p1 = (b - 1) / PT;
    const size_t mirror_stride = (size_t)p.num_pages * p.n_kv * PT;
    const uint16_t* mk = static_cast<const uint16_t*>(p.mirror_k_scale) + (size_t)owner * mirror_stride;
    const uint16_t* mv = static_cast<const uint16_t*>(p.mirror_v_scale) + (size_t)owner * mirror_stride;
    uint16_t* dk = static_cast<uint16_t*>(p.peer_k_scale[owner]);
    uint16_t* dv = static_cast<uint16_t*>(p.peer_v_scale[owner]);
    const int runs = (p1 - p0 + 1) * p.n_kv;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < runs; i += gridDim.y * blockDim.x) {
        const int pi = p0 + i / p.n_kv, head = i % p.n_kv;
        if (pi >= p.max_pages) continue;
        const int page = p.page_table[(size_t)e * p.max_pages + pi];
        if (page < 0 || page >= p.num_pages) continue;      // the append kernel has already raised PIKV_ST_BAD_PAGE
        const int lo = max(a - pi * PT, 0), hi = min(b - pi * PT, PT);
        const size_t off = ((size_t)page * p.n_kv + head) * PT;
        if (lo == 0 && hi == PT) {
            const uint4* sk = reinterpret_cast<const uint4*>(mk + off);
            const uint4* sv = reinterpret_cast<const uint4*>(mv + off);
            uint4* tk = reinterpret_cast<uint4*>(dk + off);
            uint4* tv = reinterpret_cast<uint4*>(dv + off);
            tk[0] = sk[0]; tk[1] = sk[1];
            tv[0] = sv[0]; tv[1] = sv[1];
        } else {
            for (int r = lo; r < hi; ++r) {
                dk[off + r] = mk[off + r];
                dv[off + r] = mv[off + r];
            }
        }
    }
}

extern "C" int pikv_shard_push_scales(const pikv_shard_push_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "shard_push_scales: null params");
    PIKV_REQUIRE(p->counts_k && p->slot_base && p->page_table && p->mirror_k_scale && p->mirror_v_scale, PIKV_EINVAL,
                 "shard_push_scales: null pointer");
    PIKV_REQUIRE(p->world >= 1 && p->world <= 8 && p->rank >= 0 && p->rank < p->world && p->seqs_per_rank > 0 &&
                     p->E == p->world * p->seqs_per_rank && p->top_k > 0 && p->n_kv > 0 && p->max_pages > 0 && p->num_pages > 0,
                 PIKV_EINVAL, "shard_push_scales: bad sizes");
    for (int r = 0; r < p->world; ++r)
        PIKV_REQUIRE(p->peer_k_scale[r] && p->peer_v_scale[r], PIKV_EINVAL, "shard_push_scales: null pool pointer for rank %d", r);
    if (p->world == 1) return PIKV_OK;
    dim3 grid(p->E, 4);
    shard_push_scales_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(*p);
    count_launch(1);
    return check_launch("shard_push_scales_kernel");
}

extern "C" int pikv_kv_append_sharded(const pikv_append_sharded_params* sp, pikv_stream_t stream) {
    PIKV_REQUIRE(sp != nullptr, PIKV_EINVAL, "append_sharded: null params");
    const pikv_append_params* p = &sp->base;
    PIKV_REQUIRE(p->T >= 0 && p->n_kv > 0 && p->top_k > 0 && p->top_k <= APPEND_MAX_K, PIKV_EINVAL, "append_sharded: bad sizes");
    if (p->T == 0) return PIKV_OK;
    PIKV_REQUIRE(p->k && p->v && p->dst_seq && p->slot && p->page_table && sp->slot_base, PIKV_EINVAL,
                 "append_sharded: null input pointer");
    PIKV_REQUIRE(p->dtype == PIKV_BF16 && p->bits == 8 && p->symmetric, PIKV_EUNSUPPORTED,
                 "append_sharded: bf16 inputs, int8 symmetric codes only");
    PIKV_REQUIRE(sp->world >= 1 && sp->world <= 8 && sp->seqs_per_rank > 0 && p->num_seqs == sp->world * sp->seqs_per_rank,
                 PIKV_EINVAL, "append_sharded: world must be 1..8 and num_seqs = world * seqs_per_rank");
    PIKV_REQUIRE((long long)p->T * p->n_kv < (1ll << 28), PIKV_ELIMIT, "append_sharded: T * n_kv must stay below 2^28");
    AppendDev a;
    append_fill_common(p, a);
    a.codes[0] = a.codes[1] = nullptr; a.scale[0] = a.scale[1] = nullptr; a.zp[0] = a.zp[1] = nullptr;   // peer pools only
    a.world = sp->world; a.per = sp->seqs_per_rank; a.capacity = sp->capacity; a.slot_base = sp->slot_base;
    PIKV_REQUIRE(sp->which >= 0 && sp->which <= 2 && (sp->which == 0 || (sp->rank >= 0 && sp->rank < sp->world)), PIKV_EINVAL,
                 "append_sharded: which must be 0..2 (and rank valid when it is not 0)");
    a.rank = sp->rank; a.which = sp->which;
    PIKV_REQUIRE((sp->mirror_k_scale == nullptr) == (sp->mirror_v_scale == nullptr), PIKV_EINVAL,
                 "append_sharded: give both scale mirrors or neither");
    PIKV_REQUIRE(sp->mirror_k_scale == nullptr || (sp->rank >= 0 && sp->rank < sp->world), PIKV_EINVAL,
                 "append_sharded: rank is required with scale mirrors");
    a.mirror[0] = static_cast<uint16_t*>(sp->mirror_k_scale); a.mirror[1] = static_cast<uint16_t*>(sp->mirror_v_scale);
    a.mirror_stride = (size_t)p->num_pages * p->n_kv * PT;
    for (int r = 0; r < 8; ++r) {
        const bool on = r < sp->world;
        PIKV_REQUIRE(!on || (sp->peer_k_codes[r] && sp->peer_v_codes[r] && sp->peer_k_scale[r] && sp->peer_v_scale[r]),
                     PIKV_EINVAL, "append_sharded: null pool pointer for rank %d", r);
        a.pcodes[0][r] = on ? static_cast<uint8_t*>(sp->peer_k_codes[r]) : nullptr;
        a.pcodes[1][r] = on ? static_cast<uint8_t*>(sp->peer_v_codes[r]) : nullptr;
        a.pscale[0][r] = on ? static_cast<uint16_t*>(sp->peer_k_scale[r]) : nullptr;
        a.pscale[1][r] = on ? static_cast<uint16_t*>(sp->peer_v_scale[r]) : nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long lanes = (long long)a.T * a.n_kv * 8;
    // two CTAs per SM: the link, not the SMs, bounds this launch (one, two and three per SM measured within 5 %),
    // and kernels of the other steps in flight still find room beside them
    long long want = ceil_div64(lanes, APPEND_THREADS), cap_ctas = (long long)sm_count() * 2;
    const int grid = (int)(want < cap_ctas ? want : cap_ctas);
    if (a.top_k <= 1) kv_append_quant_kernel<__nv_bfloat16, 8, true, 1, 1><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 2) kv_append_quant_kernel<__nv_bfloat16, 8, true, 2, 1><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 4) kv_append_quant_kernel<__nv_bfloat16, 8, true, 4, 1><<<grid, APPEND_THREADS, 0, st>>>(a);
    else kv_append_quant_kernel<__nv_bfloat16, 8, true, 8, 1><<<grid, APPEND_THREADS, 0, st>>>(a);
    count_launch(1);
    return check_launch("kv_append_quant_kernel (sharded)");
}

// ---- striped expert-sharded append ---------------------------------------------------------------------
extern "C" int pikv_kv_append_striped(const pikv_append_striped_params* sp, pikv_stream_t stream) {
    PIKV_REQUIRE(sp != nullptr, PIKV_EINVAL, "append_striped: null params");
    const pikv_append_params* p = &sp->base;
    PIKV_REQUIRE(p->T >= 0 && p->n_kv > 0 && p->top_k > 0 && p->top_k <= APPEND_MAX_K, PIKV_EINVAL, "append_striped: bad sizes");
    if (p->T == 0) return PIKV_OK;
    PIKV_REQUIRE(p->k && p->v && p->dst_seq && p->slot && p->page_table && sp->expert_rot, PIKV_EINVAL,
                 "append_striped: null input pointer");
    PIKV_REQUIRE(p->dtype == PIKV_BF16 && p->bits == 8 && p->symmetric, PIKV_EUNSUPPORTED,
                 "append_striped: bf16 inputs, int8 symmetric codes only");
    PIKV_REQUIRE(sp->world >= 1 && sp->world <= 8 && sp->rank >= 0 && sp->rank < sp->world, PIKV_EINVAL,
                 "append_striped: world must be 1..8 and rank inside it");
    PIKV_REQUIRE(sp->num_experts > 0 && sp->num_streams > 0 && p->num_seqs == sp->num_experts * sp->num_streams, PIKV_EINVAL,
                 "append_striped: num_seqs must be num_experts * num_streams");
    PIKV_REQUIRE(sp->token_stream != nullptr || (sp->stream >= 0 && sp->stream < sp->num_streams), PIKV_EINVAL,
                 "append_striped: give token_stream or a valid stream");
    int log2 = -1;
    for (int b = 4; b < 27; ++b)
        if ((1 << b) == sp->stripe) log2 = b;
    PIKV_REQUIRE(log2 > 0, PIKV_EINVAL, "append_striped: stripe=%d must be a power of two >= 16", sp->stripe);
    PIKV_REQUIRE(sp->which >= 0 && sp->which <= 2, PIKV_EINVAL, "append_striped: which must be 0..2");
    PIKV_REQUIRE((long long)p->T * p->n_kv < (1ll << 28), PIKV_ELIMIT, "append_striped: T * n_kv must stay below 2^28");
    PIKV_REQUIRE((long long)p->num_pages * p->n_kv * PT < (1ll << 31), PIKV_ELIMIT, "append_striped: page pool too large for 32-bit row indices");
    AppendDev a;
    append_fill_common(p, a);
    a.codes[0] = a.codes[1] = nullptr; a.scale[0] = a.scale[1] = nullptr; a.zp[0] = a.zp[1] = nullptr;   // peer pools only
    a.world = sp->world; a.rank = sp->rank; a.which = sp->which; a.per = 1; a.capacity = 0;
    a.slot_base = sp->pair_len;
    a.st_experts = sp->num_experts; a.st_mul = sp->num_streams; a.st_add = sp->stream; a.st_log2 = log2;
    a.st_rot = sp->expert_rot; a.st_cap = sp->expert_cap; a.st_stream = sp->token_stream;
    PIKV_REQUIRE((sp->mirror_k_scale == nullptr) == (sp->mirror_v_scale == nullptr), PIKV_EINVAL,
                 "append_striped: give both scale mirrors or neither");
    a.mirror[0] = static_cast<uint16_t*>(sp->mirror_k_scale); a.mirror[1] = static_cast<uint16_t*>(sp->mirror_v_scale);
    a.mirror_stride = (size_t)p->num_pages * p->n_kv * PT;
    for (int r = 0; r < 8; ++r) {
        const bool on = r < sp->world;
        PIKV_REQUIRE(!on || (sp->peer_k_codes[r] && sp->peer_v_codes[r] && sp->peer_k_scale[r] && sp->peer_v_scale[r]),
                     PIKV_EINVAL, "append_striped: null pool pointer for rank %d", r);
        a.pcodes[0][r] = on ? static_cast<uint8_t*>(sp->peer_k_codes[r]) : nullptr;
        a.pcodes[1][r] = on ? static_cast<uint8_t*>(sp->peer_v_codes[r]) : nullptr;
        a.pscale[0][r] = on ? static_cast<uint16_t*>(sp->peer_k_scale[r]) : nullptr;
        a.pscale[1][r] = on ? static_cast<uint16_t*>(sp->peer_v_scale[r]) : nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long lanes = (long long)a.T * a.n_kv * 8;
    long long want = ceil_div64(lanes, APPEND_THREADS), cap_ctas = (long long)sm_count() * (sp->world > 1 ? 2 : 3);
    const int grid = (int)(want < cap_ctas ? want : cap_ctas);
    if (a.top_k <= 1) kv_append_quant_kernel<__nv_bfloat16, 8, true, 1, 3><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 2) kv_append_quant_kernel<__nv_bfloat16, 8, true, 2, 3><<<grid, APPEND_THREADS, 0, st>>>(a);
    else if (a.top_k <= 4) kv_append_quant_kernel<__nv_bfloat16, 8, true, 4, 3><<<grid, APPEND_THREADS, 0, st>>>(a);
    else kv_append_quant_kernel<__nv_bfloat16, 8, true, 8, 3><<<grid, APPEND_THREADS, 0, st>>>(a);
    count_launch(1);
    return check_launch("kv_append_quant_kernel (striped)");
}

// ---- scales of the rows a striped append stored on other GPUs -------------------------------------------
// The append left them in the local mirrors at the offsets they have in the owner's pools (a 2-byte store costs
// the link as much as a 128-byte one).  The step appended positions [len_before[e], len_after[e]) to the pair of
// expert e; one thread ships the scales of one (expert, 16-position page, head): two 16-byte stores per tensor
// when the step wrote the whole page, entry by entry at the two ends of the range.
__global__ void __launch_bounds__(256) striped_push_scales_kernel(pikv_striped_push_params p, int log2_stripe) {
    const int e = blockIdx.x;
    const int a = p.len_before[e];
    int b = p.len_after[e];
    if (p.expert_cap) b = min(b, p.expert_cap[e]);
    if (b <= a) return;
    const int p0 = a / PT, p1 = (b - 1) / PT;
    const size_t mirror_stride = (size_t)p.num_pages * p.n_kv * PT;
    const int pair = e * p.num_streams + p.stream;
    const int rot = (p.expert_rot[e] + p.stream) % p.world;
    const int pages_per_stripe = 1 << (log2_stripe - 4);
    const int runs = (p1 - p0 + 1) * p.n_kv;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < runs; i += gridDim.y * blockDim.x) {
        const int pi = p0 + i / p.n_kv, head = i % p.n_kv;
        const int c = pi >> (log2_stripe - 4);                       // stripe of this page
        const int owner = (rot + c) % p.world;
        if (owner == p.rank) continue;                               // written in place by the append
        const int lp = (c / p.world) * pages_per_stripe + (pi & (pages_per_stripe - 1));
        if (lp >= p.max_pages) continue;
        const int page = p.page_table[(size_t)pair * p.max_pages + lp];
        if (page < 0 || page >= p.num_pages) continue;               // the append has raised PIKV_ST_BAD_PAGE
        const int lo = max(a - pi * PT, 0), hi = min(b - pi * PT, PT);
        const size_t off = ((size_t)page * p.n_kv + head) * PT;
        const uint16_t* mk = static_cast<const uint16_t*>(p.mirror_k_scale) + (size_t)owner * mirror_stride + off;
        const uint16_t* mv = static_cast<const uint16_t*>(p.mirror_v_scale) + (size_t)owner * mirror_stride + off;
        uint16_t* dk = static_cast<uint16_t*>(p.peer_k_scale[owner]) + off;
        uint16_t* dv = static_cast<uint16_t*>(p.peer_v_scale[owner]) + off;
        if (lo == 0 && hi == PT) {
            const uint4* sk = reinterpret_cast<const uint4*>(mk);
            const uint4* sv = reinterpret_cast<const uint4*>(mv);
            reinterpret_cast<uint4*>(dk)[0] = sk[0]; reinterpret_cast<uint4*>(dk)[1] = sk[1];
            reinterpret_cast<uint4*>(dv)[0] = sv[0]; reinterpret_cast<uint4*>(dv)[1] = sv[1];
        } else {
            for (int r = lo; r < hi; ++r) {
                dk[r] = mk[r];
                dv[r] = mv[r];
            }
        }
    }
}

extern "C" int pikv_shard_push_scales_striped(const pikv_striped_push_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "push_scales_striped: null params");
    PIKV_REQUIRE(p->len_before && p->len_after && p->expert_rot && p->page_table && p->mirror_k_scale && p->mirror_v_scale,
                 PIKV_EINVAL, "push_scales_striped: null pointer");
    PIKV_REQUIRE(p->world >= 1 && p->world <= 8 && p->rank >= 0 && p->rank < p->world && p->num_experts > 0 &&
                     p->num_streams > 0 && p->stream >= 0 && p->stream < p->num_streams && p->n_kv > 0 && p->max_pages > 0 &&
                     p->num_pages > 0,
                 PIKV_EINVAL, "push_scales_striped: bad sizes");
    int log2 = -1;
    for (int b = 4; b < 27; ++b)
        if ((1 << b) == p->stripe) log2 = b;
    PIKV_REQUIRE(log2 > 0, PIKV_EINVAL, "push_scales_striped: stripe=%d must be a power of two >= 16", p->stripe);
    for (int r = 0; r < p->world; ++r)
        PIKV_REQUIRE(p->peer_k_scale[r] && p->peer_v_scale[r], PIKV_EINVAL, "push_scales_striped: null pool pointer for rank %d", r);
    if (p->world == 1) return PIKV_OK;
    dim3 grid(p->num_experts, 4);
    striped_push_scales_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(*p, log2);
    count_launch(1);
    return check_launch("striped_push_scales_kernel");
}

extern "C" int pikv_cache_gather(const int32_t* seq, const int32_t* pos, int32_t n, const int32_t* page_table,
                                 int32_t num_seqs, int32_t max_pages, int32_t num_pages, int32_t n_kv, int32_t bits,
                                 const void* codes, const void* scale, const void* zp, float* out, int8_t* codes_out,
                                 uint32_t* status, pikv_stream_t stream) {
    PIKV_REQUIRE(n >= 0 && n_kv > 0, PIKV_EINVAL, "cache_gather: bad sizes");
    if (n == 0) return PIKV_OK;
    PIKV_REQUIRE(seq && pos && page_table && codes && scale, PIKV_EINVAL, "cache_gather: null pointer");
    PIKV_REQUIRE(out || codes_out, PIKV_EINVAL, "cache_gather: no output given");
    PIKV_REQUIRE(bits == 8 || bits == 4, PIKV_EUNSUPPORTED, "cache_gather: bits=%d", bits);
    const long long lanes = (long long)n * n_kv * 8;
    cache_gather_kernel<<<(int)ceil_div64(lanes, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        seq, pos, n, page_table, num_seqs, max_pages, num_pages, n_kv, bits, static_cast<const uint8_t*>(codes),
        static_cast<const uint16_t*>(scale), static_cast<const float*>(zp), out, codes_out, status);
    count_launch(1);
    return check_launch("cache_gather_kernel");
}
