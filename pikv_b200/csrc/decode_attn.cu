// Decode attention over the quantised paged cache (8-bit symmetric or 4-bit asymmetric codes),
// dequantised in registers.
//
// The pages of all requests form one list (per KV head), cut into blocks of equal length whatever the
// lengths of the requests; a work item is (block, head).  The grid is persistent (three CTAs of four warps per
// SM) and every WARP is a worker that claims items from a counter until none is left: fast and slow SMs even
// out, there is no wave quantisation and no tail, the eight heads of a block are claimed one after the other
// (so the heads of a page are read at about the same time), and a block may start and end in the middle of a
// request.  A worker streams its pages (16 tokens x 128 channels of K and of V plus their scales and, for 4
// bits, zero points) through a private ring in shared memory filled by bulk async copies (cp.async.bulk +
// mbarrier transaction counts), so the bytes in flight do not depend on registers and the stream does not
// stop at an item boundary; per page it runs 8 + 8 mma.m16n8k16 (f16 x f16 -> f32) and an online softmax in
// the log2 domain; see decode_attn_kernel.  For every request an item touches, the worker leaves one partial
// (O, m, l) in the workspace at slot (block + request, head), unique because both indices only grow along
// the list; a last kernel merges the partials of a (request, head).  A one-CTA plan kernel in front scans the
// request lengths, picks the block length and records where every block starts.
// Codes become f16 exactly with one byte-permute (bytes: 0x6400 | (code ^ 0x80) is 1024 + code + 128)
// or one AND-OR (nibbles: 0x6400 | n is 1024 + n).  Q is scaled by a power of two so that it is exact
// in f16.  The cache's swizzle makes the 16-byte shared-memory reads of a fragment conflict-free.
#include "common.cuh"

#include <mutex>

namespace pikv {

constexpr int DA_WARPS = 4;
constexpr int DA_THREADS = DA_WARPS * 32;
constexpr int DA_CTAS_PER_SM = 3;
constexpr int DA_MAX_GROUP = 8;
constexpr int DA_MIN_BLOCK = 16;                        // pages per block, at least (more than a ring holds)
constexpr int DA_ITEMS_PER_WORKER = 8;                  // blocks aimed at per worker of a head, at most
constexpr int DA_ITEM_PAGES = 48;                       // ... while an item keeps this many pages
constexpr int DA_MAX_REQ = 12000;                       // requests per call: their page prefix is scanned in shared memory
constexpr int DA_PLAN_THREADS = 1024;
constexpr int DA_FOLD_STEPS = 8;                        // softmax steps between two folds of the carried bias term
constexpr unsigned DA_WAIT_LIMIT = 1u << 24;            // mbarrier polls before giving up

struct DecodeDev {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    int B, n_q, n_kv, G;         // B = requests
    const int* seq_ids;
    const int* seq_len;
    const int* q_rows;           // request -> row of q (null: the request's own index)
    const int* page_table;
    int num_seqs, max_pages, num_pages;
    const uint8_t* k_codes;
    const uint8_t* v_codes;
    const uint16_t* k_scale;
    const uint16_t* v_scale;
    const float* k_zp;   // 4-bit asymmetric cache only
    const float* v_zp;
    float* lse;
    float* scores;
    int score_stride;
    __half* probs16;  // [B][n_q][probs_stride] exp2(score - step maximum) as f16, or null
    float* step_max;  // [B][n_q][step_stride] the step maximum (log2 domain) of every 16-position page
    int probs_stride, step_stride;
    int* head;        // workspace header: [0] item counter, [1] pages per block, [2] blocks (written by the plan kernel)
    int* prefix;      // [B+1] pages of the requests before each request
    int2* blk_start;  // [max_blocks] (request, page inside it) at which every block starts
    float* part_o;    // [(max_blocks + B) * n_kv][G][128]
    float* part_ml;   // [(max_blocks + B) * n_kv][G][2]  (running max in the log2 domain, denominator)
    int workers, max_blocks;
    unsigned* status;
};

}  // namespace pikv
#include "shard_decode.cuh"
namespace pikv {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: returns false when the limit is hit
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned i = 0; i < DA_WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// int8 x int8 -> int32, A = 16 rows x 32 bytes (row-major), B = 32 x 8 (column-major)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

// two biased bytes (code ^ 0x80) of w selected by SEL -> two exact f16 codes
template <uint32_t SEL>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w_biased) {
    uint32_t x = __byte_perm(w_biased, 0x64646464u, SEL);          // 0x64bb64bb = (1024 + b, 1024 + b)
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&x), __half2half2(__ushort_as_half(0x6480)));  // - 1152
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Geometry of one stage of a warp's ring: a page of one head.
//   8 bit: 16 rows x 128 B of K, of V, 16 + 16 bf16 scales
//   4 bit: 16 rows x 64 B (two codes per byte, low nibble = even channel, 8-byte units swizzled by
//          row & 4), scales, 16 + 16 fp32 zero points
template <int BITS> struct DAGeom;
template <> struct DAGeom<8> { static constexpr int STAGES = 4, ROW = 128, PAGE = 16 * 128, STAGE = 2 * PAGE + 64; };
template <> struct DAGeom<4> { static constexpr int STAGES = 6, ROW = 64, PAGE = 16 * 64, STAGE = 2 * PAGE + 64 + 128; };
constexpr int DA_PBUF_BYTES = DA_MAX_GROUP * 32 * 2;    // per warp: P of two pages, [head][32 positions] f16

template <int BITS>
constexpr size_t da_smem_bytes() {
    return (size_t)DA_WARPS * DAGeom<BITS>::STAGES * DAGeom<BITS>::STAGE + DA_WARPS * DAGeom<BITS>::STAGES * sizeof(uint64_t) +
           DA_WARPS * DA_PBUF_BYTES;
}

// nibbles at bits SHIFT and SHIFT + 16 of w -> (1024 + n, 1024 + n') as two f16: one shift and one AND-OR
template <int SHIFT>
__device__ __forceinline__ uint32_t nib_pair_biased(uint32_t w) {
    return ((w >> SHIFT) & 0x000f000fu) | 0x64006400u;
}
// ... and centred: 1032 = 1024 + 8 taken off again (exact), n - 8 in [-8, 7]
template <int SHIFT>
__device__ __forceinline__ uint32_t nib_pair(uint32_t w) {
    const uint32_t x = nib_pair_biased<SHIFT>(w);
    __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&x), __half2half2(__ushort_as_half(0x6408)));
    return *reinterpret_cast<uint32_t*>(&h);
}
// two bytes of w selected by SEL -> (1024 + b, 1024 + b') as two f16
template <uint32_t SEL>
__device__ __forceinline__ uint32_t bytes_to_h2_biased(uint32_t w) { return __byte_perm(w, 0x64646464u, SEL); }

// The legacy mma.sync path is what bounds this kernel on this GPU (one m16n8k16 holds a sub-core's tensor
// pipe for about 32 cycles), so the shapes are chosen to waste as few of its rows as possible:
//   S^T[pos, head] = Kcode[pos, :] . Q[head, :]    A = the page's 16 positions (all rows used), B = Q^T:
//                                                  8 mma per page
//   O^T[ch, head] += Vcode^T[ch, pos] . P'^T[pos, head]   A = 16 channels x 16 positions, 8 mma per page
// The softmax runs on S^T (a thread owns positions r, r+8 of heads 2j, 2j+1) and, for 8-bit codes, takes two
// pages (32 positions) per step; P goes through 512 bytes of shared memory to become the B operand of the
// second product.  Nothing but exact integers enters the tensor cores on the cache side:
//   q . x   = kscale * (q . code - zp * sum(q))                        (zp = 0 for the 8-bit cache)
//   P . x_c = sum_pos P' * (bias + code_c) - sum_pos P' * (bias + zp),  P' = P * vscale
// where bias is what the code -> f16 conversion leaves on: 1152 = 1024 + 128 for the bytes of V (one
// byte-permute, no subtraction), -8 for nibbles (centred, so that code - 8 and zp - 8 are small).  The second
// sum is the same for every channel: it is carried like the softmax denominator (corr) and taken off the
// accumulators every DA_FOLD_STEPS steps, so that they never hold more than a few pages' worth of bias (the
// tensor cores' fp32 accumulation truncates: a bias of 1152 x sum(P') carried over a 32768-token context
// costs about 1e-3 of the output scale with 4-bit scales, 1e-4 with 8-bit ones).
struct DACursor {
    int r, p;           // request, page inside it
    int pages, len;     // of request r
    int row;            // page-table row of request r, or -1
};
struct DAItem {
    int blk, h, left;   // block, KV head, pages of the item not yet issued / consumed
    DACursor cur;
};

// block of page f of the per-head page list
__device__ __forceinline__ int da_block_of(int f, int blk_pages, int nblocks) { return min(f / blk_pages, nblocks - 1); }

// One CTA: pages before every request (exclusive prefix), the block length, where every block starts; clears
// the item counter.  The prefix is scanned in shared memory (B <= DA_MAX_REQ).
// SHARD: the call is a rank's part of a sharded decode step, and the request list itself comes first: wait (bounded)
// for every rank's "posted" flag, then request i = (stream i / k, choice i % k) with the rows this rank holds of
// that pair as its length (a separate one-CTA kernel for this cost 5 us a step).
template <bool SHARD>
__global__ void __launch_bounds__(DA_PLAN_THREADS) decode_plan_kernel(DecodeDev d, ShardPlan sp) {
    extern __shared__ int pre[];
    __shared__ int wtot[DA_PLAN_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = d.B;
    const int max_len = d.max_pages * PIKV_PAGE_TOKENS;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the attention kernel may be scheduled
    if constexpr (SHARD) {
        __shared__ int ok_s;
        if (tid == 0) ok_s = 1;
        __syncthreads();
        const unsigned step = *sp.seq & ~SD_FAILED;
        if (tid < sp.world && !sd_flag_wait(sp.post_flags + tid, step, sp.limit_us)) {
            ok_s = 0;
            if (sp.status) atomicOr(sp.status, PIKV_ST_WAIT_TIMEOUT);
        }
        __syncthreads();
        const bool ok = ok_s != 0;
        for (int i = tid; i < R; i += DA_PLAN_THREADS) {
            const int4 rec = __ldcg(sp.route + i);               // written by a peer during this kernel: read at L2
            const int s = i / sp.top_k, e = rec.x;
            int len = 0;
            if (ok && e >= 0 && e < sp.num_experts)
                len = striped_local_len(rec.y, (sp.expert_rot[e] + s) % sp.world, sp.rank, sp.world, sp.log2_stripe);
            sp.seq_ids[i] = (e >= 0 && e < sp.num_experts) ? e * sp.num_streams + s : 0;
            sp.seq_len[i] = len;
            sp.q_rows[i] = s;
        }
        __syncthreads();                                         // d.seq_ids / d.seq_len are these arrays
    }
    for (int i = tid; i < R; i += DA_PLAN_THREADS) {
        const int seq = d.seq_ids ? d.seq_ids[i] : i;
        const bool ok = seq >= 0 && seq < d.num_seqs;
        if (!ok && d.status) atomicOr(d.status, PIKV_ST_BAD_SEQ);
        const int len = ok ? max(0, min(d.seq_len[i], max_len)) : 0;
        pre[i + 1] = (len + PIKV_PAGE_TOKENS - 1) / PIKV_PAGE_TOKENS;
    }
    if (tid == 0) pre[0] = 0;
    __syncthreads();
    {
        const int per = (R + DA_PLAN_THREADS - 1) / DA_PLAN_THREADS;
        const int lo = 1 + tid * per, hi = min(R + 1, lo + per);
        int sum = 0;
        for (int i = lo; i < hi; ++i) sum += pre[i];
        int inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) wtot[warp] = inc;
        __syncthreads();
        int run = inc - sum;
        for (int w = 0; w < warp; ++w) run += wtot[w];
        for (int i = lo; i < hi; ++i) {
            run += pre[i];
            pre[i] = run;
        }
    }
    __syncthreads();
    const int P = pre[R];
    // blocks per worker of a head: as many as DA_ITEMS_PER_WORKER when that leaves items of DA_ITEM_PAGES pages or
    // more (long lists: fast and slow SMs even out), down to two for short lists (an item start costs a few
    // dependent loads); the last block is the short one
    const int per_head = max(1, d.workers / d.n_kv);
    const int k_items = max(2, min(DA_ITEMS_PER_WORKER, P / (per_head * DA_ITEM_PAGES)));
    const int target = max(1, min(d.max_blocks, k_items * per_head));
    const int blk_pages = max(DA_MIN_BLOCK, (P + target - 1) / target);
    const int nblocks = (P + blk_pages - 1) / blk_pages;
    if (tid == 0) {
        d.head[0] = 0;
        d.head[1] = blk_pages;
        d.head[2] = nblocks;
    }
    for (int i = tid; i <= R; i += DA_PLAN_THREADS) d.prefix[i] = pre[i];
    for (int b = tid; b < nblocks; b += DA_PLAN_THREADS) {
        const int f = b * blk_pages;
        int lo = 0, hi = R - 1;                           // last request whose first page is at or before f
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (pre[mid] <= f) lo = mid; else hi = mid - 1;
        }
        d.blk_start[b] = make_int2(lo, f - pre[lo]);
    }
}

// GS (at most four query heads per KV head): the first product runs on the INTEGER tensor cores.  The cache's
// int8 codes (or the nibbles, split into bytes by one AND and one shift-AND per eight) are the A operand as they
// lie in shared memory, with no conversion at all; the query becomes a 15-bit integer u = rint(q * 2^(13-e))
// (2^e above the head's largest |q|: 6e-5 of that maximum, far below bf16's own 2^-8) cut into two int8 limbs,
// u = 128 hi + lo, which sit in neighbouring columns of the B operand, so ONE m16n8k32 yields both limbs of the
// four heads: 4 mma per page instead of 8, exact int32 sums, and a thread then owns one head at two positions
// (the f16 path spends half its softmax on padding heads).  The second product stays in f16 (P' is not an
// integer); the rescale factors travel from the thread that owns a head's statistics to the two threads that
// own its accumulators by two shuffles per step.
template <int BITS, bool GS>
__global__ void __launch_bounds__(DA_THREADS, DA_CTAS_PER_SM) decode_attn_kernel(DecodeDev d) {
    using GEO = DAGeom<BITS>;
    constexpr int STAGES = GEO::STAGES, STAGE_BYTES = GEO::STAGE, PAGE_BYTES = GEO::PAGE, ROW = GEO::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    // [warp][stage] rings, the barriers, the P buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)DA_WARPS * STAGES * STAGE_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, j = lane & 3;
    const int G = d.G, R = d.B, n_kv = d.n_kv;
    const int max_len = d.max_pages * PIKV_PAGE_TOKENS;
    // The three kernels of a call are chained by programmatic dependent launches: the merge kernel may be scheduled
    // from here on (it waits for this grid to complete), and this kernel's own set-up runs while the plan kernel
    // finishes; nothing the plan kernel wrote is read before the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    unsigned char* ring = smem + (size_t)warp * STAGES * STAGE_BYTES;
    __half* pbuf = reinterpret_cast<__half*>(reinterpret_cast<unsigned char*>(bars + DA_WARPS * STAGES) + warp * DA_PBUF_BYTES);
    const uint32_t bar0 = smem_u32(bars + warp * STAGES);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i2 = lane; i2 < DA_PBUF_BYTES / 4; i2 += 32) reinterpret_cast<uint32_t*>(pbuf)[i2] = 0u;   // rows of absent heads stay zero
    __syncwarp();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int blk_pages = __ldg(d.head + 1), nblocks = __ldg(d.head + 2), P = __ldg(d.prefix + R);
    const int nitems = nblocks * n_kv;

    auto request = [&](int rq, int& len, int& row) {          // clamped length and page-table row of a request
        const int seq = d.seq_ids ? __ldg(d.seq_ids + rq) : rq;
        const bool ok = seq >= 0 && seq < d.num_seqs;
        len = ok ? max(0, min(__ldg(d.seq_len + rq), max_len)) : 0;
        row = ok ? seq : -1;
    };
    // the next item of the list (warp-uniform); the claims of a block's heads go to consecutive callers
    auto claim = [&]() {
        int id = 0;
        if (lane == 0) id = atomicAdd(d.head, 1);
        return __shfl_sync(0xffffffffu, id, 0);
    };
    auto load_item = [&](int id, DAItem& it) {
        it.blk = id / n_kv;
        it.h = id % n_kv;
        const int2 st = __ldg(d.blk_start + it.blk);
        it.cur.r = st.x;
        it.cur.p = st.y;
        request(it.cur.r, it.cur.len, it.cur.row);
        it.cur.pages = (it.cur.len + PIKV_PAGE_TOKENS - 1) / PIKV_PAGE_TOKENS;
        it.left = it.blk == nblocks - 1 ? P - it.blk * blk_pages : blk_pages;
    };


    // moves a cursor `by` pages on (never across more than one request boundary)
    auto advance = [&](DACursor& x, int by) {
        x.p += by;
        if (x.p < x.pages) return;
        x.p = 0;
        do {
            if (++x.r >= R) { x.pages = 1 << 30; x.row = -1; return; }
            request(x.r, x.len, x.row);
            x.pages = (x.len + PIKV_PAGE_TOKENS - 1) / PIKV_PAGE_TOKENS;
        } while (x.pages == 0);
    };
    auto issue = [&](const DACursor& x, int h, int i) {   // lane 0 only: load the page under the cursor into stage i % STAGES
        const int s = i % STAGES;
        int page = x.row >= 0 ? __ldg(d.page_table + (size_t)x.row * d.max_pages + x.p) : -1;
        if (page < 0 || page >= d.num_pages) {
            if (d.status) atomicOr(d.status, PIKV_ST_BAD_PAGE);
            page = 0;
        }
        const size_t prow = ((size_t)page * n_kv + h) * PIKV_PAGE_TOKENS;
        const uint32_t dst = smem_u32(ring + (size_t)s * STAGE_BYTES);
        const uint32_t bar = bar0 + 8 * s;
        mbar_expect_tx(bar, STAGE_BYTES);
        bulk_g2s(dst, d.k_codes + prow * ROW, PAGE_BYTES, bar);
        bulk_g2s(dst + PAGE_BYTES, d.v_codes + prow * ROW, PAGE_BYTES, bar);
        bulk_g2s(dst + 2 * PAGE_BYTES, d.k_scale + prow, 32, bar);
        bulk_g2s(dst + 2 * PAGE_BYTES + 32, d.v_scale + prow, 32, bar);
        if (BITS == 4) {
            bulk_g2s(dst + 2 * PAGE_BYTES + 64, d.k_zp + prow, 64, bar);
            bulk_g2s(dst + 2 * PAGE_BYTES + 128, d.v_zp + prow, 64, bar);
        }
    };

    // Two walkers over this worker's items: `is` issues the copies and runs up to STAGES pages ahead of `c`,
    // which does the arithmetic.  The issuing side claims the items; an item it has entered and the other has
    // not yet is parked in pend_id (it never runs more than one item ahead).
    DAItem is, c;
    int next_id = claim();
    if (next_id >= nitems) return;
    load_item(next_id, is);
    c = is;
    next_id = claim();
    int pend_id = -1;
    int issued = 0, i = 0;                                 // pages issued / consumed by this worker so far
    auto top_up = [&]() {
        while (issued - i < STAGES) {
            if (is.left == 0) {
                if (pend_id >= 0 || next_id >= nitems) return;
                load_item(next_id, is);
                pend_id = next_id;
                next_id = claim();
            }
            if (lane == 0) issue(is.cur, is.h, issued);
            advance(is.cur, 1);
            --is.left;
            ++issued;
        }
    };
    top_up();

    uint32_t qf[GS ? 8 : 16];
    float qm0 = 0.f, qm1 = 0.f;   // per head 2j, 2j+1 (GS: head j in qm0): integer dot product -> log2-domain score
    float qs0 = 0.f, qs1 = 0.f;   // 4 bit: sum of the query over its 128 channels
    // ---- Q as the B operand: thread (r, j) holds channels 32j .. 32j+32 of column r ----
    //   f16 path: column r = head r, 16 f16 pairs.   GS: column r = limb (r & 1) of head r >> 1, 32 int8 in 8 words
    auto load_q = [&](int rq, int h) {
        float qv[32];
        const int qhead = GS ? (r >> 1) : r;
        if (qhead < G) {
            const int qrow = d.q_rows ? __ldg(d.q_rows + rq) : rq;
            const __nv_bfloat16* qp = d.q + ((size_t)qrow * d.n_q + (size_t)h * G + qhead) * 128 + 32 * j;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 wq = __ldg(reinterpret_cast<const uint4*>(qp) + i);
                bf16x2_to_f32(wq.x, qv[8 * i + 0], qv[8 * i + 1]);
                bf16x2_to_f32(wq.y, qv[8 * i + 2], qv[8 * i + 3]);
                bf16x2_to_f32(wq.z, qv[8 * i + 4], qv[8 * i + 5]);
                bf16x2_to_f32(wq.w, qv[8 * i + 6], qv[8 * i + 7]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) qv[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(qv[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        if constexpr (GS) {
            const int e = amax > 0.f ? ilogbf(amax) + 1 : 0;          // amax < 2^e
            const float up = ldexpf(1.0f, 13 - e);
            int u[32], usum = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int full = (int)rintf(qv[i] * up);               // |full| <= 8192
                const int lo = ((full + 64) & 127) - 64;               // [-64, 63]
                usum += full;
                u[i] = (r & 1) ? lo : ((full - lo) >> 7);              // hi in [-64, 64]
            }
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                // the channels behind the k index of mma m: bytes of this thread's word pair (2m, 2m+1) of the K row
                // (8 bit), or the even / odd nibbles of its word m (4 bit)
                if (BITS == 8) {
                    qf[2 * m] = pack4_s8(u[8 * m], u[8 * m + 1], u[8 * m + 2], u[8 * m + 3]);
                    qf[2 * m + 1] = pack4_s8(u[8 * m + 4], u[8 * m + 5], u[8 * m + 6], u[8 * m + 7]);
                } else {
                    qf[2 * m] = pack4_s8(u[8 * m], u[8 * m + 2], u[8 * m + 4], u[8 * m + 6]);
                    qf[2 * m + 1] = pack4_s8(u[8 * m + 1], u[8 * m + 3], u[8 * m + 5], u[8 * m + 7]);
                }
            }
            const float qmul = ldexpf(1.0f, e - 13) * 0.08838834764831845f * 1.4426950408889634f;
            qm0 = __shfl_sync(0xffffffffu, qmul, 8 * j);              // lane (column 2j = head j, channels 0..31)
            if (BITS == 4) {
                usum += __shfl_xor_sync(0xffffffffu, usum, 1);
                usum += __shfl_xor_sync(0xffffffffu, usum, 2);
                qs0 = (float)__shfl_sync(0xffffffffu, usum, 8 * j);
            }
            return;
        }
        int e = 0;
        if (amax > 32768.f) e = ilogbf(amax) - 14;     // a power of two keeps the bf16 query exact in f16
        const float down = ldexpf(1.0f, -e);
#pragma unroll
        for (int i = 0; i < (GS ? 0 : 16); ++i) {
            // 8 bit: consecutive channel pairs; 4 bit: pairs (c, c + 4) inside each group of 8, the order in
            // which nib_pair() takes nibbles out of a word
            const int cc = BITS == 8 ? 2 * i : 8 * (i >> 2) + (i & 3);
            const int c2 = BITS == 8 ? cc + 1 : cc + 4;
            qf[i] = pack_h2(qv[cc] * down, qv[c2] * down);
        }
        const float qmul = ldexpf(1.0f, e) * 0.08838834764831845f * 1.4426950408889634f;
        qm0 = __shfl_sync(0xffffffffu, qmul, 8 * j);          // lane of (head 2j, j = 0)
        qm1 = __shfl_sync(0xffffffffu, qmul, 8 * j + 4);
        if (BITS == 4) {
            float qs = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) qs += qv[i] * down;
            qs += __shfl_xor_sync(0xffffffffu, qs, 1);
            qs += __shfl_xor_sync(0xffffffffu, qs, 2);
            qs0 = __shfl_sync(0xffffffffu, qs, 8 * j);
            qs1 = __shfl_sync(0xffffffffu, qs, 8 * j + 4);
        }
    };

    float o[8][4];
    // running max, denominator and carried bias term of heads 2j and 2j+1 (this thread's share of the positions)
    float m0, m1, l0, l1, corr0, corr1;
    bool timed_out = false;

    // raw S^T of one page: this thread gets positions r (t[0], t[1]) and r+8 (t[2], t[3]) of heads 2j, 2j+1,
    // scaled to the log2 domain; vw = zero point of V minus 8 at those positions (4 bit)
    auto page_scores = [&](const unsigned char* st, float (&t)[4], float& vw_lo, float& vw_hi) {
        if constexpr (GS) {
            // integer path: t[0] / t[2] = head j at positions r / r+8 (t[1], t[3] unused)
            int acc[4] = {0, 0, 0, 0};
            if (BITS == 8) {
                const unsigned char* klo = st + r * 128;
                const unsigned char* khi = st + (r + 8) * 128;
                const uint4 la = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j) ^ r));
                const uint4 lb = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j + 1) ^ r));
                const uint4 ha = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j) ^ r));
                const uint4 hb = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j + 1) ^ r));
                const uint32_t wl[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
                const uint32_t wh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
                for (int m = 0; m < 4; ++m) mma_s8(acc, wl[2 * m], wh[2 * m], wl[2 * m + 1], wh[2 * m + 1], qf[2 * m], qf[2 * m + 1]);
            } else {
                const unsigned char* klo = st + r * 64;
                const unsigned char* khi = st + (r + 8) * 64;
                const uint4 lq = *reinterpret_cast<const uint4*>(klo + 8 * ((2 * j) ^ (r & 4)));
                const uint4 hq = *reinterpret_cast<const uint4*>(khi + 8 * ((2 * j) ^ (r & 4)));
                const uint32_t wl[4] = {lq.x, lq.y, lq.z, lq.w};
                const uint32_t wh[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    mma_s8(acc, wl[m] & 0x0f0f0f0fu, wh[m] & 0x0f0f0f0fu, (wl[m] >> 4) & 0x0f0f0f0fu, (wh[m] >> 4) & 0x0f0f0f0fu,
                           qf[2 * m], qf[2 * m + 1]);
            }
            const uint16_t* ksc = reinterpret_cast<const uint16_t*>(st + 2 * PAGE_BYTES);
            const float ks_lo = __uint_as_float((uint32_t)ksc[r] << 16), ks_hi = __uint_as_float((uint32_t)ksc[r + 8] << 16);
            t[0] = (float)(acc[0] * 128 + acc[1]);
            t[2] = (float)(acc[2] * 128 + acc[3]);
            if (BITS == 4) {
                const float* kzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 64);
                const float* vzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 128);
                t[0] -= kzp[r] * qs0;
                t[2] -= kzp[r + 8] * qs0;
                vw_lo = vzp[r] - 8.f;
                vw_hi = vzp[r + 8] - 8.f;
            }
            t[0] *= ks_lo * qm0;
            t[2] *= ks_hi * qm0;
            t[1] = t[3] = -INFINITY;
            return;
        }
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};      // two accumulator chains
        if (BITS == 8) {
            const unsigned char* klo = st + r * 128;
            const unsigned char* khi = st + (r + 8) * 128;           // same swizzle key: (r + 8) & 7 = r
            const uint4 la = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j) ^ r));
            const uint4 lb = *reinterpret_cast<const uint4*>(klo + 16 * ((2 * j + 1) ^ r));
            const uint4 ha = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j) ^ r));
            const uint4 hb = *reinterpret_cast<const uint4*>(khi + 16 * ((2 * j + 1) ^ r));
            const uint32_t wl[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
            const uint32_t wh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t a = wl[kk] ^ 0x80808080u, cw = wh[kk] ^ 0x80808080u;
                mma_f16((kk & 1) ? sb : sa, bytes_to_h2<0x4140>(a), bytes_to_h2<0x4140>(cw), bytes_to_h2<0x4342>(a),
                        bytes_to_h2<0x4342>(cw), qf[2 * kk], qf[2 * kk + 1]);
            }
        } else {
            const unsigned char* klo = st + r * 64;
            const unsigned char* khi = st + (r + 8) * 64;            // (r + 8) & 4 = r & 4
            const uint4 lq = *reinterpret_cast<const uint4*>(klo + 8 * ((2 * j) ^ (r & 4)));
            const uint4 hq = *reinterpret_cast<const uint4*>(khi + 8 * ((2 * j) ^ (r & 4)));
            const uint32_t wl[4] = {lq.x, lq.y, lq.z, lq.w};
            const uint32_t wh[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
            for (int wq = 0; wq < 4; ++wq) {
                mma_f16(sa, nib_pair<0>(wl[wq]), nib_pair<0>(wh[wq]), nib_pair<4>(wl[wq]), nib_pair<4>(wh[wq]), qf[4 * wq],
                        qf[4 * wq + 1]);
                mma_f16(sb, nib_pair<8>(wl[wq]), nib_pair<8>(wh[wq]), nib_pair<12>(wl[wq]), nib_pair<12>(wh[wq]),
                        qf[4 * wq + 2], qf[4 * wq + 3]);
            }
        }
        const uint16_t* ksc = reinterpret_cast<const uint16_t*>(st + 2 * PAGE_BYTES);
        const float ks_lo = __uint_as_float((uint32_t)ksc[r] << 16), ks_hi = __uint_as_float((uint32_t)ksc[r + 8] << 16);
        t[0] = sa[0] + sb[0]; t[1] = sa[1] + sb[1]; t[2] = sa[2] + sb[2]; t[3] = sa[3] + sb[3];
        if (BITS == 4) {
            const float* kzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 64);
            const float* vzp = reinterpret_cast<const float*>(st + 2 * PAGE_BYTES + 128);
            const float z_lo = kzp[r] - 8.f, z_hi = kzp[r + 8] - 8.f;          // the codes entered as code - 8
            t[0] -= z_lo * qs0; t[1] -= z_lo * qs1; t[2] -= z_hi * qs0; t[3] -= z_hi * qs1;
            vw_lo = vzp[r] - 8.f;
            vw_hi = vzp[r + 8] - 8.f;
        }
        t[0] *= ks_lo * qm0; t[1] *= ks_lo * qm1; t[2] *= ks_hi * qm0; t[3] *= ks_hi * qm1;
    };
    // masks the positions past the sequence end and writes the raw scores out when asked
    auto page_mask_scores = [&](int pos0, float (&t)[4]) {
        if (pos0 + PIKV_PAGE_TOKENS > c.cur.len) {
            if (pos0 + r >= c.cur.len) t[0] = t[1] = -INFINITY;
            if (pos0 + r + 8 >= c.cur.len) t[2] = t[3] = -INFINITY;
        }
        if (d.scores) {
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                if (GS && (cc & 1)) continue;
                const int hh = GS ? j : 2 * j + (cc & 1), pp = r + 8 * (cc >> 1);
                if (hh < G && pos0 + pp < c.cur.len && pos0 + pp < d.score_stride)
                    d.scores[((size_t)c.cur.r * d.n_q + (size_t)c.h * G + hh) * d.score_stride + pos0 + pp] = t[cc] * 0.6931471805599453f;
            }
        }
    };
    // O^T += (bias + Vcode)^T . P'^T for one page; pb0 / pb1 = P'[head r][positions 2j, 2j+1] / [2j+8, 2j+9]
    auto page_pv = [&](const unsigned char* st, uint32_t pb0, uint32_t pb1) {
        const unsigned char* vbase = st + PAGE_BYTES;
        const int pp[4] = {2 * j, 2 * j + 1, 8 + 2 * j, 9 + 2 * j};
        if (BITS == 8) {
            const uint4 v0 = *reinterpret_cast<const uint4*>(vbase + pp[0] * 128 + 16 * (r ^ (pp[0] & 7)));
            const uint4 v1 = *reinterpret_cast<const uint4*>(vbase + pp[1] * 128 + 16 * (r ^ (pp[1] & 7)));
            const uint4 v2 = *reinterpret_cast<const uint4*>(vbase + pp[2] * 128 + 16 * (r ^ (pp[2] & 7)));
            const uint4 v3 = *reinterpret_cast<const uint4*>(vbase + pp[3] * 128 + 16 * (r ^ (pp[3] & 7)));
            const uint32_t vw0[4] = {v0.x, v0.y, v0.z, v0.w}, vw1[4] = {v1.x, v1.y, v1.z, v1.w};
            const uint32_t vw2[4] = {v2.x, v2.y, v2.z, v2.w}, vw3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const int wi = m >> 1;
                // bytes (2*(m&1)) and (2*(m&1)+1) of the two positions of a pair, interleaved, then code + 128
                const uint32_t ta = ((m & 1) ? __byte_perm(vw0[wi], vw1[wi], 0x7362) : __byte_perm(vw0[wi], vw1[wi], 0x5140)) ^ 0x80808080u;
                const uint32_t tb = ((m & 1) ? __byte_perm(vw2[wi], vw3[wi], 0x7362) : __byte_perm(vw2[wi], vw3[wi], 0x5140)) ^ 0x80808080u;
                // channel 16r+2m (a0, a2) and 16r+2m+1 (a1, a3); positions 2j, 2j+1 (a0, a1) and 8+2j, 9+2j (a2, a3)
                mma_f16(o[m], bytes_to_h2_biased<0x4140>(ta), bytes_to_h2_biased<0x4342>(ta), bytes_to_h2_biased<0x4140>(tb),
                        bytes_to_h2_biased<0x4342>(tb), pb0, pb1);
            }
        } else {
            // channels 16r .. 16r+15 of the four positions: one 8-byte unit each
            const uint2 v0 = *reinterpret_cast<const uint2*>(vbase + pp[0] * 64 + 8 * (r ^ (pp[0] & 4)));
            const uint2 v1 = *reinterpret_cast<const uint2*>(vbase + pp[1] * 64 + 8 * (r ^ (pp[1] & 4)));
            const uint2 v2 = *reinterpret_cast<const uint2*>(vbase + pp[2] * 64 + 8 * (r ^ (pp[2] & 4)));
            const uint2 v3 = *reinterpret_cast<const uint2*>(vbase + pp[3] * 64 + 8 * (r ^ (pp[3] & 4)));
#pragma unroll
            for (int hb = 0; hb < 4; ++hb) {
                // bytes 2hb', 2hb'+1 of word wq of both positions of a pair: (p.b, p.b', p'.b, p'.b')
                const int wq = hb >> 1;
                const uint32_t sel = (hb & 1) ? 0x7632u : 0x5410u;
                const uint32_t ga = __byte_perm(wq ? v0.y : v0.x, wq ? v1.y : v1.x, sel);
                const uint32_t gb = __byte_perm(wq ? v2.y : v2.x, wq ? v3.y : v3.x, sel);
                const int m = 2 * hb;   // byte m of the unit: channels 16r+2m (low nibble), 16r+2m+1 (high nibble)
                mma_f16(o[m], nib_pair<0>(ga), nib_pair<4>(ga), nib_pair<0>(gb), nib_pair<4>(gb), pb0, pb1);
                mma_f16(o[m + 1], nib_pair<8>(ga), nib_pair<12>(ga), nib_pair<8>(gb), nib_pair<12>(gb), pb0, pb1);
            }
        }
    };
    // takes the carried bias term off the accumulators: its sum over the 8 lanes that share a head pair
    auto fold_bias = [&]() {
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            corr0 += __shfl_xor_sync(0xffffffffu, corr0, sh);
            corr1 += __shfl_xor_sync(0xffffffffu, corr1, sh);
        }
        float b0 = BITS == 8 ? corr0 * 1152.f : corr0, b1 = BITS == 8 ? corr1 * 1152.f : corr1;
        if constexpr (GS) {
            // statistics of head h live in the lanes with j == h; the accumulators of heads 2j, 2j+1 here
            const float mine = b0;
            b0 = __shfl_sync(0xffffffffu, mine, (lane & ~3) | ((2 * j) & 3));
            b1 = __shfl_sync(0xffffffffu, mine, (lane & ~3) | ((2 * j + 1) & 3));
        }
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            o[m][0] -= b0; o[m][1] -= b1; o[m][2] -= b0; o[m][3] -= b1;
        }
        corr0 = corr1 = 0.f;
    };

    // 8 bit: two pages (32 positions) per step of the online softmax, i.e. one max reduction and one rescale of
    // O for both; the 4-bit kernel is faster with one
    constexpr int PPS = BITS == 8 ? 2 : 1;
    while (!timed_out) {
        if (c.left == 0) {                                 // next item, if the issuing side has entered one
            if (pend_id < 0) top_up();
            if (pend_id < 0) break;
            load_item(pend_id, c);
            pend_id = -1;
            top_up();
        }
        // ---- one request inside the item, or the part of it the item covers ----
        const int seg = min(c.cur.pages - c.cur.p, c.left);
        load_q(c.cur.r, c.h);
#pragma unroll
        for (int m = 0; m < 8; ++m)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) o[m][cc] = 0.f;
        m0 = m1 = -INFINITY;
        l0 = l1 = corr0 = corr1 = 0.f;
        int since_fold = 0;
        for (int s = 0; s < seg; s += PPS) {
            const bool two = PPS == 2 && s + 1 < seg;                // warp-uniform
            const int ia = i, ib = i + 1;
            const int sA = ia % STAGES, sB = ib % STAGES;
            if (!mbar_wait(bar0 + 8 * sA, (uint32_t)(ia / STAGES) & 1u) ||
                (two && !mbar_wait(bar0 + 8 * sB, (uint32_t)(ib / STAGES) & 1u))) {
                timed_out = true;
                break;
            }
            const unsigned char* stA = ring + (size_t)sA * STAGE_BYTES;
            const unsigned char* stB = ring + (size_t)sB * STAGE_BYTES;
            const int posA = (c.cur.p + s) * PIKV_PAGE_TOKENS, posB = posA + PIKV_PAGE_TOKENS;
            float tA[4], tB[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            float vwA_lo = 0.f, vwA_hi = 0.f, vwB_lo = 0.f, vwB_hi = 0.f;
            page_scores(stA, tA, vwA_lo, vwA_hi);
            page_mask_scores(posA, tA);
            if (two) {
                page_scores(stB, tB, vwB_lo, vwB_hi);
                page_mask_scores(posB, tB);
            }
            // ---- online softmax (log2 domain); the 8 lanes with the same j hold the positions of a head pair
            //      (GS: of head j, in t[0] and t[2]) ----
            float mx0 = fmaxf(fmaxf(tA[0], tA[2]), fmaxf(tB[0], tB[2])), mx1 = fmaxf(fmaxf(tA[1], tA[3]), fmaxf(tB[1], tB[3]));
#pragma unroll
            for (int sh = 4; sh < 32; sh <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                if (!GS) mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0, mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
            float al0 = exp2f(m0 - mu0), al1 = GS ? 1.f : exp2f(m1 - mu1);
            m0 = mn0;
            m1 = mn1;
            float la = 0.f, lb = 0.f, ca = 0.f, cb = 0.f;
            // P' = P * vscale, rounded to f16 as the tensor cores will see it; pbuf is [head][32 positions]
            auto page_probs = [&](const unsigned char* st, const float (&t)[4], float vw_lo, float vw_hi, int base, int pos0) {
                const uint16_t* vsc = reinterpret_cast<const uint16_t*>(st + 2 * PAGE_BYTES + 32);
                const float vs_lo = __uint_as_float((uint32_t)vsc[r] << 16), vs_hi = __uint_as_float((uint32_t)vsc[r + 8] << 16);
                if constexpr (GS) {
                    const float p0 = exp2f(t[0] - mu0), p2 = exp2f(t[2] - mu0);
                    if (d.probs16 && j < G) {
                        // the H2O update needs exp(score - lse) summed over the heads of the group: lse is known only at
                        // the end, so the probabilities go out relative to this step's maximum (f16: uniform relative
                        // precision), with the maximum of every page beside them
                        const size_t hq = (size_t)c.cur.r * d.n_q + (size_t)c.h * G + j;
                        if (pos0 + r < c.cur.len && pos0 + r < d.probs_stride) d.probs16[hq * d.probs_stride + pos0 + r] = __float2half_rn(p0);
                        if (pos0 + r + 8 < c.cur.len && pos0 + r + 8 < d.probs_stride) d.probs16[hq * d.probs_stride + pos0 + r + 8] = __float2half_rn(p2);
                        if (r == 0 && (pos0 >> 4) < d.step_stride) d.step_max[hq * d.step_stride + (pos0 >> 4)] = mu0;
                    }
                    la += p0 + p2;
                    const __half h0 = __float2half_rn(p0 * vs_lo), h2 = __float2half_rn(p2 * vs_hi);
                    if (BITS == 8) ca += __half2float(h0) + __half2float(h2);
                    else ca += __half2float(h0) * vw_lo + __half2float(h2) * vw_hi;
                    pbuf[j * 32 + base + r] = h0;
                    pbuf[j * 32 + base + r + 8] = h2;
                    return;
                }
                const float p0 = exp2f(t[0] - mu0), p1 = exp2f(t[1] - mu1), p2 = exp2f(t[2] - mu0), p3 = exp2f(t[3] - mu1);
                if (d.probs16) {
                    const float pp[4] = {p0, p1, p2, p3};
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const int hh = 2 * j + (cc & 1), ps = pos0 + r + 8 * (cc >> 1);
                        if (hh >= G) continue;
                        const size_t hq = (size_t)c.cur.r * d.n_q + (size_t)c.h * G + hh;
                        if (ps < c.cur.len && ps < d.probs_stride) d.probs16[hq * d.probs_stride + ps] = __float2half_rn(pp[cc]);
                        if (r == 0 && cc < 2 && (pos0 >> 4) < d.step_stride) d.step_max[hq * d.step_stride + (pos0 >> 4)] = (cc & 1) ? mu1 : mu0;
                    }
                }
                la += p0 + p2;
                lb += p1 + p3;
                const __half h0 = __float2half_rn(p0 * vs_lo), h1 = __float2half_rn(p1 * vs_lo);
                const __half h2 = __float2half_rn(p2 * vs_hi), h3 = __float2half_rn(p3 * vs_hi);
                if (BITS == 8) {
                    ca += __half2float(h0) + __half2float(h2);           // x 1152 when it is folded
                    cb += __half2float(h1) + __half2float(h3);
                } else {
                    ca += __half2float(h0) * vw_lo + __half2float(h2) * vw_hi;
                    cb += __half2float(h1) * vw_lo + __half2float(h3) * vw_hi;
                }
                pbuf[(2 * j) * 32 + base + r] = h0;
                pbuf[(2 * j + 1) * 32 + base + r] = h1;
                pbuf[(2 * j) * 32 + base + r + 8] = h2;
                pbuf[(2 * j + 1) * 32 + base + r + 8] = h3;
            };
            page_probs(stA, tA, vwA_lo, vwA_hi, 0, posA);
            if (two) page_probs(stB, tB, vwB_lo, vwB_hi, 16, posB);
            l0 = l0 * al0 + la;
            l1 = l1 * al1 + lb;
            corr0 = corr0 * al0 + ca;
            corr1 = corr1 * al1 + cb;
            if constexpr (GS) {
                // the accumulators of heads 2j, 2j+1 live here, their rescale factors in the lanes with j' = head
                const float mine = al0;
                al0 = __shfl_sync(0xffffffffu, mine, (lane & ~3) | ((2 * j) & 3));
                al1 = __shfl_sync(0xffffffffu, mine, (lane & ~3) | ((2 * j + 1) & 3));
            }
            // rescale O: this thread's columns are query heads 2j and 2j+1
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                o[m][0] *= al0; o[m][1] *= al1; o[m][2] *= al0; o[m][3] *= al1;
            }
            __syncwarp();
            page_pv(stA, *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 2 * j),
                    *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 2 * j + 8));
            if (two)
                page_pv(stB, *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 16 + 2 * j),
                        *reinterpret_cast<const uint32_t*>(pbuf + r * 32 + 24 + 2 * j));
            __syncwarp();
            i += two ? 2 : 1;
            top_up();                                      // refill the stages just freed
            if (BITS == 8 && ++since_fold == DA_FOLD_STEPS) {      // (centred nibbles leave next to no bias)
                fold_bias();
                since_fold = 0;
            }
        }
        if (timed_out) break;
        // ---- this item's partial of the request: slot (block + request, head) ----
        fold_bias();
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
            l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        }
        {
            const size_t slot = ((size_t)c.blk + c.cur.r) * n_kv + c.h;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int qh = 2 * j + hh;
                if (qh >= G) continue;
                float4* po = reinterpret_cast<float4*>(d.part_o + ((slot * G + qh) * 128 + 16 * r));
#pragma unroll
                for (int m4 = 0; m4 < 4; ++m4)       // channels 16r + 4 m4 .. + 3
                    po[m4] = make_float4(o[2 * m4][hh], o[2 * m4][2 + hh], o[2 * m4 + 1][hh], o[2 * m4 + 1][2 + hh]);
                if (!GS && r == 0) {
                    d.part_ml[(slot * G + qh) * 2 + 0] = hh ? m1 : m0;
                    d.part_ml[(slot * G + qh) * 2 + 1] = hh ? l1 : l0;
                }
            }
            if (GS && r == 0 && j < G) {             // the statistics of head j
                d.part_ml[(slot * G + j) * 2 + 0] = m0;
                d.part_ml[(slot * G + j) * 2 + 1] = l0;
            }
        }
        c.left -= seg;
        advance(c.cur, seg);
    }
    if (timed_out) {
        // give the copies already issued one more bounded chance to land before the block leaves
        if (lane == 0 && d.status) atomicOr(d.status, PIKV_ST_WAIT_TIMEOUT);
        for (int ii = i; ii < issued; ++ii) (void)mbar_wait(bar0 + 8 * (ii % STAGES), (uint32_t)(ii / STAGES) & 1u);
    }
}

// Merge of the partials of the blocks g0..g1 that covered request rq, for query head (h, qh), by ONE WARP: lane i owns
// channels 4i..4i+3.  The statistics of up to 32 blocks are loaded by one warp-wide access and the partial outputs
// four blocks at a time (512 contiguous bytes each), so the loads of a request that many workers shared are in flight
// together.  acc = sum_g o_g 2^(m_g - M), l = sum_g l_g 2^(m_g - M).
__device__ __forceinline__ void da_merge_blocks(const DecodeDev& d, int rq, int h, int qh, int g0, int g1, int lane, float& M,
                                                float4& acc, float& l) {
    M = -INFINITY;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    l = 0.f;
    auto slot = [&](int g) { return (((size_t)g + rq) * d.n_kv + h) * d.G + qh; };
    if (g1 - g0 < 32) {
        // the common case: all blocks' statistics in one warp-wide load, then the outputs
        const int cnt = g1 - g0 + 1;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (lane < cnt) ml = *reinterpret_cast<const float2*>(d.part_ml + slot(g0 + lane) * 2);
        float mm = ml.x;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        M = mm;
        const float w_l = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - M), l_l = ml.y;
        int i = 0;
        for (; i + 4 <= cnt; i += 4) {
            float4 o4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) o4[u] = reinterpret_cast<const float4*>(d.part_o + slot(g0 + i + u) * 128)[lane];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float w = __shfl_sync(0xffffffffu, w_l, i + u);
                acc.x += o4[u].x * w; acc.y += o4[u].y * w; acc.z += o4[u].z * w; acc.w += o4[u].w * w;
                l += __shfl_sync(0xffffffffu, l_l, i + u) * w;
            }
        }
        for (; i < cnt; ++i) {
            const float4 o = reinterpret_cast<const float4*>(d.part_o + slot(g0 + i) * 128)[lane];
            const float w = __shfl_sync(0xffffffffu, w_l, i);
            acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
            l += __shfl_sync(0xffffffffu, l_l, i) * w;
        }
        return;
    }
    for (int gb = g0; gb <= g1; gb += 32) {
        const int g = gb + lane;
        float mm = g <= g1 ? d.part_ml[slot(g) * 2] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        M = fmaxf(M, mm);
    }
    for (int gb = g0; gb <= g1; gb += 32) {
        const int cnt = min(32, g1 - gb + 1);
        float w_l = 0.f, l_l = 0.f;
        if (lane < cnt) {
            const float2 ml = *reinterpret_cast<const float2*>(d.part_ml + slot(gb + lane) * 2);
            w_l = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - M);
            l_l = ml.y;
        }
        for (int i = 0; i < cnt; ++i) {
            const float4 o = reinterpret_cast<const float4*>(d.part_o + slot(gb + i) * 128)[lane];
            const float w = __shfl_sync(0xffffffffu, w_l, i);
            acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
            l += __shfl_sync(0xffffffffu, l_l, i) * w;
        }
    }
}

constexpr int DA_MERGE_THREADS = 128;     // four warps, one (request, query head) unit each

// One warp per (request, query head): merges the partials of the workers that covered the unit.
__global__ void __launch_bounds__(DA_MERGE_THREADS) decode_merge_kernel(DecodeDev d) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (DA_MERGE_THREADS / 32) + (threadIdx.x >> 5);
    if (unit >= d.B * d.n_q) return;
    const int rq = unit / d.n_q, qg = unit % d.n_q;
    const int h = qg / d.G, qh = qg % d.G;
    const int blk_pages = d.head[1], nblocks = d.head[2];
    const int pages = d.prefix[rq + 1] - d.prefix[rq];
    const size_t bq = (size_t)rq * d.n_q + qg;
    uint2* out2 = reinterpret_cast<uint2*>(d.out + bq * 128) + lane;      // four bf16 channels
    if (pages == 0) {
        *out2 = make_uint2(0u, 0u);
        if (lane == 0 && d.lse) d.lse[bq] = -INFINITY;
        return;
    }
    // the blocks that covered the request
    const int g0 = da_block_of(d.prefix[rq], blk_pages, nblocks), g1 = da_block_of(d.prefix[rq + 1] - 1, blk_pages, nblocks);
    float M, l;
    float4 acc;
    da_merge_blocks(d, rq, h, qh, g0, g1, lane, M, acc, l);
    const __nv_bfloat162 lo = __floats2bfloat162_rn(l > 0.f ? acc.x / l : 0.f, l > 0.f ? acc.y / l : 0.f);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(l > 0.f ? acc.z / l : 0.f, l > 0.f ? acc.w / l : 0.f);
    *out2 = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    if (lane == 0 && d.lse) d.lse[bq] = (l > 0.f) ? M * 0.6931471805599453f + logf(l) : -INFINITY;
}

// The same merge on an expert-sharded box: request i = (stream i / top_k, choice i % top_k) of a decode step
// whose rows are striped over the ranks; what this rank holds of it gives a NORMALISED partial output and its
// log-sum-exp, stored straight into the buffers of the stream's home rank (peer pointers, plain stores) at
// [local stream][choice][this rank].  A persistent grid: every warp walks its share of the units, every CTA makes
// its stores visible system-wide ONCE (a system-scope fence per unit cost 110 us for the 16384 units of a step)
// and counts itself; the last CTA to finish raises this rank's "done" flag on every rank.
__global__ void __launch_bounds__(DA_MERGE_THREADS) decode_return_kernel(DecodeDev d, ShardReturn t) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int units = d.B * d.n_q;
    const int blk_pages = d.head[1], nblocks = d.head[2];
    for (int unit = blockIdx.x * (DA_MERGE_THREADS / 32) + (threadIdx.x >> 5); unit < units;
         unit += gridDim.x * (DA_MERGE_THREADS / 32)) {
        const int rq = unit / d.n_q, qg = unit % d.n_q;
        const int h = qg / d.G, qh = qg % d.G;
        const int pages = d.prefix[rq + 1] - d.prefix[rq];
        if (pages <= 0) continue;
        const int g0 = da_block_of(d.prefix[rq], blk_pages, nblocks), g1 = da_block_of(d.prefix[rq + 1] - 1, blk_pages, nblocks);
        float M, l;
        float4 acc;
        da_merge_blocks(d, rq, h, qh, g0, g1, lane, M, acc, l);
        const int stream = rq / t.top_k, jsel = rq % t.top_k;
        const int home = stream / t.streams_per_rank, sl = stream % t.streams_per_rank;
        const size_t slot = (((size_t)sl * t.top_k + jsel) * t.world + t.rank) * d.n_q + qg;
        reinterpret_cast<float4*>(t.peer_part_o[home] + slot * 128)[lane] =
            l > 0.f ? make_float4(acc.x / l, acc.y / l, acc.z / l, acc.w / l) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane == 0) t.peer_part_lse[home][slot] = (l > 0.f) ? M * 0.6931471805599453f + logf(l) : -INFINITY;
    }
    // completion: every CTA counts itself after its stores are visible system-wide; the last one signals
    // (one thread per destination for the flags: system-scope release stores one after another cost 2 us each)
    __shared__ unsigned raise_s, step_s;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(t.counter, 1u);
        raise_s = 0u;
        if (prev == gridDim.x - 1) {
            *t.counter = 0;
            __threadfence_system();
            step_s = *t.seq;
            raise_s = 1u;
        }
    }
    __syncthreads();
    if (raise_s != 0u && threadIdx.x < t.world)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.peer_done_flags[threadIdx.x] + t.rank), "r"(step_s) : "memory");
}

static int da_workers() { return sm_count() * DA_CTAS_PER_SM * DA_WARPS; }

// launch configuration of a kernel that may start before the previous kernel of the stream has finished (it orders
// itself with griddepcontrol.wait)
static cudaLaunchConfig_t da_pdl_config(int grid, int block, size_t smem, cudaStream_t st, cudaLaunchAttribute* attr) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

// workspace: header, request prefix, block starts, partials of (max_blocks + B) x n_kv slots
struct DALayout {
    size_t prefix, blk_start, part_o, part_ml, total;
};
static DALayout da_layout(int B, int n_q, int n_kv, int max_blocks) {
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    DALayout l;
    l.prefix = 256;
    l.blk_start = l.prefix + up((size_t)(B + 1) * sizeof(int));
    l.part_o = l.blk_start + up((size_t)max_blocks * sizeof(int2));
    const size_t slots = ((size_t)max_blocks + B) * n_kv, G = (size_t)(n_q / n_kv);
    l.part_ml = l.part_o + slots * G * 128 * sizeof(float);
    l.total = l.part_ml + slots * G * 2 * sizeof(float);
    return l;
}
static int da_default_blocks(int n_kv) { return DA_ITEMS_PER_WORKER * max(1, da_workers() / n_kv); }
// the most blocks a workspace of `bytes` has room for (0: not even one)
static int da_blocks_for(size_t bytes, int B, int n_q, int n_kv) {
    int lo = 0, hi = da_default_blocks(n_kv);
    while (lo < hi) {
        const int mid = (lo + hi + 1) / 2;
        if (da_layout(B, n_q, n_kv, mid).total <= bytes) lo = mid; else hi = mid - 1;
    }
    return lo;
}

}  // namespace pikv

using namespace pikv;

extern "C" int pikv_decode_attn_default_splits(int32_t B, int32_t n_kv, int32_t max_ctx) {
    (void)B; (void)n_kv; (void)max_ctx;
    return 1;
}

extern "C" size_t pikv_decode_attn_workspace_bytes(int32_t B, int32_t n_q, int32_t n_kv, int32_t max_ctx,
                                                   int32_t splits) {
    (void)max_ctx; (void)splits;
    if (B <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0) return 0;
    return da_layout(B, n_q, n_kv, da_default_blocks(n_kv)).total;
}

int pikv::decode_attn_run(const pikv_decode_params* p, cudaStream_t st, int bits, const int* q_rows, const ShardReturn* ret,
                          const ShardPlan* plan) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "decode_attn: null params");
    PIKV_REQUIRE(p->q && (p->out || ret) && p->seq_len && p->page_table, PIKV_EINVAL, "decode_attn: null pointer");
    PIKV_REQUIRE(p->k_codes && p->v_codes && p->k_scale && p->v_scale, PIKV_EINVAL, "decode_attn: null cache pointer");
    PIKV_REQUIRE(p->B > 0 && p->n_q > 0 && p->n_kv > 0 && p->n_q % p->n_kv == 0, PIKV_EINVAL, "decode_attn: bad head counts");
    PIKV_REQUIRE(p->n_q / p->n_kv <= DA_MAX_GROUP, PIKV_EUNSUPPORTED, "decode_attn: %d query heads per KV head (max %d)",
                 p->n_q / p->n_kv, DA_MAX_GROUP);
    PIKV_REQUIRE(p->num_seqs > 0 && p->max_pages > 0 && p->num_pages > 0, PIKV_EINVAL, "decode_attn: bad cache geometry");
    PIKV_REQUIRE(p->n_kv <= da_workers(), PIKV_ELIMIT, "decode_attn: n_kv=%d exceeds the %d workers of the grid", p->n_kv, da_workers());
    PIKV_REQUIRE((long long)p->B * p->max_pages < (1ll << 31), PIKV_ELIMIT, "decode_attn: B * max_pages must stay below 2^31");
    PIKV_REQUIRE(p->B <= DA_MAX_REQ, PIKV_ELIMIT, "decode_attn: at most %d streams per call (got %d)", DA_MAX_REQ, p->B);
    PIKV_REQUIRE((long long)p->B * p->n_q < (1ll << 21), PIKV_ELIMIT, "decode_attn: B * n_q too large for one call");
    DecodeDev d;
    d.q = static_cast<const __nv_bfloat16*>(p->q);
    d.out = static_cast<__nv_bfloat16*>(p->out);
    d.B = p->B; d.n_q = p->n_q; d.n_kv = p->n_kv; d.G = p->n_q / p->n_kv;
    d.seq_ids = p->seq_ids; d.seq_len = p->seq_len; d.q_rows = q_rows; d.page_table = p->page_table;
    d.num_seqs = p->num_seqs; d.max_pages = p->max_pages; d.num_pages = p->num_pages;
    d.k_codes = static_cast<const uint8_t*>(p->k_codes); d.v_codes = static_cast<const uint8_t*>(p->v_codes);
    d.k_scale = static_cast<const uint16_t*>(p->k_scale); d.v_scale = static_cast<const uint16_t*>(p->v_scale);
    d.k_zp = static_cast<const float*>(p->k_zp); d.v_zp = static_cast<const float*>(p->v_zp);
    PIKV_REQUIRE(bits == 8 || (d.k_zp && d.v_zp), PIKV_EINVAL, "decode_attn_q4: the 4-bit cache needs k_zp and v_zp");
    d.lse = p->lse; d.scores = p->scores; d.score_stride = p->score_stride; d.status = p->status;
    PIKV_REQUIRE(d.scores == nullptr || d.score_stride > 0, PIKV_EINVAL, "decode_attn: score_stride");
    d.probs16 = static_cast<__half*>(p->probs16); d.step_max = p->step_max;
    d.probs_stride = p->probs_stride; d.step_stride = p->step_stride;
    PIKV_REQUIRE(d.probs16 == nullptr || (d.step_max != nullptr && d.probs_stride > 0 && d.step_stride > 0 && d.lse != nullptr),
                 PIKV_EINVAL, "decode_attn: probs16 needs step_max, both strides and lse");
    PIKV_REQUIRE(p->workspace != nullptr, PIKV_EINVAL, "decode_attn: null workspace");
    PIKV_REQUIRE((reinterpret_cast<uintptr_t>(p->workspace) & 15) == 0, PIKV_EINVAL, "decode_attn: workspace must be 16-byte aligned");
    d.workers = da_workers();
    d.max_blocks = da_blocks_for(p->workspace_bytes, p->B, p->n_q, p->n_kv);
    PIKV_REQUIRE(d.max_blocks >= 1, PIKV_EINVAL, "decode_attn: workspace too small (%zu bytes at least, %zu for full speed)",
                 da_layout(p->B, p->n_q, p->n_kv, 1).total, da_layout(p->B, p->n_q, p->n_kv, da_default_blocks(p->n_kv)).total);
    const DALayout lay = da_layout(p->B, p->n_q, p->n_kv, d.max_blocks);
    unsigned char* ws = static_cast<unsigned char*>(p->workspace);
    d.head = reinterpret_cast<int*>(ws);
    d.prefix = reinterpret_cast<int*>(ws + lay.prefix);
    d.blk_start = reinterpret_cast<int2*>(ws + lay.blk_start);
    d.part_o = reinterpret_cast<float*>(ws + lay.part_o);
    d.part_ml = reinterpret_cast<float*>(ws + lay.part_ml);
    if (plan != nullptr) decode_plan_kernel<true><<<1, DA_PLAN_THREADS, (size_t)(p->B + 1) * sizeof(int), st>>>(d, *plan);
    else decode_plan_kernel<false><<<1, DA_PLAN_THREADS, (size_t)(p->B + 1) * sizeof(int), st>>>(d, ShardPlan{});
    int rc = check_launch("decode_plan_kernel");
    if (rc != PIKV_OK) return rc;
    const int grid = d.workers / DA_WARPS;
    const bool gs = d.G <= 4;      // integer first product (see decode_attn_kernel)
    cudaLaunchAttribute attr[1];   // programmatic dependent launch of the attention and the merge kernel
#define PIKV_DA_LAUNCH(BITS, GS)                                                                                          \
    do {                                                                                                                  \
        const size_t smem = da_smem_bytes<BITS>();                                                                        \
        auto kern = decode_attn_kernel<BITS, GS>;                                                                         \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)            \
            return check_launch("decode_attn smem attribute");                                                            \
        cudaLaunchConfig_t cfg = da_pdl_config(grid, DA_THREADS, smem, st, attr);                                         \
        (void)cudaLaunchKernelEx(&cfg, kern, d);                                                                          \
    } while (0)
    if (bits == 8 && gs) PIKV_DA_LAUNCH(8, true);
    else if (bits == 8) PIKV_DA_LAUNCH(8, false);
    else if (gs) PIKV_DA_LAUNCH(4, true);
    else PIKV_DA_LAUNCH(4, false);
#undef PIKV_DA_LAUNCH
    rc = check_launch(bits == 8 ? "decode_attn_kernel<8>" : "decode_attn_kernel<4>");
    if (rc != PIKV_OK) return rc;
    const int units = p->B * p->n_q, per_cta = DA_MERGE_THREADS / 32;
    const int merge_ctas = (units + per_cta - 1) / per_cta;
    // the sharded return walks its units with a grid that is resident at once (one system-scope fence per CTA)
    cudaLaunchConfig_t mcfg = da_pdl_config(ret != nullptr ? min(merge_ctas, sm_count() * 8) : merge_ctas, DA_MERGE_THREADS, 0, st, attr);
    if (ret != nullptr) {
        (void)cudaLaunchKernelEx(&mcfg, decode_return_kernel, d, *ret);
        rc = check_launch("decode_return_kernel");
    } else {
        (void)cudaLaunchKernelEx(&mcfg, decode_merge_kernel, d);
        rc = check_launch("decode_merge_kernel");
    }
    count_launch(3);
    return rc;
}

extern "C" int pikv_decode_attn_q8(const pikv_decode_params* p, pikv_stream_t stream) {
    return decode_attn_run(p, static_cast<cudaStream_t>(stream), 8, nullptr, nullptr, nullptr);
}

extern "C" int pikv_decode_attn_q4(const pikv_decode_params* p, pikv_stream_t stream) {
    return decode_attn_run(p, static_cast<cudaStream_t>(stream), 4, nullptr, nullptr, nullptr);
}

// ---- decode attention for callers that must not allocate --------------------------------------------
// Some hosts of this library cannot call cudaMalloc when they need attention: a serving process that
// handed all of HBM to its own page pool at start-up, a plug-in that runs inside someone else's
// allocator-free region, code between cudaStreamBeginCapture and EndCapture.  For them the workers'
// partials live in this fixed array inside the library image.  Every GPU that loads the library keeps
// these 8 MiB until the process exits, and every call on a device shares them.
constexpr size_t DA_STATIC_SCRATCH_BYTES = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[DA_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address comes from the runtime, once per
// device, with that device current.
static int decode_static_scratch_ptr(void** out) {
    static void* ptrs[64];
    static bool have[64];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("decode_attn_static: cannot identify the current device");
        return PIKV_ECUDA;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("decode_attn_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return PIKV_ECUDA;
        }
        ptrs[dev] = p;
        have[dev] = true;
    }
    *out = ptrs[dev];
    return PIKV_OK;
}

extern "C" size_t pikv_decode_attn_static_scratch_bytes(void) { return DA_STATIC_SCRATCH_BYTES; }

extern "C" int pikv_decode_attn_q8_static(const pikv_decode_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "decode_attn_static: null params");
    PIKV_REQUIRE(p->B > 0 && p->n_q > 0 && p->n_kv > 0 && p->n_q % p->n_kv == 0 && p->max_pages > 0, PIKV_EINVAL,
                 "decode_attn_static: bad sizes");
    // the built-in array is smaller than the workspace the regular entry point asks for: fewer, longer blocks
    const size_t need = da_layout(p->B, p->n_q, p->n_kv, max(1, da_workers() / p->n_kv)).total;
    PIKV_REQUIRE(need <= DA_STATIC_SCRATCH_BYTES, PIKV_ELIMIT,
                 "decode_attn_static: %d streams x %d query heads need %zu bytes of scratch for the partial results, the "
                 "built-in array holds %zu; split the batch or use pikv_decode_attn_q8 with your own workspace",
                 p->B, p->n_q, need, DA_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    const int rc = decode_static_scratch_ptr(&scratch);
    if (rc != PIKV_OK) return rc;
    pikv_decode_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = DA_STATIC_SCRATCH_BYTES;
    return pikv_decode_attn_q8(&q, stream);
}
