// H2O scoring and eviction: score accumulate, segmented top-k select, page compaction.
//
// Select: one CTA per segment.  The segment's scores are staged once in shared memory as
// order-preserving 32-bit keys.  Segments that fit in shared memory take the bucketed path
// (select_bucketed): keys that are already in ascending order (timestamps of an append-only cache) are
// answered with two binary searches and range marks; otherwise one histogram over 4096 buckets that are
// linear in key space between the segment's smallest and largest key (float bits are a log scale, so
// neither uniform nor heavy-tailed scores pile into a few buckets), one pass that marks everything above
// the bucket holding the m-th largest key and lists that bucket's keys, and an exact rank among the listed
// keys with ties going to the lowest index.  Longer segments, and the rare bucket too full to rank, take
// the 8-bit radix select over the bits in which the keys differ (select_top_m).  The same routines run on
// the timestamps; both results are OR-ed into one keep bitmap from which the evict mask and the ascending
// kept-index list are written.
#include "common.cuh"

static int h2o_select_variant_for_tests();

namespace pikv {

constexpr int SEL_THREADS = 1024;          // keys staged in shared memory: one CTA per SM
constexpr int SEL_THREADS_STREAM = 512;    // keys re-read from memory: small CTAs, several per SM
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int SEL_SMEM_KEYS = 45056;   // keys staged in shared memory up to this length (with the bitmap, list and buckets: 218 KB)

__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
    const uint4 r = ld_stream_16(p);
    return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z), __uint_as_float(r.w));
}

__device__ __forceinline__ uint32_t order_key(float f) {
    // negative floats: all bits flipped; the others: sign bit set (an arithmetic shift and one three-input logic op)
    uint32_t b = __float_as_uint(f);
    if ((b << 1) == 0u) b = 0u;          // -0 and +0 are one value, as in a comparison of the floats
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}

constexpr int SEL_BUCKETS = 4096;      // first-level buckets of the bucketed path (4 per thread)
constexpr int SEL_RANK_CAP = 768;      // listed keys ranked pairwise up to this many; more: radix select instead

struct SelShared {
    int hist[256];
    uint32_t kmin, kmax;  // bucketed path: smallest and largest key, ascending-order flag, chosen bucket
    int sorted, bucket, above, bucket_cnt;
    int warp_tot[SEL_WARPS];
    uint32_t warp_or[SEL_WARPS], warp_and[SEL_WARPS];
    int width;            // number of low key bits in which the segment's keys differ
    uint32_t prefix;      // key bits fixed so far
    int remaining;        // how many still to take among keys matching the prefix
    int eq_total;         // size of the bin chosen by the last pass (after the last digit: keys equal to the threshold)
    int cand_n;           // entries in the candidate list
    int total;
};

constexpr int SEL_CAND_CAP = 4096;     // candidate list (keys that matched the first digit), shared memory

// One pass of the radix select finished: warp 0 finds the bin holding the rem-th largest key among the
// keys that matched so far and narrows prefix / remaining; eq_total = size of that bin.
__device__ __forceinline__ void select_pick_bin(SelShared& sh, uint32_t prefix, int shift, int lane) {
    // lane handles bins [lane*8, lane*8+8); scan from the top bin down
    int local[8], sum = 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        local[b] = sh.hist[lane * 8 + b];
        sum += local[b];
    }
    // suffix sum over lanes: above = number of keys in bins owned by higher lanes
    int suffix = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_down_sync(0xffffffffu, suffix, o);
        if (lane + o < 32) suffix += v;
    }
    const int above = suffix - sum;
    const int rem = sh.remaining;
    // the target bin is the highest bin d with count(bins > d) < rem <= count(bins >= d)
    int cum = above;
    int found = -1, found_above = 0, found_cnt = 0;
#pragma unroll
    for (int b = 7; b >= 0; --b) {
        if (found < 0 && cum < rem && rem <= cum + local[b]) {
            found = lane * 8 + b;
            found_above = cum;
            found_cnt = local[b];
        }
        cum += local[b];
    }
    if (found >= 0) {
        sh.prefix = prefix | ((uint32_t)found << shift);
        sh.remaining = rem - found_above;
        sh.eq_total = found_cnt;
    }
}

// Marks in keepw (one bit per element) the m largest of src[0..n), ties to the lowest index.
// STAGED: the keys are copied to shared memory once and read from there; otherwise every scan reads the
// scores again (from L2 after the first one), which needs almost no shared memory and lets two CTAs share
// an SM.  Either way four keys are read at a time, and after the first digit only the keys of the chosen
// bin (a short list in shared memory) are looked at again.
template <bool STAGED, int NT>
__device__ void select_top_m(const float* __restrict__ src, int n, int m, uint32_t* keys, uint32_t* cand, uint32_t* keepw,
                             SelShared& sh) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (m <= 0) return;
    if (m >= n) {
        for (int w = tid; w < (n + 31) / 32; w += NT) {
            int rem = n - w * 32;
            keepw[w] |= rem >= 32 ? 0xffffffffu : ((1u << rem) - 1u);
        }
        __syncthreads();
        return;
    }
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    const float4* src4 = reinterpret_cast<const float4*>(src);
    const uint4* keys4 = reinterpret_cast<const uint4*>(keys);
    const int n4 = (STAGED || aligned) ? n / 4 : 0;          // whole groups of four keys
    auto global4 = [&](int i) {
        const float4 f = __ldg(src4 + i);
        return make_uint4(order_key(f.x), order_key(f.y), order_key(f.z), order_key(f.w));
    };
    auto key4 = [&](int i) { return STAGED ? keys4[i] : global4(i); };
    auto key1 = [&](int i) { return STAGED ? keys[i] : order_key(__ldg(src + i)); };
    // first scan: find the bits in which the keys differ at all (and stage them).  The scores of one segment
    // share their leading (sign / exponent) bits, and a radix digit taken from those would send most keys to
    // one or two bins.  The digits start at the first differing bit.
    uint32_t any = 0u, all = 0xffffffffu;
    if (aligned) {
        for (int i = tid; i < n / 4; i += NT) {
            const uint4 u = global4(i);
            if (STAGED) reinterpret_cast<uint4*>(keys)[i] = u;
            any |= u.x | u.y | u.z | u.w;
            all &= u.x & u.y & u.z & u.w;
        }
    }
    for (int i = (aligned ? 4 * (n / 4) : 0) + tid; i < n; i += NT) {
        const uint32_t u = order_key(src[i]);
        if (STAGED) keys[i] = u;
        any |= u;
        all &= u;
    }
    any = __reduce_or_sync(0xffffffffu, any);
    all = __reduce_and_sync(0xffffffffu, all);
    if (lane == 0) {
        sh.warp_or[warp] = any;
        sh.warp_and[warp] = all;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t o = 0u, a = 0xffffffffu;
        for (int w = 0; w < (NT / 32); ++w) {
            o |= sh.warp_or[w];
            a &= sh.warp_and[w];
        }
        const int width = 32 - __clz(o ^ a);                 // bits [width-1 .. 0] vary; 0: all keys equal
        sh.width = width;
        sh.prefix = width >= 32 ? 0u : (a & (0xffffffffu << width));
        sh.remaining = m;
        sh.eq_total = n;
        sh.cand_n = 0;
    }
    __syncthreads();
    // radix select over the varying bits, most significant digit first, 8 bits at a time
    bool use_list = false;
    int pass = 0;
    for (int top = sh.width; top > 0; ++pass) {
        const int bits = min(8, top);
        const int shift = top - bits;
        for (int i = tid; i < 256; i += NT) sh.hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        const uint32_t himask = top >= 32 ? 0u : (0xffffffffu << top);
        const uint32_t dmask = (1u << bits) - 1u;
        if (use_list) {
            const int cn = sh.cand_n;
            for (int i = tid; i < cn; i += NT) {
                const uint32_t u = cand[i];
                if ((u & himask) == prefix) atomicAdd(&sh.hist[(u >> shift) & dmask], 1);
            }
        } else {
            // second pass with a short chosen bin: the matching keys also go to the candidate list
            const bool fill = pass == 1 && sh.eq_total <= SEL_CAND_CAP;
            auto one = [&](uint32_t u) {
                if ((u & himask) == prefix) {
                    atomicAdd(&sh.hist[(u >> shift) & dmask], 1);
                    if (fill) cand[atomicAdd(&sh.cand_n, 1)] = u;
                }
            };
            for (int i = tid; i < n4; i += NT) {
                const uint4 u = key4(i);
                one(u.x); one(u.y); one(u.z); one(u.w);
            }
            for (int i = 4 * n4 + tid; i < n; i += NT) one(key1(i));
            use_list = fill;
        }
        __syncthreads();
        if (warp == 0) select_pick_bin(sh, prefix, shift, lane);
        __syncthreads();
        top = shift;
    }
    const uint32_t kth = sh.prefix;      // the m-th largest key
    const int need_eq = sh.remaining;    // how many keys equal to kth to keep (lowest indices)
    if (need_eq == sh.eq_total && (n4 == n / 4)) {
        // every key equal to the threshold is kept: one pass, four keys per thread, eight lanes per keep word
        const int n4r = (n + 3) / 4;
        for (int i0 = 0; i0 < n4r; i0 += NT) {
            const int i = i0 + tid;
            uint32_t nib = 0u;
            if (i < n4) {
                const uint4 u = key4(i);
                nib = (u.x >= kth ? 1u : 0u) | (u.y >= kth ? 2u : 0u) | (u.z >= kth ? 4u : 0u) | (u.w >= kth ? 8u : 0u);
            } else if (i < n4r) {
                for (int e = 0; e < 4; ++e)
                    if (4 * i + e < n && key1(4 * i + e) >= kth) nib |= 1u << e;
            }
            uint32_t word = nib << (4 * (lane & 7));
            word |= __shfl_xor_sync(0xffffffffu, word, 1);
            word |= __shfl_xor_sync(0xffffffffu, word, 2);
            word |= __shfl_xor_sync(0xffffffffu, word, 4);
            if ((lane & 7) == 0 && word && i < n4r) keepw[i >> 3] |= word;
        }
        __syncthreads();
        return;
    }
    // ties at the threshold of which only some are kept: in-order count of equal keys; warp w owns the
    // contiguous range [w*per, (w+1)*per)
    const int tiles = (n + 31) / 32;
    const int tiles_per = (tiles + (NT / 32) - 1) / (NT / 32);
    const int t0 = warp * tiles_per, t1 = min(tiles, t0 + tiles_per);
    int eq_cnt = 0;
    for (int t = t0; t < t1; ++t) {
        const int i = t * 32 + lane;
        uint32_t u = 0;
        bool in = i < n;
        if (in) u = key1(i);
        eq_cnt += __popc(__ballot_sync(0xffffffffu, in && u == kth));
    }
    if (lane == 0) sh.warp_tot[warp] = eq_cnt;
    __syncthreads();
    int eq_before = 0;
    for (int w = 0; w < warp; ++w) eq_before += sh.warp_tot[w];
    for (int t = t0; t < t1; ++t) {
        const int i = t * 32 + lane;
        uint32_t u = 0;
        bool in = i < n;
        if (in) u = key1(i);
        const bool gt = in && u > kth;
        const bool eq = in && u == kth;
        const unsigned eqb = __ballot_sync(0xffffffffu, eq);
        const int my_rank = eq_before + __popc(eqb & ((1u << lane) - 1u));
        const bool keep = gt || (eq && my_rank < need_eq);
        const unsigned kb = __ballot_sync(0xffffffffu, keep);
        if (lane == 0 && kb) keepw[t] |= kb;
        eq_before += __popc(eqb);
    }
    __syncthreads();
}

// marks [a, b) in the keep bitmap (all threads)
template <int NT>
__device__ __forceinline__ void mark_range(uint32_t* keepw, int a, int b) {
    if (b <= a) return;
    for (int w = (a >> 5) + threadIdx.x; w <= ((b - 1) >> 5); w += NT) {
        const int lo = max(a - w * 32, 0), hi = min(b - w * 32, 32);
        const uint32_t bits = (hi >= 32 ? 0xffffffffu : ((1u << hi) - 1u)) & ~((1u << lo) - 1u);
        atomicOr(&keepw[w], bits);
    }
}

// Bucketed select for a segment staged in shared memory; same contract as select_top_m.  hist4k: SEL_BUCKETS ints.
template <int NT>
__device__ void select_bucketed(const float* __restrict__ src, int n, int m, uint32_t* keys, uint32_t* cand, uint32_t* keepw,
                                int* hist4k, SelShared& sh) {
    static_assert(NT * 4 == SEL_BUCKETS, "four buckets per thread");
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (m <= 0) return;
    if (m >= n) {
        mark_range<NT>(keepw, 0, n);
        __syncthreads();
        return;
    }
    // ---- stage the keys; smallest, largest ----
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    if (aligned) {
        // eight 16-byte loads in flight per thread: with one CTA per SM nothing else hides the latency of a round trip
        const float4* src4 = reinterpret_cast<const float4*>(src);
        const int n4s = n / 4;
        for (int i0 = tid; i0 < n4s; i0 += 8 * NT) {
            float4 f[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (i0 + q * NT < n4s) f[q] = ld_stream_f4(src4 + i0 + q * NT);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (i0 + q * NT < n4s) {
                    const uint4 u = make_uint4(order_key(f[q].x), order_key(f[q].y), order_key(f[q].z), order_key(f[q].w));
                    reinterpret_cast<uint4*>(keys)[i0 + q * NT] = u;
                    kmin = min(min(kmin, u.x), min(u.y, min(u.z, u.w)));
                    kmax = max(max(kmax, u.x), max(u.y, max(u.z, u.w)));
                }
            }
        }
    }
    for (int i = (aligned ? 4 * (n / 4) : 0) + tid; i < n; i += NT) {
        const uint32_t u = order_key(src[i]);
        keys[i] = u;
        kmin = min(kmin, u);
        kmax = max(kmax, u);
    }
    kmin = __reduce_min_sync(0xffffffffu, kmin);
    kmax = __reduce_max_sync(0xffffffffu, kmax);
    if (lane == 0) {
        sh.warp_or[warp] = kmax;
        sh.warp_and[warp] = kmin;
    }
    if (tid == 0) sh.sorted = 1;
    for (int i = tid; i < SEL_BUCKETS; i += NT) hist4k[i] = 0;
    __syncthreads();
    if (tid == 0) {
        uint32_t lo = 0xffffffffu, hi = 0u;
        for (int w = 0; w < NT / 32; ++w) {
            hi = max(hi, sh.warp_or[w]);
            lo = min(lo, sh.warp_and[w]);
        }
        sh.kmin = lo;
        sh.kmax = hi;
        sh.cand_n = 0;
    }
    // ---- already ascending?  (a thread looks at four neighbouring pairs) ----
    {
        bool ok = true;
        const uint4* k4 = reinterpret_cast<const uint4*>(keys);
        for (int i = tid; 4 * i < n - 1; i += NT) {
            if (4 * i + 4 < n) {
                const uint4 u = k4[i];
                ok &= u.x <= u.y && u.y <= u.z && u.z <= u.w && u.w <= keys[4 * i + 4];
            } else {
                for (int q = 4 * i; q < n - 1; ++q) ok &= keys[q] <= keys[q + 1];
            }
        }
        if (!__all_sync(0xffffffffu, ok) && lane == 0) sh.sorted = 0;
    }
    __syncthreads();
    kmin = sh.kmin;
    kmax = sh.kmax;
    if (sh.sorted || kmin == kmax) {
        // ascending keys: the m largest are the tail; of the run equal to the threshold the lowest indices are kept
        const uint32_t kth = keys[n - m];
        int a = 0, b = n;                        // a = first index with key >= kth, b = first index with key > kth
        {
            int lo = 0, hi = n - m;
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (keys[mid] >= kth) hi = mid; else lo = mid + 1; }
            a = lo;
            lo = n - m; hi = n;
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (keys[mid] > kth) hi = mid; else lo = mid + 1; }
            b = lo;
        }
        mark_range<NT>(keepw, b, n);
        mark_range<NT>(keepw, a, a + (m - (n - b)));
        __syncthreads();
        return;
    }
    // ---- histogram over buckets linear in key space ----
    const float scale = 4095.0f / (float)(kmax - kmin);
    auto bucket_of = [&](uint32_t u) { return min(SEL_BUCKETS - 1, (int)((float)(u - kmin) * scale)); };
    const uint4* keys4 = reinterpret_cast<const uint4*>(keys);
    const int n4 = n / 4;
    for (int i = tid; i < n4; i += NT) {
        const uint4 u = keys4[i];
        atomicAdd(&hist4k[bucket_of(u.x)], 1);
        atomicAdd(&hist4k[bucket_of(u.y)], 1);
        atomicAdd(&hist4k[bucket_of(u.z)], 1);
        atomicAdd(&hist4k[bucket_of(u.w)], 1);
    }
    for (int i = 4 * n4 + tid; i < n; i += NT) atomicAdd(&hist4k[bucket_of(keys[i])], 1);
    __syncthreads();
    // ---- the bucket holding the m-th largest key: suffix sums, thread t owns buckets 4t .. 4t+3 ----
    {
        const int c0 = hist4k[4 * tid], c1 = hist4k[4 * tid + 1], c2 = hist4k[4 * tid + 2], c3 = hist4k[4 * tid + 3];
        const int sum = c0 + c1 + c2 + c3;
        int suffix = sum;                                    // inclusive suffix over the lanes of the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_down_sync(0xffffffffu, suffix, o);
            if (lane + o < 32) suffix += v;
        }
        if (lane == 0) sh.warp_tot[warp] = suffix;
        __syncthreads();
        int above = suffix - sum;                            // keys in the buckets of higher threads
        for (int w = warp + 1; w < NT / 32; ++w) above += sh.warp_tot[w];
        const int cs[4] = {c0, c1, c2, c3};
        int cum = above;
#pragma unroll
        for (int b = 3; b >= 0; --b) {
            if (cum < m && m <= cum + cs[b]) {
                sh.bucket = 4 * tid + b;
                sh.above = cum;
                sh.bucket_cnt = cs[b];
            }
            cum += cs[b];
        }
    }
    __syncthreads();
    const int bstar = sh.bucket, rem = m - sh.above, cn = sh.bucket_cnt;
    if (cn > SEL_CAND_CAP) {
        // a bucket too full to list (scores with one far outlier): the radix select handles any distribution
        select_top_m<true, NT>(src, n, m, keys, cand, keepw, sh);
        return;
    }
    // ---- mark everything above the bucket, list the bucket's indices ----
    {
        const int n4r = (n + 3) / 4;
        for (int i0 = 0; i0 < n4r; i0 += NT) {
            const int i = i0 + tid;
            uint32_t nib = 0u, eq = 0u;
            if (i < n4) {
                const uint4 u = keys4[i];
                const int b0 = bucket_of(u.x), b1 = bucket_of(u.y), b2 = bucket_of(u.z), b3 = bucket_of(u.w);
                nib = (b0 > bstar ? 1u : 0u) | (b1 > bstar ? 2u : 0u) | (b2 > bstar ? 4u : 0u) | (b3 > bstar ? 8u : 0u);
                eq = (b0 == bstar ? 1u : 0u) | (b1 == bstar ? 2u : 0u) | (b2 == bstar ? 4u : 0u) | (b3 == bstar ? 8u : 0u);
            } else if (i < n4r) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (4 * i + e < n) {
                        const int b = bucket_of(keys[4 * i + e]);
                        nib |= (b > bstar ? 1u : 0u) << e;
                        eq |= (b == bstar ? 1u : 0u) << e;
                    }
                }
            }
            uint32_t word = nib << (4 * (lane & 7));
            word |= __shfl_xor_sync(0xffffffffu, word, 1);
            word |= __shfl_xor_sync(0xffffffffu, word, 2);
            word |= __shfl_xor_sync(0xffffffffu, word, 4);
            if ((lane & 7) == 0 && word && i < n4r) atomicOr(&keepw[i >> 3], word);
            // listed indices: one shared-memory atomic per warp
            const int c = __popc(eq);
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            int base = 0;
            if (lane == 31 && inc) base = atomicAdd(&sh.cand_n, inc);
            base = __shfl_sync(0xffffffffu, base, 31) + inc - c;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (eq >> e & 1u) cand[base++] = 4 * i + e;
        }
    }
    __syncthreads();
    if (cn <= SEL_RANK_CAP) {
        // ---- exact rank among the listed keys: larger key first, lower index first among equals ----
        for (int i = tid; i < cn; i += NT) {
            const int idx = cand[i];
            const uint32_t ki = keys[idx];
            int rank = 0;
            for (int q = 0; q < cn; ++q) {
                const int iq = cand[q];
                const uint32_t kq = keys[iq];
                rank += (kq > ki || (kq == ki && iq < idx)) ? 1 : 0;
            }
            if (rank < rem) atomicOr(&keepw[idx >> 5], 1u << (idx & 31));
        }
        __syncthreads();
        return;
    }
    // ---- many listed keys: 8-bit radix select over the list for the rem-th largest, then lowest indices among equals ----
    if (tid == 0) {
        sh.prefix = 0u;
        sh.remaining = rem;
        sh.eq_total = cn;
    }
    __syncthreads();
    for (int top = 32; top > 0; top -= 8) {
        const int shift = top - 8;
        for (int i = tid; i < 256; i += NT) sh.hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sh.prefix;
        const uint32_t himask = top >= 32 ? 0u : (0xffffffffu << top);
        for (int i = tid; i < cn; i += NT) {
            const uint32_t u = keys[cand[i]];
            if ((u & himask) == prefix) atomicAdd(&sh.hist[(u >> shift) & 255u], 1);
        }
        __syncthreads();
        if (warp == 0) select_pick_bin(sh, prefix, shift, lane);
        __syncthreads();
    }
    {
        const uint32_t kth = sh.prefix;
        const int need_eq = sh.remaining;
        for (int i = tid; i < cn; i += NT) {
            const int idx = cand[i];
            const uint32_t ki = keys[idx];
            bool keep = ki > kth;
            if (ki == kth) {
                int before = 0;                              // equal keys with a lower index
                for (int q = 0; q < cn; ++q) before += (keys[cand[q]] == kth && cand[q] < idx) ? 1 : 0;
                keep = before < need_eq;
            }
            if (keep) atomicOr(&keepw[idx >> 5], 1u << (idx & 31));
        }
    }
    __syncthreads();
}

template <bool STAGED, int NT>
__global__ void __launch_bounds__(NT) h2o_select_kernel(const float* acc, const float* ts, int stride,
                                                                 const int* seg_len, int n_all, int num_heavy,
                                                                 int num_recent, uint8_t* evict_mask, int* keep_idx,
                                                                 int keep_stride, int* kept_count, bool radix_only) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ SelShared sh;
    const int seg = blockIdx.x;
    int n = seg_len ? seg_len[seg] : n_all;
    n = max(0, min(n, stride));
    const int words_cap = (stride + 31) / 32;
    uint32_t* keepw = reinterpret_cast<uint32_t*>(smem_raw);
    // keys start on a 16-byte boundary (they are read four at a time); the candidate list follows them
    uint32_t* keys = keepw + ((words_cap + 3) & ~3);
    uint32_t* cand = keys + (STAGED ? ((stride + 3) & ~3) : 0);   // unstaged: the list follows the bitmap
    int* hist4k = reinterpret_cast<int*>(cand + SEL_CAND_CAP);     // staged: first-level buckets
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int w = tid; w < words_cap; w += NT) keepw[w] = 0u;
    __syncthreads();
    const float* a = acc + (size_t)seg * stride;
    const float* t = ts + (size_t)seg * stride;
    if (n > 0) {
        if (STAGED && !radix_only) {
            if constexpr (NT * 4 == SEL_BUCKETS) {
                select_bucketed<NT>(a, n, min(num_heavy, n), keys, cand, keepw, hist4k, sh);
                select_bucketed<NT>(t, n, min(num_recent, n), keys, cand, keepw, hist4k, sh);
            }
        } else {
            select_top_m<STAGED, NT>(a, n, min(num_heavy, n), keys, cand, keepw, sh);
            select_top_m<STAGED, NT>(t, n, min(num_recent, n), keys, cand, keepw, sh);
        }
    }
    // outputs: evict mask bytes and ascending kept indices.  A warp owns a contiguous run of 128-position tiles;
    // a lane handles four neighbouring positions of a tile (one 4-byte mask store when the row is 4-byte aligned).
    const int tiles = (stride + 127) / 128;
    const int tiles_per = (tiles + (NT / 32) - 1) / (NT / 32);
    const int t0 = warp * tiles_per, t1 = min(tiles, t0 + tiles_per);
    int cnt = 0;
    for (int w = 4 * t0 + lane; w < min(4 * t1, words_cap); w += 32) cnt += __popc(keepw[w]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) sh.warp_tot[warp] = cnt;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += sh.warp_tot[w];
    const bool vec_ok = (stride & 3) == 0 && evict_mask != nullptr && (reinterpret_cast<uintptr_t>(evict_mask) & 3) == 0;
    for (int tt = t0; tt < t1; ++tt) {
        const int wi = 4 * tt + (lane >> 3);
        const uint32_t nib = wi < words_cap ? (keepw[wi] >> (4 * (lane & 7))) & 0xfu : 0u;
        const int i = tt * 128 + 4 * lane;
        if (evict_mask) {
            if (vec_ok && i + 3 < stride) {
                const uint32_t bytes = ((nib & 1u) ? 0u : 1u) | ((nib & 2u) ? 0u : 0x100u) | ((nib & 4u) ? 0u : 0x10000u) |
                                       ((nib & 8u) ? 0u : 0x1000000u);
                *reinterpret_cast<uint32_t*>(evict_mask + (size_t)seg * stride + i) = bytes;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (i + e < stride) evict_mask[(size_t)seg * stride + i + e] = (nib >> e & 1u) ? 0 : 1;
            }
        }
        const int c = __popc(nib);
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        if (keep_idx) {
            int rpos = before + inc - c;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (nib >> e & 1u) {
                    if (rpos < keep_stride) keep_idx[(size_t)seg * keep_stride + rpos] = i + e;
                    ++rpos;
                }
            }
        }
        before += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (tid == 0 && kept_count) {
        int tot = 0;
        for (int w = 0; w < (NT / 32); ++w) tot += sh.warp_tot[w];
        kept_count[seg] = tot;
    }
}

// ---- streaming select ---------------------------------------------------------------------------------
// The default select.  The scores are never staged as a whole: every pass re-reads them (after the first pass
// from L2) with coalesced 16-byte loads.  Per score array the m-th largest key and the number of keys equal to
// it that are kept (lowest indices first) are found first:
//   pass 1  smallest and largest key, and whether the keys are already ascending (timestamps of an append-only
//           cache): then the m largest are the tail of the segment and no search is needed;
//   pass 2  histogram over 4096 buckets of 2^s consecutive key values above the smallest key (s chosen so that
//           the largest key falls into the last buckets); the bucket holding the m-th largest key is found from
//           suffix sums;
//   pass 3  the keys of that bucket are listed in shared memory (a few dozen for smooth score distributions) and
//           the bucket is narrowed on the list, 12 bits at a time, down to one key value.  A bucket with more
//           keys than the list holds is narrowed by another pass 2 over the segment instead.
// In the last pass a thread owns whole 32-position words of the segment (a warp's 32 words are loaded coalesced
// and transposed through a swizzled 4 KiB tile of shared memory), so every decision about a position is a bit of
// a register word: ties are resolved with a block-wide count of the equal keys in index order (skipped when all
// of them are kept), and the evict mask and the ascending kept-index list need no atomics and no bit gathering
// across lanes.  Small CTAs, four per SM: the segments of an SM overlap each other's barriers and load latencies.
constexpr int SS_THREADS = 256;
constexpr int SS_BUCKETS = 4096;
constexpr int SS_LIST_CAP = 1024;
constexpr int SS_RANK_CAP = 256;                    // listed keys ranked by counting up to this many
constexpr int SS_BPT = SS_BUCKETS / SS_THREADS;     // buckets a thread owns in the suffix sums

struct SsResult {
    int mode;            // 0: nothing kept, 1: every position, 2: positions >= lo, 3: keys above kth + need_eq keys equal to it
    uint32_t kth;
    int need_eq, all_eq, lo;
    int raw;             // the array's float bits serve as keys (no set sign bit), see ss_key
};

struct SsShared {
    // the search (histogram, candidate list) and the last pass (transpose tiles) never overlap in time
    union {
        uint4 tile[SS_THREADS / 32][256];           // per warp: 32 words x 8 chunks of 16 bytes, chunk c of word r at c ^ (r & 7)
        struct {
            int hist[SS_BUCKETS];
            uint32_t list[SS_LIST_CAP];
        };
    };
    uint32_t red_a[SS_THREADS / 32], red_b[SS_THREADS / 32];
    int red_i[SS_THREADS / 32];
    int list_n, bucket, above, bucket_cnt, sorted, need_count, negative;
    uint32_t kmin, kmax;
    SsResult res[2];
};

// RAW: every value of the array has its sign bit clear (scores and timestamps normally do); then the float bits
// themselves order like the values and no conversion is needed.  Keys of the two kinds are never mixed: everything
// about one array (range, threshold, comparisons) lives in one key space.
template <bool RAW>
__device__ __forceinline__ uint32_t ss_key(float f) { return RAW ? __float_as_uint(f) : order_key(f); }
template <bool RAW>
__device__ __forceinline__ uint4 ss_keys4(const float4 f) {
    return make_uint4(ss_key<RAW>(f.x), ss_key<RAW>(f.y), ss_key<RAW>(f.z), ss_key<RAW>(f.w));
}

// one(key) for every key of src[0..n), in no particular order; four 16-byte loads in flight per thread
template <int NT, bool RAW, class F>
__device__ __forceinline__ void ss_for_keys(const float* __restrict__ src, int n, bool aligned, F&& one) {
    if (aligned) {
        const float4* src4 = reinterpret_cast<const float4*>(src);
        const int n4 = n >> 2;
        int i0 = threadIdx.x;
        for (; i0 + 7 * NT < n4; i0 += 8 * NT) {                  // eight loads in flight, no bounds checks
            float4 f[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) f[u] = __ldg(src4 + i0 + u * NT);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint4 k = ss_keys4<RAW>(f[u]);
                one(k.x); one(k.y); one(k.z); one(k.w);
            }
        }
        for (; i0 < n4; i0 += NT) {
            const uint4 k = ss_keys4<RAW>(__ldg(src4 + i0));
            one(k.x); one(k.y); one(k.z); one(k.w);
        }
        for (int i = 4 * n4 + threadIdx.x; i < n; i += NT) one(ss_key<RAW>(__ldg(src + i)));
    } else {
        for (int i = threadIdx.x; i < n; i += NT) one(ss_key<RAW>(__ldg(src + i)));
    }
}

// exclusive prefix of v over the CTA in thread order, and the total; red: NT / 32 ints of shared memory
template <int NT>
__device__ __forceinline__ int ss_block_scan(int v, int* red, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) red[warp] = inc;
    __syncthreads();
    int before = 0, tot = 0;
#pragma unroll
    for (int q = 0; q < NT / 32; ++q) {
        const int x = red[q];
        before += q < warp ? x : 0;
        tot += x;
    }
    __syncthreads();
    total = tot;
    return before + inc - v;
}

// bucket holding the rem-th largest counted key: suffix sums over hist, thread t owns buckets [t * SS_BPT, ...)
template <int NT>
__device__ __forceinline__ void ss_pick_bucket(SsShared& sh, int rem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int c[SS_BPT], sum = 0;
#pragma unroll
    for (int q = 0; q < SS_BPT / 4; ++q) {
        const int4 v = reinterpret_cast<const int4*>(sh.hist)[tid * (SS_BPT / 4) + q];
        c[4 * q] = v.x; c[4 * q + 1] = v.y; c[4 * q + 2] = v.z; c[4 * q + 3] = v.w;
        sum += v.x + v.y + v.z + v.w;
    }
    int suffix = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(0xffffffffu, suffix, o);
        if (lane + o < 32) suffix += v;
    }
    if (lane == 0) sh.red_i[warp] = suffix;
    if (tid == 0) sh.bucket = -1;
    __syncthreads();
    int cum = suffix - sum;
    for (int q = warp + 1; q < NT / 32; ++q) cum += sh.red_i[q];
#pragma unroll
    for (int b = SS_BPT - 1; b >= 0; --b) {
        if (cum < rem && rem <= cum + c[b]) {
            sh.bucket = tid * SS_BPT + b;
            sh.above = cum;
            sh.bucket_cnt = c[b];
        }
        cum += c[b];
    }
    __syncthreads();
}

__device__ __forceinline__ int ss_shift_for(uint32_t width) {      // (width >> s) < SS_BUCKETS
    return max(0, (32 - __clz(width)) - 12);
}

// Where the m largest of src[0..n) are, ties to the lowest index: fills *out (shared memory) for the last pass.
// ASCENDING_CHECK: whether pass 1 also tests for ascending keys (worth it for timestamps; for scores it only costs)
// RAW: the float bits are taken as keys; returns false (nothing decided) when pass 1 meets a set sign bit, and the
// caller runs the converting instance instead.
template <int NT, bool ASCENDING_CHECK, bool RAW>
__device__ bool ss_find(const float* __restrict__ src, int n, int m, bool aligned, SsShared& sh, SsResult* out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (m <= 0 || m >= n) {
        if (tid == 0) {
            out->mode = m <= 0 ? 0 : 1;
            out->raw = RAW;
        }
        __syncthreads();
        return true;
    }
    // ---- pass 1: smallest, largest, ascending? ----
    {
        uint32_t mn = 0xffffffffu, mx = 0u, signs = 0u;
        bool ok = true;
        if (aligned) {
            const float4* src4 = reinterpret_cast<const float4*>(src);
            const int n4 = n >> 2;
            int i0 = 0;
            // whole iterations: every vector exists and has a successor key, no bounds tests; eight loads in flight
            for (; i0 + 8 * NT <= n4 && 4 * (i0 + 8 * NT) < n; i0 += 8 * NT) {
                float4 f[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) f[u] = __ldg(src4 + i0 + u * NT + tid);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint4 k = ss_keys4<RAW>(f[u]);
                    if (ASCENDING_CHECK) {
                        uint32_t next = __shfl_down_sync(0xffffffffu, k.x, 1);
                        if (lane == 31) next = ss_key<RAW>(__ldg(src + 4 * (size_t)(i0 + u * NT + tid) + 4));
                        ok &= k.x <= k.y && k.y <= k.z && k.z <= k.w && k.w <= next;
                    }
                    mn = min(mn, min(min(k.x, k.y), min(k.z, k.w)));
                    mx = max(mx, max(max(k.x, k.y), max(k.z, k.w)));
                    if (RAW) signs |= k.x | k.y | k.z | k.w;
                }
            }
            for (; i0 < n4; i0 += 4 * NT) {                      // the same trip count in every thread (shuffles inside)
                float4 f[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * NT + tid;
                    f[u] = i < n4 ? __ldg(src4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * NT + tid;
                    const bool on = i < n4;
                    const uint4 k = ss_keys4<RAW>(f[u]);
                    if (ASCENDING_CHECK) {
                        uint32_t next = __shfl_down_sync(0xffffffffu, k.x, 1);      // the key after this thread's four
                        const bool has_next = 4 * i + 4 < n;
                        if (on && has_next && (lane == 31 || i + 1 >= n4)) next = ss_key<RAW>(__ldg(src + 4 * (size_t)i + 4));
                        if (on) ok &= k.x <= k.y && k.y <= k.z && k.z <= k.w && (!has_next || k.w <= next);
                    }
                    if (on) {
                        mn = min(mn, min(min(k.x, k.y), min(k.z, k.w)));
                        mx = max(mx, max(max(k.x, k.y), max(k.z, k.w)));
                        if (RAW) signs |= k.x | k.y | k.z | k.w;
                    }
                }
            }
            if (tid == 0) {                                       // the last n % 4 keys
                for (int i = 4 * n4; i < n; ++i) {
                    const uint32_t u = ss_key<RAW>(__ldg(src + i));
                    mn = min(mn, u);
                    mx = max(mx, u);
                    if (RAW) signs |= u;
                    if (ASCENDING_CHECK && i + 1 < n) ok &= u <= ss_key<RAW>(__ldg(src + i + 1));
                }
            }
        } else {
            for (int i = tid; i < n; i += NT) {
                const uint32_t u = ss_key<RAW>(__ldg(src + i));
                mn = min(mn, u);
                mx = max(mx, u);
                if (RAW) signs |= u;
                if (ASCENDING_CHECK && i + 1 < n) ok &= u <= ss_key<RAW>(__ldg(src + i + 1));
            }
        }
        if (!ASCENDING_CHECK) ok = false;
        mn = __reduce_min_sync(0xffffffffu, mn);
        mx = __reduce_max_sync(0xffffffffu, mx);
        const bool all_ok = __all_sync(0xffffffffu, ok);
        const bool negative = RAW && __any_sync(0xffffffffu, (signs >> 31) != 0u);
        if (lane == 0) {
            sh.red_a[warp] = mn;
            sh.red_b[warp] = mx;
            sh.red_i[warp] = (all_ok ? 1 : 0) | (negative ? 2 : 0);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t lo = 0xffffffffu, hi = 0u;
            int so = 1, neg = 0;
            for (int q = 0; q < NT / 32; ++q) {
                lo = min(lo, sh.red_a[q]);
                hi = max(hi, sh.red_b[q]);
                so &= sh.red_i[q] & 1;
                neg |= sh.red_i[q] & 2;
            }
            sh.kmin = lo;
            sh.kmax = hi;
            sh.sorted = so;
            sh.need_count = 0;
            sh.negative = neg;
            out->raw = RAW;
            if (neg) {
                // the caller repeats the search with converted keys
            } else if (so || lo == hi) {
                // ascending keys: the m largest are the tail; of a run of equal keys across the cut the lowest indices stay
                const uint32_t kth = ss_key<RAW>(src[n - m]);
                if (ss_key<RAW>(src[n - m - 1]) != kth) {
                    out->mode = 2;
                    out->lo = n - m;
                } else {
                    out->mode = 3;
                    out->kth = kth;
                    out->all_eq = 0;
                    out->need_eq = m;                    // all keys equal; otherwise m minus the keys above kth (counted below)
                    sh.need_count = lo != hi;
                }
            }
        }
        __syncthreads();
    }
    if (RAW && sh.negative) return false;
    if (sh.sorted || sh.kmin == sh.kmax) {
        if (sh.need_count) {
            const uint32_t kth = out->kth;
            int gt = 0;
            ss_for_keys<NT, RAW>(src, n, aligned, [&](uint32_t u) { gt += u > kth ? 1 : 0; });
            int total;
            (void)ss_block_scan<NT>(gt, sh.red_i, total);
            if (tid == 0) out->need_eq = m - total;
            __syncthreads();
        }
        return true;
    }
    // ---- passes 2 and 3: narrow [lo, lo + width] around the m-th largest key ----
    // The first histogram covers only the top 2^27 key values below the largest key (sixteen binades of positive
    // scores): a few low outliers must not widen the buckets of the range the m-th largest key lives in.  If fewer
    // than m keys fall into it (a far outlier at the top), the whole key range is taken instead.
    uint32_t lo = sh.kmin, width = sh.kmax - sh.kmin;
    bool clamped = width > 0x07ffffffu;
    if (clamped) {
        lo = sh.kmax - 0x07ffffffu;
        width = 0x07ffffffu;
    }
    int rem = m;
    bool on_list = false;
    int list_n = 0;
    while (true) {
        const int s = ss_shift_for(width);
        for (int i = tid; i < SS_BUCKETS; i += NT) sh.hist[i] = 0;
        __syncthreads();
        if (on_list) {
            for (int i = tid; i < list_n; i += NT) {
                const uint32_t d = sh.list[i] - lo;
                if (d <= width) atomicAdd(&sh.hist[d >> s], 1);
            }
        } else {
            ss_for_keys<NT, RAW>(src, n, aligned, [&](uint32_t u) {
                const uint32_t d = u - lo;
                if (d <= width) atomicAdd(&sh.hist[d >> s], 1);
            });
        }
        __syncthreads();
        ss_pick_bucket<NT>(sh, rem);
        const int b = sh.bucket, cnt = sh.bucket_cnt;
        if (b < 0) {
            if (clamped) {                             // fewer than m keys in the clamped range
                clamped = false;
                lo = sh.kmin;
                width = sh.kmax - sh.kmin;
                __syncthreads();
                continue;
            }
            if (tid == 0) out->mode = 0;               // cannot happen for 1 <= rem <= keys in range
            __syncthreads();
            return true;
        }
        clamped = false;
        rem -= sh.above;
        const uint32_t nlo = lo + ((uint32_t)b << s);
        const uint32_t span = s > 0 ? ((1u << s) - 1u) : 0u;
        width = min(lo + width - nlo, span);
        lo = nlo;
        if (s == 0) {
            if (tid == 0) {
                out->mode = 3;
                out->kth = lo;
                out->need_eq = rem;
                out->all_eq = rem == cnt;
            }
            __syncthreads();
            return true;
        }
        if (!on_list && cnt <= SS_LIST_CAP) {
            if (tid == 0) sh.list_n = 0;
            __syncthreads();
            ss_for_keys<NT, RAW>(src, n, aligned, [&](uint32_t u) {
                if (u - lo <= width) {
                    const int at = atomicAdd(&sh.list_n, 1);
                    if (at < SS_LIST_CAP) sh.list[at] = u;
                }
            });
            __syncthreads();
            list_n = min(sh.list_n, SS_LIST_CAP);
            on_list = true;
            if (list_n <= SS_RANK_CAP) {
                // a short list: the rem-th largest key by counting, for every listed key, the keys above it and the
                // keys equal to it (one round instead of a histogram per 12 bits)
                for (int i = tid; i < list_n; i += NT) {
                    const uint32_t ki = sh.list[i];
                    int g = 0, ge = 0;
                    for (int q = 0; q < list_n; ++q) {
                        const uint32_t kq = sh.list[q];
                        g += kq > ki ? 1 : 0;
                        ge += kq >= ki ? 1 : 0;
                    }
                    if (g < rem && rem <= ge) {          // every copy of the key writes the same values
                        out->mode = 3;
                        out->kth = ki;
                        out->need_eq = rem - g;
                        out->all_eq = (rem - g) == (ge - g);
                    }
                }
                __syncthreads();
                return true;
            }
        }
        __syncthreads();
    }
}

// gt / eq words of word w for one array's result.  The warp's 32 words start at word wb; `tile` is the warp's
// staging tile.  All lanes of the warp call this together (mode 3 synchronises the warp).
template <int NT>
__device__ __forceinline__ void ss_word_bits(const SsResult& r, const float* __restrict__ src, int w, int wb, int n, bool aligned,
                                             uint32_t valid, uint4* tile, uint32_t& gt, uint32_t& eq) {
    const int lane = threadIdx.x & 31;
    gt = 0u;
    eq = 0u;
    if (r.mode == 1) {
        gt = valid;
    } else if (r.mode == 2) {
        const int a = r.lo - 32 * w;                   // first kept bit of this word
        gt = a <= 0 ? valid : (a >= 32 ? 0u : (valid & ~((1u << a) - 1u)));
    } else if (r.mode == 3) {
        uint32_t k[32];
        if (aligned && 32 * wb + 1024 <= n) {
            // the warp's 32 words: eight coalesced loads, swizzled tile, one word per lane
            const float4* src4 = reinterpret_cast<const float4*>(src) + 8 * (size_t)wb;
            float4 f[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) f[q] = __ldg(src4 + q * 32 + lane);
            __syncwarp();
            if (r.raw) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int row = 4 * q + (lane >> 3), c = lane & 7;
                    tile[row * 8 + (c ^ (row & 7))] = ss_keys4<true>(f[q]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int row = 4 * q + (lane >> 3), c = lane & 7;
                    tile[row * 8 + (c ^ (row & 7))] = ss_keys4<false>(f[q]);
                }
            }
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 u = tile[lane * 8 + (c ^ (lane & 7))];
                k[4 * c] = u.x; k[4 * c + 1] = u.y; k[4 * c + 2] = u.z; k[4 * c + 3] = u.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const float v = (valid >> e & 1u) ? __ldg(src + 32 * (size_t)w + e) : 0.f;
                k[e] = r.raw ? ss_key<true>(v) : ss_key<false>(v);
            }
        }
        const uint32_t kth = r.kth;
        if (r.all_eq) {
            // every key equal to the threshold is kept: one comparison per key (k >= kth), gathered through the carry
            // flag (the subtraction leaves "no borrow" in it, the add-with-carry shifts it into the word), last key first
#pragma unroll
            for (int e = 31; e >= 0; --e) {
                uint32_t tmp;
                asm("{\n\tsub.cc.u32 %1, %2, %3;\n\taddc.u32 %0, %0, %0;\n\t}" : "+r"(gt), "=r"(tmp) : "r"(k[e]), "r"(kth));
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                gt |= (k[e] > kth ? 1u : 0u) << e;
                eq |= (k[e] == kth ? 1u : 0u) << e;
            }
        }
        gt &= valid;
        eq &= valid;
    }
}

__device__ __forceinline__ uint32_t ss_lowest_bits(uint32_t word, int cnt) {      // the cnt lowest set bits of word
    if (cnt <= 0) return 0u;
    if (cnt >= __popc(word)) return word;
    uint32_t r = 0u;
    for (int i = 0; i < cnt; ++i) {
        const uint32_t b = word & (0u - word);
        r |= b;
        word ^= b;
    }
    return r;
}

template <int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) h2o_select_stream_kernel(const float* acc, const float* ts, int stride,
                                                                           const int* seg_len, int n_all, int num_heavy,
                                                                           int num_recent, uint8_t* evict_mask, int* keep_idx,
                                                                           int keep_stride, int* kept_count) {
    extern __shared__ __align__(16) unsigned char ss_raw[];
    SsShared& sh = *reinterpret_cast<SsShared*>(ss_raw);
    const int seg = blockIdx.x, tid = threadIdx.x, warp = tid >> 5;
    int n = seg_len ? seg_len[seg] : n_all;
    n = max(0, min(n, stride));
    const float* a = acc + (size_t)seg * stride;
    const float* t = ts + (size_t)seg * stride;
    const bool al_a = (reinterpret_cast<uintptr_t>(a) & 15) == 0, al_t = (reinterpret_cast<uintptr_t>(t) & 15) == 0;
    // the timestamps first: they are read once, the scores up to four times, and read last the scores are the
    // array still in L2 when the later passes come back to them
    if (!ss_find<NT, true, true>(t, n, min(num_recent, n), al_t, sh, &sh.res[1]))
        ss_find<NT, true, false>(t, n, min(num_recent, n), al_t, sh, &sh.res[1]);
    if (!ss_find<NT, false, true>(a, n, min(num_heavy, n), al_a, sh, &sh.res[0]))
        ss_find<NT, false, false>(a, n, min(num_heavy, n), al_a, sh, &sh.res[0]);
    __syncthreads();
    const SsResult ra = sh.res[0], rt = sh.res[1];
    const bool ties_a = ra.mode == 3 && !ra.all_eq, ties_t = rt.mode == 3 && !rt.all_eq;
    uint8_t* mrow = evict_mask ? evict_mask + (size_t)seg * stride : nullptr;
    const bool mask_vec = mrow != nullptr && (reinterpret_cast<uintptr_t>(mrow) & 15) == 0;
    int* krow = keep_idx ? keep_idx + (size_t)seg * keep_stride : nullptr;
    const int words_cap = (stride + 31) >> 5;
    int eq_a_before = 0, eq_t_before = 0, kept_before = 0;
    for (int w0 = 0; w0 < words_cap; w0 += NT) {
        const int w = w0 + tid, wb = w0 + 32 * warp;
        const int left = n - 32 * w;
        const uint32_t valid = (w >= words_cap || left <= 0) ? 0u : (left >= 32 ? 0xffffffffu : ((1u << left) - 1u));
        uint32_t gta, eqa, gtt, eqt;
        ss_word_bits<NT>(ra, a, w, wb, n, al_a, valid, sh.tile[warp], gta, eqa);
        ss_word_bits<NT>(rt, t, w, wb, n, al_t, valid, sh.tile[warp], gtt, eqt);
        uint32_t keep = gta | gtt;
        if (ties_a || ties_t) {
            // equal keys in index order: packed counts of both arrays (a chunk holds at most 32 * NT < 65536 positions)
            int total;
            const int packed = (ties_a ? __popc(eqa) : 0) | ((ties_t ? __popc(eqt) : 0) << 16);
            const int before = ss_block_scan<NT>(packed, sh.red_i, total);
            keep |= ties_a ? ss_lowest_bits(eqa, ra.need_eq - (eq_a_before + (before & 0xffff))) : eqa;
            keep |= ties_t ? ss_lowest_bits(eqt, rt.need_eq - (eq_t_before + (before >> 16))) : eqt;
            eq_a_before += total & 0xffff;
            eq_t_before += total >> 16;
        } else {
            keep |= eqa | eqt;
        }
        int total;
        int rpos = kept_before + ss_block_scan<NT>(__popc(keep), sh.red_i, total);
        kept_before += total;
        if (w < words_cap) {
            if (mrow) {
                const uint32_t ev = ~keep;
                if (mask_vec && (stride & 15) == 0 && 32 * w + 32 <= stride) {
                    uint32_t by[8];
#pragma unroll
                    for (int g = 0; g < 8; ++g) by[g] = (((ev >> (4 * g)) & 0xfu) * 0x00204081u) & 0x01010101u;
                    uint4* mp = reinterpret_cast<uint4*>(mrow + 32 * (size_t)w);
                    mp[0] = make_uint4(by[0], by[1], by[2], by[3]);
                    mp[1] = make_uint4(by[4], by[5], by[6], by[7]);
                } else {
                    for (int e = 0; e < 32 && 32 * w + e < stride; ++e) mrow[32 * (size_t)w + e] = (ev >> e) & 1u;
                }
            }
            if (krow) {
                uint32_t bits = keep;
                while (bits) {
                    const int e = __ffs(bits) - 1;
                    bits &= bits - 1u;
                    if (rpos < keep_stride) krow[rpos] = 32 * w + e;
                    ++rpos;
                }
            }
        }
    }
    if (tid == 0 && kept_count) kept_count[seg] = kept_before;
}

__global__ void h2o_accumulate_kernel(float* acc, float* ts, int n, const int* idx, const float* w, int m, float now,
                                      unsigned* status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int j = idx ? idx[i] : i;
    if (j < 0 || j >= n) {
        if (status) atomicOr(status, PIKV_ST_BAD_INDEX);
        return;
    }
    acc[j] = __fadd_rn(acc[j], w[i]);
    ts[j] = now;
}
__global__ void h2o_decay_kernel(float* acc, int n, float decay) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] = __fmul_rn(acc[i], decay);
}

// ---- compaction ---------------------------------------------------------------------
struct CompactDev {
    pikv_compact_params p;
    int heads_per;   // heads moved per segment
};

// Eight lanes move one row (16 bytes each of K and of V); a group handles COMPACT_ITEMS rows per tile.  The chain
// kept index -> page ids -> row is three dependent loads deep: a CTA walks several tiles of its segment as a software
// pipeline, loading the kept indices of tile t+2 and the page ids of tile t+1 while the rows of tile t are in flight.
// A bare gather of this pattern (scattered 128-byte rows, one in sixteen, contiguous writes) runs at 5.9 TB/s; what
// separates this kernel from it is instruction count (the launch was issue-bound at 104 warp instructions per row
// before the loop was slimmed: no division by the head count, 32-bit pool rows, one predicated side load per lane) and
// the sector-sized reads behind the 2- and 4-byte side values.  Two rows per group at five CTAs per SM measured best
// (four rows at three CTAs: 139 us, one row at eight: 131 us, two at five: 127 us).
constexpr int COMPACT_ITEMS = 2;
constexpr int COMPACT_TILE = 256 / 8 * COMPACT_ITEMS;     // rows (x head slots) of one tile

struct CompactTile {          // what a group knows about its COMPACT_ITEMS rows of one tile
    int j[COMPACT_ITEMS], spos[COMPACT_ITEMS], spage[COMPACT_ITEMS], dpage[COMPACT_ITEMS];
};

// PER_HEAD: one segment per (sequence, head) and one head slot per row (no division by the head count in the loop).
// The six side values of a row (two scales, two zero points, score, timestamp) are moved by lanes 0..5 of its group:
// every lane fixes its source, destination, element size and index kind once, so the loop has one predicated load
// and one store per row for them instead of a six-way branch.
template <bool PER_HEAD>
__global__ void __launch_bounds__(256, 5) h2o_compact_kernel(CompactDev c) {
    const pikv_compact_params& p = c.p;
    const int seg = blockIdx.x;
    const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
    const int seq = PER_HEAD ? seg / p.n_kv : seg;
    const int seg_head = PER_HEAD ? seg % p.n_kv : 0;
    constexpr int PTK = PIKV_PAGE_TOKENS;
    if (seq >= p.num_seqs) {
        if (p.status && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(p.status, PIKV_ST_BAD_INDEX);
        return;
    }
    const int heads_per = PER_HEAD ? 1 : c.heads_per;
    const int items_cap = p.keep_stride * heads_per;              // (row, head slot) items of a segment, at most
    const int tiles = (items_cap + COMPACT_TILE - 1) / COMPACT_TILE;
    const int dstride = p.dst_score_stride > 0 ? p.dst_score_stride : p.score_stride;
    const bool has_zp = p.src_k_zp && p.dst_k_zp, has_acc = p.src_acc && p.dst_acc, has_ts = p.src_ts && p.dst_ts;
    // this lane's side value: element size (0: none), whether it is indexed by the pool row or by the score position
    const unsigned char* side_src = nullptr;
    unsigned char* side_dst = nullptr;
    int side_size = 0;
    const bool side_by_row = sub < 4;
    if (sub == 0) side_src = static_cast<const unsigned char*>(p.src_k_scale), side_dst = static_cast<unsigned char*>(p.dst_k_scale), side_size = 2;
    else if (sub == 1) side_src = static_cast<const unsigned char*>(p.src_v_scale), side_dst = static_cast<unsigned char*>(p.dst_v_scale), side_size = 2;
    else if (sub == 2 && has_zp) side_src = static_cast<const unsigned char*>(p.src_k_zp), side_dst = static_cast<unsigned char*>(p.dst_k_zp), side_size = 4;
    else if (sub == 3 && has_zp) side_src = static_cast<const unsigned char*>(p.src_v_zp), side_dst = static_cast<unsigned char*>(p.dst_v_zp), side_size = 4;
    else if (sub == 4 && has_acc) side_src = reinterpret_cast<const unsigned char*>(p.src_acc + (size_t)seg * p.score_stride), side_dst = reinterpret_cast<unsigned char*>(p.dst_acc + (size_t)seg * dstride), side_size = 4;
    else if (sub == 5 && has_ts) side_src = reinterpret_cast<const unsigned char*>(p.src_ts + (size_t)seg * p.score_stride), side_dst = reinterpret_cast<unsigned char*>(p.dst_ts + (size_t)seg * dstride), side_size = 4;
    const int* keep_row = p.keep_idx + (size_t)seg * p.keep_stride;
    const int* spt_row = p.src_page_table + (size_t)seq * p.max_pages;
    const int* dpt_row = p.dst_page_table + (size_t)seq * p.max_pages;
    const unsigned char* sk = static_cast<const unsigned char*>(p.src_k_codes);
    const unsigned char* sv = static_cast<const unsigned char*>(p.src_v_codes);
    unsigned char* dk = static_cast<unsigned char*>(p.dst_k_codes);
    unsigned char* dv = static_cast<unsigned char*>(p.dst_v_codes);
    const bool b8 = p.bits == 8;

    // stage 1: the kept indices of a tile (speculative: rows past the kept count are dropped in stage 2)
    auto load_idx = [&](int tile, CompactTile& t) {
#pragma unroll
        for (int i = 0; i < COMPACT_ITEMS; ++i) {
            const int item = tile * COMPACT_TILE + i * 32 + grp;
            t.j[i] = PER_HEAD ? item : item / heads_per;
            t.spos[i] = (tile < tiles && t.j[i] < p.keep_stride) ? __ldg(keep_row + t.j[i]) : -1;
        }
    };
    // stage 2: page ids (spos < 0 afterwards: nothing to move)
    auto load_pages = [&](int kept, CompactTile& t) {
#pragma unroll
        for (int i = 0; i < COMPACT_ITEMS; ++i) {
            bool on = t.spos[i] >= 0 && t.j[i] < kept;
            if (t.j[i] < kept && (t.spos[i] < 0 || t.spos[i] / PTK >= p.max_pages || t.j[i] / PTK >= p.max_pages ||
                                  (p.score_stride > 0 && t.spos[i] >= p.score_stride))) {
                if (p.status && sub == 0) atomicOr(p.status, PIKV_ST_BAD_INDEX);
                on = false;
            }
            t.spage[i] = on ? __ldg(spt_row + t.spos[i] / PTK) : 0;
            t.dpage[i] = on ? __ldg(dpt_row + t.j[i] / PTK) : 0;
            if (!on) t.spos[i] = -1;
        }
    };

    const int kept = min(__ldg(p.kept_count + seg), p.keep_stride);
    CompactTile cur, nxt, nxt2;
    int tile = blockIdx.y;
    load_idx(tile, cur);
    load_idx(tile + gridDim.y, nxt);
    load_pages(kept, cur);
    for (; tile < tiles; tile += gridDim.y) {
        load_idx(tile + 2 * gridDim.y, nxt2);
        // stage 3: the rows of this tile
        uint4 kc[COMPACT_ITEMS], vc[COMPACT_ITEMS];
        uint32_t side[COMPACT_ITEMS];
        unsigned dprow[COMPACT_ITEMS];        // destination pool row (pools hold fewer than 2^31 rows)
#pragma unroll
        for (int i = 0; i < COMPACT_ITEMS; ++i) {
            bool on = cur.spos[i] >= 0;
            if (on && ((unsigned)cur.spage[i] >= (unsigned)p.num_pages || (unsigned)cur.dpage[i] >= (unsigned)p.num_pages)) {
                if (p.status && sub == 0) atomicOr(p.status, PIKV_ST_BAD_PAGE);
                on = false;
                cur.spos[i] = -1;
            }
            kc[i] = vc[i] = make_uint4(0u, 0u, 0u, 0u);
            side[i] = 0u;
            dprow[i] = 0u;
            if (!on) continue;
            int hs = 0;
            if (!PER_HEAD) hs = (tile * COMPACT_TILE + i * 32 + grp) % heads_per;
            const int head = PER_HEAD ? seg_head : hs;
            const int srow = cur.spos[i] % PTK, drow = cur.j[i] % PTK;
            const unsigned sprow = ((unsigned)cur.spage[i] * (unsigned)p.n_kv + (unsigned)head) * PTK + (unsigned)srow;
            dprow[i] = ((unsigned)cur.dpage[i] * (unsigned)p.n_kv + (unsigned)head) * PTK + (unsigned)drow;
            if (b8) {
                const size_t so = (size_t)sprow * 128 + 16 * swz8_chunk(srow, sub);
                kc[i] = ld_stream_16(sk + so);
                vc[i] = ld_stream_16(sv + so);
            } else {
                const size_t so = (size_t)sprow * 64 + 8 * swz4_unit(srow, sub);
                const uint2 a2 = *reinterpret_cast<const uint2*>(sk + so);
                const uint2 b2 = *reinterpret_cast<const uint2*>(sv + so);
                kc[i].x = a2.x; kc[i].y = a2.y;
                vc[i].x = b2.x; vc[i].y = b2.y;
            }
            if (side_size != 0 && (side_by_row || hs == 0)) {
                const size_t at = side_by_row ? (size_t)sprow : (size_t)cur.spos[i];
                side[i] = side_size == 2 ? (uint32_t)*reinterpret_cast<const uint16_t*>(side_src + at * 2)
                                         : *reinterpret_cast<const uint32_t*>(side_src + at * 4);
            }
        }
        load_pages(kept, nxt);                 // the next tile's indices have had a tile's time to arrive
#pragma unroll
        for (int i = 0; i < COMPACT_ITEMS; ++i) {
            if (cur.spos[i] < 0) continue;
            const int drow = cur.j[i] % PTK;
            if (b8) {
                const size_t dofs = (size_t)dprow[i] * 128 + 16 * swz8_chunk(drow, sub);
                *reinterpret_cast<uint4*>(dk + dofs) = kc[i];
                *reinterpret_cast<uint4*>(dv + dofs) = vc[i];
            } else {
                const size_t dofs = (size_t)dprow[i] * 64 + 8 * swz4_unit(drow, sub);
                *reinterpret_cast<uint2*>(dk + dofs) = make_uint2(kc[i].x, kc[i].y);
                *reinterpret_cast<uint2*>(dv + dofs) = make_uint2(vc[i].x, vc[i].y);
            }
            int hs = 0;
            if (!PER_HEAD) hs = (tile * COMPACT_TILE + i * 32 + grp) % heads_per;
            if (side_size != 0 && (side_by_row || hs == 0)) {
                const size_t at = side_by_row ? (size_t)dprow[i] : (size_t)cur.j[i];
                if (side_size == 2) *reinterpret_cast<uint16_t*>(side_dst + at * 2) = (uint16_t)side[i];
                else *reinterpret_cast<uint32_t*>(side_dst + at * 4) = side[i];
            }
        }
        cur = nxt;
        nxt = nxt2;
    }
}

// acc[b, kvh, pos] += sum over the group's query heads of exp(score - lse)
__global__ void h2o_accumulate_attn_kernel(const float* scores, int score_stride, const float* lse, const int* seq_len,
                                           int B, int n_q, int n_kv, float* acc, int acc_stride) {
    const int pos = blockIdx.x * blockDim.x + threadIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / n_kv, h = bh % n_kv;
    const int len = seq_len ? seq_len[b] : score_stride;
    if (pos >= len || pos >= acc_stride) return;
    const int g = n_q / n_kv;
    float s = 0.f;
    for (int i = 0; i < g; ++i) {
        const int qh = h * g + i;
        s += expf(scores[((size_t)b * n_q + qh) * score_stride + pos] - lse[(size_t)b * n_q + qh]);
    }
    acc[(size_t)bh * acc_stride + pos] += s;
}

// the same increment from the decode kernel's compact output: f16 probabilities relative to the maximum of their
// softmax step, that maximum per 16-position page (log2 domain), and the final log-sum-exp.  A thread owns eight
// consecutive positions (one 16-byte load per query head, the step's factor once per thread, acc as two float4);
// rows that are not 16-byte aligned, and the ragged end of a row, take the scalar path.
__global__ void __launch_bounds__(256) h2o_accumulate_probs_kernel(const __half* probs, int probs_stride, const float* step_max,
                                                                   int step_stride, const float* lse, const int* seq_len, int B,
                                                                   int n_q, int n_kv, float* acc, int acc_stride, int vec_ok) {
    const int pos0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    const int bh = blockIdx.y;
    const int b = bh / n_kv, h = bh % n_kv;
    int len = seq_len ? seq_len[b] : probs_stride;
    len = min(min(len, acc_stride), min(probs_stride, step_stride * 16));
    if (pos0 >= len) return;
    const int g = n_q / n_kv;
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const bool full = vec_ok && pos0 + 8 <= len;
    for (int i = 0; i < g; ++i) {
        const size_t hq = (size_t)b * n_q + (size_t)h * g + i;
        const float f = exp2f(step_max[hq * step_stride + (pos0 >> 4)] - lse[hq] * 1.4426950408889634f);
        if (full) {
            const uint4 v = ld_stream_16(probs + hq * probs_stride + pos0);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                s[2 * q] += p2.x * f;
                s[2 * q + 1] += p2.y * f;
            }
        } else {
            for (int e = 0; e < 8 && pos0 + e < len; ++e) s[e] += __half2float(probs[hq * probs_stride + pos0 + e]) * f;
        }
    }
    float* arow = acc + (size_t)bh * acc_stride + pos0;
    if (full) {
        float4 a0 = reinterpret_cast<float4*>(arow)[0], a1 = reinterpret_cast<float4*>(arow)[1];
        a0.x += s[0]; a0.y += s[1]; a0.z += s[2]; a0.w += s[3];
        a1.x += s[4]; a1.y += s[5]; a1.z += s[6]; a1.w += s[7];
        reinterpret_cast<float4*>(arow)[0] = a0;
        reinterpret_cast<float4*>(arow)[1] = a1;
    } else {
        for (int e = 0; e < 8 && pos0 + e < len; ++e) arow[e] += s[e];
    }
}

}  // namespace pikv

using namespace pikv;

// 0: the streaming select; 1: radix select on keys staged in shared memory; 2: radix select on re-read scores;
// 3: bucketed select on staged keys (1 and 3 fall back to 2 for segments longer than shared memory holds).
// Process-wide, for tests: the four routines must agree bit for bit.
static int g_h2o_select_variant = 0;
static int h2o_select_variant_for_tests() { return g_h2o_select_variant; }
extern "C" int pikv_h2o_select_variant(int32_t variant) {
    PIKV_REQUIRE(variant >= 0 && variant <= 3, PIKV_EINVAL, "h2o_select_variant: 0..3");
    g_h2o_select_variant = variant;
    return PIKV_OK;
}

extern "C" int pikv_h2o_accumulate(float* acc, float* ts, int32_t n, const int32_t* idx, const float* w, int32_t m,
                                   float now, float decay, uint32_t* status, pikv_stream_t stream) {
    PIKV_REQUIRE(acc && ts && w, PIKV_EINVAL, "h2o_accumulate: null pointer");
    PIKV_REQUIRE(n > 0 && m >= 0 && (idx != nullptr || m <= n), PIKV_EINVAL, "h2o_accumulate: bad sizes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int launches = 0;
    if (decay != 1.0f) {
        h2o_decay_kernel<<<ceil_div(n, 256), 256, 0, st>>>(acc, n, decay);
        ++launches;
    }
    if (m > 0) {
        h2o_accumulate_kernel<<<ceil_div(m, 256), 256, 0, st>>>(acc, ts, n, idx, w, m, now, status);
        ++launches;
    }
    count_launch(launches);
    return check_launch("h2o_accumulate");
}

extern "C" int pikv_h2o_select(const float* acc, const float* ts, int32_t segments, int32_t stride,
                               const int32_t* seg_len, int32_t n, int32_t num_heavy, int32_t num_recent,
                               uint8_t* evict_mask, int32_t* keep_idx, int32_t keep_stride, int32_t* kept_count,
                               pikv_stream_t stream) {
    PIKV_REQUIRE(acc && ts, PIKV_EINVAL, "h2o_select: null scores");
    PIKV_REQUIRE(segments > 0 && stride > 0 && n >= 0 && n <= stride, PIKV_EINVAL, "h2o_select: bad sizes");
    PIKV_REQUIRE(num_heavy >= 0 && num_recent >= 0, PIKV_EINVAL, "h2o_select: negative counts");
    PIKV_REQUIRE(keep_idx == nullptr || keep_stride > 0, PIKV_EINVAL, "h2o_select: keep_stride");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t words = (size_t)(stride + 31) / 32 * 4;
    const int variant = h2o_select_variant_for_tests();
    if (variant == 0) {
        auto kern = h2o_select_stream_kernel<SS_THREADS>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SsShared)) != cudaSuccess)
            return check_launch("h2o_select smem attribute");
        kern<<<segments, SS_THREADS, sizeof(SsShared), st>>>(acc, ts, stride, seg_len, n, num_heavy, num_recent, evict_mask,
                                                             keep_idx, keep_stride, kept_count);
        count_launch(1);
        return check_launch("h2o_select_stream_kernel");
    }
    // the staged routines when the segment fits in shared memory; longer segments re-read the scores from L2
    const bool staged = stride <= SEL_SMEM_KEYS && variant != 2;
    const bool radix_only = variant == 1;
    if (staged) {
        size_t smem = ((words + 15) & ~(size_t)15) + (size_t)((stride + 3) & ~3) * 4 + (size_t)SEL_CAND_CAP * 4 +
                      (size_t)SEL_BUCKETS * 4;
        auto kern = h2o_select_kernel<true, SEL_THREADS>;
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("h2o_select smem attribute");
        kern<<<segments, SEL_THREADS, smem, st>>>(acc, ts, stride, seg_len, n, num_heavy, num_recent, evict_mask,
                                                  keep_idx, keep_stride, kept_count, radix_only);
    } else {
        PIKV_REQUIRE(words <= 200 * 1024, PIKV_ELIMIT, "h2o_select: stride=%d too long", stride);
        const size_t smem = ((words + 15) & ~(size_t)15) + (size_t)SEL_CAND_CAP * 4;
        auto kern = h2o_select_kernel<false, SEL_THREADS_STREAM>;
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("h2o_select smem attribute");
        kern<<<segments, SEL_THREADS_STREAM, smem, st>>>(acc, ts, stride, seg_len, n, num_heavy, num_recent, evict_mask,
                                                   keep_idx, keep_stride, kept_count, true);
    }
    count_launch(1);
    return check_launch("h2o_select_kernel");
}

extern "C" int pikv_h2o_compact(const pikv_compact_params* p, pikv_stream_t stream) {
    PIKV_REQUIRE(p != nullptr, PIKV_EINVAL, "h2o_compact: null params");
    PIKV_REQUIRE(p->keep_idx && p->kept_count && p->src_page_table && p->dst_page_table, PIKV_EINVAL,
                 "h2o_compact: null index pointer");
    PIKV_REQUIRE(p->src_k_codes && p->src_v_codes && p->src_k_scale && p->src_v_scale && p->dst_k_codes &&
                     p->dst_v_codes && p->dst_k_scale && p->dst_v_scale,
                 PIKV_EINVAL, "h2o_compact: null cache pointer");
    PIKV_REQUIRE(p->num_seqs > 0 && p->n_kv > 0 && p->keep_stride > 0 && p->max_pages > 0, PIKV_EINVAL,
                 "h2o_compact: bad sizes");
    PIKV_REQUIRE(p->bits == 8 || p->bits == 4, PIKV_EUNSUPPORTED, "h2o_compact: bits=%d", p->bits);
    PIKV_REQUIRE((p->src_acc == nullptr) == (p->dst_acc == nullptr) && (p->src_ts == nullptr) == (p->dst_ts == nullptr), PIKV_EINVAL,
                 "h2o_compact: scores / timestamps need both a source and a destination");
    PIKV_REQUIRE((p->src_acc == nullptr && p->src_ts == nullptr) ||
                     (p->score_stride > 0 && (p->dst_score_stride == 0 || p->dst_score_stride >= p->keep_stride) &&
                      (p->dst_score_stride != 0 || p->score_stride >= p->keep_stride)),
                 PIKV_EINVAL, "h2o_compact: score_stride=%d dst_score_stride=%d keep_stride=%d", p->score_stride,
                 p->dst_score_stride, p->keep_stride);
    CompactDev c;
    c.p = *p;
    c.heads_per = p->per_head ? 1 : p->n_kv;
    const int segments = p->per_head ? p->num_seqs * p->n_kv : p->num_seqs;
    const long long lanes = (long long)p->keep_stride * c.heads_per * 8;
    // a CTA walks up to four tiles of its segment (software pipeline); enough CTAs to fill the GPU a few times over
    const long long tiles = ceil_div64(lanes, 256 * COMPACT_ITEMS);
    long long per_seg = ceil_div64(tiles, 4);                        // four tiles per CTA ...
    const long long fill = (long long)sm_count() * 12 / segments;    // ... unless that leaves SMs idle
    if (per_seg < fill) per_seg = fill;
    if (per_seg > tiles) per_seg = tiles;
    if (per_seg < 1) per_seg = 1;
    dim3 grid(segments, (unsigned)per_seg);
    PIKV_REQUIRE((long long)p->num_pages * p->n_kv * PIKV_PAGE_TOKENS < (1ll << 31), PIKV_ELIMIT,
                 "h2o_compact: the pools must hold fewer than 2^31 rows");
    if (p->per_head) h2o_compact_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(c);
    else h2o_compact_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(c);
    count_launch(1);
    return check_launch("h2o_compact_kernel");
}

extern "C" int pikv_h2o_accumulate_probs(const void* probs16, int32_t probs_stride, const float* step_max, int32_t step_stride,
                                         const float* lse, const int32_t* seq_len, int32_t B, int32_t n_q, int32_t n_kv,
                                         float* acc, int32_t acc_stride, pikv_stream_t stream) {
    PIKV_REQUIRE(probs16 && step_max && lse && acc, PIKV_EINVAL, "h2o_accumulate_probs: null pointer");
    PIKV_REQUIRE(B > 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && probs_stride > 0 && step_stride > 0 && acc_stride > 0,
                 PIKV_EINVAL, "h2o_accumulate_probs: bad sizes");
    dim3 grid(ceil_div(min(probs_stride, acc_stride), 256 * 8), B * n_kv);
    // eight positions of a page never straddle two softmax steps; vector accesses need 16-byte aligned rows
    const int vec_ok = (reinterpret_cast<uintptr_t>(probs16) & 15) == 0 && (probs_stride & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(acc) & 15) == 0 && (acc_stride & 3) == 0;
    h2o_accumulate_probs_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(probs16), probs_stride, step_max, step_stride, lse, seq_len, B, n_q, n_kv, acc, acc_stride,
        vec_ok);
    count_launch(1);
    return check_launch("h2o_accumulate_probs_kernel");
}

extern "C" int pikv_h2o_accumulate_attn(const float* scores, int32_t score_stride, const float* lse,
                                        const int32_t* seq_len, int32_t B, int32_t n_q, int32_t n_kv, float* acc,
                                        int32_t acc_stride, pikv_stream_t stream) {
    PIKV_REQUIRE(scores && lse && acc, PIKV_EINVAL, "h2o_accumulate_attn: null pointer");
    PIKV_REQUIRE(B > 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && score_stride > 0 && acc_stride > 0, PIKV_EINVAL,
                 "h2o_accumulate_attn: bad sizes");
    dim3 grid(ceil_div(min(score_stride, acc_stride), 256), B * n_kv);
    h2o_accumulate_attn_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(scores, score_stride, lse, seq_len, B,
                                                                                  n_q, n_kv, acc, acc_stride);
    count_launch(1);
    return check_launch("h2o_accumulate_attn_kernel");
}
