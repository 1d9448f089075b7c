// Pieces the decode-attention kernels and the sharded decode exchange share.
#pragma once

#include "common.cuh"

namespace pikv {

// where decode_return_kernel sends what this rank holds of every request of a sharded decode step
struct ShardReturn {
    int world, rank, top_k, streams_per_rank;
    float* peer_part_o[8];       // rank r's [streams_per_rank][top_k][world][n_q][128]
    float* peer_part_lse[8];     // rank r's [streams_per_rank][top_k][world][n_q]
    unsigned* peer_done_flags[8];  // rank r's [world]
    unsigned* counter;           // this rank's completion counter (device word, zero between launches)
    const unsigned* seq;         // this rank's step number
};

// what the plan kernel of a sharded decode call needs to build the request list itself: request i = (stream i / k,
// choice i % k), its length = the rows this rank holds of that pair
struct ShardPlan {
    int world, rank, num_experts, num_streams, top_k, log2_stripe;
    unsigned limit_us;             // bound of the wait for the ranks' "posted" flags
    const unsigned* post_flags;    // this rank's [world]
    const unsigned* seq;           // this rank's step number
    const int4* route;             // this rank's copy of the routing records [num_streams * top_k]
    const int* expert_rot;         // [num_experts]
    unsigned* status;
    int* seq_ids;                  // out [num_streams * top_k]: the same arrays the decode call reads
    int* seq_len;
    int* q_rows;
};

int decode_attn_run(const pikv_decode_params* p, cudaStream_t st, int bits, const int* q_rows, const ShardReturn* ret,
                    const ShardPlan* plan);

constexpr unsigned SD_FAILED = 0x80000000u;      // top bit of a rank's step number: a wait of that rank ran out

#ifdef __CUDACC__
__device__ __forceinline__ void sd_flag_store(unsigned* flag, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
// polls a flag word a peer writes until it shows `want`, about a microsecond per poll, limit_us polls at most
__device__ __forceinline__ bool sd_flag_wait(const unsigned* flag, unsigned want, unsigned limit_us) {
    for (unsigned spins = 0;; ++spins) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
        if (seen == want) return true;
        if (spins >= limit_us) return false;
        __nanosleep(1000);
    }
}
// rows of the first `len` rows of a striped pair that rank `rank` stores (see pikv_kv_append_striped)
__device__ __forceinline__ int striped_local_len(int len, int rot, int rank, int world, int log2_stripe) {
    const int full = len >> log2_stripe, tail = len & ((1 << log2_stripe) - 1);
    const int first = (rank - rot + world) % world;
    const int n_full = full > first ? (full - first + world - 1) / world : 0;
    return (n_full << log2_stripe) + ((full % world) == first ? tail : 0);
}
#endif

}  // namespace pikv
