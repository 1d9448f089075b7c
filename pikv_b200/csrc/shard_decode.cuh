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

int decode_attn_run(const pikv_decode_params* p, cudaStream_t st, int bits, const int* q_rows, const ShardReturn* ret);

#ifdef __CUDACC__
// rows of the first `len` rows of a striped pair that rank `rank` stores (see pikv_kv_append_striped)
__device__ __forceinline__ int striped_local_len(int len, int rot, int rank, int world, int log2_stripe) {
    const int full = len >> log2_stripe, tail = len & ((1 << log2_stripe) - 1);
    const int first = (rank - rot + world) % world;
    const int n_full = full > first ? (full - first + world - 1) / world : 0;
    return (n_full << log2_stripe) + ((full % world) == first ? tail : 0);
}
#endif

}  // namespace pikv
