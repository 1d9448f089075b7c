/*
 * pikv_b200 - C ABI of the B200 (sm_100a) routed KV-cache kernels.
 *
 * One shared object, libpikv_b200.so.  Every entry point takes plain device
 * pointers and sizes, enqueues its kernels on the stream it is given and
 * returns immediately with 0 or a negative PIKV_E* code; pikv_last_error()
 * gives the message for the calling thread.  The library never allocates
 * device memory (scratch is passed in by the caller, sized by the matching
 * *_workspace_bytes function), never synchronises the device and has no CPU
 * fallback.
 *
 * The reference project's native boundary is a set of
 *   extern "C" void launch_<kernel>(const float* ..., int dims..., cudaStream_t)
 * functions with no return code (core/cuda/pikv_routing_kernel.cu:404-511,
 * core/cuda/pikv_compression_kernel.cu:463-623,
 * core/cuda/pikv_scheduling_kernel.cu:504-676) bound from
 * core/single/pikv_kernels.py.  Each declaration below names the launcher(s)
 * and the Python operator whose arithmetic it replaces.
 */
#ifndef PIKV_B200_H
#define PIKV_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PIKV_ABI_VERSION 1

/* status codes */
#define PIKV_OK            0
#define PIKV_EINVAL       -1  /* bad argument (null pointer, size out of range) */
#define PIKV_EUNSUPPORTED -2  /* shape / dtype combination not built           */
#define PIKV_ECUDA        -3  /* a CUDA runtime call failed at launch          */
#define PIKV_ELIMIT       -4  /* size beyond a documented fixed limit          */

/* element types of activations / K / V inputs */
#define PIKV_F32  0
#define PIKV_BF16 1

/* how expert_mask enters the logits (gate) */
#define PIKV_MASK_NONE    0
#define PIKV_MASK_SINGLE  1   /* l + (1-mask) * -1e9        core/single/pikv_routing.py:70          */
#define PIKV_MASK_MODULE  2   /* l + (1-mask) * FLT_LOWEST  core/single/module/pikv_routing.py:133  */
#define PIKV_MASK_BIAS    3   /* l + mask                   core/single/routing_strategy.py:46      */

/* bits set in the device status word that kernels OR into (never trap) */
#define PIKV_ST_BAD_SEQ     1u   /* destination sequence id out of range        */
#define PIKV_ST_BAD_PAGE    2u   /* page-table entry out of range               */
#define PIKV_ST_BAD_INDEX   8u   /* gather / scatter index out of range         */
#define PIKV_ST_WAIT_TIMEOUT 16u /* a bounded in-kernel wait ran out; result invalid */

/* tokens per cache page and the head width the cache kernels are built for */
#define PIKV_PAGE_TOKENS 16
#define PIKV_HEAD_DIM    128

typedef void* pikv_stream_t;   /* a cudaStream_t */

int         pikv_abi_version(void);
const char* pikv_last_error(void);
/* number of kernels this library has launched in the calling process */
uint64_t    pikv_launch_count(void);

/* ------------------------------------------------------------------------
 * Router gate: logits tail + softmax + top-k + load-balance counts + slots.
 *
 * Replaces launch_topk_routing_kernel / launch_load_balancing_kernel /
 * launch_adaptive_routing_kernel / launch_expert_capacity_kernel
 * (core/cuda/pikv_routing_kernel.cu:404-511) and the PyTorch tail of
 * BaseRouter.forward (core/single/pikv_routing.py:65-79,155), the running
 * per-expert position loop of core/single/module/pikv_routing.py:88-104 and
 * its usage counters (:154-160).
 *
 * Either `act`+`w2` (the gate net's last Linear: logits = act . w2^T + b2,
 * fp32 accumulate) or `logits_in` is given.  Then, per token:
 *   l = l / temperature ; l *= correction[e] ; mask ; p = softmax(l)
 *   top-k of p (ties: lowest expert index) ; w = p_top / (sum p_top + eps)
 * and, over the batch in (token, k) order, slot = slot_base[e] + running
 * count of earlier selections of e, or -1 once slot >= capacity.
 * ---------------------------------------------------------------------- */
typedef struct {
    const void*  act;          /* [T,H] dtype, or NULL                          */
    const void*  w2;           /* [E,H] dtype                                   */
    const float* b2;           /* [E] or NULL                                   */
    const float* logits_in;    /* [T,E] fp32, used when act == NULL             */
    int32_t dtype, T, H, E, top_k;
    const float* expert_mask;  /* [E] or NULL                                   */
    int32_t mask_mode;
    const float* correction;   /* [E] or NULL                                   */
    float temperature;         /* 1.0 = off                                     */
    float renorm_eps;
    int32_t capacity;          /* slots per expert; <=0: no limit               */
    const int32_t* slot_base;  /* [E] current length per expert, or NULL        */
    /* outputs (any may be NULL except topk_idx) */
    float*   probs;            /* [T,E]                                         */
    int32_t* topk_idx;         /* [T,k]                                         */
    float*   topk_w;           /* [T,k]                                         */
    int32_t* slot;             /* [T,k]                                         */
    int32_t* counts_k;         /* [k,E] selections of e in column j (dropped or not) */
    float*   prob_sum;         /* [E] sum over tokens of p[t,e]                 */
    int32_t* new_len;          /* [E] min(slot_base + count, capacity)          */
    void*    workspace;        /* pikv_gate_workspace_bytes(T,E,top_k)          */
    size_t   workspace_bytes;
    int32_t  phase;            /* PIKV_GATE_WHOLE (0), _SCORE or _SLOTS, see below */
} pikv_gate_params;

/* The gate is two kernels: scoring (logits, softmax, top-k, ranks local to each CTA's chunk of
 * tokens, per-chunk counters) and the slot finalisation (prefix over the chunks -> slot,
 * counts_k, prob_sum, new_len).  phase = PIKV_GATE_SCORE launches only the first and leaves
 * slot holding chunk-local ranks; PIKV_GATE_SLOTS, called later with the same parameters and
 * the same workspace (the caller orders it after the first: same stream or an event), only
 * the second.  For callers that keep the scoring kernels of consecutive batches back to back
 * on one stream and run the short finalisation beside them on another. */
#define PIKV_GATE_WHOLE 0
#define PIKV_GATE_SCORE 1
#define PIKV_GATE_SLOTS 2
/* OR-ed into phase: run bf16 activations through the fp32-product SIMT kernel instead of the tensor-core
 * one (the tests compare the two kernels with it; callers have no reason to set it). */
#define PIKV_GATE_FORCE_SIMT 0x100

size_t pikv_gate_workspace_bytes(int32_t T, int32_t E, int32_t top_k);
int    pikv_gate_fused(const pikv_gate_params* p, pikv_stream_t stream);
/* bf16 activations run on the tcgen05 kernel (TMA + tensor memory), fp32 ones on the SIMT
 * kernel.  Reads and clears the tensor-core kernel's sticky error word (non-zero: a bounded
 * mbarrier wait ran out and the outputs are invalid); waits for the work queued before it. */
int    pikv_gate_error_state(void);

/* The whole gate net in one kernel: logits = relu(x . w1^T + b1) . w2^T + b2, then the same tail and outputs as
 * pikv_gate_fused (the router's nn.Sequential(Linear, ReLU, Linear), core/single/pikv_routing.py:34-38, whose
 * first layer is the one dense contraction of "route": [T,K] x [K,H] on tcgen05 tensor cores, fp32 accumulation
 * in tensor memory).  The hidden activations never go to HBM: each 128-token tile keeps them in shared memory,
 * 256 hidden units at a time, as the operand of the second product.
 *   p: as for pikv_gate_fused with H = hidden units (inputs of w2 [E,H]); p->act is ignored; bf16; E <= 32;
 *   T <= 131072 per call; phase PIKV_GATE_WHOLE.
 *   x [T,K] bf16, w1 [H,K] bf16, b1 [H] fp32 or NULL. */
int pikv_gate_mlp_fused(const pikv_gate_params* p, const void* x, int32_t K, const void* w1, const float* b1,
                        pikv_stream_t stream);

/* Dense [T,E,capacity] dispatch / combine tensors (zero-filled by this call)
 * for callers that read them.  position_mode 0: slot as given (running count,
 * core/single/module/pikv_routing.py:93-104); 1: the positions
 * core/single/pikv_routing.py:107-128 produces ("number of earlier k-columns
 * in which this expert was chosen by any token"), from counts_k. */
int pikv_dispatch_scatter(const int32_t* topk_idx, const float* topk_w, const int32_t* slot,
                          const int32_t* counts_k, int32_t T, int32_t E, int32_t top_k,
                          int32_t capacity, int32_t position_mode,
                          float* dispatch, float* combine, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Routed KV append fused with per-(token, head) group quantisation.
 *
 * Replaces launch_quantization_compression_kernel
 * (core/cuda/pikv_compression_kernel.cu:485-505) and the row insert of
 * launch_lru_cache_management_kernel (core/cuda/pikv_scheduling_kernel.cu:504-525);
 * arithmetic = QuantizedCompressor._quantize_tensor
 * (core/single/module/pikv_compression.py:945-1012) applied to each
 * [1, 128] slice, row placement = CacheSchedulingManager.update_cache
 * (core/single/cache_scheduling.py:430-436) per destination sequence.
 *
 * Cache layout (all pools indexed by physical page id):
 *   codes  [pages][n_kv][16 tokens][128 * bits / 8] bytes; inside one token row
 *          the 16-byte chunk c is stored at chunk (c ^ (token_in_page & 7))
 *          for 8-bit codes, and the 8-byte unit u at unit (u ^ (token_in_page & 4))
 *          for 4-bit codes (two codes per byte, low nibble = even channel)
 *   scale  [pages][n_kv][16] bf16
 *   zp     [pages][n_kv][16] fp32 (asymmetric only; the reference's zero point is an
 *          integer-valued fp32 that a constant group drives to millions, so it is kept exact)
 * A "sequence" is whatever owns a page-table row: an expert, a decode stream,
 * or an (expert, stream) pair.
 * ---------------------------------------------------------------------- */
typedef struct {
    const void* k;             /* [T, n_kv*128] dtype                           */
    const void* v;
    int32_t dtype, T, n_kv, top_k;
    const int32_t* dst_seq;    /* [T,k] destination sequence (= topk_idx)       */
    const int32_t* slot;       /* [T,k] position in that sequence, <0 = dropped */
    const int32_t* page_table; /* [num_seqs, max_pages] physical page ids       */
    int32_t num_seqs, max_pages, num_pages;
    int32_t bits, symmetric;   /* (8,1) (8,0) (4,1) (4,0)                       */
    void* k_codes; void* v_codes;
    void* k_scale; void* v_scale;   /* bf16                                     */
    void* k_zp;    void* v_zp;      /* fp32, asymmetric only                    */
    uint32_t* status;          /* device word, OR-ed with PIKV_ST_* (may be NULL) */
} pikv_append_params;

int pikv_kv_append_quant(const pikv_append_params* p, pikv_stream_t stream);

/* The prefill side of the cache: the same append with the rotary position embedding of
 * RotaryEmbedding.forward (core/single/pikv_attention.py:329-390) applied to K in registers before it is
 * quantised, so the rotated K is never written in bf16 (the step PiKVAttention.forward performs between
 * k_proj and _update_cache, core/single/pikv_attention.py:226-247).  Head dim 128, halves split at 64:
 *   k'[c]      = k[c] * cos[pos][c] - k[c + 64] * sin[pos][c]        c < 64
 *   k'[c + 64] = k[c + 64] * cos[pos][c] + k[c] * sin[pos][c]
 * rope_cos / rope_sin: [max_pos][64] fp32 tables from the caller (the reference's cos_cached / sin_cached);
 * positions [T] (NULL: the token index).  bf16 in, int8 symmetric codes.  V is stored as by
 * pikv_kv_append_quant. */
int pikv_kv_append_rope(const pikv_append_params* p, const float* rope_cos, const float* rope_sin,
                        const int32_t* positions, int32_t max_pos, pikv_stream_t stream);

/* Gate + append as one call: pikv_gate_fused followed by pikv_kv_append_quant with
 * dst_seq = the gate's topk_idx and slot = the gate's slot (those two fields of `append` are
 * ignored), same outputs.  For bf16 K/V and int8 symmetric codes the stand-alone slot
 * finalisation is folded into the append kernel (every CTA rebuilds the prefix of the
 * gate's per-chunk counters in shared memory), which saves a launch and a dependent kernel
 * boundary; other combinations run the two entry points back to back. */
int pikv_route_append(const pikv_gate_params* gate, const pikv_append_params* append, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Expert-sharded routed append: quantise and store straight into the page pools of
 * the GPU that owns each destination sequence, through peer-mapped pointers (plain
 * stores over NVLink; no staging buffer, no multicast).  Replaces the
 * replicate-everything + all_reduce of DistributedPiKVMoE.forward
 * (core/distributed/distributed_pikv.py:174-194) for the cache-append side.
 *   base: k, v, dst_seq (GLOBAL sequence ids, owner = id / seqs_per_rank), slot (rank
 *   of the row inside (this GPU, sequence), i.e. the gate's slot with capacity 0),
 *   page_table = [num_seqs = world * seqs_per_rank][max_pages] with page ids local to
 *   the owner, num_pages = pages per GPU; bf16 in, int8 symmetric out; the pool
 *   pointers of `base` are ignored.
 *   slot_base [num_seqs]: position of this GPU's first row in every sequence (from
 *   pikv_shard_plan); rows landing at >= capacity are dropped.
 *   peer_*[r]: the pools of rank r as seen from this GPU (own pools at r = rank).
 * The caller orders the step against the other GPUs (all ranks must finish the call
 * before any rank reads the rows, e.g. a barrier collective on the same stream).
 * pikv_shard_plan turns the all-gathered selection counts [world][E] into slot_base
 * for this rank and advances len_all [E] (kept identically on every rank).
 * ---------------------------------------------------------------------- */
typedef struct {
    pikv_append_params base;
    int32_t world, seqs_per_rank, capacity;
    const int32_t* slot_base;
    void* peer_k_codes[8]; void* peer_v_codes[8]; void* peer_k_scale[8]; void* peer_v_scale[8];
    int32_t rank;              /* this GPU's rank (used when which != 0)                 */
    int32_t which;             /* 0: every destination; 1: only sequences this rank owns;
                                  2: only the other ranks'                                */
    void* mirror_k_scale;      /* optional, both or neither: local bf16 [world][pool entries] */
    void* mirror_v_scale;      /* buffers; the scales of rows stored on OTHER GPUs go there (at
                                  the offset they have in the owner's pool) instead of over the
                                  link, and pikv_shard_push_scales ships them afterwards         */
} pikv_append_sharded_params;

int pikv_kv_append_sharded(const pikv_append_sharded_params* p, pikv_stream_t stream);

/* NVLink moves packets, not bytes: a 2-byte scale store costs about as much as a 128-byte row
 * store (measured: one side store per row takes the row stores from 692 to 430 GB/s).  With scale
 * mirrors the sharded append keeps the scales of remote rows in local memory, and this call, on the
 * same stream after it, ships them 32 bytes (one page of one head) at a time: this rank's rows of
 * sequence e are the slots [slot_base[e], slot_base[e] + sum_j counts_k[j][e]), cut at capacity. */
typedef struct {
    const int32_t* counts_k;   /* [top_k][E], this rank's gate output               */
    const int32_t* slot_base;  /* [E], from pikv_shard_exchange_plan / pikv_shard_plan */
    const int32_t* page_table; /* [E][max_pages], page ids local to the owner          */
    int32_t top_k, E, world, rank, seqs_per_rank, capacity, n_kv, max_pages, num_pages;
    const void* mirror_k_scale; const void* mirror_v_scale;
    void* peer_k_scale[8]; void* peer_v_scale[8];
} pikv_shard_push_params;

int pikv_shard_push_scales(const pikv_shard_push_params* p, pikv_stream_t stream);
int pikv_shard_plan(const int32_t* gathered, int32_t world, int32_t E, int32_t rank, int32_t capacity,
                    int32_t* len_all, int32_t* slot_base, pikv_stream_t stream);

/* The all-gather of the selection counts and pikv_shard_plan as ONE kernel over peer memory, so
 * that a sharded step is made of this library's kernels only (no collective library call, nothing
 * on the host): every rank stores its counts into slot (step % PIKV_XCHG_RING) of every rank's
 * gather buffer over NVLink, raises the step number in every rank's flag word, waits (about two
 * seconds at most, then PIKV_ST_WAIT_TIMEOUT is raised in *status and the step's rows are dropped)
 * for all ranks' flags and computes slot_base / len_all.  All ranks must call it once per step, in
 * the same order.  gather [PIKV_XCHG_RING][world][E] int32 and flags [PIKV_XCHG_RING][world] uint32
 * live in memory every rank has mapped (peer_*[r] = rank r's copy as seen from this GPU) and start
 * zeroed, as does *seq, this rank's step counter.  start_empty != 0: lengths restart from zero.
 * Failure is shared: a rank whose wait ran out marks itself failed (top bit of *seq) and sets the top
 * bit of the flags it raises from then on; a rank that sees that bit fails at once, drops its rows and
 * raises PIKV_ST_WAIT_TIMEOUT too.  So within one more step every rank's status word shows the failure;
 * from the failing step on the sharded cache is invalid on every rank, until a step with start_empty
 * (which clears the marks) restarts it.  wait_limit_us: microseconds a wait may take (<= 0: the
 * default, PIKV_DEFAULT_WAIT_US).
 * Replaces the exchange of DistributedPiKVMoE.forward (core/distributed/distributed_pikv.py:174-194)
 * for the routing counts. */
#define PIKV_XCHG_RING 4
#define PIKV_DEFAULT_WAIT_US 2000000
typedef struct {
    const int32_t* counts_k;   /* [top_k][E], this rank's gate output             */
    int32_t top_k, E, world, rank, capacity, start_empty;
    int32_t*  peer_gather[8];
    uint32_t* peer_flags[8];
    uint32_t* seq;
    int32_t*  len_all;         /* [E] replicated lengths, advanced identically on every rank */
    int32_t*  slot_base;       /* [E] out: position of this rank's first row in every sequence */
    uint32_t* status;          /* may be NULL */
    int32_t   wait_limit_us;
} pikv_shard_exchange_params;

int pikv_shard_exchange_plan(const pikv_shard_exchange_params* p, pikv_stream_t stream);

/* Barrier across the ranks over peer-mapped flag words (flags [world] uint32 per rank, zeroed at start;
 * *seq this rank's barrier counter, zeroed): when the kernel ends on a rank, everything queued before the
 * barrier call on every rank's stream has completed, peer stores included.  The wait is bounded like every
 * other wait of this library (PIKV_ST_WAIT_TIMEOUT in *status, the kernel returns).  Stands in for the
 * implicit synchronisation of the all_reduce in DistributedPiKVMoE.forward
 * (core/distributed/distributed_pikv.py:196). */
typedef struct {
    int32_t world, rank;
    uint32_t* peer_flags[8];
    uint32_t* seq;
    uint32_t* status;          /* may be NULL */
    int32_t   wait_limit_us;   /* <= 0: PIKV_DEFAULT_WAIT_US */
} pikv_peer_barrier_params;

int pikv_peer_barrier(const pikv_peer_barrier_params* p, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Striped expert-sharded append: the cache of a pair (expert e, stream s) is cut into stripes of `stripe`
 * rows and stripe c lives on rank (expert_rot[e] + s + c) mod world, behind that rank's earlier stripes of
 * the pair (slot (c / world) * stripe + row % stripe).  Spreads both the experts and the long caches of
 * popular experts evenly over the GPUs; replaces the contiguous expert blocks of
 * core/distributed/distributed_pikv.py:91-96 for the cache.  The rank that gates a stream's tokens (its
 * home) quantises their rows and stores each straight into its owner's pages over peer pointers.
 *   base: k, v [T, n_kv*128] bf16; dst_seq [T,k] = EXPERT of every (token, j); slot [T,k] = row position
 *   inside the pair, minus pair_len[e] when pair_len is given (so the gate's slot with capacity 0 and no
 *   slot_base can be passed as it is, or its slot with slot_base = the pair lengths and pair_len = NULL);
 *   page_table [num_experts * num_streams][max_pages], the same on every rank (sequence id = e *
 *   num_streams + s, page ids local to the owner, every rank lays its pool out alike); int8 symmetric.
 *   stream: the stream all T tokens belong to, or token_stream [T] for mixed batches.
 *   expert_cap [E] (optional): rows at positions >= expert_cap[e] are dropped.
 *   which: 0 every row, 1 only rows this rank owns, 2 only the others'.
 * The caller orders the step against the other GPUs before anyone reads the rows (pikv_peer_barrier).
 * ---------------------------------------------------------------------- */
typedef struct {
    pikv_append_params base;
    int32_t world, rank, stripe, num_experts, num_streams, stream, which;
    const int32_t* token_stream;
    const int32_t* pair_len;
    const int32_t* expert_rot;
    const int32_t* expert_cap;
    void* peer_k_codes[8]; void* peer_v_codes[8]; void* peer_k_scale[8]; void* peer_v_scale[8];
    void* mirror_k_scale;      /* optional, both or neither: local bf16 [world][pool entries] buffers that take */
    void* mirror_v_scale;      /* the scales of rows stored on OTHER GPUs; pikv_shard_push_scales_striped ships them */
} pikv_append_striped_params;

int pikv_kv_append_striped(const pikv_append_striped_params* p, pikv_stream_t stream);

/* Ships the scales a striped append (one stream, with mirrors) left in the local mirrors to their owners, 32
 * bytes (one page of one head) at a time: the step appended the positions [len_before[e], min(len_after[e],
 * expert_cap[e])) to the pair of expert e and this stream.  Same stream, after the append. */
typedef struct {
    const int32_t* len_before; const int32_t* len_after;   /* [E] */
    const int32_t* expert_rot; const int32_t* expert_cap;  /* [E]; expert_cap may be NULL */
    const int32_t* page_table;                             /* [E * num_streams][max_pages] */
    int32_t world, rank, stripe, num_experts, num_streams, stream, n_kv, max_pages, num_pages;
    const void* mirror_k_scale; const void* mirror_v_scale;
    void* peer_k_scale[8]; void* peer_v_scale[8];
} pikv_striped_push_params;

int pikv_shard_push_scales_striped(const pikv_striped_push_params* p, pikv_stream_t stream);

/* Read rows back in logical order, dequantised: out[i] = (code - zp) * scale for
 * sequence seq[i], position pos[i]; out is [n, n_kv*128] fp32, codes_out
 * (optional) [n, n_kv*128] int8 unpacked codes.  Used by tests, checkpointing
 * and the host-side read path (PiKVMoE's cached rows). */
int pikv_cache_gather(const int32_t* seq, const int32_t* pos, int32_t n,
                      const int32_t* page_table, int32_t num_seqs, int32_t max_pages, int32_t num_pages,
                      int32_t n_kv, int32_t bits,
                      const void* codes, const void* scale, const void* zp,
                      float* out, int8_t* codes_out, uint32_t* status, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Block-wide fake quantisation: every column group of width group_size is
 * one block with min/max over ALL rows.  Bit-exact drop-in arithmetic of
 * QuantizedCompressor.forward (core/single/pikv_compression.py:474-506,
 * core/single/module/pikv_compression.py:1014-1051); replaces
 * launch_quantization_compression_kernel.
 *   qmin/qmax: code range; symmetric selects the scale formula.
 *   params_in (optional, [G][2] = scale, zero point): static mode, skip the
 *   statistics pass.  params_out (optional) [G][2].  sq_err (optional) [G]:
 *   sum over the block of (x - dq)^2 (mean = / (N*width)).
 * ---------------------------------------------------------------------- */
size_t pikv_quant_block_workspace_bytes(int32_t N, int32_t H, int32_t group_size);
int pikv_quant_block(const void* x, int32_t dtype, int32_t N, int32_t H, int32_t group_size,
                     int32_t qmin, int32_t qmax, int32_t symmetric,
                     const float* params_in, float* params_out,
                     float* dq_out, float* q_out, float* sq_err,
                     void* workspace, size_t workspace_bytes, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * H2O scoring and eviction.
 *
 * pikv_h2o_accumulate: acc[idx] += w ; ts[idx] = now
 *   (H2OScheduler.update_attention_scores, core/single/cache_scheduling.py:69-73;
 *   decay != 1 multiplies all n scores first, core/single/module/pikv_scheduling.py:119-125;
 *   replaces launch_cache_access_update_kernel, core/cuda/pikv_scheduling_kernel.cu:614-627).
 *   idx == NULL means idx = 0..m-1.  Indices must be distinct.
 * pikv_h2o_select: per segment keep the num_heavy largest scores and the
 *   num_recent largest timestamps, ties to the lowest index
 *   (H2OScheduler.select_eviction_candidates, core/single/cache_scheduling.py:75-99).
 *   acc, ts: [segments, stride]; seg_len[s] <= stride valid entries (NULL: all n).
 *   evict_mask [segments, stride] uint8 (1 = evict; entries past the length = 1),
 *   keep_idx [segments, keep_stride] ascending, kept_count [segments].
 * pikv_h2o_compact: copy the kept rows of a paged cache, in ascending order,
 *   to positions 0..kept-1 of the destination sequences' pages, together with
 *   their scores and timestamps (CacheSchedulingManager.update_cache evict
 *   branch, core/single/cache_scheduling.py:418-424; replaces
 *   launch_cache_compaction_kernel, core/cuda/pikv_scheduling_kernel.cu:629-652).
 *   A sequence owns n_kv segments (one per KV head) when per_head != 0 and
 *   segment s = seq * n_kv + head; otherwise one segment per sequence.
 *   Source and destination pages must not overlap.
 * ---------------------------------------------------------------------- */
int pikv_h2o_accumulate(float* acc, float* ts, int32_t n, const int32_t* idx, const float* w, int32_t m,
                        float now, float decay, uint32_t* status, pikv_stream_t stream);

int pikv_h2o_select(const float* acc, const float* ts, int32_t segments, int32_t stride,
                    const int32_t* seg_len, int32_t n, int32_t num_heavy, int32_t num_recent,
                    uint8_t* evict_mask, int32_t* keep_idx, int32_t keep_stride, int32_t* kept_count,
                    pikv_stream_t stream);

/* Testing aid: which select routine pikv_h2o_select runs (all give identical results).  0 (default): the
 * streaming select (threads own 32-position words, scores re-read from L2, bucket narrowing); 1: radix select on
 * keys staged in shared memory; 2: radix select re-reading the scores; 3: bucketed select on staged keys. */
int pikv_h2o_select_variant(int32_t variant);

typedef struct {
    const int32_t* keep_idx;   /* [segments, keep_stride]                        */
    const int32_t* kept_count; /* [segments]                                     */
    int32_t keep_stride, num_seqs, n_kv, per_head, bits;
    const int32_t* src_page_table; const int32_t* dst_page_table;  /* [num_seqs, max_pages] */
    int32_t max_pages, num_pages;
    const void* src_k_codes; const void* src_v_codes; const void* src_k_scale; const void* src_v_scale;
    const void* src_k_zp; const void* src_v_zp;
    void* dst_k_codes; void* dst_v_codes; void* dst_k_scale; void* dst_v_scale;
    void* dst_k_zp; void* dst_v_zp;
    const float* src_acc; const float* src_ts;   /* [segments, score_stride] or NULL */
    float* dst_acc; float* dst_ts;               /* [segments, dst_score_stride] or NULL: the kept positions' values,
                                                    at 0 .. kept - 1 of every row                                */
    int32_t score_stride;
    int32_t dst_score_stride;                    /* 0: same as score_stride; otherwise at least keep_stride   */
    uint32_t* status;
} pikv_compact_params;

int pikv_h2o_compact(const pikv_compact_params* p, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Decode attention over the int8 paged cache, dequantised in registers.
 *
 * out[b,h,:] = softmax(q[b,h,:] . K[b,h/g]^T / sqrt(128)) V[b,h/g] with
 * K = code * scale (core/single/module/pikv_compression.py:1006), arithmetic
 * of PiKVAttention._compute_attention (core/single/pikv_attention.py:117-123,
 * 163,188).  g = n_q / n_kv query heads share one KV head.  The pages of all
 * (stream, KV head) units form one list that a persistent grid cuts into equal
 * ranges, one per warp, whatever the streams' lengths; a warp leaves one partial
 * result per unit it touched in `workspace` and a second kernel merges them.
 *   q, out: [B, n_q, 128] bf16.  seq_ids [B] (NULL: b) selects the page-table
 *   row, seq_len [B] its valid length.  B <= 12000 per call.
 *   lse (optional) [B, n_q] fp32 log-sum-exp of the scaled scores.
 *   scores (optional) [B, n_q, score_stride] fp32 raw scaled scores, consumed by
 *   pikv_h2o_accumulate_attn.
 *   splits: ignored (the kernel balances the pages over the GPU by itself); kept
 *   so that existing callers compile.
 *   workspace: pikv_decode_attn_workspace_bytes(B, n_q, n_kv, ., .) bytes, 16-byte aligned.
 * ---------------------------------------------------------------------- */
typedef struct {
    const void* q; void* out;
    int32_t B, n_q, n_kv;
    const int32_t* seq_ids; const int32_t* seq_len;
    const int32_t* page_table; int32_t num_seqs, max_pages, num_pages;
    const void* k_codes; const void* v_codes; const void* k_scale; const void* v_scale;
    int32_t splits;            /* ignored                                        */
    float* lse;
    float* scores; int32_t score_stride;
    void* workspace; size_t workspace_bytes;
    uint32_t* status;
    const void* k_zp; const void* v_zp;   /* fp32 zero points, 4-bit asymmetric cache only */
    /* compact score output for the H2O update (optional; needs lse): f16 exp2(score_log2 - maximum of the softmax
     * step) [B, n_q, probs_stride] and that maximum for every 16-position page [B, n_q, step_stride] (step_stride
     * >= ceil(context / 16)); half the bytes of `scores`, consumed by pikv_h2o_accumulate_probs */
    void* probs16; float* step_max; int32_t probs_stride, step_stride;
} pikv_decode_params;

size_t pikv_decode_attn_workspace_bytes(int32_t B, int32_t n_q, int32_t n_kv, int32_t max_ctx, int32_t splits);
int    pikv_decode_attn_default_splits(int32_t B, int32_t n_kv, int32_t max_ctx);
int    pikv_decode_attn_q8(const pikv_decode_params* p, pikv_stream_t stream);
/* The same over the 4-bit asymmetric cache (K = (code - zp) * scale, codes 0..15, two per byte):
 * half the code bytes per token; k_zp / v_zp are required. */
int    pikv_decode_attn_q4(const pikv_decode_params* p, pikv_stream_t stream);

/* Same computation for callers that cannot allocate device memory at the point where they need
 * attention (a server that gave all of HBM to its own pool at start-up, a plug-in inside an
 * allocator-free region, code inside a stream capture).  It has no counterpart in the reference.
 * The partial results go to an 8 MiB array built into the library (held by every GPU that loads it,
 * until exit) instead of `workspace`, which is ignored; the call makes no cudaMalloc / cudaFree and
 * calls no allocating routine.  The array is smaller than the workspace the regular entry point asks for, so the
 * kernel cuts the page list into fewer, longer blocks; one block per worker of a KV head must still fit
 * (64 streams x 32 query / 8 KV heads need 4.8 MB of the pikv_decode_attn_static_scratch_bytes() = 8 MiB),
 * otherwise the call is refused with PIKV_ELIMIT before anything is launched.  The first call on each device looks the array's address up
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls on a device
 * share the array: it needs no clearing (every partial a launch reads was written by that launch),
 * but two calls whose kernels overlap on the GPU (different streams) race on it. */
size_t pikv_decode_attn_static_scratch_bytes(void);
int    pikv_decode_attn_q8_static(const pikv_decode_params* p, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Decode step over the striped expert-sharded cache (pikv_kv_append_striped).  Stream s lives on its home
 * rank s / streams_per_rank, which holds its query, its top-k experts and weights and the lengths of its
 * pairs.  One step, the same three calls in the same order on every rank (all on one stream per rank):
 *   pikv_shard_decode_post     home: routing records {expert, pair length, weight} of its streams to every
 *                              rank, query rows to the ranks that own a stripe of a selected pair
 *   pikv_shard_decode_attn     owner: waits for every rank's post, builds the local request list (request
 *                              i = stream i / k, choice i % k; seq_ids / seq_len / q_rows are caller-given
 *                              scratch of num_streams * top_k ints each), runs the decode-attention kernel
 *                              over the rows it holds and stores each request's normalised partial output
 *                              and log-sum-exp into the home rank's buffers
 *   pikv_shard_decode_combine  home: waits for every rank's partials; per (stream, choice) merges the ranks'
 *                              partials by log-sum-exp, then mode 0: out = sum_j w_j * attention_j, the
 *                              combine of DistributedPiKVMoE.forward (expert output times routing weight,
 *                              summed over experts and ranks, core/distributed/distributed_pikv.py:174-194);
 *                              mode 1: one softmax over the union of the k caches.
 * Everything crosses NVLink as plain stores into peer-mapped buffers followed by flag words (no collective
 * library call, no multicast); every wait is bounded by wait_limit_us and raises PIKV_ST_WAIT_TIMEOUT.
 * Buffers per rank (pikv_shard_decode_buffer_bytes(what, ...): 0 q, 1 route, 2 post flags, 3 partial outputs,
 * 4 partial log-sum-exps, 5 done flags), zeroed at start, mapped on every rank; seq (1 word) and counters
 * (2 words) are local device words, zeroed at start.  `cache` of pikv_shard_decode_attn carries the local
 * page pools, the replicated page table, n_q / n_kv and the workspace (sized for B = num_streams * top_k).
 * ---------------------------------------------------------------------- */
typedef struct {
    int32_t world, rank, num_experts, num_streams, top_k, n_q, stripe, streams_per_rank;
    const int32_t* expert_rot;
    void*     peer_q[8];
    void*     peer_route[8];
    uint32_t* peer_post_flags[8];
    float*    peer_part_o[8];
    float*    peer_part_lse[8];
    uint32_t* peer_done_flags[8];
    uint32_t* seq;
    uint32_t* counters;
    uint32_t* status;
    int32_t   wait_limit_us;
} pikv_shard_decode_ctx;

size_t pikv_shard_decode_buffer_bytes(int32_t what, int32_t world, int32_t num_streams, int32_t top_k, int32_t n_q);
int pikv_shard_decode_post(const pikv_shard_decode_ctx* c, const void* q_local, const int32_t* topk_idx,
                           const float* topk_w, const int32_t* pair_len, pikv_stream_t stream);
int pikv_shard_decode_attn(const pikv_shard_decode_ctx* c, const pikv_decode_params* cache, int32_t* seq_ids,
                           int32_t* seq_len, int32_t* q_rows, pikv_stream_t stream);
int pikv_shard_decode_combine(const pikv_shard_decode_ctx* c, const int32_t* topk_idx, const float* topk_w,
                              const int32_t* pair_len, void* out, float* lse_out, int32_t mode, pikv_stream_t stream);

/* acc[b, kvh, pos] += sum over the g query heads of exp(score - lse): the H2O
 * accumulated-attention increment (core/single/pikv_moe.py:241-245 column sums
 * fed to core/single/cache_scheduling.py:69-73).  acc: [B*n_kv, acc_stride]. */
int pikv_h2o_accumulate_attn(const float* scores, int32_t score_stride, const float* lse,
                             const int32_t* seq_len, int32_t B, int32_t n_q, int32_t n_kv,
                             float* acc, int32_t acc_stride, pikv_stream_t stream);
/* The same increment from the decode kernel's compact output (probs16 / step_max of pikv_decode_params):
 * acc[b, kvh, pos] += sum over the group's query heads of probs16 * 2^(step_max[pos / 16] - lse / ln 2). */
int pikv_h2o_accumulate_probs(const void* probs16, int32_t probs_stride, const float* step_max, int32_t step_stride,
                              const float* lse, const int32_t* seq_len, int32_t B, int32_t n_q, int32_t n_kv,
                              float* acc, int32_t acc_stride, pikv_stream_t stream);

/* ------------------------------------------------------------------------
 * Low-rank projection on tcgen05 tensor cores (bf16 operands, fp32 accumulate
 * in tensor memory): y[M,N] = act(x[M,K] . w[N,K]^T + bias).
 * Projection (N = rank, relu=1) and reconstruction (K = rank, relu=0) of
 * SVDCompressor.forward (core/single/pikv_compression.py:336-349), the
 * encoder/decoder layers of PyramidCompressor (:101-127) and the cache
 * compressor's two Linears (core/single/kv_cache_compression.py:38-39);
 * replaces launch_svd_compression_kernel / launch_pyramid_compression_kernel
 * (core/cuda/pikv_compression_kernel.cu:507-553).
 *   x, w bf16 row-major (K contiguous), K % 16 == 0, N % 16 == 0, N <= 256 per
 *   call column block (larger N is tiled internally); out bf16 or fp32.
 *   residual (optional) [M,N] bf16 added after the activation.
 * ---------------------------------------------------------------------- */
int pikv_lowrank_project(const void* x, const void* w, const float* bias, const void* residual,
                         void* out, int32_t out_dtype, int32_t M, int32_t N, int32_t K, int32_t relu,
                         pikv_stream_t stream);
/* Reads and clears the sticky device error word of the projection kernel (non-zero: a
 * bounded mbarrier wait ran out and the output is invalid).  Copies from the device, so
 * it waits for the work queued before it. */
int pikv_lowrank_error_state(void);

/* ------------------------------------------------------------------------
 * Expert-sharded exchange helpers (token all-to-all over NVLink via NCCL runs
 * in the host layer between these two calls).
 * pikv_a2a_pack quantises each routed (token, j) K/V row and writes a
 * fixed-size record into the send buffer, grouped by destination rank in
 * (token, j) order; pikv_a2a_unpack stores received records into the local
 * paged cache.  Replaces the replicate-everything + all_reduce design of
 * DistributedPiKVMoE.forward (core/distributed/distributed_pikv.py:174-194).
 * Record (int8 symmetric): header {int32 seq, int32 slot} + K codes
 * [n_kv*128] + V codes [n_kv*128] + K scales [n_kv] bf16 + V scales [n_kv] bf16.
 * ---------------------------------------------------------------------- */
size_t pikv_a2a_record_bytes(int32_t n_kv);
/* Record index of (token, j): send_pos[t,j] when send_pos is given, else seq_prefix[dst_seq] + slot
 * (records grouped by destination sequence, (token, j) order inside a sequence - with experts owned
 * in contiguous blocks that is also grouped by destination rank).  slot < 0 or send_pos < 0 skips. */
int pikv_a2a_pack(const void* k, const void* v, int32_t dtype, int32_t T, int32_t n_kv, int32_t top_k,
                  const int32_t* dst_seq, const int32_t* slot, const int32_t* seq_prefix,
                  const int32_t* send_pos, void* send_buf, pikv_stream_t stream);
/* Stores records into the local cache at sequence (header.seq - seq_offset) and position
 * header.slot + seg_base[segment, local sequence], where segment s covers records
 * [seg_start[s], seg_start[s+1]) (one segment per source rank; seg_start / seg_base may be NULL:
 * no offset).  Records whose final position is >= capacity (> 0) are dropped silently, like the
 * truncation of core/single/cache_scheduling.py:431-435. */
int pikv_a2a_unpack(const void* recv_buf, int32_t n_records, int32_t n_kv,
                    const int32_t* page_table, int32_t num_seqs, int32_t max_pages, int32_t num_pages,
                    int32_t seq_offset, int32_t capacity,
                    const int32_t* seg_start, const int32_t* seg_base, int32_t n_seg,
                    void* k_codes, void* v_codes, void* k_scale, void* v_scale,
                    uint32_t* status, pikv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PIKV_B200_H */
