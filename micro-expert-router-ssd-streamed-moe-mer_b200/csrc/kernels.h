// Internal interface between the C-ABI layer (mer_abi.cu) and the kernel files.
// Not part of the public boundary; see include/mer_b200.h for that.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define MER_BLOCK_ELEMS 32
#define MER_Q4_BLOCK_BYTES 18
#define MER_Q8_BLOCK_BYTES 34
#define MER_NONE 0xFFFFFFFFu
#define MER_MAX_CTAS1 257  /* per-phase stride of MoeDispatch::item_bounds: up to 256 CTAs + 1 */

// Router parameters resident on the device (one per installed layer).
struct RouterDev {
  const float *w;                // [E x D]
  const float *correction_bias;  // [E] or null
  const float *logit_bias;       // [E] or null
  uint32_t num_experts, top_k;
  int scoring, normalise;
  uint32_t n_group, topk_group;
  float scaling;
  uint32_t shared_expert_id;  // global id or MER_NONE
  uint32_t id_base;           // layer * num_experts
  const float *shared_scale;  // [n_tokens] mixing weight of the shared expert (its sigmoid gate scalar), or null = 1
};

#define MER_EP_MAX_WORLD 16

// One MoE dispatch: P = n_tokens * slots pairs (token, slot); pair p belongs to token p / slots.
// Pairs are grouped by expert: group g covers perm[offsets[g] .. offsets[g+1]) and runs expert
// group_expert[g].
struct MoeDispatch {
  const uint8_t *const *expert_ptr;  // global id -> payload in the HBM slot arena, null = not resident
  uint32_t max_experts;
  int dtype;
  uint32_t D, F;
  uint32_t n_tokens, slots, n_groups;
  const float *x;           // [n_tokens x D]
  uint32_t *pair_expert;    // [P] global id or MER_NONE
  float *pair_weight;       // [P]
  uint32_t *group_expert;   // [n_groups]
  uint32_t *offsets;        // [n_groups + 1]
  uint32_t *perm;           // [P]
  uint32_t *group_count;    // [n_groups] zero between dispatches: per-group pair counts of the grid-wide grouping,
  uint32_t *group_cursor;   //   and its scatter cursors (both null: always group in one CTA)
  float *h;                 // [P x F]   silu(gate) * up
  float *y;                 // [P x D]   per-pair expert outputs
  float *out;               // [n_tokens x D]
  uint32_t *status;         // device status word (MER_DEVSTAT_* bits)
  uint32_t *counters;       // scratch counters: [0..n_tokens) per-token arrivals, [max_tokens] global arrivals
  float *logits;            // [n_tokens x E] scratch
  float swiglu_limit;       // <= 0 = off
  uint32_t scratch_pairs;   // pair capacity the streaming scratch was sized for
  uint32_t max_group_tokens;  // upper bound on the pairs of any one group in this dispatch
  uint32_t active_groups_hint;  // expected number of non-empty groups (shapes the work split)
  uint32_t expected_pairs;      // expected number of pairs that reach a group (0 = all of them; fewer under expert parallelism)
  // token passes of the streaming FFN (null when the generic kernels run): groups cut into runs of at most
  // tokens_per_pass pairs, built by the grouping kernels; amax = per-pair max |h| cell, zeroed there too
  uint32_t *pass_group, *pass_start, *pass_count, *n_passes, *amax;
  uint32_t tokens_per_pass;
  // Work split of the streaming kernels, built with the passes: item_bounds[phase * MER_MAX_CTAS1 + b] = first item of
  // CTA b in that phase (b = 0 .. n_ctas), items weighted by the tokens of their pass (null: the GEMM path).
  uint32_t *item_bounds;
  uint32_t items_per_pass[2];  // items per pass in the gate/up and the down phase (K splits x tile groups)
  uint32_t n_ctas;
  const float *y_parts;     // set by the streaming FFN: K-split partials [y_nparts][P x D] of the per-pair outputs,
  uint32_t y_nparts;        //   or null / 1 when `y` already holds them
  int fuse_combine;         // in: a weighted combine into `out` follows the expert FFN; the FFN launch may do it itself
  int combined;             // out: it did (launch_combine then does nothing)
  int fuse_reduce;          // in: the caller wants final per-pair outputs in `y` for the grouped pairs (no K-split partials left)
  uint32_t gemm_bn;         // > 0: the tcgen05 GEMM path runs this dispatch with passes of gemm_bn tokens
  int packed;               // 1: slots hold the tile-major fragment layout (layout.cuh), 0: the flat block stream
  // Residual stream: when set, the combine writes out = (residual + sum over the routed slots) + shared-expert slot,
  // in that order (add_residual after the routed sum, then the shared expert: model.rs:2742-2763).
  const float *residual;    // [n_tokens x D] or null
  uint32_t routed_slots;    // slots below this index are routed experts (used with `residual`)
  // Expert-parallel push (push_tokens_per_rank > 0): tokens are numbered over all ranks, rank j brought tokens
  // [j * tpr, (j + 1) * tpr), and the output of pair (token, slot) belongs in the per-pair output region of the token's
  // home rank, row (token % tpr) * slots + slot.  The GEMM kernels' down epilogue stores there directly (peer stores
  // over NVLink while the tile's successors are still being multiplied); other kernel families write `y` and a copy
  // kernel moves the rows.
  uint8_t *push_y[MER_EP_MAX_WORLD];
  uint32_t push_tokens_per_rank;
};

// Where the down projection's output row of pair p goes.
__device__ __forceinline__ float *pair_output_row(const MoeDispatch &d, float *y, uint32_t pair) {
  if (d.push_tokens_per_rank == 0) return y + (size_t)pair * d.D;
  const uint32_t tok = pair / d.slots, sl = pair - tok * d.slots;
  const uint32_t home = tok / d.push_tokens_per_rank, t = tok - home * d.push_tokens_per_rank;
  return reinterpret_cast<float *>(d.push_y[home]) + ((size_t)t * d.slots + sl) * d.D;
}

// Expert-parallel view of one rank: where every rank's exchange buffer is mapped and how experts
// and tokens are partitioned.  Offsets are the same on every rank.
struct EpDev {
  uint8_t *peer[MER_EP_MAX_WORLD];  // exchange buffer of rank j as mapped here (own buffer at [rank])
  uint32_t rank, world;
  uint32_t experts_per_rank;  // rank j owns the local expert indices [j*epr, (j+1)*epr) of every layer ...
  const uint16_t *owner;      // ... unless a placement table is installed: owner[global expert id] (same on every rank)
  uint32_t top_k;             // slots >= top_k are the shared expert (runs on the token's own rank)
  uint32_t id_base;           // layer * experts_per_layer of the layer in flight
  uint32_t tokens_per_rank;   // tokens every rank contributes to the step in flight
  size_t off_flags, off_x, off_ids, off_y;  // byte offsets inside an exchange buffer
  uint64_t wait_ns;           // limit of every wait on a peer
};

// kernels_ep.cu
cudaError_t launch_ep_filter(const EpDev &ep, const uint32_t *ids_all, const float *w_all, uint32_t n_pairs, uint32_t slots,
                             uint32_t *pair_expert, float *pair_weight, cudaStream_t s, int *launches);
// `epoch_counter`: device word, advanced by one by the signal kernel each of these launches starts with.
// `group_count` non-null: the kernel also counts the local pairs per group (n_routed = routed experts of the layer), which
// is the grouping kernels' first step (launch_groups_layer with `counted`).
cudaError_t launch_ep_gather(const EpDev &ep, uint32_t *epoch_counter, uint32_t D, uint32_t slots, float *x_all, uint32_t *pair_expert,
                             float *pair_weight, uint32_t *status, uint32_t *group_count, uint32_t n_routed, cudaStream_t s,
                             int *launches);
cudaError_t launch_ep_combine(const EpDev &ep, uint32_t *epoch_counter, uint32_t D, uint32_t slots, const uint32_t *ids, const float *w,
                              const float *residual, float *out, uint32_t *status, cudaStream_t s, int *launches);
// Copies the per-pair output rows of the grouped (= local) pairs from d.y to their tokens' home ranks (d.push_*).
cudaError_t launch_ep_push_rows(const MoeDispatch &d, cudaStream_t s, int *launches);

// NCCL all-to-all mode: pack every pair into the send segment of its expert's owner (segment d = rows [d * seg_rows, ...),
// cursors[d] counts its rows, pos[p] = row the pair went to); combine from the rows that came back.
cudaError_t launch_a2a_pack(const EpDev &ep, uint32_t D, uint32_t slots, uint32_t n_pairs, uint32_t seg_rows, const float *x,
                            const uint32_t *ids, uint32_t *cursors, float *send_x, uint32_t *send_meta, uint32_t *pos, cudaStream_t s,
                            int *launches);
cudaError_t launch_a2a_combine(uint32_t n_tokens, uint32_t D, uint32_t slots, uint32_t routed_slots, const uint32_t *pos, const float *w,
                               const float *ret_y, const float *residual, float *out, cudaStream_t s, int *launches);

// kernels_generic.cu
// Groups pairs by expert for a whole layer whose routing is already in d.pair_expert (+ pass table).
// `counted`: the pairs per group are already in d.group_count (only honoured when groups_layer_on_grid(d)).
bool groups_layer_on_grid(const MoeDispatch &d);
cudaError_t launch_groups_layer(const RouterDev &r, const MoeDispatch &d, cudaStream_t s, int *launches, bool counted = false);
// group = false: route only (the caller groups later, e.g. after gathering other ranks' tokens)
cudaError_t launch_router(const RouterDev &r, const MoeDispatch &d, uint32_t max_tokens, cudaStream_t s, int *launches,
                          bool group = true);
cudaError_t launch_groups_from_pairs(const MoeDispatch &d, cudaStream_t s, int *launches);
cudaError_t launch_ffn_generic(const MoeDispatch &d, cudaStream_t s, int *launches, cudaEvent_t ev_mid);
cudaError_t launch_combine(const MoeDispatch &d, cudaStream_t s, int *launches);
// Pre-MoE steps on n_tokens rows of x: RMSNorm (rms_weight != null: xn = x * rsqrt(mean(x^2) + eps) * weight) and the
// shared expert's gate scalar (shared_gate != null: scale[t] = sigmoid(shared_gate . xn[t])).
cudaError_t launch_pre_moe(const float *x, uint32_t n_tokens, uint32_t D, const float *rms_weight, float eps, const float *shared_gate,
                           float *xn, float *shared_scale, cudaStream_t s, int *launches);
cudaError_t launch_dequant(int dtype, const uint8_t *src, float *dst, size_t n_weights, cudaStream_t s);
// Dequantises projection `matrix` (0 gate, 1 up, 2 down) of a packed expert into row-major f32.
cudaError_t launch_dequant_packed(int dtype, const uint8_t *expert, int matrix, uint32_t D, uint32_t F, float *dst, cudaStream_t s);
// Flat gate||up||down block stream -> tile-major fragment layout (same bytes, permuted).
cudaError_t launch_repack(int dtype, const uint8_t *flat, uint8_t *packed, uint32_t D, uint32_t F, cudaStream_t s);
cudaError_t launch_raw_matvec(int dtype, const uint8_t *w, const float *x, float *y, size_t rows, size_t cols, cudaStream_t s);
cudaError_t launch_f16_to_f32(const uint16_t *src, float *dst, size_t n, cudaStream_t s);
cudaError_t launch_f32_to_f16(const float *src, uint16_t *dst, size_t n, cudaStream_t s);

// kernels_stream.cu: streaming tensor-core expert FFN for block-aligned shapes.
bool stream_ffn_supported(int dtype, uint32_t D, uint32_t F);
size_t stream_ffn_scratch_bytes(uint32_t max_pairs, uint32_t D, uint32_t F);
cudaError_t launch_ffn_stream(MoeDispatch &d, void *scratch, int sm_count, cudaStream_t s, int *launches, cudaEvent_t ev_mid);
// Points d.pass_* / d.amax into the scratch and picks tokens_per_pass for this dispatch (call before grouping).
void stream_bind(MoeDispatch &d, void *scratch, int sm_count);
cudaError_t launch_reduce_parts(const MoeDispatch &d, cudaStream_t s, int *launches);

// kernels_gemm.cu: tcgen05 / TMEM grouped GEMM for groups of a dozen tokens and more.
bool gemm_ffn_supported(int dtype, uint32_t D, uint32_t F);
size_t gemm_ffn_scratch_bytes(uint32_t max_tokens, uint32_t max_pairs, uint32_t D, uint32_t F);
// Tokens per pass (16..128) for this dispatch, or 0 when its groups are too small for the GEMM path.
uint32_t gemm_pick_bn(const MoeDispatch &d, uint32_t min_mean_tokens);
void gemm_bind(MoeDispatch &d, void *stream_scratch, int sm_count, uint32_t bn);
cudaError_t launch_ffn_gemm(MoeDispatch &d, void *gemm_scratch, size_t gemm_scratch_bytes, uint32_t max_tokens, int sm_count,
                            cudaStream_t s, int *launches, cudaEvent_t ev_mid);
