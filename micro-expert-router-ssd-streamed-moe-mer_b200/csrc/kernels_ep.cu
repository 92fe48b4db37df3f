// Expert-parallel kernels: one process per GPU, experts of every layer partitioned contiguously
// over the ranks.  Two ways to move tokens:
//   (1) the host runs the collectives (all-gather of x and routing, reduce-scatter of partial
//       outputs) and this file only filters the gathered routing down to the local experts;
//   (2) the ranks exchange through peer memory: every rank publishes its tokens and routing in an
//       exchange buffer the other ranks have mapped; a rank pulls the token rows it needs with plain
//       peer loads (no TMA, no multicast) after a flag barrier (a one-CTA signal kernel raises this
//       rank's flag on every peer, then all CTAs of the gather kernel wait for the flags of the ranks
//       they read).  Per-pair expert outputs travel the other way as plain peer stores: the owner of
//       the expert writes them into the exchange buffer of the token's home rank (the GEMM kernels'
//       down epilogue directly, k_ep_push_rows for the other kernel families), raises its flag, and
//       the combine kernel reads local memory once every rank's flag is up.
//   (3) NCCL all-to-all: every (token, slot) pair is packed into the send segment of the rank that owns its expert
//       (k_a2a_pack), the library exchanges the segments with grouped ncclSend / ncclRecv, the owners run their
//       experts over the rows they received and send the outputs back the same way; k_a2a_combine sums each
//       token's pairs in slot order from the returned rows.
// Every wait on a peer is bounded by wall-clock time; on expiry the kernel latches
// MER_DEVSTAT_TIMEOUT and carries on without the peer's data (the host then fails the call).
#include "../../include/mer_b200.h"
#include "kernels.h"

namespace {

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t ld_flag(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until flag >= epoch (epochs grow monotonically; compared as signed distance so that a
// wrap after 2^31 steps is harmless).  Returns false when the time limit ran out.
__device__ bool wait_flag(const uint32_t *flag, uint32_t epoch, uint64_t limit_ns) {
  if ((int32_t)(ld_flag(flag) - epoch) >= 0) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 64; i++) {
      if ((int32_t)(ld_flag(flag) - epoch) >= 0) return true;
      __nanosleep(200);
    }
    if (global_ns() - t0 > limit_ns) return false;
  }
}

// Rank that holds routed expert e of the layer in flight.
__device__ __forceinline__ uint32_t expert_owner(const EpDev &ep, uint32_t e) {
  return ep.owner ? (uint32_t)__ldg(ep.owner + e) : (e - ep.id_base) / ep.experts_per_rank;
}
__device__ __forceinline__ bool pair_is_local(const EpDev &ep, uint32_t e, uint32_t slot, uint32_t src_rank) {
  if (e == MER_NONE) return false;
  if (slot >= ep.top_k) return src_rank == ep.rank;  // shared expert: replicated, runs where the token lives
  return expert_owner(ep, e) == ep.rank;
}

// (1) Routing gathered by the host: keep the pairs whose expert lives here, blank the rest.
__global__ void k_ep_filter(EpDev ep, const uint32_t *__restrict__ ids_all, const float *__restrict__ w_all, uint32_t n_pairs,
                            uint32_t slots, uint32_t *__restrict__ pair_expert, float *__restrict__ pair_weight) {
  const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  const uint32_t token = p / slots, slot = p % slots;
  const uint32_t e = ids_all[p];
  const bool local = pair_is_local(ep, e, slot, token / ep.tokens_per_rank);
  pair_expert[p] = local ? e : MER_NONE;
  pair_weight[p] = local ? w_all[p] : 0.0f;
}

// (2a) Tells every peer that this rank's exchange buffer holds the data of the next epoch.  A kernel of its own, launched
// after the kernels that wrote the data (stream order: the data is in this GPU's memory by then) and before the kernel
// whose CTAs wait for the peers' flags, so that no waiting CTA can ever stand in the way of the signal.  The epoch
// counter lives in device memory (one step per signal), which lets the whole layer be replayed as a CUDA graph.
__global__ void k_ep_signal(EpDev ep, uint32_t *epoch_counter) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = *epoch_counter = *epoch_counter + 1;
  __syncthreads();
  const uint32_t j = threadIdx.x;
  if (j >= ep.world) return;
  __threadfence_system();
  uint32_t *flag = reinterpret_cast<uint32_t *>(ep.peer[j] + ep.off_flags) + ep.rank;
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(flag), "r"(s_epoch) : "memory");
}

// (2b) Pulls the tokens of every rank that hit a local expert: routing (filtered) for all tokens,
// x rows only for tokens with at least one local pair.  One CTA per (source rank, token).
__global__ void __launch_bounds__(256) k_ep_gather(EpDev ep, const uint32_t *__restrict__ epoch_counter, uint32_t D, uint32_t slots,
                                                   float *__restrict__ x_all, uint32_t *__restrict__ pair_expert,
                                                   float *__restrict__ pair_weight, uint32_t *status, uint32_t *group_count,
                                                   uint32_t n_routed) {
  const uint32_t src = blockIdx.y, t = blockIdx.x;
  __shared__ int s_ok, s_any;
  const uint32_t epoch = __ldcg(epoch_counter);  // set by the signal kernel in front of this one
  if (threadIdx.x == 0) {
    const uint32_t *flags = reinterpret_cast<const uint32_t *>(ep.peer[ep.rank] + ep.off_flags);
    s_ok = wait_flag(flags + src, epoch, ep.wait_ns);
    if (!s_ok) atomicOr(status, MER_DEVSTAT_TIMEOUT);
    __threadfence_system();  // the peer's data is read only after its flag was seen
    s_any = 0;
  }
  __syncthreads();
  const uint32_t tg = src * ep.tokens_per_rank + t;  // global token index
  if (!s_ok) {
    if (threadIdx.x < slots) pair_expert[tg * slots + threadIdx.x] = MER_NONE, pair_weight[tg * slots + threadIdx.x] = 0.0f;
    return;
  }
  const uint8_t *base = ep.peer[src];
  if (threadIdx.x < slots) {
    const uint32_t e = __ldcg(reinterpret_cast<const uint32_t *>(base + ep.off_ids) + t * slots + threadIdx.x);
    const bool local = pair_is_local(ep, e, threadIdx.x, src);
    pair_expert[tg * slots + threadIdx.x] = local ? e : MER_NONE;
    pair_weight[tg * slots + threadIdx.x] = local ? 1.0f : 0.0f;
    if (local) {
      s_any = 1;
      // the grouping kernels' count step, done here: group = local expert index, or the shared-expert group
      if (group_count) atomicAdd(group_count + (threadIdx.x >= ep.top_k ? n_routed : e - ep.id_base), 1u);
    }
  }
  __syncthreads();
  if (!s_any) return;
  const float4 *srcx = reinterpret_cast<const float4 *>(base + ep.off_x) + (size_t)t * (D / 4);
  float4 *dst = reinterpret_cast<float4 *>(x_all) + (size_t)tg * (D / 4);
  for (uint32_t i = threadIdx.x; i < D / 4; i += blockDim.x) dst[i] = __ldcg(srcx + i);
}

// (2c) out[t] = sum over slots, in slot order, of weight * y (same order and rounding as k_combine).  The rank that
// owns a pair's expert has pushed y into this rank's exchange buffer, row (token, slot); the kernel waits for every
// rank's flag (raised after its expert launches) and then reads local memory only.
// One CTA per token, a thread four consecutive values.
__global__ void __launch_bounds__(256) k_ep_combine(EpDev ep, const uint32_t *__restrict__ epoch_counter, uint32_t D, uint32_t slots,
                                                    const uint32_t *__restrict__ ids, const float *__restrict__ w,
                                                    const float *__restrict__ residual, float *__restrict__ out, uint32_t *status) {
  const uint32_t t = blockIdx.x;
  __shared__ int s_ok;
  __shared__ const float *s_row[64];
  __shared__ float s_w[64];
  const uint32_t epoch = __ldcg(epoch_counter);  // set by the signal kernel in front of this one
  if (threadIdx.x < 32) {
    // lanes share the ranks to wait for
    const uint32_t *flags = reinterpret_cast<const uint32_t *>(ep.peer[ep.rank] + ep.off_flags);
    int ok = 1;
    for (uint32_t j = threadIdx.x; j < ep.world; j += 32) ok &= (int)wait_flag(flags + j, epoch, ep.wait_ns);
    ok = __all_sync(0xffffffffu, ok);
    __threadfence_system();
    if (threadIdx.x == 0) {
      s_ok = ok;
      if (!ok) atomicOr(status, MER_DEVSTAT_TIMEOUT);
    }
  }
  // where each slot's row lives (null = skipped slot), resolved once per token: the owners of the experts pushed the
  // rows into this rank's own buffer
  if (threadIdx.x >= 32 && threadIdx.x < 32 + slots && threadIdx.x < 96) {
    const uint32_t sl = threadIdx.x - 32;
    const uint32_t e = ids[t * slots + sl];
    const float wt = w[t * slots + sl];
    const float *row = nullptr;
    if (e != MER_NONE && wt != 0.0f) row = reinterpret_cast<const float *>(ep.peer[ep.rank] + ep.off_y) + ((size_t)t * slots + sl) * D;
    s_row[sl] = row;
    s_w[sl] = wt;
  }
  __syncthreads();
  for (uint32_t i4 = threadIdx.x; i4 < D / 4; i4 += blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    if (s_ok) {
      // eight slots at a time: all their (mostly remote) loads are issued before the first one is consumed; the sum
      // itself stays in slot order
      for (uint32_t s0 = 0; s0 <= slots; s0 += 8) {
        float4 y[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float *row = s0 + j < slots ? s_row[s0 + j] : nullptr;
          y[j] = row ? __ldcg(reinterpret_cast<const float4 *>(row) + i4) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const uint32_t sl = s0 + j;
          if (sl > slots) break;
          if (residual && sl == min(ep.top_k, slots)) {  // hidden + routed sum, before the shared expert's slot
            const float4 r = __ldg(reinterpret_cast<const float4 *>(residual) + (size_t)t * (D / 4) + i4);
            acc.x = __fadd_rn(r.x, acc.x), acc.y = __fadd_rn(r.y, acc.y), acc.z = __fadd_rn(r.z, acc.z), acc.w = __fadd_rn(r.w, acc.w);
          }
          if (sl == slots || !s_row[sl]) continue;
          const float wt = s_w[sl];
          acc.x = __fadd_rn(acc.x, __fmul_rn(wt, y[j].x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(wt, y[j].y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(wt, y[j].z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(wt, y[j].w));
        }
      }
    }
    reinterpret_cast<float4 *>(out)[(size_t)t * (D / 4) + i4] = acc;
  }
}

// (2d) Kernel families that leave the per-pair outputs in the local array: one CTA per grouped pair copies its row to
// the token's home rank.
__global__ void __launch_bounds__(256) k_ep_push_rows(MoeDispatch d) {
  const uint32_t i = blockIdx.x;
  if (i >= d.offsets[d.n_groups]) return;
  const uint32_t pair = d.perm[i];
  const float4 *src = reinterpret_cast<const float4 *>(d.y + (size_t)pair * d.D);
  float4 *dst = reinterpret_cast<float4 *>(pair_output_row(d, nullptr, pair));
  for (uint32_t k = threadIdx.x; k < d.D / 4; k += blockDim.x) dst[k] = __ldcg(src + k);
}

// (3a) One warp per (token, slot) pair: claim the next row of the owner's send segment, copy the token's row and the
// expert id there, remember where the pair went.  Segment d starts at row d * seg_rows.  The order of the pairs
// inside a segment is whatever the atomics give; nothing depends on it.
__global__ void __launch_bounds__(256) k_a2a_pack(EpDev ep, uint32_t D, uint32_t slots, uint32_t n_pairs, uint32_t seg_rows,
                                                  const float *__restrict__ x, const uint32_t *__restrict__ ids,
                                                  uint32_t *__restrict__ cursors, float *__restrict__ send_x,
                                                  uint32_t *__restrict__ send_meta, uint32_t *__restrict__ pos) {
  const uint32_t p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (p >= n_pairs) return;
  const uint32_t token = p / slots, slot = p % slots;
  const uint32_t e = ids[p];
  if (e == MER_NONE) {
    if (lane == 0) pos[p] = MER_NONE;
    return;
  }
  const uint32_t dest = slot >= ep.top_k ? ep.rank : expert_owner(ep, e);  // the shared expert runs at home
  uint32_t row = 0;
  if (lane == 0) row = dest * seg_rows + atomicAdd(cursors + dest, 1u);
  row = __shfl_sync(0xffffffffu, row, 0);
  if (lane == 0) pos[p] = row, send_meta[row] = e;
  const float4 *src = reinterpret_cast<const float4 *>(x) + (size_t)token * (D / 4);
  float4 *dst = reinterpret_cast<float4 *>(send_x) + (size_t)row * (D / 4);
  for (uint32_t i = lane; i < D / 4; i += 32) dst[i] = __ldg(src + i);
}

// (3b) out[t] = sum over slots, in slot order, of weight * y, y of a pair = the row that came back for it
// (same order and rounding as k_combine).  One CTA per token.
__global__ void __launch_bounds__(256) k_a2a_combine(uint32_t D, uint32_t slots, uint32_t routed_slots, const uint32_t *__restrict__ pos,
                                                     const float *__restrict__ w, const float *__restrict__ ret_y,
                                                     const float *__restrict__ residual, float *__restrict__ out) {
  const uint32_t t = blockIdx.x;
  for (uint32_t i4 = threadIdx.x; i4 < D / 4; i4 += blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (uint32_t sl = 0; sl <= slots; sl++) {
      if (residual && sl == min(routed_slots, slots)) {  // hidden + routed sum, before the shared expert's slot
        const float4 r = __ldg(reinterpret_cast<const float4 *>(residual) + (size_t)t * (D / 4) + i4);
        acc.x = __fadd_rn(r.x, acc.x), acc.y = __fadd_rn(r.y, acc.y), acc.z = __fadd_rn(r.z, acc.z), acc.w = __fadd_rn(r.w, acc.w);
      }
      if (sl == slots) break;
      const uint32_t row = pos[t * slots + sl];
      const float wt = w[t * slots + sl];
      if (row == MER_NONE || wt == 0.0f) continue;
      const float4 y = __ldcg(reinterpret_cast<const float4 *>(ret_y) + (size_t)row * (D / 4) + i4);
      acc.x = __fadd_rn(acc.x, __fmul_rn(wt, y.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(wt, y.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(wt, y.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(wt, y.w));
    }
    reinterpret_cast<float4 *>(out)[(size_t)t * (D / 4) + i4] = acc;
  }
}

}  // namespace

cudaError_t launch_a2a_pack(const EpDev &ep, uint32_t D, uint32_t slots, uint32_t n_pairs, uint32_t seg_rows, const float *x,
                            const uint32_t *ids, uint32_t *cursors, float *send_x, uint32_t *send_meta, uint32_t *pos, cudaStream_t s,
                            int *launches) {
  k_a2a_pack<<<(n_pairs + 7) / 8, 256, 0, s>>>(ep, D, slots, n_pairs, seg_rows, x, ids, cursors, send_x, send_meta, pos);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_a2a_combine(uint32_t n_tokens, uint32_t D, uint32_t slots, uint32_t routed_slots, const uint32_t *pos, const float *w,
                               const float *ret_y, const float *residual, float *out, cudaStream_t s, int *launches) {
  k_a2a_combine<<<n_tokens, 256, 0, s>>>(D, slots, routed_slots, pos, w, ret_y, residual, out);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_ep_push_rows(const MoeDispatch &d, cudaStream_t s, int *launches) {
  k_ep_push_rows<<<d.n_tokens * d.slots, 256, 0, s>>>(d);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_ep_filter(const EpDev &ep, const uint32_t *ids_all, const float *w_all, uint32_t n_pairs, uint32_t slots,
                             uint32_t *pair_expert, float *pair_weight, cudaStream_t s, int *launches) {
  k_ep_filter<<<(n_pairs + 255) / 256, 256, 0, s>>>(ep, ids_all, w_all, n_pairs, slots, pair_expert, pair_weight);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_ep_gather(const EpDev &ep, uint32_t *epoch_counter, uint32_t D, uint32_t slots, float *x_all, uint32_t *pair_expert,
                             float *pair_weight, uint32_t *status, uint32_t *group_count, uint32_t n_routed, cudaStream_t s,
                             int *launches) {
  k_ep_signal<<<1, 32, 0, s>>>(ep, epoch_counter);  // this rank's tokens and routing are published
  dim3 grid(ep.tokens_per_rank, ep.world);
  k_ep_gather<<<grid, 256, 0, s>>>(ep, epoch_counter, D, slots, x_all, pair_expert, pair_weight, status, group_count, n_routed);
  if (launches) (*launches) += 2;
  return cudaGetLastError();
}

cudaError_t launch_ep_combine(const EpDev &ep, uint32_t *epoch_counter, uint32_t D, uint32_t slots, const uint32_t *ids, const float *w,
                              const float *residual, float *out, uint32_t *status, cudaStream_t s, int *launches) {
  k_ep_signal<<<1, 32, 0, s>>>(ep, epoch_counter);  // this rank's expert outputs are published
  k_ep_combine<<<ep.tokens_per_rank, 256, 0, s>>>(ep, epoch_counter, D, slots, ids, w, residual, out, status);
  if (launches) (*launches) += 2;
  return cudaGetLastError();
}
