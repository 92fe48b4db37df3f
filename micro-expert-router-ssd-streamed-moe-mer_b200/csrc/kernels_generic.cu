// Router, token->expert grouping, generic (any-shape) expert FFN, combine, dequant dump.
//
// The generic FFN kernels are the slow, shape-agnostic path: one warp per output row, one
// weight per lane per step, fp32 FMA.  They handle rows that straddle blocks (d_model or
// d_ff not a multiple of 32, e.g. the reference's 37x45 test shape) and are the on-device
// cross-check for the streaming kernels.
#include "kernels.h"

#include <cuda_fp16.h>
#include <math_constants.h>

#include <climits>

#include "../../include/mer_b200.h"
#include "layout.cuh"

namespace {

__device__ __forceinline__ float f16_bits_to_f32(uint16_t v) { return __half2float(__ushort_as_half(v)); }

// One dequantised weight of a flat block stream: d * (q - 8) (Q4_0) or d * q (Q8_0); the
// product is exact in fp32 (11-bit significand times a <= 8-bit integer).
template <int DT>
__device__ __forceinline__ float decode_weight(const uint8_t *__restrict__ base, size_t flat) {
  size_t blk = flat >> 5;
  uint32_t j = (uint32_t)flat & 31u;
  if (DT == MER_DTYPE_Q8_0) {
    const uint8_t *b = base + blk * MER_Q8_BLOCK_BYTES;
    float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(b));
    return __fmul_rn(d, (float)(int8_t)b[2 + j]);
  } else {
    const uint8_t *b = base + blk * MER_Q4_BLOCK_BYTES;
    float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(b));
    uint32_t byte = b[2 + (j & 15u)];
    int q = (int)(j < 16u ? (byte & 15u) : (byte >> 4)) - 8;
    return __fmul_rn(d, (float)q);
  }
}

// Weight (matrix, row, col) of a resident expert in either slot layout.
template <int DT>
__device__ __forceinline__ float weight_at(const MoeDispatch &d, const uint8_t *__restrict__ base, int matrix, uint32_t row,
                                           uint32_t col) {
  if (d.packed) {
    PackedAddr a = packed_locate<DT>(d.D, d.F, matrix, row, col);
    float sc = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(base + a.scale));
    uint32_t byte = base[a.quant];
    int q = DT == MER_DTYPE_Q8_0 ? (int)(int8_t)byte : (int)((col & 16u) ? (byte >> 4) : (byte & 15u)) - 8;
    return __fmul_rn(sc, (float)q);
  }
  const size_t bb = DT == MER_DTYPE_Q8_0 ? MER_Q8_BLOCK_BYTES : MER_Q4_BLOCK_BYTES;
  const size_t proj = ((size_t)d.D * d.F + 31) / 32 * bb;
  const uint32_t K = matrix < 2 ? d.D : d.F;
  return decode_weight<DT>(base + (size_t)matrix * proj, (size_t)row * K + col);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float clamp_gate(float g, float limit) {
  if (limit > 0.0f && isfinite(limit) && g == g) g = fminf(fmaxf(g, -limit), limit);  // NaN stays NaN
  return g;
}

// Order of f32::total_cmp as a signed integer key (gating.rs:283-294 compares with total_cmp).
__device__ __forceinline__ int total_key(float f) {
  int b = __float_as_int(f);
  return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}
__device__ __forceinline__ bool better(int ka, uint32_t ia, int kb, uint32_t ib) {
  return ka > kb || (ka == kb && ia < ib);
}

// ---------------------------------------------------------------------------------------
// Router.  One CTA computes the logits of 8 experts for a tile of 4 tokens (every warp takes an
// eighth of the columns of all 8 rows, so W is read once per token tile and each lane has many
// independent loads in flight).  The last CTA to finish a token tile scores, filters and picks
// top-k for its tokens, one warp per token (LinearGate::route_with_scratch, gating.rs:395-476);
// the last tile overall groups the (token, slot) pairs by expert.
// ---------------------------------------------------------------------------------------
constexpr int ROUTER_THREADS = 256;
constexpr int ROUTER_ROWS = ROUTER_THREADS / 32;  // expert rows per CTA
constexpr int ROUTER_TT = 4;                      // tokens per CTA
constexpr uint32_t SMALL_P = 4096;                // pair keys staged in shared memory below this many pairs
constexpr uint32_t STABLE_G = 512;
constexpr uint32_t GRID_GROUPING_PAIRS = 8192;    // from this many pairs the grouping runs grid-wide (count / scan / scatter)                // stable (token, slot)-ordered grouping up to this many groups

// Cuts every group into passes of at most d.tokens_per_pass pairs (the unit the streaming FFN works
// on) and clears the per-pair max cells.  One CTA of 256 threads; `off` = the group offsets.
__device__ void build_passes_block(const MoeDispatch &d, const uint32_t *off) {
  __shared__ uint32_t s_pcnt[257];
  __shared__ uint8_t s_cost[1024];  // cost of each of the first 1024 passes (the weighted work split below)
  const uint32_t tpp = d.tokens_per_pass, P = d.n_tokens * d.slots;
  const uint32_t tpp_shift = 31 - __clz(tpp);  // tokens per pass is a power of two (4 or 8; 16 .. 128 for the GEMM kernels)
#pragma unroll 1
  for (uint32_t i = threadIdx.x; i < P; i += 256) d.amax[i] = 0;
  const uint32_t per = (d.n_groups + 255) / 256;
  const uint32_t g0 = threadIdx.x * per, g1 = min(g0 + per, d.n_groups);
  uint32_t mine = 0;
#pragma unroll 1
  for (uint32_t g = g0; g < g1; g++) mine += (off[g + 1] - off[g] + tpp - 1) >> tpp_shift;
  s_pcnt[threadIdx.x + 1] = mine;
  if (threadIdx.x == 0) s_pcnt[0] = 0;
  __syncthreads();
  if (threadIdx.x < 32) {  // inclusive scan of 256 counts by one warp, 8 per lane
    uint32_t v[8], run = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) run += s_pcnt[1 + threadIdx.x * 8 + i], v[i] = run;
    uint32_t incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (threadIdx.x >= (uint32_t)o) incl += up;
    }
    const uint32_t base = incl - run;
#pragma unroll
    for (int i = 0; i < 8; i++) s_pcnt[1 + threadIdx.x * 8 + i] = base + v[i];
  }
  __syncthreads();
  uint32_t np = s_pcnt[threadIdx.x];
#pragma unroll 1
  for (uint32_t g = g0; g < g1; g++) {
    const uint32_t beg = off[g], end = off[g + 1];
#pragma unroll 1
    for (uint32_t st = beg; st < end; st += tpp) {
      const uint32_t cnt = min(tpp, end - st);
      d.pass_group[np] = g;
      d.pass_start[np] = st;
      d.pass_count[np] = cnt;
      if (np < 1024) s_cost[np] = cnt > 4 ? 13 : 10;
      np++;
    }
  }
  if (threadIdx.x == 0) {
    d.n_passes[0] = s_pcnt[256];
    d.n_passes[1] = d.n_passes[2] = 0;  // arrival counters of the streaming kernels' grid-wide barriers
  }
  if (!d.item_bounds) return;
  // ---- work split of the streaming kernels: one contiguous item range per CTA and phase.  An item of a pass with
  // more than four tokens multiplies two token tiles instead of one, which measures as ~1.3x the time: cost 13 vs 10.
  __shared__ uint32_t s_cum[1025];
  const uint32_t n_passes = s_pcnt[256], G = d.n_ctas;
  __syncthreads();  // s_cost[] written above is read back below
  const bool weighted = n_passes <= 1024 && tpp == 8;
  if (weighted) {
    // inclusive scan of the pass costs: 4 per thread, then the same warp scan as above over the 256 partial sums
    uint32_t c[4], run = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t q = threadIdx.x * 4 + i;
      c[i] = q < n_passes ? (uint32_t)s_cost[q] : 0u;
      run += c[i];
    }
    s_pcnt[threadIdx.x + 1] = run;
    __syncthreads();
    if (threadIdx.x < 32) {
      uint32_t v[8], r2 = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) r2 += s_pcnt[1 + threadIdx.x * 8 + i], v[i] = r2;
      uint32_t incl = r2;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (threadIdx.x >= (uint32_t)o) incl += up;
      }
      const uint32_t base = incl - r2;
#pragma unroll
      for (int i = 0; i < 8; i++) s_pcnt[1 + threadIdx.x * 8 + i] = base + v[i];
    }
    __syncthreads();
    uint32_t acc = s_pcnt[threadIdx.x];  // cost of all passes before this thread's four
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t q = threadIdx.x * 4 + i;
      if (q <= 1024) s_cum[q] = acc;
      acc += c[i];
    }
    if (threadIdx.x == 255) s_cum[1024] = acc;
    __syncthreads();
  }
#pragma unroll 1
  for (uint32_t i = threadIdx.x; i < 2 * (G + 1); i += 256) {
    const uint32_t phase = i / (G + 1), b = i % (G + 1);
    const uint32_t ipp = d.items_per_pass[phase];
    const uint64_t n_items = (uint64_t)n_passes * ipp;
    uint32_t bound;
    if (!weighted) {
      bound = (uint32_t)(n_items * b / G);
    } else if ((uint64_t)s_cum[n_passes] * ipp * G <= 0xFFFFFFFFull) {
      // the usual case: everything fits 32 bits (64-bit divisions cost a few hundred cycles each, and this loop sits
      // on the critical path of every decode layer)
      const uint32_t total = s_cum[n_passes] * ipp, target = total * b / G;
      uint32_t lo = 0, hi = n_passes;  // largest pass index with cum[pass] * ipp <= target
#pragma unroll 1
      while (lo < hi) {
        const uint32_t mid = (lo + hi + 1) >> 1;
        if (s_cum[mid] * ipp <= target) lo = mid; else hi = mid - 1;
      }
      if (lo >= n_passes) {
        bound = (uint32_t)n_items;
      } else {
        const uint32_t w = s_cum[lo + 1] - s_cum[lo];
        const uint32_t rem = target - s_cum[lo] * ipp;
        bound = lo * ipp + min(ipp, (rem + w - 1) / w);
      }
    } else {
      const uint64_t total = (uint64_t)s_cum[n_passes] * ipp, target = total * b / G;
      uint32_t lo = 0, hi = n_passes;
#pragma unroll 1
      while (lo < hi) {
        const uint32_t mid = (lo + hi + 1) >> 1;
        if ((uint64_t)s_cum[mid] * ipp <= target) lo = mid; else hi = mid - 1;
      }
      if (lo >= n_passes) {
        bound = (uint32_t)n_items;
      } else {
        const uint32_t w = s_cum[lo + 1] - s_cum[lo];
        const uint64_t rem = target - (uint64_t)s_cum[lo] * ipp;
        bound = lo * ipp + (uint32_t)min((uint64_t)ipp, (rem + w - 1) / w);
      }
    }
    d.item_bounds[phase * MER_MAX_CTAS1 + b] = bound;
  }
}

// Group of pair p: local expert index, the shared-expert group, or MER_NONE for an unfilled / foreign slot.
__device__ __forceinline__ uint32_t pair_group_key(const RouterDev &r, const MoeDispatch &d, uint32_t p) {
  const uint32_t e = __ldcg(d.pair_expert + p);
  if (e == MER_NONE) return MER_NONE;
  if ((p % d.slots) >= r.top_k || e == r.shared_expert_id) return r.num_experts;  // shared-expert slot (or a dispatched row of it)
  return e - r.id_base;
}

// Grouping of a large dispatch in three grid-wide steps (count, scan, scatter) instead of one CTA.  The order of
// the pairs inside a group is whatever the atomics give; every pair's result is independent of its position.
__global__ void __launch_bounds__(256) k_group_count(RouterDev r, MoeDispatch d) {
  const uint32_t P = d.n_tokens * d.slots;
  for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < P; p += gridDim.x * blockDim.x) {
    const uint32_t k = pair_group_key(r, d, p);
    if (k != MER_NONE) atomicAdd(d.group_count + k, 1u);
  }
}
__global__ void __launch_bounds__(256) k_group_scan(RouterDev r, MoeDispatch d) {
  const uint32_t G = d.n_groups;
  for (uint32_t g = threadIdx.x; g < G; g += blockDim.x) d.group_expert[g] = (g < r.num_experts) ? r.id_base + g : r.shared_expert_id;
  // the counts go through shared memory in slabs: one thread adds them up, everybody loads and stores
  __shared__ uint32_t s_cnt[1024];
  __shared__ uint32_t s_run;
  if (threadIdx.x == 0) s_run = 0;
  for (uint32_t g0 = 0; g0 < G; g0 += 1024) {
    const uint32_t n = min(1024u, G - g0);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
      s_cnt[i] = d.group_count[g0 + i];
      d.group_count[g0 + i] = 0;  // zero again for the next dispatch's count
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t acc = s_run;
      for (uint32_t i = 0; i < n; i++) {
        const uint32_t c = s_cnt[i];
        s_cnt[i] = acc;
        acc += c;
      }
      s_run = acc;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) d.offsets[g0 + i] = s_cnt[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) d.offsets[G] = s_run;
  __threadfence_block();
  __syncthreads();
  if (d.pass_group) build_passes_block(d, d.offsets);
}
__global__ void __launch_bounds__(256) k_group_scatter(RouterDev r, MoeDispatch d) {
  const uint32_t P = d.n_tokens * d.slots;
  for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < P; p += gridDim.x * blockDim.x) {
    const uint32_t k = pair_group_key(r, d, p);
    if (k != MER_NONE) d.perm[d.offsets[k] + atomicAdd(d.group_cursor + k, 1u)] = p;
  }
}
// Clears the scatter cursors after use, so that group_count / group_cursor are zero between dispatches.
__global__ void k_group_clear(MoeDispatch d) {
  for (uint32_t g = threadIdx.x; g < d.n_groups; g += blockDim.x) d.group_cursor[g] = 0;
}

// Runs in one CTA after every token has been routed: groups pairs by expert.
__device__ void build_groups_layer(const RouterDev &r, const MoeDispatch &d, uint32_t *s_u32) {
  const uint32_t P = d.n_tokens * d.slots;
  const uint32_t G = d.n_groups;
  const uint32_t tid = threadIdx.x, nt = blockDim.x, warp = tid >> 5, lane = tid & 31;
  uint32_t *s_off = s_u32;                    // [G + 1]
  uint32_t *s_cnt = s_u32 + G + 1;            // [8 warps][G] (stable path) or [G]
  const bool stable = G <= STABLE_G;
  uint32_t *s_key = s_cnt + (stable ? ROUTER_ROWS * G : G);  // [min(P, SMALL_P)]
  const bool staged = P <= SMALL_P;
  auto key_global = [&](uint32_t p) -> uint32_t {
    uint32_t e = __ldcg(d.pair_expert + p);
    if (e == MER_NONE) return MER_NONE;
    if ((p % d.slots) >= r.top_k || e == r.shared_expert_id) return r.num_experts;  // shared-expert slot (or a dispatched row of it)
    return e - r.id_base;
  };
  auto key_of = [&](uint32_t p) -> uint32_t { return staged ? s_key[p] : key_global(p); };
#pragma unroll 1
  for (uint32_t g = tid; g < G; g += nt) d.group_expert[g] = (g < r.num_experts) ? r.id_base + g : r.shared_expert_id;
#pragma unroll 1
  for (uint32_t i = tid; i < (stable ? ROUTER_ROWS * G : G); i += nt) s_cnt[i] = 0;
  if (staged)
#pragma unroll 1
    for (uint32_t p = tid; p < P; p += nt) s_key[p] = key_global(p);
  __syncthreads();
  if (stable) {
    // every warp owns a contiguous run of pairs, so (warp, position in run) order = (token, slot) order
    const uint32_t chunk = ((P + ROUTER_ROWS - 1) / ROUTER_ROWS + 31) / 32 * 32;
    const uint32_t p0 = warp * chunk, p1 = min(P, p0 + chunk);
#pragma unroll 1
    for (uint32_t p = p0 + lane; p < p1; p += 32) {
      uint32_t k = key_of(p);
      if (k != MER_NONE) atomicAdd(&s_cnt[warp * G + k], 1u);
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t g = tid; g < G; g += nt) {  // per group: exclusive scan over the warps, total into s_off
      uint32_t run = 0;
#pragma unroll 1
      for (uint32_t w = 0; w < ROUTER_ROWS; w++) {
        uint32_t c = s_cnt[w * G + g];
        s_cnt[w * G + g] = run;
        run += c;
      }
      s_off[g] = run;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the group totals
      const uint32_t per = (G + 31) / 32;
      uint32_t run = 0;
#pragma unroll 1
      for (uint32_t i = 0; i < per; i++) {
        uint32_t g = lane * per + i;
        if (g < G) run += s_off[g];
      }
      uint32_t incl = run;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= (uint32_t)o) incl += up;
      }
      uint32_t base = incl - run;
#pragma unroll 1
      for (uint32_t i = 0; i < per; i++) {
        uint32_t g = lane * per + i;
        if (g < G) {
          uint32_t c = s_off[g];
          s_off[g] = base;
          base += c;
        }
      }
      if (lane == 31) s_off[G] = incl;
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t pb = p0; pb < p1; pb += 32) {
      const uint32_t p = pb + lane;
      const uint32_t k = p < p1 ? key_of(p) : MER_NONE;
      const uint32_t same = __match_any_sync(0xffffffffu, k);
      if (k != MER_NONE) {
        const uint32_t rank = __popc(same & ((1u << lane) - 1));
        d.perm[s_off[k] + s_cnt[warp * G + k] + rank] = p;
      }
      __syncwarp();
      if (k != MER_NONE && (same & ((1u << lane) - 1)) == 0) s_cnt[warp * G + k] += __popc(same);
      __syncwarp();
    }
  } else {
#pragma unroll 1
    for (uint32_t p = tid; p < P; p += nt) {
      uint32_t k = key_of(p);
      if (k != MER_NONE) atomicAdd(&s_cnt[k], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t acc = 0;
#pragma unroll 1
      for (uint32_t g = 0; g < G; g++) {
        s_off[g] = acc;
        acc += s_cnt[g];
        s_cnt[g] = 0;
      }
      s_off[G] = acc;
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t p = tid; p < P; p += nt) {
      uint32_t k = key_of(p);
      if (k != MER_NONE) d.perm[s_off[k] + atomicAdd(&s_cnt[k], 1u)] = p;
    }
  }
  __syncthreads();
#pragma unroll 1
  for (uint32_t g = tid; g <= G; g += nt) d.offsets[g] = s_off[g];
  if (d.pass_group) build_passes_block(d, s_off);
}

// Scoring, group filter, top-k and mixing weights of one token by one warp.
// s_score / s_sel / s_ok are this warp's shared arrays of E entries; logits are already in s_score.
__device__ void route_token(const RouterDev &r, const MoeDispatch &d, uint32_t token, float *s_score, float *s_sel,
                            uint8_t *s_ok, uint32_t *s_groups, float *s_gscore, bool count_groups) {
  const uint32_t E = r.num_experts, lane = threadIdx.x & 31;
  constexpr int REG_E = 8;  // up to 32 * REG_E experts: selection keys live in registers
  const bool small = E <= 32 * REG_E;
  float cbias[REG_E];  // correction bias, fetched now so that its latency hides behind the scoring
#pragma unroll
  for (int j = 0; j < REG_E; j++) cbias[j] = (small && r.correction_bias && lane + 32 * j < E) ? __ldg(r.correction_bias + lane + 32 * j) : 0.0f;
  if (r.logit_bias)
#pragma unroll 1
    for (uint32_t i = lane; i < E; i += 32) s_score[i] += __ldg(r.logit_bias + i);
  __syncwarp();
  if (r.scoring == MER_SCORE_SOFTMAX) {
    // softmax_inplace (transformer.rs:2747-2819)
    float mx = -CUDART_INF_F;
    int nan = 0;
#pragma unroll 1
    for (uint32_t i = lane; i < E; i += 32) {
      float v = s_score[i];
      if (v != v)
        nan = 1;
      else if (v > mx)
        mx = v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      nan |= __shfl_xor_sync(0xffffffffu, nan, o);
    }
    if (nan || !isfinite(mx)) {
#pragma unroll 1
      for (uint32_t i = lane; i < E; i += 32) s_score[i] = 1.0f / (float)E;
      if (lane == 0) atomicOr(d.status, MER_DEVSTAT_NONFINITE_ROUTER);
    } else {
#pragma unroll 1
      for (uint32_t i = lane; i < E; i += 32) s_score[i] = expf(s_score[i] - mx);
      __syncwarp();
      float sum = 0.0f;
      if (lane == 0) {  // the reference sums left to right; keep that order
        if ((E & 3u) == 0) {
          const float4 *s4 = reinterpret_cast<const float4 *>(s_score);  // E % 4 == 0 keeps every warp's array 16-byte aligned
#pragma unroll 4
          for (uint32_t i = 0; i < E / 4; i++) {
            const float4 v = s4[i];
            sum += v.x, sum += v.y, sum += v.z, sum += v.w;
          }
        } else {
#pragma unroll 1
          for (uint32_t i = 0; i < E; i++) sum += s_score[i];
        }
      }
      sum = __shfl_sync(0xffffffffu, sum, 0);
      if (sum > 0.0f)
#pragma unroll 1
        for (uint32_t i = lane; i < E; i += 32) s_score[i] = s_score[i] / sum;
    }
  } else {
#pragma unroll 1
    for (uint32_t i = lane; i < E; i += 32) s_score[i] = 1.0f / (1.0f + expf(-s_score[i]));
  }
  __syncwarp();
  if (small) {
#pragma unroll
    for (int j = 0; j < REG_E; j++) {
      const uint32_t i = lane + 32 * j;
      if (i < E) s_sel[i] = r.correction_bias ? s_score[i] + cbias[j] : s_score[i], s_ok[i] = 1;
    }
  } else {
#pragma unroll 1
    for (uint32_t i = lane; i < E; i += 32) {
      s_sel[i] = r.correction_bias ? s_score[i] + r.correction_bias[i] : s_score[i];
      s_ok[i] = 1;
    }
  }
  __syncwarp();
  // group_filter_shape + select_top_groups (gating.rs:335-376)
  const uint32_t ng = r.n_group < 1 ? 1 : r.n_group;
  const bool grouped = ng > 1 && r.topk_group > 0 && r.topk_group < ng && (E % ng) == 0 && ng <= 64;
  if (grouped) {
    const uint32_t gs = E / ng;
#pragma unroll 1
    for (uint32_t gi = lane; gi < ng; gi += 32) {
      float top1 = -CUDART_INF_F, top2 = -CUDART_INF_F;
#pragma unroll 1
      for (uint32_t i = 0; i < gs; i++) {
        float s = s_sel[gi * gs + i];
        if (s > top1) {
          top2 = top1;
          top1 = s;
        } else if (s > top2) {
          top2 = s;
        }
      }
      s_gscore[gi] = top1 + (isfinite(top2) ? top2 : 0.0f);
    }
    __syncwarp();
    if (lane == 0) {
      uint64_t taken = 0;
#pragma unroll 1
      for (uint32_t n = 0; n < r.topk_group; n++) {
        int bk = 0;
        uint32_t bi = MER_NONE;
#pragma unroll 1
        for (uint32_t g = 0; g < ng; g++) {
          if (taken >> g & 1) continue;
          int k = total_key(s_gscore[g]);
          if (bi == MER_NONE || better(k, g, bk, bi)) bk = k, bi = g;
        }
        taken |= 1ull << bi;
        s_groups[n] = bi;
      }
    }
    __syncwarp();
#pragma unroll 1
    for (uint32_t i = lane; i < E; i += 32) {
      bool ok = false;
#pragma unroll 1
      for (uint32_t n = 0; n < r.topk_group; n++) ok |= (s_groups[n] == i / gs);
      s_ok[i] = ok;
    }
    __syncwarp();
  }
  // top-k by (selection desc, id asc), non-finite skipped (gating.rs:315-333, 429-441)
  const uint32_t S = d.slots, k = r.top_k;
  uint32_t my_id = MER_NONE;  // lane i keeps the i-th pick
  uint32_t n_sel = 0;
  if (small) {
    // keys in registers: lane l holds experts l, l + 32, ...; a taken or disallowed expert bids INT_MIN
    int keys[REG_E];
#pragma unroll
    for (int j = 0; j < REG_E; j++) {
      const uint32_t i = lane + 32 * j;
      const float sv = i < E ? s_sel[i] : 0.0f;
      keys[j] = (i < E && s_ok[i] && isfinite(sv)) ? total_key(sv) : INT_MIN;
    }
#pragma unroll 1
    for (uint32_t n = 0; n < k; n++) {
      int bk = INT_MIN;
      uint32_t bj = 0;
#pragma unroll
      for (int j = 0; j < REG_E; j++)
        if (keys[j] > bk) bk = keys[j], bj = j;  // ascending j keeps the lowest id on ties
      const int top_key = __reduce_max_sync(0xffffffffu, bk);
      if (top_key == INT_MIN) break;  // nothing left to pick
      const uint32_t top_id = __reduce_min_sync(0xffffffffu, bk == top_key ? lane + 32 * bj : MER_NONE);
      if (lane == (top_id & 31u)) {
#pragma unroll
        for (int j = 0; j < REG_E; j++)
          if ((uint32_t)j == (top_id >> 5)) keys[j] = INT_MIN;
      }
      if (lane == (n & 31)) my_id = top_id;
      n_sel++;
    }
  } else {
#pragma unroll 1
    for (uint32_t n = 0; n < k; n++) {
      int bk = 0;
      uint32_t bi = MER_NONE;
#pragma unroll 1
      for (uint32_t i = lane; i < E; i += 32) {
        float s = s_sel[i];
        if (!s_ok[i] || !isfinite(s)) continue;
        int key = total_key(s);
        if (bi == MER_NONE || key > bk) bk = key, bi = i;  // ascending scan keeps the lowest id on ties
      }
      // warp arg-max by (key desc, id asc): two warp reductions; lanes without a candidate bid the lowest key
      const int my_key = bi == MER_NONE ? INT_MIN : bk;
      const int top_key = __reduce_max_sync(0xffffffffu, my_key);
      const uint32_t top_id = __reduce_min_sync(0xffffffffu, (bi != MER_NONE && my_key == top_key) ? bi : MER_NONE);
      bk = top_key, bi = top_id;
      if (bi == MER_NONE) break;
      if (lane == 0) s_ok[bi] = 0;
      if (lane == (n & 31)) my_id = bi;
      n_sel++;
      __syncwarp();
    }
  }
  // mixing weights = unbiased scores; renormalise; scale (gating.rs:443-474)
  float w = (lane < n_sel && my_id != MER_NONE) ? s_score[my_id] : 0.0f;
  if (r.normalise) {
    float sum = 0.0f;
#pragma unroll 1
    for (uint32_t i = 0; i < n_sel; i++) sum += __shfl_sync(0xffffffffu, w, i);  // slot order
    if (isfinite(sum) && sum > 0.0f) w = w / sum;
  }
  if (r.scaling != 1.0f && isfinite(r.scaling)) w = w * r.scaling;
  if (lane < k) {
    bool have = lane < n_sel;
    d.pair_expert[(size_t)token * S + lane] = have ? r.id_base + my_id : MER_NONE;
    d.pair_weight[(size_t)token * S + lane] = have ? w : 0.0f;
    if (count_groups && have) atomicAdd(d.group_count + my_id, 1u);  // the grid-wide grouping's count step, done here
  }
  if (lane == 0) {
    if (n_sel < k) atomicOr(d.status, MER_DEVSTAT_SHORT_SELECTION);
    if (S > k) {
      if (count_groups) atomicAdd(d.group_count + E, 1u);
      d.pair_expert[(size_t)token * S + k] = r.shared_expert_id;
      d.pair_weight[(size_t)token * S + k] = r.shared_scale ? r.shared_scale[token] : 1.0f;
    }
  }
}

// Router logits of a large batch as a tiled fp32 GEMM: logits[t][e] = x[t] . w[e].  A CTA computes 32 tokens x 64
// experts; K runs in chunks of 256 values that cp.async double-buffers in shared memory.  Eight warps split every
// chunk (32 values of K each); a thread holds 8 tokens x 8 experts (rows ty + 4 i and tx + 8 j: neighbouring lanes read
// neighbouring rows, whose stride of 260 floats keeps every 128-bit load conflict-free), i.e. 16 shared 128-bit loads per 256 FMAs (the
// 4 x 4 form before it, 8 loads per 64 FMAs, was bound by shared-memory bandwidth: 45 us for 1 GFLOP).  The eight
// partial sums are added at the end in warp order.  k_router then runs with `pre` set and only scores / selects.
constexpr int RL_WARPS = 8, RL_THREADS = 32 * RL_WARPS;
constexpr int RL_TT = 32, RL_TE = 64, RL_KC = 32 * RL_WARPS, RL_LD = RL_KC + 4;  // row stride = 4 mod 32 floats: conflict-free 128-bit loads
constexpr size_t RL_BUF = (size_t)(RL_TT + RL_TE) * RL_LD;                       // floats per buffer
constexpr size_t RL_SMEM = 2 * RL_BUF * 4;
__global__ void __launch_bounds__(RL_THREADS) k_router_logits_tiled(RouterDev r, MoeDispatch d, uint32_t ksplit) {
  extern __shared__ __align__(16) float sm[];
  const uint32_t E = r.num_experts, D = d.D, T = d.n_tokens;
  const uint32_t t0 = blockIdx.y * RL_TT, e0 = blockIdx.x * RL_TE;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, ty = lane >> 3, tx = lane & 7;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;
  // global -> shared: a thread copies one 16-byte piece of every fourth row (64 pieces per 256-value row)
  const uint32_t lr = tid >> 6, lc = (tid & 63) * 4;
  auto issue_chunk = [&](uint32_t k0, uint32_t buf) {
    float *xs = sm + buf * RL_BUF, *ws = xs + RL_TT * RL_LD;
#pragma unroll
    for (int i = 0; i < RL_TT / 4; i++) {
      const uint32_t row = 4 * i + lr;
      const float *src = d.x + (size_t)min(t0 + row, T - 1) * D + k0 + lc;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(xs + row * RL_LD + lc)), "l"(src) : "memory");
    }
#pragma unroll
    for (int j = 0; j < RL_TE / 4; j++) {
      const uint32_t row = 4 * j + lr;
      const float *src = r.w + (size_t)min(e0 + row, E - 1) * D + k0 + lc;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(ws + row * RL_LD + lc)), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // A batch of a few hundred tokens makes too few tiles for the SMs: blockIdx.z then takes one of `ksplit` slices of K
  // and writes its partial logits to set z of d.logits ([ksplit][T][E]); k_router adds the sets in order.
  const uint32_t n_chunks = D / RL_KC / ksplit, c_base = blockIdx.z * n_chunks;
  issue_chunk(c_base * RL_KC, 0);
  for (uint32_t c = 0; c < n_chunks; c++) {
    if (c + 1 < n_chunks) {
      issue_chunk((c_base + c + 1) * RL_KC, (c + 1) & 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");  // chunk c has landed (this thread's pieces)
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();  // ... and everybody else's
    const float *xs = sm + (c & 1) * RL_BUF, *ws = xs + RL_TT * RL_LD;
#pragma unroll 2
    for (int kk = 0; kk < RL_KC / RL_WARPS; kk += 4) {
      const int k = warp * (RL_KC / RL_WARPS) + kk;
      float4 a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; i++) a[i] = *reinterpret_cast<const float4 *>(xs + (ty + 4 * i) * RL_LD + k);
#pragma unroll
      for (int j = 0; j < 8; j++) b[j] = *reinterpret_cast<const float4 *>(ws + (tx + 8 * j) * RL_LD + k);
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
        }
    }
    __syncthreads();  // the buffer may be refilled two iterations from now
  }
  // partial sums of warps 1..7 through shared memory (the operand buffers are done with), added to warp 0's in warp order
  float *red = sm;  // [RL_WARPS - 1][RL_TT * RL_TE]
  static_assert((RL_WARPS - 1) * RL_TT * RL_TE <= 2 * RL_BUF, "the partial sums fit the operand buffers");
  if (warp > 0) {
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
      for (int j = 0; j < 8; j++) red[(warp - 1) * RL_TT * RL_TE + (ty + 4 * i) * RL_TE + tx + 8 * j] = acc[i][j];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float v = acc[i][j];
#pragma unroll
        for (int g = 0; g < RL_WARPS - 1; g++) v += red[g * RL_TT * RL_TE + (ty + 4 * i) * RL_TE + tx + 8 * j];
        const uint32_t t = t0 + ty + 4 * i, e = e0 + tx + 8 * j;
        if (t < T && e < E) d.logits[((size_t)blockIdx.z * T + t) * E + e] = v;
      }
  }
}

__global__ void __launch_bounds__(ROUTER_THREADS) k_router(RouterDev r, MoeDispatch d, uint32_t max_tokens, int pre, int group_here) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const uint32_t E = r.num_experts, D = d.D;
  const uint32_t tile = blockIdx.y, t0 = tile * ROUTER_TT;
  const uint32_t n_here = min((uint32_t)ROUTER_TT, d.n_tokens - t0);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t e0 = blockIdx.x * ROUTER_ROWS;
  __shared__ float s_part[ROUTER_ROWS][ROUTER_TT][ROUTER_ROWS + 1];  // [row][token][warp]
  __shared__ float s_logit[ROUTER_TT][ROUTER_ROWS];                  // used when one CTA covers all experts
  const bool single = gridDim.x == 1 && !pre;

  if (pre) {
    // logits are already in d.logits (k_router_logits_tiled)
  } else if ((D & 1023u) == 0) {
    const uint32_t slice4 = D / 4 / ROUTER_ROWS;  // float4 per warp slice
    float acc[ROUTER_ROWS][ROUTER_TT];
#pragma unroll
    for (int rr = 0; rr < ROUTER_ROWS; rr++)
#pragma unroll
      for (int tt = 0; tt < ROUTER_TT; tt++) acc[rr][tt] = 0.0f;
#pragma unroll 2
    for (uint32_t i = lane; i < slice4; i += 32) {
      float4 b[ROUTER_TT], a[ROUTER_ROWS];
#pragma unroll
      for (int tt = 0; tt < ROUTER_TT; tt++) {
        b[tt] = make_float4(0, 0, 0, 0);
        if ((uint32_t)tt < n_here) b[tt] = __ldg(reinterpret_cast<const float4 *>(d.x + (size_t)(t0 + tt) * D) + warp * slice4 + i);
      }
#pragma unroll
      for (int rr = 0; rr < ROUTER_ROWS; rr++) {
        const uint32_t row = min(e0 + rr, E - 1);
        a[rr] = __ldg(reinterpret_cast<const float4 *>(r.w + (size_t)row * D) + warp * slice4 + i);
      }
#pragma unroll
      for (int rr = 0; rr < ROUTER_ROWS; rr++)
#pragma unroll
        for (int tt = 0; tt < ROUTER_TT; tt++) {
          acc[rr][tt] = fmaf(a[rr].x, b[tt].x, acc[rr][tt]);
          acc[rr][tt] = fmaf(a[rr].y, b[tt].y, acc[rr][tt]);
          acc[rr][tt] = fmaf(a[rr].z, b[tt].z, acc[rr][tt]);
          acc[rr][tt] = fmaf(a[rr].w, b[tt].w, acc[rr][tt]);
        }
    }
#pragma unroll
    for (int rr = 0; rr < ROUTER_ROWS; rr++)
#pragma unroll
      for (int tt = 0; tt < ROUTER_TT; tt++) {
        float v = warp_sum(acc[rr][tt]);
        if (lane == 0) s_part[rr][tt][warp] = v;
      }
    __syncthreads();
    if (threadIdx.x < ROUTER_ROWS * ROUTER_TT) {
      const uint32_t rr = threadIdx.x / ROUTER_TT, tt = threadIdx.x % ROUTER_TT;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < ROUTER_ROWS; w++) v += s_part[rr][tt][w];
      if (single)
        s_logit[tt][rr] = v;
      else if (e0 + rr < E && tt < n_here)
        d.logits[(size_t)(t0 + tt) * E + e0 + rr] = v;
    }
  } else {
    // any d_model: warp = expert row, tokens one after the other
    const uint32_t e = e0 + warp;
    for (uint32_t tt = 0; tt < n_here; tt++) {
      float acc = 0.0f;
      if (e < E) {
        const float *w = r.w + (size_t)e * D, *x = d.x + (size_t)(t0 + tt) * D;
        for (uint32_t i = lane; i < D; i += 32) acc = fmaf(__ldg(w + i), __ldg(x + i), acc);
        acc = warp_sum(acc);
      }
      if (lane == 0 && e < E) {
        if (single)
          s_logit[tt][warp] = acc;
        else
          d.logits[(size_t)(t0 + tt) * E + e] = acc;
      }
    }
  }
  __shared__ uint32_t s_flag;
  __syncthreads();
  if (!single && !pre) {
    if (threadIdx.x == 0) {
      __threadfence();
      uint32_t prev = atomicAdd(&d.counters[tile], 1u);
      s_flag = (prev == gridDim.x - 1);
      if (s_flag) d.counters[tile] = 0;  // re-arm for the next launch
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
  }

  // ---- this CTA holds the last logits of the token tile: one warp routes one token ----
  __shared__ uint32_t s_groups[ROUTER_TT][64];
  __shared__ float s_gscore[ROUTER_TT][64];
  if (warp < n_here) {
    float *s_score = reinterpret_cast<float *>(smem_raw) + (size_t)warp * 2 * E;  // [E] scores (become mixing weights)
    float *s_sel = s_score + E;                                                    // [E] selection scores
    uint8_t *s_ok = smem_raw + (size_t)ROUTER_TT * 2 * E * 4 + (size_t)warp * E;    // [E] allowed & not yet taken
    const uint32_t token = t0 + warp;
    if (pre > 1) {  // the logits kernel split K: add its partial sets in order
      for (uint32_t i = lane; i < E; i += 32) {
        float v = __ldcg(d.logits + (size_t)token * E + i);
        for (int z = 1; z < pre; z++) v += __ldcg(d.logits + ((size_t)z * d.n_tokens + token) * E + i);
        s_score[i] = v;
      }
    } else {
      for (uint32_t i = lane; i < E; i += 32) s_score[i] = single ? s_logit[warp][i] : __ldcg(d.logits + (size_t)token * E + i);
    }
    __syncwarp();
    route_token(r, d, token, s_score, s_sel, s_ok, s_groups[warp], s_gscore[warp], group_here == 2);
  }
  if (group_here != 1) return;  // a large dispatch is grouped by the grid-wide kernels that follow (2: their count step is done above)
  __syncthreads();
  const uint32_t n_tiles = gridDim.y;
  if (n_tiles > 1) {
    if (threadIdx.x == 0) {
      __threadfence();
      uint32_t prev = atomicAdd(&d.counters[max_tokens], 1u);
      s_flag = (prev == n_tiles - 1);
      if (s_flag) d.counters[max_tokens] = 0;
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
  }
  build_groups_layer(r, d, reinterpret_cast<uint32_t *>(smem_raw));
}

// Routing of a whole layer supplied by the caller (pair_expert already filled): group by expert.
__global__ void __launch_bounds__(ROUTER_THREADS) k_groups_layer(RouterDev r, MoeDispatch d) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  build_groups_layer(r, d, reinterpret_cast<uint32_t *>(smem_raw));
}

// Routing supplied by the caller: mode 0 = every pair is its own group, mode 1 = one group.
__global__ void k_groups_from_pairs(MoeDispatch d, int single_group) {
  const uint32_t P = d.n_tokens * d.slots;
  for (uint32_t p = threadIdx.x; p < P; p += blockDim.x) {
    d.perm[p] = p;
    if (!single_group) {
      d.group_expert[p] = d.pair_expert[p];
      d.offsets[p] = p;
    }
  }
  if (threadIdx.x == 0) {
    if (single_group) {
      d.group_expert[0] = d.pair_expert[0];
      d.offsets[0] = 0;
      d.offsets[1] = P;
    } else {
      d.offsets[P] = P;
    }
  }
  if (d.pass_group) {
    __syncthreads();  // the offsets written above are read back by the whole block
    build_passes_block(d, d.offsets);
  }
}

// ---------------------------------------------------------------------------------------
// Generic expert FFN.
// ---------------------------------------------------------------------------------------
constexpr int GEN_TG = 4;  // tokens of a group handled per pass over a weight row

__device__ __forceinline__ const uint8_t *group_weights(const MoeDispatch &d, uint32_t g) {
  uint32_t eid = d.group_expert[g];
  const uint8_t *base = (eid < d.max_experts) ? d.expert_ptr[eid] : nullptr;
  if (!base && threadIdx.x == 0) atomicOr(d.status, MER_DEVSTAT_RESIDENCY_MISS);
  return base;
}

template <int DT>
__global__ void __launch_bounds__(256) k_gate_up_generic(MoeDispatch d) {
  const uint32_t g = blockIdx.y;
  const uint32_t beg = d.offsets[g], end = d.offsets[g + 1];
  if (beg == end) return;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t r = blockIdx.x * 8 + warp;
  const uint8_t *base = group_weights(d, g);
  if (r >= d.F) return;
  if (!base) {  // fail closed: the pair contributes zeros and the host reports the miss
    for (uint32_t t = beg + lane; t < end; t += 32) d.h[(size_t)d.perm[t] * d.F + r] = 0.0f;
    return;
  }
  for (uint32_t t0 = beg; t0 < end; t0 += GEN_TG) {
    uint32_t pair[GEN_TG];
    const float *xs[GEN_TG];
    float ag[GEN_TG], au[GEN_TG];
#pragma unroll
    for (int t = 0; t < GEN_TG; t++) {
      pair[t] = (t0 + t < end) ? d.perm[t0 + t] : MER_NONE;
      xs[t] = d.x + (size_t)(pair[t] == MER_NONE ? 0 : pair[t] / d.slots) * d.D;
      ag[t] = au[t] = 0.0f;
    }
    for (uint32_t c = lane; c < d.D; c += 32) {
      float wg = weight_at<DT>(d, base, 0, r, c), wu = weight_at<DT>(d, base, 1, r, c);
#pragma unroll
      for (int t = 0; t < GEN_TG; t++) {
        float xv = __ldg(xs[t] + c);
        ag[t] = fmaf(wg, xv, ag[t]);
        au[t] = fmaf(wu, xv, au[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < GEN_TG; t++) {
      float gsum = warp_sum(ag[t]), usum = warp_sum(au[t]);
      if (lane == 0 && pair[t] != MER_NONE)
        d.h[(size_t)pair[t] * d.F + r] = silu_f(clamp_gate(gsum, d.swiglu_limit)) * usum;
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(256) k_down_generic(MoeDispatch d) {
  const uint32_t g = blockIdx.y;
  const uint32_t beg = d.offsets[g], end = d.offsets[g + 1];
  if (beg == end) return;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t r = blockIdx.x * 8 + warp;
  const uint8_t *base = group_weights(d, g);  // latches the residency miss: the slot may have gone since gate/up ran
  if (r >= d.D) return;
  if (!base) {
    for (uint32_t t = beg + lane; t < end; t += 32) d.y[(size_t)d.perm[t] * d.D + r] = 0.0f;
    return;
  }
  for (uint32_t t0 = beg; t0 < end; t0 += GEN_TG) {
    uint32_t pair[GEN_TG];
    const float *hs[GEN_TG];
    float acc[GEN_TG];
#pragma unroll
    for (int t = 0; t < GEN_TG; t++) {
      pair[t] = (t0 + t < end) ? d.perm[t0 + t] : MER_NONE;
      hs[t] = d.h + (size_t)(pair[t] == MER_NONE ? d.perm[beg] : pair[t]) * d.F;
      acc[t] = 0.0f;
    }
    for (uint32_t c = lane; c < d.F; c += 32) {
      float w = weight_at<DT>(d, base, 2, r, c);
#pragma unroll
      for (int t = 0; t < GEN_TG; t++) acc[t] = fmaf(w, hs[t][c], acc[t]);
    }
#pragma unroll
    for (int t = 0; t < GEN_TG; t++) {
      float s = warp_sum(acc[t]);
      if (lane == 0 && pair[t] != MER_NONE) d.y[(size_t)pair[t] * d.D + r] = s;
    }
  }
}

// out[token] = sum over slots, in slot order, of weight * y (combine_outputs_into,
// inference.rs:4472-4491; zero weights and unfilled slots skipped as engine.rs:5575-5581).
// Multiply and add round separately, as the reference's `*dst += weight * *v` does.
__global__ void __launch_bounds__(256) k_combine(MoeDispatch d) {
  const uint32_t token = blockIdx.y;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.D) return;
  float acc = 0.0f;
  for (uint32_t s = 0; s < d.slots; s++) {
    if (d.residual && s == d.routed_slots) acc = __fadd_rn(d.residual[(size_t)token * d.D + i], acc);  // hidden + routed sum
    size_t p = (size_t)token * d.slots + s;
    float w = d.pair_weight[p];
    if (d.pair_expert[p] == MER_NONE || w == 0.0f) continue;
    float yv;
    if (d.y_parts && d.y_nparts > 1) {  // the streaming FFN left K-split partials: add them in split order
      const size_t n = (size_t)d.n_tokens * d.slots * d.D;
      yv = d.y_parts[p * d.D + i];
#pragma unroll 8
      for (uint32_t k = 1; k < d.y_nparts; k++) yv += d.y_parts[(size_t)k * n + p * d.D + i];
    } else {
      yv = d.y[p * d.D + i];
    }
    acc = __fadd_rn(acc, __fmul_rn(w, yv));
  }
  if (d.residual && d.routed_slots >= d.slots) acc = __fadd_rn(d.residual[(size_t)token * d.D + i], acc);
  d.out[(size_t)token * d.D + i] = acc;
}

// The same sum for final per-pair outputs (no K-split partials) and d_model % 4 == 0: one CTA per token, a thread four
// consecutive values; the rows of eight slots are loaded before the first is consumed (the one-value-per-thread form
// above moved 150 MB at 3 TB/s on a 2048-token batch).  Order and rounding are unchanged.
__global__ void __launch_bounds__(256) k_combine_rows4(MoeDispatch d) {
  const uint32_t token = blockIdx.x, S = d.slots;
  __shared__ float s_w[64];
  if (threadIdx.x < S && threadIdx.x < 64) {
    const size_t p = (size_t)token * S + threadIdx.x;
    const float w = d.pair_weight[p];
    s_w[threadIdx.x] = d.pair_expert[p] == MER_NONE ? 0.0f : w;  // a zero weight skips the slot
  }
  __syncthreads();
  const float4 *y4 = reinterpret_cast<const float4 *>(d.y) + (size_t)token * S * (d.D / 4);
  const float4 *res4 = d.residual ? reinterpret_cast<const float4 *>(d.residual) + (size_t)token * (d.D / 4) : nullptr;
  for (uint32_t i4 = threadIdx.x; i4 < d.D / 4; i4 += blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (uint32_t s0 = 0; s0 <= S; s0 += 8) {
      float4 y[8];
#pragma unroll
      for (int j = 0; j < 8; j++)
        y[j] = (s0 + j < S && s_w[s0 + j] != 0.0f) ? __ldcs(y4 + (size_t)(s0 + j) * (d.D / 4) + i4) : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const uint32_t sl = s0 + j;
        if (sl > S) break;
        if (res4 && sl == min(d.routed_slots, S)) {  // hidden + routed sum, before the shared expert's slot
          const float4 r = __ldg(res4 + i4);
          acc.x = __fadd_rn(r.x, acc.x), acc.y = __fadd_rn(r.y, acc.y), acc.z = __fadd_rn(r.z, acc.z), acc.w = __fadd_rn(r.w, acc.w);
        }
        if (sl == S) continue;
        const float wt = s_w[sl];
        if (wt == 0.0f) continue;
        acc.x = __fadd_rn(acc.x, __fmul_rn(wt, y[j].x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(wt, y[j].y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(wt, y[j].z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(wt, y[j].w));
      }
    }
    reinterpret_cast<float4 *>(d.out)[(size_t)token * (d.D / 4) + i4] = acc;
  }
}

// RMSNorm of every token row and / or the shared expert's gate scalar (RmsNorm::forward_inplace, transformer.rs:62-74;
// SharedExpert::forward, transformer.rs:2224-2231).  One CTA per token; sums are block tree reductions (the
// reference adds left to right: rounding differs in the last bits only).
__global__ void __launch_bounds__(256) k_pre_moe(const float *__restrict__ x, uint32_t D, const float *__restrict__ rms_weight, float eps,
                                                 const float *__restrict__ shared_gate, float *__restrict__ xn,
                                                 float *__restrict__ shared_scale) {
  __shared__ float s_red[8];
  __shared__ float s_bcast;
  const uint32_t token = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *row = x + (size_t)token * D;
  auto block_sum = [&](float v) -> float {
    v = warp_sum(v);
    __syncthreads();  // s_red / s_bcast of a previous reduction have been read
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int w = 0; w < 8; w++) t += s_red[w];
      s_bcast = t;
    }
    __syncthreads();
    return s_bcast;
  };
  float scale = 1.0f;
  if (rms_weight) {
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
    sq = block_sum(sq);
    scale = 1.0f / sqrtf(sq / (float)D + eps);
  }
  float dot = 0.0f;
  for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) {
    float v = row[i];
    if (rms_weight) {
      v = __fmul_rn(__fmul_rn(v, scale), rms_weight[i]);  // x * scale * weight, rounded after each product
      xn[(size_t)token * D + i] = v;
    }
    if (shared_gate) dot = fmaf(shared_gate[i], v, dot);
  }
  if (shared_gate) {
    dot = block_sum(dot);
    if (threadIdx.x == 0) shared_scale[token] = 1.0f / (1.0f + expf(-dot));
  }
}

template <int DT>
__global__ void k_dequant(const uint8_t *__restrict__ src, float *__restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = decode_weight<DT>(src, i);
}

template <int DT>
__global__ void k_dequant_packed(const uint8_t *__restrict__ expert, int matrix, uint32_t D, uint32_t F, float *__restrict__ dst) {
  const uint32_t rows = matrix < 2 ? F : D, cols = matrix < 2 ? D : F;
  size_t n = (size_t)rows * cols;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint32_t row = (uint32_t)(i / cols), col = (uint32_t)(i % cols);
    PackedAddr a = packed_locate<DT>(D, F, matrix, row, col);
    float sc = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(expert + a.scale));
    uint32_t byte = expert[a.quant];
    int q = DT == MER_DTYPE_Q8_0 ? (int)(int8_t)byte : (int)((col & 16u) ? (byte >> 4) : (byte & 15u)) - 8;
    dst[i] = __fmul_rn(sc, (float)q);
  }
}

// One thread per source block: copies its scale and its quant bytes to their packed places.
template <int DT>
__global__ void k_repack(const uint8_t *__restrict__ flat, uint8_t *__restrict__ packed, uint32_t D, uint32_t F) {
  constexpr uint32_t BB = DT == MER_DTYPE_Q8_0 ? MER_Q8_BLOCK_BYTES : MER_Q4_BLOCK_BYTES;
  const size_t per_matrix = (size_t)D * F / 32;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < 3 * per_matrix; i += stride) {
    const int matrix = (int)(i / per_matrix);
    const size_t blk = i % per_matrix;
    const uint32_t K = matrix < 2 ? D : F;
    const uint32_t row = (uint32_t)(blk / (K / 32)), kb = (uint32_t)(blk % (K / 32));
    const uint16_t *src = reinterpret_cast<const uint16_t *>(flat + i * BB);  // blocks are 2-byte aligned
    PackedAddr a0 = packed_locate<DT>(D, F, matrix, row, kb * 32);
    *reinterpret_cast<uint16_t *>(packed + a0.scale) = src[0];
    if (DT == MER_DTYPE_Q4_0) {
#pragma unroll
      for (uint32_t t = 0; t < 4; t++) {  // quant bytes 4t..4t+3 hold elements 4t.. (low) and 16+4t.. (high)
        PackedAddr a = packed_locate<DT>(D, F, matrix, row, kb * 32 + 4 * t);
        *reinterpret_cast<uint32_t *>(packed + a.quant) = (uint32_t)src[1 + 2 * t] | ((uint32_t)src[2 + 2 * t] << 16);
      }
    } else {
#pragma unroll
      for (uint32_t t = 0; t < 4; t++) {
        PackedAddr a = packed_locate<DT>(D, F, matrix, row, kb * 32 + 8 * t);
        uint2 v;
        v.x = (uint32_t)src[1 + 4 * t] | ((uint32_t)src[2 + 4 * t] << 16);
        v.y = (uint32_t)src[3 + 4 * t] | ((uint32_t)src[4 + 4 * t] << 16);
        *reinterpret_cast<uint2 *>(packed + a.quant) = v;
      }
    }
  }
}

// Raw block-stream matvec for the qualification cases: one warp per row.
template <int DT>
__global__ void k_raw_matvec(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, size_t rows,
                             size_t cols) {
  size_t r = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  uint32_t lane = threadIdx.x & 31;
  if (r >= rows) return;
  float acc = 0.0f;
  for (size_t c = lane; c < cols; c += 32) acc = fmaf(decode_weight<DT>(w, r * cols + c), x[c], acc);
  acc = warp_sum(acc);
  if (lane == 0) y[r] = acc;
}

__global__ void k_f16_to_f32(const uint16_t *__restrict__ src, float *__restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = f16_bits_to_f32(src[i]);
}
__global__ void k_f32_to_f16(const float *__restrict__ src, uint16_t *__restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __half_as_ushort(__float2half_rn(src[i]));
}

}  // namespace

cudaError_t launch_router(const RouterDev &r, const MoeDispatch &d, uint32_t max_tokens, cudaStream_t s,
                          int *launches, bool group) {
  const uint32_t E = r.num_experts, G = d.n_groups;
  const uint32_t P = d.n_tokens * d.slots;
  size_t smem_topk = (size_t)ROUTER_TT * E * 9;
  size_t smem_grp = (size_t)(G + 1 + (G <= STABLE_G ? ROUTER_ROWS * G : G) + (P <= SMALL_P ? P : 0)) * 4;
  size_t smem = smem_topk > smem_grp ? smem_topk : smem_grp;
  smem = (smem + 15) & ~(size_t)15;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k_router, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  const bool tiled = d.n_tokens >= 256 && (d.D % RL_KC) == 0;  // from a few hundred tokens: logits as a tiled GEMM first
  uint32_t ksplit = 1;
  if (tiled) {
    dim3 lgrid((E + RL_TE - 1) / RL_TE, (d.n_tokens + RL_TT - 1) / RL_TT);
    // split K over blockIdx.z while the tiles alone leave SMs idle (the partial sets must fit the logits scratch,
    // which holds max_tokens x 4096 floats, and a slice is a whole number of chunks)
    const uint32_t n_chunks = d.D / RL_KC, tiles = lgrid.x * lgrid.y;
    for (uint32_t ks = 2; ks <= 8 && ks <= n_chunks; ks++)
      if (n_chunks % ks == 0 && tiles * ks <= 160 && (size_t)ks * E <= 4096) ksplit = ks;
    lgrid.z = ksplit;
    cudaError_t e = cudaFuncSetAttribute(k_router_logits_tiled, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RL_SMEM);
    if (e != cudaSuccess) return e;
    k_router_logits_tiled<<<lgrid, RL_THREADS, RL_SMEM, s>>>(r, d, ksplit);
    if (launches) (*launches)++;
  }
  dim3 grid(tiled ? 1 : (E + ROUTER_ROWS - 1) / ROUTER_ROWS, (d.n_tokens + ROUTER_TT - 1) / ROUTER_TT);
  const bool grid_grouping = group && P >= GRID_GROUPING_PAIRS && d.group_count != nullptr;
  k_router<<<grid, ROUTER_THREADS, smem, s>>>(r, d, max_tokens, tiled ? (int)ksplit : 0, grid_grouping ? 2 : group ? 1 : 0);
  if (launches) (*launches)++;
  if (grid_grouping) {  // the router has counted the pairs per group
    const unsigned blocks = (P + 1023) / 1024;
    k_group_scan<<<1, 256, 0, s>>>(r, d);
    k_group_scatter<<<blocks, 256, 0, s>>>(r, d);
    k_group_clear<<<1, 256, 0, s>>>(d);
    if (launches) (*launches) += 3;
  }
  return cudaGetLastError();
}

bool groups_layer_on_grid(const MoeDispatch &d) { return d.n_tokens * d.slots >= GRID_GROUPING_PAIRS && d.group_count != nullptr; }

cudaError_t launch_groups_layer(const RouterDev &r, const MoeDispatch &d, cudaStream_t s, int *launches, bool counted) {
  const uint32_t G = d.n_groups, P = d.n_tokens * d.slots;
  if (groups_layer_on_grid(d)) {  // a large dispatch: count / scan / scatter over the grid
    const unsigned blocks = (P + 1023) / 1024;
    if (!counted) k_group_count<<<blocks, 256, 0, s>>>(r, d);
    k_group_scan<<<1, 256, 0, s>>>(r, d);
    k_group_scatter<<<blocks, 256, 0, s>>>(r, d);
    k_group_clear<<<1, 256, 0, s>>>(d);
    if (launches) (*launches) += counted ? 3 : 4;
    return cudaGetLastError();
  }
  size_t smem = (size_t)(G + 1 + (G <= STABLE_G ? ROUTER_ROWS * G : G) + (P <= SMALL_P ? P : 0)) * 4;
  smem = (smem + 15) & ~(size_t)15;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k_groups_layer, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  k_groups_layer<<<1, ROUTER_THREADS, smem, s>>>(r, d);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_groups_from_pairs(const MoeDispatch &d, cudaStream_t s, int *launches) {
  k_groups_from_pairs<<<1, 256, 0, s>>>(d, d.n_groups == 1);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_ffn_generic(const MoeDispatch &d, cudaStream_t s, int *launches, cudaEvent_t ev_mid) {
  dim3 g1((d.F + 7) / 8, d.n_groups), g2((d.D + 7) / 8, d.n_groups);
  if (d.dtype == MER_DTYPE_Q8_0) {
    k_gate_up_generic<MER_DTYPE_Q8_0><<<g1, 256, 0, s>>>(d);
    if (ev_mid) cudaEventRecord(ev_mid, s);
    k_down_generic<MER_DTYPE_Q8_0><<<g2, 256, 0, s>>>(d);
  } else {
    k_gate_up_generic<MER_DTYPE_Q4_0><<<g1, 256, 0, s>>>(d);
    if (ev_mid) cudaEventRecord(ev_mid, s);
    k_down_generic<MER_DTYPE_Q4_0><<<g2, 256, 0, s>>>(d);
  }
  if (launches) (*launches) += 2;
  return cudaGetLastError();
}

cudaError_t launch_combine(const MoeDispatch &d, cudaStream_t s, int *launches) {
  if (d.combined) return cudaSuccess;  // the expert FFN launch already did it
  if (!(d.y_parts && d.y_nparts > 1) && (d.D & 3u) == 0 && d.slots <= 64) {
    k_combine_rows4<<<d.n_tokens, 256, 0, s>>>(d);
  } else {
    dim3 grid((d.D + 255) / 256, d.n_tokens);
    k_combine<<<grid, 256, 0, s>>>(d);
  }
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_pre_moe(const float *x, uint32_t n_tokens, uint32_t D, const float *rms_weight, float eps, const float *shared_gate,
                           float *xn, float *shared_scale, cudaStream_t s, int *launches) {
  if (!rms_weight && !shared_gate) return cudaSuccess;
  k_pre_moe<<<n_tokens, 256, 0, s>>>(x, D, rms_weight, eps, shared_gate, xn, shared_scale);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_dequant(int dtype, const uint8_t *src, float *dst, size_t n, cudaStream_t s) {
  int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (blocks < 1) blocks = 1;
  if (dtype == MER_DTYPE_Q8_0)
    k_dequant<MER_DTYPE_Q8_0><<<blocks, 256, 0, s>>>(src, dst, n);
  else
    k_dequant<MER_DTYPE_Q4_0><<<blocks, 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}

cudaError_t launch_dequant_packed(int dtype, const uint8_t *expert, int matrix, uint32_t D, uint32_t F, float *dst, cudaStream_t s) {
  if (dtype == MER_DTYPE_Q8_0)
    k_dequant_packed<MER_DTYPE_Q8_0><<<148 * 8, 256, 0, s>>>(expert, matrix, D, F, dst);
  else
    k_dequant_packed<MER_DTYPE_Q4_0><<<148 * 8, 256, 0, s>>>(expert, matrix, D, F, dst);
  return cudaGetLastError();
}

cudaError_t launch_repack(int dtype, const uint8_t *flat, uint8_t *packed, uint32_t D, uint32_t F, cudaStream_t s) {
  if (dtype == MER_DTYPE_Q8_0)
    k_repack<MER_DTYPE_Q8_0><<<148 * 8, 256, 0, s>>>(flat, packed, D, F);
  else
    k_repack<MER_DTYPE_Q4_0><<<148 * 8, 256, 0, s>>>(flat, packed, D, F);
  return cudaGetLastError();
}

cudaError_t launch_raw_matvec(int dtype, const uint8_t *w, const float *x, float *y, size_t rows, size_t cols, cudaStream_t s) {
  unsigned blocks = (unsigned)((rows + 7) / 8);
  if (dtype == MER_DTYPE_Q8_0)
    k_raw_matvec<MER_DTYPE_Q8_0><<<blocks, 256, 0, s>>>(w, x, y, rows, cols);
  else
    k_raw_matvec<MER_DTYPE_Q4_0><<<blocks, 256, 0, s>>>(w, x, y, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_f16_to_f32(const uint16_t *src, float *dst, size_t n, cudaStream_t s) {
  k_f16_to_f32<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}
cudaError_t launch_f32_to_f16(const float *src, uint16_t *dst, size_t n, cudaStream_t s) {
  k_f32_to_f16<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}
