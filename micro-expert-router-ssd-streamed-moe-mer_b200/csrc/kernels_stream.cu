// Streaming expert FFN for decode-sized token groups (a few tokens per expert): HBM-bound.
//
// Data flow per projection phase (gate/up, then down):
//   * Experts are resident in the tile-major fragment layout of layout.cuh (the reference's bytes,
//     permuted at admission).  A stage of the ring is two contiguous 16-row tile chunks, each moved
//     global -> shared memory by ONE bulk async copy (cp.async.bulk, completion on an mbarrier):
//     every byte of an expert is read from HBM once, as a linear stream.
//   * Warps unpack the integer part of the weights straight into f16 mma.sync A fragments.  A
//     4-bit or 8-bit field masked into the low mantissa bits of an f16 IS the subnormal value
//     q * 2^-24 (q * 2^-20 for a field at bits 4..7), so unpacking is one LOP3 per two weights and
//     the integers are exact.  The zero point (8 for Q4_0, 128 for the sign-flipped Q8_0 byte) is
//     folded in as the accumulator's initial value -zp * sum(x_block).
//   * Activations are pre-split into f16 hi + lo parts (22+ significant bits) after an exact
//     power-of-two per-token scaling; hi and lo are two columns of the n=8 MMA tile, so one tile
//     carries 4 tokens.  Products are exact, accumulation is fp32 in the tensor core.
//   * The per-block f16 scale d is applied in fp32 when a block's partial is folded into the row
//     accumulator: acc += d * partial (the ordering of matmul_q4_0.wgsl:65-85 in the reference).
//
// Work is cut into items (token pass, K split, group of 16 tiles).  Each of the 16 consumer warps of
// a CTA owns one 16-row tile of the item over the item's K range: no warp ever waits for another
// one's partial sums (an earlier version split K across warps and lost a third of its time at the
// hand-off barrier).  Load balance comes from splitting K across CTAs instead: partial sums go to
// scratch and the next kernel adds them (k_h_finalize applies SiLU(gate)*up, the combine kernel sums
// the down partials), always in the same order, so results are deterministic.  Each persistent CTA
// takes a contiguous item range and rebuilds activation fragments only when its (pass, K split)
// changes; no atomics on data, no inter-CTA waits.  Every mbarrier wait is bounded: on expiry the
// warp stops computing, the CTA latches MER_DEVSTAT_TIMEOUT, drains its copies in flight and returns.
#include "kernels.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "../../include/mer_b200.h"
#include "layout.cuh"
#include "ptx.cuh"

namespace {

constexpr int CONSUMER_WARPS = 16;
constexpr int PRODUCER_WARPS = 2;  // each issues the bulk copies of half a stage's tiles: one warp alone was busy ~90 % of the time
constexpr int THREADS = (CONSUMER_WARPS + PRODUCER_WARPS) * 32;
constexpr uint32_t HEADER_BYTES = 1024;  // mbarriers and per-pass token tables at the start of shared memory
constexpr float POW2_24 = 16777216.0f;

constexpr int TAIL_NONE = 0, TAIL_FINALIZE = 1, TAIL_COMBINE = 2, TAIL_REDUCE = 3;

struct StreamParams {
  MoeDispatch d;
  int phase;                 // 0 = gate/up (+SiLU*mul), 1 = down
  const float *act;          // activations, row-major fp32: x [n_tokens x D] (gate/up) or h [P x F] (down)
  uint32_t act_per_pair;     // 1: rows indexed by pair (down); 0: by token = pair / slots (gate/up)
  uint32_t rows;             // output rows of the projection (F for gate/up, D for down)
  uint32_t kb_total;         // 32-weight blocks per row
  uint32_t kb_split;         // blocks per K split (kb_total when n_ksplit == 1)
  uint32_t n_ksplit;
  uint32_t kc;               // blocks per pipeline stage
  uint32_t n_stages;
  uint32_t chunk_stride;     // bytes between the 16-row tile chunks of a stage (kc * 16 * block bytes)
  uint32_t frag_cols;        // fragment arrays held in shared memory: 2 * min(4 * NT, most tokens of any group)
  uint32_t frag_stride;      // bytes between (token, part) fragment arrays in shared memory
  float *out;                // phase 0: h [P x F], or gate/up partials [n_ksplit][P][2][F] when K is split;
                             // phase 1: y partials [n_ksplit][P x D]
  int tail;                  // work done by the whole grid after a grid-wide barrier (cooperative launch):
                             // TAIL_FINALIZE (phase 0, K split): h = SiLU(sum gate) * sum up and the row maxima;
                             // TAIL_COMBINE (phase 1): out[token] = weighted sum of its pairs' outputs in slot order;
                             // TAIL_REDUCE (phase 1, K split): y[pair] = sum of its partials, grouped pairs only
  uint32_t *grid_counter;    // arrival counter of that barrier, zeroed by the grouping kernel
};

// D = A * B + C with separate C so that a seed / zero needs no register moves.
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1, float c0, float c1, float c2, float c3) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory"); }


// ------------------------------------------------------------------- activation fragments
// Position of block element j in the per-block fragment order, and the extra exact scale of
// that slot (Q4_0 high nibbles sit 4 mantissa bits higher, so their activations carry 2^-4).
template <int DT>
__device__ __forceinline__ void frag_slot(uint32_t j, uint32_t &pos, float &slot_scale) {
  if (DT == MER_DTYPE_Q4_0) {
    uint32_t hi = j >> 4, jj = j & 15u, t = jj >> 2, e = jj & 3u;
    // thread t order: [4t, 4t+2, 4t+1, 4t+3 | same +16]
    uint32_t within = (e == 0) ? 0 : (e == 2) ? 1 : (e == 1) ? 2 : 3;
    pos = t * 8 + hi * 4 + within;
    slot_scale = hi ? 0.0625f : 1.0f;
  } else {
    uint32_t t = j >> 3, e = j & 7u, half = e >> 2, ee = e & 3u;
    uint32_t within = (ee == 0) ? 0 : (ee == 2) ? 1 : (ee == 1) ? 2 : 3;
    pos = t * 8 + half * 4 + within;
    slot_scale = 1.0f;
  }
}

__device__ __forceinline__ float nan_max(float a, float b) { return (b > a || b != b) ? b : a; }  // NaN sticks

// ------------------------------------------------------------------------ weight unpacking
// Eight weights of one row slot of one block -> four f16x2 registers holding the integer fields as
// subnormals: {MMA0.k(2t,2t+1), MMA0.k(2t+8,2t+9), MMA1.k(2t,2t+1), MMA1.k(2t+8,2t+9)}.
__device__ __forceinline__ void unpack_q4(uint32_t v, uint32_t (&r)[4]) {
  const uint32_t v8 = v >> 8;
  r[0] = v & 0x000F000Fu;   // low nibbles of bytes 0, 2  -> elements 4t, 4t+2
  r[1] = v8 & 0x000F000Fu;  // low nibbles of bytes 1, 3  -> elements 4t+1, 4t+3
  r[2] = v & 0x00F000F0u;   // high nibbles -> elements 16 + ... (x16, undone on the activation side)
  r[3] = v8 & 0x00F000F0u;
}
__device__ __forceinline__ void unpack_q8(uint32_t lo, uint32_t hi, uint32_t (&r)[4]) {
  // int8 -> biased unsigned byte (q + 128) in the low mantissa bits
  r[0] = (lo ^ 0x80808080u) & 0x00FF00FFu;
  r[1] = ((lo >> 8) ^ 0x00808080u) & 0x00FF00FFu;
  r[2] = (hi ^ 0x80808080u) & 0x00FF00FFu;
  r[3] = ((hi >> 8) ^ 0x00808080u) & 0x00FF00FFu;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2 *>(&v)); }

template <int DT>
struct BlockBytes {
  static constexpr uint32_t value = DT == MER_DTYPE_Q4_0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES;
};

// --------------------------------------------------------------------------- main kernel
template <int DT, int NT>
__device__ __forceinline__ void ffn_stream_body(const StreamParams &p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr uint32_t BB = BlockBytes<DT>::value;
  constexpr uint32_t TP = 4 * NT;
  const MoeDispatch &d = p.d;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // shared memory carve-up
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // [n_stages]
  uint64_t *empty = full + p.n_stages;                   // [n_stages]
  uint32_t *s_abort = reinterpret_cast<uint32_t *>(empty + p.n_stages);
  uint32_t *s_pair = reinterpret_cast<uint32_t *>(smem + 160);  // [TP] pair index of each token of the current pass
  float *s_un = reinterpret_cast<float *>(smem + 192);          // [TP] its 2^24 / scale
  uint32_t *s_amax = reinterpret_cast<uint32_t *>(smem + 224);  // [TP] max |activation| of its row, as float bits
  // per-block accumulator seeds, [TP][kb_split + 2]: the four token rows a warp reads together (one per t) must not start
  // in the same bank (a stride of 32 blocks put every 64-bit read four-deep on one bank pair: 25 % more shared-memory
  // wavefronts in the whole gate/up phase)
  const uint32_t seed_stride = p.kb_split + 2;
  float *s_init = reinterpret_cast<float *>(smem + HEADER_BYTES);
  uint8_t *s_frag = reinterpret_cast<uint8_t *>(s_init + seed_stride * TP);  // [TP*2][frag_stride]
  s_frag = reinterpret_cast<uint8_t *>(((size_t)s_frag + 127) & ~(size_t)127);
  uint8_t *s_stage = s_frag + (size_t)p.frag_cols * p.frag_stride;          // [n_stages][16 tiles][chunk_stride]
  const uint32_t stage_bytes = CONSUMER_WARPS * p.chunk_stride;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.n_stages; s++) {
      mbar_init(&full[s], PRODUCER_WARPS);
      mbar_init(&empty[s], CONSUMER_WARPS);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint32_t n_tiles = p.rows / ((p.phase == 0 ? 8u : 16u) * CONSUMER_WARPS);  // items per (pass, K split)
  const uint32_t n_passes = *d.n_passes;
  const uint64_t n_items = (uint64_t)n_passes * p.n_ksplit * n_tiles;
  // the grouping kernel cut the item list into one contiguous range per CTA, balanced by the tokens of the passes
  const uint32_t *bounds = d.item_bounds + p.phase * MER_MAX_CTAS1 + blockIdx.x;
  const uint32_t item_beg = min((uint32_t)n_items, bounds[0]), item_end = min((uint32_t)n_items, bounds[1]);
  if (item_beg >= item_end) return;
  const size_t proj_bytes = (size_t)d.D * d.F / 32 * BB;
  const size_t tile_bytes = (size_t)p.kb_total * 16 * BB;  // one packed 16-row tile, all of K

  // items are ordered (pass, K split, tile); a CTA decodes its first item once and then steps
  uint32_t tile = item_beg % n_tiles, ks = (item_beg / n_tiles) % p.n_ksplit, pp = item_beg / n_tiles / p.n_ksplit;
  auto next_item = [&]() {
    if (++tile == n_tiles) {
      tile = 0;
      if (++ks == p.n_ksplit) ks = 0, ++pp;
    }
  };
  auto kb_range = [&](uint32_t ks, uint32_t &kb0, uint32_t &kbn) {
    kb0 = ks * p.kb_split;
    kbn = min(p.kb_split, p.kb_total - kb0);
  };

  if (warp >= CONSUMER_WARPS) {
    // ------------------------------ producer warps: warp h, lane m < 8 copies the chunk of tile 8h + m of every stage
    constexpr uint32_t TILES_PER_PRODUCER = CONSUMER_WARPS / PRODUCER_WARPS;
    const uint32_t my_tile = (warp - CONSUMER_WARPS) * TILES_PER_PRODUCER + (lane % TILES_PER_PRODUCER);
    uint32_t stage = 0, round = 0;
    bool ok = true;
    for (uint32_t item = item_beg; item < item_end && ok; item++, next_item()) {
      uint32_t kb0, kbn;
      kb_range(ks, kb0, kbn);
      uint32_t eid = d.group_expert[d.pass_group[pp]];
      const uint8_t *base = (eid < d.max_experts) ? d.expert_ptr[eid] : nullptr;
      if (!base) continue;  // consumers skip the same item
      // item -> packed tiles 16*tile .. 16*tile + 15 of the phase's region; lane m < 16 copies tile m's chunk
      const uint8_t *src = base + (p.phase == 0 ? 0 : 2 * proj_bytes) + (size_t)(CONSUMER_WARPS * tile + my_tile) * tile_bytes;
      for (uint32_t c0 = 0; c0 < kbn && ok; c0 += p.kc) {
        uint32_t nb = min(p.kc, kbn - c0);
        if (round > 0) ok = mbar_wait(&empty[stage], (round - 1) & 1);
        if (*(volatile uint32_t *)s_abort) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(&full[stage], TILES_PER_PRODUCER * nb * 16 * BB);
        __syncwarp();
        if (lane < TILES_PER_PRODUCER)
          bulk_g2s(s_stage + (size_t)stage * stage_bytes + my_tile * p.chunk_stride, src + (size_t)(kb0 + c0) * 16 * BB, nb * 16 * BB,
                   &full[stage]);
        if (++stage == p.n_stages) stage = 0, round++;
      }
    }
    if (!ok) {
      if (lane == 0) {
        *(volatile uint32_t *)s_abort = 1;
        atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
      }
      // drain: give copies already in flight a bounded chance to land before the CTA's memory is released
      for (uint32_t s = 0; s < p.n_stages; s++) (void)mbar_wait(&full[s], 0), (void)mbar_wait(&full[s], 1);
    }
    return;
  }

  // ---------------------------------------------------------------------- consumer warps
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t piece16 = packed_piece(g, t) * 16;  // byte offset of this lane's 16-byte piece inside a block record
  const uint32_t stage0 = smem_u32(s_stage) + warp * p.chunk_stride;  // this warp's tile chunk in stage 0
  const uint32_t frag0 = smem_u32(s_frag) + t * 16, init0 = smem_u32(s_init);
  uint32_t stage = 0, round = 0;
  uint32_t cur_pp = MER_NONE, cur_ks = MER_NONE;
  // A warp whose bounded wait expired goes "dead": it stops computing and waiting but still walks
  // the same loop structure, so the named barriers below always see all consumer warps.
  bool dead = false;

  // Fragment columns and seeds of tokens beyond a pass's count hold stale data (or lie past the
  // arrays when the dispatch has few tokens per group).  That is harmless: an MMA output column
  // depends on its own B column only, and the columns of absent tokens are never written out.
  uint32_t pstart = 0, pcount = 0;
  bool resident = false;

  for (uint32_t item = item_beg; item < item_end; item++, next_item()) {
    uint32_t kb0, kbn;
    kb_range(ks, kb0, kbn);

    if (pp != cur_pp || ks != cur_ks) {
      // new activation fragments: first, everyone must be done with the old ones
      if (pp != cur_pp) {
        pstart = d.pass_start[pp], pcount = d.pass_count[pp];
        const uint32_t eid = d.group_expert[d.pass_group[pp]];
        resident = eid < d.max_experts && d.expert_ptr[eid] != nullptr;
      }
      if (threadIdx.x < TP) s_amax[threadIdx.x] = 0;  // nobody reads it before the barrier below
      consumer_sync();
      cur_pp = pp, cur_ks = ks;
      // The pass's activation rows become MMA B fragments here, in shared memory: an exact power-of-two
      // scaling that puts max |a| of the row in [256, 512), an f16 hi/lo split in fragment order, and the
      // per-block accumulator seed -zp * 2^-24 * sum(block).  Warps share the rows: 16 / pcount per row; every
      // warp looks up its own row, so the only barriers are the one above, one for the row maxima (gate/up
      // phase) and the final one.
      const uint32_t K = p.kb_total * 32;
      const uint32_t wpt = CONSUMER_WARPS / pcount;  // warps per row (pcount <= 8)
      const uint32_t my_tok = warp / wpt, my_sub = warp % wpt;
      const bool has_row = my_tok < pcount;
      const float *row = nullptr;
      uint32_t my_pair = 0;
      if (has_row) {
        my_pair = d.perm[pstart + my_tok];
        row = p.act + (size_t)(p.act_per_pair ? my_pair : my_pair / d.slots) * K;
      }
      if (threadIdx.x < TP) s_pair[threadIdx.x] = threadIdx.x < pcount ? d.perm[pstart + threadIdx.x] : 0u;  // for the epilogues
      float row_max = 0.0f;
      if (p.phase == 0) {  // the row maximum is not known yet: one pass over the row
        float mx = 0.0f;
        if (has_row) {
          const float4 *r4 = reinterpret_cast<const float4 *>(row);
#pragma unroll 1
          for (uint32_t i = my_sub * 32 + lane; i < K / 4; i += wpt * 32) {
            const float4 v = __ldg(r4 + i);
            mx = nan_max(nan_max(nan_max(nan_max(mx, fabsf(v.x)), fabsf(v.y)), fabsf(v.z)), fabsf(v.w));
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (has_row && lane == 0) atomicMax(&s_amax[my_tok], (mx != mx) ? 0x7fc00000u : __float_as_uint(mx));
        consumer_sync();
        if (has_row) row_max = __uint_as_float(s_amax[my_tok]);
      } else if (has_row) {
        row_max = __uint_as_float(d.amax[my_pair]);  // collected by the gate/up epilogue or its finalize step
      }
      float row_scale = 1.0f;
      if (row_max > 0.0f && isfinite(row_max)) {
        int e;
        frexpf(row_max, &e);               // row_max = m * 2^e, m in [0.5, 1)
        row_scale = ldexpf(1.0f, 9 - e);   // row_max * scale in [256, 512)
      } else if (row_max != row_max || isinf(row_max)) {
        row_scale = row_max;  // non-finite activations poison the row, as they would in fp32
      }
      if (has_row && my_sub == 0 && lane == 0) s_un[my_tok] = POW2_24 / row_scale;
      if (has_row) {
        const float sc = row_scale;
        const float zp = DT == MER_DTYPE_Q4_0 ? 8.0f : 128.0f;
        uint8_t *hi_dst = s_frag + (size_t)(2 * my_tok) * p.frag_stride, *lo_dst = hi_dst + p.frag_stride;
        float *seed_dst = s_init + (size_t)my_tok * seed_stride;
        // float4 groups of this K split: 8 per block; a warp converts 4 blocks per step
#pragma unroll 1
        for (uint32_t q = my_sub * 32 + lane; q < kbn * 8; q += wpt * 32) {
          float4 v = __ldg(reinterpret_cast<const float4 *>(row + (size_t)kb0 * 32) + q);
          v.x *= sc, v.y *= sc, v.z *= sc, v.w *= sc;  // exact (power of two) unless it overflows
          const uint32_t kbl = q >> 3, j0 = (q & 7u) * 4;
          uint32_t pos;
          float ss;
          frag_slot<DT>(j0, pos, ss);  // the four elements land at pos + {0, 2, 1, 3}
          const float vs[4] = {v.x * ss, v.z * ss, v.y * ss, v.w * ss};
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const __half h = __float2half_rn(vs[i]);
            hi[i] = __half_as_ushort(h);
            lo[i] = __half_as_ushort(__float2half_rn(vs[i] - __half2float(h)));
          }
          *reinterpret_cast<uint2 *>(hi_dst + kbl * 64 + pos * 2) = make_uint2(hi[0] | hi[1] << 16, hi[2] | hi[3] << 16);
          *reinterpret_cast<uint2 *>(lo_dst + kbl * 64 + pos * 2) = make_uint2(lo[0] | lo[1] << 16, lo[2] | lo[3] << 16);
          float sum = (v.x + v.y) + (v.z + v.w);  // eight consecutive lanes hold one block
#pragma unroll
          for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
          if ((lane & 7) == 0) seed_dst[kbl] = -zp * sum * (1.0f / POW2_24);
        }
      }
      consumer_sync();  // fragments, seeds, s_pair, s_un visible to every warp
    }
    const size_t n_pairs = (size_t)d.n_tokens * d.slots;
    const bool split_gate_up = p.phase == 0 && p.n_ksplit > 1;
    if (!resident) {
      if (threadIdx.x == 0) atomicOr(d.status, MER_DEVSTAT_RESIDENCY_MISS);
      // fail closed: zero outputs for this item
      const uint32_t rows_here = (p.phase == 0 ? 8u : 16u) * CONSUMER_WARPS;
      for (uint32_t i = threadIdx.x; i < rows_here * pcount; i += CONSUMER_WARPS * 32) {
        const uint32_t pair = d.perm[pstart + i / rows_here], row = tile * rows_here + i % rows_here;
        if (split_gate_up) {
          float *gp = p.out + ((size_t)ks * n_pairs + pair) * 2 * d.F;
          gp[row] = 0.0f, gp[d.F + row] = 0.0f;
        } else if (p.phase == 0) {
          p.out[(size_t)pair * d.F + row] = 0.0f;
        } else {
          p.out[((size_t)ks * n_pairs + pair) * d.D + row] = 0.0f;
        }
      }
      continue;
    }

    // per-item loop invariants: where column g / token t of each N-tile lives (unused ones read zeros)
    uint32_t fa[NT], ia[NT];
#pragma unroll
    for (int n = 0; n < NT; n++) {
      fa[n] = frag0 + (n * 8 + g) * p.frag_stride;  // column g of N-tile n = (token n*4 + g/2, part g&1)
      ia[n] = init0 + (n * 4 + t) * seed_stride * 4;
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    const uint32_t n_live = (pcount + 3) >> 2;  // N-tiles that hold tokens

    // two adjacent blocks (kb, kb + 1; kb even) of both row slots against every live N-tile.
    // rec = shared address of the pair's first record in this warp's tile chunk.
    auto do_pair = [&](uint32_t rec, uint32_t kb) {
      uint32_t a0[4], a0h[4], a1[4], a1h[4];  // block kb: slots g / g+8; block kb+1: slots g / g+8
      float2 d0, d1;                          // {scale slot g, scale slot g+8} of each block
      if (DT == MER_DTYPE_Q4_0) {
        const uint4 w = lds128(rec + piece16);
        const uint2 sc = lds64(rec + 512 + g * 8);
        unpack_q4(w.x, a0), unpack_q4(w.y, a0h), unpack_q4(w.z, a1), unpack_q4(w.w, a1h);
        d0 = h2_to_f2(sc.x), d1 = h2_to_f2(sc.y);
      } else {
        const uint4 w0 = lds128(rec + piece16), w1 = lds128(rec + 544 + piece16);
        const uint32_t sc0 = lds32(rec + 512 + g * 4), sc1 = lds32(rec + 544 + 512 + g * 4);
        unpack_q8(w0.x, w0.y, a0), unpack_q8(w0.z, w0.w, a0h), unpack_q8(w1.x, w1.y, a1), unpack_q8(w1.z, w1.w, a1h);
        d0 = h2_to_f2(sc0), d1 = h2_to_f2(sc1);
      }
#pragma unroll
      for (int n = 0; n < NT; n++) {
        if (n > 0 && (uint32_t)n >= n_live) break;  // uniform
        const uint4 bf0 = lds128(fa[n] + kb * 64), bf1 = lds128(fa[n] + kb * 64 + 64);
        const uint2 sd = lds64(ia[n] + kb * 4);
        const float seed0 = __uint_as_float(sd.x), seed1 = __uint_as_float(sd.y);
        float c1[4], c2[4], e1[4], e2[4];
        mma_f16(c1, a0[0], a0h[0], a0[1], a0h[1], bf0.x, bf0.y, seed0, 0.0f, seed0, 0.0f);
        mma_f16(e1, a1[0], a1h[0], a1[1], a1h[1], bf1.x, bf1.y, seed1, 0.0f, seed1, 0.0f);
        mma_f16(c2, a0[2], a0h[2], a0[3], a0h[3], bf0.z, bf0.w, c1[0], c1[1], c1[2], c1[3]);
        mma_f16(e2, a1[2], a1h[2], a1[3], a1h[3], bf1.z, bf1.w, e1[0], e1[1], e1[2], e1[3]);
        acc[n][0] = fmaf(d0.x, c2[0], acc[n][0]);
        acc[n][1] = fmaf(d0.x, c2[1], acc[n][1]);
        acc[n][2] = fmaf(d0.y, c2[2], acc[n][2]);
        acc[n][3] = fmaf(d0.y, c2[3], acc[n][3]);
        acc[n][0] = fmaf(d1.x, e2[0], acc[n][0]);
        acc[n][1] = fmaf(d1.x, e2[1], acc[n][1]);
        acc[n][2] = fmaf(d1.y, e2[2], acc[n][2]);
        acc[n][3] = fmaf(d1.y, e2[3], acc[n][3]);
      }
    };

    for (uint32_t c0 = 0; c0 < kbn; c0 += p.kc) {
      const uint32_t nb = min(p.kc, kbn - c0);
      if (!dead && !mbar_wait(&full[stage], round & 1)) dead = true;
      dead = __any_sync(0xffffffffu, dead);
      if (!dead) {
        constexpr uint32_t PAIR_BYTES = 2 * 16 * BB;  // 576 (Q4_0) / 1088 (Q8_0)
        const uint32_t np = nb >> 1;                  // block pairs in this chunk
        uint32_t rec = stage0 + stage * stage_bytes;
        uint32_t kb = c0;
        // two pairs per iteration keep independent MMA chains in flight
#pragma unroll 1
        for (uint32_t pr = 0; pr < np; pr += 2, rec += 2 * PAIR_BYTES, kb += 4) {
          do_pair(rec, kb);
          if (pr + 1 < np) do_pair(rec + PAIR_BYTES, kb + 2);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == p.n_stages) stage = 0, round++;
    }

    // ---- item epilogue: this warp's tile is complete over the item's K range; write it out
    if (!dead) {
      const uint32_t ptile = CONSUMER_WARPS * tile + warp;  // packed tile index within the phase's region
#pragma unroll
      for (int n = 0; n < NT; n++) {
        if (n > 0 && (uint32_t)n >= n_live) break;
        const uint32_t tok = n * 4 + t;
        const bool valid = tok < pcount;
        const uint32_t pair = valid ? s_pair[tok] : 0;
        const float un = valid ? s_un[tok] : 0.0f;
        const float r_lo = (acc[n][0] + acc[n][1]) * un, r_hi = (acc[n][2] + acc[n][3]) * un;  // row slots g and g+8
        if (split_gate_up) {
          // K is split across CTAs: leave gate and up partial sums; k_h_finalize adds them and applies SiLU
          if (valid) {
            float *gp = p.out + ((size_t)ks * n_pairs + pair) * 2 * d.F + ptile * 8 + g;
            gp[0] = r_lo;
            gp[d.F] = r_hi;
          }
        } else if (p.phase == 0) {
          // slots 0..7 of a gate/up tile are gate rows, slots 8..15 the matching up rows
          float gate = r_lo;
          if (d.swiglu_limit > 0.0f && isfinite(d.swiglu_limit) && gate == gate)
            gate = fminf(fmaxf(gate, -d.swiglu_limit), d.swiglu_limit);
          const float hval = __fdividef(gate, 1.0f + __expf(-gate)) * r_hi;
          if (valid) p.out[(size_t)pair * d.F + ptile * 8 + g] = hval;
          const float ah = fabsf(hval);
          uint32_t bits = !valid ? 0u : (ah != ah) ? 0x7fc00000u : __float_as_uint(ah);
          // max over the 8 rows held by the lanes that share t (all lanes take part in the shuffles)
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
          if (valid && g == 0) atomicMax(d.amax + pair, bits);
        } else if (valid) {
          float *yo = p.out + ((size_t)ks * n_pairs + pair) * d.D + ptile * 16;
          yo[g] = r_lo;
          yo[g + 8] = r_hi;
        }
      }
    }
  }
  if (dead && lane == 0) {
    *(volatile uint32_t *)s_abort = 1;
    atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
  }
}

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Grid-wide barrier of a cooperative launch: every CTA arrives once; waits are bounded by wall-clock time.
__device__ bool grid_barrier(uint32_t *counter, uint32_t *status) {
  __shared__ int s_ok;
  __syncthreads();  // this CTA's stores are issued
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    const uint64_t t0 = global_ns();
    bool ok = true;
    while (*(volatile uint32_t *)counter < gridDim.x) {
      __nanosleep(64);
      if (global_ns() - t0 > 2000000000ull) {
        ok = false;
        break;
      }
    }
    __threadfence();
    if (!ok) atomicOr(status, MER_DEVSTAT_TIMEOUT);
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

// After all CTAs have left their partial sums: the same arithmetic as k_h_finalize / k_combine, spread over the grid.
__device__ void ffn_stream_tail(const StreamParams &p) {
  const MoeDispatch &d = p.d;
  if (!grid_barrier(p.grid_counter, d.status)) return;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t P = d.n_tokens * d.slots;
  if (p.tail == TAIL_FINALIZE) {
    const float *parts = p.out;
    const uint32_t F = d.F, fchunks = (F + 127) / 128;
    const uint32_t gw = blockIdx.x * (THREADS / 32) + warp, nw = gridDim.x * (THREADS / 32);
#pragma unroll 1
    for (uint32_t u = gw; u < P * fchunks; u += nw) {  // a warp: 128 consecutive values of one pair's row
      const uint32_t pair = u / fchunks, f0 = (u % fchunks) * 128 + lane * 4;
      float mx = 0.0f;
      if (f0 < F) {
        float4 g = make_float4(0, 0, 0, 0), up = make_float4(0, 0, 0, 0);
#pragma unroll 1
        for (uint32_t k = 0; k < p.n_ksplit; k++) {
          const float *base = parts + ((size_t)k * P + pair) * 2 * F;
          const float4 a = __ldcg(reinterpret_cast<const float4 *>(base + f0)), b = __ldcg(reinterpret_cast<const float4 *>(base + F + f0));
          g.x += a.x, g.y += a.y, g.z += a.z, g.w += a.w;
          up.x += b.x, up.y += b.y, up.z += b.z, up.w += b.w;
        }
        const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {up.x, up.y, up.z, up.w};
        float hv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float gate = gv[i];
          if (d.swiglu_limit > 0.0f && isfinite(d.swiglu_limit) && gate == gate) gate = fminf(fmaxf(gate, -d.swiglu_limit), d.swiglu_limit);
          hv[i] = __fdividef(gate, 1.0f + __expf(-gate)) * uv[i];
          mx = nan_max(mx, fabsf(hv[i]));
        }
        *reinterpret_cast<float4 *>(d.h + (size_t)pair * F + f0) = make_float4(hv[0], hv[1], hv[2], hv[3]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) atomicMax(d.amax + pair, (mx != mx) ? 0x7fc00000u : __float_as_uint(mx));
    }
  } else if (p.tail == TAIL_COMBINE) {
    const uint32_t D4 = d.D / 4;
    const float4 *yp = reinterpret_cast<const float4 *>(p.n_ksplit > 1 ? p.out : d.y);
    const size_t part4 = (size_t)P * D4;
#pragma unroll 1
    for (uint32_t e = blockIdx.x * THREADS + threadIdx.x; e < d.n_tokens * D4; e += gridDim.x * THREADS) {
      const uint32_t token = e / D4, i4 = e % D4;
      float4 acc = make_float4(0, 0, 0, 0);
      auto add_residual = [&]() {  // hidden + routed sum, before the shared expert's slot (model.rs:2742-2763)
        const float4 r = __ldg(reinterpret_cast<const float4 *>(d.residual) + (size_t)token * D4 + i4);
        acc.x = __fadd_rn(r.x, acc.x), acc.y = __fadd_rn(r.y, acc.y), acc.z = __fadd_rn(r.z, acc.z), acc.w = __fadd_rn(r.w, acc.w);
      };
#pragma unroll 1
      for (uint32_t sl = 0; sl < d.slots; sl++) {
        if (d.residual && sl == d.routed_slots) add_residual();
        const size_t pr = (size_t)token * d.slots + sl;
        const float w = d.pair_weight[pr];
        if (d.pair_expert[pr] == MER_NONE || w == 0.0f) continue;
        float4 yv = __ldcg(yp + pr * D4 + i4);
#pragma unroll 1
        for (uint32_t k = 1; k < p.n_ksplit; k++) {
          const float4 t = __ldcg(yp + (size_t)k * part4 + pr * D4 + i4);
          yv.x += t.x, yv.y += t.y, yv.z += t.z, yv.w += t.w;
        }
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, yv.x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, yv.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, yv.z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, yv.w));
      }
      if (d.residual && d.routed_slots >= d.slots) add_residual();
      reinterpret_cast<float4 *>(d.out)[(size_t)token * D4 + i4] = acc;
    }
  } else if (p.tail == TAIL_REDUCE) {
    // per-pair outputs of the pairs that ran here (under expert parallelism: a fraction of all pairs)
    const uint32_t D4 = d.D / 4, n_here = d.offsets[d.n_groups];
    const float4 *yp = reinterpret_cast<const float4 *>(p.out);
    const size_t part4 = (size_t)P * D4;
#pragma unroll 1
    for (uint32_t e = blockIdx.x * THREADS + threadIdx.x; e < n_here * D4; e += gridDim.x * THREADS) {
      const size_t pr = d.perm[e / D4];
      const uint32_t i4 = e % D4;
      float4 yv = __ldcg(yp + pr * D4 + i4);
#pragma unroll 1
      for (uint32_t k = 1; k < p.n_ksplit; k++) {
        const float4 t = __ldcg(yp + (size_t)k * part4 + pr * D4 + i4);
        yv.x += t.x, yv.y += t.y, yv.z += t.z, yv.w += t.w;
      }
      reinterpret_cast<float4 *>(d.y)[pr * D4 + i4] = yv;
    }
  }
}

template <int DT, int NT>
__global__ void __launch_bounds__(THREADS, 1) k_ffn_stream(StreamParams p) {
  ffn_stream_body<DT, NT>(p);
  if (p.tail != TAIL_NONE) ffn_stream_tail(p);
}

// h = SiLU(clamp(sum of gate partials)) * (sum of up partials), partials added in K-split order, plus the
// row maximum of |h| that the down phase scales its activations by.  grid = (pairs, ceil(F / 1024)).
__global__ void __launch_bounds__(256) k_h_finalize(const float *__restrict__ parts, uint32_t n_ksplit, uint32_t n_pairs, uint32_t F,
                                                    float limit, float *__restrict__ h, uint32_t *__restrict__ amax) {
  const uint32_t pair = blockIdx.x;
  const uint32_t f0 = blockIdx.y * 1024 + threadIdx.x * 4;
  float mx = 0.0f;
  if (f0 < F) {
    float4 g = make_float4(0, 0, 0, 0), u = make_float4(0, 0, 0, 0);
#pragma unroll 4
    for (uint32_t k = 0; k < n_ksplit; k++) {
      const float *base = parts + ((size_t)k * n_pairs + pair) * 2 * F;
      const float4 a = *reinterpret_cast<const float4 *>(base + f0), b = *reinterpret_cast<const float4 *>(base + F + f0);
      g.x += a.x, g.y += a.y, g.z += a.z, g.w += a.w;
      u.x += b.x, u.y += b.y, u.z += b.z, u.w += b.w;
    }
    float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w}, hv[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float gate = gv[i];
      if (limit > 0.0f && isfinite(limit) && gate == gate) gate = fminf(fmaxf(gate, -limit), limit);
      hv[i] = __fdividef(gate, 1.0f + __expf(-gate)) * uv[i];
      mx = nan_max(mx, fabsf(hv[i]));
    }
    *reinterpret_cast<float4 *>(h + (size_t)pair * F + f0) = make_float4(hv[0], hv[1], hv[2], hv[3]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = nan_max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) atomicMax(amax + pair, (mx != mx) ? 0x7fc00000u : __float_as_uint(mx));
}

__global__ void k_reduce_ksplit(const float *__restrict__ part, float *__restrict__ y, size_t n, uint32_t n_ksplit) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = part[i];
  for (uint32_t k = 1; k < n_ksplit; k++) acc += part[(size_t)k * n + i];
  y[i] = acc;
}

struct Plan {
  uint32_t nt, kc, n_stages, chunk_stride, frag_stride, kb_split, n_ksplit, frag_cols;
  size_t smem;
};

constexpr size_t SMEM_LIMIT = 226 * 1024;  // 227 KB per CTA less the kernel's static shared memory
constexpr uint32_t MAX_KSPLIT = 64;

// Shapes one phase.  An item is 16 tiles (one per warp) over one K split.
//  * K split: the largest split (whole K, K/2, K/4, ... in multiples of 8 blocks, at least 16 blocks)
//    that still leaves about eight items per CTA for the expected number of active experts, within
//    `max_ksplit` (what the partial-sum scratch can hold);
//  * a stage holds 4 block pairs per warp if at least three stages then fit, else 2, else 1;
//  * fragment arrays are sized by the most tokens any group can hold in this dispatch.
Plan make_plan(int dtype, uint32_t kb_total, uint32_t packed_tiles, uint32_t nt, uint32_t max_group_tokens,
               uint32_t active_groups, int n_ctas, uint32_t max_ksplit) {
  const uint32_t bb = dtype == MER_DTYPE_Q4_0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES;
  const uint32_t tp = 4 * nt;
  Plan pl{};
  if (packed_tiles % CONSUMER_WARPS) return pl;
  const uint64_t items_per_split = (uint64_t)active_groups * (packed_tiles / CONSUMER_WARPS);
  uint32_t n_ksplit = 1, kb_split = kb_total;
  if (max_ksplit > MAX_KSPLIT) max_ksplit = MAX_KSPLIT;
  // Pick the K split that minimises the busiest CTA's estimated time, in units of one block step (16 tiles x one
  // block of K).  A CTA gets ceil(items / CTAs) items of kb_split block steps each, pays a fixed cost per item
  // (epilogue) and one activation-fragment rebuild per (pass, K split) unit its contiguous range touches; a rebuild
  // measures about 4 us, i.e. ~10 block steps of Q8_0 or ~20 of Q4_0 at the rate one SM streams.
  {
    const double rebuild = dtype == MER_DTYPE_Q4_0 ? 20.0 : 10.0, per_item = 2.0;
    const uint32_t tile_groups = packed_tiles / CONSUMER_WARPS;
    double best = 1e30;
    uint32_t seen_split = 0;
    for (uint32_t n = 1; n <= max_ksplit; n++) {
      uint32_t split = ((kb_total + n - 1) / n + 7) / 8 * 8;
      if (split > kb_total) split = kb_total;
      if (n > 1 && split < 16) break;
      if (split == seen_split) continue;  // same split as a smaller n
      seen_split = split;
      const uint32_t nn = (kb_total + split - 1) / split;
      if (nn > max_ksplit) continue;
      const uint64_t items = items_per_split * nn;
      const double per_cta = (double)((items + n_ctas - 1) / n_ctas);
      const double units = (per_cta - 1.0) / tile_groups + 1.0;
      const double cost = per_cta * (split + per_item) + units * rebuild + 0.5 * nn;  // last term: partial sums, and ties go to fewer splits
      if (cost < best) best = cost, kb_split = split, n_ksplit = nn;
    }
  }
  // shared memory also bounds a split: the fragment arrays of one split must leave room for the ring
  for (;;) {
    const uint32_t frag_cols = 2 * (max_group_tokens < tp ? max_group_tokens : tp);
    const uint32_t frag_stride = kb_split * 64 + 64;
    const size_t fixed = HEADER_BYTES + (size_t)(kb_split + 2) * tp * 4 + 128 + (size_t)frag_cols * frag_stride;
    if (fixed < SMEM_LIMIT) {
      const size_t avail = SMEM_LIMIT - fixed;
      for (uint32_t ppw = 4; ppw >= 1; ppw >>= 1) {
        uint32_t kc = 2 * ppw;
        if (kc > kb_split) kc = kb_split;
        const uint32_t chunk = kc * 16 * bb;
        const size_t stage = (size_t)CONSUMER_WARPS * chunk;
        uint32_t n_stages = (uint32_t)(avail / stage);
        if (n_stages > 8) n_stages = 8;
        if (n_stages >= 3 || (ppw == 1 && n_stages >= 2)) {
          pl = Plan{nt, kc, n_stages, chunk, frag_stride, kb_split, n_ksplit, frag_cols, fixed + n_stages * stage};
          return pl;
        }
      }
    }
    // does not fit: halve the split (more partial sums) if the scratch allows
    const uint32_t next_split = ((kb_split + 1) / 2 + 7) / 8 * 8;
    if (next_split >= kb_split || next_split < 8) return pl;
    const uint32_t next_n = (kb_total + next_split - 1) / next_split;
    if (next_n > max_ksplit) return pl;
    kb_split = next_split, n_ksplit = next_n;
  }
}

struct ScratchLayout {
  size_t amax, npass, pgroup, pstart, pcount, bounds, parts, parts_bytes, total;
};

// `parts` holds the K-split partial sums of whichever phase is running: gate/up partials
// [n_ksplit][P][2][F], then (after k_h_finalize has consumed them) down partials [n_ksplit][P][D].
ScratchLayout scratch_layout(uint32_t max_pairs, uint32_t D, uint32_t F) {
  ScratchLayout L{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += (bytes + 255) & ~(size_t)255;
    return o;
  };
  L.amax = take((size_t)max_pairs * 4);
  L.npass = take(256);
  L.pgroup = take((size_t)max_pairs * 4);
  L.pstart = take((size_t)max_pairs * 4);
  L.pcount = take((size_t)max_pairs * 4);
  L.bounds = take((size_t)2 * MER_MAX_CTAS1 * 4);
  // room for 8 splits of the largest batch, but never less than 64 splits of an 8-pair dispatch, capped at 1 GiB
  const size_t per_pair = (size_t)(2 * F > D ? 2 * F : D) * 4;
  size_t want = (size_t)8 * max_pairs * per_pair;
  const size_t small = (size_t)MAX_KSPLIT * 8 * per_pair;
  if (want < small) want = small;
  if (want > ((size_t)1 << 30)) want = (size_t)1 << 30;
  if (want < (size_t)max_pairs * per_pair) want = (size_t)max_pairs * per_pair;
  L.parts_bytes = want;
  L.parts = take(want);
  L.total = off;
  return L;
}

template <int DT>
cudaError_t launch_phase(const StreamParams &p, uint32_t nt, size_t smem, int grid, cudaStream_t s) {
  void (*kern)(StreamParams) = nt == 2 ? k_ffn_stream<DT, 2> : k_ffn_stream<DT, 1>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (p.tail != TAIL_NONE) {
    // the tail waits for every CTA of the grid: a cooperative launch guarantees that they are all resident
    StreamParams q = p;
    void *args[] = {&q};
    return cudaLaunchCooperativeKernel((const void *)kern, dim3(grid), dim3(THREADS), args, smem, s);
  }
  kern<<<grid, THREADS, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

bool stream_ffn_supported(int dtype, uint32_t D, uint32_t F) {
  if (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0) return false;
  if (D == 0 || F == 0 || D % 256 != 0 || F % 256 != 0) return false;  // 16-byte aligned rows, whole 16-tile groups
  Plan a = make_plan(dtype, D / 32, F / 8, 1, 4, 1, 148, MAX_KSPLIT), b = make_plan(dtype, F / 32, D / 16, 1, 4, 1, 148, MAX_KSPLIT);
  return a.n_stages >= 2 && b.n_stages >= 2;
}

size_t stream_ffn_scratch_bytes(uint32_t max_pairs, uint32_t D, uint32_t F) { return scratch_layout(max_pairs, D, F).total; }

namespace {
struct Plans {
  uint32_t nt;
  Plan gate_up, down;
};
// Token-pass width and both phase plans of a dispatch (pure function of its shape and hints).
Plans plan_dispatch(const MoeDispatch &d, int sm_count) {
  const uint32_t P = d.n_tokens * d.slots;
  const ScratchLayout L = scratch_layout(d.scratch_pairs, d.D, d.F);
  const uint32_t mgt = d.max_group_tokens ? d.max_group_tokens : P, act = d.active_groups_hint ? d.active_groups_hint : 1;
  // how many K splits of partial sums the scratch can hold for this dispatch
  const uint32_t cap_gu = (uint32_t)std::min<size_t>(MAX_KSPLIT, L.parts_bytes / ((size_t)P * 2 * d.F * 4));
  const uint32_t cap_dn = (uint32_t)std::min<size_t>(MAX_KSPLIT, L.parts_bytes / ((size_t)P * d.D * 4));
  Plans pl{};
  pl.nt = mgt > 4 ? 2u : 1u;
  pl.gate_up = make_plan(d.dtype, d.D / 32, d.F / 8, pl.nt, mgt, act, sm_count, cap_gu);
  pl.down = make_plan(d.dtype, d.F / 32, d.D / 16, pl.nt, mgt, act, sm_count, cap_dn);
  if (pl.nt == 2 && (pl.gate_up.n_stages < 3 || pl.down.n_stages < 3)) {  // eight tokens per pass do not fit: four per pass
    pl.nt = 1;
    pl.gate_up = make_plan(d.dtype, d.D / 32, d.F / 8, pl.nt, mgt, act, sm_count, cap_gu);
    pl.down = make_plan(d.dtype, d.F / 32, d.D / 16, pl.nt, mgt, act, sm_count, cap_dn);
  }
  return pl;
}
}  // namespace

void stream_bind(MoeDispatch &d, void *scratch, int sm_count) {
  if (sm_count > MER_MAX_CTAS1 - 1) sm_count = MER_MAX_CTAS1 - 1;
  uint8_t *base = static_cast<uint8_t *>(scratch);
  const ScratchLayout L = scratch_layout(d.scratch_pairs, d.D, d.F);
  d.n_passes = reinterpret_cast<uint32_t *>(base + L.npass);
  d.pass_group = reinterpret_cast<uint32_t *>(base + L.pgroup);
  d.pass_start = reinterpret_cast<uint32_t *>(base + L.pstart);
  d.pass_count = reinterpret_cast<uint32_t *>(base + L.pcount);
  d.amax = reinterpret_cast<uint32_t *>(base + L.amax);
  const Plans pl = plan_dispatch(d, sm_count);
  d.tokens_per_pass = 4 * pl.nt;
  d.item_bounds = reinterpret_cast<uint32_t *>(base + L.bounds);
  d.items_per_pass[0] = pl.gate_up.n_ksplit * (d.F / 8 / CONSUMER_WARPS);
  d.items_per_pass[1] = pl.down.n_ksplit * (d.D / 16 / CONSUMER_WARPS);
  d.n_ctas = (uint32_t)sm_count;
}

cudaError_t launch_ffn_stream(MoeDispatch &d, void *scratch, int sm_count, cudaStream_t s, int *launches, cudaEvent_t ev_mid) {
  if (sm_count > MER_MAX_CTAS1 - 1) sm_count = MER_MAX_CTAS1 - 1;  // the per-CTA work split holds at most 256 ranges
  const uint32_t P = d.n_tokens * d.slots;
  uint8_t *base = static_cast<uint8_t *>(scratch);
  const ScratchLayout L = scratch_layout(d.scratch_pairs, d.D, d.F);
  const Plans pl = plan_dispatch(d, sm_count);
  const Plan &pg = pl.gate_up, &pd = pl.down;
  const uint32_t nt = pl.nt;
  if (pg.n_stages < 2 || pd.n_stages < 2 || !d.pass_group || d.tokens_per_pass != 4 * nt) return cudaErrorInvalidConfiguration;
  float *parts = reinterpret_cast<float *>(base + L.parts);
  cudaError_t e;
  int n = 0;
  StreamParams p{};
  p.d = d;
  // phase 0: gate/up, activations = x by token
  p.phase = 0, p.act = d.x, p.act_per_pair = 0;
  p.rows = d.F, p.kb_total = d.D / 32, p.kb_split = pg.kb_split, p.n_ksplit = pg.n_ksplit, p.kc = pg.kc;
  p.n_stages = pg.n_stages, p.chunk_stride = pg.chunk_stride, p.frag_stride = pg.frag_stride, p.frag_cols = pg.frag_cols;
  p.out = pg.n_ksplit > 1 ? parts : d.h;
  auto launch = [&](size_t smem) {
    return d.dtype == MER_DTYPE_Q4_0 ? launch_phase<MER_DTYPE_Q4_0>(p, nt, smem, sm_count, s)
                                     : launch_phase<MER_DTYPE_Q8_0>(p, nt, smem, sm_count, s);
  };
  // K split: the partial sums are finished (SiLU(gate) * up, row maxima) by the same launch after a grid-wide barrier;
  // where a cooperative launch is refused, by a second kernel
  p.tail = pg.n_ksplit > 1 ? TAIL_FINALIZE : TAIL_NONE, p.grid_counter = d.n_passes + 1;
  e = launch(pg.smem);
  if (e != cudaSuccess && p.tail != TAIL_NONE) {
    cudaGetLastError();
    p.tail = TAIL_NONE;
    e = launch(pg.smem);
    if (e == cudaSuccess) {
      k_h_finalize<<<dim3(P, (d.F + 1023) / 1024), 256, 0, s>>>(parts, pg.n_ksplit, P, d.F, d.swiglu_limit, d.h, d.amax);
      e = cudaGetLastError();
      n++;
    }
  }
  if (e != cudaSuccess) return e;
  n++;
  if (ev_mid) cudaEventRecord(ev_mid, s);
  // phase 1: down, activations = h by pair, scaled by the row maxima collected above
  p.phase = 1, p.act = d.h, p.act_per_pair = 1;
  p.rows = d.D, p.kb_total = d.F / 32, p.kb_split = pd.kb_split, p.n_ksplit = pd.n_ksplit, p.kc = pd.kc;
  p.n_stages = pd.n_stages, p.chunk_stride = pd.chunk_stride, p.frag_stride = pd.frag_stride, p.frag_cols = pd.frag_cols;
  p.out = pd.n_ksplit > 1 ? parts : d.y;
  // the weighted combine of the layer rides on the same launch when the caller asked for it
  p.tail = d.fuse_combine ? TAIL_COMBINE : (d.fuse_reduce && pd.n_ksplit > 1) ? TAIL_REDUCE : TAIL_NONE;
  p.grid_counter = d.n_passes + 2;
  d.combined = 0;
  bool reduced = false;
  e = launch(pd.smem);
  if (e == cudaSuccess && p.tail == TAIL_COMBINE) d.combined = 1;
  if (e == cudaSuccess && p.tail == TAIL_REDUCE) reduced = true;
  if (e != cudaSuccess && p.tail != TAIL_NONE) {
    cudaGetLastError();
    p.tail = TAIL_NONE;
    e = launch(pd.smem);
  }
  if (e != cudaSuccess) return e;
  n++;
  // the per-pair outputs are the K-split partials until somebody adds them: the combine kernel does, or
  // launch_reduce_parts for entry points that return per-pair outputs
  d.y_parts = (pd.n_ksplit > 1 && !reduced) ? parts : nullptr;
  d.y_nparts = pd.n_ksplit;
  if (launches) *launches += n;
  return cudaSuccess;
}

cudaError_t launch_reduce_parts(const MoeDispatch &d, cudaStream_t s, int *launches) {
  if (!d.y_parts || d.y_nparts <= 1) return cudaSuccess;
  size_t cnt = (size_t)d.n_tokens * d.slots * d.D;
  k_reduce_ksplit<<<(unsigned)((cnt + 255) / 256), 256, 0, s>>>(d.y_parts, d.y, cnt, d.y_nparts);
  if (launches) (*launches)++;
  return cudaGetLastError();
}
