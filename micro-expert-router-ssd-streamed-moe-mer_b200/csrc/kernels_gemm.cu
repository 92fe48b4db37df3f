// Grouped expert FFN for token groups of a dozen tokens and more (prefill, expert-parallel decode):
// tcgen05 tensor-core GEMM per (expert, 128 weight rows, up to 128 tokens) with TMEM accumulators.
//
//   D[128 weight rows x N tokens] += A[128 x 32] * B[N x 32]^T      per 32-value block of K
//
//   * A never touches shared memory as an operand: the packed Q4_0 / Q8_0 tile chunks of layout.cuh
//     are streamed global -> shared by bulk async copies, eight warps dequantise them block by block into
//     two f16 operands, hi = f16(d*q) and lo = d*q - hi (exact: an 11-bit scale times an 8-bit integer
//     has at most 19 significant bits), and store them straight into TENSOR MEMORY (tcgen05.st; a thread
//     owns one weight row), from where the MMA reads its A operand.  Eight A stages live in TMEM beside
//     the two accumulators.
//   * B is the activation tile as f16 hi + lo parts (22 significant bits after an exact power-of-two
//     per-row scaling), laid out in the K-major no-swizzle core-matrix order by k_gemm_act_image (per core-matrix
//     column of K the hi pieces of the pass's rows, then the lo pieces; as wide as the pass, not as the widest one)
//     and fetched with one bulk copy per 64 values of K, two per stage, into a two-stage shared-memory ring.
//   * Three products per 16 values of K (hi*hi, hi*lo, lo*hi; lo*lo is below fp32 resolution) accumulate
//     in fp32 in TMEM, so the result matches the fp32 reference to ~1e-4 of the output RMS instead of f16's 2e-3.
//     A group of at most 64 tokens issues them as two instructions: W_hi * [x_hi | x_lo] with twice the width
//     (two column sets of the accumulator, added in the epilogue) and W_lo * x_hi.
//   * Warp roles: 0 = producer of the activation stages, 1 = MMA issuer (one elected lane issues predicated
//     instructions; every operand is computed in uniform registers) and TMEM owner,
//     2..9 = epilogue (four warps per accumulator buffer: tcgen05.ld, un-scaling, SiLU(gate)*up or plain store; two
//     buffers let the epilogue of one item overlap the MMAs of the next two),
//     10..17 = dequantisers (a warp reaches the 32 TMEM lanes of its quarter; the two warps of a quarter
//     take alternate blocks), 18 = producer of the weight stages (lanes 0..7 copy one packed tile each).
// Every wait is bounded; on expiry the CTA latches MER_DEVSTAT_TIMEOUT, stops issuing work, waits
// (bounded) for its copies and MMAs in flight, frees its TMEM and returns.
#include <cuda_fp16.h>

#include <type_traits>

#include "../../include/mer_b200.h"
#include "kernels.h"
#include "layout.cuh"
#include "ptx.cuh"

namespace {

constexpr int G_WARPS = 19, G_THREADS = G_WARPS * 32;
constexpr int W_PRODUCER = 0, W_MMA = 1, W_EPI0 = 2, W_DQ0 = 10, W_WEIGHTS = 18;
constexpr int EPI_WARPS = 4, DQ_WARPS = 8;  // EPI_WARPS per accumulator
constexpr uint32_t RAW_BLOCKS = 4;       // blocks of K per weight stage (per packed tile: one bulk copy)
constexpr uint32_t G_HEADER = 5120;      // mbarriers, TMEM base, and from byte 1024 the epilogue groups' per-pass tables (2 KB each)
constexpr uint32_t TMEM_COLS = 512;      // [0, 256): two accumulator buffers of up to 128 columns; [256, 512): A stages
constexpr uint32_t TMEM_A0 = 256, A_STAGES = 8, A_STAGE_COLS = 32;  // a stage = one block: 16 columns hi + 16 columns lo
constexpr uint32_t MAX_RING = 8;
// The MMA issuer synchronises with its producers once per GROUP blocks of K: it waits for a whole group of A stages
// and for the group's activation stage (both complete the same barrier, a_full: eight dequantiser arrivals, the
// producer's expect-tx arrival and the bytes of its two copies), issues the group's MMAs and commits done[], which releases
// both.  A waiter is never two phases behind a done[] barrier: the issuer leads its producers by at most two groups.
constexpr uint32_t GROUP = 4, DONE_RING = 8;
static_assert(GROUP == RAW_BLOCKS, "a weight stage holds exactly one group of blocks");
constexpr float POW2_SCALE_TARGET = 9;   // activations are scaled so that the row maximum lies in [256, 512)

struct GemmParams {
  MoeDispatch d;
  int phase;               // 0 = gate/up (+SiLU*mul), 1 = down
  const uint8_t *act_img;  // [pass][K / 64] images of {hi, lo} activation tiles
  const float *unscale;    // [pass][bn] 1 / scale of each token row
  uint32_t rows;           // F (gate/up) or D (down)
  uint32_t kb_total;       // 32-value blocks per weight row
  uint32_t bn;             // token columns per pass (16, 32, 64 or 128)
  uint32_t b_lbo;          // bn * 16 + 32: a chunk slot of the activation ring and of the image array holds 16 of these
  uint32_t n_raw, n_b;     // ring depths (weights, activations)
  float *out;              // phase 0: h [P x F]; phase 1: y [P x D]
};

// ------------------------------------------------------------------------------ tcgen05 PTX
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// One lane of a converged warp.  The MMA warp runs its loops and waits with all 32 lanes, so that every address and
// descriptor it computes is warp-uniform; the lane elected ONCE at the start issues the tcgen05.mma / tcgen05.commit
// instructions, as predicated instructions (no branch around them).  Measured on the way here: the whole loop inside
// `if (lane == 0)` cost ~85 cycles of issue time per MMA, an elect.sync + branch around every single MMA ~65, either
// of them more than a narrow MMA takes to execute.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ void tc_commit(uint32_t leader, uint64_t *bar) {
  asm volatile(
      "{\n .reg .pred q;\n setp.ne.b32 q, %1, 0;\n"
      " @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar)),
      "r"(leader)
      : "memory");
}
// K-major, no swizzle: 8-row x 16-byte core matrices; LBO = step between core matrices along K,
// SBO = step between 8-row groups.  Bits: start >> 4 [0,14), LBO >> 4 [16,30), SBO >> 4 [32,46), version 1 [46,48).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// f16 x f16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
// A operand read from tensor memory (lane = row, a 32-bit column = two consecutive values of K), B through a descriptor.
// Called by the whole (converged) warp; only the lane with leader != 0 issues.
__device__ __forceinline__ void tc_mma_ts(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 q, %5, 0;\n setp.ne.b32 p, %4, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts_acc(uint32_t leader, uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc) {
  tc_mma_ts(leader, d_tmem, a_tmem, b, idesc, 1u);
}
// 32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
      "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
      "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// Two integers held as the f16 values 1024 + b (b in the low mantissa bits) -> hi = f16(d * (b - zp)),
// lo = d * (b - zp) - hi.  Every step is exact except the rounding that defines hi.
__device__ __forceinline__ void dq2(uint32_t biased, __half2 zp1024, __half2 d2, uint32_t &hi, uint32_t &lo) {
  const __half2 q = __hsub2(bits_h2(biased), zp1024);
  const __half2 h = __hmul2(d2, q);
  hi = h2_bits(h);
  lo = h2_bits(__hfma2(d2, q, __hneg2(h)));
}

// Token columns a pass occupies in its activation image and in the accumulator: its count rounded up to 16, at most bn.
__host__ __device__ constexpr uint32_t pass_width(uint32_t bn, uint32_t count) {
  const uint32_t w = (count + 15u) & ~15u;
  return w < bn ? w : bn;
}
// Bytes between two K core-matrix columns of a pass's image: the hi rows, then the lo rows, then a 32-byte skew.
__host__ __device__ constexpr uint32_t pass_lbo(uint32_t width) { return 2u * width * 16u + 32u; }
// The passes of a group of at most MERGE_TOKENS tokens (always a single pass) multiply W_hi by [x_hi | x_lo] in one
// instruction of twice the pass's width (two column sets of one accumulator buffer, added in the epilogue): two
// instructions per 16 values of K instead of three.  The rule looks at the group, not at the pass, so that the order
// of a token's additions depends only on how many tokens its expert received, never on which pass it landed in:
// results stay bit-identical from run to run although large dispatches are grouped with atomics.
constexpr uint32_t MERGE_TOKENS = 64;

struct Ring {
  uint32_t stage = 0, round = 0, n;
  __device__ explicit Ring(uint32_t n_) : n(n_) {}
  __device__ void advance() {
    if (++stage == n) stage = 0, round++;
  }
};

template <int DT>
__global__ void __launch_bounds__(G_THREADS, 1) k_ffn_gemm(GemmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr uint32_t BB = DT == MER_DTYPE_Q4_0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES;
  constexpr uint32_t TILE_RAW = RAW_BLOCKS * 16 * BB;  // bytes of RAW_BLOCKS blocks of one packed tile (2304 / 4352)
  constexpr uint32_t RAW_BYTES = 8 * TILE_RAW;
  const MoeDispatch &d = p.d;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t m_tiles = p.rows / (p.phase == 0 ? 64u : 128u);  // 128-row MMA tiles (8 packed tiles each)
  const uint32_t n_chunks = p.kb_total / 2, n_groups = p.kb_total / GROUP;
  const uint32_t n_passes = *d.n_passes;
  // Items (pass, 128-row tile) are dealt round-robin: the CTAs running at any moment work on a dozen
  // neighbouring passes, so the activation images they all re-read stay in L2.
  const uint32_t n_items = n_passes * m_tiles;
  const uint32_t item_beg = blockIdx.x, item_step = gridDim.x;
  if (item_beg >= n_items) return;

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  uint64_t *raw_full = bars, *raw_empty = bars + 8, *a_full = bars + 16, *done = bars + 24,
           *acc_full = bars + 48, *acc_empty = bars + 50, *drain = bars + 52;
  uint32_t *s_tmem = reinterpret_cast<uint32_t *>(smem + 512);
  volatile uint32_t *s_abort = reinterpret_cast<volatile uint32_t *>(smem + 516);
  uint8_t *s_raw = smem + G_HEADER;
  uint8_t *s_b = s_raw + p.n_raw * RAW_BYTES;
  const uint32_t b_stage = 16 * p.b_lbo;  // ring slot and image slot of one 64-value chunk of K: what the widest pass needs

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < MAX_RING; s++) {
      mbar_init(&raw_full[s], 1), mbar_init(&raw_empty[s], DQ_WARPS);  // filled by the weight producer, left by every dequantiser warp
      mbar_init(&a_full[s], DQ_WARPS + 1), mbar_init(&done[s], 1);  // per group: every dequantiser warp + the activation producer
    }
    for (uint32_t s = 0; s < 2; s++) mbar_init(&acc_full[s], 1), mbar_init(&acc_empty[s], EPI_WARPS);
    mbar_init(drain, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == W_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The CTA owns all 512 columns of its SM's tensor memory, so the allocation starts at lane 0, column 0.  Using the
  // constant instead of the value read back lets every TMEM address below be computed in uniform registers: with the
  // loaded value each MMA took ~57 cycles to issue, with the constant ~35.  Should the allocator ever answer otherwise,
  // the kernel gives the columns back, latches the error status and leaves.
  constexpr uint32_t tmem_base = 0;
  if (*s_tmem != tmem_base) {
    if (warp == W_MMA) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*s_tmem), "r"(TMEM_COLS) : "memory");
    if (threadIdx.x == 0) atomicOr(p.d.status, MER_DEVSTAT_TIMEOUT);
    return;
  }

  const size_t proj_bytes = (size_t)d.D * d.F / 32 * BB;
  const size_t tile_bytes = (size_t)p.kb_total * 16 * BB;
  const size_t region = p.phase == 0 ? 0 : 2 * proj_bytes;
  auto expert_base = [&](uint32_t pass) -> const uint8_t * {
    const uint32_t eid = d.group_expert[d.pass_group[pass]];
    return eid < d.max_experts ? d.expert_ptr[eid] : nullptr;
  };
  bool ok = true;

  if (warp == W_PRODUCER) {
    // ------------------------------------------------------------------------ producer of the activation stages
    // one stage = one group of blocks of K of the pass's activation image: two chunks of 64 values, one bulk copy each.
    // A stage is free again when the MMAs of the group that used it have run: the issuer's done[] commit says so.
    Ring rb(p.n_b);
    uint32_t pg = 0;  // groups issued so far, over all items (the issuer counts the same way)
    for (uint32_t item = item_beg; item < n_items && ok; item += item_step) {
      const uint32_t pass = item / m_tiles;
      if (!expert_base(pass)) continue;
      const uint8_t *bsrc = p.act_img + (size_t)pass * n_chunks * b_stage;
      const uint32_t bytes = 8 * pass_lbo(pass_width(p.bn, __ldg(d.pass_count + pass)));  // a narrow pass has a small image
      for (uint32_t gi = 0; gi < n_groups && ok; gi++, pg++) {
        if (pg >= p.n_b) {
          const uint32_t sp = pg - p.n_b;
          ok = mbar_wait(&done[sp % DONE_RING], (sp / DONE_RING) & 1);
        }
        if (*s_abort) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(&a_full[rb.stage], 2 * bytes);  // stage = group parity: the barrier the group's A stages complete too
        __syncwarp();
        if (lane < 2)
          bulk_g2s(s_b + ((size_t)rb.stage * 2 + lane) * b_stage, bsrc + ((size_t)gi * 2 + lane) * b_stage, bytes, &a_full[rb.stage]);
        rb.advance();
      }
    }
    if (!ok) {
      if (lane == 0) *s_abort = 1, atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
      // copies already in flight get a bounded chance to land before the CTA's shared memory is released
      for (uint32_t s = 0; s < p.n_b; s++) (void)mbar_wait(&a_full[s], 0), (void)mbar_wait(&a_full[s], 1);
    }
  } else if (warp == W_MMA) {
    // -------------------------------------------------------------------------- MMA issuer
    // The whole warp walks the loops and waits (every value it computes is warp-uniform); the elected lane issues.
    // one step = one 32-value block of K: two instructions of 16 values for each of the three operand pairings
    Ring rb(p.n_b);
    const uint32_t leader = elect_one();  // the warp is converged here; the same lane issues from now on
    uint32_t n_done = 0;  // items issued so far: accumulator buffer = n_done & 1, its k-th use has k = n_done >> 1
    uint32_t grp = 0;     // groups of GROUP blocks issued so far, over all items; A-stage half = grp & 1
    // B descriptors differ only in their start-address field: one base, then 64-bit adds of (byte offset >> 4).
    // (The ring lies well inside the 256 KB the 14-bit field spans, so the adds never carry out of it.)
    const uint32_t stage16 = b_stage >> 4;
    // One item's K loop for a pass of WIDTH columns.  WIDTH is a template argument because everything the MMA instruction
    // takes (descriptors, TMEM addresses) must sit in uniform registers: values derived from kernel parameters and
    // constants are computed there directly, values derived from a loaded pass count had to be moved over per
    // instruction (measured: +25 % issue time).
    auto run_item = [&](auto width_tag, auto merged_tag) {
      constexpr uint32_t width = decltype(width_tag)::value, lbo = pass_lbo(width);
      constexpr bool merged = decltype(merged_tag)::value;
      constexpr uint32_t idesc = instr_desc(width), idesc2 = instr_desc(2 * width);
      constexpr uint32_t half16 = (4 * lbo) >> 4, j16 = (2 * lbo) >> 4, lo16 = width;  // the lo rows follow the hi rows: width * 16 bytes
      const uint64_t b_desc0 = smem_desc(smem_u32(s_b), lbo, 128);
      const uint32_t buf = n_done & 1, use = n_done >> 1;
      const uint32_t d_tmem = tmem_base + buf * 128;
      for (uint32_t st = 0; st < p.kb_total && ok; st += GROUP, grp++) {
        const uint32_t ag = grp & 1;
        if (st == 0 && use > 0) ok = mbar_wait(&acc_empty[buf], (use - 1) & 1);  // the buffer's previous item has been drained
        if (ok) ok = mbar_wait(&a_full[ag], (grp >> 1) & 1);
        if (*s_abort) ok = false;
        ok = __all_sync(0xffffffffu, ok);  // warp-uniform by construction; the vote also tells the compiler so
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (uint32_t b4 = 0; b4 < GROUP; b4++) {
          const uint32_t a_hi = tmem_base + TMEM_A0 + (ag * GROUP + b4) * A_STAGE_COLS, a_lo = a_hi + 16;
          const uint64_t b_blk = b_desc0 + (uint64_t)((rb.stage * 2 + (b4 >> 1)) * stage16 + (b4 & 1) * half16);
#pragma unroll
          for (uint32_t j = 0; j < 2; j++) {  // 16 values of K per instruction: 8 TMEM columns of A, two core-matrix columns of B
            const uint64_t dbh = b_blk + (uint64_t)(j * j16), dbl = dbh + lo16;
            const uint32_t acc = (b4 == 0 && j == 0) ? (st != 0) : 1u;  // the item's first MMA overwrites the accumulator
            if (merged) {
              tc_mma_ts(leader, d_tmem, a_hi + j * 8, dbh, idesc2, acc);  // columns [0, width): W_hi x_hi; [width, 2 width): W_hi x_lo
            } else {
              tc_mma_ts(leader, d_tmem, a_hi + j * 8, dbh, idesc, acc);
              tc_mma_ts_acc(leader, d_tmem, a_hi + j * 8, dbl, idesc);
            }
            tc_mma_ts_acc(leader, d_tmem, a_lo + j * 8, dbh, idesc);
          }
        }
        rb.advance();
        tc_commit(leader, &done[grp % DONE_RING]);  // frees the group's A stages and its activation stage
        if (st + GROUP >= p.kb_total) tc_commit(leader, &acc_full[buf]);
      }
      n_done++;
    };
    for (uint32_t item = item_beg; item < n_items && ok; item += item_step) {
      const uint32_t pass = item / m_tiles;
      if (!expert_base(pass)) continue;
      // the MMA is as wide as the pass has tokens (rounded up to 16 columns): a ragged last pass of a group costs
      // its share, not a full tile
      const uint32_t grp_id = __ldg(d.pass_group + pass);
      const bool merged = __ldg(d.offsets + grp_id + 1) - __ldg(d.offsets + grp_id) <= MERGE_TOKENS;
      const uint32_t w16 = pass_width(p.bn, __ldg(d.pass_count + pass)) >> 4;
      using T = std::true_type;
      using F = std::false_type;
      if (merged) {
        switch (w16) {
          case 1: run_item(std::integral_constant<uint32_t, 16>{}, T{}); break;
          case 2: run_item(std::integral_constant<uint32_t, 32>{}, T{}); break;
          case 3: run_item(std::integral_constant<uint32_t, 48>{}, T{}); break;
          default: run_item(std::integral_constant<uint32_t, 64>{}, T{}); break;
        }
      } else {
        switch (w16) {
          case 1: run_item(std::integral_constant<uint32_t, 16>{}, F{}); break;
          case 2: run_item(std::integral_constant<uint32_t, 32>{}, F{}); break;
          case 3: run_item(std::integral_constant<uint32_t, 48>{}, F{}); break;
          case 4: run_item(std::integral_constant<uint32_t, 64>{}, F{}); break;
          case 5: run_item(std::integral_constant<uint32_t, 80>{}, F{}); break;
          case 6: run_item(std::integral_constant<uint32_t, 96>{}, F{}); break;
          case 7: run_item(std::integral_constant<uint32_t, 112>{}, F{}); break;
          default: run_item(std::integral_constant<uint32_t, 128>{}, F{}); break;
        }
      }
    }
    if (!ok && lane == 0) *s_abort = 1, atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
    __syncwarp();
    // nothing may still be writing TMEM when it is freed
    tc_commit(leader, drain);
    (void)mbar_wait(drain, 0);
    __syncwarp();
  } else if (warp == W_WEIGHTS) {
    // ------------------------------------------------------------------------ producer of the weight stages
    // one stage = one group of RAW_BLOCKS blocks of the item's eight packed tiles; lane m < 8 copies tile m's chunk
    Ring raw(p.n_raw);
    for (uint32_t item = item_beg; item < n_items && ok; item += item_step) {
      const uint8_t *base = expert_base(item / m_tiles);
      if (!base) continue;
      const uint8_t *src = base + region + (size_t)((item % m_tiles) * 8 + (lane & 7)) * tile_bytes;
      for (uint32_t gi = 0; gi < n_groups && ok; gi++) {
        if (raw.round > 0) ok = mbar_wait(&raw_empty[raw.stage], (raw.round - 1) & 1);  // every dequantiser warp has left the stage
        if (*s_abort) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(&raw_full[raw.stage], RAW_BYTES);
        __syncwarp();
        if (lane < 8) bulk_g2s(s_raw + raw.stage * RAW_BYTES + lane * TILE_RAW, src + (size_t)gi * TILE_RAW, TILE_RAW, &raw_full[raw.stage]);
        raw.advance();
      }
    }
    if (!ok) {
      if (lane == 0) *s_abort = 1, atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
      // weight copies already in flight get a bounded chance to land before the CTA's shared memory is released
      for (uint32_t s = 0; s < p.n_raw; s++) (void)mbar_wait(&raw_full[s], 0), (void)mbar_wait(&raw_full[s], 1);
    }
  } else if (warp >= W_DQ0) {
    // ------------------------------------------------------------------------ dequantisers
    // A thread owns one weight row of the item: TMEM lane 32 * (warp % 4) + lane, i.e. packed tile 2q + lane / 16,
    // row slot lane % 16.  Per block it reads the row's 32 quants from the tile chunk in shared memory and stores
    // 16 columns of hi and 16 of lo.  The two warps of a quarter take alternate blocks.
    Ring raw(p.n_raw);
    uint32_t gblk = 0;  // blocks of K seen so far, over all items (A stage = gblk % A_STAGES)
    const uint32_t q = warp & 3, mine = (warp - W_DQ0) >> 2;
    const uint32_t T = 2 * q + (lane >> 4), g = lane & 7, half = (lane >> 3) & 1;
    const __half2 zp = DT == MER_DTYPE_Q4_0 ? __floats2half2_rn(1032.0f, 1032.0f) : __floats2half2_rn(1152.0f, 1152.0f);
    for (uint32_t item = item_beg; item < n_items && ok; item += item_step) {
      const uint32_t pass = item / m_tiles;
      if (!expert_base(pass)) continue;
      // one group (= one weight stage) at a time: this warp's two blocks of it, one wait on each side
      for (uint32_t gi = 0; gi < n_groups && ok; gi++, gblk += GROUP) {
        ok = mbar_wait(&raw_full[raw.stage], raw.round & 1);
        if (ok && gblk >= A_STAGES) {
          // the group's A stages were last read by the MMAs of group gblk / GROUP - 2
          const uint32_t sp = gblk / GROUP - A_STAGES / GROUP;
          ok = mbar_wait(&done[sp % DONE_RING], (sp / DONE_RING) & 1);
        }
        if (*s_abort) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tile_src = smem_u32(s_raw) + raw.stage * RAW_BYTES + T * TILE_RAW;
#pragma unroll
        for (uint32_t hb = 0; hb < GROUP / 2; hb++) {
          const uint32_t sub = mine + 2 * hb;  // block of the group handled here
          uint32_t v[32];  // [0, 16): hi, values (2c, 2c+1) of the block in column c; [16, 32): lo
          if (DT == MER_DTYPE_Q8_0) {
            const uint32_t src = tile_src + sub * 544;
            const uint32_t sc2 = lds32(src + 512 + g * 4);
            const __half2 dd = __half2half2(half ? __high2half(bits_h2(sc2)) : __low2half(bits_h2(sc2)));
#pragma unroll
            for (int t = 0; t < 4; t++) {  // values 8t .. 8t+7
              const uint2 w = lds64(src + packed_piece(g, t) * 16 + half * 8);
              const uint32_t w0 = w.x ^ 0x80808080u, w1 = w.y ^ 0x80808080u;
              dq2(__byte_perm(w0, 0x64646464u, 0x4140), zp, dd, v[4 * t + 0], v[16 + 4 * t + 0]);
              dq2(__byte_perm(w0, 0x64646464u, 0x4342), zp, dd, v[4 * t + 1], v[16 + 4 * t + 1]);
              dq2(__byte_perm(w1, 0x64646464u, 0x4140), zp, dd, v[4 * t + 2], v[16 + 4 * t + 2]);
              dq2(__byte_perm(w1, 0x64646464u, 0x4342), zp, dd, v[4 * t + 3], v[16 + 4 * t + 3]);
            }
          } else {
            // block-pair record: 16 bytes per (g, t) = words (slot g, blk 0), (slot g+8, blk 0), (slot g, blk 1), (slot g+8, blk 1);
            // byte i of a word holds values 4t+i (low nibble) and 16+4t+i (high nibble) of its block
            const uint32_t src = tile_src + (sub >> 1) * 576, blk = sub & 1;
            const uint32_t sc2 = lds32(src + 512 + g * 8 + blk * 4);
            const __half2 dd = __half2half2(half ? __high2half(bits_h2(sc2)) : __low2half(bits_h2(sc2)));
#pragma unroll
            for (int t = 0; t < 4; t++) {
              const uint32_t w = lds32(src + packed_piece(g, t) * 16 + (blk * 2 + half) * 4);
              const uint32_t lows = w & 0x0F0F0F0Fu, highs = (w >> 4) & 0x0F0F0F0Fu;
              dq2(__byte_perm(lows, 0x64646464u, 0x4140), zp, dd, v[2 * t + 0], v[16 + 2 * t + 0]);
              dq2(__byte_perm(lows, 0x64646464u, 0x4342), zp, dd, v[2 * t + 1], v[16 + 2 * t + 1]);
              dq2(__byte_perm(highs, 0x64646464u, 0x4140), zp, dd, v[8 + 2 * t + 0], v[24 + 2 * t + 0]);
              dq2(__byte_perm(highs, 0x64646464u, 0x4342), zp, dd, v[8 + 2 * t + 1], v[24 + 2 * t + 1]);
            }
          }
          tc_st32(tmem_base + ((q * 32u) << 16) + TMEM_A0 + ((gblk + sub) % A_STAGES) * A_STAGE_COLS, v);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&a_full[(gblk / GROUP) & 1]);
          mbar_arrive(&raw_empty[raw.stage]);
        }
        raw.advance();
      }
    }
    if (!ok && lane == 0) *s_abort = 1, atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
  } else {
    // ---------------------------------------------------------------------------- epilogue
    // Two groups of four warps, one per accumulator buffer: group e drains the items whose running number is e mod 2,
    // so the epilogues of two consecutive items may overlap each other as well as the MMAs that follow.
    const uint32_t q = warp & 3;         // a warp reads the TMEM lanes 32 * (warp % 4) ..
    const uint32_t row = q * 32 + lane;  // row of the item's 128-row tile
    const uint32_t buf = (warp - W_EPI0) >> 2, gw = (warp - W_EPI0) & 3;  // group, warp within the group
    uint32_t *s_pair = reinterpret_cast<uint32_t *>(smem + 1024 + buf * 2048);
    float *s_un = reinterpret_cast<float *>(smem + 1024 + buf * 2048 + 512);
    float **s_row = reinterpret_cast<float **>(smem + 1024 + buf * 2048 + 1024);  // down phase: each token's output row
    uint32_t n_item = 0, used = 0;  // resident items seen by the CTA; uses of this group's buffer
    // A group whose bounded wait expired goes "dead": it stops touching TMEM and waiting but keeps walking the items, so
    // that the group's named barriers always see all four warps.
    bool dead = false;
    for (uint32_t item = item_beg; item < n_items; item += item_step) {
      const uint32_t pass = item / m_tiles, mt = item % m_tiles;
      const bool resident = expert_base(pass) != nullptr;
      if (resident) {
        if ((n_item++ & 1) != buf) continue;  // the other group's item
      } else if (buf != 0) {
        continue;  // items of missing experts are zero-filled by group 0
      }
      const uint32_t pstart = d.pass_start[pass], pcount = d.pass_count[pass];
      // The pass's pair indices and un-scale factors go to shared memory (one column per thread of the group), fetched
      // before the accumulator is waited for so that their latency hides behind the item's MMAs; the column loop then
      // reads them as broadcasts.
      {
        const uint32_t c = gw * 32 + lane;
        const bool have = c < pcount;
        const uint32_t pr = have ? __ldg(d.perm + pstart + c) : 0u;
        const float un = have ? __ldg(p.unscale + (size_t)pass * p.bn + c) : 0.0f;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + buf) : "memory");  // the group has finished reading the previous item's tables
        s_pair[c] = pr, s_un[c] = un;
        if (p.phase == 1) s_row[c] = have ? pair_output_row(d, p.out, pr) : nullptr;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + buf) : "memory");
      }
      if (resident && !dead) {
        ok = mbar_wait(&acc_full[buf], used & 1);
        used++;
        if (*s_abort) ok = false;
        if (!__all_sync(0xffffffffu, ok)) dead = true;
        tc_fence_after();
      } else if (!resident && warp == W_EPI0 && lane == 0) {
        atomicOr(d.status, MER_DEVSTAT_RESIDENCY_MISS);  // fail closed: zeros below
      }
      const uint32_t acc_addr = tmem_base + ((q * 32u) << 16) + buf * 128;
      const uint32_t width = pass_width(p.bn, pcount);
      const uint32_t grp_id = d.pass_group[pass];
      const bool merged = d.offsets[grp_id + 1] - d.offsets[grp_id] <= MERGE_TOKENS;
      const bool is_gate = (lane & 8) == 0;
      const bool clamp = d.swiglu_limit > 0.0f && isfinite(d.swiglu_limit);
      for (uint32_t cbase = 0; cbase < pcount; cbase += 32) {  // 32 columns (tokens) at a time
        uint32_t v[32];
        float val[32];
        if (resident && !dead) {
          tc_ld32(acc_addr + cbase, v);
#pragma unroll
          for (int i = 0; i < 32; i++) val[i] = __uint_as_float(v[i]);
          if (merged) {  // the W_hi x_lo column set of the same tokens
            tc_ld32(acc_addr + width + cbase, v);
#pragma unroll
            for (int i = 0; i < 32; i++) val[i] += __uint_as_float(v[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) val[i] = 0.0f;
        }
        // the steps run column-batched (all multiplies, then all shuffles, ...): warp-synchronous operations are kept in
        // program order, so a column-by-column loop would serialise on the latency of every single one
#pragma unroll
        for (int i = 0; i < 32; i++) val[i] *= s_un[cbase + i];
        if (p.phase == 0) {
          // rows come in packed tiles of 16: slots 0..7 gate rows, 8..15 the matching up rows
          float up[32];
#pragma unroll
          for (int i = 0; i < 32; i++) up[i] = __shfl_down_sync(0xffffffffu, val[i], 8);
#pragma unroll
          for (int i = 0; i < 32; i++) {
            float gate = val[i];
            if (clamp && gate == gate) gate = fminf(fmaxf(gate, -d.swiglu_limit), d.swiglu_limit);
            val[i] = __fdividef(gate, 1.0f + __expf(-gate)) * up[i];
          }
          float *dst = p.out + (mt * 8 + (row >> 4)) * 8 + (lane & 7);
#pragma unroll
          for (int i = 0; i < 32; i++)
            if (is_gate && cbase + i < pcount) dst[(size_t)s_pair[cbase + i] * d.F] = val[i];
        } else {
          const uint32_t off = mt * 128 + row;
#pragma unroll
          for (int i = 0; i < 32; i++)
            if (cbase + i < pcount) s_row[cbase + i][off] = val[i];
        }
      }
      if (resident && !dead) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
    }
    if (dead && lane == 0) *s_abort = 1, atomicOr(d.status, MER_DEVSTAT_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Per-token row maximum of |x| (the gate/up activations' scale source).  One warp per token.
__global__ void __launch_bounds__(256) k_row_amax(const float *__restrict__ x, uint32_t n_tokens, uint32_t K, uint32_t *__restrict__ amax) {
  const uint32_t tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (tok >= n_tokens) return;
  const float4 *r4 = reinterpret_cast<const float4 *>(x + (size_t)tok * K);
  float mx = 0.0f;
  bool nan = false;
  for (uint32_t i = lane; i < K / 4; i += 32) {
    const float4 v = __ldg(r4 + i);
    nan |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
    mx = fmaxf(fmaxf(fmaxf(fmaxf(mx, fabsf(v.x)), fabsf(v.y)), fabsf(v.z)), fabsf(v.w));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  nan = __any_sync(0xffffffffu, nan);
  if (lane == 0) amax[tok] = nan ? 0x7fc00000u : __float_as_uint(mx);
}

// Row maxima of the grouped rows of h only (perm lists them): in an expert-parallel dispatch most pairs belong to other
// ranks and their rows of h are never written or read.
__global__ void __launch_bounds__(256) k_row_amax_grouped(MoeDispatch d, const float *__restrict__ h, uint32_t K, uint32_t *__restrict__ amax) {
  const uint32_t i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= d.offsets[d.n_groups]) return;
  const uint32_t pair = d.perm[i];
  const float4 *r4 = reinterpret_cast<const float4 *>(h + (size_t)pair * K);
  float mx = 0.0f;
  bool nan = false;
  for (uint32_t k = lane; k < K / 4; k += 32) {
    const float4 v = __ldg(r4 + k);
    nan |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
    mx = fmaxf(fmaxf(fmaxf(fmaxf(mx, fabsf(v.x)), fabsf(v.y)), fabsf(v.z)), fabsf(v.w));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  nan = __any_sync(0xffffffffu, nan);
  if (lane == 0) amax[pair] = nan ? 0x7fc00000u : __float_as_uint(mx);
}

// Builds, for every token pass, the activation operand images the GEMM kernel copies chunk by chunk.  A chunk is 64
// values of K = 8 core-matrix columns; a column holds the pass's rows as 16-byte pieces, the f16 hi parts of all rows
// first, then the lo parts (+32 B skew): [hi row 0 .. hi row w-1 | lo row 0 .. lo row w-1], w = the pass's width
// (its token count rounded up to 16), so one descriptor of 2w rows covers [x_hi | x_lo] and a narrow pass is a small
// image.  grid = (pass capacity, K / 64).
__global__ void __launch_bounds__(256) k_gemm_act_image(MoeDispatch d, int phase, const float *__restrict__ act, uint32_t K, uint32_t bn,
                                                        uint32_t b_lbo, const uint32_t *__restrict__ amax_tok, uint8_t *__restrict__ img,
                                                        float *__restrict__ unscale) {
  const uint32_t pass = blockIdx.x, chunk = blockIdx.y;
  if (pass >= *d.n_passes) return;
  const uint32_t pstart = d.pass_start[pass], pcount = d.pass_count[pass];
  const uint32_t n_chunks = K / 64;
  uint8_t *dst0 = img + ((size_t)pass * n_chunks + chunk) * 16 * b_lbo;  // slots are as large as the widest pass needs
  const uint32_t width = pass_width(bn, pcount), lbo = pass_lbo(width);
  // per row of the pass, once: where it comes from and its scale
  __shared__ float s_scale[128];
  __shared__ uint32_t s_src[128];
  for (uint32_t j = threadIdx.x; j < width; j += blockDim.x) {
    float sc = 0.0f;  // rows beyond the pass's count are zero rows
    uint32_t rowi = 0;
    if (j < pcount) {
      const uint32_t pair = d.perm[pstart + j];
      rowi = phase == 0 ? pair / d.slots : pair;
      const float mx = __uint_as_float(phase == 0 ? amax_tok[rowi] : d.amax[pair]);
      sc = 1.0f;
      if (mx > 0.0f && isfinite(mx)) {
        int e;
        frexpf(mx, &e);
        sc = ldexpf(1.0f, (int)POW2_SCALE_TARGET - e);  // mx * sc in [256, 512)
      } else if (mx != mx || isinf(mx)) {
        sc = mx;  // non-finite activations poison the row, as they would in fp32
      }
    }
    s_scale[j] = sc, s_src[j] = rowi;
    if (chunk == 0) unscale[(size_t)pass * bn + j] = j < pcount ? 1.0f / sc : 0.0f;
  }
  __syncthreads();
  for (uint32_t idx = threadIdx.x; idx < width * 8; idx += blockDim.x) {
    const uint32_t k8 = idx / width, j = idx - k8 * width;
    uint4 hi = make_uint4(0, 0, 0, 0), lo = make_uint4(0, 0, 0, 0);
    if (j < pcount) {
      const float sc = s_scale[j];
      const float4 *src = reinterpret_cast<const float4 *>(act + (size_t)s_src[j] * K + chunk * 64 + k8 * 8);
      const float4 a = __ldg(src), b = __ldg(src + 1);
      const float vs[8] = {a.x * sc, a.y * sc, a.z * sc, a.w * sc, b.x * sc, b.y * sc, b.z * sc, b.w * sc};
      uint32_t h[4], l[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const __half2 hh = __floats2half2_rn(vs[2 * i], vs[2 * i + 1]);
        const float2 back = __half22float2(hh);
        h[i] = h2_bits(hh);
        l[i] = h2_bits(__floats2half2_rn(vs[2 * i] - back.x, vs[2 * i + 1] - back.y));
      }
      hi = make_uint4(h[0], h[1], h[2], h[3]), lo = make_uint4(l[0], l[1], l[2], l[3]);
    }
    uint8_t *dst = dst0 + (size_t)k8 * lbo + j * 16;
    *reinterpret_cast<uint4 *>(dst) = hi;
    *reinterpret_cast<uint4 *>(dst + width * 16) = lo;
  }
}

struct GemmPlan {
  uint32_t n_raw, n_b, b_lbo;
  size_t smem;
};

GemmPlan gemm_plan(int dtype, uint32_t bn) {
  const uint32_t tile_raw = RAW_BLOCKS * 16 * (dtype == MER_DTYPE_Q4_0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES);
  GemmPlan pl{};
  pl.b_lbo = bn * 16 + 32;
  pl.n_raw = 4, pl.n_b = 2;  // weight stages (one group each); activation stages (one group = two chunk slots each)
  pl.smem = G_HEADER + (size_t)pl.n_raw * 8 * tile_raw + (size_t)pl.n_b * 2 * 16 * pl.b_lbo;
  return pl;
}

struct GemmScratch {
  uint32_t *amax_tok;
  float *unscale;
  uint8_t *img;
  size_t img_bytes;
};

GemmScratch gemm_scratch(void *scratch, size_t scratch_bytes, uint32_t max_tokens, uint32_t max_pairs) {
  GemmScratch g{};
  uint8_t *p = reinterpret_cast<uint8_t *>(scratch);
  g.amax_tok = reinterpret_cast<uint32_t *>(p);
  size_t off = ((size_t)max_tokens * 4 + 255) & ~(size_t)255;
  g.unscale = reinterpret_cast<float *>(p + off);
  off += ((size_t)3 * max_pairs * 4 + 128 * 4 + 255) & ~(size_t)255;
  g.img = p + off;
  g.img_bytes = scratch_bytes > off ? scratch_bytes - off : 0;
  return g;
}

}  // namespace

bool gemm_ffn_supported(int dtype, uint32_t D, uint32_t F) {
  return (dtype == MER_DTYPE_Q4_0 || dtype == MER_DTYPE_Q8_0) && D % 256 == 0 && F % 256 == 0;
}

// Activation images: rows padded to whole passes (at most 3 x max_pairs rows), 4 bytes per value plus the skew.
size_t gemm_ffn_scratch_bytes(uint32_t max_tokens, uint32_t max_pairs, uint32_t D, uint32_t F) {
  const size_t kmax = D > F ? D : F;
  const size_t rows = (size_t)3 * max_pairs + 128;
  return (((size_t)max_tokens * 4 + 255) & ~(size_t)255) + ((rows * 4 + 255) & ~(size_t)255) + rows * kmax * 4 + (rows / 16 + 1) * (kmax / 64) * 512 +
         4096;
}

// Tokens per pass for a dispatch: about 1.5 x the mean group size, within what the image scratch holds.
// Returns 0 when the dispatch is better served by the streaming kernels.
uint32_t gemm_pick_bn(const MoeDispatch &d, uint32_t min_mean_tokens) {
  const uint64_t P = (uint64_t)d.n_tokens * d.slots;
  const uint32_t groups = d.active_groups_hint ? d.active_groups_hint : 1;
  const uint64_t mean = (d.expected_pairs ? d.expected_pairs : P) / groups;
  if (mean < min_mean_tokens) return 0;
  uint32_t bn = mean <= 12 ? 16 : mean <= 24 ? 32 : mean <= 56 ? 64 : 128;
  const uint64_t gmax = d.n_groups < P ? d.n_groups : P;
  while (bn > 16 && P + gmax * (bn - 1) > (uint64_t)3 * d.scratch_pairs) bn >>= 1;
  if (P + gmax * (bn - 1) > (uint64_t)3 * d.scratch_pairs + 128) return 0;
  return bn;
}

void gemm_bind(MoeDispatch &d, void *stream_scratch, int sm_count, uint32_t bn) {
  stream_bind(d, stream_scratch, sm_count);  // pass tables and the per-pair max cells live in the streaming scratch
  d.tokens_per_pass = bn;
}

cudaError_t launch_ffn_gemm(MoeDispatch &d, void *gemm_scratch_ptr, size_t gemm_scratch_bytes, uint32_t max_tokens, int sm_count,
                            cudaStream_t s, int *launches, cudaEvent_t ev_mid) {
  const uint32_t bn = d.tokens_per_pass;
  const GemmPlan pl = gemm_plan(d.dtype, bn);
  const GemmScratch gs = gemm_scratch(gemm_scratch_ptr, gemm_scratch_bytes, max_tokens, d.scratch_pairs);
  const uint32_t P = d.n_tokens * d.slots;
  const uint32_t gmax = d.n_groups < P ? d.n_groups : P;
  const uint32_t pass_cap = P / bn + gmax;  // upper bound on the number of passes
  auto kern = d.dtype == MER_DTYPE_Q4_0 ? k_ffn_gemm<MER_DTYPE_Q4_0> : k_ffn_gemm<MER_DTYPE_Q8_0>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return e;

  k_row_amax<<<(d.n_tokens + 7) / 8, 256, 0, s>>>(d.x, d.n_tokens, d.D, gs.amax_tok);
  for (int phase = 0; phase < 2; phase++) {
    const uint32_t K = phase == 0 ? d.D : d.F;
    const float *act = phase == 0 ? d.x : d.h;
    k_gemm_act_image<<<dim3(pass_cap, K / 64), 256, 0, s>>>(d, phase, act, K, bn, pl.b_lbo, gs.amax_tok, gs.img, gs.unscale);
    GemmParams p{};
    p.d = d, p.phase = phase, p.act_img = gs.img, p.unscale = gs.unscale;
    p.rows = phase == 0 ? d.F : d.D;
    p.kb_total = K / 32;
    p.bn = bn, p.b_lbo = pl.b_lbo, p.n_raw = pl.n_raw, p.n_b = pl.n_b;
    p.out = phase == 0 ? d.h : d.y;
    kern<<<sm_count, G_THREADS, pl.smem, s>>>(p);
    if (phase == 0) {
      // row maxima of h = SiLU(gate) * up, the scale source of the down phase's operand image (the GEMM epilogue does
      // not collect them: a warp reduction per column sat on its critical path)
      k_row_amax_grouped<<<(P + 7) / 8, 256, 0, s>>>(d, d.h, d.F, d.amax);
      if (ev_mid) cudaEventRecord(ev_mid, s);
    }
  }
  d.y_parts = nullptr, d.y_nparts = 1;
  if (launches) (*launches) += 6;
  return cudaGetLastError();
}
