// Resident (HBM slot) layout of an expert: "tile-major fragment order".
//
// The bytes of the reference's gate||up||down block stream are kept one for one (same scales,
// same quants, same total size); only their order changes at admission so that the streaming
// kernels read every operand with aligned 128-bit shared-memory loads:
//
//   region 0, gate/up: F/8 tiles.  Tile tt holds 16 row slots: slots 0..7 = gate rows 8tt..8tt+7,
//                      slots 8..15 = up rows 8tt..8tt+7 (so SiLU(gate)*up pairs up inside a thread).
//   region 1, down:    D/16 tiles.  Tile tt holds down rows 16tt..16tt+15.
//   A tile stores its K/32 blocks in order; all 16 row slots of a block sit together:
//     Q8_0 block record, 544 B = 16 x 34:
//        [lane L = g*4+t][16 B] = quants 8t..8t+7 of row slot g, then of row slot g+8      (512 B)
//        [g][2 x f16]           = scale of slot g, scale of slot g+8                        (32 B)
//     Q4_0 block-pair record, 576 B = 2 x 16 x 18 (blocks 2p and 2p+1):
//        [lane L][16 B] = quant bytes 4t..4t+3 of (slot g, blk 2p), (slot g+8, blk 2p),
//                         (slot g, blk 2p+1), (slot g+8, blk 2p+1)                          (512 B)
//        [g][4 x f16]   = scales in the same order                                          (64 B)
//   (g = lane / 4 and t = lane % 4 are the mma.sync m16n8k16 fragment coordinates.)
//   Inside a record the 16-byte piece of lane L = (g, t) sits at position g*4 + ((t + g/2) % 4), not at L: the
//   streaming kernels read one piece per lane (any bijection is conflict-free for them), while the GEMM kernels'
//   dequantisers read the four pieces of ONE row slot in four steps, all lanes at the same t; the rotation spreads the
//   eight row slots of a step over all 32 banks of shared memory (without it: 8-way bank conflicts).
//
// Shapes whose rows are not multiples of 256 columns keep the reference's flat stream.
#pragma once

#include <stdint.h>

#include "kernels.h"

struct PackedAddr {
  size_t quant;  // byte offset of the quant byte that holds the weight
  size_t scale;  // byte offset of the f16 block scale
};

// Position (in 16-byte pieces) of the piece of fragment lane (g, t) inside a block record.
__host__ __device__ inline uint32_t packed_piece(uint32_t g, uint32_t t) { return g * 4u + ((t + (g >> 1)) & 3u); }

// Location of weight (matrix, row, col) inside a packed expert. matrix: 0 gate, 1 up, 2 down.
template <int DT>
__host__ __device__ inline PackedAddr packed_locate(uint32_t D, uint32_t F, int matrix, uint32_t row, uint32_t col) {
  const uint32_t bb = DT == 0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES;
  const size_t proj = (size_t)D * F / 32 * bb;
  uint32_t K, tile, slot;
  size_t region;
  if (matrix < 2) {
    K = D, tile = row >> 3, slot = (row & 7u) + 8u * (uint32_t)matrix, region = 0;
  } else {
    K = F, tile = row >> 4, slot = row & 15u, region = 2 * proj;
  }
  const uint32_t g = slot & 7u, half = slot >> 3, kb = col >> 5, j = col & 31u;
  const size_t tile_base = region + (size_t)tile * (K / 32) * 16 * bb;
  PackedAddr a;
  if (DT == 0) {
    const size_t rec = tile_base + (size_t)(kb >> 1) * 576;
    const uint32_t bip = kb & 1u, jj = j & 15u, t = jj >> 2;
    a.quant = rec + (size_t)packed_piece(g, t) * 16 + bip * 8 + half * 4 + (jj & 3u);
    a.scale = rec + 512 + g * 8 + bip * 4 + half * 2;
  } else {
    const size_t rec = tile_base + (size_t)kb * 544;
    const uint32_t t = j >> 3;
    a.quant = rec + (size_t)packed_piece(g, t) * 16 + half * 8 + (j & 7u);
    a.scale = rec + 512 + g * 4 + half * 2;
  }
  return a;
}
