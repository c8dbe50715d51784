// Shared-memory tile geometry and tcgen05 descriptors of one attention tile,
// used by both the flash-attention kernel and the single-tile probe so that the
// probe validates exactly the descriptor arithmetic the kernel runs on.
//
// A tile is 128 rows x D bf16 columns, brought in by TMA as D/64 "stripes": each
// stripe is a 128-row x 64-column (128-byte) box in the 128-byte swizzle, 16 KiB,
// stripes laid one after the other (reference: fab_load_tile,
// test/gpu/blackwell/flash_attention_defs.jl:275-281).
//
//  * Q and K are consumed K-major (the contraction runs along D, the contiguous
//    axis): 8-row groups are 1024 bytes apart (stride), a 16-element K step is
//    +32 bytes inside the 128-byte row, the next 64 columns are the next stripe
//    (+16 KiB)  (flash_attention_defs.jl:298-300, 736-741).
//  * V is consumed MN-major as the B operand of P*V (the contraction runs along
//    the 128 key rows, N = D along the contiguous axis): 8 key rows are 1024
//    bytes apart (stride), the next 64 columns of D are one stripe apart
//    (leading = 16 KiB), a 16-row K step is +2048 bytes
//    (flash_attention_defs.jl:342, 742-744).
//  * P lives in tensor memory as packed bf16 pairs: 16 K-elements = 8 columns per
//    k16 step (flash_attention_defs.jl:341).
#pragma once
#include "sm100_prims.cuh"

namespace ptxb200 {

constexpr int kAttnRows = 128;          // rows of a Q sub-tile and of a K/V tile
constexpr int kStripeBytes = 16384;     // 128 rows x 128 bytes

template <int D>
struct AttnTile {
  static_assert(D == 64 || D == 128, "head dimension");
  static constexpr int kStripes = D / 64;
  static constexpr int kTileBytes = kAttnRows * D * 2;
  static constexpr int kQKAtoms = D / 16;         // k16 steps of S = Q K^T
  static constexpr int kPVAtoms = kAttnRows / 16; // k16 steps of O = P V

  static constexpr uint32_t kIdescQK = make_idesc_bf16_f32(128, 128, false, false);
  static constexpr uint32_t kIdescPV = make_idesc_bf16_f32(128, D, false, true);

#if defined(__CUDACC__)
  // Descriptor high words (constants of the two operand layouts).
  static constexpr uint32_t kKMajorHi = sdesc_hi(1024, kLayoutB128);
  static constexpr uint32_t kVHi = sdesc_hi(1024, kLayoutB128);
  // Low word of the K-major descriptor of a Q or K tile at `tile_smem`, k16 step kk.
  static __device__ __forceinline__ uint32_t kmajor_lo(uint32_t tile_smem, int kk) {
    return sdesc_lo(tile_smem, 16) + (uint32_t)((kk >> 2) * (kStripeBytes >> 4) + (kk & 3) * 2);
  }
  // Low word of the MN-major B-operand descriptor of a V tile, k16 step kk.
  static __device__ __forceinline__ uint32_t v_lo(uint32_t tile_smem, int kk) {
    return sdesc_lo(tile_smem, kStripeBytes) + (uint32_t)(kk * (2048 >> 4));
  }
  // Tensor-memory address of P's k16 step kk, P starting at column `p_col`.
  static __device__ __forceinline__ uint32_t p_tmem(uint32_t tmem, uint32_t p_col, int kk) {
    return tmem + p_col + kk * 8;
  }
  // One thread: TMA-load the tile whose first row is `row` into `dst_smem`.
  static __device__ __forceinline__ void load(uint32_t dst_smem, const void* tmap, int row,
                                              uint32_t bar) {
#pragma unroll
    for (int s = 0; s < kStripes; ++s)
      tma_load_2d(dst_smem + s * kStripeBytes, tmap, s * 64, row, bar);
  }
  // The same from a 3-D map (slice = batch*head): rows past the end of the slice's
  // sequence come in as zeros.
  static __device__ __forceinline__ void load3(uint32_t dst_smem, const void* tmap, int row, int slice,
                                               uint32_t bar) {
#pragma unroll
    for (int s = 0; s < kStripes; ++s)
      tma_load_3d(dst_smem + s * kStripeBytes, tmap, s * 64, row, slice, bar);
  }
#endif
};

}  // namespace ptxb200
