// Accumulator -> C stores shared by the GEMM kernels: one thread holds 32 consecutive
// fp32 accumulator columns of one output row (what tcgen05.ld 32x32b.x32 delivers) and
// writes them as fp32, or rounded to bf16, with 128-bit stores.
#pragma once
#include "sm100_prims.cuh"

namespace ptxb200 {

template <bool kF32Out>
__device__ __forceinline__ void store_acc_chunk(void* __restrict__ c_out, size_t row, int ldc, int col,
                                                const uint32_t (&v)[32]) {
  if (kF32Out) {
    float* dst = reinterpret_cast<float*>(c_out) + row * (size_t)ldc + col;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      st_global_v4(dst + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_out) + row * (size_t)ldc + col;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t p0 = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
      const uint32_t p1 = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
      const uint32_t p2 = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
      const uint32_t p3 = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
      st_global_v4(dst + 8 * i, p0, p1, p2, p3);
    }
  }
}

}  // namespace ptxb200
