// gemm_bf16: C[M,N] = A[M,K] * B[K,N] on sm_100a, bf16 operands, fp32
// accumulation in tensor memory, bf16 (or fp32) output.
//
// What the reference does for this path
// (test/gpu/blackwell/gemm_highperf_blackwell.jl:69-199 and :317-468): one
// 128x256 output tile per CTA (or a persistent loop over tiles), a 4-stage TMA
// ring of 128x64 A and 256x64 B^T boxes in 128-byte-swizzled shared memory, four
// m128n256k16 tcgen05.mma per ring stage issued by one thread, slot release by
// tcgen05.commit, and a 128-thread fp32 epilogue that runs only after the whole
// K loop and, in the persistent variant, is followed by a CTA-wide barrier, so
// the tensor pipe idles during every epilogue.
//
// What this kernel does instead: one persistent CTA per SM with three roles on
// separate warps -- a TMA producer warp, an MMA-issue warp and four epilogue
// warps -- and TWO 256-column accumulators in tensor memory. While the epilogue
// warps drain accumulator t (tcgen05.ld -> bf16 pack -> 128-bit stores), the MMA
// warp is already accumulating tile t+1 into the other one, so the tensor pipe
// never waits for an epilogue. Tiles are walked in an L2-friendly order
// (bands of kGroupM row-tiles, column-tiles inside a band) so that the ~148
// tiles in flight share A row panels and B column panels in the 126 MB L2.
//
// Uniform grouped GEMM (the reference's grid-z = group kernel,
// test/gpu/blackwell/grouped_gemm.jl:43-158): G problems of one shape with A stacked
// as [G*M, K], B^T as [G*N, K] and C as [G*M, N] are one more factor of the same
// persistent tile loop -- tile -> (group, row-tile, column-tile), the group folded
// into the TMA row coordinates -- so small groups fill the machine together instead
// of one launch (or one grid-z slice) each. A B^T box that runs past its group's N
// rows brings in the next group's rows (or zero fill past the end); those columns
// are computed and never stored.
//
// Algorithmic work per launch: 2*G*M*N*K flop; compulsory bytes G*((M*K + N*K)*2 +
// M*N*sizeof(out)).
#include "host_common.h"
#include "sm100_prims.cuh"

namespace ptxb200 {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;                       // one 128-byte swizzle row of bf16
constexpr int kStages = 4;
constexpr int kAStageBytes = kBM * kBK * 2;   // 16 KiB
constexpr int kBStageBytes = kBN * kBK * 2;   // 32 KiB
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kThreads = 192;                 // warp 0 producer, warp 1 MMA, warps 2-5 epilogue
constexpr int kAccCols = 256;                 // fp32 columns per accumulator
constexpr int kTmemCols = 512;                // two accumulators
constexpr int kGroupM = 16;                   // row-tiles per rasterisation band

// Shared-memory map (offsets from a 1024-byte aligned base).
constexpr int kOffA = 0;
constexpr int kOffB = kOffA + kStages * kAStageBytes;
constexpr int kOffBars = kOffB + kStages * kBStageBytes;  // full[4] empty[4] acc_full[2] acc_empty[2]
constexpr int kOffTmemSlot = kOffBars + 12 * 8;
constexpr int kOffAbort = kOffTmemSlot + 8;
constexpr int kSmemBytes = kOffAbort + 8 + 1024;          // + slack for manual 1024-B alignment

// Wait sites reported in the status word.
enum : uint32_t { kSiteEmpty = 1, kSiteFull = 2, kSiteAccEmpty = 3, kSiteAccFull = 4 };

// Tile index -> (row-tile, column-tile): bands of kGroupM row-tiles, column-major
// inside a band, so concurrently running CTAs cover a compact block of C.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band_tiles = kGroupM * tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * kGroupM;
  const int rows_in_band = min(tiles_m - first_m, kGroupM);
  const int r = tile - band * band_tiles;
  tm = first_m + r % rows_in_band;
  tn = r / rows_in_band;
}

template <bool kF32Out>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            void* __restrict__ c_out, int M, int N, int K, int ldc, int groups,
            uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));

  const uint32_t a_base = base + kOffA;
  const uint32_t b_base = base + kOffB;
  const uint32_t bar_full = base + kOffBars;
  const uint32_t bar_empty = bar_full + kStages * 8;
  const uint32_t bar_acc_full = bar_empty + kStages * 8;
  const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kOffAbort);
  const WaitCtx wctx{status, abort_flag};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int tiles_m = M / kBM;
  const int tiles_n = (N + kBN - 1) / kBN;
  const int tiles_per_group = tiles_m * tiles_n;
  const int total_tiles = tiles_per_group * groups;
  const int kiters = K / kBK;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int tm, tn;
        const int g = tile / tiles_per_group;
        tile_coords(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
        const int a_row = g * M + tm * kBM;
        const int b_row = g * N + tn * kBN;
        for (int k = 0; k < kiters; ++k, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          mbar_wait(bar_empty + 8 * s, ph ^ 1u, wctx, kSiteEmpty);
          mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
          tma_load_2d(a_base + s * kAStageBytes, &tmap_a, k * kBK, a_row, bar_full + 8 * s);
          tma_load_2d(b_base + s * kBStageBytes, &tmap_b, k * kBK, b_row, bar_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    // The whole warp walks the loop converged; the tcgen05 instructions elect their
    // issuing lane themselves (see tc_mma_ss_warp).
    {
      constexpr uint32_t idesc = make_idesc_bf16_f32(kBM, kBN, false, false);
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++t) {
        const uint32_t buf = t & 1u;
        const uint32_t aph = (t >> 1) & 1u;
        mbar_wait_warp(bar_acc_empty + 8 * buf, aph ^ 1u, wctx, kSiteAccEmpty);
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * kAccCols;
        for (int k = 0; k < kiters; ++k, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          mbar_wait_warp(bar_full + 8 * s, ph, wctx, kSiteFull);
          tc_fence_after();
          const uint32_t da = sdesc_lo(a_base + s * kAStageBytes, 16);
          const uint32_t db = sdesc_lo(b_base + s * kBStageBytes, 16);
          constexpr uint32_t dhi = sdesc_hi(1024, kLayoutB128);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // +32 bytes (2 descriptor units) per 16-element K step inside the swizzle row
            tc_mma_ss_warp(d_tmem, da + 2 * kk, dhi, db + 2 * kk, dhi, idesc, (k | kk) != 0 ? 1u : 0u);
          }
          tc_commit_warp(bar_empty + 8 * s);   // slot free once these MMAs have read it
        }
        tc_commit_warp(bar_acc_full + 8 * buf);  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 ----------------
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may touch
    const int row_in_tile = quad * 32 + lane;
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++t) {
      int tm, tn;
      const int g = tile / tiles_per_group;
      tile_coords(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = t & 1u;
      const uint32_t aph = (t >> 1) & 1u;
      mbar_wait(bar_acc_full + 8 * buf, aph, wctx, kSiteAccFull);
      tc_fence_after();
      const size_t row = (size_t)g * M + (size_t)tm * kBM + row_in_tile;
      const int col0 = tn * kBN;
      const uint32_t t_row = tmem_addr(tmem, quad * 32, buf * kAccCols);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(t_row + c * 32, v);
        tc_wait_ld_bind(v);
        const int col = col0 + c * 32;
        if (col < N) {
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
      }
      // every TMEM read of this accumulator has completed (wait::ld above)
      tc_fence_before();
      mbar_arrive(bar_acc_empty + 8 * buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

int launch_gemm(const DeviceCtx& ctx, void* C, const void* A, const void* Bt, int groups, int M, int N,
                int K, int ldc, unsigned flags, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = encode_tmap_bf16_2d(&ta, A, (uint64_t)groups * M, (uint64_t)K, (uint64_t)K * 2, kBM, kBK);
  if (rc != PTXB200_OK) return rc;
  rc = encode_tmap_bf16_2d(&tb, Bt, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K * 2, kBN, kBK);
  if (rc != PTXB200_OK) return rc;

  const int tiles = groups * (M / kBM) * ((N + kBN - 1) / kBN);
  const int grid = tiles < ctx.sm_count ? tiles : ctx.sm_count;
  uint32_t* status = ctx.workspace + kWsStatus;
  if (flags & PTXB200_GEMM_F32_OUT) {
    static bool attr_done_f32[64] = {false};
    if (!attr_done_f32[ctx.device & 63]) {
      PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      attr_done_f32[ctx.device & 63] = true;
    }
    gemm_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, C, M, N, K, ldc, groups, status);
  } else {
    static bool attr_done_bf16[64] = {false};
    if (!attr_done_bf16[ctx.device & 63]) {
      PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      attr_done_bf16[ctx.device & 63] = true;
    }
    gemm_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, C, M, N, K, ldc, groups, status);
  }
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

}  // namespace ptxb200
