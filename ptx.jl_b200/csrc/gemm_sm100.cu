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
// Few tiles, long K (the reference leaves this: one tile per CTA,
// gemm_highperf_blackwell.jl:27-32). With fewer tiles than half the SMs the launch would
// run on a fraction of the machine, so the tiles are cut along K: their k-iterations
// form one line that is dealt out evenly to at least twice as many CTAs, a CTA's share
// being a run of whole tiles with a partial tile at either end. A partial accumulator
// is parked in a slab of fp32 scratch, and a second small kernel sums each tile's slabs
// in segment order and writes C. The order of the sums is fixed, so results are
// reproducible from launch to launch (they differ in the last bits from the unsplit
// order).
//
// Algorithmic work per launch: 2*G*M*N*K flop; compulsory bytes G*((M*K + N*K)*2 +
// M*N*sizeof(out)).
#include <map>
#include <mutex>
#include <utility>

#include "gemm_epilogue.cuh"
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

// The work of one CTA: first its whole tiles of the data-parallel part (tile =
// blockIdx.x + i * gridDim.x below dp_tiles), then its share [it, end) of the
// k-iteration line of the stream-K tiles. The three roles walk the same sequence.
struct Sched {
  int dp_tiles;        // tiles handed out whole
  int sk_tiles;        // tiles cut along K (tile indices dp_tiles .. dp_tiles + sk_tiles - 1)
  int sk_ctas;         // CTAs that share the k-iteration line (the first sk_ctas of the grid)
  int kiters;          // K / kBK
  float* slabs;        // [2 * sk_ctas][kBM * kBN] fp32 partial accumulators
};
struct Unit {
  int tile;            // global tile index
  int k0, k1;          // k-iterations [k0, k1) of that tile
  int slab;            // partial units: which of this CTA's two slabs (0: its share starts here, 1: not)
};
struct UnitIter {
  int i = 0;
  long long it = 0, end = 0, begin = 0;
  __device__ __forceinline__ void init(const Sched& s) {
    const long long total = (long long)s.sk_tiles * s.kiters;
    if ((int)blockIdx.x < s.sk_ctas) {
      begin = it = total * blockIdx.x / s.sk_ctas;
      end = total * (blockIdx.x + 1) / s.sk_ctas;
    }
  }
  __device__ __forceinline__ bool next(const Sched& s, Unit& u) {
    const int tile = blockIdx.x + i * gridDim.x;
    if (tile < s.dp_tiles) {
      ++i;
      u = {tile, 0, s.kiters, 0};
      return true;
    }
    if (it < end) {
      const int t = (int)(it / s.kiters);
      const int k0 = (int)(it - (long long)t * s.kiters);
      const long long left = end - it;
      const int len = left < s.kiters - k0 ? (int)left : s.kiters - k0;
      u = {s.dp_tiles + t, k0, k0 + len, it == begin ? 0 : 1};
      it += len;
      return true;
    }
    return false;
  }
};
// CTA whose share of the stream-K line holds iteration x: the largest c with
// floor(c * total / ctas) <= x.
__device__ __forceinline__ int sk_owner(long long x, long long total, int ctas) {
  return (int)(((x + 1) * ctas - 1) / total);
}
// Slab element of accumulator (row, col): 16-byte column groups outermost, rows
// innermost, so that a warp's 32 rows of one group are 512 contiguous bytes.
__device__ __forceinline__ size_t slab_index(int row, int col4) { return ((size_t)col4 * kBM + row) * 4; }

template <bool kF32Out>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            void* __restrict__ c_out, int M, int N, int K, int ldc, int groups,
            const Sched sched, uint32_t* status) {
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

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      uint32_t it = 0;
      UnitIter units;
      units.init(sched);
      Unit u;
      while (units.next(sched, u)) {
        int tm, tn;
        const int g = u.tile / tiles_per_group;
        tile_coords(u.tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
        const int a_row = g * M + tm * kBM;
        const int b_row = g * N + tn * kBN;
        for (int k = u.k0; k < u.k1; ++k, ++it) {
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
      UnitIter units;
      units.init(sched);
      Unit u;
      for (; units.next(sched, u); ++t) {
        const uint32_t buf = t & 1u;
        const uint32_t aph = (t >> 1) & 1u;
        mbar_wait_warp(bar_acc_empty + 8 * buf, aph ^ 1u, wctx, kSiteAccEmpty);
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * kAccCols;
        for (int k = u.k0; k < u.k1; ++k, ++it) {
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
            tc_mma_ss_warp(d_tmem, da + 2 * kk, dhi, db + 2 * kk, dhi, idesc,
                           (k != u.k0 || kk != 0) ? 1u : 0u);
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
    UnitIter units;
    units.init(sched);
    Unit u;
    for (; units.next(sched, u); ++t) {
      int tm, tn;
      const int g = u.tile / tiles_per_group;
      tile_coords(u.tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = t & 1u;
      const uint32_t aph = (t >> 1) & 1u;
      mbar_wait(bar_acc_full + 8 * buf, aph, wctx, kSiteAccFull);
      tc_fence_after();
      const size_t row = (size_t)g * M + (size_t)tm * kBM + row_in_tile;
      const int col0 = tn * kBN;
      const uint32_t t_row = tmem_addr(tmem, quad * 32, buf * kAccCols);
      const bool whole = u.k0 == 0 && u.k1 == sched.kiters;
      if (whole) {
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(t_row + c * 32, v);
          tc_wait_ld_bind(v);
          const int col = col0 + c * 32;
          if (col < N) store_acc_chunk<kF32Out>(c_out, row, ldc, col, v);
        }
        // every TMEM read of this accumulator has completed (wait::ld above)
        tc_fence_before();
        mbar_arrive(bar_acc_empty + 8 * buf);
        continue;
      }
      // ---- a part of a tile cut along K: park the partial sums; sk_reduce_kernel adds
      // the parts up in segment order and writes C
      float* slab = sched.slabs + (size_t)(2 * blockIdx.x + u.slab) * (kBM * kBN);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(t_row + c * 32, v);
        tc_wait_ld_bind(v);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          __stcg(reinterpret_cast<float4*>(slab + slab_index(row_in_tile, c * 8 + i)),
                 make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])));
      }
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

// Second step of a launch that cut tiles along K: C = sum of each tile's parts, in
// segment order. One thread per (tile, row, 4 columns); consecutive threads take
// consecutive rows, which is the contiguous axis of the slabs.
template <bool kF32Out>
__global__ void __launch_bounds__(256)
sk_reduce_kernel(void* __restrict__ c_out, int M, int N, int ldc, int tiles_m, int tiles_n,
                 const Sched sched) {
  const int tiles_per_group = tiles_m * tiles_n;
  const long long total = (long long)sched.sk_tiles * sched.kiters;
  const long long n_items = (long long)sched.sk_tiles * (kBN / 4) * kBM;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_items;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(idx % kBM);
    const int col4 = (int)((idx / kBM) % (kBN / 4));
    const int t_local = (int)(idx / ((long long)kBM * (kBN / 4)));
    const int tile = sched.dp_tiles + t_local;
    int tm, tn;
    const int g = tile / tiles_per_group;
    tile_coords(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
    const int col = tn * kBN + col4 * 4;
    if (col >= N) continue;
    const long long x0 = (long long)t_local * sched.kiters;
    const int c_first = sk_owner(x0, total, sched.sk_ctas);
    const int nseg = sk_owner(x0 + sched.kiters - 1, total, sched.sk_ctas) - c_first + 1;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int seg = 0; seg < nseg; ++seg) {
      const int cta = c_first + seg;
      const long long cta_begin = total * cta / sched.sk_ctas;
      const float* part = sched.slabs + (size_t)(2 * cta + (cta_begin >= x0 ? 0 : 1)) * (kBM * kBN);
      const float4 q = __ldcg(reinterpret_cast<const float4*>(part + slab_index(r, col4)));
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    const size_t row = (size_t)g * M + (size_t)tm * kBM + r;
    if (kF32Out) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(c_out) + row * (size_t)ldc + col) = acc;
    } else {
      uint2 pk;
      pk.x = pack_bf16x2(acc.x, acc.y);
      pk.y = pack_bf16x2(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(c_out) + row * (size_t)ldc + col) = pk;
    }
  }
}

}  // namespace

namespace {

// The fp32 slabs for tiles cut along K come from the library's per-(device, stream)
// scratch (scratch_acquire): launches on one stream run one after the other, launches
// on different streams may overlap and must not share them. A launch needs two slabs
// per CTA.
constexpr int kSkMinIters = 8;   // a CTA's share of the k-iteration line is at least this long

}  // namespace

int launch_gemm(const DeviceCtx& ctx, void* C, const void* A, const void* Bt, int groups, int M, int N,
                int K, int ldc, unsigned flags, cudaStream_t stream) {
  // enough 256x256 tiles for every pair of SMs: the CTA-pair kernel (gemm2_sm100.cu)
  if (!(flags & PTXB200_GEMM_ONE_CTA) && gemm_pair_eligible(ctx, groups, M, N, K))
    return launch_gemm_pair(ctx, C, A, Bt, groups, M, N, K, ldc, flags, stream);
  CUtensorMap ta, tb;
  int rc = encode_tmap_bf16_2d(&ta, A, (uint64_t)groups * M, (uint64_t)K, (uint64_t)K * 2, kBM, kBK);
  if (rc != PTXB200_OK) return rc;
  rc = encode_tmap_bf16_2d(&tb, Bt, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K * 2, kBN, kBK);
  if (rc != PTXB200_OK) return rc;

  const int tiles_m = M / kBM, tiles_n = (N + kBN - 1) / kBN;
  const int tiles = groups * tiles_m * tiles_n;
  Sched sched;
  sched.kiters = K / kBK;
  sched.dp_tiles = tiles;
  sched.sk_tiles = 0;
  sched.sk_ctas = 0;
  sched.slabs = nullptr;
  int grid = tiles < ctx.sm_count ? tiles : ctx.sm_count;
  ScratchLease lease;
  // Few tiles, long K: cut every tile along K so that at least twice as many CTAs work.
  // (Cutting only the tiles of a sparse LAST wave was built too and measured slower
  // than leaving them whole: parking and re-reading two partial tiles per CTA costs
  // more than the idle SMs of that wave.)
  if (!(flags & PTXB200_GEMM_NO_SPLIT) && tiles * 2 <= ctx.sm_count) {
    const long long line = (long long)tiles * sched.kiters;
    long long ctas = line / kSkMinIters;
    if (ctas > ctx.sm_count) ctas = ctx.sm_count;
    if (ctas >= 2 * tiles) {
      if ((rc = scratch_acquire(ctx, stream, kScratchGemmSlabs, (size_t)2 * ctas * kBM * kBN * sizeof(float),
                                &lease)) != PTXB200_OK)
        return rc;
      sched.slabs = reinterpret_cast<float*>(lease.ptr);
      sched.dp_tiles = 0;
      sched.sk_tiles = tiles;
      sched.sk_ctas = (int)ctas;
      grid = (int)ctas;
    }
  }
  uint32_t* status = status_word(ctx, stream);
  static PerDeviceOnce attr_once;
  rc = attr_once.run(ctx.device, []() -> int {
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    return PTXB200_OK;
  });
  if (rc != PTXB200_OK) return rc;
  if (flags & PTXB200_GEMM_F32_OUT)
    gemm_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, C, M, N, K, ldc, groups, sched, status);
  else
    gemm_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, C, M, N, K, ldc, groups, sched, status);
  PTXB200_CUDA_TRY(cudaGetLastError());
  if (sched.sk_tiles > 0) {
    const long long items = (long long)sched.sk_tiles * (kBN / 4) * kBM;
    const int rgrid = (int)((items + 255) / 256);
    if (flags & PTXB200_GEMM_F32_OUT)
      sk_reduce_kernel<true><<<rgrid, 256, 0, stream>>>(C, M, N, ldc, tiles_m, tiles_n, sched);
    else
      sk_reduce_kernel<false><<<rgrid, 256, 0, stream>>>(C, M, N, ldc, tiles_m, tiles_n, sched);
    PTXB200_CUDA_TRY(cudaGetLastError());
    if ((rc = scratch_mark_used(lease, stream)) != PTXB200_OK) return rc;
  }
  return PTXB200_OK;
}

}  // namespace ptxb200
