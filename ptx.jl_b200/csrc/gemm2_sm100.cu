// gemm_bf16 on CTA pairs: one 256x256 output tile per pair of SMs, issued as
// tcgen05.mma.cta_group::2.
//
// Why a second GEMM kernel. The single-CTA kernel (gemm_sm100.cu) streams 48 KiB
// from L2 into shared memory per 128x256x64 block of work; at the tensor pipe's rate
// that is ~17 TB/s over the 148 SMs, and a profile of 8192^3 shows the pipe active
// 82 % of the time with the rest spent waiting for operands. A CTA pair splits one
// 256x256 tile so that each SM holds only ITS 128 rows of A and ITS 128 rows of B^T
// per k-step (32 KiB for the same work: a third less traffic, and a six-deep ring in
// the same shared memory); the pair's leader issues m256n256k16 instructions that
// read both halves, and each SM ends up with its 128 rows of the 256-column
// accumulator in its own tensor memory. The reference has no counterpart (its GEMM is
// cta_group::1 throughout, test/gpu/blackwell/gemm_highperf_blackwell.jl:69-199).
//
// Roles in EACH CTA of the pair (192 threads): warp 0 TMA producer, warp 1 MMA
// (issues only in the leader; in both it owns the tensor-memory allocation), warps 2-5
// epilogue. Barriers live at the same shared-memory offsets in both CTAs:
//   full[s]      leader's only: two arrivals (each CTA's producer posts its own byte
//                count) plus the bytes of both CTAs' TMA loads, which name the leader's
//                barrier (cta_group::2 loads may signal the peer's barrier);
//   empty[s]     own: the leader commits to its own and to the peer's;
//   acc_full[b]  own: likewise two commits by the leader;
//   acc_empty[b] leader's only: 128 epilogue threads of each CTA arrive (remotely from
//                the peer) once their rows of the accumulator are in registers.
// No load is multicast; the peer's barriers are reached through mapa-translated
// addresses. Every wait is bounded as in the single-CTA kernel, and the pair meets at a
// cluster barrier before the first remote arrival and before exit.
//
// Work per launch: 2*G*M*N*K flop; compulsory bytes G*((M*K + N*K)*2 + M*N*sizeof(out)).
#include "gemm_epilogue.cuh"
#include "host_common.h"
#include "sm100_prims.cuh"

namespace ptxb200 {
namespace {

constexpr int kBM2 = 256;                      // rows of the pair's tile (128 per CTA)
constexpr int kBN2 = 256;                      // columns of the pair's tile
constexpr int kBK2 = 64;
constexpr int kStages2 = 6;
constexpr int kAStage2 = 128 * kBK2 * 2;       // this CTA's 128 rows of A: 16 KiB
constexpr int kBStage2 = 128 * kBK2 * 2;       // this CTA's 128 rows of B^T: 16 KiB
constexpr int kStage2 = kAStage2 + kBStage2;
constexpr int kThreads2 = 192;
constexpr int kAccCols2 = 256;
#ifndef PTXB200_GEMM2_GROUP_M
#define PTXB200_GEMM2_GROUP_M 8
#endif
constexpr int kGroupM2 = PTXB200_GEMM2_GROUP_M;   // row-tiles (of 256) per rasterisation band

constexpr int kOffA2 = 0;
constexpr int kOffB2 = kOffA2 + kStages2 * kAStage2;
constexpr int kOffBars2 = kOffB2 + kStages2 * kBStage2;   // full[6] empty[6] acc_full[2] acc_empty[2]
constexpr int kOffTmemSlot2 = kOffBars2 + (2 * kStages2 + 4) * 8;
constexpr int kOffAbort2 = kOffTmemSlot2 + 8;
constexpr int kSmemBytes2 = kOffAbort2 + 8;    // the base must be 1024-byte aligned (checked)

enum : uint32_t { kSite2Empty = 18, kSite2Full = 19, kSite2AccEmpty = 20, kSite2AccFull = 21 };

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `smem_addr` (an address in this CTA's shared memory) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
// TMA tile load into this CTA's shared memory whose bytes are counted on a barrier
// that may be the pair leader's (`cluster_bar`).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, int c0, int c1,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Converged warp, elected lane: D[tmem of both CTAs] (+)= A * B over the pair.
__device__ __forceinline__ void tc_mma_ss_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on `cluster_bar` (any CTA of the pair) once every MMA issued so far is done.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(cluster_bar)
      : "memory");
}

__device__ __forceinline__ void tile_coords2(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band_tiles = kGroupM2 * tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * kGroupM2;
  const int rows_in_band = min(tiles_m - first_m, kGroupM2);
  const int r = tile - band * band_tiles;
  tm = first_m + r % rows_in_band;
  tn = r / rows_in_band;
}

template <bool kF32Out>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 void* __restrict__ c_out, int M, int N, int K, int ldc, int groups, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t rank = cluster_ctarank();        // 0: the pair's leader
  const bool leader = rank == 0;

  const uint32_t a_base = base + kOffA2;
  const uint32_t b_base = base + kOffB2;
  const uint32_t bar_full = base + kOffBars2;
  const uint32_t bar_empty = bar_full + kStages2 * 8;
  const uint32_t bar_acc_full = bar_empty + kStages2 * 8;
  const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemSlot2);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kOffAbort2);
  const WaitCtx wctx{status, abort_flag};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // the swizzled tiles need a 1024-byte aligned base; both CTAs of a pair see the same offset
  const bool misaligned = (base & 1023u) != 0;
  if (misaligned && threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0u, kStatusTimeoutTag | (17u << 8));

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(bar_full + 8 * s, 2);      // one arrival per CTA of the pair (used in the leader)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 256);   // 128 epilogue threads per CTA (used in the leader)
    }
    mbar_fence_init();
  }
  if (warp == 1 && !misaligned) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers exist before anything remote is signalled
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int tiles_m = (M + kBM2 - 1) / kBM2;   // M % 128 == 0: the last row-tile may be its first half only
  const int tiles_n = (N + kBN2 - 1) / kBN2;
  const int tiles_per_group = tiles_m * tiles_n;
  const int total_tiles = tiles_per_group * groups;
  const int kiters = K / kBK2;
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  if (misaligned) {
    // nothing was allocated; leave together
  } else if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      const uint32_t leader_full = map_to_cta(bar_full, 0);
      uint32_t it = 0;
      for (int tile = pair; tile < total_tiles; tile += pairs) {
        int tm, tn;
        const int g = tile / tiles_per_group;
        tile_coords2(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
        const int a_row = g * M + tm * kBM2 + (int)rank * 128;
        const int b_row = g * N + tn * kBN2 + (int)rank * 128;
        for (int k = 0; k < kiters; ++k, ++it) {
          const uint32_t s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1u;
          mbar_wait(bar_empty + 8 * s, ph ^ 1u, wctx, kSite2Empty);
          mbar_arrive_expect_tx_cluster(leader_full + 8 * s, kStage2);
          tma_load_2d_pair(a_base + s * kAStage2, &tmap_a, k * kBK2, a_row, leader_full + 8 * s);
          tma_load_2d_pair(b_base + s * kBStage2, &tmap_b, k * kBK2, b_row, leader_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue (leader only; converged warp, elected lane) ----------------
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16_f32(kBM2, kBN2, false, false);
      const uint32_t peer_empty = map_to_cta(bar_empty, 1);
      const uint32_t peer_acc_full = map_to_cta(bar_acc_full, 1);
      uint32_t it = 0, t = 0;
      for (int tile = pair; tile < total_tiles; tile += pairs, ++t) {
        const uint32_t buf = t & 1u;
        const uint32_t aph = (t >> 1) & 1u;
        mbar_wait_warp(bar_acc_empty + 8 * buf, aph ^ 1u, wctx, kSite2AccEmpty);
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * kAccCols2;
        for (int k = 0; k < kiters; ++k, ++it) {
          const uint32_t s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1u;
          mbar_wait_warp(bar_full + 8 * s, ph, wctx, kSite2Full);
          tc_fence_after();
          const uint32_t da = sdesc_lo(a_base + s * kAStage2, 16);
          const uint32_t db = sdesc_lo(b_base + s * kBStage2, 16);
          constexpr uint32_t dhi = sdesc_hi(1024, kLayoutB128);
#pragma unroll
          for (int kk = 0; kk < kBK2 / 16; ++kk)
            tc_mma_ss_pair(d_tmem, da + 2 * kk, dhi, db + 2 * kk, dhi, idesc, (k | kk) != 0 ? 1u : 0u);
          tc_commit_pair(bar_empty + 8 * s);      // this CTA's slot
          tc_commit_pair(peer_empty + 8 * s);     // the peer's slot
        }
        tc_commit_pair(bar_acc_full + 8 * buf);
        tc_commit_pair(peer_acc_full + 8 * buf);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): this CTA's 128 rows of the tile ----------------
    const int quad = warp & 3;
    const int row_in_half = quad * 32 + lane;
    const uint32_t leader_acc_empty = map_to_cta(bar_acc_empty, 0);
    uint32_t t = 0;
    for (int tile = pair; tile < total_tiles; tile += pairs, ++t) {
      int tm, tn;
      const int g = tile / tiles_per_group;
      tile_coords2(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = t & 1u;
      const uint32_t aph = (t >> 1) & 1u;
      mbar_wait(bar_acc_full + 8 * buf, aph, wctx, kSite2AccFull);
      tc_fence_after();
      const size_t row = (size_t)g * M + (size_t)tm * kBM2 + rank * 128 + row_in_half;
      // in a half-filled last row-tile the peer's 128 rows lie past M (its A box read the
      // next group's rows or zero fill): computed, not stored
      const bool rows_valid = tm * kBM2 + (int)rank * 128 < M;
      const int col0 = tn * kBN2;
      const uint32_t t_row = tmem_addr(tmem, quad * 32, buf * kAccCols2);
#pragma unroll 1
      for (int c = 0; c < kBN2 / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(t_row + c * 32, v);
        tc_wait_ld_bind(v);
        const int col = col0 + c * 32;
        if (col < N && rows_valid) store_acc_chunk<kF32Out>(c_out, row, ldc, col, v);
      }
      tc_fence_before();
      mbar_arrive_cluster(leader_acc_empty + 8 * buf);
    }
  }

  // Neither CTA may leave (or free tensor memory) while the other can still signal
  // its barriers or while the leader's instructions still read its shared memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1 && !misaligned) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
}

}  // namespace

bool gemm_pair_eligible(const DeviceCtx& ctx, int groups, int M, int N, int K) {
  (void)K;
  // worth it once every pair of SMs has a tile (M % 128 == 0 is the entry points' contract;
  // a last row-tile may be half-filled)
  const long long tiles = (long long)groups * ((M + kBM2 - 1) / kBM2) * ((N + kBN2 - 1) / kBN2);
  return tiles >= ctx.sm_count / 2;
}

int launch_gemm_pair(const DeviceCtx& ctx, void* C, const void* A, const void* Bt, int groups, int M, int N,
                     int K, int ldc, unsigned flags, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = encode_tmap_bf16_2d(&ta, A, (uint64_t)groups * M, (uint64_t)K, (uint64_t)K * 2, 128, kBK2);
  if (rc != PTXB200_OK) return rc;
  rc = encode_tmap_bf16_2d(&tb, Bt, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K * 2, 128, kBK2);
  if (rc != PTXB200_OK) return rc;
  const long long tiles = (long long)groups * ((M + kBM2 - 1) / kBM2) * ((N + kBN2 - 1) / kBN2);
  const int max_pairs = ctx.sm_count / 2;
  const int pairs = tiles < max_pairs ? (int)tiles : max_pairs;
  uint32_t* status = status_word(ctx, stream);
  const int f32 = (flags & PTXB200_GEMM_F32_OUT) ? 1 : 0;
  static PerDeviceOnce attr_once;
  rc = attr_once.run(ctx.device, []() -> int {
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemBytes2));
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemBytes2));
    return PTXB200_OK;
  });
  if (rc != PTXB200_OK) return rc;
  if (f32)
    gemm_pair_kernel<true><<<2 * pairs, kThreads2, kSmemBytes2, stream>>>(ta, tb, C, M, N, K, ldc, groups, status);
  else
    gemm_pair_kernel<false><<<2 * pairs, kThreads2, kSmemBytes2, stream>>>(ta, tb, C, M, N, K, ldc, groups, status);
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

}  // namespace ptxb200
