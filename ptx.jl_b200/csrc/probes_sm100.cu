// Bring-up probes with known answers (ptxb200_selftest). They restate, as small
// CUDA kernels, what the reference checks with its single-instruction runtime
// tests: TMEM store->load identity (test/gpu/blackwell/tcgen05_roundtrip.jl:22-88)
// and one tcgen05.mma on known operands (tcgen05_mma_probe.jl:39-131,
// tcgen05_b128_probe.jl) -- here on non-uniform data and on exactly the operand
// forms the attention kernel uses: 128-byte-swizzled K-major Q/K tiles loaded by
// TMA, P as a tensor-memory A operand, V as an MN-major shared-memory B operand.
#include "attn_tiles.cuh"
#include "host_common.h"

namespace ptxb200 {
namespace {

constexpr uint32_t kSiteProbe = 15;

// ---- probe 0: TMEM round trip -------------------------------------------------
__global__ void __launch_bounds__(128, 1) tmem_roundtrip_kernel(uint32_t* out) {
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t row = warp * 32 + lane;
  const uint32_t t_row = tmem_addr(tmem, warp * 32, 0);
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = ((row << 16) | (uint32_t)(c * 32 + i)) ^ 0x5A5A0000u;
    tmem_st32(t_row + c * 32, v);
  }
  tc_wait_st();
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(t_row + c * 32, v);
    tc_wait_ld_bind(v);
#pragma unroll
    for (int i = 0; i < 32; ++i) out[row * 128 + c * 32 + i] = v[i];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}

// ---- probes 1, 2: one attention tile -------------------------------------------
// S = Q K^T (128 x 128) into TMEM columns 128..255, O = P V (128 x D) into columns
// 256..256+D, P (given, bf16) stored into TMEM columns 0..63 by the threads.
template <int D>
__global__ void __launch_bounds__(128, 1)
attn_tile_probe_kernel(const __grid_constant__ CUtensorMap tmap_q,
                       const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const uint32_t* __restrict__ p_bf16x2,
                       float* __restrict__ out_s, float* __restrict__ out_o, uint32_t* status) {
  using T = AttnTile<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem = base + T::kTileBytes;
  const uint32_t v_smem = base + 2 * T::kTileBytes;
  const uint32_t bar_tma = base + 3 * T::kTileBytes;
  const uint32_t bar_mma = bar_tma + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 3 * T::kTileBytes + 16);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + 3 * T::kTileBytes + 24);
  const WaitCtx wctx{status, abort_flag};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar_tma, 3 * T::kTileBytes);
    T::load(q_smem, &tmap_q, 0, bar_tma);
    T::load(k_smem, &tmap_k, 0, bar_tma);
    T::load(v_smem, &tmap_v, 0, bar_tma);
  }

  // P row of this thread -> TMEM columns 0..63 (packed bf16 pairs)
  const uint32_t row = warp * 32 + lane;
  const uint32_t t_row = tmem_addr(tmem, warp * 32, 0);
  for (int c = 0; c < 2; ++c) {
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = p_bf16x2[row * 64 + c * 32 + i];
    tmem_st32(t_row + c * 32, v);
  }
  tc_wait_st();
  tc_fence_before();
  __syncthreads();

  if (threadIdx.x == 0) {
    mbar_wait(bar_tma, 0, wctx, kSiteProbe);
    tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < T::kQKAtoms; ++kk)
      tc_mma_ss(tmem + 128, T::kmajor_lo(q_smem, kk), T::kKMajorHi, T::kmajor_lo(k_smem, kk),
                T::kKMajorHi, T::kIdescQK,
                kk != 0 ? 1u : 0u);
#pragma unroll
    for (int kk = 0; kk < T::kPVAtoms; ++kk)
      tc_mma_ts(tmem + 256, T::p_tmem(tmem, 0, kk), T::v_lo(v_smem, kk), T::kVHi, T::kIdescPV,
                kk != 0 ? 1u : 0u);
    tc_commit(bar_mma);
  }
  mbar_wait(bar_mma, 0, wctx, kSiteProbe);
  tc_fence_after();

  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(t_row + 128 + c * 32, v);
    tc_wait_ld_bind(v);
#pragma unroll
    for (int i = 0; i < 32; ++i) out_s[row * 128 + c * 32 + i] = __uint_as_float(v[i]);
  }
  for (int c = 0; c < D / 32; ++c) {
    uint32_t v[32];
    tmem_ld32(t_row + 256 + c * 32, v);
    tc_wait_ld_bind(v);
#pragma unroll
    for (int i = 0; i < 32; ++i) out_o[row * D + c * 32 + i] = __uint_as_float(v[i]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int D>
int launch_tile_probe(const DeviceCtx& ctx, void* out_s, void* out_o, const void* q, const void* k,
                      const void* v, const void* p, cudaStream_t stream) {
  using T = AttnTile<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_tmap_bf16_2d(&tq, q, 128, D, D * 2, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_2d(&tk, k, 128, D, D * 2, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_2d(&tv, v, 128, D, D * 2, 128, 64)) != PTXB200_OK) return rc;
  const int smem_bytes = 3 * T::kTileBytes + 64 + 1024;
  PTXB200_CUDA_TRY(cudaFuncSetAttribute(attn_tile_probe_kernel<D>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  attn_tile_probe_kernel<D><<<1, 128, smem_bytes, stream>>>(
      tq, tk, tv, reinterpret_cast<const uint32_t*>(p), reinterpret_cast<float*>(out_s),
      reinterpret_cast<float*>(out_o), status_word(ctx, stream));
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

// A bounded wait on a barrier that nobody arrives on: the wait gives up after its
// limit, records its first-blame code (site 15) in the status word and the kernel
// returns normally. What the host-side reporting is tested against.
__global__ void __launch_bounds__(32, 1) wait_expiry_kernel(uint32_t* out, uint32_t* status) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ uint32_t abort_word;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const WaitCtx wctx{status, &abort_word};
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(bar, 0, wctx, 15);
  __syncwarp();
  // a second wait in the same CTA returns at once through the abort flag
  bool ok2 = true;
  if (threadIdx.x == 1) ok2 = mbar_wait(bar, 0, wctx, 15);
  if (threadIdx.x == 0) out[0] = ok ? 1u : 0u;
  if (threadIdx.x == 1) out[1] = ok2 ? 1u : 0u;
  if (threadIdx.x == 0) out[2] = 0xD0E5u;   // the kernel ran to its end
}

// Throughput of the exponential unit of one SM, the second bound of the attention kernel
// (its softmax needs one ex2 per score: as many MUFU cycles per 128 x 128 tile as the tensor
// pipe needs at head dim 128, twice as many at head dim 64). One CTA of 16 warps; five
// passes, each timed with clock64 from the barrier before it to the barrier after it:
//   pass 0-2: 4, 8, 16 warps issue nothing but independent ex2.approx.ftz (8 chains each)
//   pass 3-4: 8, 16 warps run the softmax's inner mix per pair of scores -- one packed
//             fma (scale and basis), two ex2, one packed add (row sum), one bf16x2 pack
//   pass 5-6: 8, 16 warps issue ex2.approx.ftz.bf16x2 (two exponentials per instruction)
// out[2 * pass] = cycles, out[2 * pass + 1] = ex2 executed by the pass (all warps).
constexpr int kEx2Iters = 2048;
__global__ void __launch_bounds__(512, 1) ex2_throughput_kernel(uint32_t* out, float seed) {
  const int warp = threadIdx.x >> 5;
  __shared__ long long t_start;
  float sink = 0.0f;
  for (int pass = 0; pass < 7; ++pass) {
    const int warps = pass == 0 ? 4 : (pass == 1 || pass == 3 || pass == 5) ? 8 : 16;
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_start));
    __syncthreads();
    if (warp < warps) {
      if (pass < 3) {
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = seed - 0.01f * (float)(i + (threadIdx.x & 31));
#pragma unroll 1
        for (int r = 0; r < kEx2Iters; ++r) {
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i] = ex2_approx(a[i]) - 1.5f;   // stays in (-1.5, 0): never saturates
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sink += a[i];
      } else if (pass >= 5) {
        // packed bf16 form: one instruction, two exponentials
        uint32_t a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = pack_bf16x2(seed - 0.01f * i, seed - 0.02f * (threadIdx.x & 31));
#pragma unroll 1
        for (int r = 0; r < kEx2Iters; ++r) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t e;
            asm volatile("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(e) : "r"(a[i]));
            a[i] = e ^ 0x80008000u;   // negate both halves: stays in (-2, 0)
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sink += __uint_as_float(a[i] & 0x3F800000u);
      } else {
        float2 x[4], sum = make_float2(0.0f, 0.0f);
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = make_float2(seed - 0.1f * i, seed - 0.05f * i - 0.01f * (threadIdx.x & 31));
        const float2 sc = make_float2(0.999f, 0.999f), ng = make_float2(-0.01f, -0.01f);
#pragma unroll 1
        for (int r = 0; r < kEx2Iters; ++r) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 y = __ffma2_rn(x[i], sc, ng);
            float2 e;
            e.x = ex2_approx(y.x);
            e.y = ex2_approx(y.y);
            sum = __fadd2_rn(sum, e);
            acc ^= pack_bf16x2(e.x, e.y);
            x[i] = make_float2(e.x - 1.5f, e.y - 1.5f);
          }
        }
        sink += sum.x + sum.y + __uint_as_float(acc & 0x3F800000u);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      long long t_end;
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_end));
      out[2 * pass] = (uint32_t)(t_end - t_start);
      out[2 * pass + 1] = (uint32_t)(warps * 32 * kEx2Iters * 8 * (pass >= 5 ? 2 : 1));
    }
  }
  if (sink == 12345.678f) out[15] = 1;   // keeps the arithmetic alive
}

}  // namespace

int launch_selftest(const DeviceCtx& ctx, int which, void* out_s, void* out_o, const void* q,
                    const void* k, const void* v, const void* p, cudaStream_t stream) {
  switch (which) {
    case 0:
      tmem_roundtrip_kernel<<<1, 128, 0, stream>>>(reinterpret_cast<uint32_t*>(out_s));
      PTXB200_CUDA_TRY(cudaGetLastError());
      return PTXB200_OK;
    case 1: return launch_tile_probe<128>(ctx, out_s, out_o, q, k, v, p, stream);
    case 2: return launch_tile_probe<64>(ctx, out_s, out_o, q, k, v, p, stream);
    case 3:
      wait_expiry_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<uint32_t*>(out_s), status_word(ctx, stream));
      PTXB200_CUDA_TRY(cudaGetLastError());
      return PTXB200_OK;
    case 4:
      ex2_throughput_kernel<<<1, 512, 0, stream>>>(reinterpret_cast<uint32_t*>(out_s), -0.75f);
      PTXB200_CUDA_TRY(cudaGetLastError());
      return PTXB200_OK;
    default: return PTXB200_E_INVALID;
  }
}

}  // namespace ptxb200
