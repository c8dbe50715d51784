// Row-wise fp32 kernels either side of attention in a transformer block: softmax,
// RMS norm, layer norm (one output row from one input row) and SwiGLU (elementwise).
//
// The reference ships these as one-CTA-per-row kernels with the row held in
// registers between the reduction passes (test/gpu/softmax.jl:30-140,
// test/gpu/rms_norm.jl:30-106, test/gpu/layer_norm.jl:24-122,
// test/gpu/swiglu.jl:31-69): N must be a multiple of block*4 and at most
// block*64. All four are bound by HBM: 8 bytes per element (one fp32 read, one fp32
// write; the weight vectors stay in cache), 12 for SwiGLU.
//
// What is kept: one read of X, the row in registers across the passes, 128-bit
// accesses. What is different:
//   * the threads that share a row are chosen from the row length: one warp per row
//     up to 2048 columns (reductions are five shuffles, no shared memory, no block
//     barrier; four rows per CTA), 256 threads up to 8192, 1024 threads up to 32768;
//   * any N that is a multiple of 4 (ragged rows are guarded per 128-bit access);
//   * a persistent grid sized from the SM count, rows handed out round-robin, so
//     small rows do not pay one CTA launch each;
//   * X and Y are accessed with the streaming cache hints (read once, written
//     once), the weight vectors through the read-only path;
//   * one reduction per row instead of two: softmax merges (max, sum of exponentials)
//     pairs by the online-softmax rule and rescales once; layer norm merges (count,
//     mean, centred sum of squares) triples by Chan's rule, which also keeps its
//     accuracy for rows with a large mean, where the reference's E[x^2] - mean^2
//     cancels. With several warps per row that is one block barrier per row.
#include "host_common.h"
#include "sm100_prims.cuh"

namespace ptxb200 {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

enum RowOp : int { kOpSoftmax = 0, kOpRmsNorm = 1, kOpLayerNorm = 2 };

struct RowParams {
  float* y;
  const float* x;
  const float* w;      // rms_norm, layer_norm
  const float* bias;   // layer_norm
  int rows;
  int n4;              // N / 4
  float inv_n;
  float eps;
};

// Reductions over the kTpr threads that share a row. Each op needs exactly one:
// a sum (RMS norm), a (max, sum of exponentials) pair merged with the online-softmax
// rule, or a (count, mean, M2) triple merged with Chan's rule (layer norm). With
// more than one warp per row the warps' partials meet in shared memory behind ONE
// block barrier: `red` alternates between two buffers from row to row, so a warp
// writing the next row's partials cannot overrun a reader of this row's (it would
// first have to pass the next row's barrier, which the reader also has to reach).
struct Pair { float m, s; };          // running max and sum of 2^((x - m) log2 e)
struct Moments { float n, mean, m2; };

__device__ __forceinline__ Pair merge(Pair a, Pair b) {
  const float m = fmaxf(a.m, b.m);
  // a side that holds only padding has m = -inf and s = 0; (-inf) - (-inf) must not reach ex2
  const float fa = a.m == m ? 1.0f : ex2_approx((a.m - m) * kLog2e);
  const float fb = b.m == m ? 1.0f : ex2_approx((b.m - m) * kLog2e);
  return {m, a.s * fa + b.s * fb};
}
__device__ __forceinline__ Moments merge(Moments a, Moments b) {
  const float n = a.n + b.n;
  const float rb = n > 0.0f ? b.n / n : 0.0f;
  const float d = b.mean - a.mean;
  return {n, a.mean + d * rb, a.m2 + b.m2 + d * d * a.n * rb};
}
__device__ __forceinline__ float merge(float a, float b) { return a + b; }

__device__ __forceinline__ float shfl_xor(float v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ Pair shfl_xor(Pair v, int o) { return {shfl_xor(v.m, o), shfl_xor(v.s, o)}; }
__device__ __forceinline__ Moments shfl_xor(Moments v, int o) {
  return {shfl_xor(v.n, o), shfl_xor(v.mean, o), shfl_xor(v.m2, o)};
}
__device__ __forceinline__ float identity(float) { return 0.0f; }
__device__ __forceinline__ Pair identity(Pair) { return {-INFINITY, 0.0f}; }
__device__ __forceinline__ Moments identity(Moments) { return {0.0f, 0.0f, 0.0f}; }

template <int kTpr, typename T>
__device__ __forceinline__ T row_reduce(T v, T* red /* [2][32] */, int parity) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = merge(v, shfl_xor(v, o));
  if (kTpr > 32) {
    constexpr int kWarps = kTpr / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* buf = red + parity * 32;
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    v = lane < kWarps ? buf[lane] : identity(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = merge(v, shfl_xor(v, o));
  }
  return v;
}

// kTpr threads per row, up to kVec 128-bit accesses per thread.
template <int kOp, int kTpr, int kVec>
__global__ void __launch_bounds__(kTpr == 32 ? 128 : kTpr)
rowwise_kernel(const RowParams p) {
  __shared__ float red_raw[2 * 32 * 3];
  constexpr int kRowsPerCta = kTpr == 32 ? 4 : 1;
  const int t = threadIdx.x % kTpr;                 // position within the row's thread group
  const int sub = threadIdx.x / kTpr;               // which of the CTA's rows
  const float4* w4 = reinterpret_cast<const float4*>(p.w);
  const float4* b4 = reinterpret_cast<const float4*>(p.bias);
  int parity = 0;

  for (int row0 = blockIdx.x * kRowsPerCta; row0 < p.rows;
       row0 += gridDim.x * kRowsPerCta, parity ^= 1) {
    const int row = row0 + sub;
    const bool live = row < p.rows;   // a CTA's last group of rows may be partial (warp-per-row only)
    const float4* x4 = reinterpret_cast<const float4*>(p.x) + (size_t)(live ? row : 0) * p.n4;
    float4* y4 = reinterpret_cast<float4*>(p.y) + (size_t)(live ? row : 0) * p.n4;

    float4 v[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int c = t + i * kTpr;
      const float fill = kOp == kOpSoftmax ? -INFINITY : 0.0f;
      v[i] = (live && c < p.n4) ? __ldcs(x4 + c) : make_float4(fill, fill, fill, fill);
    }

    if (kOp == kOpSoftmax) {
      float m = -INFINITY;
#pragma unroll
      for (int i = 0; i < kVec; ++i) m = fmaxf(fmaxf(m, fmaxf(v[i].x, v[i].y)), fmaxf(v[i].z, v[i].w));
      // exponentials against this thread's own maximum, rescaled once the row's is known
      const float neg = m == -INFINITY ? 0.0f : -m * kLog2e;
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        v[i].x = ex2_approx(fmaf(v[i].x, kLog2e, neg));
        v[i].y = ex2_approx(fmaf(v[i].y, kLog2e, neg));
        v[i].z = ex2_approx(fmaf(v[i].z, kLog2e, neg));
        v[i].w = ex2_approx(fmaf(v[i].w, kLog2e, neg));
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);   // padding lanes hold 2^-inf = 0
      }
      const Pair tot = row_reduce<kTpr>(Pair{m, s}, reinterpret_cast<Pair*>(red_raw), parity);
      const float f = (m == tot.m ? 1.0f : ex2_approx((m - tot.m) * kLog2e)) / tot.s;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const int c = t + i * kTpr;
        if (live && c < p.n4)
          __stcs(y4 + c, make_float4(v[i].x * f, v[i].y * f, v[i].z * f, v[i].w * f));
      }
    } else if (kOp == kOpRmsNorm) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < kVec; ++i)
        s += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      s = row_reduce<kTpr>(s, red_raw, parity);
      const float rstd = rsqrtf(s * p.inv_n + p.eps);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const int c = t + i * kTpr;
        if (live && c < p.n4) {
          const float4 w = __ldg(w4 + c);
          __stcs(y4 + c, make_float4(v[i].x * rstd * w.x, v[i].y * rstd * w.y, v[i].z * rstd * w.z,
                                     v[i].w * rstd * w.w));
        }
      }
    } else {
      // this thread's own count, mean and centred sum of squares
      float s = 0.0f, cnt = 0.0f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);   // padding lanes hold zeros
        if (t + i * kTpr < p.n4) cnt += 4.0f;
      }
      const float mean_t = cnt > 0.0f ? s / cnt : 0.0f;
      float q = 0.0f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        if (t + i * kTpr < p.n4) {
          const float dx = v[i].x - mean_t, dy = v[i].y - mean_t, dz = v[i].z - mean_t, dw = v[i].w - mean_t;
          q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
      }
      const Moments tot = row_reduce<kTpr>(Moments{cnt, mean_t, q}, reinterpret_cast<Moments*>(red_raw), parity);
      const float rstd = rsqrtf(tot.m2 * p.inv_n + p.eps);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const int c = t + i * kTpr;
        if (live && c < p.n4) {
          const float4 w = __ldg(w4 + c);
          const float4 b = __ldg(b4 + c);
          __stcs(y4 + c, make_float4(fmaf((v[i].x - tot.mean) * rstd, w.x, b.x),
                                     fmaf((v[i].y - tot.mean) * rstd, w.y, b.y),
                                     fmaf((v[i].z - tot.mean) * rstd, w.z, b.z),
                                     fmaf((v[i].w - tot.mean) * rstd, w.w, b.w)));
        }
      }
    }
  }
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // g * sigmoid(g) * u with exp(-g) = 2^(-g log2 e) (test/gpu/swiglu.jl:33-40)
  return g * rcp_approx(1.0f + ex2_approx(-g * kLog2e)) * u;
}

constexpr int kSwigluThreads = 256;
constexpr int kSwigluUnroll = 4;   // independent 128-bit load pairs in flight per thread

__global__ void __launch_bounds__(kSwigluThreads)
swiglu_kernel(float* __restrict__ out, const float* __restrict__ gate, const float* __restrict__ up,
              size_t n4) {
  const float4* g4 = reinterpret_cast<const float4*>(gate);
  const float4* u4 = reinterpret_cast<const float4*>(up);
  float4* o4 = reinterpret_cast<float4*>(out);
  const size_t stride = (size_t)gridDim.x * kSwigluThreads;
  for (size_t base = (size_t)blockIdx.x * kSwigluThreads + threadIdx.x; base < n4;
       base += stride * kSwigluUnroll) {
    float4 g[kSwigluUnroll], u[kSwigluUnroll];
#pragma unroll
    for (int i = 0; i < kSwigluUnroll; ++i) {
      const size_t c = base + i * stride;
      if (c < n4) {
        g[i] = __ldcs(g4 + c);
        u[i] = __ldcs(u4 + c);
      }
    }
#pragma unroll
    for (int i = 0; i < kSwigluUnroll; ++i) {
      const size_t c = base + i * stride;
      if (c < n4)
        __stcs(o4 + c, make_float4(silu_mul(g[i].x, u[i].x), silu_mul(g[i].y, u[i].y),
                                   silu_mul(g[i].z, u[i].z), silu_mul(g[i].w, u[i].w)));
    }
  }
}

template <int kOp, int kTpr, int kVec>
int launch_one(const DeviceCtx& ctx, const RowParams& p, cudaStream_t stream) {
  constexpr int kRowsPerCta = kTpr == 32 ? 4 : 1;
  constexpr int kThreads = kTpr == 32 ? 128 : kTpr;
  // enough resident CTAs per SM to keep ~2048 threads' worth of loads in flight
  const int ctas_per_sm = 2048 / kThreads > 8 ? 8 : 2048 / kThreads;
  const long long want = ((long long)p.rows + kRowsPerCta - 1) / kRowsPerCta;
  const long long cap = (long long)ctx.sm_count * ctas_per_sm;
  const int grid = (int)(want < cap ? want : cap);
  rowwise_kernel<kOp, kTpr, kVec><<<grid, kThreads, 0, stream>>>(p);
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

template <int kOp>
int dispatch(const DeviceCtx& ctx, const RowParams& p, cudaStream_t stream) {
  const int n4 = p.n4;
  if (n4 <= 32 * 16) {
    const int per = (n4 + 31) / 32;
    if (per <= 1) return launch_one<kOp, 32, 1>(ctx, p, stream);
    if (per <= 2) return launch_one<kOp, 32, 2>(ctx, p, stream);
    if (per <= 4) return launch_one<kOp, 32, 4>(ctx, p, stream);
    if (per <= 8) return launch_one<kOp, 32, 8>(ctx, p, stream);
    return launch_one<kOp, 32, 16>(ctx, p, stream);
  }
  if (n4 <= 256 * 8) {
    const int per = (n4 + 255) / 256;
    if (per <= 4) return launch_one<kOp, 256, 4>(ctx, p, stream);
    return launch_one<kOp, 256, 8>(ctx, p, stream);
  }
  const int per = (n4 + 1023) / 1024;
  if (per <= 4) return launch_one<kOp, 1024, 4>(ctx, p, stream);
  return launch_one<kOp, 1024, 8>(ctx, p, stream);
}

}  // namespace

int launch_rowwise(const DeviceCtx& ctx, int op, float* y, const float* x, const float* w,
                   const float* bias, int rows, int n, float eps, cudaStream_t stream) {
  RowParams p;
  p.y = y;
  p.x = x;
  p.w = w;
  p.bias = bias;
  p.rows = rows;
  p.n4 = n / 4;
  p.inv_n = 1.0f / (float)n;
  p.eps = eps;
  switch (op) {
    case kOpSoftmax: return dispatch<kOpSoftmax>(ctx, p, stream);
    case kOpRmsNorm: return dispatch<kOpRmsNorm>(ctx, p, stream);
    case kOpLayerNorm: return dispatch<kOpLayerNorm>(ctx, p, stream);
    default: return PTXB200_E_INVALID;
  }
}

int launch_swiglu(const DeviceCtx& ctx, float* out, const float* gate, const float* up, size_t n,
                  cudaStream_t stream) {
  const size_t n4 = n / 4;
  const size_t per_cta = (size_t)kSwigluThreads * kSwigluUnroll;
  const size_t want = (n4 + per_cta - 1) / per_cta;
  const size_t cap = (size_t)ctx.sm_count * 8;
  const int grid = (int)(want < cap ? want : cap);
  swiglu_kernel<<<grid, kSwigluThreads, 0, stream>>>(out, gate, up, n4);
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

}  // namespace ptxb200
