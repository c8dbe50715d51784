// Host-side plumbing shared by the entry points: per-device context (SM count,
// capability, status/workspace words), tensor-map encoding through the driver
// entry point, and error bookkeeping.
//
// Reference counterpart: ext/CUDACoreExt.jl:44-71,114-140 (cuTensorMapEncodeTiled
// call and descriptor upload). Here the 128-byte tensor map is passed to the
// kernel by value as a __grid_constant__ parameter, so there is no upload step
// and no per-call device allocation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <vector>

#include "../../include/ptxb200.h"

namespace ptxb200 {

// Words of the per-device workspace (uint32 each): one first-blame status word per
// stream that has launched through the library on the device (slot 0 .. kWsStatusSlots-1,
// handed out in order of first use; once every slot is taken further streams share
// slots by hash).
enum : int {
  kWsStatusSlots = 128,
  kWsWords = 256,
};

struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  uint32_t* workspace = nullptr;  // kWsWords uint32 on the device, zero-initialised once
};

// Device address of the status word that launches on `stream` report to.
uint32_t* status_word(const DeviceCtx& ctx, cudaStream_t stream);

// Runs `f` (returning PTXB200_OK or an error code) once per device ordinal, under a lock;
// later calls for that device return PTXB200_OK at once. For the per-kernel
// cudaFuncSetAttribute calls of the launchers.
class PerDeviceOnce {
 public:
  template <class F>
  int run(int device, F&& f) {
    if (device < 0) return PTXB200_E_INVALID;
    std::lock_guard<std::mutex> lock(mu_);
    if ((int)done_.size() <= device) done_.resize(device + 1, 0);
    if (!done_[device]) {
      const int rc = f();
      if (rc != PTXB200_OK) return rc;
      done_[device] = 1;
    }
    return PTXB200_OK;
  }

 private:
  std::mutex mu_;
  std::vector<char> done_;
};

// Scratch memory the library keeps per (device, stream, purpose) for kernels that park
// partial results in global memory: launches on one stream run one after the other and
// may share a buffer, launches on different streams may overlap and must not.
//  * scratch_acquire returns a buffer of at least `bytes` for (current device, stream,
//    kind), allocating or growing it when needed (cudaMalloc: the first such launch on a
//    stream must come outside stream capture).
//  * scratch_mark_used, called after the kernels that use the buffer are enqueued, records
//    an event so that the buffer can later be recycled safely.
//  * At most kScratchMaxEntries buffers exist per process: when a new (device, stream,
//    kind) needs one and the table is full, the least recently used entry is waited for
//    (its event) and freed. Everything is freed by ptxb200_shutdown.
enum : int { kScratchGemmSlabs = 0, kScratchAttnParts = 1 };
constexpr int kScratchMaxEntries = 16;
struct ScratchLease {
  void* ptr = nullptr;
  int entry = -1;
  bool fresh = false;      // allocated by this call: contents undefined
  uint32_t epoch = 0;      // counts the leases of this buffer, from 1; never 0
};
int scratch_acquire(const DeviceCtx& ctx, cudaStream_t stream, int kind, size_t bytes, ScratchLease* out);
int scratch_mark_used(const ScratchLease& lease, cudaStream_t stream);
void scratch_release_all();

// Context of the device current in the calling thread (created on first use).
// Returns PTXB200_OK or a negative code.
int current_ctx(DeviceCtx** out);

// Every cached context (for shutdown).
int release_all_ctx();

// Record / fetch the calling thread's last CUDA error text.
void set_cuda_error(const char* what, cudaError_t e);
void set_error_text(const char* what);
const char* get_cuda_error();

// 2-D row-major bf16 tensor map: `rows` x `cols` elements, row pitch
// `row_pitch_bytes`, box `box_rows` x `box_cols`, 128-byte swizzle.
// (ext/CUDACoreExt.jl:114-131: dims innermost-first = (cols, rows).)
int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols);

// 3-D bf16 tensor map over `slices` contiguous row-major matrices of `rows` x `cols`
// (one per batch*head), box 1 x `box_rows` x `box_cols`, 128-byte swizzle. Rows past
// the end of a slice read as zeros instead of the next slice's rows.
int encode_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t slices, uint64_t rows, uint64_t cols,
                        uint32_t box_rows, uint32_t box_cols);

#define PTXB200_CUDA_TRY(expr)                         \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) {                           \
      ::ptxb200::set_cuda_error(#expr, _e);            \
      return PTXB200_E_CUDA;                           \
    }                                                  \
  } while (0)

// Kernel launchers (one per .cu file).
int launch_gemm(const DeviceCtx& ctx, void* C, const void* A, const void* Bt, int groups, int M, int N,
                int K, int ldc, unsigned flags, cudaStream_t stream);
int launch_fa_fwd(const DeviceCtx& ctx, void* O, void* lse, const void* Q, const void* K,
                  const void* V, int B, int H, int H_kv, int S, int D, float sm_scale, int causal,
                  unsigned flags, void* dbg, uint32_t* status, cudaStream_t stream);
// The work distribution launch_fa_fwd would pick, as plain ints (fa_fwd_sm100.cu).
int describe_fa_plan(int BH, int S, int causal, unsigned flags, int sm_count, int* out, int cap);
// CTA-pair GEMM (gemm2_sm100.cu): whether it applies to a shape, and its launcher.
bool gemm_pair_eligible(const DeviceCtx& ctx, int groups, int M, int N, int K);
int launch_gemm_pair(const DeviceCtx& ctx, void* C, const void* A, const void* Bt, int groups, int M, int N,
                     int K, int ldc, unsigned flags, cudaStream_t stream);
// Row-wise fp32 kernels; op: 0 softmax, 1 RMS norm, 2 layer norm.
int launch_rowwise(const DeviceCtx& ctx, int op, float* y, const float* x, const float* w,
                   const float* bias, int rows, int n, float eps, cudaStream_t stream);
int launch_swiglu(const DeviceCtx& ctx, float* out, const float* gate, const float* up, size_t n,
                  cudaStream_t stream);
int launch_selftest(const DeviceCtx& ctx, int which, void* out_s, void* out_o, const void* q,
                    const void* k, const void* v, const void* p, cudaStream_t stream);

}  // namespace ptxb200
