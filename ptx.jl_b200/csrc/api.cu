// C-ABI entry points and host plumbing of libptxb200. See include/ptxb200.h for
// the contract of each call.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "host_common.h"
#include "sm100_prims.cuh"

namespace ptxb200 {

// ---------------------------------------------------------------------------
// error text
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_cuda_error(const char* what, cudaError_t e) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}
void set_error_text(const char* what) { snprintf(g_err, sizeof(g_err), "%s", what); }
const char* get_cuda_error() { return g_err; }

// ---------------------------------------------------------------------------
// per-device contexts
// ---------------------------------------------------------------------------
static std::mutex g_mu;
static std::vector<DeviceCtx*> g_ctx;  // indexed by device ordinal
// status slot of every stream seen per device (guarded by g_mu)
static std::vector<std::unordered_map<cudaStream_t, int>> g_slots;

int current_ctx(DeviceCtx** out) {
  int dev = -1;
  PTXB200_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_mu);
  if ((int)g_ctx.size() <= dev) {
    g_ctx.resize(dev + 1, nullptr);
    g_slots.resize(dev + 1);
  }
  if (g_ctx[dev] == nullptr) {
    DeviceCtx c;
    c.device = dev;
    PTXB200_CUDA_TRY(cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev));
    PTXB200_CUDA_TRY(cudaDeviceGetAttribute(&c.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    PTXB200_CUDA_TRY(cudaDeviceGetAttribute(&c.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (c.cc_major != 10) {
      set_error_text("current device is not compute capability 10.x (sm_100a code only)");
      return PTXB200_E_DEVICE;
    }
    PTXB200_CUDA_TRY(cudaMalloc((void**)&c.workspace, kWsWords * sizeof(uint32_t)));
    PTXB200_CUDA_TRY(cudaMemset(c.workspace, 0, kWsWords * sizeof(uint32_t)));
    g_ctx[dev] = new DeviceCtx(c);
  }
  *out = g_ctx[dev];
  return PTXB200_OK;
}

uint32_t* status_word(const DeviceCtx& ctx, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto& slots = g_slots[ctx.device];
  auto it = slots.find(stream);
  if (it == slots.end()) {
    const int next = (int)slots.size();
    // every slot taken: share by hash (a status read may then name a neighbour's failure)
    const int slot = next < kWsStatusSlots
                         ? next
                         : (int)((reinterpret_cast<uintptr_t>(stream) * 0x9E3779B97F4A7C15ull) >> 57) % kWsStatusSlots;
    it = slots.emplace(stream, slot).first;
  }
  return ctx.workspace + it->second;
}

int release_all_ctx() {
  scratch_release_all();
  std::lock_guard<std::mutex> lock(g_mu);
  int prev = -1;
  cudaGetDevice(&prev);
  for (DeviceCtx*& c : g_ctx) {
    if (c == nullptr) continue;
    if (cudaSetDevice(c->device) == cudaSuccess && c->workspace != nullptr) cudaFree(c->workspace);
    delete c;
    c = nullptr;
  }
  for (auto& m : g_slots) m.clear();
  if (prev >= 0) cudaSetDevice(prev);
  return PTXB200_OK;
}

// ---------------------------------------------------------------------------
// scratch buffers per (device, stream, purpose)
// ---------------------------------------------------------------------------
namespace {
struct ScratchEntry {
  bool live = false;
  int device = -1;
  cudaStream_t stream = nullptr;
  int kind = 0;
  void* ptr = nullptr;
  size_t bytes = 0;
  uint32_t epoch = 0;
  cudaEvent_t done = nullptr;   // recorded behind the last launch that used the buffer
  bool recorded = false;
  unsigned long long last_use = 0;
};
std::mutex g_scratch_mu;
ScratchEntry g_scratch[kScratchMaxEntries];
unsigned long long g_scratch_clock = 0;

// Waits for the entry's last user and frees its buffer (its device must be current or
// is made current for the call). Lock held by the caller.
void scratch_drop(ScratchEntry& e) {
  if (!e.live) return;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != e.device) cudaSetDevice(e.device);
  if (e.recorded) cudaEventSynchronize(e.done);
  if (e.ptr != nullptr) cudaFree(e.ptr);
  if (e.done != nullptr) cudaEventDestroy(e.done);
  if (prev >= 0 && prev != e.device) cudaSetDevice(prev);
  e = ScratchEntry();
}
}  // namespace

int scratch_acquire(const DeviceCtx& ctx, cudaStream_t stream, int kind, size_t bytes, ScratchLease* out) {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  int hit = -1, free_slot = -1, lru = -1;
  for (int i = 0; i < kScratchMaxEntries; ++i) {
    ScratchEntry& e = g_scratch[i];
    if (!e.live) {
      if (free_slot < 0) free_slot = i;
      continue;
    }
    if (e.device == ctx.device && e.stream == stream && e.kind == kind) hit = i;
    if (lru < 0 || e.last_use < g_scratch[lru].last_use) lru = i;
  }
  if (hit >= 0 && g_scratch[hit].bytes < bytes) {
    scratch_drop(g_scratch[hit]);   // too small: wait for its last user, then allocate anew
    free_slot = hit;
    hit = -1;
  }
  out->fresh = false;
  if (hit < 0) {
    out->fresh = true;
    if (free_slot < 0) {
      scratch_drop(g_scratch[lru]);
      free_slot = lru;
    }
    ScratchEntry& e = g_scratch[free_slot];
    PTXB200_CUDA_TRY(cudaMalloc(&e.ptr, bytes));
    cudaError_t ee = cudaEventCreateWithFlags(&e.done, cudaEventDisableTiming);
    if (ee != cudaSuccess) {
      cudaFree(e.ptr);
      e = ScratchEntry();
      set_cuda_error("cudaEventCreateWithFlags", ee);
      return PTXB200_E_CUDA;
    }
    e.live = true;
    e.device = ctx.device;
    e.stream = stream;
    e.kind = kind;
    e.bytes = bytes;
    hit = free_slot;
  }
  g_scratch[hit].last_use = ++g_scratch_clock;
  if (++g_scratch[hit].epoch == 0) g_scratch[hit].epoch = 1;
  out->epoch = g_scratch[hit].epoch;
  out->ptr = g_scratch[hit].ptr;
  out->entry = hit;
  return PTXB200_OK;
}

int scratch_mark_used(const ScratchLease& lease, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (lease.entry < 0 || lease.entry >= kScratchMaxEntries) return PTXB200_E_INVALID;
  ScratchEntry& e = g_scratch[lease.entry];
  if (!e.live || e.ptr != lease.ptr) return PTXB200_OK;   // recycled meanwhile by another thread's eviction
  PTXB200_CUDA_TRY(cudaEventRecord(e.done, stream));
  e.recorded = true;
  return PTXB200_OK;
}

void scratch_release_all() {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  for (ScratchEntry& e : g_scratch) scratch_drop(e);
}

// ---------------------------------------------------------------------------
// tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

int encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error_text("cuTensorMapEncodeTiled: driver entry point not found");
    return PTXB200_E_DRIVER;
  }
  cuuint64_t dims[2] = {cols, rows};               // innermost first
  cuuint64_t strides[1] = {row_pitch_bytes};       // stride of dim 1; dim 0 is implicit
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return PTXB200_E_DRIVER;
  }
  return PTXB200_OK;
}

int encode_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t slices, uint64_t rows, uint64_t cols,
                        uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error_text("cuTensorMapEncodeTiled: driver entry point not found");
    return PTXB200_E_DRIVER;
  }
  cuuint64_t dims[3] = {cols, rows, slices};                       // innermost first
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};             // bytes, of dims 1 and 2
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
    return PTXB200_E_DRIVER;
  }
  return PTXB200_OK;
}

}  // namespace ptxb200

using namespace ptxb200;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" {

int ptxb200_version(void) { return 100; /* 0.1.0 */ }

const char* ptxb200_last_cuda_error(void) { return get_cuda_error(); }

const char* ptxb200_strerror(int code) {
  switch (code) {
    case PTXB200_OK: return "ok";
    case PTXB200_E_INVALID: return "invalid argument (null pointer, non-positive size or unknown flag)";
    case PTXB200_E_SHAPE: return "shape outside the supported contract";
    case PTXB200_E_ALIGN: return "pointer or leading dimension is not 16-byte aligned";
    case PTXB200_E_CUDA: return "CUDA runtime error (see ptxb200_last_cuda_error)";
    case PTXB200_E_DRIVER: return "cuTensorMapEncodeTiled unavailable or failed";
    case PTXB200_E_DEVICE: return "current device is not compute capability 10.x";
    case PTXB200_E_CAPACITY: return "request exceeds a fixed capacity of this entry point";
    default: break;
  }
  if (code > 0 && ((uint32_t)code & 0xFF000000u) == kStatusTimeoutTag) {
    static thread_local char buf[160];
    static const char* const sites[] = {
        "?",            "gemm:empty",    "gemm:full",    "gemm:acc_empty", "gemm:acc_full",
        "fa:load.q_free", "fa:load.kv_free", "fa:mma.q_full", "fa:mma.kv_full", "fa:mma.p_full",
        "fa:mma.o_ready", "fa:softmax.s_full", "fa:corr.alpha", "fa:corr.l_ready",
        "fa:corr.o_done", "probe", "-", "shared memory base not 1024-byte aligned",
        "gemm2:empty", "gemm2:full", "gemm2:acc_empty", "gemm2:acc_full",
        "fa:softmax.l_free", "fa:corr.combine_piece",
    };
    unsigned site = ((unsigned)code >> 8) & 0xFFu;
    const char* name = site < sizeof(sites) / sizeof(sites[0]) ? sites[site] : "?";
    snprintf(buf, sizeof(buf),
             "device-side bounded wait ran out at site %u (%s), cta%%128=%u, parity=%u; outputs "
             "of that launch are invalid",
             site, name, ((unsigned)code >> 1) & 0x7Fu, (unsigned)code & 1u);
    return buf;
  }
  return "unknown code";
}

int gemm_bf16(void* C, const void* A, const void* Bt, int M, int N, int K, int ldc, unsigned flags,
              void* stream) {
  if (C == nullptr || A == nullptr || Bt == nullptr) return PTXB200_E_INVALID;
  if (M <= 0 || N <= 0 || K <= 0 || ldc < N) return PTXB200_E_INVALID;
  if (flags & ~(PTXB200_GEMM_F32_OUT | PTXB200_GEMM_NO_SPLIT | PTXB200_GEMM_ONE_CTA)) return PTXB200_E_INVALID;
  if (M % 128 != 0 || N % 128 != 0 || K % 64 != 0) return PTXB200_E_SHAPE;
  const size_t esz = (flags & PTXB200_GEMM_F32_OUT) ? 4 : 2;
  if (!aligned16(C) || !aligned16(A) || !aligned16(Bt) || ((size_t)ldc * esz) % 16 != 0)
    return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_gemm(*ctx, C, A, Bt, 1, M, N, K, ldc, flags, (cudaStream_t)stream);
}

int gemm_bf16_grouped(void* C, const void* A, const void* Bt, int G, int M, int N, int K, int ldc,
                      unsigned flags, void* stream) {
  if (C == nullptr || A == nullptr || Bt == nullptr) return PTXB200_E_INVALID;
  if (G <= 0 || M <= 0 || N <= 0 || K <= 0 || ldc < N) return PTXB200_E_INVALID;
  if (flags & ~(PTXB200_GEMM_F32_OUT | PTXB200_GEMM_NO_SPLIT | PTXB200_GEMM_ONE_CTA)) return PTXB200_E_INVALID;
  if (M % 128 != 0 || N % 64 != 0 || K % 64 != 0) return PTXB200_E_SHAPE;
  if ((long long)G * M >= (1ll << 31) || (long long)G * N >= (1ll << 31)) return PTXB200_E_SHAPE;
  const size_t esz = (flags & PTXB200_GEMM_F32_OUT) ? 4 : 2;
  if (!aligned16(C) || !aligned16(A) || !aligned16(Bt) || ((size_t)ldc * esz) % 16 != 0)
    return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_gemm(*ctx, C, A, Bt, G, M, N, K, ldc, flags, (cudaStream_t)stream);
}

namespace {
int rowwise_entry(int op, void* y, const void* x, const void* w, const void* bias, int rows, int n,
                  float eps, void* stream) {
  if (y == nullptr || x == nullptr || (op >= 1 && w == nullptr) || (op == 2 && bias == nullptr))
    return PTXB200_E_INVALID;
  if (rows <= 0 || n <= 0) return PTXB200_E_INVALID;
  if (op >= 1 && !(eps >= 0.0f)) return PTXB200_E_INVALID;
  if (n % 4 != 0 || n > 32768) return PTXB200_E_SHAPE;
  if (!aligned16(y) || !aligned16(x) || (w != nullptr && !aligned16(w)) ||
      (bias != nullptr && !aligned16(bias)))
    return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_rowwise(*ctx, op, (float*)y, (const float*)x, (const float*)w, (const float*)bias,
                        rows, n, eps, (cudaStream_t)stream);
}
}  // namespace

int softmax_f32(void* Y, const void* X, int rows, int N, void* stream) {
  return rowwise_entry(0, Y, X, nullptr, nullptr, rows, N, 0.0f, stream);
}

int rms_norm_f32(void* Y, const void* X, const void* W, int rows, int N, float eps, void* stream) {
  return rowwise_entry(1, Y, X, W, nullptr, rows, N, eps, stream);
}

int layer_norm_f32(void* Y, const void* X, const void* W, const void* Bias, int rows, int N,
                   float eps, void* stream) {
  return rowwise_entry(2, Y, X, W, Bias, rows, N, eps, stream);
}

int swiglu_f32(void* out, const void* gate, const void* up, long long n, void* stream) {
  if (out == nullptr || gate == nullptr || up == nullptr) return PTXB200_E_INVALID;
  if (n <= 0) return PTXB200_E_INVALID;
  if (n % 4 != 0) return PTXB200_E_SHAPE;
  if (!aligned16(out) || !aligned16(gate) || !aligned16(up)) return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_swiglu(*ctx, (float*)out, (const float*)gate, (const float*)up, (size_t)n,
                       (cudaStream_t)stream);
}

int fa_fwd_bf16_ex(void* O, void* lse, const void* Q, const void* K, const void* V, int B, int H,
                   int H_kv, int S, int D, float sm_scale, int causal, unsigned flags, void* dbg,
                   void* stream) {
  if (O == nullptr || Q == nullptr || K == nullptr || V == nullptr) return PTXB200_E_INVALID;
  if (B <= 0 || H <= 0 || H_kv <= 0 || S <= 0 || D <= 0) return PTXB200_E_INVALID;
  if (causal != 0 && causal != 1) return PTXB200_E_INVALID;
  if (flags & ~(PTXB200_FA_NO_LAZY_RESCALE | PTXB200_FA_SINGLE_BLOCKS | PTXB200_FA_NO_TAIL_SPLIT |
                PTXB200_FA_ALWAYS_TAIL_SPLIT)) return PTXB200_E_INVALID;
  if (!(sm_scale > 0.0f) || !(sm_scale < 1e30f)) return PTXB200_E_INVALID;
  if ((D != 64 && D != 128) || H % H_kv != 0) return PTXB200_E_SHAPE;
  if ((long long)B * H * S >= (1ll << 31)) return PTXB200_E_SHAPE;
  if (!aligned16(O) || !aligned16(Q) || !aligned16(K) || !aligned16(V)) return PTXB200_E_ALIGN;
  if ((dbg != nullptr && !aligned16(dbg)) || (lse != nullptr && !aligned16(lse))) return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_fa_fwd(*ctx, O, lse, Q, K, V, B, H, H_kv, S, D, sm_scale, causal, flags, dbg,
                       status_word(*ctx, (cudaStream_t)stream), (cudaStream_t)stream);
}

int fa_fwd_bf16(void* O, const void* Q, const void* K, const void* V, int B, int H, int S, int D,
                float sm_scale, int causal, unsigned flags, void* dbg, void* stream) {
  return fa_fwd_bf16_ex(O, nullptr, Q, K, V, B, H, H, S, D, sm_scale, causal, flags, dbg, stream);
}

int ptxb200_fa_plan(int B, int H, int S, int causal, unsigned flags, int sm_count, int* out, int cap) {
  if (B <= 0 || H <= 0 || S <= 0 || sm_count <= 0 || cap < 0 || (out == nullptr && cap > 0)) return PTXB200_E_INVALID;
  if (causal != 0 && causal != 1) return PTXB200_E_INVALID;
  if (flags & ~(PTXB200_FA_NO_LAZY_RESCALE | PTXB200_FA_SINGLE_BLOCKS | PTXB200_FA_NO_TAIL_SPLIT |
                PTXB200_FA_ALWAYS_TAIL_SPLIT)) return PTXB200_E_INVALID;
  if ((long long)B * H * S >= (1ll << 31)) return PTXB200_E_SHAPE;
  const int n = describe_fa_plan(B * H, S, causal, flags, sm_count, out, cap);
  return n < 0 ? PTXB200_E_CAPACITY : n;
}

int ptxb200_sync_status(void* stream) {
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t* slot = status_word(*ctx, s);
  uint32_t word = 0;
  PTXB200_CUDA_TRY(cudaMemcpyAsync(&word, slot, sizeof(word), cudaMemcpyDeviceToHost, s));
  PTXB200_CUDA_TRY(cudaStreamSynchronize(s));
  if (word != 0) {
    PTXB200_CUDA_TRY(cudaMemsetAsync(slot, 0, sizeof(word), s));
    PTXB200_CUDA_TRY(cudaStreamSynchronize(s));
  }
  return (int)word;
}

int ptxb200_device_status(void) {
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  PTXB200_CUDA_TRY(cudaDeviceSynchronize());
  uint32_t words[kWsStatusSlots];
  PTXB200_CUDA_TRY(cudaMemcpy(words, ctx->workspace, sizeof(words), cudaMemcpyDeviceToHost));
  uint32_t first = 0;
  for (int i = 0; i < kWsStatusSlots && first == 0; ++i) first = words[i];
  if (first != 0) PTXB200_CUDA_TRY(cudaMemset(ctx->workspace, 0, sizeof(words)));
  return (int)first;
}

int ptxb200_selftest(int which, void* out_s, void* out_o, const void* q, const void* k,
                     const void* v, const void* p, void* stream) {
  if (which < 0 || which > 4) return PTXB200_E_INVALID;
  if (out_s == nullptr) return PTXB200_E_INVALID;
  if (which != 0 && which != 3 && which != 4 && (out_o == nullptr || q == nullptr || k == nullptr || v == nullptr || p == nullptr))
    return PTXB200_E_INVALID;
  if (!aligned16(out_s) || !aligned16(out_o) || !aligned16(q) || !aligned16(k) || !aligned16(v) ||
      !aligned16(p))
    return PTXB200_E_ALIGN;
  DeviceCtx* ctx = nullptr;
  int rc = current_ctx(&ctx);
  if (rc != PTXB200_OK) return rc;
  return launch_selftest(*ctx, which, out_s, out_o, q, k, v, p, (cudaStream_t)stream);
}

int ptxb200_shutdown(void) { return release_all_ctx(); }

}  // extern "C"
