// sm_100a building blocks shared by every kernel in this library: mbarrier
// verbs with BOUNDED waits, TMA tile loads, tensor-memory (TMEM) allocation and
// access, tcgen05.mma issue/commit, and the descriptor bit packers.
//
// Reference counterparts (jool-space/PTX.jl), restated here as inline PTX in
// CUDA C++ rather than through a Julia DSL:
//   src/lib/mbarriers.jl:52-111          mbarrier verb API
//   src/lib/tcgen05_descriptor.jl:81-122 instruction descriptor (f16/bf16 -> f32)
//   src/lib/tcgen05_descriptor.jl:580-619 shared-memory matrix descriptor
//   src/lib/tcgen05_layout.jl:36,41      TMEM lane addressing
//   src/lib/wait_registers.jl:38-71      tying tcgen05.ld results to wait::ld
//   test/gpu/blackwell/flash_attention_defs.jl:224-267  bounded wait + first blame
//
// Every wait in this file is bounded. A wait that runs out records a
// first-blame code in a global status word, raises a CTA-wide abort flag so the
// remaining waits of that CTA return at once, and then reports success so the
// pipeline drains, TMEM is released and the kernel returns. Nothing traps.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ptxb200 {

// ---------------------------------------------------------------------------
// Descriptor packers (host + device constexpr).
// ---------------------------------------------------------------------------

// Swizzle codes of the 3-bit layout field at bits [63:61] of the shared-memory
// matrix descriptor (src/lib/tcgen05_descriptor.jl:49-55).
enum : uint32_t {
  kLayoutNone = 0, kLayoutB128Base32B = 1, kLayoutB128 = 2, kLayoutB64 = 4, kLayoutB32 = 6
};

// 32-bit instruction descriptor for kind::f16 with bf16 A/B and an fp32
// accumulator. a_mn / b_mn select the MN-major ("transposed") operand form.
__host__ __device__ constexpr uint32_t make_idesc_bf16_f32(uint32_t m, uint32_t n,
                                                           bool a_mn, bool b_mn) {
  return (1u << 4)                       // D format = f32
         | (1u << 7)                     // A format = bf16
         | (1u << 10)                    // B format = bf16
         | ((a_mn ? 1u : 0u) << 15)      // A major axis
         | ((b_mn ? 1u : 0u) << 16)      // B major axis
         | ((n >> 3) << 17)              // N / 8
         | ((m >> 4) << 24);             // M / 16
}

// 64-bit shared-memory matrix descriptor. All three byte quantities must be
// multiples of 16; the descriptor stores them divided by 16 in 14-bit fields.
__host__ __device__ constexpr uint64_t make_sdesc(uint32_t smem_addr, uint32_t leading_bytes,
                                                  uint32_t stride_bytes, uint32_t layout) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4)
         | ((uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16)
         | ((uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32)
         | (1ull << 46)                  // fixed 0b001 at bits [48:46]
         | ((uint64_t)layout << 61);
}

// Known answers held by the reference's host tests
// (test/host/tcgen05_descriptors.jl:136-141, test/host/tcgen05_layout.jl:78-92).
static_assert(make_sdesc(0, 16, 1024, kLayoutB128) == 0x4000404000010000ull,
              "K-major 128B-swizzle descriptor constant");
static_assert(make_idesc_bf16_f32(128, 256, false, false) ==
                  ((1u << 4) | (1u << 7) | (1u << 10) | (32u << 17) | (8u << 24)),
              "idesc formula");
static_assert(make_idesc_bf16_f32(128, 128, false, true) ==
                  ((1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (16u << 17) | (8u << 24)),
              "idesc formula, MN-major B");

// Descriptors travel as (lo, hi) 32-bit halves: every per-step variation (the
// start address) lives in `lo`, `hi` is a constant of the layout, so stepping
// through a tile costs one 32-bit add per operand.
__host__ __device__ constexpr uint32_t sdesc_lo(uint32_t smem_addr, uint32_t leading_bytes) {
  return (uint32_t)(make_sdesc(smem_addr, leading_bytes, 0, 0) & 0xFFFFFFFFull);
}
__host__ __device__ constexpr uint32_t sdesc_hi(uint32_t stride_bytes, uint32_t layout) {
  return (uint32_t)(make_sdesc(0, 0, stride_bytes, layout) >> 32);
}
static_assert((((uint64_t)sdesc_hi(1024, kLayoutB128) << 32) | sdesc_lo(0, 16)) ==
                  0x4000404000010000ull, "split descriptor equals the packed one");

// TMEM address = (lane << 16) + column (src/lib/tcgen05_layout.jl:36).
__host__ __device__ constexpr uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}
static_assert(tmem_addr(0, 5, 0) == (5u << 16), "lane bits sit at [31:16]");
static_assert(tmem_addr(0x00070000u, 31, 0) == 0x00070000u + 0x1F0000u, "lane 31");

// Status word layout written on a wait that ran out: 0x32000000 | site<<8 | aux
// (top bit clear: the host returns the word as a positive int).
constexpr uint32_t kStatusTimeoutTag = 0x32000000u;
static_assert((kStatusTimeoutTag >> 31) == 0, "status codes are positive ints");

#if defined(__CUDACC__)

// ---------------------------------------------------------------------------
// Small utilities
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Per-CTA control block in shared memory used by the bounded waits.
struct WaitCtx {
  uint32_t* status;          // global first-blame word (may be shared by many CTAs)
  volatile uint32_t* abort;  // shared-memory flag: nonzero once any wait of this CTA ran out
};

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  // Make the initialised barriers visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wall-clock bound on any single wait. Far above the longest legitimate wait
// (a whole work item is a few hundred microseconds), far below a watchdog.
constexpr uint64_t kWaitLimitNs = 1500ull * 1000ull * 1000ull;

// Bounded wait on phase `parity`. Returns true on completion, false if the wait
// ran out (or the CTA was already aborting); callers carry on either way.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                            uint32_t site) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort != 0) return false;
    if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      *ctx.abort = 1;
      if (ctx.status != nullptr)
        atomicCAS(ctx.status, 0u,
                  kStatusTimeoutTag | (site << 8) | ((blockIdx.x & 0x7Fu) << 1) | (parity & 1u));
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          uint32_t site) {
  if (mbar_try_wait(bar, parity)) return true;   // already complete: the common case on hot paths
  return mbar_wait_slow(bar, parity, ctx, site);
}

// ---------------------------------------------------------------------------
// Flags in global memory between CTAs of one launch (release / acquire at GPU scope).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.global.release.gpu.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.acquire.gpu.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *flag == want (written by another CTA of the same launch with
// st_release_gpu). Same expiry behaviour as mbar_wait: first blame, CTA abort flag,
// return false.
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, uint32_t want, const WaitCtx& ctx,
                                          uint32_t site) {
  if (ld_acquire_gpu(flag) == want) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_gpu(flag) == want) return true;
    if (*ctx.abort != 0) return false;
    if ((++spins & 15u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      *ctx.abort = 1;
      if (ctx.status != nullptr)
        atomicCAS(ctx.status, 0u, kStatusTimeoutTag | (site << 8) | ((blockIdx.x & 0x7Fu) << 1));
      return false;
    }
    __nanosleep(64);
  }
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor) 2-D tile load, completion counted in bytes on an
// mbarrier. c0 is the innermost (contiguous) coordinate, in elements; c0 times
// the element size must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// 3-D form: c0 innermost (elements, c0 * element size a multiple of 16 bytes), c1 the
// row, c2 the slice. Coordinates past an extent read the fill value (zero).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tmap) : "memory");
}

// ---------------------------------------------------------------------------
// TMEM allocation (one whole warp executes these)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 ordering
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// One thread: make `bar` complete (one arrival) when every tcgen05 operation
// this thread has issued so far has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                          uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]; A is read from tensor memory.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Bounded wait for a whole converged warp: every lane polls once and the warp
// branches on the vote (a uniform branch: no divergence bookkeeping on the hot
// path); only if the phase is not complete yet does lane 0 run the bounded loop.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                               uint32_t site) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_slow(bar, parity, ctx, site);
  return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

// Warp-level forms: EVERY lane of a converged warp calls these with identical
// operands; one elected lane issues the instruction. tcgen05.mma / commit are
// warp-scope, uniform-datapath instructions: issued from a converged warp with the
// election inside the instruction's predicate, the descriptors stay in uniform
// registers and an MMA costs a few issue cycles; issued by one diverged thread
// (an `if (lane == 0)` around the whole loop) each MMA costs ~50 cycles of that
// thread. In isolation that is 2150 vs 2650 cycles per pair of attention tiles; in
// the attention kernel itself, next to seven busy warps per scheduler, the converged
// form measured slower, so only the GEMM uses these.
__device__ __forceinline__ void tc_mma_ss_warp(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit_warp(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
      : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers, 32 lanes x 32-bit shape: the executing warp touches lanes
// 32*(warp_id % 4) .. +31, thread i <-> lane i, register k <-> column k.
// Results of a load are undefined until tcgen05.wait::ld; tc_wait_ld_bind ties
// the destination registers to that wait so they cannot be consumed earlier.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld_bind(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]),
                 "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld_bind16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// ---------------------------------------------------------------------------
// Numerics
// ---------------------------------------------------------------------------
// Two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in bits [15:0].
// The PTX operand order is (hi, lo) (src/wrappers/cvt.jl:27-38).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for two values on the FMA pipe (no MUFU): x = n + f with n = floor(x),
// 2^f by a degree-3 minimax polynomial on [0,1) (max relative error 7.5e-5, far
// below the bf16 rounding that follows), n added into the exponent field.
// floor comes from adding 1.5*2^23 in round-down mode, which leaves n in the low
// mantissa bits; (bits << 23) drops the constant's bits, so one shift-add per value
// finishes the job. Inputs below -126 are clamped (the polynomial dips just below 1
// at f = 0, so n = -127 would borrow from the sign bit; 2^-126 is zero for every
// purpose here).
// Same role as the reference's fab_exp_pair_emu
// (test/gpu/blackwell/flash_attention_defs.jl:355-387); coefficients derived here
// by a Remez exchange on the relative error.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float kMagic = 12582912.0f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -126.0f);
  x.y = fmaxf(x.y, -126.0f);
  const float2 r = __fadd2_rd(x, make_float2(kMagic, kMagic));
  const float2 fl = __fadd2_rn(r, make_float2(-kMagic, -kMagic));
  const float2 f = __ffma2_rn(fl, make_float2(-1.0f, -1.0f), x);
  float2 p = __ffma2_rn(f, make_float2(0.07802452f, 0.07802452f), make_float2(0.22606716f, 0.22606716f));
  p = __ffma2_rn(p, f, make_float2(0.69583356f, 0.69583356f));
  p = __ffma2_rn(p, f, make_float2(0.99992520f, 0.99992520f));
  float2 e;
  e.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(r.x) << 23));
  e.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(r.y) << 23));
  return e;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

#endif  // __CUDACC__
}  // namespace ptxb200
