// fa_fwd_bf16: O = softmax(Q K^T * scale [+ causal mask]) V on sm_100a.
//
// The reference kernel for this path is fab_kernel!
// (test/gpu/blackwell/flash_attention_defs.jl:621-961): head dim 128, non-causal
// only, 256 query rows per work item as two 128-row stages, S and O in tensor
// memory, P written back over S as bf16 and consumed from tensor memory by the
// second product, a "stale basis" softmax that starts from basis 0 and defers the
// row-max decision by one tile.
//
// This kernel keeps the tensor-memory residency (it is what the hardware wants)
// but is its own design in what it computes and how the roles talk:
//   * exact online softmax: every tile's exponentials use a basis that already
//     includes that tile's row maximum (no basis-0 first tile, so large logits
//     cannot overflow); O is rescaled only when the maximum grew by more than
//     2^8 (the slack cancels exactly in the final O / l);
//   * head dim 64 and 128, causal and non-causal, from one template;
//   * causal work items skip the key tiles above the diagonal per 128-row stage,
//     mask only the diagonal tile, and are handed out longest first within a head;
//   * the exponentials of a tile are split between two warps and two pipes: the
//     stage's softmax warp does key columns 0-95 on the MUFU, the correction warp
//     of the same rows does columns 96-127 with a polynomial on the FMA pipe (0-79 and
//     80-127 in the head-dim-64 kernel without masking code, where the MUFU binds);
//   * a protocol of mbarrier phases in which no producer can run two phases ahead
//     of its consumer: within an item each producer's next arrival is downstream of
//     an MMA issue that waited for the consumer's previous arrival, so no padding
//     commits and no split-by-parity barriers are needed; across items, where a
//     stage may run a short item ahead, the row sums are handed over through l_free;
//   * every wait is bounded and reports to a status word;
//   * where whole items dealt round robin would leave SMs idle through the last round
//     (fewer items than SMs, long sequences), that round is cut along the key axis into
//     equal shares for all SMs; the pieces of an item meet unnormalised in per-CTA scratch
//     slots and are merged by the log-sum-exp rule in the CTA that holds the item's first
//     keys (attn_sched.cuh, the kTail instantiations of the kernel, plan_schedule below).
//
// Roles (512 threads): warps 0-3 / 4-7 softmax of stage 0 / 1 (thread = one row),
// warps 8-11 correction (O rescale, their share of the exponentials, epilogue),
// warp 12 MMA issue, warp 13 TMA loads, warps 14-15 idle (they only take part in
// the register re-split).
//
// Barriers: q_full[2], q_free[2], kv_full[n], kv_free[n] (TMA ring); s_full[2] (MMA ->
// softmax and correction warps); basis[2] (softmax -> correction, every tile: the
// row's basis -m*c, from whose change the O rescale factor follows);
// p_full[stage][half]: half 0 completes with 128 softmax arrivals (P columns 0-31
// stored) plus 128 correction arrivals (O rescaled for this tile, or free after the
// previous item's epilogue), half 1 with 128 softmax arrivals (columns 32-47) plus
// 128 correction arrivals (columns 48-63); l_ready[2], o_done[2], l_free[2] (end of item).
//
// Tensor memory (512 columns x 128 lanes of 32 bit):
//   S0 at 0, S1 at 128 (fp32, 128 columns each; P_s overwrites the first 64
//   columns of S_s as packed bf16), O0 at 256, O1 at 256 + D.
//
// Algorithmic work per launch: 4*B*H*S*S*D flop non-causal, 2*B*H*S*S*D causal
// (softmax excluded; the reference's convention, bench/flash_attention.jl:107-108).
#include <math.h>

#include <mutex>
#include <utility>
#include <vector>

#include "attn_sched.cuh"
#include "attn_tiles.cuh"
#include "host_common.h"

namespace ptxb200 {
namespace {

constexpr int kThreads = 512;
#ifndef PTXB200_FA_REGS_SOFTMAX
#define PTXB200_FA_REGS_SOFTMAX 168
#define PTXB200_FA_REGS_CORRECTION 104
#define PTXB200_FA_REGS_OTHER 72
#endif
constexpr int kRegsSoftmax = PTXB200_FA_REGS_SOFTMAX;
constexpr int kRegsCorrection = PTXB200_FA_REGS_CORRECTION;
constexpr int kRegsOther = PTXB200_FA_REGS_OTHER;
static_assert(256 * kRegsSoftmax + 128 * kRegsCorrection + 128 * kRegsOther <= 65536,
              "register re-split must fit the register file");
// Head dim 64: the exponential unit is the binding pipe there (one ex2 per score, half the
// tensor work per score), so the correction warps take 48 instead of 32 of a tile's 128 key
// columns onto the FMA pipe and get the registers for it. (At head dim 128 the same
// split measured 2.4 % slower non-causal and spilled in the causal kernel.)
constexpr int kRegsSoftmax64 = 160, kRegsCorrection64 = 120;
static_assert(256 * kRegsSoftmax64 + 128 * kRegsCorrection64 + 128 * kRegsOther <= 65536,
              "register re-split must fit the register file");
// (only in the plain kernel: the causal and the ragged-length kernels measured a quarter to a
// third slower with it at head dim 64, and the kernels with a cut last round spill with it)
template <int D, bool kOther> constexpr int kHelperCols = (D == 64 && !kOther) ? 48 : 32;   // key columns per tile on the correction warps

// Which of the 16 element pairs of every 32-column chunk take the FMA-pipe
// polynomial exp2 instead of the MUFU ex2 (bit i = pair i). The MUFU pipe
// (16 ex2/clk/SM) needs as many cycles per tile as the tensor pipe at D = 128 and
// twice as many at D = 64; moving a fraction of the exponentials to the FMA pipe
// takes it off the critical path.
#ifndef PTXB200_FA_EMU_MASK
#define PTXB200_FA_EMU_MASK 0x0000u
#endif
constexpr uint32_t kEmuMask = PTXB200_FA_EMU_MASK;
// The last 32 key columns of every tile are exponentiated by the correction warps
// with the FMA-pipe polynomial, in parallel with the softmax warps' MUFU work on the
// first 96: the softmax phase of a stage is latency-bound in a single warp per
// scheduler, the correction warps' issue slots are otherwise idle, and the MUFU
// pipe is co-critical with the tensor pipe.
constexpr int kSoftmaxChunks = 3;   // 32-column chunks done by the softmax warps
#ifndef PTXB200_FA_BATCH
#define PTXB200_FA_BATCH 8
#endif
constexpr int kBatch = PTXB200_FA_BATCH;   // element pairs per exp batch

enum : uint32_t {
  kSiteLoadQFree = 5, kSiteLoadKvFree = 6, kSiteMmaQFull = 7, kSiteMmaKvFull = 8,
  kSiteMmaPFull = 9, kSiteSoftmaxSFull = 11, kSiteCorrAlpha = 12,
  kSiteCorrLReady = 13, kSiteCorrODone = 14, kSiteSoftmaxLFree = 22, kSiteCombinePart = 23
};

// Timestamp hooks for offline latency studies; compiled out of the product build.
#ifdef PTXB200_FA_TIMING
#define FA_TSTAMP(cond, rec, tile, ev)                                            \
  do {                                                                            \
    if ((cond) && (tile) < 16 && p.dbg != nullptr) {                              \
      long long t_;                                                               \
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_));                          \
      p.dbg[16 + (((rec) * 16 + (tile)) * 8 + (ev))] = (uint32_t)t_;              \
    }                                                                             \
  } while (0)
#else
#define FA_TSTAMP(cond, rec, tile, ev) do {} while (0)
#endif
// Per-CTA wall-clock marks (globaltimer, ns, low 32 bits) into dbg[64 + 4 * cta + k]: kernel
// entry, roles start, roles done. The caller's dbg buffer must then hold 64 + 4 * grid words.
// Offline studies only; compiled out of the product build.
#ifdef PTXB200_FA_CTA_TIMES
#define FA_CTA_TIME(k)                                                                     \
  do {                                                                                     \
    if (threadIdx.x == 256 && p.dbg != nullptr) p.dbg[64 + 4 * blockIdx.x + (k)] = (uint32_t)globaltimer_ns(); \
  } while (0)
#else
#define FA_CTA_TIME(k) do {} while (0)
#endif

template <int D>
struct FaCfg {
  using T = AttnTile<D>;
#ifndef PTXB200_FA_SLOTS128
#define PTXB200_FA_SLOTS128 5
#endif
  static constexpr int kSlots = (D == 128) ? PTXB200_FA_SLOTS128 : 8;   // K/V ring slots (one tile each)
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kOffQ + 2 * T::kTileBytes;
  static constexpr int kOffStats = kOffKV + kSlots * T::kTileBytes;  // alpha[2][128], l[2][128]
  static constexpr int kOffBars = kOffStats + 4 * 128 * 4;   // basis[2][128], l[2][128]
  // barrier indices (8 bytes each)
  static constexpr int kBarQFull = 0;                  // [2]  TMA tx
  static constexpr int kBarQFree = 2;                  // [2]  tcgen05.commit behind a stage's last Q K^T of an item
  static constexpr int kBarKvFull = 4;                 // [kSlots] TMA tx
  static constexpr int kBarKvFree = kBarKvFull + kSlots;   // [kSlots] tcgen05.commit
  static constexpr int kBarSFull = kBarKvFree + kSlots;    // [2] tcgen05.commit
  static constexpr int kBarPFull = kBarSFull + 2;      // [2 stages][2 halves] 128 softmax + 128 correction threads
  static constexpr int kBarAlpha = kBarPFull + 4;      // [2] basis published: 128 softmax threads
  static constexpr int kBarLReady = kBarAlpha + 2;     // [2] 128 softmax threads
  static constexpr int kBarODone = kBarLReady + 2;     // [2] tcgen05.commit
  static constexpr int kBarLFree = kBarODone + 2;      // [2] 128 correction threads: the item's row sums are read
  static constexpr int kNumBars = kBarLFree + 2;
  static constexpr int kOffTmemSlot = kOffBars + kNumBars * 8;
  static constexpr int kOffAbort = kOffTmemSlot + 8;
  static constexpr int kOffSegs = kOffAbort + 8;     // a cut last round: this CTA's segment count, then FaSeg[kTailMaxSegs]
  static constexpr int kSmemBytes = kOffSegs + 8 + kTailMaxSegs * (int)sizeof(FaSeg);   // the base must be 1024-byte aligned (checked)
  static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB a CTA can opt in to");
  static constexpr uint32_t kColS = 0;                 // + stage * 128
  static constexpr uint32_t kColO = 256;               // + stage * D
};

struct FaParams {
  __nv_bfloat16* o;
  int seqlen;        // S
  int num_mblocks;   // ceil(S / 256)
  int bh;            // B * H
  int total_work;    // num_mblocks * bh
  float scale_log2;  // sm_scale * log2(e)
  float rescale_threshold;  // in log2 units of the scaled scores
  uint32_t* status;
  uint32_t* dbg;
  uint32_t* cta_flags;  // only read by the kCtaFlags variant: one word per CTA
  float* lse;           // optional: log-sum-exp of the scaled scores per query row
  int heads_q;          // query heads per batch entry
  int heads_kv;         // key/value heads per batch entry (divides heads_q)
  int pair_mode;        // causal only: items are dealt out in pairs (see ItemIter)
  // Launches whose last round is cut along the key axis (the kTail kernels) only:
  FaSched sched;          // the round-robin part and the cut part of the distribution (attn_sched.cuh)
  float* parts;           // one slot of parked pieces per CTA
  uint32_t* part_flags;   // part_flags[c] == epoch once CTA c's slot is complete
  uint32_t epoch;         // differs from every earlier launch on the same scratch
};

// One piece of work as the roles see it: key tiles j0 .. j0 + nt[s] - 1 of stage s of item
// (mb, bh). jlast[s] is the index, relative to j0, of the stage's final tile of the ITEM
// (the only one that can hold masked keys); it lies outside [0, nt[s]) when this piece does
// not contain that tile. Without a cut last round every piece is a whole item: j0 = 0,
// jlast[s] = nt[s] - 1, kind = kWhole.
struct WorkItem {
  int mb, bh, j0;
  int nt[2];
  int jlast[2];
  int kind;      // kWhole, kWriter (piece parked in scratch), kCombiner (merges the parked pieces)
  int n_other;   // kCombiner: pieces parked by the next n_other CTAs
};
enum : int { kWhole = 0, kWriter = 1, kCombiner = 2 };

// The work items of one CTA, in order. An item is (m_block, batch*head): 256 query
// rows of one head.
//  * Non-causal: item w = blockIdx.x + i * gridDim.x with m_block varying fastest, so
//    CTAs that run together share one head's K/V in L2
//    (flash_attention_defs.jl:80-82); all items are equally long.
//  * Causal: item m_block visits 2*m_block + 2 key tiles. A CTA takes PAIRS of items of
//    one head -- block n-1-t and then block t -- so every pair is 2n + 2 tiles long
//    whatever t is: the CTAs stay in step without any sorting, the ceil(n/2) CTAs that
//    share a head work on it at the same time, and the heads in flight (about
//    2 * 148 / n of them) keep their K/V in L2 until all their pairs are done. (Handing
//    out single items longest-first within a head balances the load as well but lets
//    the items of a head drift apart in time: at S = 8192 the kernel then read K and V
//    4.9 times from HBM. Sorting all items by length was slower still.) A pair is a
//    coarse unit when a launch has few of them; the host compares the two static
//    schedules' longest CTA and falls back to single items where pairs lose more than
//    a tenth (causal_pair_mode below).
template <bool kCausal>
struct ItemIter {
  int v = 0;   // items this CTA has taken so far
  // `units` = how many items (or pairs) are dealt round robin: all of them, or the full
  // rounds only when the last round is cut
  __device__ __forceinline__ bool next(const FaParams& p, int& mb, int& bh, const int units) {
    if (!kCausal || !p.pair_mode) {
      const int w = blockIdx.x + v * gridDim.x;
      if (w >= units) return false;
      ++v;
      bh = w / p.num_mblocks;
      // causal without pairing (small launches, where a pair is too coarse a unit):
      // longest blocks of a head first
      mb = kCausal ? p.num_mblocks - 1 - (w % p.num_mblocks) : w % p.num_mblocks;
      return true;
    }
    const int pairs_per_head = (p.num_mblocks + 1) >> 1;
    while (true) {
      const int q = blockIdx.x + (v >> 1) * gridDim.x;
      if (q >= units) return false;
      bh = q / pairs_per_head;
      const int t = q - bh * pairs_per_head;
      const int far = p.num_mblocks - 1 - t;
      const bool second = (v & 1) != 0;
      ++v;
      if (!second) { mb = far; return true; }
      if (t != far) { mb = t; return true; }
      // the middle block of an odd count has no partner: on to the next pair
    }
  }
  // true while the item just returned by next() is this CTA's first
  __device__ __forceinline__ bool on_first() const { return v == 1; }
};
template <bool V> struct BoolTag { static constexpr bool value = V; };

// Key tiles each stage of the item visits.
template <bool kCausal>
__device__ __forceinline__ void tile_counts(const FaParams& p, int mb, int& nt0, int& nt1) {
  const int nt_all = (p.seqlen + kAttnRows - 1) / kAttnRows;   // the last tile may be partly past the end
  if (kCausal) {
    nt0 = min(2 * mb + 1, nt_all);
    nt1 = min(2 * mb + 2, nt_all);   // equals nt0 in a last block that has only its first stage
  } else {
    nt0 = nt1 = nt_all;
  }
}

// The pieces of work of one CTA, in order. kTail = false: the whole items ItemIter deals
// out. kTail = true: the items of the full rounds, then this CTA's segments of the cut last
// round from the table in shared memory (fa_fwd_kernel's prologue fills it: int count, pad,
// FaSeg[kTailMaxSegs]).
template <bool kCausal, bool kTail>
struct WorkIter {
  ItemIter<kCausal> rr;
  int tail_i = -1;   // kTail: -1 while the round-robin part lasts, then the next table entry
  __device__ __forceinline__ bool next(const FaParams& p, const uint8_t* seg_table, WorkItem& w) {
    if (!kTail || tail_i < 0) {
      const int units = kTail ? p.sched.full_units
                              : ((kCausal && p.pair_mode) ? p.bh * ((p.num_mblocks + 1) >> 1) : p.total_work);
      if (rr.next(p, w.mb, w.bh, units)) {
        tile_counts<kCausal>(p, w.mb, w.nt[0], w.nt[1]);
        w.j0 = 0;
        w.jlast[0] = w.nt[0] - 1;
        w.jlast[1] = w.nt[1] - 1;
        w.kind = kWhole;
        w.n_other = 0;
        return true;
      }
      if (!kTail) return false;
      tail_i = 0;
    }
    if (tail_i >= *reinterpret_cast<const int*>(seg_table)) return false;
    const FaSeg g = reinterpret_cast<const FaSeg*>(seg_table + 8)[tail_i];
    ++tail_i;
    w.mb = g.mb;
    w.bh = g.bh;
    w.j0 = g.j0;
    int full0, full1;   // the item's tiles per stage
    tile_counts<kCausal>(p, g.mb, full0, full1);
    w.nt[0] = min(g.j1, full0) - g.j0;
    w.nt[1] = g.j1 - g.j0;
    w.jlast[0] = full0 - 1 - g.j0;
    w.jlast[1] = full1 - 1 - g.j0;
    w.kind = g.j0 > 0 ? kWriter : (g.j1 < g.len ? kCombiner : kWhole);
    w.n_other = g.n_other;
    return true;
  }
  // true while the piece just returned by next() is this CTA's first
  __device__ __forceinline__ bool on_first() const { return rr.v == 1 || (rr.v == 0 && tail_i == 1); }
};

// Where a position of the tail line falls, for a whole warp: lane l holds the running
// step count behind units l, l + 32, ... of the tail (at most 8 per lane), so the unit that
// contains position x is the number of units that end at or before x, and its start is
// the largest of those ends.
struct WarpLocator {
  int incl[8];
  __device__ __forceinline__ void operator()(int x, int& u, int& st) const {
    int cnt = 0, below = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (incl[k] <= x) {
        ++cnt;
        below = max(below, incl[k]);
      }
    u = __reduce_add_sync(0xffffffffu, cnt);
    st = __reduce_max_sync(0xffffffffu, below);
  }
};

// One converged warp: this CTA's segments of the tail line into shared memory
// (int count, pad, FaSeg[kTailMaxSegs]). The host has checked, with the same code, that
// no CTA of the launch needs more than kTailMaxSegs.
// Non-causal launches: every unit is one item of nt_all steps, so a position's unit is a division.
struct UniformLocator {
  int len;
  __device__ __forceinline__ void operator()(int x, int& u, int& st) const {
    u = x / len;
    st = u * len;
  }
};

__device__ __noinline__ void tail_table(const FaSched sc, uint8_t* table) {
  const int lane = threadIdx.x & 31;
  if (!sc.causal) {
    UniformLocator loc{sc.nt_all};
    FaSeg* segs = reinterpret_cast<FaSeg*>(table + 8);
    const int n = fa_tail_segments(sc, (int)blockIdx.x, loc, segs);
    if (lane == 0) *reinterpret_cast<int*>(table) = n < kTailMaxSegs ? n : kTailMaxSegs;
    __syncwarp();
    return;
  }
  WarpLocator loc;
  int carry = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int u = k * 32 + lane;
    int len = 0;
    if (u < sc.tail_units) {
      int la, lb;
      fa_unit_lens(sc, sc.full_units + u, la, lb);
      len = la + lb;
    }
    int incl = len;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    loc.incl[k] = u < sc.tail_units ? carry + incl : 0x7fffffff;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  FaSeg* segs = reinterpret_cast<FaSeg*>(table + 8);
  const int n = fa_tail_segments(sc, (int)blockIdx.x, loc, segs);   // every lane writes the same values
  if (lane == 0) *reinterpret_cast<int*>(table) = n < kTailMaxSegs ? n : kTailMaxSegs;
  __syncwarp();
}

// The MMA-issue thread (one lane of warp 12).
//
// Its instruction stream is what paces the tensor pipe: with the ring slot changing
// every tile, forming the slot's descriptors costs this one thread about 320 clk per
// tile pair on top of 2050 clk of tensor time (measured in isolation). Two ways
// around that were built and measured no better in the full kernel: one switch per
// tile over the slot with every descriptor an immediate (faster in isolation, slower
// here, most of all for causal shapes), and issuing from the converged warp with an
// elected lane (the GEMM kernel's scheme).
template <int D, bool kCausal, bool kConv, bool kTail>
__device__ __forceinline__ void fa_mma_role(const FaParams& p, uint32_t base, uint32_t tmem,
                                            const WaitCtx& wctx, const uint8_t* seg_table) {
  using C = FaCfg<D>;
  using T = AttnTile<D>;
  constexpr int kSlots = C::kSlots;
  const uint32_t q_smem = base + C::kOffQ;
  const uint32_t kv_smem = base + C::kOffKV;
  const uint32_t bars = base + C::kOffBars;
  auto bar = [bars](int idx) -> uint32_t { return bars + 8u * (uint32_t)idx; };

  auto wait = [&](uint32_t b, uint32_t parity, uint32_t site) {
    if (kConv) mbar_wait_warp(b, parity, wctx, site); else mbar_wait(b, parity, wctx, site);
  };
  auto commit = [&](uint32_t b) { if (kConv) tc_commit_warp(b); else tc_commit(b); };
  [[maybe_unused]] const bool stamp_lane = !kConv || (threadIdx.x & 31) == 0;

  uint32_t slot = 0;      // ring slot of the next K/V tile
  uint32_t ring_ph = 0;   // phase of that slot's kv_full barrier
  uint32_t item_i = 0;
  uint32_t cnt_pv[2] = {0, 0};   // P*V products issued per stage (p_full phases)
  uint32_t kv_count = 0;

  // S_stage = Q_stage K^T with K in ring slot KS.
  auto qk = [&](int stage, uint32_t KS) {
    const uint32_t qa = q_smem + stage * T::kTileBytes;
    const uint32_t ka = kv_smem + KS * T::kTileBytes;
#pragma unroll
    for (int kk = 0; kk < T::kQKAtoms; ++kk)
      if (kConv)
        tc_mma_ss_warp(tmem + C::kColS + stage * 128, T::kmajor_lo(qa, kk), T::kKMajorHi,
                       T::kmajor_lo(ka, kk), T::kKMajorHi, T::kIdescQK, kk != 0 ? 1u : 0u);
      else
        tc_mma_ss(tmem + C::kColS + stage * 128, T::kmajor_lo(qa, kk), T::kKMajorHi,
                  T::kmajor_lo(ka, kk), T::kKMajorHi, T::kIdescQK, kk != 0 ? 1u : 0u);
    commit(bar(C::kBarSFull + stage));
  };
  // O_stage (+)= P_stage V with V in ring slot VS, issued per 64-column half of P as
  // the softmax publishes it: k16 steps 0-3 run while the second half is still being
  // exponentiated (the reference's split-P idea, flash_attention_defs.jl:36-50).
  auto pv = [&](int stage, uint32_t VS, bool accumulate, uint32_t parity) {
    const uint32_t va = kv_smem + VS * T::kTileBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      wait(bar(C::kBarPFull + 2 * stage + h), parity, kSiteMmaPFull);
      tc_fence_after();
#pragma unroll
      for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
        if (kConv)
          tc_mma_ts_warp(tmem + C::kColO + stage * D, T::p_tmem(tmem, C::kColS + stage * 128, kk),
                         T::v_lo(va, kk), T::kVHi, T::kIdescPV, (accumulate || kk != 0) ? 1u : 0u);
        else
          tc_mma_ts(tmem + C::kColO + stage * D, T::p_tmem(tmem, C::kColS + stage * 128, kk),
                    T::v_lo(va, kk), T::kVHi, T::kIdescPV, (accumulate || kk != 0) ? 1u : 0u);
    }
  };
  auto advance = [&](uint32_t n) {
    slot += n;
    kv_count += n;
    if (slot >= (uint32_t)kSlots) { slot -= kSlots; ring_ph ^= 1u; }
  };
  // First scores of an item for one stage: S_s = Q_s K_0^T with K_0 in slot KS (already
  // waited for). `qph` is the phase of the item's Q loads, `nt_s` the stage's tile count.
  auto first_qk = [&](int stage, uint32_t KS, uint32_t qph, int nt_s) {
    wait(bar(C::kBarQFull + stage), qph, kSiteMmaQFull);
    tc_fence_after();
    qk(stage, KS);
    if (nt_s == 1) commit(bar(C::kBarQFree + stage));   // also the stage's last Q K^T
  };

  // First tile of an item with the pipeline empty: K_0 sits in the current slot.
  auto start_item = [&](uint32_t qph, const int (&nts)[2]) {
    wait(bar(C::kBarKvFull + slot), ring_ph, kSiteMmaKvFull);
    first_qk(0, slot, qph, nts[0]);
    first_qk(1, slot, qph, nts[1]);
    commit(bar(C::kBarKvFree + slot));
    advance(1);
  };

  // At head dim 128 the items form one stream: a stage's first Q K^T of the NEXT item is
  // issued right behind its last P V of this one (for a causal item's shorter first
  // stage, a whole tile earlier), so the stages keep alternating across the boundary
  // instead of draining and refilling the pipeline once per item. A stage may therefore
  // be a whole short item ahead of the correction warps; the per-item hand-overs that
  // allow for it are the per-stage q_free and the l_free barrier. At head dim 64, where
  // the MUFU rather than the issue order bounds a tile, this measured slower on causal
  // problems, so there each item starts behind the previous one's last P V.
  constexpr bool kStream = (D == 128);
  WorkIter<kCausal, kTail> items;
  WorkItem w, w2;
  int nt[2] = {0, 0};
  bool have = items.next(p, seg_table, w);
  if (have) {
    nt[0] = w.nt[0];
    nt[1] = w.nt[1];
    start_item(0u, nt);
  }
  while (have) {
    int nt2[2] = {0, 0};
    const bool have2 = items.next(p, seg_table, w2);
    if (have2) {
      nt2[0] = w2.nt[0];
      nt2[1] = w2.nt[1];
    }
    const bool chain = kStream && have2;
    const uint32_t qph2 = (item_i + 1u) & 1u;
    const int nt_max = nt[1];
    for (int j = 0; j < nt_max; ++j) {
      // V_j sits in slot VS; behind it K_{j+1}, or a chained next item's K_0 after the last tile
      const uint32_t VS = slot;
      const uint32_t KS = (VS + 1 == (uint32_t)kSlots) ? 0u : VS + 1;
      const bool last = (j + 1 == nt_max);
      const bool need_k = !last || chain;
      FA_TSTAMP(stamp_lane && blockIdx.x == 0 && item_i == 0, 2, j, 6);
      wait(bar(C::kBarKvFull + VS), ring_ph, kSiteMmaKvFull);
      if (need_k) wait(bar(C::kBarKvFull + KS), KS == 0 ? (ring_ph ^ 1u) : ring_ph, kSiteMmaKvFull);
      FA_TSTAMP(stamp_lane && blockIdx.x == 0 && item_i == 0, 2, j, 7);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (!kCausal || j < nt[s]) {
          FA_TSTAMP(stamp_lane && blockIdx.x == 0 && item_i == 0, 2, j, 3 * s + 0);
          pv(s, VS, j > 0, cnt_pv[s] & 1u);
          ++cnt_pv[s];
          FA_TSTAMP(stamp_lane && blockIdx.x == 0 && item_i == 0, 2, j, 3 * s + 1);
          if (j + 1 < nt[s]) {
            qk(s, KS);
            if (j + 2 == nt[s]) commit(bar(C::kBarQFree + s));   // the stage's last Q K^T of this item
          } else {
            commit(bar(C::kBarODone + s));
          }
          FA_TSTAMP(stamp_lane && blockIdx.x == 0 && item_i == 0, 2, j, 3 * s + 2);
        }
        if (last && chain) first_qk(s, KS, qph2, nt2[s]);
      }
      commit(bar(C::kBarKvFree + VS));
      if (need_k) commit(bar(C::kBarKvFree + KS));
      advance(need_k ? 2u : 1u);
    }
    have = have2;
    nt[0] = nt2[0]; nt[1] = nt2[1];
    ++item_i;
    if (have && !kStream) start_item(item_i & 1u, nt);
  }
  if (p.dbg != nullptr && blockIdx.x == 0 && stamp_lane) {
    p.dbg[1] = kv_count;
    p.dbg[2] = cnt_pv[0];
    p.dbg[3] = cnt_pv[1];
  }
}

// kCtaFlags: additionally mark, in p.cta_flags[blockIdx.x], every CTA in which a
// bounded wait ran out (used by the entry point that keeps its scratch in a static
// device array).
// kRagged (non-causal only): the sequence length is not a multiple of 128, so the last key
// tile holds keys past the end that must be masked. A variant of its own because the
// masking code, though it runs once per item, costs the common case 1-2 % when compiled in.
// kTail: the launch's last round of items is cut along the key axis (attn_sched.cuh): the
// CTA runs its segments of that round after its whole items, parks or merges pieces in the
// epilogue. A variant of its own so that launches without a cut run exactly the code they
// ran before the cut existed.
template <int D, bool kCausal, bool kCtaFlags = false, bool kRagged = false, bool kTail = false>
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using C = FaCfg<D>;
  using T = AttnTile<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0) {
    // the 128-byte swizzle needs 1024-byte aligned tiles; every thread leaves before
    // any barrier or allocation exists
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0u, kStatusTimeoutTag | (17u << 8));
    return;
  }

  const uint32_t q_smem = base + C::kOffQ;
  const uint32_t kv_smem = base + C::kOffKV;
  float* stats_neg = reinterpret_cast<float*>(smem + C::kOffStats);            // [2][128]
  float* stats_l = stats_neg + 256;                                            // [2][128]
  const uint32_t bars = base + C::kOffBars;
  auto bar = [bars](int idx) -> uint32_t { return bars + 8u * (uint32_t)idx; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::kOffAbort);
  const WaitCtx wctx{p.status, abort_flag};
  const uint8_t* seg_table = smem + C::kOffSegs;   // kTail: int count, pad, FaSeg[kTailMaxSegs]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(C::kBarQFull + 0), 1);
    mbar_init(bar(C::kBarQFull + 1), 1);
    mbar_init(bar(C::kBarQFree + 0), 1);
    mbar_init(bar(C::kBarQFree + 1), 1);
    for (int s = 0; s < C::kSlots; ++s) {
      mbar_init(bar(C::kBarKvFull + s), 1);
      mbar_init(bar(C::kBarKvFree + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(C::kBarSFull + s), 1);
      mbar_init(bar(C::kBarPFull + 2 * s + 0), 256);   // softmax warps (P half 0) + correction warps (O ready)
      mbar_init(bar(C::kBarPFull + 2 * s + 1), 256);   // softmax warps + correction warps
      mbar_init(bar(C::kBarAlpha + s), 128);
      mbar_init(bar(C::kBarLReady + s), 128);
      mbar_init(bar(C::kBarODone + s), 1);
      mbar_init(bar(C::kBarLFree + s), 128);
    }
    mbar_fence_init();
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  FA_CTA_TIME(0);
  if (kTail && warp == 14) tail_table(p.sched, smem + C::kOffSegs);
  tc_fence_before();
  __syncthreads();
  FA_CTA_TIME(1);
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= 12) {
    // =====================================================================
    // warpgroup 3: TMA loads (warp 13) and MMA issue (warp 12)
    // =====================================================================
    setmaxnreg_dec<kRegsOther>();
    if (warp == 13) {
      if (elect_one()) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
        uint32_t kv_it = 0, item_i = 0;
        auto kv_load = [&](const void* tmap, int row, int slice) {
          const uint32_t s = kv_it % C::kSlots;
          const uint32_t ph = (kv_it / C::kSlots) & 1u;
          mbar_wait(bar(C::kBarKvFree + s), ph ^ 1u, wctx, kSiteLoadKvFree);
          mbar_arrive_expect_tx(bar(C::kBarKvFull + s), T::kTileBytes);
          T::load3(kv_smem + s * T::kTileBytes, tmap, row, slice, bar(C::kBarKvFull + s));
          ++kv_it;
        };
        WorkIter<kCausal, kTail> items;
        for (WorkItem w; items.next(p, seg_table, w); ++item_i) {
          const int mb = w.mb, bh = w.bh, nt1 = w.nt[1];
          const int kv_row0 = kTail ? w.j0 * kAttnRows : 0;   // first key tile of this piece of the item
          // grouped heads: query head h reads key/value head h / (heads_q / heads_kv)
          const int b_idx = bh / p.heads_q;
          const int kv_head = (bh - b_idx * p.heads_q) / (p.heads_q / p.heads_kv);
          const int kv_slice = b_idx * p.heads_kv + kv_head;
          const int q_row0 = mb * 2 * kAttnRows;   // within the head's sequence; rows past its end load as zeros
          // a stage's Q may be overwritten once its last S = Q K^T of the previous item has run
          mbar_wait(bar(C::kBarQFree + 0), (item_i & 1u) ^ 1u, wctx, kSiteLoadQFree);
          mbar_arrive_expect_tx(bar(C::kBarQFull + 0), T::kTileBytes);
          T::load3(q_smem, &tmap_q, q_row0, bh, bar(C::kBarQFull + 0));
          kv_load(&tmap_k, kv_row0, kv_slice);
          mbar_wait(bar(C::kBarQFree + 1), (item_i & 1u) ^ 1u, wctx, kSiteLoadQFree);
          mbar_arrive_expect_tx(bar(C::kBarQFull + 1), T::kTileBytes);
          T::load3(q_smem + T::kTileBytes, &tmap_q, q_row0 + kAttnRows, bh, bar(C::kBarQFull + 1));
          for (int j = 0; j < nt1; ++j) {
            FA_TSTAMP(blockIdx.x == 0 && items.on_first(), 3, j, 0);
            kv_load(&tmap_v, kv_row0 + j * kAttnRows, kv_slice);
            FA_TSTAMP(blockIdx.x == 0 && items.on_first(), 3, j, 1);
            if (j + 1 < nt1) kv_load(&tmap_k, kv_row0 + (j + 1) * kAttnRows, kv_slice);
          }
        }
        if (p.dbg != nullptr && blockIdx.x == 0) p.dbg[0] = kv_it;
      }
    } else if (warp == 12) {
#ifdef PTXB200_FA_MMA_CONVERGED
      fa_mma_role<D, kCausal, true, kTail>(p, base, tmem, wctx, seg_table);
#else
      if (elect_one()) fa_mma_role<D, kCausal, false, kTail>(p, base, tmem, wctx, seg_table);
#endif
    }
  } else if (warp < 8) {
    // =====================================================================
    // softmax: warpgroup `stage` owns the 128 rows of that stage; one row
    // per thread, the whole 128-column tile of scores in registers.
    // =====================================================================
    setmaxnreg_inc<(kHelperCols<D, kCausal || kRagged || kTail> == 48 ? kRegsSoftmax64 : kRegsSoftmax)>();
    const int stage = warp >> 2;
    const int row = tid & 127;
    const uint32_t t_row = tmem_addr(tmem, (warp & 3) * 32, C::kColS + stage * 128);
    const float scale_log2 = p.scale_log2;
    uint32_t cnt_s = 0, items_done = 0;
    WorkIter<kCausal, kTail> items;
    for (WorkItem w; items.next(p, seg_table, w);) {
      const int ntiles = stage ? w.nt[1] : w.nt[0];
      // the stage's final tile of the item: the piece's last tile, unless the item is cut there
      const int jlast = kTail ? (stage ? w.jlast[1] : w.jlast[0]) : ntiles - 1;
      [[maybe_unused]] const int kv_tail =   // keys in the sequence's last tile (non-causal)
          p.seqlen - ((kTail ? (p.seqlen + kAttnRows - 1) / kAttnRows : ntiles) - 1) * kAttnRows;
      [[maybe_unused]] const bool stamp = blockIdx.x == 0 && items.on_first() && row == 0;
      float m_run = -INFINITY;
      float l_run = 0.0f;
#pragma unroll 1
      for (int j = 0; j < ntiles; ++j) {
        FA_TSTAMP(stamp, stage, j, 0);
        mbar_wait(bar(C::kBarSFull + stage), cnt_s & 1u, wctx, kSiteSoftmaxSFull);
        ++cnt_s;
        tc_fence_after();
        FA_TSTAMP(stamp, stage, j, 1);
        uint32_t v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_row + c * 32, v[c]);
#pragma unroll
        for (int c = 0; c < 4; ++c) tc_wait_ld_bind(v[c]);
        FA_TSTAMP(stamp, stage, j, 2);

        if (kCausal && j == jlast) {
          // diagonal tile: key (local) column i is kept iff i <= row (keys past the end of
          // the sequence lie beyond every valid row's diagonal)
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > row) v[c][i] = 0xFF800000u;  // -inf
        }
        if (kRagged && !kCausal && j == jlast && kv_tail < kAttnRows) {
          // last tile of a sequence that is not a multiple of 128: its keys past the end
          // loaded as zeros and must not count
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= kv_tail) v[c][i] = 0xFF800000u;  // -inf
        }

        float mx[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float m = fmaxf(__uint_as_float(v[c][0]), __uint_as_float(v[c][1]));
#pragma unroll
          for (int i = 2; i < 32; i += 2)
            m = max3(m, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
          mx[c] = m;
        }
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));

        float alpha = 1.0f;
        if (j == 0) {
          m_run = m_tile;
        } else {
          const float m_new = fmaxf(m_run, m_tile);
          if ((m_new - m_run) * scale_log2 > p.rescale_threshold) {
            alpha = ex2_approx((m_run - m_new) * scale_log2);
            m_run = m_new;
          }
          l_run *= alpha;
        }
        const float neg = -m_run * scale_log2;
        // the basis goes to the correction warps: they exponentiate their share of the
        // columns against it and derive the O rescale factor from its change
        stats_neg[stage * 128 + row] = neg;
        mbar_arrive(bar(C::kBarAlpha + stage));

        FA_TSTAMP(stamp, stage, j, 3);
        const float2 scale2 = make_float2(scale_log2, scale_log2);
        const float2 neg2 = make_float2(neg, neg);
        float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int c = 0; c < kSoftmaxChunks; ++c) {
          uint32_t pk[16];
          // batches of kBatch pairs: all scaled inputs, then all exponentials back to
          // back (so the MUFU latency of one is hidden behind the issue of the next),
          // then the sums and the bf16 packing
          constexpr int kPairsLast = (128 - kHelperCols<D, kCausal || kRagged || kTail> - 64) / 2;   // pairs of the third chunk: 16, or 8 at D = 64
#pragma unroll
          for (int b = 0; b < 16; b += kBatch) {
            if (c == 2 && b >= kPairsLast) break;
            float2 x[kBatch], e[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
              x[i] = __ffma2_rn(make_float2(__uint_as_float(v[c][2 * (b + i)]),
                                            __uint_as_float(v[c][2 * (b + i) + 1])), scale2, neg2);
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
              if ((kEmuMask >> (b + i)) & 1u) {
                e[i] = exp2_poly2(x[i]);
              } else {
                e[i].x = ex2_approx(x[i].x);
                e[i].y = ex2_approx(x[i].y);
              }
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
              sum2[i & 1] = __fadd2_rn(sum2[i & 1], e[i]);
              pk[b + i] = pack_bf16x2(e[i].x, e[i].y);
            }
          }
          if (c == 2 && kPairsLast == 8) {
            uint32_t pk8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) pk8[i] = pk[i];
            tmem_st8(t_row + 32, pk8);
          } else {
            tmem_st16(t_row + c * 16, pk);
          }
          if (c == 1 || c == kSoftmaxChunks - 1) {
            // this warp's share of a 64-column half of P is in tensor memory: publish it
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(C::kBarPFull + 2 * stage + (c >> 1)));
            FA_TSTAMP(stamp, stage, j, 4 + (c >> 1));
          }
        }
        l_run += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      }
      // the correction warps must have read the previous item's row sum (a stage may
      // run a whole short item ahead of them)
      if (items_done > 0) mbar_wait(bar(C::kBarLFree + stage), (items_done - 1u) & 1u, wctx, kSiteSoftmaxLFree);
      ++items_done;
      stats_l[stage * 128 + row] = l_run;
      mbar_arrive(bar(C::kBarLReady + stage));
    }
    if (p.dbg != nullptr && blockIdx.x == 0 && row == 0) p.dbg[6 + stage] = cnt_s;
  } else {
    // =====================================================================
    // correction warps: rescale O when a row maximum moved, exponentiate key
    // columns 96-127 of every tile on the FMA pipe, and run the epilogue
    // =====================================================================
    // 104 registers is below the 128 the kernel launches with: a release, like the
    // MMA/load warpgroup's, that the two softmax warpgroups' increase draws on
    setmaxnreg_dec<(kHelperCols<D, kCausal || kRagged || kTail> == 48 ? kRegsCorrection64 : kRegsCorrection)>();
    const int row = tid & 127;
    const uint32_t t_lane = tmem_addr(tmem, (warp & 3) * 32, 0);
    mbar_arrive(bar(C::kBarPFull + 0));   // O is free for the first item
    mbar_arrive(bar(C::kBarPFull + 2));
    uint32_t cnt_a[2] = {0, 0};
    uint32_t cnt_h[2] = {0, 0};   // S tiles seen per stage
    uint32_t item_i = 0;
    WorkIter<kCausal, kTail> items;
    for (WorkItem w; items.next(p, seg_table, w); ++item_i) {
      const int mb = w.mb, bh = w.bh;
      const int nt[2] = {w.nt[0], w.nt[1]};
      const int nt_max = nt[1];
      float l_part[2] = {0.0f, 0.0f};   // row sums of the columns this thread exponentiates
      float neg_prev[2] = {0.0f, 0.0f};
#pragma unroll 1
      for (int j = 0; j < nt_max; ++j) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (j < nt[s]) {
            uint32_t sv[32];
            [[maybe_unused]] uint32_t sw[16];   // head dim 64: key columns 80..95 as well
            // Only a stage's last tile can hold masked keys: those above the diagonal
            // (causal) or past the end of the sequence (non-causal, S % 128 != 0). `keep`
            // is the last key column this row keeps there.
            const int j_abs = kTail ? w.j0 + j : j;   // the tile's index within the head's sequence
            const bool mask_tile = j == (kTail ? w.jlast[s] : nt[s] - 1) &&
                                   (kCausal || (kRagged && p.seqlen - j_abs * kAttnRows < kAttnRows));
            const int keep = kCausal ? row : p.seqlen - j_abs * kAttnRows - 1;
            {
              // fetch this row's last 32 scores while the softmax warp forms the maximum
              mbar_wait(bar(C::kBarSFull + s), cnt_h[s] & 1u, wctx, kSiteSoftmaxSFull);
              ++cnt_h[s];
              tc_fence_after();
              if (kHelperCols<D, kCausal || kRagged || kTail> == 48) tmem_ld16(t_lane + C::kColS + s * 128 + 80, sw);
              tmem_ld32(t_lane + C::kColS + s * 128 + 96, sv);
              if (kHelperCols<D, kCausal || kRagged || kTail> == 48) tc_wait_ld_bind16(sw);
              tc_wait_ld_bind(sv);
            }
            mbar_wait(bar(C::kBarAlpha + s), cnt_a[s] & 1u, wctx, kSiteCorrAlpha);
            ++cnt_a[s];
            const float neg = stats_neg[s * 128 + row];
            // alpha = 2^((m_old - m_new) * c) = 2^(neg_new - neg_old); exactly 1 when the basis stood
            const float alpha = (j == 0 || neg == neg_prev[s]) ? 1.0f : ex2_approx(neg - neg_prev[s]);
            neg_prev[s] = neg;
            if (j > 0) {
              if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                  uint32_t o[32];
                  const uint32_t a = t_lane + C::kColO + s * D + c * 32;
                  tmem_ld32(a, o);
                  tc_wait_ld_bind(o);
#pragma unroll
                  for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                  tmem_st32(a, o);
                }
                tc_wait_st();
              }
              tc_fence_before();
              mbar_arrive(bar(C::kBarPFull + 2 * s));
            }
            {
              const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
              const float2 neg2 = make_float2(neg, neg);
              float2 sum2 = make_float2(0.0f, 0.0f);
              uint32_t pk[16];
              [[maybe_unused]] uint32_t pk8[8];
              // two copies of the loop, so that the tiles without masked keys (all but one
              // per stage) carry no per-element compares
              auto exps = [&](auto masked) {
                if (kHelperCols<D, kCausal || kRagged || kTail> == 48) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    float2 e = exp2_poly2(__ffma2_rn(
                        make_float2(__uint_as_float(sw[2 * i]), __uint_as_float(sw[2 * i + 1])), scale2, neg2));
                    if (decltype(masked)::value) {
                      if (80 + 2 * i > keep) e.x = 0.0f;
                      if (80 + 2 * i + 1 > keep) e.y = 0.0f;
                    }
                    sum2 = __fadd2_rn(sum2, e);
                    pk8[i] = pack_bf16x2(e.x, e.y);
                  }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  float2 e = exp2_poly2(__ffma2_rn(
                      make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), scale2, neg2));
                  if (decltype(masked)::value) {
                    // masked keys weigh exactly zero (the polynomial bottoms out at 2^-126)
                    if (96 + 2 * i > keep) e.x = 0.0f;
                    if (96 + 2 * i + 1 > keep) e.y = 0.0f;
                  }
                  sum2 = __fadd2_rn(sum2, e);
                  pk[i] = pack_bf16x2(e.x, e.y);
                }
              };
              if (mask_tile) exps(BoolTag<true>{}); else exps(BoolTag<false>{});
              if (kHelperCols<D, kCausal || kRagged || kTail> == 48) tmem_st8(t_lane + C::kColS + s * 128 + 40, pk8);   // P columns of keys 80..95
              tmem_st16(t_lane + C::kColS + s * 128 + 48, pk);   // P columns of keys 96..127
              tc_wait_st();
              tc_fence_before();
              mbar_arrive(bar(C::kBarPFull + 2 * s + 1));
              l_part[s] = l_part[s] * alpha + (sum2.x + sum2.y);
            }
          }
        }
      }
      if constexpr (!kTail) {
        // ---- epilogue: O / l -> bf16 -> global ----
        const int q_row0 = bh * p.seqlen + mb * 2 * kAttnRows;
  #pragma unroll
        for (int s = 0; s < 2; ++s) {
          // rows past the end of the sequence were computed on zero-filled queries: not written
          const bool row_valid = mb * 2 * kAttnRows + s * kAttnRows + row < p.seqlen;
          mbar_wait(bar(C::kBarODone + s), item_i & 1u, wctx, kSiteCorrODone);
          mbar_wait(bar(C::kBarLReady + s), item_i & 1u, wctx, kSiteCorrLReady);
          tc_fence_after();
          const float l_total = stats_l[s * 128 + row] + l_part[s];
          mbar_arrive(bar(C::kBarLFree + s));   // the softmax warps may publish the next item's sum
          const float inv_l = 1.0f / l_total;
          if (p.lse != nullptr && row_valid) {
            // sum_j 2^(s_j c) = 2^(m c) * l with basis -m c in neg_prev: natural log of it
            p.lse[q_row0 + s * kAttnRows + row] = (log2f(l_total) - neg_prev[s]) * 0.6931471805599453f;
          }
          __nv_bfloat16* dst = p.o + (size_t)(q_row0 + s * kAttnRows + row) * D;
  #pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_lane + C::kColO + s * D + c * 32, o);
            tc_wait_ld_bind(o);
            if (c == D / 32 - 1) {
              // last read of O_s: the next item may overwrite it
              tc_fence_before();
              mbar_arrive(bar(C::kBarPFull + 2 * s));
            }
  #pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t p0 = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
              const uint32_t p1 = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
              const uint32_t p2 = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
              const uint32_t p3 = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
              if (row_valid) st_global_v4(dst + c * 32 + 8 * i, p0, p1, p2, p3);
            }
          }
        }
      } else {
        // A piece of an item cut along the key axis is either parked in this CTA's scratch
        // slot, unnormalised -- fp32 O, row sum l and basis b with O = sum_j 2^(s_j c - b) v_j
        // -- or, in the CTA that holds the item's first keys, merged with the pieces the
        // following CTAs parked:
        //   B = max_p b_p,  O = sum_p 2^(b_p - B) O_p,  l = sum_p 2^(b_p - B) l_p,  out = O / l.
        const int q_row0 = bh * p.seqlen + mb * 2 * kAttnRows;
        constexpr int kStageFloats = 256 + kAttnRows * D;   // l[128], b[128], O as [D/4][128 rows][4]
        float* const my_slot = p.parts + (size_t)blockIdx.x * (2 * kStageFloats);
        if (w.kind == kCombiner) {
          // the other pieces are complete once their CTAs' flags carry this launch's epoch
          for (int k = 1; k <= w.n_other; ++k)
            flag_wait(p.part_flags + blockIdx.x + k, p.epoch, wctx, kSiteCombinePart);
        }
  #pragma unroll
        for (int s = 0; s < 2; ++s) {
          // rows past the end of the sequence were computed on zero-filled queries: not written
          const bool row_valid = mb * 2 * kAttnRows + s * kAttnRows + row < p.seqlen;
          mbar_wait(bar(C::kBarODone + s), item_i & 1u, wctx, kSiteCorrODone);
          mbar_wait(bar(C::kBarLReady + s), item_i & 1u, wctx, kSiteCorrLReady);
          tc_fence_after();
          float l_total = stats_l[s * 128 + row] + l_part[s];
          mbar_arrive(bar(C::kBarLFree + s));   // the softmax warps may publish the next item's sum
          if (w.kind == kWriter) {
            float* const dst = my_slot + s * kStageFloats;
            dst[row] = l_total;
            dst[128 + row] = -neg_prev[s];
  #pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(t_lane + C::kColO + s * D + c * 32, o);
              tc_wait_ld_bind(o);
              if (c == D / 32 - 1) {
                // last read of O_s: the next item may overwrite it
                tc_fence_before();
                mbar_arrive(bar(C::kBarPFull + 2 * s));
              }
  #pragma unroll
              for (int i = 0; i < 8; ++i)
                st_global_v4(dst + 256 + ((c * 8 + i) * kAttnRows + row) * 4, o[4 * i], o[4 * i + 1], o[4 * i + 2],
                             o[4 * i + 3]);
            }
            continue;
          }
          float basis = -neg_prev[s];   // log2 basis of this CTA's O and l
          float w_own = 1.0f;
          if (w.kind == kCombiner) {
            const float b_own = basis;
            for (int k = 1; k <= w.n_other; ++k)
              basis = fmaxf(basis, __ldcg(my_slot + (size_t)k * (2 * kStageFloats) + s * kStageFloats + 128 + row));
            w_own = ex2_approx(b_own - basis);
            l_total *= w_own;
            for (int k = 1; k <= w.n_other; ++k) {
              const float* src = my_slot + (size_t)k * (2 * kStageFloats) + s * kStageFloats;
              l_total += __ldcg(src + row) * ex2_approx(__ldcg(src + 128 + row) - basis);
            }
          }
          const float inv_l = 1.0f / l_total;
          if (p.lse != nullptr && row_valid) {
            // sum_j 2^(s_j c) = 2^b * l with b the basis: natural log of it
            p.lse[q_row0 + s * kAttnRows + row] = (log2f(l_total) + basis) * 0.6931471805599453f;
          }
          __nv_bfloat16* dst = p.o + (size_t)(q_row0 + s * kAttnRows + row) * D;
  #pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_lane + C::kColO + s * D + c * 32, o);
            tc_wait_ld_bind(o);
            if (c == D / 32 - 1) {
              // last read of O_s: the next item may overwrite it
              tc_fence_before();
              mbar_arrive(bar(C::kBarPFull + 2 * s));
            }
            if (w.kind == kCombiner) {
  #pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * w_own);
  #pragma unroll 1
              for (int k = 1; k <= w.n_other; ++k) {
                const float* src = my_slot + (size_t)k * (2 * kStageFloats) + s * kStageFloats;
                const float wk = ex2_approx(__ldcg(src + 128 + row) - basis);
  #pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float4 part = __ldcg(reinterpret_cast<const float4*>(src + 256 + ((c * 8 + i) * kAttnRows + row) * 4));
                  o[4 * i + 0] = __float_as_uint(fmaf(part.x, wk, __uint_as_float(o[4 * i + 0])));
                  o[4 * i + 1] = __float_as_uint(fmaf(part.y, wk, __uint_as_float(o[4 * i + 1])));
                  o[4 * i + 2] = __float_as_uint(fmaf(part.z, wk, __uint_as_float(o[4 * i + 2])));
                  o[4 * i + 3] = __float_as_uint(fmaf(part.w, wk, __uint_as_float(o[4 * i + 3])));
                }
              }
            }
  #pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t p0 = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
              const uint32_t p1 = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
              const uint32_t p2 = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
              const uint32_t p3 = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
              if (row_valid) st_global_v4(dst + c * 32 + 8 * i, p0, p1, p2, p3);
            }
          }
        }
        if (w.kind == kWriter) {
          // both stages of the piece are in the slot: make them visible, then raise the flag
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (row == 0) st_release_gpu(p.part_flags + blockIdx.x, p.epoch);
        }
      }
    }
    if (p.dbg != nullptr && blockIdx.x == 0 && row == 0) {
      p.dbg[8] = cnt_a[0];
      p.dbg[9] = cnt_a[1];
      p.dbg[10] = item_i;
    }
  }

  tc_fence_before();
  __syncthreads();
  FA_CTA_TIME(3);
  if (warp == 12) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (kCtaFlags) {
    if (tid == 0 && *abort_flag != 0) p.cta_flags[blockIdx.x] = 1u;
  }
}

// Longest per-CTA tile count of the two static causal schedules; pairs unless they
// are more than a tenth longer.
int causal_pair_mode(int bh, int nmb, int nt_all, int sm_count) {
  const long long items = (long long)bh * nmb;
  const int pairs_per_head = (nmb + 1) / 2;
  const long long pairs = (long long)bh * pairs_per_head;
  if (items > (1 << 20)) return 1;   // enough work for either; skip the simulation
  // key tiles of block mb over both stages (tile_counts)
  auto len = [&](int mb) {
    const int nt0 = 2 * mb + 1 < nt_all ? 2 * mb + 1 : nt_all, nt1 = 2 * mb + 2 < nt_all ? 2 * mb + 2 : nt_all;
    return (long long)(nt0 + nt1);
  };
  const int grid_i = items < sm_count ? (int)items : sm_count;
  const int grid_p = pairs < sm_count ? (int)pairs : sm_count;
  long long worst_i = 0, worst_p = 0;
  for (int c = 0; c < grid_i; ++c) {
    long long sum = 0;
    for (long long w = c; w < items; w += grid_i) sum += len(nmb - 1 - (int)(w % nmb));
    worst_i = sum > worst_i ? sum : worst_i;
  }
  for (int c = 0; c < grid_p; ++c) {
    long long sum = 0;
    for (long long q = c; q < pairs; q += grid_p) {
      const int t = (int)(q % pairs_per_head), far = nmb - 1 - t;
      sum += len(far) + (t != far ? len(t) : 0);
    }
    worst_p = sum > worst_p ? sum : worst_p;
  }
  return worst_p * 10 <= worst_i * 11 ? 1 : 0;
}

// ---------------------------------------------------------------------------
// Choosing the distribution of a launch (host)
// ---------------------------------------------------------------------------
struct HostLocator {   // the tail line's unit starts as a plain array
  const int* starts;   // starts[u] = first step of tail unit u; starts[n] = one past the end
  int n;
  __host__ __device__ void operator()(int x, int& u, int& st) const {
    int lo = 0, hi = n;   // starts[lo] <= x < starts[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) / 2;
      if (starts[mid] <= x) lo = mid; else hi = mid;
    }
    u = lo;
    st = starts[lo];
  }
};

// Steps the busiest CTA runs when units [0, units) are dealt round robin to `grid` CTAs.
long long worst_round_robin(const FaSched& sc, int units, int grid) {
  long long worst = 0;
  for (int c = 0; c < grid; ++c) {
    long long sum = 0;
    for (int q = c; q < units; q += grid) {
      int la, lb;
      fa_unit_lens(sc, q, la, lb);
      sum += la + lb;
    }
    worst = sum > worst ? sum : worst;
  }
  return worst;
}

constexpr int kSplitOverheadSteps = 3;   // what a second segment, parking and merging cost a CTA, in steps (measured: 2.5-3)
constexpr int kSplitMaxRounds = 64;      // beyond this many full rounds the tail is noise: not split

// Round robin over whole units (the reference's distribution), or the same with the last,
// partly filled round cut along the key axis when that shortens the busiest CTA's work by
// more than the overhead of the cut.
FaSched plan_schedule(int bh, int nmb, int nt_all, int causal, unsigned flags, int sm_count, bool may_split) {
  FaSched legacy;
  legacy.num_mblocks = nmb;
  legacy.bh = bh;
  legacy.nt_all = nt_all;
  legacy.causal = causal;
  legacy.pair_mode = (causal && !(flags & PTXB200_FA_SINGLE_BLOCKS)) ? causal_pair_mode(bh, nmb, nt_all, sm_count) : 0;
  const long long legacy_units = (long long)bh * (legacy.pair_mode ? (nmb + 1) / 2 : nmb);
  legacy.grid = legacy_units < sm_count ? (int)legacy_units : sm_count;
  legacy.full_units = (int)legacy_units;
  legacy.tail_units = legacy.tail_steps = legacy.tail_ctas = 0;
  if (!may_split || (flags & PTXB200_FA_NO_TAIL_SPLIT) || sm_count > 256) return legacy;

  struct Key {
    int bh, nmb, nt_all, causal, sm;
    unsigned flags;
    bool operator==(const Key& o) const {
      return bh == o.bh && nmb == o.nmb && nt_all == o.nt_all && causal == o.causal && sm == o.sm && flags == o.flags;
    }
  };
  static std::mutex mu;
  static std::vector<std::pair<Key, FaSched>> cache;   // the last few shapes: the decision walks every tail CTA
  const Key key{bh, nmb, nt_all, causal, sm_count, flags};
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& kv : cache)
      if (kv.first == key) return kv.second;
  }
  auto remember = [&](const FaSched& sc) {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 16) cache.erase(cache.begin());
    cache.emplace_back(key, sc);
    return sc;
  };

  FaSched sc = legacy;
  sc.pair_mode = (causal && !(flags & PTXB200_FA_SINGLE_BLOCKS)) ? 1 : 0;   // pairs keep a head's CTAs together; the cut balances them
  const long long units = (long long)bh * (sc.pair_mode ? (nmb + 1) / 2 : nmb);
  if (units > (long long)kSplitMaxRounds * sm_count) return remember(legacy);
  sc.grid = sm_count;
  sc.full_units = (int)(units / sm_count) * sm_count;
  sc.tail_units = (int)units - sc.full_units;
  if (sc.tail_units == 0) return remember(legacy);
  std::vector<int> starts(sc.tail_units + 1, 0);
  int longest_item = 0;
  for (int u = 0; u < sc.tail_units; ++u) {
    int la, lb;
    fa_unit_lens(sc, sc.full_units + u, la, lb);
    starts[u + 1] = starts[u] + la + lb;
    longest_item = la > longest_item ? la : longest_item;
    longest_item = lb > longest_item ? lb : longest_item;
  }
  sc.tail_steps = starts.back();
  if ((long long)sc.tail_steps * (sm_count + 1) >= (1ll << 31)) return remember(legacy);   // cut positions are 32-bit products
  int span_min = (longest_item + kTailMaxParts - 3) / (kTailMaxParts - 2);   // at most kTailMaxParts pieces per item
  if (span_min < 2 * fa_min_seg(causal)) span_min = 2 * fa_min_seg(causal);
  sc.tail_ctas = sc.tail_steps / span_min < sm_count ? sc.tail_steps / span_min : sm_count;
  if (sc.tail_ctas < 2) return remember(legacy);
  // the kernel's per-CTA table and the combiner's reads are bounded: walk every tail CTA,
  // and take the busiest one's steps from the walk (cuts snap to item edges, so spans differ)
  HostLocator loc{starts.data(), (int)starts.size() - 1};
  int tail_worst = 0;
  for (int c = 0; c < sc.tail_ctas; ++c) {
    FaSeg segs[kTailMaxSegs];
    const int n = fa_tail_segments(sc, c, loc, segs);
    if (n > kTailMaxSegs) return remember(legacy);
    int steps = 0;
    for (int i = 0; i < n; ++i) {
      if (segs[i].n_other + 1 > kTailMaxParts) return remember(legacy);
      steps += segs[i].j1 - segs[i].j0;
    }
    tail_worst = steps > tail_worst ? steps : tail_worst;
  }
  const long long split_worst = worst_round_robin(sc, sc.full_units, sc.grid) + tail_worst + kSplitOverheadSteps;
  const long long legacy_worst = worst_round_robin(legacy, legacy.full_units, legacy.grid);
  if (!(flags & PTXB200_FA_ALWAYS_TAIL_SPLIT) && split_worst * 100 > legacy_worst * 92)
    return remember(legacy);   // cut only for a gain of a twelfth or more
  return remember(sc);
}

constexpr size_t kPartsHeaderBytes = 4096;   // one flag word per CTA, ahead of the slots

template <int D>
constexpr size_t parts_slot_bytes() { return (size_t)2 * (256 + kAttnRows * D) * sizeof(float); }

template <int D, bool kCausal>
int launch_variant(const DeviceCtx& ctx, const CUtensorMap& tq, const CUtensorMap& tk,
                   const CUtensorMap& tv, const FaParams& p, cudaStream_t stream) {
  using C = FaCfg<D>;
  static PerDeviceOnce attr_once;   // one per <D, kCausal> instantiation
  const int rc = attr_once.run(ctx.device, []() -> int {
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(fa_fwd_kernel<D, kCausal>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          C::kSmemBytes));
    PTXB200_CUDA_TRY(cudaFuncSetAttribute(fa_fwd_kernel<D, kCausal, false, false, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          C::kSmemBytes));
    if (!kCausal) {
      PTXB200_CUDA_TRY(cudaFuncSetAttribute(fa_fwd_kernel<D, false, false, true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            C::kSmemBytes));
      PTXB200_CUDA_TRY(cudaFuncSetAttribute(fa_fwd_kernel<D, false, false, true, true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            C::kSmemBytes));
    }
    return PTXB200_OK;
  });
  if (rc != PTXB200_OK) return rc;
  const bool ragged = !kCausal && p.seqlen % kAttnRows != 0;
  if (p.sched.tail_units > 0) {
    // the last round is cut: every SM gets a CTA
    const int grid = p.sched.grid;
    if (ragged)
      fa_fwd_kernel<D, false, false, true, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
    else
      fa_fwd_kernel<D, kCausal, false, false, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  } else {
    const int units = (kCausal && p.pair_mode) ? p.bh * ((p.num_mblocks + 1) / 2) : p.total_work;   // what ItemIter deals out
    const int grid = units < ctx.sm_count ? units : ctx.sm_count;
    if (ragged)
      fa_fwd_kernel<D, false, false, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
    else
      fa_fwd_kernel<D, kCausal><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  }
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

// The parameters every entry point fills the same way. `sc` is the distribution
// plan_schedule chose: without a cut last round only its pair_mode is used.
void fill_params(FaParams& p, void* O, void* lse, int B, int H, int H_kv, int S, float sm_scale, unsigned flags,
                 void* dbg, uint32_t* status, const FaSched& sc) {
  p.o = reinterpret_cast<__nv_bfloat16*>(O);
  p.seqlen = S;
  p.num_mblocks = (S + 255) / 256;
  p.bh = B * H;
  p.total_work = p.num_mblocks * p.bh;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.rescale_threshold = (flags & PTXB200_FA_NO_LAZY_RESCALE) ? 0.0f : 8.0f;
  p.status = status;
  p.dbg = reinterpret_cast<uint32_t*>(dbg);
  p.cta_flags = nullptr;
  p.lse = reinterpret_cast<float*>(lse);
  p.heads_q = H;
  p.heads_kv = H_kv;
  p.pair_mode = sc.pair_mode;
  p.sched = sc;
  p.parts = nullptr;
  p.part_flags = nullptr;
  p.epoch = 0;
}

}  // namespace

int launch_fa_fwd(const DeviceCtx& ctx, void* O, void* lse, const void* Q, const void* K,
                  const void* V, int B, int H, int H_kv, int S, int D, float sm_scale, int causal,
                  unsigned flags, void* dbg, uint32_t* status, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_tmap_bf16_3d(&tq, Q, (uint64_t)B * H, S, D, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_3d(&tk, K, (uint64_t)B * H_kv, S, D, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_3d(&tv, V, (uint64_t)B * H_kv, S, D, 128, 64)) != PTXB200_OK) return rc;
  FaParams p;
  fill_params(p, O, lse, B, H, H_kv, S, sm_scale, flags, dbg, status,
              plan_schedule(B * H, (S + 255) / 256, (S + kAttnRows - 1) / kAttnRows, causal, flags, ctx.sm_count, true));
  ScratchLease lease;
  if (p.sched.tail_units > 0) {
    // one slot of parked pieces and one flag per CTA, kept per (device, stream)
    const size_t slot = D == 128 ? parts_slot_bytes<128>() : parts_slot_bytes<64>();
    if ((rc = scratch_acquire(ctx, stream, kScratchAttnParts, kPartsHeaderBytes + (size_t)ctx.sm_count * slot,
                              &lease)) != PTXB200_OK)
      return rc;
    if (lease.fresh) PTXB200_CUDA_TRY(cudaMemsetAsync(lease.ptr, 0, kPartsHeaderBytes, stream));
    p.part_flags = reinterpret_cast<uint32_t*>(lease.ptr);
    p.parts = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(lease.ptr) + kPartsHeaderBytes);
    p.epoch = lease.epoch;
  }
  if (D == 128) {
    rc = causal ? launch_variant<128, true>(ctx, tq, tk, tv, p, stream)
                : launch_variant<128, false>(ctx, tq, tk, tv, p, stream);
  } else {
    rc = causal ? launch_variant<64, true>(ctx, tq, tk, tv, p, stream)
                : launch_variant<64, false>(ctx, tq, tk, tv, p, stream);
  }
  if (rc != PTXB200_OK) return rc;
  if (p.sched.tail_units > 0) return scratch_mark_used(lease, stream);
  return PTXB200_OK;
}

// The distribution plan_schedule picks and every tail CTA's segments, for tests on a
// machine without a GPU. out: 10 ints of FaSched (num_mblocks, bh, nt_all, causal, pair_mode,
// grid, full_units, tail_units, tail_steps, tail_ctas), then per tail CTA its segment count
// followed by 6 ints per segment (mb, bh, j0, j1, len, n_other). Returns the ints written,
// or -1 if `cap` is too small.
int describe_fa_plan(int BH, int S, int causal, unsigned flags, int sm_count, int* out, int cap) {
  const int nmb = (S + 255) / 256, nt_all = (S + kAttnRows - 1) / kAttnRows;
  const FaSched sc = plan_schedule(BH, nmb, nt_all, causal, flags, sm_count, true);
  int n = 0;
  auto put = [&](int v) {
    if (n < cap) out[n] = v;
    ++n;
  };
  put(sc.num_mblocks); put(sc.bh); put(sc.nt_all); put(sc.causal); put(sc.pair_mode);
  put(sc.grid); put(sc.full_units); put(sc.tail_units); put(sc.tail_steps); put(sc.tail_ctas);
  if (sc.tail_units > 0) {
    std::vector<int> starts(sc.tail_units + 1, 0);
    for (int u = 0; u < sc.tail_units; ++u) {
      int la, lb;
      fa_unit_lens(sc, sc.full_units + u, la, lb);
      starts[u + 1] = starts[u] + la + lb;
    }
    HostLocator loc{starts.data(), (int)starts.size() - 1};
    for (int c = 0; c < sc.tail_ctas; ++c) {
      FaSeg segs[kTailMaxSegs];
      const int k = fa_tail_segments(sc, c, loc, segs);
      put(k);
      for (int i = 0; i < k && i < kTailMaxSegs; ++i) {
        put(segs[i].mb); put(segs[i].bh); put(segs[i].j0); put(segs[i].j1); put(segs[i].len); put(segs[i].n_other);
      }
    }
  }
  return n <= cap ? n : -1;
}

}  // namespace ptxb200

// ===========================================================================
// fa_fwd_bf16_noalloc: the same kernel with its scratch in a static device array
// ===========================================================================
//
// fa_fwd_bf16 keeps its scratch -- the status word its bounded waits report to --
// in a per-device workspace that the library cudaMalloc's on first use. Some
// callers must not trigger an allocation: a serving loop whose device memory was
// carved up front (a later cudaMalloc is an error there, or fails on a full
// device), a latency-critical section that cannot take cudaMalloc's implicit
// synchronisation, a host runtime (such as a Julia session with its own memory
// pool) that wants to own every byte on the device. For them this entry point keeps the scratch in
// the array below. The array is part of the loaded module: every GPU that loads
// this library holds its kNoAllocScratchBytes until the process exits.
//
// Layout (uint32 words): [0] status word (first-blame code of a wait that ran
// out, as in fa_fwd_bf16), [1..15] reserved, [16 .. 16 + kNoAllocMaxCtas) one flag
// per CTA, set when a wait of that CTA ran out.
//
// The host-side name of a __device__ array is not a device address; the address
// the kernel gets comes from cudaGetSymbolAddress, asked once per device with
// that device current.
namespace ptxb200 {
namespace {

constexpr int kNoAllocMaxCtas = 240;                                 // one CTA per SM
constexpr int kNoAllocFlagBase = 16;
constexpr int kNoAllocScratchWords = kNoAllocFlagBase + kNoAllocMaxCtas;   // 256 words
constexpr int kNoAllocScratchBytes = kNoAllocScratchWords * 4;             // 1 KiB
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocScratchWords];

struct NoAllocDevice {
  bool ready = false;
  uint32_t* scratch = nullptr;   // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
constexpr int kNoAllocMaxDevices = 64;
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
std::mutex g_noalloc_mu;

static_assert(kNoAllocScratchBytes == 1024, "documented size of the static scratch array");

template <int D, bool kCausal>
int noalloc_prepare() {   // opt in to the large dynamic shared memory of one variant
  PTXB200_CUDA_TRY(cudaFuncSetAttribute(fa_fwd_kernel<D, kCausal, true>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        FaCfg<D>::kSmemBytes));
  return PTXB200_OK;
}

template <int D, bool kCausal>
int noalloc_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                   const FaParams& p, int grid, cudaStream_t stream) {
  using C = FaCfg<D>;
  fa_fwd_kernel<D, kCausal, true><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  PTXB200_CUDA_TRY(cudaGetLastError());
  return PTXB200_OK;
}

}  // namespace
}  // namespace ptxb200

extern "C" int fa_fwd_bf16_noalloc(void* O, const void* Q, const void* K, const void* V, int B,
                                   int H, int S, int D, float sm_scale, int causal,
                                   unsigned flags, void* stream_v) {
  using namespace ptxb200;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (O == nullptr || Q == nullptr || K == nullptr || V == nullptr) return PTXB200_E_INVALID;
  if (B <= 0 || H <= 0 || S <= 0 || D <= 0) return PTXB200_E_INVALID;
  if (causal != 0 && causal != 1) return PTXB200_E_INVALID;
  if (flags & ~(PTXB200_FA_NO_LAZY_RESCALE | PTXB200_FA_SINGLE_BLOCKS | PTXB200_FA_NO_TAIL_SPLIT |
                PTXB200_FA_ALWAYS_TAIL_SPLIT)) return PTXB200_E_INVALID;
  if (!(sm_scale > 0.0f) || !(sm_scale < 1e30f)) return PTXB200_E_INVALID;
  if ((D != 64 && D != 128) || (S % 128 != 0 && !causal)) return PTXB200_E_SHAPE;
  if ((long long)B * H * S >= (1ll << 31)) return PTXB200_E_SHAPE;
  if (!aligned16(O) || !aligned16(Q) || !aligned16(K) || !aligned16(V)) return PTXB200_E_ALIGN;
  cudaStream_t stream = (cudaStream_t)stream_v;

  int dev = -1;
  PTXB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    set_error_text("fa_fwd_bf16_noalloc: device ordinal beyond the 64 this entry point tracks");
    return PTXB200_E_CAPACITY;
  }
  NoAllocDevice nd;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice& slot = g_noalloc_dev[dev];
    if (!slot.ready) {
      // one-time set-up for this device (it is the current one): capability, SM
      // count and the DEVICE address of the static scratch array. Because the first
      // call on a device does this, that call should come before any stream capture.
      int cc_major = 0;
      PTXB200_CUDA_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev));
      if (cc_major != 10) {
        set_error_text("current device is not compute capability 10.x (sm_100a code only)");
        return PTXB200_E_DEVICE;
      }
      PTXB200_CUDA_TRY(cudaDeviceGetAttribute(&slot.sm_count, cudaDevAttrMultiProcessorCount, dev));
      void* ptr = nullptr;
      PTXB200_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
      slot.scratch = reinterpret_cast<uint32_t*>(ptr);
      int rc;
      if ((rc = noalloc_prepare<128, false>()) != PTXB200_OK) return rc;
      if ((rc = noalloc_prepare<128, true>()) != PTXB200_OK) return rc;
      if ((rc = noalloc_prepare<64, false>()) != PTXB200_OK) return rc;
      if ((rc = noalloc_prepare<64, true>()) != PTXB200_OK) return rc;
      slot.ready = true;
    }
    nd = slot;
  }

  FaParams p;
  // whole items only: cutting the last round along the key axis needs scratch in proportion
  // to the SM count, which this entry point does not have
  fill_params(p, O, nullptr, B, H, H, S, sm_scale, flags, nullptr, nd.scratch,
              plan_schedule(B * H, (S + 255) / 256, (S + kAttnRows - 1) / kAttnRows, causal, flags, nd.sm_count, false));
  p.cta_flags = nd.scratch + kNoAllocFlagBase;
  const int units = (causal && p.pair_mode) ? p.bh * ((p.num_mblocks + 1) / 2) : p.total_work;
  const int grid = units < nd.sm_count ? units : nd.sm_count;
  if (grid > kNoAllocMaxCtas) {
    set_error_text("fa_fwd_bf16_noalloc: launch needs more CTAs than the 240 flag slots of the "
                   "static scratch array");
    return PTXB200_E_CAPACITY;
  }

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_tmap_bf16_3d(&tq, Q, (uint64_t)B * H, S, D, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_3d(&tk, K, (uint64_t)B * H, S, D, 128, 64)) != PTXB200_OK) return rc;
  if ((rc = encode_tmap_bf16_3d(&tv, V, (uint64_t)B * H, S, D, 128, 64)) != PTXB200_OK) return rc;

  // The array keeps what the previous call left: the status word and the flags of
  // the CTAs this launch uses must start at zero.
  PTXB200_CUDA_TRY(cudaMemsetAsync(nd.scratch, 0, (size_t)(kNoAllocFlagBase + grid) * 4, stream));

  if (D == 128) {
    return causal ? noalloc_launch<128, true>(tq, tk, tv, p, grid, stream)
                  : noalloc_launch<128, false>(tq, tk, tv, p, grid, stream);
  }
  return causal ? noalloc_launch<64, true>(tq, tk, tv, p, grid, stream)
                : noalloc_launch<64, false>(tq, tk, tv, p, grid, stream);
}


// Reads back what fa_fwd_bf16_noalloc launches on the current device left in the static
// array, without allocating: waits for `stream`, copies the status word and the per-CTA
// flags to the caller's host memory and returns the word (0 = every wait completed).
extern "C" int fa_fwd_bf16_noalloc_status(uint32_t* cta_flags_out, int max_flags, void* stream_v) {
  using namespace ptxb200;
  if (max_flags < 0 || (cta_flags_out == nullptr && max_flags > 0)) return PTXB200_E_INVALID;
  cudaStream_t stream = (cudaStream_t)stream_v;
  int dev = -1;
  PTXB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    set_error_text("fa_fwd_bf16_noalloc_status: device ordinal beyond the 64 this entry point tracks");
    return PTXB200_E_CAPACITY;
  }
  uint32_t* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_dev[dev].ready) scratch = g_noalloc_dev[dev].scratch;
  }
  const int n_flags = max_flags < kNoAllocMaxCtas ? max_flags : kNoAllocMaxCtas;
  if (scratch == nullptr) {
    // no fa_fwd_bf16_noalloc launch on this device yet: nothing to report
    PTXB200_CUDA_TRY(cudaStreamSynchronize(stream));
    for (int i = 0; i < n_flags; ++i) cta_flags_out[i] = 0;
    return PTXB200_OK;
  }
  uint32_t host[kNoAllocScratchWords];
  PTXB200_CUDA_TRY(cudaMemcpyAsync(host, scratch, sizeof(host), cudaMemcpyDeviceToHost, stream));
  PTXB200_CUDA_TRY(cudaStreamSynchronize(stream));
  for (int i = 0; i < n_flags; ++i) cta_flags_out[i] = host[kNoAllocFlagBase + i];
  if (host[0] != 0) {
    // first blame is consumed by this read, as with ptxb200_sync_status
    PTXB200_CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(uint32_t), stream));
    PTXB200_CUDA_TRY(cudaStreamSynchronize(stream));
  }
  return (int)host[0];
}
