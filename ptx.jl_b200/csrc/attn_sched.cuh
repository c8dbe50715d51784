// Work distribution of the attention kernel: which (query block, batch*head) items a CTA
// runs, and how the LAST, partly filled round of items is cut along the key axis so that
// every SM stays busy until the end.
//
// The reference deals whole items (m_block, bh) to its persistent CTAs round robin
// (test/gpu/blackwell/flash_attention_defs.jl:269-272) and accepts an idle tail: with U
// units on G CTAs the last round has R = U mod G units and G - R CTAs wait for it. Here
// the units of that last round are laid end to end on a line of key-tile STEPS (a step =
// one 128-key tile for both 128-row stages of an item), the line is cut into tail_ctas
// equal spans, and CTA c runs span c: the end of one item, possibly whole items, the
// start of another. A CTA that holds the first steps of an item it does not finish is
// that item's COMBINER; every other piece is the first thing its CTA runs in the tail, is
// written out unnormalised (fp32 O, row sum, basis) to that CTA's slot in global scratch,
// and is merged by the combiner. The rules that keep this simple:
//   * a cut of a causal item never leaves a piece shorter than two steps: it snaps to the
//     item's start or end instead, so the item's shorter first stage is never empty
//     (non-causal items can be cut anywhere);
//   * spans are at least twice that long, so no span snaps to nothing;
//   * every piece that is not an item's first is the FIRST segment of its CTA, hence one
//     scratch slot per CTA, and the pieces of an item sit in consecutive CTAs.
// Everything here compiles for host and device: the host runs the same code to decide
// whether a launch splits (and to verify the per-CTA segment count), tests run it on CPU.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define PTXB200_HD __host__ __device__ __forceinline__
#else
#define PTXB200_HD inline
#endif

namespace ptxb200 {

// Shortest piece of a cut item, in steps.
PTXB200_HD int fa_min_seg(int causal) { return causal ? 2 : 1; }
constexpr int kTailMaxSegs = 8;   // segments a CTA's span may hold (table size in shared memory)
constexpr int kTailMaxParts = 8;  // pieces one item is cut into at most (bounds the combiner's reads)

// What the kernel needs to know about the distribution (part of its parameters).
struct FaSched {
  int num_mblocks;   // 256-row query blocks per head
  int bh;            // batch * heads
  int nt_all;        // 128-key tiles per head
  int causal;
  int pair_mode;     // causal: units are pairs of blocks (n-1-t, t) of one head
  int grid;          // CTAs launched
  int full_units;    // units [0, full_units) are dealt round robin: unit q = cta + v * grid
  int tail_units;    // units [full_units, full_units + tail_units) are cut along the line
  int tail_steps;    // length of that line
  int tail_ctas;     // CTAs [0, tail_ctas) share the line equally
};

// One piece of work for a CTA: key tiles [j0, j1) of item (mb, bh), whose last stage has
// `len` tiles in all. j0 == 0 && j1 == len: a whole item. j0 > 0: a piece written to
// scratch. j0 == 0 && j1 < len: the combiner's piece; n_other more pieces follow in the
// next n_other CTAs.
struct FaSeg {
  int mb, bh, j0, j1, len, n_other;
};

// Steps of an item = key tiles its second stage visits (the first stage of a causal item
// visits one fewer, unless the sequence ends first).
PTXB200_HD int fa_item_steps(int mb, int nt_all, int causal) {
  if (!causal) return nt_all;
  const int x = 2 * mb + 2;
  return x < nt_all ? x : nt_all;
}
PTXB200_HD int fa_num_units(const FaSched& s) {
  return (s.causal && s.pair_mode) ? s.bh * ((s.num_mblocks + 1) >> 1) : s.bh * s.num_mblocks;
}
// Items of unit q, in the order they run: (bh, mb_a) and, for a pair, (bh, mb_b); mb_b = -1 if none.
PTXB200_HD void fa_unit_items(const FaSched& s, int q, int& bh, int& mb_a, int& mb_b) {
  const int n = s.num_mblocks;
  if (!s.causal || !s.pair_mode) {
    bh = q / n;
    const int r = q - bh * n;
    mb_a = s.causal ? n - 1 - r : r;   // causal single blocks: longest first within a head
    mb_b = -1;
    return;
  }
  const int pph = (n + 1) >> 1;
  bh = q / pph;
  const int t = q - bh * pph;
  const int far = n - 1 - t;
  mb_a = far;
  mb_b = (t != far) ? t : -1;          // the middle block of an odd count has no partner
}
PTXB200_HD void fa_unit_lens(const FaSched& s, int q, int& len_a, int& len_b) {
  int bh, mb_a, mb_b;
  fa_unit_items(s, q, bh, mb_a, mb_b);
  len_a = fa_item_steps(mb_a, s.nt_all, s.causal);
  len_b = mb_b >= 0 ? fa_item_steps(mb_b, s.nt_all, s.causal) : 0;
}

// A cut at line position x inside the unit that starts at `st` with items of len_a and
// len_b steps: moved to the nearest item edge if it would leave a piece shorter than
// min_seg.
PTXB200_HD int fa_snap(int x, int st, int len_a, int len_b, int min_seg) {
  int s0 = st, len = len_a;
  if (x - st >= len_a && len_b > 0) {
    s0 = st + len_a;
    len = len_b;
  }
  const int j = x - s0;
  if (j < min_seg) return s0;
  if (len - j < min_seg) return s0 + len;
  return x;
}

// Cut k of the tail line, k in [0, tail_ctas]. `loc(x, u, st)` sets u to the tail unit
// (0-based within the tail) whose steps contain line position x and st to its start.
template <class Loc>
PTXB200_HD int fa_tail_cut(const FaSched& s, int k, Loc& loc) {
  if (k <= 0) return 0;
  if (k >= s.tail_ctas) return s.tail_steps;
  // (k * tail_steps fits 32 bits for every launch the host lets through: both are bounded by
  // the SM count times the steps of a few hundred units)
  const int raw = (int)((unsigned)k * (unsigned)s.tail_steps / (unsigned)s.tail_ctas);
  int u, st, len_a, len_b;
  loc(raw, u, st);
  fa_unit_lens(s, s.full_units + u, len_a, len_b);
  return fa_snap(raw, st, len_a, len_b, fa_min_seg(s.causal));
}

// The segments of CTA `cta` in the tail, in order, into segs[0 .. kTailMaxSegs); returns
// how many there are (a count above kTailMaxSegs means the table is too small: the host
// then does not split this launch).
template <class Loc>
PTXB200_HD int fa_tail_segments(const FaSched& s, int cta, Loc& loc, FaSeg* segs) {
  if (cta >= s.tail_ctas) return 0;
  const int b0 = fa_tail_cut(s, cta, loc);
  const int b1 = fa_tail_cut(s, cta + 1, loc);
  int n = 0, pos = b0;
  int u, st;
  if (pos < b1) loc(pos, u, st);
  while (pos < b1) {
    int bh, mb_a, mb_b, len_a, len_b;
    fa_unit_items(s, s.full_units + u, bh, mb_a, mb_b);
    fa_unit_lens(s, s.full_units + u, len_a, len_b);
    // the item of this unit that holds pos
    const bool second = (pos - st >= len_a) && len_b > 0;
    const int s0 = second ? st + len_a : st;
    const int len = second ? len_b : len_a;
    FaSeg g;
    g.mb = second ? mb_b : mb_a;
    g.bh = bh;
    g.j0 = pos - s0;
    g.len = len;
    g.j1 = (b1 - s0 < len) ? b1 - s0 : len;
    g.n_other = 0;
    pos = s0 + g.j1;
    if (g.j0 == 0 && g.j1 < len) {
      // this CTA combines the item: count the pieces that follow in the next CTAs
      int k = cta + 2, cnt = 1;
      while (fa_tail_cut(s, k, loc) < s0 + len) {
        ++cnt;
        ++k;
      }
      g.n_other = cnt;
    }
    if (n < kTailMaxSegs) segs[n] = g;
    ++n;
    if (pos >= st + len_a + len_b) {   // on to the next unit
      st += len_a + len_b;
      ++u;
    }
  }
  return n;
}

}  // namespace ptxb200
