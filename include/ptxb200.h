/*
 * ptxb200 -- C ABI of the sm_100a (B200) native library for the one hot path of
 * jool-space/PTX.jl: the tcgen05 flash-attention forward kernel and the
 * tcgen05 bf16 GEMM it is built from.
 *
 * Everything here is plain C: raw device pointers, ints and a CUDA stream
 * handle passed as void* (a cudaStream_t / CUstream; NULL = the legacy default
 * stream). No torch or C++ types cross this boundary.
 *
 * Conventions shared by every entry point
 *   - Work is enqueued asynchronously on `stream`, on the CUDA device that is
 *     current in the calling thread. The caller owns every buffer and keeps it
 *     alive until the stream has passed the enqueued work (the reference states
 *     the same ownership rule: src/lib/tensor_map.jl:40-42,173-178,
 *     bench/flash_attention.jl:38-40).
 *   - Return value: 0 = enqueued. Negative = the call was rejected on the host
 *     and nothing was launched (see PTXB200_E_*). Device-side trouble (a bounded
 *     wait inside a kernel ran out) never traps or hangs; it is recorded in a
 *     per-device status word that ptxb200_sync_status() returns as a positive
 *     code (0x32000000 | site << 8 | aux).
 *   - All device pointers must be 16-byte aligned (TMA and 128-bit stores).
 *   - Only compute capability 10.x devices are accepted. There is no CPU or
 *     library fallback: on any other device the calls return
 *     PTXB200_E_DEVICE.
 */
#ifndef PTXB200_H_
#define PTXB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTXB200_OK 0
#define PTXB200_E_INVALID (-1)   /* null pointer, non-positive size, bad flag       */
#define PTXB200_E_SHAPE (-2)     /* shape outside the supported contract           */
#define PTXB200_E_ALIGN (-3)     /* pointer or leading dimension not 16-B aligned   */
#define PTXB200_E_CUDA (-4)      /* a CUDA runtime call failed (see ptxb200_last_cuda_error) */
#define PTXB200_E_DRIVER (-5)    /* cuTensorMapEncodeTiled unavailable or failed    */
#define PTXB200_E_DEVICE (-6)    /* current device is not compute capability 10.x   */
#define PTXB200_E_CAPACITY (-7)  /* request exceeds a fixed, documented capacity    */

/* gemm_bf16 flags */
#define PTXB200_GEMM_F32_OUT 0x1u /* write C as fp32 (the reference kernel's output type) */
#define PTXB200_GEMM_NO_SPLIT 0x2u /* never cut tiles along K: every C element is one
                                      accumulation in k order whatever the tile count
                                      (see "Few tiles, long K" at gemm_bf16) */
#define PTXB200_GEMM_ONE_CTA 0x4u  /* always the one-CTA-per-tile kernel, never the CTA-pair one */

/* fa_fwd_bf16 flags */
#define PTXB200_FA_NO_LAZY_RESCALE 0x1u /* rescale O on every row-max increase (no 2^8 slack) */
#define PTXB200_FA_SINGLE_BLOCKS 0x2u   /* causal: hand out single 256-row blocks, longest first, instead
                                           of equal-length pairs of blocks (same results bit for bit) */
#define PTXB200_FA_ALWAYS_TAIL_SPLIT 0x8u /* cut the last round whenever it can be cut, whether or not the
                                            library expects it to pay (tests, measurements) */
#define PTXB200_FA_NO_TAIL_SPLIT 0x4u   /* never cut the items of the last, partly filled round along the
                                           key axis (see "Last round" at fa_fwd_bf16): every output row is
                                           then one accumulation in key order whatever the SM count */

/* Library version: major*10000 + minor*100 + patch. */
int ptxb200_version(void);

/* Human-readable text for a return code (negative host codes and positive
 * device status codes). Never returns NULL. */
const char* ptxb200_strerror(int code);

/* Text of the last CUDA runtime / driver error seen by the calling thread inside
 * this library ("" if none). */
const char* ptxb200_last_cuda_error(void);

/*
 * C[M,N] = A[M,K] * B[K,N], bf16 operands, fp32 accumulation in tensor memory,
 * bf16 (default) or fp32 (PTXB200_GEMM_F32_OUT) output.
 *
 *   A   [M,K] row-major bf16 (K contiguous)
 *   Bt  B stored column-major, i.e. B transposed: [N,K] row-major bf16
 *   C   [M,N] row-major with leading dimension ldc (elements), ldc >= N
 *
 * Shape contract: M % 128 == 0, N % 128 == 0, K % 64 == 0, all > 0;
 * ldc * sizeof(element) % 16 == 0.
 *
 * Few tiles, long K: when the 128x256 output tiles number at most half the SMs and
 * K is long enough, every tile is cut along K and shared by at least twice as many
 * SMs; the partial sums meet in fp32 scratch that the library keeps per (device,
 * stream) -- 256 KiB per CTA of the launch, at most 38 MB, allocated (cudaMalloc) by
 * the first launch on a stream that needs it, so make that launch outside stream
 * capture or pass PTXB200_GEMM_NO_SPLIT; at most 16 such buffers exist per process (the
 * least recently used one is waited for and freed when a 17th stream asks), all freed
 * by ptxb200_shutdown -- and a second small kernel on the same stream adds them up.
 * Results stay reproducible from launch to launch; they differ in the last bits from
 * the unsplit summation order, which PTXB200_GEMM_NO_SPLIT keeps. No reference
 * counterpart (test/gpu/blackwell/gemm_highperf_blackwell.jl:27-32 leaves it).
 *
 * Replaces the reference's _run_ghb launch of _ghb_gemm_kernel! /
 * _ghb_persistent_kernel! (test/gpu/blackwell/gemm_highperf_blackwell.jl:69-199,
 * 230-269, 317-468): same operand packing (A K-fast, B as [N,K] K-fast), same
 * fp32 accumulation; the reference writes fp32 only.
 */
int gemm_bf16(void* C, const void* A, const void* Bt, int M, int N, int K, int ldc,
              unsigned flags, void* stream);

/*
 * Uniform grouped GEMM: C[g] = A[g] * B[g] for g in [0, G), every group of the
 * same shape, in one launch.
 *
 *   A   [G*M, K] row-major bf16: group g is rows g*M .. g*M+M-1
 *   Bt  [G*N, K] row-major bf16: group g's B transposed is rows g*N .. g*N+N-1
 *   C   [G*M, N] row-major with leading dimension ldc (elements), ldc >= N
 *
 * Shape contract: G > 0, M % 128 == 0, N % 64 == 0, K % 64 == 0;
 * ldc * sizeof(element) % 16 == 0. Flags as gemm_bf16.
 *
 * Replaces the reference's _run_ggb launch of _grouped_gemm_bw_kernel!
 * (test/gpu/blackwell/grouped_gemm.jl:43-158, 208-232): same stacked operand
 * packing (_ggb_pack_A / _ggb_pack_B, :185-206), grid-z = group there, one more
 * factor of the persistent tile loop here; the reference writes fp32 only and fixes
 * N = 64.
 */
int gemm_bf16_grouped(void* C, const void* A, const void* Bt, int G, int M, int N, int K, int ldc,
                      unsigned flags, void* stream);

/*
 * Row-wise fp32 kernels either side of attention in a transformer block. X and Y
 * are [rows, N] row-major fp32, W and Bias are [N] fp32; one read of X and one
 * write of Y per call. Shape contract: rows > 0, N % 4 == 0, 4 <= N <= 32768;
 * every pointer 16-byte aligned (so every row is). Asynchronous on `stream`.
 *
 *   softmax_f32     Y[r,i] = exp(X[r,i] - max_i X[r,:]) / sum_i exp(X[r,i] - max)
 *                   replaces _softmax_v4_kernel! (test/gpu/softmax.jl:30-140)
 *   rms_norm_f32    Y[r,i] = X[r,i] * W[i] / sqrt(mean_i X[r,:]^2 + eps)
 *                   replaces _rms_norm_v4_kernel! (test/gpu/rms_norm.jl:30-106)
 *   layer_norm_f32  Y[r,i] = (X[r,i] - mean) / sqrt(var + eps) * W[i] + Bias[i]
 *                   (biased variance) replaces _layer_norm_v4_kernel!
 *                   (test/gpu/layer_norm.jl:24-122)
 *   swiglu_f32      out[k] = gate[k] / (1 + exp(-gate[k])) * up[k] over n elements,
 *                   n % 4 == 0; replaces _swiglu_v4_kernel! (test/gpu/swiglu.jl:31-69)
 *
 * The reference kernels take N (or F) and the block size as compile-time values
 * with N % (block*4) == 0 and launch one CTA per row; these take them at run time.
 */
int softmax_f32(void* Y, const void* X, int rows, int N, void* stream);
int rms_norm_f32(void* Y, const void* X, const void* W, int rows, int N, float eps, void* stream);
int layer_norm_f32(void* Y, const void* X, const void* W, const void* Bias, int rows, int N,
                   float eps, void* stream);
int swiglu_f32(void* out, const void* gate, const void* up, long long n, void* stream);

/*
 * O = softmax(Q K^T * sm_scale [+ causal mask]) V, row-wise, per (batch, head).
 *
 *   Q, K, V, O  [B,H,S,D] row-major bf16 == a 2-D (B*H*S, D) matrix, D contiguous
 *               (the reference's layout: flash_attention_defs.jl:90, 979-986)
 *   D           64 or 128
 *   S           any length >= 1 (work is cut in 256-row items of 128-key tiles; rows
 *               and keys past the end of a sequence are loaded as zeros through
 *               per-head tensor maps, masked out of the softmax and not written.
 *               The reference asserts S % 256 == 0 and more:
 *               bench/flash_attention.jl:43-47)
 *   causal      0: every key; 1: key j is kept for query i iff j <= i
 *               (mask convention of test/gpu/ampere/flash_attention.jl:176-186)
 *   dbg         NULL, or 64 uint32 words on the device that receive per-role
 *               progress counters of CTA 0 (diagnostics only)
 *
 * Scores are accumulated in fp32, the softmax runs in fp32 with the row maximum
 * subtracted, P is rounded to bf16 for the second product, O is accumulated in
 * fp32 and rounded once to bf16.
 *
 * Last round: work is dealt to one persistent CTA per SM in 256-row items, round robin
 * (the reference's distribution, flash_attention_defs.jl:269-272). When the last round
 * would leave SMs idle -- items % SMs != 0, most of all when there are fewer items than
 * SMs -- and cutting pays, the items of that round are cut along the key axis into equal
 * shares for all SMs; the pieces of an item meet, unnormalised and in fp32, in scratch
 * that the library keeps per (device, stream) (about 133 KB per SM at D = 128, allocated
 * with cudaMalloc by the first such launch on a stream -- make it outside stream capture
 * -- and freed by ptxb200_shutdown; see gemm_bf16 for the table's bound), and the CTA
 * that holds an item's first keys merges them by the log-sum-exp rule before the one
 * rounding to bf16. Results stay reproducible from launch to launch on one GPU model;
 * they differ in the last bits from the uncut key order, which PTXB200_FA_NO_TAIL_SPLIT
 * keeps. The CTAs of such a launch wait for one another's pieces (bounded, like every
 * wait here), so they must be able to run at the same time: do not run other work that
 * occupies the GPU's SMs for seconds concurrently with it.
 *
 * Replaces the reference's fab_setup launch closure of fab_kernel!
 * (bench/flash_attention.jl:41-85; test/gpu/blackwell/flash_attention_defs.jl:
 * 621-961), which covers D = 128, non-causal only.
 */
int fa_fwd_bf16(void* O, const void* Q, const void* K, const void* V, int B, int H, int S, int D,
                float sm_scale, int causal, unsigned flags, void* dbg, void* stream);

/*
 * fa_fwd_bf16 with two additions next to the reference's path (its kernel has
 * neither: one K/V head per query head, no statistics output --
 * flash_attention_defs.jl:621-630):
 *   H_kv  number of key/value heads per batch entry; must divide H. Query head h
 *         attends to key/value head h / (H / H_kv) (grouped-query attention).
 *         K and V are [B, H_kv, S, D].
 *   lse   NULL, or B*H*S floats on the device that receive, per query row,
 *         log(sum_j exp(q.k_j * sm_scale)) over the kept keys (natural log) --
 *         what a backward pass or a split-sequence combine needs.
 * Everything else as fa_fwd_bf16 (which is this call with lse = NULL, H_kv = H).
 */
int fa_fwd_bf16_ex(void* O, void* lse, const void* Q, const void* K, const void* V, int B, int H,
                   int H_kv, int S, int D, float sm_scale, int causal, unsigned flags, void* dbg,
                   void* stream);

/*
 * fa_fwd_bf16 without any allocation. (No counterpart in the reference: its
 * launch closure allocates nothing per call either, but its set-up uploads three
 * descriptor blobs into freshly allocated device memory.)
 *
 * Who needs it: a caller that must not cause a device allocation at the point
 * where it launches attention -- a serving loop that carved up all device memory
 * beforehand and treats any later cudaMalloc as an error (or would simply fail,
 * the device being full), a latency-critical section where the implicit
 * synchronisation of cudaMalloc is unacceptable, or a host runtime with its own
 * device memory pool (a Julia or Python session) that wants every byte on the GPU
 * to come from that pool. fa_fwd_bf16 is unsuitable there because its first call
 * on a device cudaMalloc's the library's small workspace.
 *
 * How: the kernel's scratch (the status word of its bounded waits plus one
 * "this CTA timed out" flag per CTA) lives in a 1 KiB array that is part of the
 * loaded library image, so every GPU that loads libptxb200.so holds that 1 KiB
 * until the process exits. This function never calls cudaMalloc, cudaFree or any
 * allocating routine. Arguments, layout, shape contract and results are those of
 * fa_fwd_bf16 (same kernel code); there is no dbg argument.
 *
 * Limits and rules
 *   - Non-causal calls need S % 128 == 0 here (PTXB200_E_SHAPE otherwise); fa_fwd_bf16
 *     takes any S.
 *   - Capacity: at most 240 CTAs (one per SM) and device ordinals 0..63; beyond
 *     that the call returns PTXB200_E_CAPACITY and launches nothing.
 *   - The first call on each device looks up the array's device address and sets
 *     kernel attributes. Make that first call outside any stream capture.
 *   - All calls on one device share the one array. The function clears what must
 *     start at zero on `stream` before each launch, so calls that follow each
 *     other on a stream are fine; calls that can overlap on the GPU (different
 *     streams, or different host threads launching on the same device) race on
 *     the status word and flags. The attention results themselves do not depend
 *     on the scratch contents unless a wait runs out.
 *   - ptxb200_sync_status() reports on fa_fwd_bf16/gemm_bf16 launches only; it
 *     does not read this array (it would allocate the workspace). Use
 *     fa_fwd_bf16_noalloc_status() below.
 */
int fa_fwd_bf16_noalloc(void* O, const void* Q, const void* K, const void* V, int B, int H, int S,
                        int D, float sm_scale, int causal, unsigned flags, void* stream);

/*
 * The status read-back that goes with fa_fwd_bf16_noalloc, and like it allocates
 * nothing (no counterpart in the reference; its beacon read-back,
 * flash_attention_defs.jl:989-998, copies a buffer the caller allocated).
 *
 * Waits for `stream`, then copies the static array of the current device to the host:
 * returns its status word -- 0 if every bounded wait of the fa_fwd_bf16_noalloc
 * launches since the last read completed, else the positive first-blame code
 * (ptxb200_strerror decodes it; the outputs of that launch are invalid) -- and clears
 * the word when it was nonzero. If cta_flags_out is not NULL it receives
 * min(max_flags, 240) words, word i nonzero iff a wait ran out in CTA i of the most
 * recent launch (each launch clears the flags it uses). Before any
 * fa_fwd_bf16_noalloc call on the device it returns 0. The sharing rule of the
 * array applies: a read that overlaps a launch on another stream races with it.
 */
int fa_fwd_bf16_noalloc_status(uint32_t* cta_flags_out, int max_flags, void* stream);

/*
 * The work distribution fa_fwd_bf16 would use for a problem on a GPU with `sm_count`
 * SMs, computed on the host (no GPU needed; diagnostics and tests). out receives 10 ints
 * -- 256-row blocks per head, batch*heads, 128-key tiles per head, causal, pairs,
 * CTAs, units dealt round robin, units of the cut last round, steps of that round,
 * CTAs sharing it -- then, per CTA of a cut last round, its segment count and 6 ints per
 * segment (block, batch*head, first tile, end tile, tiles of the item, pieces parked by
 * following CTAs). Returns the ints written, PTXB200_E_CAPACITY if cap is too small.
 * The reference's distribution is the round robin of flash_attention_defs.jl:269-272.
 */
int ptxb200_fa_plan(int B, int H, int S, int causal, unsigned flags, int sm_count, int* out, int cap);

/*
 * Synchronise `stream`, then return and clear that stream's status word on the
 * current device: 0 if every kernel enqueued on `stream` through this library since
 * the last call ran to completion normally, a positive code if a bounded device-side
 * wait ran out (the affected outputs are then invalid), PTXB200_E_CUDA if the stream
 * itself reports an error. Each stream that launches through the library gets a word of
 * its own (the first 128 streams per device; beyond that, streams share words by hash
 * and a read may then report a neighbour's failure). Replaces the reference's beacon
 * buffer read-back (flash_attention_defs.jl:224-267, 989-998).
 */
int ptxb200_sync_status(void* stream);

/*
 * The same for every stream at once: synchronises the current DEVICE, returns the
 * first nonzero status word of any stream that launched through this library on it
 * (0 if none) and clears them all. For callers that launch on several streams and check
 * once at the end. No reference counterpart beyond the one above.
 */
int ptxb200_device_status(void);

/*
 * Bring-up probes with known answers, restating the reference's single-
 * instruction runtime tests (test/gpu/blackwell/tcgen05_roundtrip.jl:22-88,
 * tcgen05_mma_probe.jl:39-131, tcgen05_b128_probe.jl). `which`:
 *   0  TMEM store -> load identity. out: 128*128 uint32, out[r*128+c] must equal
 *      (r << 16 | c) ^ 0x5A5A0000.
 *   1  one attention tile, D = 128:  out_s = Q K^T (128x128 fp32) and
 *      out_o = P V (128xD fp32) with P (bf16, 128x128) read from tensor memory
 *      and V as an MN-major shared-memory operand.
 *   2  the same with D = 64.
 *   3  a bounded wait that nothing satisfies (the native counterpart of reading the
 *      reference's beacons after a stuck wait, bench/flash_attention.jl:163-179): one
 *      thread waits on a barrier nobody arrives on, gives up after the wait limit
 *      (1.5 s), and the kernel returns. out: 3 uint32 = {0, 0, 0xD0E5} (both waits
 *      report failure, the kernel reached its end); the next ptxb200_sync_status
 *      returns the positive code of wait site 15 ("probe").
 *   4  throughput of one SM's exponential unit (no reference counterpart; the
 *      reference's kernel comments assume 16 ex2 per clock per SM,
 *      flash_attention_defs.jl:355-387): one CTA of 16 warps runs seven timed passes --
 *      4, 8 and 16 warps of nothing but ex2.approx, then 8 and 16 warps of the softmax's
 *      inner mix (packed fma, two ex2, packed add, bf16 pack), then 8 and 16 warps of the
 *      packed ex2.approx.ftz.bf16x2 (two exponentials per instruction). out: 16 uint32;
 *      out[2k] = cycles of pass k, out[2k+1] = ex2 executed in it.
 * For 1 and 2: q,k,v are (128, D) bf16, p is (128,128) bf16, all row-major.
 * Unused pointers may be NULL for probes 0, 3 and 4.
 */
int ptxb200_selftest(int which, void* out_s, void* out_o, const void* q, const void* k,
                     const void* v, const void* p, void* stream);

/* Release the per-device workspaces this library allocated. Optional. */
int ptxb200_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* PTXB200_H_ */
