"""TEST INFRASTRUCTURE -- numpy restatement of the reference's CPU checkers and a
ctypes binding of the C restatement (oracle/attention_oracle.c).

numpy versions (authoritative for small cases; they follow the reference line by
line):
  attention_ref_numpy  fab_cpu_ref   test/gpu/blackwell/flash_attention_defs.jl:967-976
                       fam_cpu_ref   test/gpu/ampere/flash_attention.jl:284-299 (causal)
  gemm_ref_numpy       _ghb_cpu_ref  test/gpu/blackwell/gemm_highperf_blackwell.jl:224-228
bf16 rounding is round-to-nearest-even on the fp32 bit pattern, as Julia's
BFloat16(x) conversion does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_DIR, "liboracle.so")
_lib = None


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 array -> uint16 bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = ((u & 0x7F800000) == 0x7F800000) & ((u & 0x007FFFFF) != 0)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x0040, r)
    return r.astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> fp32."""
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _quantise(x: np.ndarray) -> np.ndarray:
    return from_bf16_bits(to_bf16_bits(x))


def attention_ref_numpy(Q: np.ndarray, K: np.ndarray, V: np.ndarray, sm_scale: float,
                        causal: bool = False) -> np.ndarray:
    """One (batch, head) slice: Q, K, V are (S, D) fp32; returns fp32 (S, D).

    Qb = Float32.(BFloat16.(Q)) ...; scores = (Qb * Kb') .* sm_scale;
    [causal: scores[r, c] = -Inf for c > r]; rmax; ex = exp.(scores .- rmax);
    (ex ./ sum(ex)) * Vb
    """
    Qb, Kb, Vb = _quantise(Q), _quantise(K), _quantise(V)
    scores = (Qb @ Kb.T).astype(np.float32) * np.float32(sm_scale)
    if causal:
        S = scores.shape[0]
        scores = np.where(np.triu(np.ones((S, S), dtype=bool), k=1), np.float32(-np.inf), scores)
    rmax = scores.max(axis=1, keepdims=True)
    ex = np.exp(scores - rmax, dtype=np.float32)
    return ((ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)) @ Vb).astype(np.float32)


def attention_lse_numpy(Q: np.ndarray, K: np.ndarray, sm_scale: float, causal: bool = False) -> np.ndarray:
    """Per query row log(sum_j exp(q.k_j * sm_scale)) over the kept keys, float64 on
    bf16-quantised inputs: the row statistic behind fab_cpu_ref's normalisation
    (rmax + log(sum(ex)) in test/gpu/blackwell/flash_attention_defs.jl:972-975)."""
    Qb, Kb = _quantise(Q).astype(np.float64), _quantise(K).astype(np.float64)
    scores = (Qb @ Kb.T) * float(sm_scale)
    if causal:
        S = scores.shape[0]
        scores = np.where(np.triu(np.ones((S, S), dtype=bool), k=1), -np.inf, scores)
    rmax = scores.max(axis=1, keepdims=True)
    return (rmax[:, 0] + np.log(np.exp(scores - rmax).sum(axis=1))).astype(np.float32)


def gemm_ref_numpy(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """A (M,K), B (K,N) fp32 -> fp32 (M,N) on bf16-quantised inputs."""
    return (_quantise(A) @ _quantise(B)).astype(np.float32)


# ----------------------------- row-wise neighbours ------------------------------
# Restatements of the reference's CPU references for its row-wise kernels, float64
# inside like theirs. Parity unpinned in the same sense as the attention oracle:
# the reference's tests hold tolerances (atol 1e-4, rtol 1e-3), not output vectors.

def softmax_ref_numpy(X: np.ndarray) -> np.ndarray:
    """softmax_ref, test/gpu/softmax.jl:139-149."""
    x = X.astype(np.float64)
    x = x - x.max(axis=1, keepdims=True)
    e = np.exp(x)
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def rms_norm_ref_numpy(X: np.ndarray, W: np.ndarray, eps: float) -> np.ndarray:
    """rms_norm_ref, test/gpu/rms_norm.jl:109-119."""
    x = X.astype(np.float64)
    ms = (x * x).sum(axis=1, keepdims=True) / x.shape[1]
    return (x * (1.0 / np.sqrt(ms + np.float64(np.float32(eps)))) * W.astype(np.float64)).astype(np.float32)


def layer_norm_ref_numpy(X: np.ndarray, W: np.ndarray, B: np.ndarray, eps: float) -> np.ndarray:
    """layer_norm_ref, test/gpu/layer_norm.jl:125-136 (biased variance)."""
    x = X.astype(np.float64)
    m = x.sum(axis=1, keepdims=True) / x.shape[1]
    v = ((x - m) ** 2).sum(axis=1, keepdims=True) / x.shape[1]
    return ((x - m) * (1.0 / np.sqrt(v + np.float64(np.float32(eps)))) * W.astype(np.float64)
            + B.astype(np.float64)).astype(np.float32)


def swiglu_ref_numpy(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """swiglu_ref, test/gpu/swiglu.jl:70-75."""
    g = gate.astype(np.float64)
    return (g * (1.0 / (1.0 + np.exp(-g))) * up.astype(np.float64)).astype(np.float32)


# ----------------------------- C restatement -----------------------------------

def build_c_oracle(force: bool = False) -> str:
    src = os.path.join(_DIR, "attention_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(_LIB_PATH):
        r = subprocess.run(["make", "-C", _DIR, "-B", "liboracle.so"], stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + r.stdout)
    return _LIB_PATH


def _c():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build_c_oracle()
        L = ctypes.CDLL(_LIB_PATH)
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.oracle_attention_fwd.restype = ci
        L.oracle_attention_fwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, cf, ci, ci]
        L.oracle_gemm.restype = ci
        L.oracle_gemm.argtypes = [vp, vp, vp, ci, ci, ci, ci]
        L.oracle_num_threads.restype = ci
        _lib = L
    return _lib


def c_oracle_threads() -> int:
    return int(_c().oracle_num_threads())


def attention_ref_c(q_bits: np.ndarray, k_bits: np.ndarray, v_bits: np.ndarray, sm_scale: float,
                    causal: bool = False, nthreads: int = 0) -> np.ndarray:
    """q/k/v: uint16 bf16 bit patterns of shape (BH, S, D). Returns fp32 (BH, S, D)."""
    q_bits, k_bits, v_bits = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q_bits, k_bits, v_bits))
    BH, S, D = q_bits.shape
    out = np.empty((BH, S, D), dtype=np.float32)
    rc = _c().oracle_attention_fwd(q_bits.ctypes.data, k_bits.ctypes.data, v_bits.ctypes.data,
                                   out.ctypes.data, BH, S, D, ctypes.c_float(sm_scale), int(causal), nthreads)
    if rc != 0:
        raise RuntimeError("oracle_attention_fwd failed")
    return out


def gemm_ref_c(a_bits: np.ndarray, bt_bits: np.ndarray, nthreads: int = 0) -> np.ndarray:
    """a: (M,K), bt: (N,K) uint16 bf16 bit patterns. Returns fp32 (M,N)."""
    a_bits, bt_bits = (np.ascontiguousarray(a, dtype=np.uint16) for a in (a_bits, bt_bits))
    M, K = a_bits.shape
    N = bt_bits.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    rc = _c().oracle_gemm(a_bits.ctypes.data, bt_bits.ctypes.data, out.ctypes.data, M, N, K, nthreads)
    if rc != 0:
        raise RuntimeError("oracle_gemm failed")
    return out
