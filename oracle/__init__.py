"""TEST INFRASTRUCTURE -- CPU oracle for the attention / GEMM hot path and its row-wise neighbours.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm
may import this package. See oracle/attention_oracle.c for what it restates and
for the parity-pinning statement ("parity unpinned" for floating-point outputs:
the reference holds no golden outputs and cannot run where this was written).
"""
from .oracle import (attention_ref_numpy, attention_lse_numpy, attention_ref_c, gemm_ref_numpy, gemm_ref_c,  # noqa: F401
                     to_bf16_bits, from_bf16_bits, build_c_oracle, c_oracle_threads,
                     softmax_ref_numpy, rms_norm_ref_numpy, layer_norm_ref_numpy, swiglu_ref_numpy)
