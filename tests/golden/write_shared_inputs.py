"""Writes seeded Q, K, V as raw bf16 bit patterns, [B*H*S, D] row-major, for backends that
cannot share a random-number stream (Julia's MersenneTwister cannot be reproduced from
Python): the Julia bench twin (julia/bench/flash_attention_native.jl, PTX_FA_INPUTS) and
the Julia oracle (oracle/attention_oracle.jl) read these bytes; the Python tests regenerate
them from the same seed. Also writes the C oracle's fp32 output for a byte-level comparison.

  python tests/golden/write_shared_inputs.py <prefix> [B H S D seed sigma_qk causal]

Defaults: the CPU-runnable configuration (B=1, H=4, S=256, D=64, N(0,1), seed 20260001).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main(argv):
    import oracle
    prefix = argv[1]
    B, H, S, D, seed = (int(x) for x in (argv[2:7] if len(argv) >= 7 else (1, 4, 256, 64, 20260001)))
    sigma = float(argv[7]) if len(argv) > 7 else 1.0
    causal = bool(int(argv[8])) if len(argv) > 8 else False
    rng = np.random.Generator(np.random.Philox(seed))
    q, k, v = (oracle.to_bf16_bits((rng.standard_normal((B * H, S, D)) * s).astype(np.float32))
               for s in (sigma, sigma, 1.0))
    for name, arr in (("q", q), ("k", k), ("v", v)):
        arr.tofile(f"{prefix}_{name}.bin")
    oracle.build_c_oracle()
    o = oracle.attention_ref_c(q, k, v, 1.0 / np.sqrt(D), causal)
    o.astype(np.float32).tofile(f"{prefix}_o_c_f32.bin")
    print(f"wrote {prefix}_{{q,k,v}}.bin ({q.nbytes} bytes each) and {prefix}_o_c_f32.bin")


if __name__ == "__main__":
    main(sys.argv)
