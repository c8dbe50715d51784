"""Generates the committed golden fixtures under tests/golden/.

The reference (Julia) cannot run where these were made and holds no golden output
vectors for the attention / GEMM path, so the expected outputs here come from an
INDEPENDENT implementation: float64 arithmetic in PyTorch on the bf16-quantised
inputs (a different library and precision from both the CPU oracle and the CUDA
kernels). Inputs are stored as bf16 bit patterns so every consumer sees the same
bytes. Run:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def attention_f64(q, k, v, scale, causal):
    q, k, v = q.double(), k.double(), v.double()
    s = torch.einsum("bhid,bhjd->bhij", q, k) * scale
    if causal:
        S = s.shape[-1]
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    return torch.einsum("bhij,bhjd->bhid", torch.softmax(s, dim=-1), v).float().numpy()


def make_attention(name, B, H, S, D, seed, sigma_qk, sigma_v=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, S, D, generator=g) * sigma_qk).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, generator=g) * sigma_qk).to(torch.bfloat16)
    v = (torch.randn(B, H, S, D, generator=g) * sigma_v).to(torch.bfloat16)
    scale = 1.0 / D ** 0.5
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q=bits(q), k=bits(k), v=bits(v),
                        o=attention_f64(q, k, v, scale, False),
                        o_causal=attention_f64(q, k, v, scale, True),
                        sm_scale=np.float32(scale), seed=np.int64(seed))


def make_gemm(name, M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.rand(M, K, generator=g) * 2 - 1).to(torch.bfloat16)
    bt = (torch.rand(N, K, generator=g) * 2 - 1).to(torch.bfloat16)
    c = (a.double() @ bt.double().t()).float().numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), a=bits(a), bt=bits(bt), c=c, seed=np.int64(seed))


if __name__ == "__main__":
    # the CPU-runnable reference configuration: B=1 H=4 S=256 D=64, N(0,1), seed 20260001
    make_attention("attn_b1_h4_s256_d64", 1, 4, 256, 64, 20260001, 1.0)
    # a D=128 case at the reference's smallest test shape and input scale
    make_attention("attn_b1_h1_s256_d128", 1, 1, 256, 128, 7919 + 131 + 256, 0.5)
    # rescale-heavy input (scale 2.0), two KV tiles per query block and more
    make_attention("attn_b1_h1_s512_d128_scale2", 1, 1, 512, 128, 4242, 2.0)
    make_gemm("gemm_128_256_192", 128, 256, 192, 20260005)
    # Known answers held by the reference's own host tests and probes.
    known = {
        "sdesc_kmajor_b128": "0x4000404000010000",          # test/host/tcgen05_descriptors.jl:136-141
        "sdesc_fields": {"addr_shift": 0, "leading_shift": 16, "stride_shift": 32,
                         "fixed_bit": 46, "layout_shift": 61, "unit_bytes": 16},
        "layout_codes": {"NONE": 0, "B128_BASE32B": 1, "B128": 2, "B64": 4, "B32": 6},
        "idesc_fields": {"d_f32": [4, 1], "a_bf16": [7, 1], "b_bf16": [10, 1], "a_major_bit": 15,
                         "b_major_bit": 16, "n_shift": 17, "n_div": 8, "m_shift": 24, "m_div": 16},
        "tmem_lane_shift": 16,                                # test/host/tcgen05_layout.jl:13-33
        "fa_barrier_arena_bytes_reference": 248,              # test/host/barrier_sets.jl:33
        "mma_probe_ones_k16": 16.0,                           # tcgen05_mma_probe.jl:122-129
        "accum_probe_4x": 64.0,                               # tcgen05_accum_probe.jl:136
        "tensor_map": {"dtype_bf16": 9, "swizzle_128b": 3},  # src/lib/tensor_map.jl:57-87
    }
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(known, f, indent=1)
    for fn in sorted(os.listdir(HERE)):
        print(fn, os.path.getsize(os.path.join(HERE, fn)))
