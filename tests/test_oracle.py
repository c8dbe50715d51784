"""The CPU oracle (numpy and C restatements of the reference's CPU checkers)
against the committed golden fixtures, against each other, and on edge cases."""
import json
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")

ATTN_FIXTURES = ["attn_b1_h4_s256_d64", "attn_b1_h1_s256_d128", "attn_b1_h1_s512_d128_scale2"]


@pytest.mark.parametrize("name", ATTN_FIXTURES)
@pytest.mark.parametrize("causal", [False, True])
def test_attention_oracles_match_golden(oracle_mod, name, causal):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    q, k, v = z["q"], z["k"], z["v"]
    B, H, S, D = q.shape
    gold = z["o_causal" if causal else "o"].reshape(B * H, S, D)
    scale = float(z["sm_scale"])
    c = oracle_mod.attention_ref_c(q.reshape(B * H, S, D), k.reshape(B * H, S, D), v.reshape(B * H, S, D), scale, causal)
    # fp32 oracle vs float64 golden: rounding of fp32 dot products and exp only
    np.testing.assert_allclose(c, gold, rtol=2e-4, atol=2e-5)
    f = oracle_mod.from_bf16_bits
    for i in range(B * H):
        n = oracle_mod.attention_ref_numpy(f(q).reshape(B * H, S, D)[i], f(k).reshape(B * H, S, D)[i],
                                           f(v).reshape(B * H, S, D)[i], scale, causal)
        np.testing.assert_allclose(n, gold[i], rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(n, c[i], rtol=1e-4, atol=1e-5)


def test_gemm_oracles_match_golden(oracle_mod):
    z = np.load(os.path.join(GOLDEN, "gemm_128_256_192.npz"))
    c = oracle_mod.gemm_ref_c(z["a"], z["bt"])
    np.testing.assert_allclose(c, z["c"], rtol=1e-5, atol=1e-4)
    f = oracle_mod.from_bf16_bits
    n = oracle_mod.gemm_ref_numpy(f(z["a"]), f(z["bt"]).T)
    np.testing.assert_allclose(n, z["c"], rtol=1e-5, atol=1e-4)


def test_bf16_rounding_is_round_to_nearest_even(oracle_mod):
    import torch
    x = torch.randn(200000, generator=torch.Generator().manual_seed(3)) * 37.0
    special = torch.tensor([0.0, -0.0, 1.0, 1.00390625, 1.001953125, 1.005859375, float("inf"), -float("inf"),
                            3.3895314e38, 1e-40, 65504.0])
    x = torch.cat([x, special])
    want = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = oracle_mod.to_bf16_bits(x.numpy())
    assert np.array_equal(got, want)
    # ties: 1 + 2^-8 is exactly halfway between 1 and 1 + 2^-7 -> rounds to even (1.0)
    assert oracle_mod.to_bf16_bits(np.array([1.00390625], np.float32))[0] == 0x3F80
    assert oracle_mod.to_bf16_bits(np.array([1.01171875], np.float32))[0] == 0x3F82  # tie -> even mantissa
    assert np.isnan(oracle_mod.from_bf16_bits(oracle_mod.to_bf16_bits(np.array([np.nan], np.float32))))[0]
    y = oracle_mod.from_bf16_bits(got)
    assert np.array_equal(oracle_mod.to_bf16_bits(y), got)   # idempotent


def test_attention_edge_cases(oracle_mod):
    rng = np.random.default_rng(11)
    S, D = 64, 16
    Q, K, V = (rng.standard_normal((S, D)).astype(np.float32) for _ in range(3))
    # causal: the first row attends to key 0 only
    o = oracle_mod.attention_ref_numpy(Q, K, V, 0.25, True)
    np.testing.assert_allclose(o[0], oracle_mod.from_bf16_bits(oracle_mod.to_bf16_bits(V))[0], rtol=1e-6)
    # V = ones -> every output is 1 (rows of P sum to one)
    o1 = oracle_mod.attention_ref_numpy(Q, K, np.ones_like(V), 0.25, False)
    np.testing.assert_allclose(o1, 1.0, rtol=1e-6)
    # large logits stay finite thanks to the max subtraction
    ob = oracle_mod.attention_ref_numpy(Q * 50, K * 50, V, 1.0, False)
    assert np.isfinite(ob).all()
    qb, kb, vb = (oracle_mod.to_bf16_bits(x)[None] for x in (Q * 50, K * 50, V))
    np.testing.assert_allclose(oracle_mod.attention_ref_c(qb, kb, vb, 1.0, False)[0], ob, rtol=1e-4, atol=1e-5)
    # bad arguments are refused by the C side
    with pytest.raises(RuntimeError):
        oracle_mod.attention_ref_c(np.zeros((1, 4, 8), np.uint16), np.zeros((1, 4, 8), np.uint16),
                                   np.zeros((1, 4, 8), np.uint16), 1.0)   # D % 16 != 0


def test_c_oracle_thread_count_does_not_change_results(oracle_mod):
    rng = np.random.default_rng(5)
    q, k, v = (oracle_mod.to_bf16_bits(rng.standard_normal((3, 128, 64)).astype(np.float32)) for _ in range(3))
    a = oracle_mod.attention_ref_c(q, k, v, 0.125, True, nthreads=1)
    b = oracle_mod.attention_ref_c(q, k, v, 0.125, True, nthreads=4)
    assert np.array_equal(a, b)


def test_known_answers_file_is_consistent():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        known = json.load(f)
    s = known["sdesc_fields"]
    val = (16 // s["unit_bytes"]) << s["leading_shift"] | (1024 // s["unit_bytes"]) << s["stride_shift"] \
        | 1 << s["fixed_bit"] | known["layout_codes"]["B128"] << s["layout_shift"]
    assert val == int(known["sdesc_kmajor_b128"], 16)
    assert known["mma_probe_ones_k16"] == 16.0 and known["accum_probe_4x"] == 64.0


def test_rowwise_oracles_known_answers(oracle_mod):
    """Closed-form cases of the row-wise references (their only pins: the reference's
    tests hold tolerances, not vectors)."""
    o = oracle_mod
    N = 64
    np.testing.assert_allclose(o.softmax_ref_numpy(np.zeros((3, N), np.float32)), 1.0 / N, rtol=1e-7)
    x = np.log(np.arange(1, 5, dtype=np.float64)).astype(np.float32)[None, :]
    np.testing.assert_allclose(o.softmax_ref_numpy(x), np.arange(1, 5)[None, :] / 10.0, rtol=1e-6)
    ones = np.ones((2, N), np.float32)
    w = np.linspace(0.5, 1.5, N).astype(np.float32)
    np.testing.assert_allclose(o.rms_norm_ref_numpy(3 * ones, w, 0.0), np.broadcast_to(w, (2, N)), rtol=1e-6)
    ramp = np.tile(np.array([-1.0, 1.0], np.float32), N // 2)[None, :]          # mean 0, variance 1
    b = np.full(N, 0.25, np.float32)
    np.testing.assert_allclose(o.layer_norm_ref_numpy(ramp + 5.0, w, b, 0.0), ramp * w + b, rtol=1e-6)
    g = np.array([0.0, np.log(3.0), -np.log(3.0)], np.float32)
    u = np.array([2.0, 2.0, 2.0], np.float32)
    np.testing.assert_allclose(o.swiglu_ref_numpy(g, u), [0.0, 2 * np.log(3.0) * 0.75, -2 * np.log(3.0) * 0.25],
                               rtol=1e-6, atol=1e-7)
