"""fa_fwd_bf16 parity against the CPU oracle, through the C ABI.

The small shapes and input scales are the reference's own runtime cases
(test/gpu/blackwell/flash_attention.jl:202-221: (1,1,256), (1,2,512), (2,4,1024)
with input scale 0.5 for Q,K and 1 for V, plus the rescale-heavy scale 2.0 case;
causal and D = 64 cases follow test/gpu/ampere/flash_attention.jl:350-360).
Tolerance: max abs <= 2e-2 and mean abs <= 2e-3 against the fp32 oracle.
"""
import numpy as np
import pytest
import torch

from util import ATTN_MAX_ABS, ATTN_MEAN_ABS, attn_errors, bits, seeded_qkv

pytestmark = pytest.mark.gpu


def _run(pkg, gpu, oracle_mod, B, H, S, D, causal, sigma_qk, sigma_v=1.0, flags=0, seed=None):
    seed = seed if seed is not None else B * 7919 + H * 131 + S
    q, k, v = seeded_qkv(B, H, S, D, seed, sigma_qk, sigma_v)
    o = pkg.ops.fa_fwd(q.to(gpu), k.to(gpu), v.to(gpu), causal=causal, flags=flags)
    status = pkg.ops.sync_status()
    assert status == 0, pkg.native.strerror(status)
    ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(k).reshape(B * H, S, D),
                                     bits(v).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
    return attn_errors(o, ref)


@pytest.mark.parametrize("B,H,S", [(1, 1, 256), (1, 2, 512), (2, 4, 1024)])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
def test_reference_shapes(pkg, gpu, oracle_mod, B, H, S, D, causal):
    mx, mean = _run(pkg, gpu, oracle_mod, B, H, S, D, causal, sigma_qk=0.5)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("flags", [0, 1])
def test_rescale_heavy(pkg, gpu, oracle_mod, D, causal, flags):
    """Input scale 2.0 makes row maxima move by far more than 2^8 between tiles, so
    the O-rescale path runs (flash_attention.jl:210-221); flags=1 rescales on every
    increase of the maximum."""
    mx, mean = _run(pkg, gpu, oracle_mod, 1, 2, 512, D, causal, sigma_qk=2.0, flags=flags)
    assert mx <= 5e-2 and mean <= 4e-3, (mx, mean)   # the reference's gate for this input


@pytest.mark.parametrize("D,causal", [(128, False), (128, True), (64, False), (64, True)])
def test_many_items_per_cta(pkg, gpu, oracle_mod, D, causal):
    """More work items than SMs: every role walks its persistent loop several times
    (phase bookkeeping across items), including the causal longest-first order."""
    mx, mean = _run(pkg, gpu, oracle_mod, 2, 40, 768, D, causal, sigma_qk=1.0)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("S", [128, 256, 300])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
def test_many_short_items_per_cta(pkg, gpu, oracle_mod, S, D, causal):
    """A dozen one- and two-tile items per CTA: the per-item hand-overs (Q buffers, row
    sums, O accumulators) turn over as fast as they can, with a stage free to start the
    next item while the other and the correction warps still finish this one."""
    mx, mean = _run(pkg, gpu, oracle_mod, 8, 222, S, D, causal, sigma_qk=1.0)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("S", [128, 384, 640])
@pytest.mark.parametrize("D,causal", [(128, False), (128, True), (64, True)])
def test_odd_number_of_128_row_blocks(pkg, gpu, oracle_mod, S, D, causal):
    """S a multiple of 128 but not of 256 (the reference asserts these away,
    bench/flash_attention.jl:43-47): the last work item of every head has only its
    first stage, whose second stage lies over the next head's first rows: a stray
    write there would corrupt that head's output and show up here."""
    B, H = 2, 3
    q, k, v = seeded_qkv(B, H, S, D, 900 + S, 1.0)
    o = torch.full((B, H, S, D), 7.0, dtype=torch.bfloat16, device=gpu)
    pkg.ops.fa_fwd(q.to(gpu), k.to(gpu), v.to(gpu), causal=causal, out=o)
    assert pkg.ops.sync_status() == 0
    ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(k).reshape(B * H, S, D),
                                     bits(v).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
    mx, mean = attn_errors(o, ref)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)


def test_cpu_runnable_config_shape(pkg, gpu, oracle_mod):
    """B=1 H=4 S=256 D=64 non-causal, N(0,1) inputs: the configuration sized for a CPU run."""
    mx, mean = _run(pkg, gpu, oracle_mod, 1, 4, 256, 64, False, sigma_qk=1.0, seed=20260001)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)


def test_large_logits_do_not_overflow(pkg, gpu, oracle_mod):
    """Scores of several hundred: a softmax that exponentiated the first tile
    without subtracting its maximum would overflow; this one must not."""
    mx, mean = _run(pkg, gpu, oracle_mod, 1, 1, 512, 128, False, sigma_qk=6.0)
    assert np.isfinite(mx) and mx <= 5e-2, (mx, mean)


@pytest.mark.parametrize("causal", [False, True])
def test_full_size_properties(pkg, gpu, causal):
    """Size-independent properties at a headline-sized slice (S = 4096, D = 128):
    with V = all ones every output is exactly 1 (rows of P sum to 1); with one-hot
    structure in V the output rows are convex combinations, so 0 <= O <= 1; and a
    second launch on the same inputs is bit-identical (no race)."""
    B, H, S, D = 1, 8, 4096, 128
    q, k, _ = seeded_qkv(B, H, S, D, 99, 1.0)
    q, k = q.to(gpu), k.to(gpu)
    ones = torch.ones(B, H, S, D, dtype=torch.bfloat16, device=gpu)
    o = pkg.ops.fa_fwd(q, k, ones, causal=causal)
    assert pkg.ops.sync_status() == 0
    assert torch.allclose(o.float(), torch.ones_like(o, dtype=torch.float32), atol=2 ** -7)
    v = (torch.rand(B, H, S, D, device=gpu) < 0.5).to(torch.bfloat16)
    o1 = pkg.ops.fa_fwd(q, k, v, causal=causal)
    o2 = pkg.ops.fa_fwd(q, k, v, causal=causal)
    assert pkg.ops.sync_status() == 0
    assert torch.equal(o1, o2)
    assert float(o1.float().min()) >= 0.0 and float(o1.float().max()) <= 1.0 + 2 ** -7
    if causal:
        # the first query row attends to key 0 only
        assert torch.equal(o1[:, :, 0, :], v[:, :, 0, :])


@pytest.mark.parametrize("S", [1, 7, 100, 127, 129, 200, 255, 257, 1000, 2049])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
def test_any_sequence_length(pkg, gpu, oracle_mod, S, D, causal):
    """Sequence lengths that are no multiple of the 128-row tile (the reference asserts
    S % 256 == 0): rows and keys past the end load as zeros through the per-head tensor
    maps; the keys are masked out of the softmax, the rows are not written. The output
    buffer is longer than needed and pre-filled, so a write past the end would show."""
    B, H = 2, 3
    q, k, v = seeded_qkv(B, H, S, D, 900 + S, 0.8)
    out = torch.full((B * H * S * D + 4096,), 7.0, dtype=torch.bfloat16, device=gpu)
    o = out[:B * H * S * D].view(B, H, S, D)
    lse = torch.full((B * H * S + 64,), 7.0, dtype=torch.float32, device=gpu)
    pkg.ops.fa_fwd(q.to(gpu), k.to(gpu), v.to(gpu), causal=causal, out=o, lse=lse[:B * H * S])
    assert pkg.ops.sync_status() == 0
    assert torch.all(out[B * H * S * D:] == 7.0) and torch.all(lse[B * H * S:] == 7.0)
    ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(k).reshape(B * H, S, D),
                                     bits(v).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
    mx, mean = attn_errors(o, ref)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)
    qf, kf = q.float().numpy().reshape(B * H, S, D), k.float().numpy().reshape(B * H, S, D)
    got_lse = lse[:B * H * S].cpu().numpy().reshape(B * H, S)
    for i in range(B * H):
        np.testing.assert_allclose(got_lse[i], oracle_mod.attention_lse_numpy(qf[i], kf[i], 1.0 / D ** 0.5, causal),
                                   atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("B,H,S,D", [
    (4, 16, 4096, 128),    # 512 pairs of 16 blocks per head on 148 CTAs
    (16, 16, 1280, 128),   # 5 blocks per head: the middle one has no partner
    (8, 32, 2304, 64),     # 9 blocks per head, D = 64
    (2, 2, 1024, 128),     # fewer pairs than CTAs
    (1, 3, 384, 64),       # S % 256 == 128: the last block has only its first stage
])
def test_causal_schedules_agree_bit_for_bit(pkg, gpu, B, H, S, D):
    """Causal work is handed out either as equal-length pairs of blocks of one head
    or as single blocks, longest first (the host picks by the longest CTA; the flag
    forces single blocks). Which CTA computes a block changes nothing in the block's
    arithmetic, so the outputs must be identical."""
    q, k, v = (t.to(gpu) for t in seeded_qkv(B, H, S, D, 4242 + S, 0.7))
    lse_a = torch.empty(B * H * S, dtype=torch.float32, device=gpu)
    lse_b = torch.empty_like(lse_a)
    # (the last round is left uncut in both: a cut changes the key order of the rows it touches)
    keep = pkg.native.FA_NO_TAIL_SPLIT
    a = pkg.ops.fa_fwd(q, k, v, causal=True, lse=lse_a, flags=keep)
    b = pkg.ops.fa_fwd(q, k, v, causal=True, lse=lse_b, flags=keep | pkg.native.FA_SINGLE_BLOCKS)
    assert pkg.ops.sync_status() == 0
    assert torch.equal(a, b) and torch.equal(lse_a, lse_b)


@pytest.mark.parametrize("name,B,H,S,D,causal,sigma", [
    ("c2", 4, 16, 4096, 128, False, 1.0),
    ("c3", 16, 16, 2048, 64, False, 1.0),
    ("c4", 8, 32, 8192, 128, True, 0.5),
])
def test_full_size_configs_against_oracle_slices(pkg, gpu, oracle_mod, name, B, H, S, D, causal, sigma):
    """The three full-size attention configurations, whole on the device, checked on
    sampled (batch, head) slices: two against the C oracle, eight against an unfused
    fp32 computation on the GPU (same bf16-quantised inputs, the oracle's formula)."""
    g = torch.Generator(device=gpu).manual_seed(len(name) * 1000 + S)
    q = (torch.randn(B, H, S, D, device=gpu, generator=g) * sigma).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, device=gpu, generator=g) * sigma).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, device=gpu, generator=g).to(torch.bfloat16)
    o = pkg.ops.fa_fwd(q, k, v, causal=causal)
    assert pkg.ops.sync_status() == 0
    scale = 1.0 / D ** 0.5
    slices = [(0, 0), (B - 1, H - 1), (B // 2, 1), (1 % B, H // 2), (B - 1, 0), (0, H - 1), (B // 3, H // 3),
              ((2 * B) // 3, (2 * H) // 3)]
    for i, (b, h) in enumerate(slices):
        qf, kf, vf = q[b, h].float(), k[b, h].float(), v[b, h].float()
        sc = (qf @ kf.t()) * scale
        if causal:
            sc = sc.masked_fill(torch.ones(S, S, dtype=torch.bool, device=gpu).triu(1), float("-inf"))
        ref = torch.softmax(sc, dim=1) @ vf
        err = (o[b, h].float() - ref).abs()
        assert float(err.max()) <= ATTN_MAX_ABS and float(err.mean()) <= ATTN_MEAN_ABS, (name, b, h, float(err.max()))
        if i < 2:
            ref_c = oracle_mod.attention_ref_c(bits(q[b, h]).reshape(1, S, D), bits(k[b, h]).reshape(1, S, D),
                                               bits(v[b, h]).reshape(1, S, D), scale, causal)
            mx, mean = attn_errors(o[b, h], ref_c)
            assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (name, b, h, mx, mean)


@pytest.mark.parametrize("D,causal,H,H_kv", [(128, False, 8, 2), (128, True, 6, 3), (64, False, 4, 1), (64, True, 8, 8)])
def test_grouped_heads_and_lse(pkg, gpu, oracle_mod, D, causal, H, H_kv):
    """fa_fwd_bf16_ex: query head h attends to key/value head h / (H / H_kv), and the
    per-row log-sum-exp comes out next to O. O is checked against the oracle on K/V
    repeated per group; LSE against float64 (tolerance: fp32 statistics of bf16 data)."""
    B, S = 2, 512
    g = torch.Generator().manual_seed(4100 + D + H)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    lse = torch.full((B, H, S), float("nan"), dtype=torch.float32, device=gpu)
    o = pkg.ops.fa_fwd(q.to(gpu), k.to(gpu), v.to(gpu), causal=causal, lse=lse)
    assert pkg.ops.sync_status() == 0
    ke = k.repeat_interleave(H // H_kv, dim=1)
    ve = v.repeat_interleave(H // H_kv, dim=1)
    ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(ke).reshape(B * H, S, D),
                                     bits(ve).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
    mx, mean = attn_errors(o, ref)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)
    got = lse.cpu().numpy().reshape(B * H, S)
    qf, kf = q.float().numpy().reshape(B * H, S, D), ke.float().numpy().reshape(B * H, S, D)
    for i in (0, B * H // 2, B * H - 1):
        want = oracle_mod.attention_lse_numpy(qf[i], kf[i], 1.0 / D ** 0.5, causal)
        np.testing.assert_allclose(got[i], want, rtol=0, atol=2e-3)
    L = pkg.native.lib()
    P = o.data_ptr()
    import ctypes
    assert L.fa_fwd_bf16_ex(P, None, P, P, P, 1, 6, 4, 256, 128, ctypes.c_float(0.1), 0, 0, None, None) == pkg.native.E_SHAPE


def _random_shapes(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        D = int(rng.choice([64, 128]))
        causal = bool(rng.integers(0, 2))
        S = int(rng.integers(1, 1400))
        H_kv = int(rng.integers(1, 5))
        H = H_kv * int(rng.integers(1, 4))
        # enough (batch, head) slices that most CTAs walk several items of different length
        B = max(1, int(rng.integers(150, 700)) // (H * max(1, (S + 255) // 256)))
        out.append((B, H, H_kv, S, D, causal, 7000 + i))
    return out


@pytest.mark.parametrize("B,H,H_kv,S,D,causal,seed", _random_shapes(16, 20260025))
def test_seeded_random_shapes(pkg, gpu, oracle_mod, B, H, H_kv, S, D, causal, seed):
    """Shapes drawn from a seeded generator: any sequence length, grouped heads, both head
    dims, causal or not, with the log-sum-exp output; O against the oracle, and the
    default schedule bit for bit against single blocks for the causal ones."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    qd, kd, vd = q.to(gpu), k.to(gpu), v.to(gpu)
    lse = torch.full((B, H, S), float("nan"), dtype=torch.float32, device=gpu)
    o = pkg.ops.fa_fwd(qd, kd, vd, causal=causal, lse=lse)
    status = pkg.ops.sync_status()
    assert status == 0, pkg.native.strerror(status)
    assert not torch.isnan(lse).any()
    ke = k.repeat_interleave(H // H_kv, dim=1)
    ve = v.repeat_interleave(H // H_kv, dim=1)
    ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(ke).reshape(B * H, S, D),
                                     bits(ve).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
    mx, mean = attn_errors(o, ref)
    assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)
    # with the last round left uncut the result is the same up to the re-association of the
    # cut rows' sums, and the two causal schedules then agree bit for bit
    keep = pkg.native.FA_NO_TAIL_SPLIT
    o1 = pkg.ops.fa_fwd(qd, kd, vd, causal=causal, flags=keep)
    assert pkg.ops.sync_status() == 0
    assert (o.float() - o1.float()).abs().max().item() <= 2 ** -6
    if causal:
        o2 = pkg.ops.fa_fwd(qd, kd, vd, causal=True, flags=keep | pkg.native.FA_SINGLE_BLOCKS)
        assert pkg.ops.sync_status() == 0
        assert torch.equal(o1, o2)


def test_rejects_bad_arguments(pkg, gpu):
    L = pkg.native.lib()
    t = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16, device=gpu)
    P = t.data_ptr()
    import ctypes
    sc = ctypes.c_float(0.1)
    assert L.fa_fwd_bf16(P, P, P, P, 1, 1, 0, 128, sc, 0, 0, None, None) == pkg.native.E_INVALID
    assert L.fa_fwd_bf16(P, P, P, P, 1, 1, 256, 96, sc, 0, 0, None, None) == pkg.native.E_SHAPE
    assert L.fa_fwd_bf16(None, P, P, P, 1, 1, 256, 128, sc, 0, 0, None, None) == pkg.native.E_INVALID
    assert L.fa_fwd_bf16(P, P + 2, P, P, 1, 1, 256, 128, sc, 0, 0, None, None) == pkg.native.E_ALIGN
    assert L.fa_fwd_bf16(P, P, P, P, 1, 1, 256, 128, sc, 2, 0, None, None) == pkg.native.E_INVALID
    assert L.fa_fwd_bf16(P, P, P, P, 1, 1, 256, 128, sc, 0, 0x80, None, None) == pkg.native.E_INVALID


# ---------------------------------------------------------------------------
# The last round cut along the key axis (no reference counterpart: the reference deals whole
# items, test/gpu/blackwell/flash_attention_defs.jl:269-272). Shapes whose item count leaves
# the last round partly filled on this GPU; each is checked against the oracle, against the
# uncut launch, and for reproducibility from launch to launch.
# ---------------------------------------------------------------------------
def _plan_header(pkg, B, H, S, causal, flags=0):
    import ctypes
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    cap = 16 + sm * 49
    buf = (ctypes.c_int * cap)()
    n = pkg.native.lib().ptxb200_fa_plan(B, H, S, int(causal), flags, sm, buf, cap)
    assert n >= 10
    return dict(zip(["nmb", "bh", "nt_all", "causal", "pair", "grid", "full", "tail_units", "tail_steps",
                     "tail_ctas"], list(buf)[:10]))


@pytest.mark.parametrize("B,H,H_kv,S,D,causal", [
    (1, 8, 8, 4096, 128, False),    # an eighth of the headline problem: 128 items for 148 SMs
    (2, 16, 16, 2048, 64, False),   # an eighth of the short-sequence configuration (D = 64)
    (1, 4, 4, 8192, 128, True),     # causal pairs of 66 steps, fewer than SMs
    (1, 5, 5, 8192, 64, True),
    (3, 4, 2, 1000, 128, False),    # ragged length, grouped heads
    (1, 7, 7, 1000, 64, True),
    (1, 1, 1, 4096, 128, False),    # one head: every item in many pieces
    (1, 2, 1, 2304, 128, True),     # odd block count: a middle block without partner
    (5, 8, 8, 1536, 128, False),    # a full round, then a cut one
    (3, 30, 30, 1280, 64, True),    # five blocks per head, a full round first
    (2, 45, 45, 1024, 64, True),    # fewer CTAs share the cut round than run the launch
])
def test_cut_last_round_matches_oracle_and_uncut_launch(pkg, gpu, oracle_mod, B, H, H_kv, S, D, causal):
    cut = pkg.native.FA_ALWAYS_TAIL_SPLIT     # (the default policy cuts only where it expects a clear gain)
    assert _plan_header(pkg, B, H, S, causal, cut)["tail_units"] > 0, "this shape is meant to exercise the cut"
    g = torch.Generator().manual_seed(B * 1000 + H * 10 + S)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H_kv, S, D, generator=g).to(torch.bfloat16)
    qd, kd, vd = q.to(gpu), k.to(gpu), v.to(gpu)
    lse = torch.full((B, H, S), float("nan"), dtype=torch.float32, device=gpu)
    lse_u = torch.empty_like(lse)
    o = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device=gpu)
    pkg.ops.fa_fwd(qd, kd, vd, causal=causal, lse=lse, out=o, flags=cut)
    o_again = pkg.ops.fa_fwd(qd, kd, vd, causal=causal, flags=cut)        # same scratch, next epoch
    o_uncut = pkg.ops.fa_fwd(qd, kd, vd, causal=causal, lse=lse_u, flags=pkg.native.FA_NO_TAIL_SPLIT)
    status = pkg.ops.sync_status()
    assert status == 0, pkg.native.strerror(status)
    assert not torch.isnan(o.float()).any() and not torch.isnan(lse).any()
    assert torch.equal(o, o_again)
    # the merge re-associates fp32 sums before the one rounding to bf16: at most a bf16 ulp apart
    assert (o.float() - o_uncut.float()).abs().max().item() <= 2 ** -6
    torch.testing.assert_close(lse, lse_u, rtol=0, atol=2e-5 * max(1.0, float(lse_u.abs().max())))
    if B * H * S * S <= 5e8:
        ke = k.repeat_interleave(H // H_kv, dim=1)
        ve = v.repeat_interleave(H // H_kv, dim=1)
        ref = oracle_mod.attention_ref_c(bits(q).reshape(B * H, S, D), bits(ke).reshape(B * H, S, D),
                                         bits(ve).reshape(B * H, S, D), 1.0 / D ** 0.5, causal)
        mx, mean = attn_errors(o, ref)
        assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (mx, mean)
    else:
        # too large for the oracle in test time: a few heads of it
        for bh in (0, B * H - 1):
            b_, h_ = divmod(bh, H)
            hk = h_ // (H // H_kv)
            ref = oracle_mod.attention_ref_c(bits(q[b_, h_])[None], bits(k[b_, hk])[None], bits(v[b_, hk])[None],
                                             1.0 / D ** 0.5, causal)
            mx, mean = attn_errors(o[b_, h_], ref)
            assert mx <= ATTN_MAX_ABS and mean <= ATTN_MEAN_ABS, (bh, mx, mean)


def test_cut_last_round_on_two_streams(pkg, gpu):
    """Scratch for the parked pieces is per stream: launches that overlap on two streams
    stay correct and reproducible."""
    B, H, S, D = 1, 8, 2048, 128
    cut = pkg.native.FA_ALWAYS_TAIL_SPLIT
    assert _plan_header(pkg, B, H, S, False, cut)["tail_units"] > 0
    sets = [[t.to(gpu) for t in seeded_qkv(B, H, S, D, 70 + i, 1.0)] for i in range(2)]
    want = [pkg.ops.fa_fwd(*s, flags=cut) for s in sets]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.empty_like(w) for w in want]
    for _ in range(20):
        for st, s, o in zip(streams, sets, outs):
            pkg.ops.fa_fwd(*s, out=o, stream=st, flags=cut)
    torch.cuda.synchronize()
    assert pkg.ops.sync_status() == 0
    for o, w in zip(outs, want):
        assert torch.equal(o, w)

