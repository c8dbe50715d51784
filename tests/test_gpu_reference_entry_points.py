"""The host-side mirrors of the reference's own drivers, run the way the reference runs
them: fab_setup / fab_check / fab_time / fab_sweep / fab_hang_debug
(bench/flash_attention.jl:41-179) and _run_ghb / _run_ggb
(test/gpu/blackwell/gemm_highperf_blackwell.jl:230-277, grouped_gemm.jl:208-244), each
with the CPU oracle handed in as the checker."""
import numpy as np
import pytest
import torch

from util import bits

pytestmark = pytest.mark.gpu


def _checker(oracle_mod):
    def ref(Q, K, V, sm_scale, causal):
        S, D = Q.shape
        q, k, v = (bits(t.to(torch.bfloat16)).reshape(1, S, D) for t in (Q, K, V))
        return torch.from_numpy(oracle_mod.attention_ref_c(q, k, v, sm_scale, causal)[0])
    return ref


@pytest.mark.parametrize("cfg", [{}, {"causal": True}, {"head_dim": 64}, {"head_dim": 64, "causal": True}])
def test_fab_check_passes_the_reference_gate(pkg, gpu, oracle_mod, cfg, capsys):
    fa = pkg.flash_attention
    # the reference's gate: rescale-heavy input scale 2.0, max abs diff < 5e-2 (:89-105)
    assert fa.fab_check(_checker(oracle_mod), cfg, B=1, H=2, S=512, input_scale=2.0, atol=5e-2)
    assert "OK" in capsys.readouterr().out


def test_fab_setup_keeps_the_reference_contract(pkg, gpu):
    fa = pkg.flash_attention
    p = fa.fab_setup(2, 4, 1024)
    assert (p.B, p.H, p.S, p.D, p.causal) == (2, 4, 1024, 128, False)
    assert p.Q.shape == (2 * 4 * 1024, 128) and p.O_d.dtype == torch.bfloat16
    assert abs(p.sm_scale - 128 ** -0.5) < 1e-7
    assert p.num_ctas == min(2 * 4 * 4, torch.cuda.get_device_properties(gpu).multi_processor_count)
    with pytest.raises(ValueError):
        fa.fab_setup(1, 1, 384)          # the reference asserts S % 256 == 0 (:43)
    p.launch()
    assert pkg.ops.sync_status() == 0


def test_fab_time_and_sweep_and_hang_debug(pkg, gpu, oracle_mod, capsys):
    fa = pkg.flash_attention
    r = fa.fab_time(B=1, H=16, S=2048, iters=5, warmup=2, warm_ms=5.0)
    assert r["ms"] > 0 and r["tflops"] > 100 and r["ctas"] == 128
    fa.fab_sweep(_checker(oracle_mod), shapes=((1, 4, 1024), (1, 2, 2048)))
    out = capsys.readouterr().out
    assert "B=1 H=4 S=1024" in out and "TF" in out
    status, counters = fa.fab_hang_debug()
    assert status == 0
    assert counters[0] == counters[1] > 0          # K/V tiles loaded == consumed by CTA 0
    assert "no timeouts" in capsys.readouterr().out


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 256)])
def test_run_ghb_reference_cases(pkg, gpu, oracle_mod, M, N, K):
    """The reference's three GEMM cases under its own tolerance (isapprox rtol = atol = 5e-2)."""
    got, A, B = pkg.gemm_highperf.run_ghb(M, N, K)
    ref = oracle_mod.gemm_ref_numpy(A.numpy(), B.numpy())
    np.testing.assert_allclose(got.numpy(), ref, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("G,M,N,K", [(1, 128, 64, 64), (2, 128, 64, 64), (4, 128, 64, 128)])
def test_run_ggb_reference_cases(pkg, gpu, oracle_mod, G, M, N, K):
    got, A3, B3 = pkg.gemm_highperf.run_ggb(G, M, N, K)
    for g in range(G):
        ref = oracle_mod.gemm_ref_numpy(A3[g].numpy(), B3[g].numpy())
        np.testing.assert_allclose(got[g].numpy(), ref, rtol=5e-2, atol=5e-2)
