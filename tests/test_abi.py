"""The C-ABI library loads, exports every symbol include/ptxb200.h declares, and
rejects bad arguments on the host (no GPU is touched by these calls)."""
import ctypes
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_exports_every_declared_symbol(pkg):
    lib = pkg.native.lib()
    declared = pkg.native.declared_symbols()
    assert set(declared) >= {"gemm_bf16", "fa_fwd_bf16", "ptxb200_version", "ptxb200_strerror",
                             "ptxb200_sync_status", "ptxb200_selftest", "ptxb200_shutdown"}
    for name in declared:
        assert hasattr(lib, name), name
    nm = subprocess.run(["nm", "-D", "--defined-only", pkg.native.LIB_PATH], stdout=subprocess.PIPE, text=True).stdout
    exported = {l.split()[-1] for l in nm.splitlines() if " T " in l}
    assert set(declared) <= exported


def test_header_is_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "ptxb200.h"\nint main(void){return PTXB200_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src),
                    "-o", str(tmp_path / "t.o")], check=True)


def test_version_and_strerror(pkg):
    lib = pkg.native.lib()
    assert lib.ptxb200_version() >= 100
    for code in (0, -1, -2, -3, -4, -5, -6, -7, 12345):
        assert lib.ptxb200_strerror(code)
    text = lib.ptxb200_strerror(0xB2000000 - (1 << 32) | 0)  # not a positive code
    assert text
    assert b"unknown" in lib.ptxb200_strerror(0x42000B02)     # wrong tag
    timeout = lib.ptxb200_strerror(0x32000B03)                # site 11, cta 1, parity 1
    assert b"fa:softmax.s_full" in timeout and b"ran out" in timeout


def test_host_side_argument_checks(pkg):
    """Shape/alignment/null errors are reported before any CUDA call is made."""
    L = pkg.native.lib()
    n = pkg.native
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 15) & ~15
    sc = ctypes.c_float(0.125)
    assert L.gemm_bf16(None, p, p, 128, 128, 64, 128, 0, None) == n.E_INVALID
    assert L.gemm_bf16(p, p, p, 0, 128, 64, 128, 0, None) == n.E_INVALID
    assert L.gemm_bf16(p, p, p, 128, 128, 64, 128, 0x10, None) == n.E_INVALID
    assert L.gemm_bf16(p, p, p, 127, 128, 64, 128, 0, None) == n.E_SHAPE
    assert L.gemm_bf16(p, p, p, 128, 64, 64, 64, 0, None) == n.E_SHAPE
    assert L.gemm_bf16(p, p, p, 128, 128, 100, 128, 0, None) == n.E_SHAPE
    assert L.gemm_bf16(p + 8, p, p, 128, 128, 64, 128, 0, None) == n.E_ALIGN
    assert L.gemm_bf16(p, p, p, 128, 128, 64, 129, 0, None) == n.E_ALIGN     # ldc*2 not 16-B multiple
    assert L.gemm_bf16_grouped(p, p, None, 2, 128, 64, 64, 64, 0, None) == n.E_INVALID
    assert L.gemm_bf16_grouped(p, p, p, 0, 128, 64, 64, 64, 0, None) == n.E_INVALID
    assert L.gemm_bf16_grouped(p, p, p, 2, 128, 32, 64, 32, 0, None) == n.E_SHAPE
    assert L.gemm_bf16_grouped(p, p, p, 2, 64, 64, 64, 64, 0, None) == n.E_SHAPE
    assert L.gemm_bf16_grouped(p, p, p, 1 << 20, 1 << 12, 64, 64, 64, 0, None) == n.E_SHAPE
    assert L.gemm_bf16_grouped(p, p, p, 2, 128, 64, 64, 68, 0, None) == n.E_ALIGN
    assert L.fa_fwd_bf16(p, p, p, None, 1, 1, 256, 128, sc, 0, 0, None, None) == n.E_INVALID
    assert L.fa_fwd_bf16(p, p, p, p, 1, 1, 256, 128, ctypes.c_float(0.0), 0, 0, None, None) == n.E_INVALID
    assert L.fa_fwd_bf16(p, p, p, p, 1, 1, 0, 128, sc, 0, 0, None, None) == n.E_INVALID
    assert L.fa_fwd_bf16(p, p, p, p, 1, 1, 256, 32, sc, 0, 0, None, None) == n.E_SHAPE
    assert L.fa_fwd_bf16(p, p, p, p, 1 << 12, 1 << 12, 256, 128, sc, 0, 0, None, None) == n.E_SHAPE
    assert L.fa_fwd_bf16(p, p + 4, p, p, 1, 1, 256, 128, sc, 0, 0, None, None) == n.E_ALIGN
    assert L.ptxb200_selftest(9, p, p, p, p, p, p, None) == n.E_INVALID


def test_missing_library_fails_loudly(pkg, monkeypatch):
    """The product path has no fallback: without the shared library the binding raises."""
    monkeypatch.setattr(pkg.native, "_lib", None)
    monkeypatch.setattr(pkg.native, "LIB_PATH", "/nonexistent/libptxb200.so")
    import pytest
    with pytest.raises(pkg.native.PtxB200Error):
        pkg.native.lib()


def test_product_never_imports_the_oracle():
    """oracle/ is test infrastructure; nothing under the package may reference it."""
    pkg_dir = os.path.join(ROOT, "ptx.jl_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, fn
