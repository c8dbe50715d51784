"""Host-only checks of the descriptor packers against independent formulas and the
reference's known answers (double-entry rule of test/host/tcgen05_descriptors.jl:1-3:
the expected encoders below are written here, not imported from the library)."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def expected_sdesc(addr, leading, stride, layout):
    # test/host/tcgen05_descriptors.jl:33-43 (_td_expected_sdesc)
    return ((addr & 0x3FFFF) >> 4) | ((leading >> 4) & 0x3FFF) << 16 | ((stride >> 4) & 0x3FFF) << 32 | 1 << 46 | layout << 61


def expected_idesc(m, n, a_mn, b_mn):
    # test/host/tcgen05_descriptors.jl:45-57 (_td_expected_idesc), bf16 operands
    return 1 << 4 | 1 << 7 | 1 << 10 | int(a_mn) << 15 | int(b_mn) << 16 | (n >> 3) << 17 | (m >> 4) << 24


@pytest.fixture(scope="module")
def dump(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("desc") / "descriptor_dump")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "ptx.jl_b200", "csrc"),
           "-I", "/usr/local/cuda/include", os.path.join(ROOT, "tests", "host", "descriptor_dump.cpp"), "-o", exe]
    subprocess.run(cmd, check=True)
    out = subprocess.run([exe], check=True, stdout=subprocess.PIPE, text=True).stdout
    return [line.split() for line in out.strip().splitlines()]


def test_known_answer_constant(dump):
    with open(os.path.join(ROOT, "tests", "golden", "known_answers.json")) as f:
        known = json.load(f)
    got = [l for l in dump if l[0] == "sdesc_b128"][0][1]
    assert int(got, 16) == int(known["sdesc_kmajor_b128"], 16) == 0x4000404000010000


def test_sdesc_matches_independent_formula(dump):
    rows = [l for l in dump if l[0] == "sdesc"]
    assert len(rows) == 4 * 4 * 3 * 5
    for _, a, l, s, y, full, lo, hi in rows:
        a, l, s, y = int(a), int(l), int(s), int(y)
        exp = expected_sdesc(a, l, s, y)
        assert int(full, 16) == exp
        assert (int(hi, 16) << 32 | int(lo, 16)) == exp      # split form used by the kernels
        assert exp & (0x7 << 46) == 1 << 46                  # fixed 0b001
        assert exp & ((0x3 << 14) | (0x3 << 30) | (0xFF << 53)) == 0  # reserved bits stay zero


def test_idesc_matches_independent_formula(dump):
    rows = [l for l in dump if l[0] == "idesc"]
    assert len(rows) == 3 * 32 * 4
    for _, m, n, am, bm, v in rows:
        assert int(v, 16) == expected_idesc(int(m), int(n), int(am), int(bm))


def test_tmem_lane_bits(dump):
    for _, lane, v in [l for l in dump if l[0] == "tmem"]:
        assert int(v, 16) == 0x00070000 + (int(lane) << 16) + 5


def test_attention_tile_geometry(dump):
    a128 = [l for l in dump if l[0] == "attn128"][0]
    a64 = [l for l in dump if l[0] == "attn64"][0]
    assert int(a128[1], 16) == expected_idesc(128, 128, False, False)
    assert int(a128[2], 16) == expected_idesc(128, 128, False, True)     # V is the MN-major B operand
    assert int(a64[2], 16) == expected_idesc(128, 64, False, True)
    assert [int(x) for x in a128[3:]] == [32768, 8, 8]                    # FAB_TILE_BYTES, 8 k16 steps
    assert [int(x) for x in a64[3:]] == [16384, 4, 8]
