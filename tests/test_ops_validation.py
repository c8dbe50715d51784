"""ops.py rejects every mis-shaped, mis-typed or misplaced buffer with ValueError BEFORE
anything is launched (a kernel given such a buffer would write out of bounds on the
device). No GPU is needed: the checks read only shape, dtype, device and contiguity, so
stand-in objects that expose those are enough; the library call itself is replaced by a
stub that fails the test if it is ever reached."""
from dataclasses import dataclass

import pytest
import torch


@dataclass
class FakeTensor:
    shape: tuple
    dtype: torch.dtype = torch.bfloat16
    device: torch.device = torch.device("cuda", 0)
    is_cuda: bool = True
    contiguous: bool = True
    strides: tuple = None

    def __post_init__(self):
        self.shape = torch.Size(self.shape)

    def is_contiguous(self):
        return self.contiguous

    def dim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def stride(self, i):
        if self.strides is not None:
            return self.strides[i]
        st = 1
        for s in self.shape[i + 1:]:
            st *= s
        return st

    def data_ptr(self):
        raise AssertionError("a pointer was taken: validation let a bad argument through")


class _NoLaunch:
    def __getattr__(self, name):
        raise AssertionError(f"library call {name} reached with invalid arguments")


@pytest.fixture()
def ops(pkg, monkeypatch):
    monkeypatch.setattr(pkg.native, "lib", lambda: _NoLaunch())
    return pkg.ops


F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32
CUDA1 = torch.device("cuda", 1)


def test_fa_fwd_rejects_bad_buffers(ops):
    q = FakeTensor((1, 2, 256, 128))
    good = dict(q=q, k=FakeTensor((1, 2, 256, 128)), v=FakeTensor((1, 2, 256, 128)))
    bad = [
        dict(out=FakeTensor((1, 2, 256, 64))),                       # too small
        dict(out=FakeTensor((1, 2, 256, 128), dtype=F32)),           # wrong element size
        dict(out=FakeTensor((1, 2, 256, 128), device=CUDA1)),        # another GPU
        dict(out=FakeTensor((1, 2, 256, 128), contiguous=False)),
        dict(out=FakeTensor((1, 2, 256, 128), is_cuda=False, device=torch.device("cpu"))),
        dict(lse=FakeTensor((1, 2, 255), dtype=F32)),                # one row short
        dict(lse=FakeTensor((1, 2, 256), dtype=BF16)),
        dict(lse=FakeTensor((1, 2, 256), dtype=F32, device=CUDA1)),
        dict(dbg=FakeTensor((32,), dtype=I32)),                      # fewer than 64 words
        dict(dbg=FakeTensor((64,), dtype=torch.int64)),
        dict(dbg=FakeTensor((64,), dtype=I32, device=CUDA1)),
        dict(k=FakeTensor((1, 2, 256, 128), device=CUDA1), v=FakeTensor((1, 2, 256, 128), device=CUDA1)),
        dict(k=FakeTensor((1, 2, 128, 128)), v=FakeTensor((1, 2, 128, 128))),   # other sequence length
        dict(q=FakeTensor((1, 2, 256, 128), dtype=F32)),
    ]
    for extra in bad:
        with pytest.raises(ValueError):
            ops.fa_fwd(**{**good, **extra})


def test_gemm_rejects_bad_buffers(ops):
    a, bt = FakeTensor((256, 128)), FakeTensor((512, 128))
    for kw in [
        dict(out=FakeTensor((256, 512), dtype=BF16), f32_out=True),     # half the bytes the kernel writes
        dict(out=FakeTensor((256, 512), dtype=F32), f32_out=False),
        dict(out=FakeTensor((128, 512))),                               # too few rows
        dict(out=FakeTensor((256, 256))),
        dict(out=FakeTensor((256, 512), strides=(512, 2))),             # not unit column stride
        dict(out=FakeTensor((256, 512), strides=(256, 1))),             # rows overlap
        dict(out=FakeTensor((256, 512), device=CUDA1)),
        dict(out=FakeTensor((256, 512), is_cuda=False, device=torch.device("cpu"))),
    ]:
        with pytest.raises(ValueError):
            ops.gemm(a, bt, **kw)
    with pytest.raises(ValueError):
        ops.gemm(a, FakeTensor((512, 128), device=CUDA1))
    g_a, g_bt = FakeTensor((4, 128, 64)), FakeTensor((4, 64, 64))
    for kw in [dict(out=FakeTensor((4, 128, 64), dtype=F32)), dict(out=FakeTensor((4, 128, 32))),
               dict(out=FakeTensor((4, 128, 64), dtype=BF16), f32_out=True),
               dict(out=FakeTensor((4, 128, 64), device=CUDA1))]:
        with pytest.raises(ValueError):
            ops.gemm_grouped(g_a, g_bt, **kw)


def test_rowwise_ops_reject_bad_buffers(ops):
    x, w, b = FakeTensor((64, 1024), dtype=F32), FakeTensor((1024,), dtype=F32), FakeTensor((1024,), dtype=F32)
    bad_outs = [FakeTensor((64, 512), dtype=F32), FakeTensor((64, 1024), dtype=BF16),
                FakeTensor((64, 1024), dtype=F32, device=CUDA1),
                FakeTensor((64, 1024), dtype=F32, contiguous=False),
                FakeTensor((64, 1024), dtype=F32, is_cuda=False, device=torch.device("cpu"))]
    for out in bad_outs:
        with pytest.raises(ValueError):
            ops.softmax(x, out=out)
        with pytest.raises(ValueError):
            ops.rms_norm(x, w, out=out)
        with pytest.raises(ValueError):
            ops.layer_norm(x, w, b, out=out)
        with pytest.raises(ValueError):
            ops.swiglu(x, FakeTensor((64, 1024), dtype=F32), out=out)
    with pytest.raises(ValueError):
        ops.rms_norm(x, FakeTensor((1024,), dtype=F32, device=CUDA1))
    with pytest.raises(ValueError):
        ops.layer_norm(x, w, FakeTensor((512,), dtype=F32))


def test_stream_of_another_device_is_rejected(ops):
    class FakeStream:
        device = CUDA1
        cuda_stream = 0
    q = FakeTensor((1, 1, 128, 64))
    with pytest.raises(ValueError):
        ops.fa_fwd(q, FakeTensor((1, 1, 128, 64)), FakeTensor((1, 1, 128, 64)), stream=FakeStream())
    with pytest.raises(ValueError):
        ops.softmax(FakeTensor((8, 64), dtype=F32), stream=FakeStream())
