"""The allocation-free mean pool (cubk_mean_pool_static_scratch) against the ordinary entry point.

Who needs it: hosts that may not call cudaMalloc on the path that runs the model -- a serving loop
that bans calls able to block on the driver's allocation lock, a plug-in inside a process that owns
all device memory, a sandbox that filters allocator calls. The variant keeps the split-sequence
partial sums in an array that is part of the library image, so the test drives it with nothing but
the caller's input and output buffers.

Collected last on purpose (file name), so that a run stopping at the first failure has already run
every other test; it must pass alone in a fresh process as well as after the others.
"""
import pytest
import torch

from cubert_b200 import kernels

pytestmark = pytest.mark.gpu


def _both(x, elem_bytes):
    """(static-scratch result, ordinary result) for a device tensor x [B, S, H]."""
    lib = kernels.load()
    b, s, h = x.shape
    stream = torch.cuda.current_stream().cuda_stream
    out_static = torch.full((b, h), float("nan"), dtype=x.dtype, device="cuda")
    out_plain = torch.full((b, h), float("nan"), dtype=x.dtype, device="cuda")
    kernels.check(lib.cubk_mean_pool_static_scratch(x.data_ptr(), elem_bytes, b, s, h, out_static.data_ptr(), stream))
    need = lib.cubk_mean_pool_scratch_bytes(b, s, h)
    scratch = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    fn = lib.cubk_mean_pool_f32 if elem_bytes == 4 else lib.cubk_mean_pool_f16
    kernels.check(fn(x.data_ptr(), b, s, h, out_plain.data_ptr(), scratch.data_ptr(), need, stream))
    torch.cuda.synchronize()
    return out_static, out_plain


@pytest.mark.parametrize("dtype,elem_bytes", [(torch.float32, 4), (torch.float16, 2)])
def test_static_scratch_matches_the_ordinary_entry_point_twice_in_a_row(dtype, elem_bytes):
    lib = kernels.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    # two calls in a row on different data and shapes: the second must not see the first one's partial sums
    shapes = [(2, 512, 1024), (3, 256, 768)]
    for (b, s, h) in shapes:
        assert 0 < lib.cubk_mean_pool_scratch_bytes(b, s, h) <= kernels.STATIC_POOL_SCRATCH_BYTES  # split path runs
        x = (torch.randn((b, s, h), device="cuda", generator=g) * 3 + 1).to(dtype)
        got, want = _both(x, elem_bytes)
        assert torch.equal(got, want)  # same kernels, same order of additions: identical bits
        ref = x.float().mean(dim=1)
        tol = 1e-5 if dtype == torch.float32 else 1e-3  # the bars of tests/test_kernels_gpu.py
        assert torch.all((got.float() - ref).abs() <= tol * torch.clamp(ref.abs(), min=0.1))
    # a shape that needs no partial sums at all goes through as well
    x = torch.randn((512, 16, 256), device="cuda", generator=g).to(dtype)
    got, want = _both(x, elem_bytes)
    assert torch.equal(got, want)


def test_static_scratch_rejects_what_does_not_fit():
    lib = kernels.load()
    stream = torch.cuda.current_stream().cuda_stream
    b, s, h = 9, 512, 4096     # binary16: 9 sequences x 5 slices x 4096 float32 sums = 720 KiB > 512 KiB
    assert lib.cubk_mean_pool_scratch_bytes(b, s, h) > kernels.STATIC_POOL_SCRATCH_BYTES
    x = torch.zeros(16, device="cuda")  # never touched: the call must refuse before launching
    rc = lib.cubk_mean_pool_static_scratch(x.data_ptr(), 2, b, s, h, x.data_ptr(), stream)
    assert rc == kernels.CUBK_ERR_SCRATCH
    assert lib.cubk_mean_pool_static_scratch(x.data_ptr(), 3, 2, 64, 64, x.data_ptr(), stream) == kernels.CUBK_ERR_INVALID_ARG
    torch.cuda.synchronize()
