"""The allocation-free FP32 matmul (tfb_matmul_f32_static) against the regular entry point.

Hosts that cannot call cudaMalloc at the call site (hard latency budgets, a runtime that owns all
device memory, teardown) use this variant, whose scratch is a fixed array inside the library. The
test calls it through the C-ABI twice in a row with different shapes — the second call reuses the
array the first one filled — and compares each result with tfb_matmul on the same inputs. It also
checks that a product beyond the array's capacity is refused rather than attempted. It does not
depend on any other test and runs last so that a failure here cannot hide one elsewhere."""
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from gpu_util import assert_device_ok, dev, lib, ptr, rel_err, stream_ptr

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5


def both(M, N, K, seed):
    A, B = dev(refdata.uniform(seed, (M, K))), dev(refdata.uniform(seed + 1, (K, N)))
    want = torch.full((M, N), float("nan"), device="cuda")
    got = torch.full((M, N), float("nan"), device="cuda")
    capi.check(lib.tfb_matmul(ptr(A), ptr(B), ptr(want), M, N, K, capi.DTYPE_F32, capi.DTYPE_F32, stream_ptr()))
    capi.check(lib.tfb_matmul_f32_static(ptr(A), ptr(B), ptr(got), M, N, K, stream_ptr()))
    assert_device_ok()
    return got.cpu().numpy(), want.cpu().numpy()


def test_static_scratch_matmul_matches_regular_entry_point_twice():
    for shape, seed in (((256, 192, 320), 1), ((64, 256, 784), 5), ((17, 23, 19), 9)):
        got, want = both(*shape, seed)
        assert rel_err(got, want) < FP32_TOL, shape


def test_static_scratch_matmul_rejects_oversized_products():
    limit = lib.tfb_matmul_f32_static_limit()
    assert limit == 16 << 20
    t = torch.zeros(16, device="cuda")
    rc = lib.tfb_matmul_f32_static(ptr(t), ptr(t), ptr(t), 4096, 4096, 4096, stream_ptr())
    assert rc == -6
    assert "scratch" in capi.last_error()
