"""The allocation-free FP32 matmul (tfb_matmul_f32_static).

Hosts that cannot call cudaMalloc at the call site (hard latency budgets, a runtime that owns all
device memory, teardown) use this variant, whose scratch is a fixed array inside the library. The
test calls it through the C-ABI twice in a row with different shapes — the second call reuses the
array the first one filled — and compares each result with the regular entry point AND with the
oracle's sequential FP32 loop on the same inputs. It checks that the calls allocate nothing (free
device memory, the library's pool and the library's scratch buffers all unchanged), that a product
beyond the array's capacity is refused rather than attempted, and that an error code recorded in this
entry point's own status word reaches tfb_device_status. It does not depend on any other test and
runs last so that a failure here cannot hide one elsewhere."""
import ctypes

import pytest
import torch

import refdata
import tensors_b200.capi as capi
from gpu_util import assert_device_ok, dev, lib, ptr, rel_err, stream_ptr

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5


def regular(A, B, M, N, K):
    C = torch.full((M, N), float("nan"), device="cuda")
    capi.check(lib.tfb_matmul(ptr(A), ptr(B), ptr(C), M, N, K, capi.DTYPE_F32, capi.DTYPE_F32, stream_ptr()))
    return C


def static(A, B, C, M, N, K):
    capi.check(lib.tfb_matmul_f32_static(ptr(A), ptr(B), ptr(C), M, N, K, stream_ptr()))


def memory_state():
    dev_idx = torch.cuda.current_device()
    torch.cuda.synchronize()
    free, _ = torch.cuda.mem_get_info()
    used, reserved = ctypes.c_uint64(0), ctypes.c_uint64(0)
    capi.check(lib.tfb_pool_stats(dev_idx, ctypes.byref(reserved), ctypes.byref(used), None, None))
    nbuf, nbytes = ctypes.c_uint64(0), ctypes.c_uint64(0)
    capi.check(lib.tfb_scratch_stats(dev_idx, ctypes.byref(nbuf), ctypes.byref(nbytes)))
    return free, used.value, reserved.value, nbuf.value, nbytes.value, torch.cuda.memory_allocated()


def test_static_scratch_matmul_two_calls_against_oracle_and_regular_entry_point(oracle):
    for (M, N, K), seed in (((256, 192, 320), 1), ((64, 256, 784), 5), ((17, 23, 19), 9)):
        a, b = refdata.uniform(seed, (M, K)), refdata.uniform(seed + 1, (K, N))
        A, B = dev(a), dev(b)
        want = regular(A, B, M, N, K)
        got = torch.full((M, N), float("nan"), device="cuda")
        static(A, B, got, M, N, K)
        assert_device_ok()
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < FP32_TOL, (M, N, K)
        assert rel_err(got.cpu().numpy(), oracle.matmul(a, b)) < FP32_TOL, (M, N, K)


def test_static_scratch_matmul_allocates_nothing():
    M, N, K = 320, 256, 512
    A, B = dev(refdata.uniform(3, (M, K))), dev(refdata.uniform(4, (K, N)))
    C = torch.empty((M, N), device="cuda")
    static(A, B, C, M, N, K)      # first call on the device: symbol look-up, kernel attributes
    before = memory_state()
    for _ in range(3):
        static(A, B, C, M, N, K)
    after = memory_state()
    assert before == after, (before, after)
    assert_device_ok()


def test_static_scratch_matmul_rejects_oversized_products():
    limit = lib.tfb_matmul_f32_static_limit()
    assert limit == 16 << 20
    t = torch.zeros(16, device="cuda")
    rc = lib.tfb_matmul_f32_static(ptr(t), ptr(t), ptr(t), 4096, 4096, 4096, stream_ptr())
    assert rc == -6
    assert "scratch" in capi.last_error()


def test_static_entry_point_errors_reach_device_status():
    # Kernels launched through the static entry point record into a status word of their own (a
    # __device__ variable). A code written there — injected from the host, no kernel is made to fail —
    # must be reported and cleared by tfb_device_status exactly like one in the regular word.
    A = dev(refdata.uniform(1, (32, 32)))
    C = torch.empty((32, 32), device="cuda")
    static(A, A, C, 32, 32, 32)
    assert_device_ok()
    for word in (1, 0):
        capi.check(lib.tfb_inject_device_status(word, 103))
        code = ctypes.c_int(0)
        assert lib.tfb_device_status(ctypes.byref(code)) == -4 and code.value == 103, word
        assert_device_ok()        # cleared by the read
