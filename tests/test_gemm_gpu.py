"""Parity of the tcgen05 GEMM (through the C-ABI) with the oracle: bit patterns of the reference's
own kernel tests, seeded cases in every operand layout, the BF16 path, fused epilogues, and the
full-size configurations through sampled rows/columns plus size-independent properties."""
import ctypes

import numpy as np
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from gpu_util import assert_device_ok, dev, gemm_ex, lib, ptr, rel_err, stream_ptr

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5   # normwise, against the reference FP32 matmul
BF16_TOL = 1e-2


@pytest.fixture(autouse=True, params=["small_products_on_cuda_cores", "tensor_cores_only"])
def product_path(request):
    """FP32 products with few rows and a long contraction run on the one-launch CUDA-core kernel by default;
    the tests run a second time with that knob off, so that the tensor-core path keeps seeing those shapes.
    Tests that only hold large products are not repeated."""
    large_only = ("test_square_sweep", "test_config1", "test_matmul_on_host_buffers", "test_few_rows_long_contraction")
    if request.param == "tensor_cores_only" and request.node.name.startswith(large_only):
        pytest.skip("large products take the tensor-core path either way")
    old = ctypes.c_int(0)
    capi.check(lib.tfb_get_tuning(capi.TUNE_SMALL_GEMM, ctypes.byref(old)))
    capi.check(lib.tfb_set_tuning(capi.TUNE_SMALL_GEMM, 1 if request.param == "small_products_on_cuda_cores" else 0))
    yield request.param
    capi.check(lib.tfb_set_tuning(capi.TUNE_SMALL_GEMM, old.value))


def tfb_matmul(a, b, in_dtype=capi.DTYPE_F32, out_dtype=capi.DTYPE_F32):
    M, K = a.shape
    N = b.shape[1]
    td = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}
    A, B = dev(a, td[in_dtype]), dev(b, td[in_dtype])
    C = torch.full((M, N), float("nan"), device="cuda", dtype=td[out_dtype])
    capi.check(lib.tfb_matmul(ptr(A), ptr(B), ptr(C), M, N, K, in_dtype, out_dtype, stream_ptr()))
    assert_device_ok()
    return C.float().cpu().numpy()


def test_reference_kernel_test_patterns(oracle, golden):
    # The cases of cuda/kernels/gemm_{naive,tiled_16x16,optimized}_test.cpp, against the golden
    # outputs of the reference's Tensor::matmul, with the tolerances those tests use or tighter.
    for name, a, b in refdata.gemm_test_patterns():
        got = tfb_matmul(a, b)
        want = golden[f"gemm_{name}"]
        assert not np.isnan(got).any(), name
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6, err_msg=name)
    got = tfb_matmul(np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6], [7, 8]], np.float32))
    assert got.tolist() == [[19.0, 22.0], [43.0, 50.0]]


def test_launcher_semantics_same_dtype_and_noop():
    # launch_gemm_* keep the input dtype for C and silently ignore empty problems and unknown dtypes
    # (cuda/kernels/gemm.cu:81,298).
    for dt, tdt, eps in ((capi.DTYPE_F16, torch.float16, 0.05), (capi.DTYPE_BF16, torch.bfloat16, 0.1)):
        A = dev(np.array([[1, 2], [3, 4]], np.float32), tdt)
        B = dev(np.array([[5, 6], [7, 8]], np.float32), tdt)
        C = torch.zeros((2, 2), device="cuda", dtype=tdt)
        capi.check(lib.tfb_gemm(ptr(A), ptr(B), ptr(C), 2, 2, 2, dt, stream_ptr()))
        assert_device_ok()
        np.testing.assert_allclose(C.float().cpu().numpy(), [[19, 22], [43, 50]], rtol=eps)
    C = torch.full((2, 2), 7.0, device="cuda")
    assert lib.tfb_gemm(ptr(C), ptr(C), ptr(C), 0, 2, 2, capi.DTYPE_F32, stream_ptr()) == 0
    assert lib.tfb_gemm(ptr(C), ptr(C), ptr(C), 2, 2, 2, 5, stream_ptr()) == 0
    assert_device_ok()
    assert torch.all(C == 7.0)


def test_bad_arguments_report_errors():
    C = torch.zeros((2, 2), device="cuda")
    assert lib.tfb_matmul(None, ptr(C), ptr(C), 2, 2, 2, 0, 0, stream_ptr()) == -1
    assert "null" in capi.last_error()
    assert lib.tfb_matmul(ptr(C), ptr(C), ptr(C), 2, 2, 2, 4, 0, stream_ptr()) == -2
    assert lib.tfb_matmul(ptr(C), ptr(C), ptr(C), -1, 2, 2, 0, 0, stream_ptr()) == -1
    assert lib.tfb_gemm_ex(ptr(C), ptr(C), ptr(C), 2, 2, 2, 1, 2, 2, 0, 0, 0, 0, None, 0, stream_ptr()) == -1
    assert lib.tfb_gemm_ex(ptr(C), ptr(C), ptr(C), 2, 2, 2, 2, 2, 2, 0, 0, 0, 0, None, 1, stream_ptr()) == -1


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("shape", [(128, 128, 128), (300, 200, 100), (17, 23, 19), (2, 2, 2), (64, 256, 784),
                                   (784, 256, 64), (1000, 10, 1024), (513, 257, 33), (1, 1, 1)])
def test_fp32_layouts_against_oracle(oracle, shape, trans_a, trans_b):
    M, N, K = shape
    a, b = refdata.uniform(100 + M, (M, K)), refdata.uniform(200 + N, (K, N))
    want = oracle.matmul(a, b)
    A = dev(np.ascontiguousarray(a.T) if trans_a else a)
    B = dev(np.ascontiguousarray(b.T) if trans_b else b)
    C = gemm_ex(A, B, M, N, K, trans_a, trans_b)
    assert_device_ok()
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    assert rel_err(got, want) < FP32_TOL


@pytest.mark.parametrize("in_dtype", [capi.DTYPE_BF16, capi.DTYPE_F16])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 512), (300, 200, 100), (17, 23, 19), (64, 256, 784)])
def test_16bit_layouts_against_oracle(oracle, shape, trans_a, trans_b, in_dtype):
    # Inputs rounded to the 16-bit type on the host, reference loop on the up-converted values.
    M, N, K = shape
    tdt = torch.bfloat16 if in_dtype == capi.DTYPE_BF16 else torch.float16
    a16 = dev(refdata.uniform(300 + M, (M, K)), tdt)
    b16 = dev(refdata.uniform(400 + N, (K, N)), tdt)
    want = oracle.matmul(a16.float().cpu().numpy(), b16.float().cpu().numpy())
    A = a16.t().contiguous() if trans_a else a16
    B = b16.t().contiguous() if trans_b else b16
    C = gemm_ex(A, B, M, N, K, trans_a, trans_b, in_dtype=in_dtype)
    assert_device_ok()
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    assert rel_err(got, want) < 1e-5          # exact products, FP32 accumulate: far inside 1e-2
    C16 = gemm_ex(A, B, M, N, K, trans_a, trans_b, in_dtype=in_dtype, out_dtype=in_dtype)
    assert rel_err(C16.float().cpu().numpy(), want) < BF16_TOL


@pytest.mark.parametrize("flags", [capi.EPI_BIAS_COL, capi.EPI_BIAS_ROW, capi.EPI_RELU,
                                   capi.EPI_BIAS_COL | capi.EPI_RELU, capi.EPI_BIAS_ROW | capi.EPI_RELU])
def test_fused_epilogues(oracle, flags):
    M, N, K = 300, 200, 100
    a, b = refdata.uniform(1, (M, K)), refdata.uniform(2, (K, N))
    bias = refdata.normal(3, (N if flags & capi.EPI_BIAS_COL else M,))
    want = oracle.matmul(a, b)
    if flags & capi.EPI_BIAS_COL:
        want = want + bias[None, :]
    if flags & capi.EPI_BIAS_ROW:
        want = want + bias[:, None]
    if flags & capi.EPI_RELU:
        want = np.maximum(want, 0)
    C = gemm_ex(dev(a), dev(b), M, N, K, bias=dev(bias), flags=flags)
    assert_device_ok()
    assert rel_err(C.cpu().numpy(), want) < FP32_TOL


def test_strided_operands_and_empty_k(oracle):
    M, N, K = 70, 50, 40
    a, b = refdata.uniform(5, (M, K + 8)), refdata.uniform(6, (K, N + 4))
    want = oracle.matmul(a[:, :K], b[:, :N])
    C = gemm_ex(dev(a), dev(b), M, N, K, lda=K + 8, ldb=N + 4)
    assert_device_ok()
    assert rel_err(C.cpu().numpy(), want) < FP32_TOL
    # K == 0: the reference loop leaves acc = 0 (tensor/Tensor.cpp:354-362)
    C = gemm_ex(dev(a), dev(b), M, N, 0, lda=K + 8, ldb=N + 4)
    assert_device_ok()
    assert torch.all(C == 0)


def test_matmul_backward_against_golden(oracle, golden):
    a, b, g = refdata.uniform(11, (96, 112)), refdata.uniform(12, (112, 80)), refdata.normal(13, (96, 80))
    A, B, G = dev(a), dev(b), dev(g)
    dA, dB = torch.empty_like(A), torch.empty_like(B)
    capi.check(lib.tfb_matmul_backward(ptr(G), ptr(A), ptr(B), ptr(dA), ptr(dB), 96, 80, 112, capi.DTYPE_F32,
                                       stream_ptr()))
    assert_device_ok()
    assert rel_err(dA.cpu().numpy(), golden["matmul_bwd_dA"]) < FP32_TOL
    assert rel_err(dB.cpu().numpy(), golden["matmul_bwd_dB"]) < FP32_TOL
    # the reference's arange known answer (autograd/ops/autograd_all_ops_test.cpp:281-328)
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.arange(6, dtype=np.float32).reshape(3, 2)
    A, B, G = dev(a), dev(b), dev(np.ones((2, 2), np.float32))
    dA, dB = torch.empty_like(A), torch.empty_like(B)
    capi.check(lib.tfb_matmul_backward(ptr(G), ptr(A), ptr(B), ptr(dA), ptr(dB), 2, 2, 3, 0, stream_ptr()))
    assert_device_ok()
    np.testing.assert_allclose(dA.cpu().numpy(), [[1, 5, 9], [1, 5, 9]], rtol=1e-6)
    np.testing.assert_allclose(dB.cpu().numpy(), [[3, 3], [5, 5], [7, 7]], rtol=1e-6)


def test_config1_2048_cubed_full_oracle(oracle):
    # FP32 GEMM 2048^3, uniform[-1,1) seed 0, via the Tensor::matmul entry point; full oracle.
    n = 2048
    a, b = refdata.uniform(0, (n, n)), refdata.uniform(1, (n, n))
    got = tfb_matmul(a, b)
    want = oracle.matmul(a, b)
    assert rel_err(got, want) < FP32_TOL
    # and both within FP32 rounding noise of the FP64 product on a sample of rows
    rows = [0, 1, 777, 2047]
    exact = a[rows].astype(np.float64) @ b.astype(np.float64)
    assert rel_err(got[rows], exact) < FP32_TOL


@pytest.mark.parametrize("n", [4096, 8192])
def test_square_sweep_sampled_rows_and_columns(oracle, n):
    # Full products at these sizes take the scalar reference loop minutes to hours; the same loop
    # is applied to 64 full rows and 64 full columns, and linearity is checked on the whole matrix.
    a, b = refdata.uniform(2, (n, n)), refdata.uniform(3, (n, n))
    A, B = dev(a), dev(b)
    C = gemm_ex(A, B, n, n, n)
    assert_device_ok()
    rows = np.linspace(0, n - 1, 64).astype(np.int64)
    cols = np.linspace(0, n - 1, 64).astype(np.int64)
    assert rel_err(C[torch.from_numpy(rows).cuda()].cpu().numpy(), oracle.matmul_rows(a, b, rows)) < FP32_TOL
    assert rel_err(C[:, torch.from_numpy(cols).cuda()].cpu().numpy(), oracle.matmul_cols(a, b, cols)) < FP32_TOL
    # size-independent properties over the full output: C·1 == A·(B·1) and linearity in A
    ones = torch.ones((n,), device="cuda", dtype=torch.float64)
    lhs = C.double() @ ones
    rhs = A.double() @ (B.double() @ ones)
    assert float((lhs - rhs).norm() / rhs.norm()) < 1e-5
    C2 = gemm_ex(A * 2.0, B, n, n, n)
    assert torch.equal(C2, C * 2.0)   # scaling by 2 is exact in every split and product
    # BF16 inputs (host-rounded), FP32 accumulate and output
    a16, b16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
    Cb = gemm_ex(a16, b16, n, n, n, in_dtype=capi.DTYPE_BF16)
    assert_device_ok()
    want = oracle.matmul_rows(a16.float().cpu().numpy(), b16.float().cpu().numpy(), rows[:16])
    assert rel_err(Cb[torch.from_numpy(rows[:16]).cuda()].cpu().numpy(), want) < BF16_TOL


@pytest.mark.parametrize("n", [1024, 2048, 16384])
def test_square_sweep_ends_fp32_and_bf16(oracle, n):
    # The remaining sizes of the sweep, both input types: 64 full rows and 64 full columns against the
    # reference's sequential FP32 loop, and the same rows against an FP64 product. At K = 16384 the
    # reference's own sequential sum sits ~7e-6 from the exact result, so the distance to FP64 is
    # reported next to the distance to the oracle: both must stay inside the budget.
    a, b = refdata.uniform(2, (n, n)), refdata.uniform(3, (n, n))
    A, B = dev(a), dev(b)
    rows = np.linspace(0, n - 1, 64).astype(np.int64)
    cols = np.linspace(0, n - 1, 64).astype(np.int64)
    rows_t, cols_t = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    C = gemm_ex(A, B, n, n, n)
    assert_device_ok()
    got_rows, got_cols = C[rows_t].cpu().numpy(), C[:, cols_t].cpu().numpy()
    exact_rows = (A[rows_t].double() @ B.double()).cpu().numpy()
    want_rows, want_cols = oracle.matmul_rows(a, b, rows), oracle.matmul_cols(a, b, cols)
    err_oracle = max(rel_err(got_rows, want_rows), rel_err(got_cols, want_cols))
    err_exact, oracle_vs_exact = rel_err(got_rows, exact_rows), rel_err(want_rows, exact_rows)
    print(f"n={n} fp32: vs oracle {err_oracle:.2e}, vs fp64 {err_exact:.2e} (oracle vs fp64 {oracle_vs_exact:.2e})")
    assert err_oracle < FP32_TOL
    assert err_exact < FP32_TOL
    del C
    a16, b16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
    Cb = gemm_ex(a16, b16, n, n, n, in_dtype=capi.DTYPE_BF16)
    assert_device_ok()
    a16h, b16h = a16.float().cpu().numpy(), b16.float().cpu().numpy()
    want = oracle.matmul_rows(a16h, b16h, rows[:16])
    assert rel_err(Cb[rows_t[:16]].cpu().numpy(), want) < BF16_TOL
    want = oracle.matmul_cols(a16h, b16h, cols[:16])
    assert rel_err(Cb[:, cols_t[:16]].cpu().numpy(), want) < BF16_TOL
    exact16 = (a16[rows_t[:16]].double() @ b16.double()).cpu().numpy()
    assert rel_err(Cb[rows_t[:16]].cpu().numpy(), exact16) < BF16_TOL


@pytest.mark.parametrize("in_dtype", [capi.DTYPE_F32, capi.DTYPE_BF16])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("shape", [(512, 384, 8192), (1024, 1024, 4096), (1024, 784, 8192), (100, 130, 3000),
                                   (256, 10, 8192)])
def test_split_k_shapes_against_oracle(oracle, shape, trans_a, trans_b, in_dtype):
    # Few output tiles and a long contraction: the K range of each tile is shared between CTAs and the
    # partial sums are added in a second kernel; bias and ReLU must still land exactly once.
    M, N, K = shape
    tdt = torch.float32 if in_dtype == capi.DTYPE_F32 else torch.bfloat16
    a16, b16 = dev(refdata.uniform(7, (M, K)), tdt), dev(refdata.uniform(8, (K, N)), tdt)
    bias = refdata.normal(9, (N,))
    want = np.maximum(oracle.matmul(a16.float().cpu().numpy(), b16.float().cpu().numpy()) + bias[None, :], 0)
    A = a16.t().contiguous() if trans_a else a16
    B = b16.t().contiguous() if trans_b else b16
    C = gemm_ex(A, B, M, N, K, trans_a, trans_b, in_dtype=in_dtype, bias=dev(bias),
                flags=capi.EPI_BIAS_COL | capi.EPI_RELU)
    assert_device_ok()
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    assert rel_err(got, want) < FP32_TOL


@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("in_dtype", [capi.DTYPE_F32, capi.DTYPE_BF16])
def test_matmul_on_host_buffers(oracle, in_dtype, pinned):
    # five row panels (the last one ragged), copies overlapped with the products inside the call
    import ctypes
    M, N, K = 2500, 300, 200
    tdt = torch.float32 if in_dtype == capi.DTYPE_F32 else torch.bfloat16
    a = torch.from_numpy(refdata.uniform(1, (M, K))).to(tdt)
    b = torch.from_numpy(refdata.uniform(2, (K, N))).to(tdt)
    c = torch.full((M, N), float("nan"))
    if pinned:
        a, b, c = a.pin_memory(), b.pin_memory(), c.pin_memory()
    for _ in range(2):   # twice: buffers and streams are reused
        capi.check(lib.tfb_matmul_host(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                                       ctypes.c_void_p(c.data_ptr()), M, N, K, in_dtype, stream_ptr()))
        torch.cuda.current_stream().synchronize()
        assert_device_ok()
        want = oracle.matmul(a.float().numpy(), b.float().numpy())
        assert rel_err(c.numpy(), want) < FP32_TOL
        c.fill_(float("nan"))
    # the same with B already on the device
    Bd = b.cuda()
    capi.check(lib.tfb_matmul_host_b_resident(ctypes.c_void_p(a.data_ptr()), ptr(Bd), ctypes.c_void_p(c.data_ptr()),
                                              M, N, K, in_dtype, stream_ptr()))
    torch.cuda.current_stream().synchronize()
    assert_device_ok()
    assert rel_err(c.numpy(), want) < FP32_TOL


@pytest.mark.parametrize("in_dtype", [capi.DTYPE_F32, capi.DTYPE_BF16])
def test_row_panels_over_the_devices_of_one_process(oracle, in_dtype):
    # Every visible GPU gets a panel (twice over when there is only one GPU: two entries on device 0 with
    # their own streams); panels are ragged, one is empty; B is replicated per device; no collective.
    import ctypes
    ndev = torch.cuda.device_count()
    devices = list(range(ndev)) * (2 if ndev == 1 else 1) + [0]
    rows = [(130 + 77 * g) for g in range(len(devices) - 1)] + [0]
    N, K = 200, 300
    tdt = torch.float32 if in_dtype == capi.DTYPE_F32 else torch.bfloat16
    a_full = torch.from_numpy(refdata.uniform(5, (sum(rows), K))).to(tdt)
    b = torch.from_numpy(refdata.uniform(6, (K, N))).to(tdt)
    want = oracle.matmul(a_full.float().numpy(), b.float().numpy())
    A, B, C, S = [], [], [], []
    r0 = 0
    for d, r in zip(devices, rows):
        A.append(a_full[r0:r0 + r].contiguous().to(f"cuda:{d}"))
        B.append(b.to(f"cuda:{d}"))
        C.append(torch.full((r, N), float("nan"), device=f"cuda:{d}"))
        S.append(torch.cuda.Stream(device=d))
        r0 += r
    n = len(devices)
    arr = lambda ts: (ctypes.c_void_p * n)(*[t.data_ptr() if t.numel() else None for t in ts])
    streams = (ctypes.c_void_p * n)(*[s.cuda_stream for s in S])
    before = torch.cuda.current_device()
    capi.check(lib.tfb_matmul_row_panels(n, (ctypes.c_int * n)(*devices), arr(A), arr(B), arr(C),
                                         (ctypes.c_int64 * n)(*rows), N, K, in_dtype, capi.DTYPE_F32, streams))
    assert torch.cuda.current_device() == before
    for s in S:
        s.synchronize()
    got = np.concatenate([c.cpu().numpy() for c in C], axis=0)
    assert not np.isnan(got).any()
    assert rel_err(got, want) < (FP32_TOL if in_dtype == capi.DTYPE_F32 else BF16_TOL)
    for d in set(devices):
        with torch.cuda.device(d):
            assert_device_ok()
    # a device index that does not exist is refused before anything is enqueued
    bad = (ctypes.c_int * n)(*([devices[0]] * (n - 1) + [ndev + 3]))
    assert lib.tfb_matmul_row_panels(n, bad, arr(A), arr(B), arr(C), (ctypes.c_int64 * n)(*rows), N, K, in_dtype,
                                     capi.DTYPE_F32, streams) == -1


@pytest.mark.parametrize("case", [
    # M, N, K, trans_a, trans_b, flags: one extent of at most 16 (tiles that are mostly padding)
    (700, 10, 1500, False, True, capi.EPI_BIAS_COL | capi.EPI_RELU),   # narrow N: a classifier head
    (256, 16, 64, False, True, capi.EPI_NONE),
    (513, 1001, 10, False, False, capi.EPI_BIAS_ROW),                  # short K, ragged columns
    (2048, 1024, 10, False, False, capi.EPI_NONE),                     # short K: the gradient behind the head
    (10, 1024, 4096, True, False, capi.EPI_NONE),                      # narrow M: the head's weight gradient
    (3, 130, 300, True, False, capi.EPI_NONE),
])
def test_narrow_products_against_oracle(oracle, case):
    M, N, K, ta, tb, flags = case
    a, b = refdata.uniform(17, (M, K)), refdata.uniform(18, (K, N))
    bias = refdata.normal(19, (M if flags & capi.EPI_BIAS_ROW else N,))
    want = oracle.matmul(a, b)
    if flags & capi.EPI_BIAS_COL:
        want = want + bias[None, :]
    if flags & capi.EPI_BIAS_ROW:
        want = want + bias[:, None]
    if flags & capi.EPI_RELU:
        want = np.maximum(want, 0)
    A, B = dev(a.T.copy() if ta else a), dev(b.T.copy() if tb else b)
    C = gemm_ex(A, B, M, N, K, ta, tb, bias=dev(bias) if flags else None, flags=flags)
    # and with both operands given as hi / lo planes
    lda, ldb = (A.shape[1] + 3) // 4 * 4, (B.shape[1] + 3) // 4 * 4
    ap = torch.full((2, A.shape[0], lda), float("nan"), device="cuda")
    bp = torch.full((2, B.shape[0], ldb), float("nan"), device="cuda")
    capi.check(lib.tfb_split_tf32(ptr(A), A.shape[0], A.shape[1], A.shape[1], ptr(ap[0]), ptr(ap[1]), lda, stream_ptr()))
    capi.check(lib.tfb_split_tf32(ptr(B), B.shape[0], B.shape[1], B.shape[1], ptr(bp[0]), ptr(bp[1]), ldb, stream_ptr()))
    C2 = torch.full((M, N), float("nan"), device="cuda")
    bias_d = dev(bias) if flags else None
    capi.check(lib.tfb_gemm_presplit(ptr(ap[0]), ptr(ap[1]), ptr(bp[0]), ptr(bp[1]), ptr(C2), M, N, K, lda, ldb, N,
                                     int(ta), int(tb), ptr(bias_d), flags, stream_ptr()))
    assert_device_ok()
    for got in (C.cpu().numpy(), C2.cpu().numpy()):
        assert not np.isnan(got).any()
        assert rel_err(got, want) < FP32_TOL


@pytest.mark.parametrize("in_dtype", [capi.DTYPE_F32, capi.DTYPE_BF16])
def test_batched_matmul_against_oracle(oracle, in_dtype):
    # N-D operands: [batch, M, K] x [batch, K, N], a shared right-hand side (stride 0: one tall product
    # under the hood) and a padded batch stride; every matrix against the oracle's 2-D loop
    tdt = torch.float32 if in_dtype == capi.DTYPE_F32 else torch.bfloat16
    tol = FP32_TOL if in_dtype == capi.DTYPE_F32 else BF16_TOL
    batch, M, N, K = 5, 96, 80, 112
    a = dev(refdata.uniform(1, (batch, M, K)), tdt)
    b = dev(refdata.uniform(2, (batch, K, N)), tdt)
    ah, bh = a.float().cpu().numpy(), b.float().cpu().numpy()
    C = torch.full((batch, M, N), float("nan"), device="cuda")
    capi.check(lib.tfb_matmul_batched(ptr(a), ptr(b), ptr(C), batch, M, N, K, M * K, K * N, M * N, in_dtype,
                                      capi.DTYPE_F32, stream_ptr()))
    assert_device_ok()
    for i in range(batch):
        assert rel_err(C[i].cpu().numpy(), oracle.matmul(ah[i], bh[i])) < tol, i
    C.fill_(float("nan"))
    capi.check(lib.tfb_matmul_batched(ptr(a), ptr(b), ptr(C), batch, M, N, K, M * K, 0, M * N, in_dtype,
                                      capi.DTYPE_F32, stream_ptr()))
    assert_device_ok()
    for i in range(batch):
        assert rel_err(C[i].cpu().numpy(), oracle.matmul(ah[i], bh[0])) < tol, i
    pad = torch.full((batch, M + 3, N), float("nan"), device="cuda")   # output matrices (M + 3) * N apart
    capi.check(lib.tfb_matmul_batched(ptr(a), ptr(b), ptr(pad), batch, M, N, K, M * K, K * N, (M + 3) * N, in_dtype,
                                      capi.DTYPE_F32, stream_ptr()))
    assert_device_ok()
    assert rel_err(pad[3, :M].cpu().numpy(), oracle.matmul(ah[3], bh[3])) < tol
    assert torch.isnan(pad[:, M:]).all()
    assert lib.tfb_matmul_batched(ptr(a), ptr(b), ptr(C), batch, M, N, K, M * K, K * N, M * N - 1, in_dtype,
                                  capi.DTYPE_F32, stream_ptr()) == -1   # overlapping outputs
    assert lib.tfb_matmul_batched(ptr(a), ptr(b), ptr(C), 0, M, N, K, 0, 0, 0, in_dtype, capi.DTYPE_F32, stream_ptr()) == 0


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(64, 256, 784), (10, 1024, 1024), (1, 7, 513), (128, 128, 600), (33, 100, 1999),
                                   (16, 1000, 2048), (1024, 10, 1024), (700, 16, 784), (1000, 7, 513)])
def test_few_rows_long_contraction_on_the_cuda_core_kernel(oracle, shape, trans_a, trans_b):
    # the window of the one-launch CUDA-core kernel (at most 128 rows — or, run transposed, at most 128 columns —
    # and 16384 outputs, K in 512..2048): every
    # operand layout, ragged tiles, K slices that do not divide evenly between the blocks of a cluster,
    # bias and ReLU; plain FP32 FMAs, so the distance to an FP64 product is checked as well
    M, N, K = shape
    a, b = refdata.uniform(11, (M, K)), refdata.uniform(12, (K, N))
    bias = refdata.normal(13, (N,))
    A, B = dev(a), dev(b)
    As = A.t().contiguous() if trans_a else A
    Bs = B.t().contiguous() if trans_b else B
    C = gemm_ex(As, Bs, M, N, K, trans_a, trans_b, bias=dev(bias), flags=capi.EPI_BIAS_COL | capi.EPI_RELU)
    assert_device_ok()
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    want = np.maximum(oracle.matmul(a, b) + bias[None, :], 0)
    assert rel_err(got, want) < FP32_TOL
    exact = np.maximum(a.astype(np.float64) @ b.astype(np.float64) + bias[None, :], 0)
    assert rel_err(got, exact) < FP32_TOL
    # operands given as TF32 planes are added back together exactly: same bits as the unsplit call
    if K % 4 == 0 and M % 4 == 0 and N % 4 == 0:
        hA, hB = torch.empty((2, *As.shape), device="cuda"), torch.empty((2, *Bs.shape), device="cuda")
        capi.check(lib.tfb_split_tf32(ptr(As), As.shape[0], As.shape[1], As.shape[1], ptr(hA[0]), ptr(hA[1]), As.shape[1], stream_ptr()))
        capi.check(lib.tfb_split_tf32(ptr(Bs), Bs.shape[0], Bs.shape[1], Bs.shape[1], ptr(hB[0]), ptr(hB[1]), Bs.shape[1], stream_ptr()))
        C2 = torch.full((M, N), float("nan"), device="cuda")
        capi.check(lib.tfb_gemm_presplit(ptr(hA[0]), ptr(hA[1]), ptr(hB[0]), ptr(hB[1]), ptr(C2), M, N, K, As.shape[1],
                                         Bs.shape[1], N, int(trans_a), int(trans_b), ptr(dev(bias)),
                                         capi.EPI_BIAS_COL | capi.EPI_RELU, stream_ptr()))
        assert_device_ok()
        assert torch.equal(C2, C)


@pytest.mark.parametrize("raw_hi", [1, 0])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True), (True, True)])
def test_operand_as_its_own_hi_plane(oracle, raw_hi, trans_a, trans_b, product_path):
    # kind::tf32 drops the low 13 mantissa bits of what it reads, so an aligned FP32 operand serves as its
    # own hi plane and only lo = x - trunc(x) is written (knob RAW_HI, default off). Both forms must sit at
    # the same distance from an FP64 product — a lo plane that does not match the hi plane it is used with
    # would show as an error near 1e-3 — for aligned operands, operands with padded rows whose padding holds
    # garbage, rows that are not a multiple of 16 bytes, and a base pointer off the 16-byte grid.
    if product_path == "tensor_cores_only":
        pytest.skip("none of these shapes is in the CUDA-core window")
    old = ctypes.c_int(0)
    capi.check(lib.tfb_get_tuning(capi.TUNE_RAW_HI, ctypes.byref(old)))
    capi.check(lib.tfb_set_tuning(capi.TUNE_RAW_HI, raw_hi))
    try:
        for (M, N, K, pad_a, pad_b, shift) in ((384, 320, 512, 0, 0, 0), (300, 200, 100, 8, 4, 0), (130, 70, 90, 3, 1, 0),
                                                 (256, 256, 256, 4, 4, 1), (1024, 1024, 1100, 0, 0, 0)):
            a, b = refdata.uniform(31, (M, K)), refdata.uniform(32, (K, N))
            sa, sb = (a.T if trans_a else a), (b.T if trans_b else b)
            hold_a = np.full((sa.shape[0], sa.shape[1] + pad_a), np.float32(1e30))
            hold_b = np.full((sb.shape[0], sb.shape[1] + pad_b), np.float32(-1e30))
            hold_a[:, :sa.shape[1]] = sa
            hold_b[:, :sb.shape[1]] = sb
            # `shift` floats in front of the matrix take its base off the 16-byte grid
            fa = torch.cat([torch.zeros(shift, device="cuda"), dev(hold_a).reshape(-1)])
            fb = torch.cat([torch.zeros(shift, device="cuda"), dev(hold_b).reshape(-1)])
            C = gemm_ex(fa[shift:], fb[shift:], M, N, K, trans_a, trans_b, lda=hold_a.shape[1], ldb=hold_b.shape[1])
            assert_device_ok()
            got = C.cpu().numpy()
            exact = a.astype(np.float64) @ b.astype(np.float64)
            assert rel_err(got, exact) < 4e-6, (M, N, K, pad_a, pad_b, shift)
            assert rel_err(got, oracle.matmul(a, b)) < FP32_TOL
    finally:
        capi.check(lib.tfb_set_tuning(capi.TUNE_RAW_HI, old.value))


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (1024, 784, 1024), (1000, 900, 1100), (130, 128, 4096), (512, 640, 520),
                                   (700, 1001, 777)])
def test_cluster_split_k_is_the_two_kernel_form_bit_for_bit(oracle, shape, trans_a, trans_b, product_path):
    # FP32 products of a few 128 x 128 tiles with two K splits: by default (knob CLUSTER_K) the two halves of
    # a tile run in the two CTAs of a cluster and meet in distributed shared memory; with the knob off they go
    # through partial sums in scratch and the reduction kernel. Both add own + peer and then apply bias and
    # ReLU, so the results must agree bit for bit; and both must match the oracle.
    if product_path == "tensor_cores_only":
        pytest.skip("none of these shapes is in the CUDA-core window")
    M, N, K = shape
    a, b = refdata.uniform(41, (M, K)), refdata.uniform(42, (K, N))
    bias = refdata.normal(43, (N,))
    A, B = dev(np.ascontiguousarray(a.T) if trans_a else a), dev(np.ascontiguousarray(b.T) if trans_b else b)
    knobs = (capi.TUNE_GEMM_TILE_N, capi.TUNE_GEMM_PAIR, capi.TUNE_GEMM_SPLIT_K, capi.TUNE_CLUSTER_K)
    old = []
    for k in knobs:
        v = ctypes.c_int(0)
        capi.check(lib.tfb_get_tuning(k, ctypes.byref(v)))
        old.append(v.value)
    out = {}
    try:
        capi.check(lib.tfb_set_tuning(capi.TUNE_GEMM_TILE_N, 128))
        capi.check(lib.tfb_set_tuning(capi.TUNE_GEMM_PAIR, 0))
        capi.check(lib.tfb_set_tuning(capi.TUNE_GEMM_SPLIT_K, 2))
        for cluster in (1, 0):
            capi.check(lib.tfb_set_tuning(capi.TUNE_CLUSTER_K, cluster))
            C = gemm_ex(A, B, M, N, K, trans_a, trans_b, bias=dev(bias), flags=capi.EPI_BIAS_COL | capi.EPI_RELU)
            assert_device_ok()
            out[cluster] = C.cpu().numpy()
    finally:
        for k, v in zip(knobs, old):
            capi.check(lib.tfb_set_tuning(k, v))
    assert not np.isnan(out[1]).any()
    assert np.array_equal(out[1], out[0])
    want = np.maximum(oracle.matmul(a, b) + bias[None, :], 0)
    assert rel_err(out[1], want) < FP32_TOL
