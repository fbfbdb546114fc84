"""Helpers for the -m gpu tests: torch supplies device memory and streams, every computation
goes through the C-ABI of libtfb.so."""
import ctypes

import numpy as np
import torch

import tensors_b200.capi as capi

lib = capi.lib
TORCH_DTYPE = {capi.DTYPE_F32: torch.float32, capi.DTYPE_F16: torch.float16, capi.DTYPE_BF16: torch.bfloat16}


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def assert_device_ok():
    code = capi.device_status()
    assert code == 0, f"a kernel recorded device error {code}"


def rel_err(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / denom) if denom > 0 else float(np.linalg.norm(got))


def gemm_ex(A, B, M, N, K, trans_a=False, trans_b=False, in_dtype=capi.DTYPE_F32, out_dtype=capi.DTYPE_F32,
            bias=None, flags=0, lda=None, ldb=None):
    """A, B: torch device tensors holding the stored matrices. Returns C [M,N] as a device tensor."""
    C = torch.full((M, N), float("nan"), device="cuda", dtype=TORCH_DTYPE[out_dtype])
    lda = lda if lda is not None else A.shape[-1]
    ldb = ldb if ldb is not None else B.shape[-1]
    capi.check(lib.tfb_gemm_ex(ptr(A), ptr(B), ptr(C), M, N, K, lda, ldb, N, int(trans_a), int(trans_b),
                               in_dtype, out_dtype, ptr(bias), flags, stream_ptr()))
    return C
