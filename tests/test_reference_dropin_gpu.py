"""The drop-in shown against the reference itself: the reference's own Tensor / autograd / allocator
sources, with the edits of oracle/dropin/apply_dropin.py applied to a temporary copy and
oracle/dropin/tfb_registrar.cpp linked in, run the reference's known answers on Device::cuda(0) tensors —
Tensor::matmul dispatches through the added registry slot into libtfb.so, and Tensor::backward walks the
reference's Engine into the patched MatmulBackward. Built by `make -C oracle dropin` where a reference
checkout exists; the prebuilt library travels with the repository snapshot."""
import ctypes
import os

import numpy as np
import pytest

import refdata

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libtf_ref_dropin.so")


@pytest.fixture(scope="module")
def dropin():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libtf_ref_dropin.so not built (needs a reference checkout at build time)")
    lib = ctypes.CDLL(LIB)
    fp = ctypes.POINTER(ctypes.c_float)
    lib.dropin_matmul.argtypes = [fp, fp, fp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    lib.dropin_matmul_backward.argtypes = [fp, fp, fp, fp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    lib.dropin_last_error.restype = ctypes.c_char_p
    return lib


def f(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def matmul(lib, a, b):
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    c = np.full((a.shape[0], b.shape[1]), np.nan, np.float32)
    rc = lib.dropin_matmul(f(a), f(b), f(c), a.shape[0], b.shape[1], a.shape[1])
    assert rc == 0, lib.dropin_last_error().decode()
    return c


def test_reference_matmul_known_answers_on_cuda_tensors(dropin, oracle):
    # tensor ops test of the reference: [[1,2],[3,4]] x [[5,6],[7,8]] = [[19,22],[43,50]]
    c = matmul(dropin, [[1, 2], [3, 4]], [[5, 6], [7, 8]])
    np.testing.assert_allclose(c, [[19, 22], [43, 50]], rtol=1e-6)
    # [[0,1,2],[3,4,5]] x [[0,1],[2,3],[4,5]] = [[10,13],[28,40]]
    c = matmul(dropin, np.arange(6).reshape(2, 3), np.arange(6).reshape(3, 2))
    np.testing.assert_allclose(c, [[10, 13], [28, 40]], rtol=1e-6)
    # an odd shape against the oracle's restatement of the reference loop
    a, b = refdata.uniform(1, (17, 19)), refdata.uniform(2, (19, 23))
    got, want = matmul(dropin, a, b), oracle.matmul(a, b)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5
    a, b = refdata.uniform(3, (300, 520)), refdata.uniform(4, (520, 260))
    got, want = matmul(dropin, a, b), oracle.matmul(a, b)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5


def test_reference_backward_known_answer_on_cuda_tensors(dropin):
    # autograd/ops/autograd_all_ops_test.cpp:281-328: c = a.matmul(b); c.backward()
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.arange(6, dtype=np.float32).reshape(3, 2)
    ga, gb = np.full_like(a, np.nan), np.full_like(b, np.nan)
    rc = dropin.dropin_matmul_backward(f(a), f(b), f(ga), f(gb), 2, 2, 3)
    assert rc == 0, dropin.dropin_last_error().decode()
    np.testing.assert_allclose(ga, [[1, 5, 9], [1, 5, 9]], rtol=1e-6)
    np.testing.assert_allclose(gb, [[3, 3], [5, 5], [7, 7]], rtol=1e-6)


def test_reference_argument_checks_survive_the_cuda_branch(dropin):
    assert dropin.dropin_matmul_shape_mismatch_throws() == 0
