"""The device-side loops of the autograd walk (fill, ReLU and its backward mask, gradient accumulation,
scaling by a device scalar): exact operations, so bit-exact against numpy — at aligned and unaligned
addresses and with ragged lengths."""
import numpy as np
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from gpu_util import assert_device_ok, lib, ptr, stream_ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 4096, 1000003])
@pytest.mark.parametrize("offset", [0, 1])
def test_vector_ops_bit_exact(n, offset):
    x = refdata.normal(11, (n + offset,))
    x[::7] = 0.0   # exact zeros exercise the x == 0 side of the mask
    g = refdata.normal(12, (n + offset,))
    X, G = torch.from_numpy(x).cuda()[offset:], torch.from_numpy(g).cuda()[offset:]
    xs, gs = x[offset:], g[offset:]
    out = torch.full((n + offset,), float("nan"), device="cuda")[offset:]

    capi.check(lib.tfb_relu_forward(ptr(X), ptr(out), n, stream_ptr()))
    assert np.array_equal(out.cpu().numpy(), np.maximum(xs, 0))
    capi.check(lib.tfb_relu_backward(ptr(X), ptr(G), ptr(out), n, stream_ptr()))
    assert np.array_equal(out.cpu().numpy(), np.where(xs > 0, gs, np.float32(0)))
    capi.check(lib.tfb_fill(ptr(out), n, 1.0, stream_ptr()))
    assert np.array_equal(out.cpu().numpy(), np.ones(n, np.float32))
    acc = torch.from_numpy(x.copy()).cuda()[offset:]
    capi.check(lib.tfb_accumulate(ptr(acc), ptr(G), n, stream_ptr()))
    assert np.array_equal(acc.cpu().numpy(), xs + gs)
    scalar = torch.tensor([0.3], device="cuda")
    capi.check(lib.tfb_scale_by_device_scalar(ptr(X), ptr(scalar), ptr(out), n, stream_ptr()))
    assert np.array_equal(out.cpu().numpy(), xs * np.float32(0.3))
    assert_device_ok()


def test_vector_ops_reject_bad_arguments():
    t = torch.zeros(8, device="cuda")
    assert lib.tfb_fill(ptr(t), -1, 1.0, stream_ptr()) == -1
    assert lib.tfb_relu_forward(None, ptr(t), 8, stream_ptr()) == -1
    assert lib.tfb_relu_backward(ptr(t), None, ptr(t), 8, stream_ptr()) == -1
    assert lib.tfb_accumulate(None, ptr(t), 8, stream_ptr()) == -1
    assert lib.tfb_scale_by_device_scalar(ptr(t), None, ptr(t), 8, stream_ptr()) == -1
    assert lib.tfb_fill(None, 0, 1.0, stream_ptr()) == 0   # nothing to do
