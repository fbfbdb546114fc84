"""Parity of the implicit-GEMM Conv2d (forward, dgrad, wgrad, bias gradient) with the oracle, with the
reference's own known answers and golden outputs, and the bit-exact im2col index map."""
import ctypes
import os

import numpy as np
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from golden.make_golden import CONV_CHANNELS_L1, CONV_CHANNELS_L2
from gpu_util import assert_device_ok, dev, lib, ptr, rel_err, stream_ptr

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5


def out_dim(n, k, s, p, d):
    return int(lib.tfb_conv_out_dim(n, k, s, p, d))


def conv_forward(x, w, b, stride=(1, 1), pad=(0, 0), dil=(1, 1), relu=False):
    N, C, H, W = x.shape
    Cout, _, kH, kW = w.shape
    oH, oW = out_dim(H, kH, stride[0], pad[0], dil[0]), out_dim(W, kW, stride[1], pad[1], dil[1])
    X, Wt = dev(x), dev(w)
    B = dev(b) if b is not None else None
    out = torch.full((N, Cout, oH, oW), float("nan"), device="cuda")
    capi.check(lib.tfb_conv2d_forward(ptr(X), ptr(Wt), ptr(B), ptr(out), N, C, H, W, Cout, kH, kW, stride[0], stride[1],
                                      pad[0], pad[1], dil[0], dil[1], int(relu), capi.DTYPE_F32, stream_ptr()))
    assert_device_ok()
    return out.cpu().numpy()


def conv_backward(x, w, g, stride=(1, 1), pad=(0, 0), dil=(1, 1)):
    N, C, H, W = x.shape
    Cout, _, kH, kW = w.shape
    X, Wt, G = dev(x), dev(w), dev(g)
    gi = torch.full(x.shape, float("nan"), device="cuda")
    gw = torch.full(w.shape, float("nan"), device="cuda")
    gb = torch.full((Cout,), float("nan"), device="cuda")
    capi.check(lib.tfb_conv2d_backward(ptr(X), ptr(Wt), ptr(G), ptr(gi), ptr(gw), ptr(gb), N, C, H, W, Cout, kH, kW,
                                       stride[0], stride[1], pad[0], pad[1], dil[0], dil[1], capi.DTYPE_F32, stream_ptr()))
    assert_device_ok()
    return gi.cpu().numpy(), gw.cpu().numpy(), gb.cpu().numpy()


@pytest.fixture(params=["default", "tma_feed", "gather_kernel"])
def feed(request):
    """By default a product with at least 16 contraction channels runs on the TMA-fed GEMM kernel (forward
    and weight gradient at any stride whose tile fits a 256-element box, input gradient at stride 1), short contractions (forward with Cin*kH*kW <= 128, input gradient with Cin <= 4, weight
    gradient with Cin*kH*kW < 32) on the CUDA-core kernels and everything else on the kernel with software gather producers.
    The CONV_TMA knob at 2 sends every product the feed can express to the first; CONV_TMA = 0 with CONV_DIRECT = 0
    everything to the last, so each kernel gets every case it can take."""
    def get(knob):
        v = ctypes.c_int(0)
        capi.check(lib.tfb_get_tuning(knob, ctypes.byref(v)))
        return v.value
    old = {k: get(k) for k in (capi.TUNE_CONV_TMA, capi.TUNE_CONV_DIRECT)}
    capi.check(lib.tfb_set_tuning(capi.TUNE_CONV_TMA, 1))
    capi.check(lib.tfb_set_tuning(capi.TUNE_CONV_DIRECT, 1))
    if request.param == "gather_kernel":
        capi.check(lib.tfb_set_tuning(capi.TUNE_CONV_TMA, 0))
        capi.check(lib.tfb_set_tuning(capi.TUNE_CONV_DIRECT, 0))
    elif request.param == "tma_feed":
        capi.check(lib.tfb_set_tuning(capi.TUNE_CONV_TMA, 2))
    yield request.param
    for k, v in old.items():
        capi.check(lib.tfb_set_tuning(k, v))


def test_reference_known_answers(feed):
    # nn/conv2d_forward_test.cpp:112-137 and nn/conv2d_backward_test.cpp:110-160
    x = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2)
    w = np.array([2.0], np.float32).reshape(1, 1, 1, 1)
    np.testing.assert_allclose(conv_forward(x, w, None).ravel(), [2, 4, 6, 8], rtol=1e-6)
    go = np.array([0.1, 0.2, 0.3, 0.4], np.float32).reshape(1, 1, 2, 2)
    gi, gw, gb = conv_backward(x, w, go)
    np.testing.assert_allclose(gi.ravel(), [0.2, 0.4, 0.6, 0.8], rtol=1e-4)
    np.testing.assert_allclose(gw.ravel(), [3.0], rtol=1e-4)
    np.testing.assert_allclose(gb.ravel(), [1.0], rtol=1e-4)


def test_reference_backward_test_patterns(oracle, feed):
    # the fill patterns of nn/conv2d_backward_test.cpp:162-300, tolerance of those tests (1e-3) or tighter
    f = np.float32
    cases = []
    w = np.arange(1, 9, dtype=f).reshape(2, 1, 2, 2)
    x = (f(0.1) * np.arange(1, 19, dtype=f)).reshape(2, 1, 3, 3)
    go = (f(0.01) * ((np.arange(16) % 11) + 1).astype(f)).reshape(2, 2, 2, 2)
    cases.append((x, w, np.array([0.1, -0.2], f), go, (0, 0)))
    w = (f(0.02) * ((np.arange(3 * 2 * 9) % 7) + 1).astype(f)).reshape(3, 2, 3, 3)
    x = (f(0.05) * ((np.arange(2 * 16) % 5) + 1).astype(f)).reshape(1, 2, 4, 4)
    go = (f(0.01) * ((np.arange(3 * 16) % 13) + 1).astype(f)).reshape(1, 3, 4, 4)
    cases.append((x, w, np.array([0.3, 0.1, -0.2], f), go, (1, 1)))
    w = np.full((1, 1, 2, 2), 0.5, f)
    x = np.arange(1, 10, dtype=f).reshape(1, 1, 3, 3)
    go = (f(0.1) * np.arange(1, 5, dtype=f)).reshape(1, 1, 2, 2)
    cases.append((x, w, None, go, (0, 0)))
    for x, w, b, go, pad in cases:
        y = conv_forward(x, w, b, pad=pad)
        np.testing.assert_allclose(y, oracle.conv2d_forward(x, w, b, pad=pad), rtol=1e-5, atol=1e-6)
        gi, gw, gb = conv_backward(x, w, go, pad=pad)
        oi, ow, ob = oracle.conv2d_backward(x, w, go, pad=pad)
        np.testing.assert_allclose(gi, oi, rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(gw, ow, rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(gb, ob, rtol=1e-4, atol=1e-6)


def test_forward_against_reference_golden(golden):
    # 3 -> 64 and 64 -> 128 channels, 3x3, pad 1, stride 1 on 32x32 images, reference Kaiming weights
    x, w1 = refdata.normal(31, (2, 3, 32, 32)), refdata.conv_weight(3, 64, 3)
    y1 = conv_forward(x, w1, None, pad=(1, 1))
    assert rel_err(y1[:, CONV_CHANNELS_L1], golden["conv_l1_Y_ch"]) < FP32_TOL
    assert rel_err(y1.astype(np.float64).sum(axis=(0, 2, 3)), golden["conv_l1_Y_sum"]) < FP32_TOL
    x2, w2 = refdata.normal(32, (1, 64, 32, 32)), refdata.conv_weight(64, 128, 3)
    y2 = conv_forward(x2, w2, None, pad=(1, 1))
    assert rel_err(y2[:, CONV_CHANNELS_L2], golden["conv_l2_Y_ch"]) < FP32_TOL
    assert rel_err(y2.astype(np.float64).sum(axis=(0, 2, 3)), golden["conv_l2_Y_sum"]) < FP32_TOL
    xs, ws = refdata.normal(33, (2, 4, 9, 11)), refdata.conv_weight(4, 6, 3)
    ys = conv_forward(xs, ws, None, (2, 2), (2, 2), (2, 2))
    assert rel_err(ys, golden["conv_s2p2d2_Y"]) < FP32_TOL


@pytest.mark.parametrize("case", [
    # N, Cin, H, W, Cout, kH, kW, stride, pad, dil
    (2, 3, 32, 32, 64, 3, 3, (1, 1), (1, 1), (1, 1)),
    (2, 64, 32, 32, 128, 3, 3, (1, 1), (1, 1), (1, 1)),
    (3, 5, 13, 17, 7, 3, 2, (2, 1), (1, 2), (1, 2)),
    (2, 4, 9, 11, 6, 3, 3, (2, 2), (2, 2), (2, 2)),
    (1, 130, 6, 5, 140, 1, 1, (1, 1), (0, 0), (1, 1)),
    (2, 2, 40, 40, 3, 5, 5, (3, 3), (2, 2), (1, 1)),
    (1, 1, 1, 1, 1, 1, 1, (1, 1), (0, 0), (1, 1)),
    # stride 1 with ragged extents: widths that are no power of two, wider than one tile, dilation,
    # asymmetric padding, channel counts with a tail block, more than one column tile
    (2, 8, 28, 28, 16, 5, 5, (1, 1), (2, 2), (1, 1)),
    (1, 3, 5, 150, 4, 3, 3, (1, 1), (1, 1), (1, 1)),
    (2, 6, 12, 10, 9, 3, 3, (1, 1), (2, 2), (2, 2)),
    (1, 40, 9, 7, 150, 2, 3, (1, 1), (0, 2), (1, 1)),
    (3, 70, 16, 16, 70, 3, 3, (1, 1), (1, 1), (1, 1)),
    (2, 4, 6, 6, 5, 3, 3, (1, 1), (0, 0), (1, 1)),
    # strides with enough channels for the TMA feed by default (forward and weight gradient; the input
    # gradient of a strided layer stays on the gather kernel): odd extents, dilation, a stride per axis,
    # an output row wider than one tile, a stride whose box would exceed 256 elements (gather kernel)
    (2, 32, 33, 31, 48, 3, 3, (2, 2), (1, 1), (1, 1)),
    (1, 64, 56, 56, 64, 3, 3, (2, 2), (1, 1), (1, 1)),
    (2, 24, 20, 70, 40, 3, 3, (1, 3), (1, 0), (1, 1)),
    (2, 16, 19, 19, 24, 3, 3, (2, 2), (2, 2), (2, 2)),
    (1, 16, 8, 300, 8, 1, 3, (1, 2), (0, 1), (1, 1)),
    (1, 16, 4, 400, 8, 1, 1, (1, 3), (0, 0), (1, 1)),
    (2, 20, 30, 30, 36, 4, 4, (4, 4), (0, 0), (1, 1)),
])
def test_forward_backward_against_oracle(oracle, case, feed):
    N, Cin, H, W, Cout, kH, kW, stride, pad, dil = case
    x = refdata.normal(1, (N, Cin, H, W))
    w = refdata.kaiming_uniform((Cout, Cin, kH, kW), Cin * kH * kW)
    b = refdata.normal(2, (Cout,)) * np.float32(0.1)
    y = conv_forward(x, w, b, stride, pad, dil)
    assert not np.isnan(y).any()
    assert rel_err(y, oracle.conv2d_forward(x, w, b, stride, pad, dil)) < FP32_TOL
    yr = conv_forward(x, w, b, stride, pad, dil, relu=True)
    assert rel_err(yr, np.maximum(oracle.conv2d_forward(x, w, b, stride, pad, dil), 0)) < FP32_TOL
    g = refdata.normal(3, y.shape)
    gi, gw, gb = conv_backward(x, w, g, stride, pad, dil)
    oi, ow, ob = oracle.conv2d_backward(x, w, g, stride, pad, dil)
    assert not (np.isnan(gi).any() or np.isnan(gw).any() or np.isnan(gb).any())
    assert rel_err(gi, oi) < FP32_TOL
    assert rel_err(gw, ow) < FP32_TOL
    assert rel_err(gb, ob) < FP32_TOL


def index_map(n_first, n_count, Cin, H, W, kH, kW, sh, sw, ph, pw, dh, dw):
    K, P = Cin * kH * kW, out_dim(H, kH, sh, ph, dh) * out_dim(W, kW, sw, pw, dw)
    out = torch.full((n_count * K * P,), -7, device="cuda", dtype=torch.int64)
    capi.check(lib.tfb_im2col_index_map(ptr(out), n_first, n_count, Cin, H, W, kH, kW, sh, sw, ph, pw, dh, dw, stream_ptr()))
    assert_device_ok()
    return out.cpu().numpy()


def test_im2col_index_map_bit_exact(oracle):
    # layer 1 of the CIFAR-shaped configuration over its entire index space (128 x 27 x 1024 entries)
    got = index_map(0, 128, 3, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1)
    want = oracle.im2col_index_range(0, got.size, 3, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1)
    assert np.array_equal(got, want)
    # layer 2 (75.5 M entries): the map repeats per sample up to the sample offset; first, middle, last
    per_n = 576 * 1024
    for n in (0, 64, 127):
        got = index_map(n, 1, 64, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1)
        want = oracle.im2col_index_range(n * per_n, per_n, 64, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1)
        assert np.array_equal(got, want)
    # strided, dilated and asymmetric cases
    for args in [(5, 13, 17, 3, 2, 2, 1, 1, 2, 1, 2), (4, 9, 11, 3, 3, 2, 2, 2, 2, 2, 2), (2, 40, 40, 5, 5, 3, 3, 2, 2, 1, 1)]:
        got = index_map(0, 3, *args)
        want = oracle.im2col_index_range(0, got.size, *args)
        assert np.array_equal(got, want)


def _own_index_tensor(N, C, H, W):
    """x[n, c, h, w] = 1 + its own linear index inside sample n (exact in FP32 and in the hi + lo split:
    at most 17 bits); 0 is left for the padding."""
    per = C * H * W
    return np.tile((np.arange(per, dtype=np.float32) + 1).reshape(1, C, H, W), (N, 1, 1, 1))


@pytest.mark.parametrize("layer", [1, 2])
def test_index_map_through_the_production_kernels_bit_exact(oracle, layer):
    # The index map of the kernels the named configuration really runs (default dispatch: layer 1 on the
    # CUDA-core kernels, layer 2 on the TMA-fed tensor-core path), forward and input gradient. The input
    # holds each element's own linear index and every filter is one-hot, so an output element IS the
    # index the kernel read (0 in the padding): integers, compared exactly with the reference formula
    # (cuda/kernels/im2col.cu:67-98, restated in the oracle; the scheme of cuda/kernels/im2col_test.cpp:75-107).
    Cin, Cout = (3, 64) if layer == 1 else (64, 128)
    N, H, W, k, pad = 4, 32, 32, 3, 1
    K, P = Cin * k * k, H * W
    per = Cin * H * W
    x = _own_index_tensor(N, Cin, H, W)
    want_map = oracle.im2col_index_range(0, N * K * P, Cin, H, W, k, k, 1, 1, pad, pad, 1, 1).reshape(N, K, P)
    sample_base = (np.arange(N, dtype=np.int64) * per).reshape(N, 1, 1)
    want_val = np.where(want_map >= 0, want_map - sample_base + 1, 0)          # [N, K, P]
    # forward: output channel j of a pass reads tap first + j and nothing else
    for first in range(0, K, Cout):
        taps = np.arange(first, min(first + Cout, K))
        w = np.zeros((Cout, K), np.float32)
        w[np.arange(len(taps)), taps] = 1.0
        y = conv_forward(x, w.reshape(Cout, Cin, k, k), None, pad=(pad, pad)).reshape(N, Cout, P)
        got = y[:, :len(taps)].astype(np.int64)
        assert np.array_equal(got, want_val[:, taps]), (layer, first)
        assert not y[:, len(taps):].any()
    # input gradient: dY holds its own index, channel c of dX receives exactly one (co, ki, kj) per pass
    dy = _own_index_tensor(N, Cout, H, W)                                      # out extent = in extent here
    for tap in range(k * k):
        w = np.zeros((Cout, Cin, k * k), np.float32)
        co_of = (np.arange(Cin) * 7 + tap * 5) % Cout
        w[co_of, np.arange(Cin), tap] = 1.0
        gi, _, _ = conv_backward(x, w.reshape(Cout, Cin, k, k), dy, pad=(pad, pad))
        want = np.zeros((N, per), np.int64)
        for c in range(Cin):
            t = c * k * k + tap
            src = want_map[:, t, :]                                            # [N, P] offsets into x, or -1
            val = (co_of[c] * P + np.arange(P, dtype=np.int64) + 1)[None, :].repeat(N, 0)
            nn, pp = np.nonzero(src >= 0)
            want[nn, src[nn, pp] - nn * per] = val[nn, pp]
        assert np.array_equal(gi.reshape(N, per).astype(np.int64), want), (layer, tap)


def test_index_map_of_a_strided_layer_on_the_tma_feed_bit_exact(oracle):
    # The same scheme for a layer whose stride and dilation are expressed by the tensor map itself
    # (traversal stride of the box, tap offsets added to its start): 32 channels, 3x3, stride 2, dilation 2,
    # pad 2, odd extents. Forward only: the input gradient of a strided layer runs on the gather kernel, whose
    # index function is pinned separately.
    N, Cin, H, W, Cout, k, st, pad, dil = 2, 32, 21, 19, 96, 3, 2, 2, 2
    oH, oW = out_dim(H, k, st, pad, dil), out_dim(W, k, st, pad, dil)
    K, P = Cin * k * k, oH * oW
    per = Cin * H * W
    x = _own_index_tensor(N, Cin, H, W)
    want_map = oracle.im2col_index_range(0, N * K * P, Cin, H, W, k, k, st, st, pad, pad, dil, dil).reshape(N, K, P)
    sample_base = (np.arange(N, dtype=np.int64) * per).reshape(N, 1, 1)
    want_val = np.where(want_map >= 0, want_map - sample_base + 1, 0)
    for first in range(0, K, Cout):
        taps = np.arange(first, min(first + Cout, K))
        w = np.zeros((Cout, K), np.float32)
        w[np.arange(len(taps)), taps] = 1.0
        y = conv_forward(x, w.reshape(Cout, Cin, k, k), None, stride=(st, st), pad=(pad, pad), dil=(dil, dil))
        y = y.reshape(N, Cout, P)
        assert np.array_equal(y[:, :len(taps)].astype(np.int64), want_val[:, taps]), first
        assert not y[:, len(taps):].any()


def test_config3_full_size_properties_and_sampled_oracle(oracle):
    # N = 128 images of 3x32x32 through both layers; the scalar oracle covers a few samples, the
    # adjoint identities <conv(x,w), g> = <x, dgrad(g)> = <w, wgrad(x,g)> cover the whole batch.
    N = 128
    x = refdata.normal(31, (N, 3, 32, 32))
    w1, w2 = refdata.conv_weight(3, 64, 3), refdata.conv_weight(64, 128, 3)
    y1 = conv_forward(x, w1, np.zeros(64, np.float32), pad=(1, 1))
    y2 = conv_forward(y1, w2, np.zeros(128, np.float32), pad=(1, 1))
    for n in (0, 127):
        assert rel_err(y1[n:n + 1], oracle.conv2d_forward(x[n:n + 1], w1, None, pad=(1, 1))) < FP32_TOL
    assert rel_err(y2[5:6], oracle.conv2d_forward(y1[5:6], w2, None, pad=(1, 1))) < FP32_TOL
    for xin, w, y in ((x, w1, y1), (y1, w2, y2)):
        g = refdata.normal(77, y.shape)
        gi, gw, gb = conv_backward(xin, w, g, pad=(1, 1))
        lhs = float(np.vdot(y.astype(np.float64), g.astype(np.float64)))
        assert abs(float(np.vdot(xin.astype(np.float64), gi.astype(np.float64))) - lhs) < 1e-5 * abs(lhs) + 1e-3
        assert abs(float(np.vdot(w.astype(np.float64), gw.astype(np.float64))) - lhs) < 1e-5 * abs(lhs) + 1e-3
        assert rel_err(gb, g.astype(np.float64).sum(axis=(0, 2, 3))) < FP32_TOL
        # sampled oracle for the gradients: two samples' worth of dgrad; wgrad of a 2-sample sub-batch
        oi, _, _ = oracle.conv2d_backward(xin[3:5], w, g[3:5], pad=(1, 1))
        assert rel_err(gi[3:5], oi) < FP32_TOL
        _, gw2, gb2 = conv_backward(xin[3:5], w, g[3:5], pad=(1, 1))
        _, ow2, ob2 = oracle.conv2d_backward(xin[3:5], w, g[3:5], pad=(1, 1))
        assert rel_err(gw2, ow2) < FP32_TOL
        assert rel_err(gb2, ob2) < FP32_TOL


def test_conv_argument_errors():
    t = torch.zeros(16, device="cuda")
    args = [ptr(t), ptr(t), None, ptr(t), 1, 1, 2, 2, 1, 1, 1, 1, 1, 0, 0, 1, 1, 0]
    assert lib.tfb_conv2d_forward(*args, 3, stream_ptr()) == -2   # Int32: not a dtype of this path
    bad = list(args)
    bad[11] = 0  # stride_h
    assert lib.tfb_conv2d_forward(*bad, capi.DTYPE_F32, stream_ptr()) == -1
    assert lib.tfb_conv2d_forward(None, ptr(t), None, ptr(t), *args[4:], capi.DTYPE_F32, stream_ptr()) == -1


def test_empty_batch(feed):
    # N = 0: nothing to compute; the weight and bias gradients of an empty batch are zeros
    t = torch.full((64,), float("nan"), device="cuda")
    gw, gb = torch.full((2 * 3 * 9,), float("nan"), device="cuda"), torch.full((2,), float("nan"), device="cuda")
    args = [0, 3, 8, 8, 2, 3, 3, 1, 1, 1, 1, 1, 1]
    capi.check(lib.tfb_conv2d_forward(ptr(t), ptr(t), None, ptr(t), *args, 0, capi.DTYPE_F32, stream_ptr()))
    capi.check(lib.tfb_conv2d_backward(ptr(t), ptr(t), ptr(t), ptr(t), ptr(gw), ptr(gb), *args, capi.DTYPE_F32,
                                       stream_ptr()))
    assert_device_ok()
    assert float(gw.abs().sum()) == 0.0 and float(gb.abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [capi.DTYPE_BF16, capi.DTYPE_F16])
@pytest.mark.parametrize("case", [(4, 16, 12, 12, 32, 3, (1, 1), (1, 1)), (2, 3, 17, 15, 8, 3, (2, 1), (1, 0)),
                                  (3, 64, 16, 16, 64, 3, (1, 1), (1, 1))])
def test_16bit_tensors_forward_and_backward(oracle, dtype, case):
    # The reference launchers' dtype surface (cuda/kernels/im2col.cu:124-157): tensors of the 16-bit type,
    # FP32 accumulation, results rounded to the tensor type. Oracle on the rounded inputs, 1e-2 budget.
    N, C, H, W, Cout, k, stride, pad = case
    tdt = torch.bfloat16 if dtype == capi.DTYPE_BF16 else torch.float16
    rnd = lambda a: torch.from_numpy(a).to(tdt).float().numpy()
    x, w = rnd(refdata.normal(1, (N, C, H, W))), rnd(refdata.conv_weight(C, Cout, k))
    b = refdata.normal(2, (Cout,)) * np.float32(0.1)
    oH, oW = out_dim(H, k, stride[0], pad[0], 1), out_dim(W, k, stride[1], pad[1], 1)
    g = rnd(refdata.normal(3, (N, Cout, oH, oW)))
    X, Wt, G, B = dev(x, tdt), dev(w, tdt), dev(g, tdt), dev(b)
    y = torch.full((N, Cout, oH, oW), float("nan"), device="cuda", dtype=tdt)
    args = (N, C, H, W, Cout, k, k, stride[0], stride[1], pad[0], pad[1], 1, 1)
    capi.check(lib.tfb_conv2d_forward(ptr(X), ptr(Wt), ptr(B), ptr(y), *args, 0, dtype, stream_ptr()))
    gi = torch.full(x.shape, float("nan"), device="cuda", dtype=tdt)
    gw = torch.full(w.shape, float("nan"), device="cuda", dtype=tdt)
    gb = torch.full((Cout,), float("nan"), device="cuda")
    capi.check(lib.tfb_conv2d_backward(ptr(X), ptr(Wt), ptr(G), ptr(gi), ptr(gw), ptr(gb), *args, dtype, stream_ptr()))
    assert_device_ok()
    tol = 1e-2
    assert rel_err(y.float().cpu().numpy(), oracle.conv2d_forward(x, w, b, stride, pad, (1, 1))) < tol
    oi, ow, ob = oracle.conv2d_backward(x, w, g, stride, pad, (1, 1))
    assert rel_err(gi.float().cpu().numpy(), oi) < tol
    assert rel_err(gw.float().cpu().numpy(), ow) < tol
    assert rel_err(gb.cpu().numpy(), ob) < tol
