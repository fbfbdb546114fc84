"""Pins the C restatement (oracle/oracle.c) to the reference: known answers from the reference's
own tests, outputs of the unmodified reference stored under tests/golden/, and — when
oracle/_ref/libtf_ref.so is present — the reference itself run live. CPU only."""
import numpy as np
import pytest

import refdata
from golden.make_golden import CONV_CHANNELS_L1, CONV_CHANNELS_L2, LINEAR_DW_ROWS


# ---- known answers written in the reference's tests ---------------------------------------
def test_known_answer_2x2(oracle):
    # cuda/kernels/gemm_naive_test.cpp:100-116
    c = oracle.matmul(np.array([[1, 2], [3, 4]]), np.array([[5, 6], [7, 8]]), mt=False)
    assert c.tolist() == [[19.0, 22.0], [43.0, 50.0]]


def test_known_answer_identity(oracle):
    # cuda/kernels/gemm_naive_test.cpp:118-144
    a = np.arange(1, 17, dtype=np.float32).reshape(4, 4)
    assert np.array_equal(oracle.matmul(a, np.eye(4)), a)


def test_known_answer_arange_grads(oracle):
    # autograd/ops/autograd_all_ops_test.cpp:281-328
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.arange(6, dtype=np.float32).reshape(3, 2)
    assert oracle.matmul(a, b).tolist() == [[10.0, 13.0], [28.0, 40.0]]
    da, db = oracle.matmul_backward(a, b, np.ones((2, 2)))
    assert da.tolist() == [[1.0, 5.0, 9.0], [1.0, 5.0, 9.0]]
    assert db.tolist() == [[3.0, 3.0], [5.0, 5.0], [7.0, 7.0]]


def test_known_answer_ones_grads(oracle):
    # autograd/ops/autograd_all_ops_test.cpp:253-268: ones(2,2)·ones(2,2), grads are all 2
    one = np.ones((2, 2), np.float32)
    da, db = oracle.matmul_backward(one, one, one)
    assert np.all(da == 2.0) and np.all(db == 2.0)


def test_known_answer_conv_1x1(oracle):
    # nn/conv2d_forward_test.cpp:112-137, nn/conv2d_backward_test.cpp:110-160
    x = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2)
    w = np.array([2.0], np.float32).reshape(1, 1, 1, 1)
    assert oracle.conv2d_forward(x, w, None).ravel().tolist() == [2.0, 4.0, 6.0, 8.0]
    go = np.array([0.1, 0.2, 0.3, 0.4], np.float32).reshape(1, 1, 2, 2)
    gi, gw, gb = oracle.conv2d_backward(x, w, go)
    np.testing.assert_allclose(gi.ravel(), [0.2, 0.4, 0.6, 0.8], rtol=1e-6)
    np.testing.assert_allclose(gw.ravel(), [3.0], rtol=1e-6)


def test_conv_backward_matches_textbook_scatter(oracle):
    # The host reference of nn/conv2d_backward_test.cpp:50-106, on that file's multi-channel case
    # (Cin=2, Cout=3, 3x3, pad 1) and its 2x2 two-sample case.
    def textbook(x, w, go, s, p, d):
        N, Cin, H, W = x.shape
        Cout, _, kH, kW = w.shape
        oH, oW = go.shape[2:]
        gi = np.zeros_like(x, dtype=np.float64)
        gw = np.zeros_like(w, dtype=np.float64)
        for n in range(N):
            for co in range(Cout):
                for oh in range(oH):
                    for ow in range(oW):
                        g = float(go[n, co, oh, ow])
                        for ci in range(Cin):
                            for ki in range(kH):
                                for kj in range(kW):
                                    ih, iw = oh * s + ki * d - p, ow * s + kj * d - p
                                    if 0 <= ih < H and 0 <= iw < W:
                                        gi[n, ci, ih, iw] += g * float(w[co, ci, ki, kj])
                                        gw[co, ci, ki, kj] += g * float(x[n, ci, ih, iw])
        return gi, gw, go.astype(np.float64).sum(axis=(0, 2, 3))

    f = np.float32
    w = (f(0.02) * ((np.arange(3 * 2 * 9) % 7) + 1).astype(f)).reshape(3, 2, 3, 3)
    x = (f(0.05) * ((np.arange(2 * 16) % 5) + 1).astype(f)).reshape(1, 2, 4, 4)
    go = (f(0.01) * ((np.arange(3 * 16) % 13) + 1).astype(f)).reshape(1, 3, 4, 4)
    gi, gw, gb = oracle.conv2d_backward(x, w, go, pad=(1, 1))
    ti, tw, tb = textbook(x, w, go, 1, 1, 1)
    np.testing.assert_allclose(gi, ti, rtol=1e-5)
    np.testing.assert_allclose(gw, tw, rtol=1e-5)
    np.testing.assert_allclose(gb, tb, rtol=1e-5)
    w = np.arange(1, 9, dtype=f).reshape(2, 1, 2, 2)
    x = (f(0.1) * np.arange(1, 19, dtype=f)).reshape(2, 1, 3, 3)
    go = (f(0.01) * ((np.arange(16) % 11) + 1).astype(f)).reshape(2, 2, 2, 2)
    gi, gw, gb = oracle.conv2d_backward(x, w, go)
    ti, tw, tb = textbook(x, w, go, 1, 0, 1)
    np.testing.assert_allclose(gi, ti, rtol=1e-5)
    np.testing.assert_allclose(gw, tw, rtol=1e-5)
    np.testing.assert_allclose(gb, tb, rtol=1e-5)


def test_im2col_matches_test_host_reference(oracle):
    # ref_im2col of cuda/kernels/im2col_test.cpp:75-107, restated in numpy, on strided / dilated cases.
    def host(x, kH, kW, sh, sw, ph, pw, dh, dw):
        N, C, H, W = x.shape
        oH = (H + 2 * ph - dh * (kH - 1) - 1) // sh + 1
        oW = (W + 2 * pw - dw * (kW - 1) - 1) // sw + 1
        col = np.zeros((N, C * kH * kW, oH * oW), np.float32)
        for n in range(N):
            for c in range(C):
                for ki in range(kH):
                    for kj in range(kW):
                        for oh in range(oH):
                            for ow in range(oW):
                                ih, iw = oh * sh + ki * dh - ph, ow * sw + kj * dw - pw
                                if 0 <= ih < H and 0 <= iw < W:
                                    col[n, (c * kH + ki) * kW + kj, oh * oW + ow] = x[n, c, ih, iw]
        return col

    x = refdata.normal(5, (2, 3, 7, 6))
    for args in [(3, 3, 1, 1, 1, 1, 1, 1), (2, 3, 2, 1, 0, 2, 1, 2), (3, 2, 1, 2, 2, 0, 2, 1)]:
        assert np.array_equal(oracle.im2col(x, *args), host(x, *args))


# ---- golden outputs of the unmodified reference ------------------------------------------------
def test_golden_gemm_patterns(oracle, golden):
    for name, a, b in refdata.gemm_test_patterns():
        assert np.array_equal(oracle.matmul(a, b, mt=False), golden[f"gemm_{name}"]), name
        assert np.array_equal(oracle.matmul(a, b, mt=True), golden[f"gemm_{name}"]), name


def test_golden_matmul_and_backward(oracle, golden):
    a, b, g = refdata.uniform(11, (96, 112)), refdata.uniform(12, (112, 80)), refdata.normal(13, (96, 80))
    assert np.array_equal(oracle.matmul(a, b), golden["matmul_96x112x80"])
    da, db = oracle.matmul_backward(a, b, g)
    assert np.array_equal(da, golden["matmul_bwd_dA"])
    assert np.array_equal(db, golden["matmul_bwd_dB"])
    assert golden["matmul_arange_C"].tolist() == [[10.0, 13.0], [28.0, 40.0]]
    assert golden["matmul_arange_dA"].tolist() == [[1.0, 5.0, 9.0], [1.0, 5.0, 9.0]]


def test_golden_kaiming_weights(golden):
    w = refdata.linear_weight(784, 256)
    assert np.array_equal(w.ravel()[:64], golden["linear_w_784_256_head"])
    assert np.allclose([w.astype(np.float64).sum(), np.abs(w).astype(np.float64).sum()],
                       golden["linear_w_784_256_sum"], rtol=0, atol=1e-9)
    assert np.abs(w).max() <= np.sqrt(1.0 / 784) + 1e-7
    cw = refdata.conv_weight(64, 128, 3)
    assert np.array_equal(cw.ravel()[:64], golden["conv_w_64_128_3_head"])
    assert np.allclose([cw.astype(np.float64).sum(), np.abs(cw).astype(np.float64).sum()],
                       golden["conv_w_64_128_3_sum"], rtol=0, atol=1e-9)


def test_golden_linear_config2(oracle, golden):
    w = refdata.linear_weight(784, 256)
    x, gy = refdata.mnist_like(21, (64, 784)), refdata.normal(22, (64, 256))
    y = oracle.linear_forward(x, w, None, relu=True)
    assert np.array_equal(y, golden["linear_c2_Y"])
    dx, dw, db = oracle.linear_backward(x, w, y, gy, relu=True)
    assert np.array_equal(dx, golden["linear_c2_dX"])
    assert np.array_equal(dw[LINEAR_DW_ROWS], golden["linear_c2_dW_rows"])
    assert np.array_equal(dw.astype(np.float64).sum(axis=1), golden["linear_c2_dW_rowsum"])
    # bias gradient: no reference implementation; check against the FP64 column sum
    dz = gy * (y > 0)
    np.testing.assert_allclose(db, dz.astype(np.float64).sum(axis=0), rtol=1e-5, atol=1e-5)


def test_golden_conv_forward(oracle, golden):
    x, w1 = refdata.normal(31, (2, 3, 32, 32)), refdata.conv_weight(3, 64, 3)
    y1 = oracle.conv2d_forward(x, w1, None, pad=(1, 1))
    assert np.array_equal(y1[:, CONV_CHANNELS_L1], golden["conv_l1_Y_ch"])
    assert np.array_equal(y1.astype(np.float64).sum(axis=(0, 2, 3)), golden["conv_l1_Y_sum"])
    x2, w2 = refdata.normal(32, (1, 64, 32, 32)), refdata.conv_weight(64, 128, 3)
    y2 = oracle.conv2d_forward(x2, w2, None, pad=(1, 1))
    assert np.array_equal(y2[:, CONV_CHANNELS_L2], golden["conv_l2_Y_ch"])
    assert np.array_equal(y2.astype(np.float64).sum(axis=(0, 2, 3)), golden["conv_l2_Y_sum"])
    xs, ws = refdata.normal(33, (2, 4, 9, 11)), refdata.conv_weight(4, 6, 3)
    assert np.array_equal(oracle.conv2d_forward(xs, ws, None, (2, 2), (2, 2), (2, 2)), golden["conv_s2p2d2_Y"])
    # the im2col + GEMM form (nn/Conv2d.cpp) differs from the direct form only by +0 terms
    y1b = oracle.conv2d_forward(x, w1, None, pad=(1, 1), via_im2col=True)
    assert np.array_equal(y1b, y1)


def test_golden_log_softmax_and_mlp(oracle, golden):
    z = refdata.normal(41, (32, 10)) * np.float32(3.0)
    assert np.array_equal(oracle.log_softmax(z), golden["log_softmax_32x10"])
    dims = (784, 64, 48, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb, lab = refdata.mnist_like(42, (32, 784)), refdata.labels(43, 32)
    loss, dws, dbs = oracle.mlp_grads(xb, lab, ws)
    assert np.float32(loss) == golden["mlp_loss"][0]
    assert np.array_equal(dws[0][[0, 7, 63]], golden["mlp_dW1_rows"])
    assert np.array_equal(dws[0].astype(np.float64).sum(axis=1), golden["mlp_dW1_rowsum"])
    assert np.array_equal(dws[1], golden["mlp_dW2"])
    assert np.array_equal(dws[2], golden["mlp_dW3"])


def test_sgd_momentum_follows_documented_update(oracle):
    # nn/optim/SGD.hpp:3-6; no reference test covers it (parity unpinned): check the formula.
    p, v, g = refdata.normal(1, (1000,)), refdata.normal(2, (1000,)), refdata.normal(3, (1000,))
    p2, v2 = oracle.sgd_momentum(p, v, g, 0.1, 0.9)
    ve = np.float32(0.9) * v + g
    assert np.array_equal(v2, ve)
    assert np.array_equal(p2, p - np.float32(0.1) * ve)


def test_thread_count_does_not_change_results(oracle):
    a, b = refdata.uniform(1, (64, 200)), refdata.uniform(2, (200, 48))
    oracle.lib.orc_set_threads(1)
    c1 = oracle.matmul(a, b)
    oracle.lib.orc_set_threads(0)
    assert np.array_equal(c1, oracle.matmul(a, b))
    rows = [0, 5, 63]
    assert np.array_equal(oracle.matmul_rows(a, b, rows), c1[rows])
    cols = [1, 47]
    assert np.array_equal(oracle.matmul_cols(a, b, cols), c1[:, cols])


def test_bf16_rounding(oracle):
    x = refdata.normal(9, (4096,))
    assert np.array_equal(oracle.round_bf16(x), refdata.from_bf16_bits(refdata.to_bf16_bits(x)))


# ---- the reference itself, live (only where oracle/_ref was built) ---------------------------------
def test_live_reference_matmul_and_backward(oracle, reference):
    a, b, g = refdata.uniform(51, (70, 130)), refdata.uniform(52, (130, 90)), refdata.normal(53, (70, 90))
    assert np.array_equal(oracle.matmul(a, b), reference.matmul(a, b))
    da, db = oracle.matmul_backward(a, b, g)
    ra, rb = reference.matmul_backward(a, b, g)
    assert np.array_equal(da, ra) and np.array_equal(db, rb)


def test_live_reference_linear_conv_mlp(oracle, reference):
    assert np.array_equal(refdata.linear_weight(100, 30), reference.linear_weight(100, 30))
    assert np.array_equal(refdata.conv_weight(3, 64, 3), reference.conv_weight(3, 64, 3))
    w = refdata.linear_weight(100, 30)
    x, g = refdata.mnist_like(54, (16, 100)), refdata.normal(55, (16, 30))
    y, dx, dw = reference.linear_fwd_bwd(x, w, g, relu=True)
    oy = oracle.linear_forward(x, w, None, True)
    odx, odw, _ = oracle.linear_backward(x, w, oy, g, True)
    assert np.array_equal(y, oy) and np.array_equal(dx, odx) and np.array_equal(dw, odw)
    xs, ws = refdata.normal(56, (2, 3, 8, 8)), refdata.conv_weight(3, 5, 3)
    assert np.array_equal(reference.conv2d_forward(xs, ws, 1, 1, 1), oracle.conv2d_forward(xs, ws, None, pad=(1, 1)))
    dims = (40, 24, 16, 10)
    wts = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb, lab = refdata.normal(57, (12, 40)), refdata.labels(58, 12)
    rl, rdw = reference.mlp_grads(xb, lab, wts)
    ol, odw, _ = oracle.mlp_grads(xb, lab, wts)
    assert np.float32(rl) == np.float32(ol)
    assert all(np.array_equal(a, b) for a, b in zip(rdw, odw))
