"""Parity of nn::Linear forward/backward, the loss kernels, SGD and the MLP step with the oracle and
with the golden outputs of the unmodified reference."""
import ctypes

import numpy as np
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from golden.make_golden import LINEAR_DW_ROWS
from gpu_util import assert_device_ok, dev, lib, ptr, rel_err, stream_ptr

pytestmark = pytest.mark.gpu
FP32_TOL = 1e-5
BF16_TOL = 1e-2


@pytest.fixture(autouse=True, params=["small_products_on_cuda_cores", "tensor_cores_only"])
def product_path(request):
    """FP32 products with few rows and a long contraction run on the one-launch CUDA-core kernel by default;
    the tests run a second time with that knob off, so that the tensor-core path keeps seeing those shapes.
    Tests that only hold large products are not repeated."""
    large_only = ("test_square_sweep", "test_config1", "test_split_k_shapes", "test_matmul_on_host_buffers")
    if request.param == "tensor_cores_only" and request.node.name.startswith(large_only):
        pytest.skip("large products take the tensor-core path either way")
    old = ctypes.c_int(0)
    capi.check(lib.tfb_get_tuning(capi.TUNE_SMALL_GEMM, ctypes.byref(old)))
    capi.check(lib.tfb_set_tuning(capi.TUNE_SMALL_GEMM, 1 if request.param == "small_products_on_cuda_cores" else 0))
    yield request.param
    capi.check(lib.tfb_set_tuning(capi.TUNE_SMALL_GEMM, old.value))


def linear_fwd_bwd(x, w, b, g, relu, dtype=capi.DTYPE_F32):
    tdt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[dtype]
    batch, in_f = x.shape
    out_f = w.shape[0]
    X, W, G = dev(x, tdt), dev(w, tdt), dev(g, tdt)
    B = dev(b) if b is not None else None
    Y = torch.full((batch, out_f), float("nan"), device="cuda", dtype=tdt)
    capi.check(lib.tfb_linear_forward(ptr(X), ptr(W), ptr(B), ptr(Y), batch, in_f, out_f, int(relu), dtype, stream_ptr()))
    dX = torch.full((batch, in_f), float("nan"), device="cuda", dtype=tdt)
    dW = torch.full((out_f, in_f), float("nan"), device="cuda", dtype=tdt)
    db = torch.full((out_f,), float("nan"), device="cuda")
    capi.check(lib.tfb_linear_backward(ptr(X), ptr(W), ptr(Y), ptr(G), ptr(dX), ptr(dW), ptr(db), batch, in_f, out_f,
                                       int(relu), dtype, stream_ptr()))
    assert_device_ok()
    return [t.float().cpu().numpy() for t in (Y, dX, dW, db)]


def test_config2_against_reference_golden(oracle, golden):
    # X 64x784 normalised pixels, W from the reference's Linear(784, 256), bias zeros, ReLU, dY ~ N(0,1)
    w = refdata.linear_weight(784, 256)
    x, g = refdata.mnist_like(21, (64, 784)), refdata.normal(22, (64, 256))
    Y, dX, dW, db = linear_fwd_bwd(x, w, np.zeros(256, np.float32), g, relu=True)
    assert rel_err(Y, golden["linear_c2_Y"]) < FP32_TOL
    # the ReLU mask must be the reference's wherever the pre-activation is not within rounding of zero
    gy = golden["linear_c2_Y"]
    assert ((Y > 0) != (gy > 0)).sum() <= 2
    assert rel_err(dX, golden["linear_c2_dX"]) < 5e-5 if ((Y > 0) != (gy > 0)).any() else rel_err(dX, golden["linear_c2_dX"]) < FP32_TOL
    assert rel_err(dW[LINEAR_DW_ROWS], golden["linear_c2_dW_rows"]) < FP32_TOL
    assert rel_err(dW.astype(np.float64).sum(axis=1), golden["linear_c2_dW_rowsum"]) < FP32_TOL
    _, _, odb = oracle.linear_backward(x, w, gy, g, relu=True)
    assert rel_err(db, odb) < FP32_TOL


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("shape", [(64, 784, 256), (33, 50, 10), (256, 1024, 10), (200, 10, 300), (1, 7, 3)])
def test_linear_with_bias_against_oracle(oracle, shape, relu):
    batch, in_f, out_f = shape
    x, w = refdata.normal(1, (batch, in_f)), refdata.linear_weight(in_f, out_f)
    b, g = refdata.normal(2, (out_f,)) * np.float32(0.1), refdata.normal(3, (batch, out_f))
    Y, dX, dW, db = linear_fwd_bwd(x, w, b, g, relu)
    oy = oracle.linear_forward(x, w, b, relu)
    assert rel_err(Y, oy) < FP32_TOL
    # use the device's own mask for the backward oracle so a sign flip at |pre-activation| ~ 1e-7
    # cannot turn into a spurious mismatch
    odx, odw, odb = oracle.linear_backward(x, w, Y, g, relu)
    assert rel_err(dX, odx) < FP32_TOL
    assert rel_err(dW, odw) < FP32_TOL
    assert rel_err(db, odb) < FP32_TOL


@pytest.mark.parametrize("shape", [(64, 784, 256), (33, 50, 10), (4096, 1024, 1024), (200, 10, 300)])
def test_linear_backward_on_saved_planes_is_bit_identical(shape):
    # forward product and backward on hi / lo planes the caller made once == the unsplit entry points
    batch, in_f, out_f = shape
    x, w = refdata.normal(1, (batch, in_f)), refdata.linear_weight(in_f, out_f)
    b, g = refdata.normal(2, (out_f,)) * np.float32(0.1), refdata.normal(3, (batch, out_f))
    Y0, dX0, dW0, db0 = linear_fwd_bwd(x, w, b, g, relu=True)
    X, W, G, B = dev(x), dev(w), dev(g), dev(b)
    ld = (in_f + 3) // 4 * 4
    xs = torch.full((2, batch, ld), float("nan"), device="cuda")
    ws = torch.full((2, out_f, ld), float("nan"), device="cuda")
    capi.check(lib.tfb_split_tf32(ptr(X), batch, in_f, in_f, ptr(xs[0]), ptr(xs[1]), ld, stream_ptr()))
    capi.check(lib.tfb_split_tf32(ptr(W), out_f, in_f, in_f, ptr(ws[0]), ptr(ws[1]), ld, stream_ptr()))
    Y = torch.full((batch, out_f), float("nan"), device="cuda")
    capi.check(lib.tfb_gemm_presplit(ptr(xs[0]), ptr(xs[1]), ptr(ws[0]), ptr(ws[1]), ptr(Y), batch, out_f, in_f, ld, ld,
                                     out_f, 0, 1, ptr(B), capi.EPI_BIAS_COL | capi.EPI_RELU, stream_ptr()))
    dX = torch.full((batch, in_f), float("nan"), device="cuda")
    dW = torch.full((out_f, in_f), float("nan"), device="cuda")
    db = torch.full((out_f,), float("nan"), device="cuda")
    capi.check(lib.tfb_linear_backward_presplit(ptr(xs[0]), ptr(xs[1]), ld, ptr(ws[0]), ptr(ws[1]), ld, ptr(Y), ptr(G),
                                                ptr(dX), ptr(dW), ptr(db), batch, in_f, out_f, 1, stream_ptr()))
    assert_device_ok()
    for got, want in ((Y, Y0), (dX, dX0), (dW, dW0), (db, db0)):
        assert np.array_equal(got.cpu().numpy(), want)
    # only the gradient that is asked for needs its operand
    capi.check(lib.tfb_linear_backward_presplit(None, None, 0, ptr(ws[0]), ptr(ws[1]), ld, ptr(Y), ptr(G), ptr(dX),
                                                None, None, batch, in_f, out_f, 1, stream_ptr()))
    assert_device_ok()
    assert np.array_equal(dX.cpu().numpy(), dX0)
    assert lib.tfb_linear_backward_presplit(None, None, 0, ptr(ws[0]), ptr(ws[1]), ld, ptr(Y), ptr(G), ptr(dX),
                                            ptr(dW), None, batch, in_f, out_f, 1, stream_ptr()) == -1   # TFB_ERR_INVALID_ARG: dW asked for without the planes of X


@pytest.mark.parametrize("dtype", [capi.DTYPE_BF16, capi.DTYPE_F16])
def test_linear_16bit(oracle, dtype):
    batch, in_f, out_f = 64, 784, 256
    tdt = torch.bfloat16 if dtype == capi.DTYPE_BF16 else torch.float16
    rnd = lambda a: torch.from_numpy(a).to(tdt).float().numpy()
    x, w, g = rnd(refdata.normal(1, (batch, in_f))), rnd(refdata.linear_weight(in_f, out_f)), rnd(refdata.normal(3, (batch, out_f)))
    b = refdata.normal(2, (out_f,)) * np.float32(0.1)
    Y, dX, dW, db = linear_fwd_bwd(x, w, b, g, True, dtype)
    assert rel_err(Y, oracle.linear_forward(x, w, b, True)) < BF16_TOL
    odx, odw, odb = oracle.linear_backward(x, w, Y, g, True)
    assert rel_err(dX, odx) < BF16_TOL
    assert rel_err(dW, odw) < BF16_TOL
    assert rel_err(db, odb) < BF16_TOL


def test_log_softmax_nll_and_sgd(oracle, golden):
    z = refdata.normal(41, (32, 10)) * np.float32(3.0)
    lab = refdata.labels(43, 32)
    Z, L = dev(z), torch.from_numpy(lab).cuda()
    dz = torch.empty_like(Z)
    loss = torch.zeros(1, device="cuda")
    capi.check(lib.tfb_log_softmax_nll(ptr(Z), ptr(L), ptr(dz), ptr(loss), 32, 10, 32, stream_ptr()))
    assert_device_ok()
    ol, odz = oracle.nll_mean(z, lab)
    assert abs(float(loss.item()) - ol) <= 1e-6 * abs(ol)
    assert rel_err(dz.cpu().numpy(), odz) < 1e-6
    # the implied log_softmax equals the reference's golden output: dz = (exp(lsm) - onehot) / N
    lsm = golden["log_softmax_32x10"]
    onehot = np.eye(10, dtype=np.float32)[lab]
    assert rel_err(dz.cpu().numpy(), (np.exp(lsm) - onehot) / 32) < 1e-6
    # data-parallel scaling: half the rows with global_rows = 32 gives the same per-row gradients
    capi.check(lib.tfb_log_softmax_nll(ptr(Z), ptr(L), ptr(dz), ptr(loss), 16, 10, 32, stream_ptr()))
    assert rel_err(dz[:16].cpu().numpy(), odz[:16]) < 1e-6
    # SGD with momentum: same IEEE operations as the host formula, bit for bit
    p, v, g = refdata.normal(1, (100003,)), refdata.normal(2, (100003,)), refdata.normal(3, (100003,))
    P, V, G = dev(p), dev(v), dev(g)
    capi.check(lib.tfb_sgd_momentum(ptr(P), ptr(V), ptr(G), p.size, 0.1, 0.9, 1.0, stream_ptr()))
    assert_device_ok()
    op, ov = oracle.sgd_momentum(p, v, g, 0.1, 0.9)
    assert np.array_equal(V.cpu().numpy(), ov)
    assert np.array_equal(P.cpu().numpy(), op)


def local_loss(m):
    """This rank's loss contribution: the slot behind the flat gradients."""
    return float(m.grads_and_loss[m.numel].item())


def test_mlp_step_against_reference_golden_and_oracle(oracle, golden):
    from tensors_b200.mlp import MLP
    dims = (784, 64, 48, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb, lab = refdata.mnist_like(42, (32, 784)), refdata.labels(43, 32)
    m = MLP(dims, ws, max_rows=32)
    m.forward_backward(dev(xb), torch.from_numpy(lab).cuda())
    assert_device_ok()
    assert abs(local_loss(m) - float(golden["mlp_loss"][0])) < 1e-5
    assert rel_err(m.weight(2, m.grads).cpu().numpy(), golden["mlp_dW3"]) < 2e-5
    assert rel_err(m.weight(1, m.grads).cpu().numpy(), golden["mlp_dW2"]) < 2e-5
    assert rel_err(m.weight(0, m.grads).cpu().numpy()[[0, 7, 63]], golden["mlp_dW1_rows"]) < 2e-5


def test_mlp_step_config5_shapes_reduced_batch(oracle):
    # 784 -> 1024 -> 1024 -> 10 at batch 256 (the named configuration uses 8192 rows), then one SGD step
    from tensors_b200.mlp import MLP
    dims = (784, 1024, 1024, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb, lab = refdata.mnist_like(7, (256, 784)), refdata.labels(8, 256)
    m = MLP(dims, ws, max_rows=256)
    p0 = m.params.clone()
    m.train_step(dev(xb), torch.from_numpy(lab).cuda(), lr=0.1, momentum=0.9)
    assert_device_ok()
    ol, odw, odb = oracle.mlp_grads(xb, lab, ws, bs=[np.zeros(d, np.float32) for d in dims[1:]])
    assert abs(float(m.loss.item()) - ol) < 1e-5
    for i in range(3):
        assert rel_err(m.weight(i, m.grads).cpu().numpy(), odw[i]) < 2e-5, i
        assert rel_err(m.bias(i, m.grads).cpu().numpy(), odb[i]) < 2e-5, i
    # velocity starts at zero: v1 = g, p1 = p0 - lr * g — the host formula, bit for bit
    op, ov = oracle.sgd_momentum(p0.cpu().numpy(), np.zeros(m.numel, np.float32), m.grads.cpu().numpy(), 0.1, 0.9)
    assert np.array_equal(m.velocity.cpu().numpy(), ov)
    assert np.array_equal(m.params.cpu().numpy(), op)


def test_mlp_graph_replay_matches_eager_steps(oracle):
    # five eager steps and two eager + three replays of the captured step must walk the same trajectory
    from tensors_b200.mlp import MLP
    dims = (784, 128, 64, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    X, L = dev(refdata.mnist_like(7, (512, 784))), torch.from_numpy(refdata.labels(8, 512)).cuda()
    eager = MLP(dims, ws, max_rows=512)
    for _ in range(5):
        eager.train_step(X, L, lr=0.1, momentum=0.9)
    graphed = MLP(dims, ws, max_rows=512)
    replay = graphed.capture_train_step(X, L, lr=0.1, momentum=0.9, warmup=2)   # 2 eager + 1 captured (not run)
    for _ in range(3):
        replay()
    assert_device_ok()
    assert torch.equal(eager.params, graphed.params)
    assert float(eager.loss.item()) == float(graphed.loss.item())


def test_mlp_steps_do_not_depend_on_programmatic_dependent_launch():
    # With the PDL knob on (default) every kernel of the step may start while its predecessor is still
    # finishing and waits inside the kernel instead; the trajectory must be bit-identical to plain stream order.
    import ctypes
    from tensors_b200.mlp import MLP
    dims = (784, 256, 192, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    X, L = dev(refdata.mnist_like(7, (1024, 784))), torch.from_numpy(refdata.labels(8, 1024)).cuda()
    old = ctypes.c_int(0)
    capi.check(lib.tfb_get_tuning(capi.TUNE_PDL, ctypes.byref(old)))
    out = {}
    try:
        for pdl in (1, 0):
            capi.check(lib.tfb_set_tuning(capi.TUNE_PDL, pdl))
            m = MLP(dims, ws, max_rows=1024)
            for _ in range(4):
                m.train_step(X, L, lr=0.1, momentum=0.9)
            replay = m.capture_train_step(X, L, lr=0.1, momentum=0.9, warmup=1)
            for _ in range(3):
                replay()
            assert_device_ok()
            out[pdl] = (m.params.clone(), float(m.loss.item()))
    finally:
        capi.check(lib.tfb_set_tuning(capi.TUNE_PDL, old.value))
    assert torch.equal(out[0][0], out[1][0])
    assert out[0][1] == out[1][1]


def test_mlp_step_with_operands_as_their_own_hi_planes(oracle):
    # The step keeps the batch, the parameters and the hidden activations as their own hi planes and
    # writes lo planes only (knob RAW_HI, default off). With the knob off it writes round-to-nearest
    # hi / lo pairs. Both must give the oracle's loss and gradients; they need not agree bit for bit.
    import ctypes
    from tensors_b200.mlp import MLP
    dims = (784, 256, 192, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    x, lab = refdata.mnist_like(17, (1500, 784)), refdata.labels(18, 1500)
    X, L = dev(x), torch.from_numpy(lab).cuda()
    ol, odw, odb = oracle.mlp_grads(x, lab, ws, bs=[np.zeros(d, np.float32) for d in dims[1:]])
    old = ctypes.c_int(0)
    capi.check(lib.tfb_get_tuning(capi.TUNE_RAW_HI, ctypes.byref(old)))
    try:
        for raw in (1, 0):
            capi.check(lib.tfb_set_tuning(capi.TUNE_RAW_HI, raw))
            m = MLP(dims, ws, max_rows=1500)
            m.forward_backward(X, L)
            assert_device_ok()
            assert abs(local_loss(m) - ol) < 1e-5, raw
            # the head: no ReLU mask behind it, so no ties
            assert rel_err(m.weight(2, m.grads).cpu().numpy(), odw[2]) < 2e-5, raw
            assert rel_err(m.bias(2, m.grads).cpu().numpy(), odb[2]) < 2e-5, raw
            for i in (0, 1):   # hidden layers: a unit at a ReLU tie may move one row (see the invariance test)
                got = m.weight(i, m.grads).cpu().numpy()
                rows = np.linalg.norm(got - odw[i], axis=1) / (np.linalg.norm(odw[i], axis=1) + 1e-30)
                assert int((rows > 5e-5).sum()) <= 2, (raw, i, np.sort(rows)[-4:])
    finally:
        capi.check(lib.tfb_set_tuning(capi.TUNE_RAW_HI, old.value))


def test_deep_mlp_finishes_every_bias_gradient_in_batches():
    # Eleven layers: the final additions of the loss and of the bias gradients run as batched launches of at
    # most eight reductions each, so this step needs two of them. Checked against a float64 autograd walk of
    # the same network (no reference counterpart has this depth); widths are small, so a ReLU tie is
    # improbable, and the tolerance would still tell a missing layer (its bias gradient would be zero or stale).
    from tensors_b200.mlp import MLP
    dims = (40, 36, 36, 32, 32, 28, 28, 24, 24, 20, 16, 10)
    L = len(dims) - 1
    rng = np.random.default_rng(5)
    ws = [(rng.standard_normal((dims[i + 1], dims[i])) * np.sqrt(2.0 / dims[i])).astype(np.float32) for i in range(L)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.1).astype(np.float32) for i in range(L)]
    x = rng.standard_normal((96, dims[0])).astype(np.float32)
    lab = rng.integers(0, dims[-1], 96).astype(np.int64)
    m = MLP(dims, ws, biases=bs, max_rows=96)
    m.forward_backward(dev(x), torch.from_numpy(lab).cuda())
    assert_device_ok()
    tw = [torch.tensor(w, dtype=torch.float64, requires_grad=True) for w in ws]
    tb = [torch.tensor(b, dtype=torch.float64, requires_grad=True) for b in bs]
    h = torch.tensor(x, dtype=torch.float64)
    for i in range(L):
        h = h @ tw[i].T + tb[i]
        if i < L - 1:
            h = torch.relu(h)
    loss = torch.nn.functional.cross_entropy(h, torch.from_numpy(lab))
    loss.backward()
    assert abs(local_loss(m) - float(loss)) < 1e-5
    for i in range(L):
        assert rel_err(m.bias(i, m.grads).cpu().numpy(), tb[i].grad.numpy()) < 1e-4, i
        assert rel_err(m.weight(i, m.grads).cpu().numpy(), tw[i].grad.numpy()) < 1e-4, i


def test_mlp_full_batch_data_parallel_invariance(oracle):
    # The named configuration at its full global batch of 8192 rows. The batch is cut into G row shards
    # as G data-parallel ranks would hold them; each shard's gradient is scaled by the GLOBAL batch, so
    # the shard gradients must add up to the one-rank gradient for every G, and the shard losses to the
    # full-batch loss, up to FP32 summation order. One caveat is inherent to ReLU: a hidden unit whose
    # pre-activation is zero to within rounding noise can land on either side of the mask when the
    # product that computes it is tiled differently, and a single such tie moves a 1024 x 1024 weight
    # gradient by ~5e-4 of its norm (its entries are sums of thousands of cancelling terms). So: the loss
    # and the last layer's gradients (no mask behind them) must agree to FP32 noise; the hidden layers'
    # must agree to a few ties' worth, and the ties are counted and checked to be exactly that.
    from tensors_b200.mlp import MLP, shard_rows
    dims, batch = (784, 1024, 1024, 10), 8192
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb, lab = refdata.mnist_like(7, (batch, 784)), refdata.labels(8, batch)
    X, L = dev(xb), torch.from_numpy(lab).cuda()
    full = MLP(dims, ws, max_rows=batch)
    full.forward_backward(X, L)
    assert_device_ok()
    g1, loss1 = full.grads.clone(), local_loss(full)
    hidden1 = [a.clone() for a in full._acts[1:3]]
    assert np.isfinite(loss1) and 2.0 < loss1 < 2.7   # ten classes, small random weights: about ln 10
    for G in (2, 4, 8):
        total, loss, ties = torch.zeros_like(g1), 0.0, 0
        m = MLP(dims, ws, max_rows=batch // G + 1)
        for r in range(G):
            b, e = shard_rows(batch, r, G)
            m.forward_backward(X[b:e], L[b:e], global_rows=batch)
            total += m.grads
            loss += local_loss(m)
            for h_full, h_shard in zip(hidden1, m._acts[1:3]):
                flipped = (h_full[b:e] > 0) != (h_shard > 0)
                ties += int(flipped.sum())
                if flipped.any():   # only values at rounding-noise level may change sides
                    assert float(torch.maximum(h_full[b:e], h_shard)[flipped].max()) < 1e-5
        assert_device_ok()
        assert abs(loss - loss1) < 1e-5, G
        assert ties <= 64, (G, ties)
        assert float((full.weight(2, total) - full.weight(2, g1)).norm() / full.weight(2, g1).norm()) < 1e-5, G
        assert float((full.bias(2, total) - full.bias(2, g1)).norm() / full.bias(2, g1).norm()) < 1e-5, G
        bound = 1e-5 + 1e-3 * ties
        assert float((total - g1).norm() / g1.norm()) < bound, (G, ties)
    # sampled oracle: the first 64 rows as one rank's shard of the global batch
    sub = MLP(dims, ws, max_rows=64)
    sub.forward_backward(X[:64], L[:64], global_rows=batch)
    ol, odw, _ = oracle.mlp_grads(xb[:64], lab[:64], ws, bs=[np.zeros(d, np.float32) for d in dims[1:]],
                                  global_rows=batch)
    assert abs(local_loss(sub) - ol) < 1e-6
    assert rel_err(sub.weight(2, sub.grads).cpu().numpy(), odw[2]) < 2e-5
