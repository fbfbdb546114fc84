"""Regenerates tests/golden/reference_outputs.npz from the UNMODIFIED reference.

Needs oracle/_ref/libtf_ref.so (`make -C oracle ref`, which compiles the reference's own CPU
sources from a reference checkout). Inputs come from tests/refdata.py generators, so only the
reference's outputs (sampled where large) are stored. Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import refdata  # noqa: E402
from oracle_lib import Reference  # noqa: E402

# Rows / channels kept from large outputs.
LINEAR_DW_ROWS = [0, 1, 17, 128, 255]
CONV_CHANNELS_L1 = [0, 1, 31, 63]
CONV_CHANNELS_L2 = [0, 64, 127]


def main():
    ref = Reference()
    out = {}

    # --- Tensor::matmul on the reference tests' fill patterns --------------------------------
    for name, a, b in refdata.gemm_test_patterns():
        out[f"gemm_{name}"] = ref.matmul(a, b)

    # --- seeded matmul + MatmulBackward --------------------------------------------------------
    a = refdata.uniform(11, (96, 112))
    b = refdata.uniform(12, (112, 80))
    g = refdata.normal(13, (96, 80))
    out["matmul_96x112x80"] = ref.matmul(a, b)
    da, db = ref.matmul_backward(a, b, g)
    out["matmul_bwd_dA"], out["matmul_bwd_dB"] = da, db
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.arange(6, dtype=np.float32).reshape(3, 2)
    da, db = ref.matmul_backward(a, b, np.ones((2, 2), np.float32))
    out["matmul_arange_C"] = ref.matmul(a, b)
    out["matmul_arange_dA"], out["matmul_arange_dB"] = da, db

    # --- Kaiming weights (first values + sums pin the generator) --------------------------------
    w = ref.linear_weight(784, 256)
    out["linear_w_784_256_head"] = w.ravel()[:64].copy()
    out["linear_w_784_256_sum"] = np.array([w.astype(np.float64).sum(), np.abs(w).astype(np.float64).sum()])
    cw = ref.conv_weight(64, 128, 3)
    out["conv_w_64_128_3_head"] = cw.ravel()[:64].copy()
    out["conv_w_64_128_3_sum"] = np.array([cw.astype(np.float64).sum(), np.abs(cw).astype(np.float64).sum()])

    # --- Linear forward + backward, the 64x784 -> 256 configuration -----------------------------
    x = refdata.mnist_like(21, (64, 784))
    gy = refdata.normal(22, (64, 256))
    y, dx, dw = ref.linear_fwd_bwd(x, w, gy, relu=True)
    out["linear_c2_Y"] = y
    out["linear_c2_dX"] = dx
    out["linear_c2_dW_rows"] = dw[LINEAR_DW_ROWS].copy()
    out["linear_c2_dW_rowsum"] = dw.astype(np.float64).sum(axis=1)

    # --- Conv2dModule forward --------------------------------------------------------------------
    x = refdata.normal(31, (2, 3, 32, 32))
    w1 = ref.conv_weight(3, 64, 3)
    y1 = ref.conv2d_forward(x, w1, 1, 1, 1)
    out["conv_l1_Y_ch"] = y1[:, CONV_CHANNELS_L1].copy()
    out["conv_l1_Y_sum"] = y1.astype(np.float64).sum(axis=(0, 2, 3))
    x2 = refdata.normal(32, (1, 64, 32, 32))
    y2 = ref.conv2d_forward(x2, cw, 1, 1, 1)
    out["conv_l2_Y_ch"] = y2[:, CONV_CHANNELS_L2].copy()
    out["conv_l2_Y_sum"] = y2.astype(np.float64).sum(axis=(0, 2, 3))
    xs = refdata.normal(33, (2, 4, 9, 11))
    ws = ref.conv_weight(4, 6, 3)
    out["conv_s2p2d2_Y"] = ref.conv2d_forward(xs, ws, 2, 2, 2)

    # --- log_softmax and the MLP step's gradients at a reduced batch ---------------------------
    z = refdata.normal(41, (32, 10)) * np.float32(3.0)
    out["log_softmax_32x10"] = ref.log_softmax(z)
    dims = (784, 64, 48, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    xb = refdata.mnist_like(42, (32, 784))
    lab = refdata.labels(43, 32)
    loss, dws = ref.mlp_grads(xb, lab, ws)
    out["mlp_loss"] = np.array([loss], np.float32)
    out["mlp_dW1_rows"] = dws[0][[0, 7, 63]].copy()
    out["mlp_dW1_rowsum"] = dws[0].astype(np.float64).sum(axis=1)
    out["mlp_dW2"] = dws[1]
    out["mlp_dW3"] = dws[2]

    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
