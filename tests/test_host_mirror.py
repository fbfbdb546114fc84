"""The C++20 host mirror of the reference interface (tensors_b200/host): builds with g++ alone, its
argument checks run without a GPU, and its reference-style known-answer checks run on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tensors_b200", "host")


def build():
    subprocess.run(["make", "-C", HOST], check=True, capture_output=True)


def test_host_mirror_builds_and_checks_arguments_without_gpu():
    build()
    r = subprocess.run([os.path.join(HOST, "host_test"), "cpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout


@pytest.mark.gpu
def test_host_mirror_known_answers_on_gpu():
    build()
    r = subprocess.run([os.path.join(HOST, "host_test"), "gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [1, 2, 4])
def test_data_parallel_mlp_step_from_plain_cpp(tmp_path, oracle, ranks):
    # train_mlp_dp_b200 drives the tfb_mlp C-ABI from C++ alone: R ranks in one process (all on one GPU
    # when fewer than R are visible), one step from the reference's own initial weights. The summed
    # gradient must be the oracle's full-batch gradient, the update the momentum formula bit for bit, and
    # every rank's replica of the parameters identical.
    import numpy as np
    import refdata
    build()
    dims, batch = (784, 128, 96, 10), 203   # ragged shards
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    bs = [np.zeros(d, np.float32) for d in dims[1:]]
    x, lab = refdata.mnist_like(5, (batch, 784)), refdata.labels(6, batch)
    prob, out = tmp_path / "problem.bin", tmp_path / "out.bin"
    with open(prob, "wb") as f:
        f.write(np.array([3, *dims, batch], np.int64).tobytes())
        for w, b in zip(ws, bs):
            f.write(np.ascontiguousarray(w, np.float32).tobytes())
            f.write(b.tobytes())
        f.write(np.ascontiguousarray(x, np.float32).tobytes())
        f.write(np.ascontiguousarray(lab, np.int64).tobytes())
    r = subprocess.run([os.path.join(HOST, "train_mlp_dp_b200"), str(prob), str(ranks), "1", str(out)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = open(out, "rb").read()
    loss = np.frombuffer(raw, np.float32, 1, 0)[0]
    numel = int(np.frombuffer(raw, np.int64, 1, 4)[0])
    params = np.frombuffer(raw, np.float32, numel, 12)
    grads = np.frombuffer(raw, np.float32, numel, 12 + 4 * numel)
    same = np.frombuffer(raw, np.int64, ranks, 12 + 8 * numel)
    assert same.tolist() == [1] * ranks
    ol, odw, odb = oracle.mlp_grads(x, lab, ws, bs=bs)
    assert abs(float(loss) - ol) < 1e-5
    from tensors_b200.mlp import flat_layout
    offsets, n = flat_layout(dims)
    assert n == numel
    p0 = np.zeros(numel, np.float32)
    for i in range(3):
        wseg = slice(offsets[2 * i], offsets[2 * i] + ws[i].size)
        bseg = slice(offsets[2 * i + 1], offsets[2 * i + 1] + bs[i].size)
        p0[wseg] = ws[i].ravel()
        # Per output unit (a row of the weight gradient and one bias-gradient entry). A hidden unit whose
        # pre-activation is zero to within rounding for some sample can fall on either side of the ReLU
        # mask (the oracle sums in another order), which moves that one unit's gradient of the layer
        # below by a whole term: at most two such units are tolerated, every other unit must agree.
        gw, ow = grads[wseg].reshape(odw[i].shape), odw[i]
        err_rows = np.linalg.norm(gw - ow, axis=1) / (np.linalg.norm(ow, axis=1) + 1e-30)   # dead units: 0 / tiny
        err_bias = np.abs(grads[bseg] - odb[i]) / (np.abs(odb[i]) + 1e-3 * np.linalg.norm(odb[i]))
        ties = int(((err_rows > 2e-5) | (err_bias > 2e-4)).sum())
        assert ties <= (2 if i < 2 else 0), (i, ties, np.sort(err_rows)[-4:], np.sort(err_bias)[-4:])
    want_p, _ = oracle.sgd_momentum(p0, np.zeros(numel, np.float32), grads, 0.1, 0.9)
    assert np.array_equal(params, want_p)


@pytest.mark.gpu
def test_gemm_bench_writes_the_reference_result_schema(tmp_path):
    # benchmarks/gemm_bench.cpp:317-359: {gpu, sm_count, peak_tflops, warmup, iters, sizes, results[...]}
    import json
    build()
    out = tmp_path / "gemm_results.json"
    r = subprocess.run([os.path.join(HOST, "gemm_bench_b200"), "--sizes", "128,512", "--iters", "3", "--output", str(out)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    d = json.load(open(out))
    assert {"gpu", "sm_count", "peak_tflops", "warmup", "iters", "sizes", "results"} <= set(d)
    assert d["sizes"] == [128, 512] and d["warmup"] == 3 and d["iters"] == 3
    assert len(d["results"]) == 2 * 3 * 3   # sizes x kernels x dtypes
    for e in d["results"]:
        assert {"size", "kernel", "time_ms", "tflops", "sol_pct"} <= set(e)
        assert e["kernel"] in ("naive", "tiled", "optimized") and e["time_ms"] > 0 and e["tflops"] > 0


@pytest.mark.gpu
def test_training_loop_on_the_host_mirror_learns():
    # Linear -> relu -> Linear -> cross_entropy -> backward -> SGD, all on the device; exits 0 when the
    # loss at least halves
    build()
    r = subprocess.run([os.path.join(HOST, "train_mlp_b200"), "100", "256", "128"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "final_loss" in r.stdout
