"""Timings of the named configurations other than the headline square GEMM (which bench.py covers):

  config 1  FP32 GEMM 2048^3 through tfb_matmul
  config 2  Linear 64x784 -> 256 forward + backward (bias, ReLU fused)
  config 3  Conv2d 128x3x32x32 -> 64 -> 128, 3x3 pad 1: forward, backward per layer
  config 4  square sweep 1024..16384, FP32 (3xTF32) and BF16
  config 5  MLP 784-1024-1024-10 training step, batch 8192 / world size (peer-memory or NCCL exchange when > 1 rank)
  config 6  probe: the GEMM kernel's rasterisation group width (A panels shared by a wave) at 8192^3, FP32 and BF16
  config 7  probe: phase timeline of the gradient-exchange kernel (flag barrier, slice, fence, flag barrier); > 1 rank
  config 8  probe: phase timeline of the GEMM kernel (prologue, first stage, last MMA, epilogue) for the products of
            an MLP shard, next to the whole call's time under CUDA-graph replay

Run:  python bench_configs.py [--configs 1,2,3,4,5] [--iters 20]
      torchrun --nproc-per-node N bench_configs.py --configs 5 [--exchange peer|nccl]
Prints one JSON line per measurement (CUDA events on the launching stream, median of `iters` after 3
warm-up runs, as the reference's benches do: benchmarks/gemm_bench.cpp:99-124).
"""
import argparse
import ctypes
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import refdata  # noqa: E402
from tensors_b200 import capi  # noqa: E402
from tensors_b200.mlp import MLP, shard_rows  # noqa: E402

lib = capi.lib
HBM_GBS = 6549.1


def p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def time_us(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(times)


def graph_us(fn, iters, warmup=3):
    """Device time of fn replayed from a CUDA graph: what is left once the host's launch calls are out
    of the way (a run of small kernels is otherwise timed at the speed of the host enqueuing them)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return time_us(g.replay, iters, warmup)


def emit(**kw):
    print(json.dumps(kw), flush=True)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(a).cuda().to(dtype)


def config1(iters):
    n = 2048
    A, B = dev(refdata.uniform(0, (n, n))), dev(refdata.uniform(1, (n, n)))
    C = torch.empty((n, n), device="cuda")
    us = time_us(lambda: capi.check(lib.tfb_matmul(p(A), p(B), p(C), n, n, n, 0, 0, stream())), iters)
    emit(config=1, what="FP32 GEMM 2048^3 via tfb_matmul (2 launches)", us=us, tflops=2 * n ** 3 / us / 1e6)


def config2(iters):
    batch, in_f, out_f = 64, 784, 256
    X, W = dev(refdata.mnist_like(21, (batch, in_f))), dev(refdata.linear_weight(in_f, out_f))
    b, G = torch.zeros(out_f, device="cuda"), dev(refdata.normal(22, (batch, out_f)))
    Y, dX = torch.empty((batch, out_f), device="cuda"), torch.empty((batch, in_f), device="cuda")
    dW, db = torch.empty((out_f, in_f), device="cuda"), torch.empty(out_f, device="cuda")
    fwd = lambda: capi.check(lib.tfb_linear_forward(p(X), p(W), p(b), p(Y), batch, in_f, out_f, 1, 0, stream()))
    bwd = lambda: capi.check(lib.tfb_linear_backward(p(X), p(W), p(Y), p(G), p(dX), p(dW), p(db), batch, in_f, out_f, 1, 0, stream()))
    uf, ub = time_us(fwd, iters), time_us(bwd, iters)
    gf, gb = graph_us(fwd, iters), graph_us(bwd, iters)
    fwd_bytes, bwd_bytes = 1.070e6, 2.14e6
    emit(config=2, what="Linear 64x784->256 forward (bias+ReLU fused)", us=uf, graph_us=gf, gbs=fwd_bytes / gf / 1e3,
         hbm_frac=fwd_bytes / gf / 1e3 / HBM_GBS, mflop=25.69)
    emit(config=2, what="Linear backward (mask+split, dX, dW, db)", us=ub, graph_us=gb, gbs=bwd_bytes / gb / 1e3,
         hbm_frac=bwd_bytes / gb / 1e3 / HBM_GBS, mflop=51.38)


EXCHANGE = "peer"
MLP_ROWS = 0
BUCKETS = 0
CONV_N, CONV_LAYERS, CONV_PASSES = 128, ("1", "2"), ("forward", "dgrad", "wgrad+dbias", "backward")


def config3(iters):
    N = CONV_N
    x = dev(refdata.normal(31, (N, 3, 32, 32)))
    for name, cin, cout, xin, alg_bytes, gflop in (("layer1 3->64", 3, 64, x, 35.1e6 * N / 128, 0.45298 * N / 128),
                                                   ("layer2 64->128", 64, 128, None, 101.0e6 * N / 128, 19.33 * N / 128)):
        if name[5] not in CONV_LAYERS:
            continue
        if xin is None:
            xin = dev(refdata.normal(32, (N, cin, 32, 32)))
        w = dev(refdata.conv_weight(cin, cout, 3))
        bias = torch.zeros(cout, device="cuda")
        y = torch.empty((N, cout, 32, 32), device="cuda")
        g = dev(refdata.normal(33, (N, cout, 32, 32)))
        gi, gw, gb = torch.empty_like(xin), torch.empty_like(w), torch.empty(cout, device="cuda")
        args = (N, cin, 32, 32, cout, 3, 3, 1, 1, 1, 1, 1, 1)
        fwd = lambda: capi.check(lib.tfb_conv2d_forward(p(xin), p(w), p(bias), p(y), *args, 0, 0, stream()))
        dgr = lambda: capi.check(lib.tfb_conv2d_backward(p(xin), p(w), p(g), p(gi), None, None, *args, 0, stream()))
        wgr = lambda: capi.check(lib.tfb_conv2d_backward(p(xin), p(w), p(g), None, p(gw), p(gb), *args, 0, stream()))
        # "backward": all three gradients in one call, as nn::Conv2d::backward computes them (the upstream
        # gradient's planes are made once for both products); two passes' worth of FLOPs
        bwd = lambda: capi.check(lib.tfb_conv2d_backward(p(xin), p(w), p(g), p(gi), p(gw), p(gb), *args, 0, stream()))
        for what, fn, passes in (("forward", fwd, 1), ("dgrad", dgr, 1), ("wgrad+dbias", wgr, 1), ("backward", bwd, 2)):
            if what not in CONV_PASSES:
                continue
            us = time_us(fn, iters)
            gus = graph_us(fn, iters)
            emit(config=3, what=f"Conv2d {name} {what}, N={N} 32x32 3x3 p1", us=us, graph_us=gus,
                 tflops=passes * gflop / gus * 1e3, gbs=passes * alg_bytes / gus / 1e3)


def config4(iters):
    for n in (1024, 2048, 4096, 8192, 16384):
        A, B = dev(refdata.uniform(2, (n, n))), dev(refdata.uniform(3, (n, n)))
        C = torch.empty((n, n), device="cuda")
        it = max(3, iters if n < 16384 else iters // 4)
        us = time_us(lambda: capi.check(lib.tfb_matmul(p(A), p(B), p(C), n, n, n, 0, 0, stream())), it)
        emit(config=4, what=f"FP32 (3xTF32) GEMM {n}^3", us=us, tflops=2 * n ** 3 / us / 1e6)
        A16, B16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
        del A, B
        us = time_us(lambda: capi.check(lib.tfb_matmul(p(A16), p(B16), p(C), n, n, n, 2, 0, stream())), it)
        emit(config=4, what=f"BF16 GEMM {n}^3 (FP32 accumulate/output)", us=us, tflops=2 * n ** 3 / us / 1e6)
        del A16, B16, C
        torch.cuda.empty_cache()


def config5(iters):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    dims, batch = (784, 1024, 1024, 10), 8192
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    b, e = shard_rows(batch, rank, world)
    if MLP_ROWS > 0:   # one rank's shard of a larger group, run alone: the per-rank compute of that group size
        b, e = 0, MLP_ROWS
    X = dev(refdata.mnist_like(7, (batch, 784))[b:e])
    labels = torch.from_numpy(refdata.labels(8, batch)[b:e]).cuda()
    m = MLP(dims, ws, max_rows=e - b, exchange=EXCHANGE)
    if BUCKETS:
        m.set_option(MLP.OPT_BUCKETS, BUCKETS)
    step = lambda: m.train_step(X, labels, lr=0.1, momentum=0.9, global_rows=batch)
    us_eager = time_us(step, iters)
    fb = time_us(lambda: m.forward_backward(X, labels, batch), iters)
    replay = m.capture_train_step(X, labels, lr=0.1, momentum=0.9, global_rows=batch)
    us = time_us(replay, iters)
    scratch = m.grads.clone()   # timing the collective must not keep summing the real gradients
    ar = time_us(lambda: dist.all_reduce(scratch), iters) if world > 1 else 0.0
    if world > 1:
        t = torch.tensor([us, fb, ar, us_eager], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us, fb, ar, us_eager = [float(v) for v in t.tolist()]
    if rank == 0:
        emit(config=5, what=f"MLP 784-1024-1024-10 step (CUDA graph replay), global batch 8192 on {world} GPU(s)", us=us,
             rows_per_rank=e - b,
             exchange=EXCHANGE if world > 1 else "none", eager_us=us_eager, forward_backward_us=fb, allreduce_us=ar,
             tflops=78.35e9 / us / 1e6, loss=float(m.loss.item()))
    m.disconnect()
    del m
    if world > 1:
        dist.destroy_process_group()


def config6(iters):
    n = 8192
    A, B = torch.rand(n, n, device="cuda") * 2 - 1, torch.rand(n, n, device="cuda") * 2 - 1
    C = torch.empty(n, n, device="cuda")
    hl = torch.empty(4, n, n, device="cuda")
    capi.check(lib.tfb_split_tf32(p(A), n, n, n, p(hl[0]), p(hl[1]), n, stream()))
    capi.check(lib.tfb_split_tf32(p(B), n, n, n, p(hl[2]), p(hl[3]), n, stream()))
    A16, B16 = A.bfloat16(), B.bfloat16()
    f32 = lambda: capi.check(lib.tfb_gemm_presplit(p(hl[0]), p(hl[1]), p(hl[2]), p(hl[3]), p(C), n, n, n, n, n, n, 0, 0,
                                                   None, 0, stream()))
    b16 = lambda: capi.check(lib.tfb_matmul(p(A16), p(B16), p(C), n, n, n, 2, 0, stream()))
    for gm in (8, 1, 2, 4, 16, 32):
        capi.check(lib.tfb_set_tuning(capi.TUNE_GEMM_GROUP_M, gm))
        for fn, name in ((f32, "fp32 (3xTF32), operands pre-split"), (b16, "bf16")):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            emit(config=6, what=f"GEMM 8192^3 {name}, raster group of {gm} M tiles", group_m=gm, ms=ms,
                 tflops=2 * n ** 3 / ms / 1e9)
    capi.check(lib.tfb_set_tuning(capi.TUNE_GEMM_GROUP_M, 0))


def config7(iters):
    import torch.distributed as dist
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world < 2:
        emit(config=7, what="exchange phase trace needs more than one rank (run under torchrun)")
        return
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    dims = (784, 1024, 1024, 10)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    m = MLP(dims, ws, max_rows=64, exchange="peer")
    m.connect()
    m.set_option(3, 1)   # TFB_MLP_OPT_TRACE_EXCHANGE
    stamps = torch.empty(5, dtype=torch.int64, device="cuda")
    for ctas in (0, 64, 32, 16):
        m.set_option(MLP.OPT_CTAS, ctas)
        for _ in range(10):
            m.exchange_update(0.0, 0.9)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(max(iters, 20)):
            m.exchange_update(0.0, 0.9)
        e1.record()
        torch.cuda.synchronize()
        capi.check(lib.tfb_memcpy(p(stamps), ctypes.c_void_p(m._ptr(8)), 40, 3, stream()))   # TFB_MLP_EXCHANGE_TRACE
        torch.cuda.synchronize()
        v = stamps.cpu().tolist()
        emit(config=7, rank=rank, world=world, exchange_ctas=ctas or "default (128)",
             us_per_exchange=e0.elapsed_time(e1) * 1e3 / max(iters, 20),
             phases_us={k: (v[i + 1] - v[i]) / 1e3 for i, k in enumerate(("flag_barrier_0", "slice_sum_update_store",
                                                                          "system_fence", "flag_barrier_1"))})
        dist.barrier()
    m.disconnect()
    del m
    dist.destroy_process_group()


def config8(iters):
    stamps = torch.zeros(8, dtype=torch.int64, device="cuda")

    def probe(M, N, K, ta, tb, what):
        A = torch.randn((K, M) if ta else (M, K), device="cuda")
        B = torch.randn((N, K) if tb else (K, N), device="cuda")
        C = torch.empty(M, N, device="cuda")
        lda, ldb = A.shape[1], B.shape[1]
        hA, hB = torch.empty(2, *A.shape, device="cuda"), torch.empty(2, *B.shape, device="cuda")
        capi.check(lib.tfb_split_tf32(p(A), A.shape[0], lda, lda, p(hA[0]), p(hA[1]), lda, stream()))
        capi.check(lib.tfb_split_tf32(p(B), B.shape[0], ldb, ldb, p(hB[0]), p(hB[1]), ldb, stream()))
        run = lambda: capi.check(lib.tfb_gemm_presplit(p(hA[0]), p(hA[1]), p(hB[0]), p(hB[1]), p(C), M, N, K, lda, ldb, N,
                                                       int(ta), int(tb), None, 0, stream()))
        us = graph_us(run, max(iters, 10))
        capi.check(lib.tfb_gemm_trace(p(stamps)))
        run()
        torch.cuda.synchronize()
        capi.check(lib.tfb_gemm_trace(None))
        v = stamps.cpu().tolist()
        names = ("prologue_done", "first_stage_landed", "last_mma_committed", "accumulator_seen", "epilogue_drained", "exit")
        emit(config=8, what=what, shape=[M, N, K], call_us_graph=us,
             kernel_phase_us={n: round((v[i + 1] - v[0]) / 1e3, 2) for i, n in enumerate(names)})

    probe(1024, 1024, 1024, False, True, "forward X W^T of a 1024-row shard")
    probe(1024, 1024, 784, False, True, "forward layer 1 of a 1024-row shard")
    probe(1024, 1024, 1024, False, False, "input gradient dZ W")
    probe(1024, 1024, 1024, True, False, "weight gradient dZ^T X")
    probe(8192, 1024, 1024, False, True, "forward X W^T, batch 8192")
    probe(2048, 2048, 2048, False, False, "2048^3")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="1,2,3,4,5")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--conv-n", type=int, default=128, help="config 3: batch size")
    ap.add_argument("--conv-layers", default="1,2", help="config 3: which layers")
    ap.add_argument("--conv-passes", default="forward,dgrad,wgrad+dbias,backward", help="config 3: which passes (backward = all three gradients in one call)")
    ap.add_argument("--buckets", type=int, default=0, help="config 5: exchange buckets (1 or 2; 0 = the handle's default)")
    ap.add_argument("--mlp-rows", type=int, default=0,
                    help="config 5 on one GPU: run only this many rows of the global batch of 8192 (the shard of one "
                         "rank of a larger group)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="config 5 with more than one rank")
    a = ap.parse_args()
    global CONV_N, CONV_LAYERS, CONV_PASSES, EXCHANGE, MLP_ROWS, BUCKETS
    EXCHANGE, MLP_ROWS, BUCKETS = a.exchange, a.mlp_rows, a.buckets
    CONV_N, CONV_LAYERS, CONV_PASSES = a.conv_n, tuple(a.conv_layers.split(",")), tuple(a.conv_passes.split(","))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    capi.check(lib.tfb_init())
    for c in a.configs.split(","):
        {"1": config1, "2": config2, "3": config3, "4": config4, "5": config5, "6": config6, "7": config7, "8": config8}[c.strip()](a.iters)
    code = capi.device_status()
    if code:
        raise SystemExit(f"device error {code}")


if __name__ == "__main__":
    main()
