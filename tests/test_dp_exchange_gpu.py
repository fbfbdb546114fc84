"""The fused gradient exchange (reduce-scatter -> SGD with momentum -> all-gather in one kernel) of the
data-parallel MLP step.

On one GPU the ranks of a group are emulated: one tfb_mlp handle per rank on the same device, their
exchange kernels run as ONE cooperative launch (tfb_mlp_exchange_update_one_device), so the flag
protocol, the slice arithmetic and the peer stores are exactly those of a real group. With two or
more GPUs the same protocol runs across processes through CUDA IPC (test_two_process_group_*).
Expected values are computed on the host: rank-order FP32 sums of the ranks' gradient buffers and the
momentum formula of nn/optim/SGD.hpp:3-6, both bit for bit."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

import refdata
import tensors_b200.capi as capi
from gpu_util import assert_device_ok, dev, lib, stream_ptr

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIMS = (784, 96, 64, 10)


def make_group(world, rows_per_rank, dims=DIMS):
    from tensors_b200.mlp import MLP
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(len(dims) - 1)]
    ms = [MLP(dims, ws, max_rows=rows_per_rank) for _ in range(world)]
    regions = (ctypes.c_void_p * world)(*[m._ptr(MLP.P_REGION) for m in ms])
    for r, m in enumerate(ms):
        capi.check(lib.tfb_mlp_connect_ptrs(m.handle, r, world, regions))
        m.set_option(MLP.OPT_KEEP_REDUCED, 1)
    handles = (ctypes.c_void_p * world)(*[m.handle.value for m in ms])
    return ms, handles


def slice_bounds(numel, rank, world):
    n_vec = numel // 4
    return 4 * (n_vec * rank // world), 4 * (n_vec * (rank + 1) // world)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_emulated_group_two_steps_bit_exact(oracle, world):
    from tensors_b200.mlp import shard_rows
    batch = 64 * world + 5   # ragged shards
    ms, handles = make_group(world, batch // world + 1)
    xb, lab = refdata.mnist_like(7, (batch, DIMS[0])), refdata.labels(8, batch)
    X, L = dev(xb), torch.from_numpy(lab).cuda()
    params = ms[0].params.cpu().numpy().copy()
    velocity = np.zeros_like(params)
    numel = ms[0].numel
    for step in range(2):
        for r, m in enumerate(ms):
            b, e = shard_rows(batch, r, world)
            m.forward_backward(X[b:e], L[b:e], global_rows=batch)
        contrib = [m.grads_and_loss.cpu().numpy().copy() for m in ms]
        capi.check(lib.tfb_mlp_exchange_update_one_device(handles, world, 0.1, 0.9, stream_ptr()))
        assert_device_ok()
        # expected: sums in rank order, then the momentum update, all in FP32
        total = contrib[0].copy()
        for c in contrib[1:]:
            total = (total + c).astype(np.float32)
        params, velocity = oracle.sgd_momentum(params, velocity, total[:numel], 0.1, 0.9)
        for r, m in enumerate(ms):
            assert np.array_equal(m.params.cpu().numpy(), params), (step, r)    # every replica, every slice
            assert float(m.loss.item()) == float(total[numel]), (step, r)
            lo, hi = slice_bounds(numel, r, world)
            assert np.array_equal(m.reduced.cpu().numpy()[lo:hi], total[lo:hi]), (step, r)
            assert np.array_equal(m.velocity.cpu().numpy()[lo:hi], velocity[lo:hi]), (step, r)


def test_emulated_group_matches_single_rank_step(oracle):
    # config 5's layer sizes; 4 ranks x 256 rows against one rank with all 1024 rows: same loss and the
    # same parameters after one step up to FP32 summation order (and ReLU ties, see the invariance test)
    from tensors_b200.mlp import MLP, shard_rows
    dims, batch, world = (784, 1024, 1024, 10), 1024, 4
    ms, handles = make_group(world, batch // world, dims)
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    one = MLP(dims, ws, max_rows=batch)
    X = dev(refdata.mnist_like(7, (batch, 784)))
    L = torch.from_numpy(refdata.labels(8, batch)).cuda()
    p0 = one.params.clone()
    one.train_step(X, L, lr=0.1, momentum=0.9)
    for r, m in enumerate(ms):
        b, e = shard_rows(batch, r, world)
        m.forward_backward(X[b:e], L[b:e], global_rows=batch)
    capi.check(lib.tfb_mlp_exchange_update_one_device(handles, world, 0.1, 0.9, stream_ptr()))
    assert_device_ok()
    assert abs(float(ms[0].loss.item()) - float(one.loss.item())) < 1e-5
    step_one, step_group = one.params - p0, ms[0].params - p0
    assert float((step_group - step_one).norm() / step_one.norm()) < 2e-3   # a few ReLU ties at most
    last = slice(one.offsets[4], one.offsets[4] + 10 * 1024)                 # no mask behind the last layer
    assert float((step_group[last] - step_one[last]).norm() / step_one[last].norm()) < 1e-5


def test_exchange_wait_runs_out_and_is_reported():
    # Rank 0 of a two-rank group runs its exchange alone: the flag rank 1 would set never arrives, the
    # wait ends at its (here 2 ms) limit, the kernel records device error 107 and returns, and the device
    # stays usable.
    from tensors_b200.mlp import MLP
    ms, _ = make_group(2, 16)
    ms[0].set_option(MLP.OPT_WAIT_NS, 2_000_000)
    p0 = ms[0].params.clone()
    capi.check(lib.tfb_mlp_exchange_update(ms[0].handle, 0.1, 0.9, stream_ptr()))
    code = ctypes.c_int(0)
    rc = lib.tfb_device_status(ctypes.byref(code))
    assert rc == -4 and code.value == 107
    assert torch.equal(ms[0].params, p0)          # nothing was updated from gradients that never arrived
    assert_device_ok()                            # the error was cleared by reading it
    a = dev(refdata.uniform(1, (64, 64)))
    c = torch.empty((64, 64), device="cuda")
    capi.check(lib.tfb_matmul(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(c.data_ptr()),
                              64, 64, 64, 0, 0, stream_ptr()))
    assert_device_ok()


def _two_process_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from tensors_b200.mlp import MLP, shard_rows
    dims, batch = (784, 256, 128, 10), 512
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    b, e = shard_rows(batch, rank, world)
    X = dev(refdata.mnist_like(7, (batch, 784))[b:e])
    L = torch.from_numpy(refdata.labels(8, batch)[b:e]).cuda()
    out = {}
    for mode in ("peer", "nccl", "peer2"):
        m = MLP(dims, ws, max_rows=e - b, exchange="peer" if mode == "peer2" else mode)
        if mode == "peer2":   # layers 1.. exchanged on a side stream while layer 0's weight gradient is computed
            m.set_option(MLP.OPT_BUCKETS, 2)
        for _ in range(3):
            m.train_step(X, L, lr=0.1, momentum=0.9, global_rows=batch)
        replay = m.capture_train_step(X, L, lr=0.1, momentum=0.9, global_rows=batch, warmup=1)
        for _ in range(2):
            replay()
        torch.cuda.synchronize()
        out[mode] = (m.params.cpu().numpy(), float(m.loss.item()), capi.device_status())
        m.disconnect()
        dist.barrier()
        del m
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), peer=out["peer"][0], nccl=out["nccl"][0], peer2=out["peer2"][0],
             losses=np.array([out["peer"][1], out["nccl"][1], out["peer2"][1]]),
             status=np.array([out["peer"][2], out["nccl"][2], out["peer2"][2]]))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_process_group_peer_exchange_equals_nccl(tmp_path):
    # Two processes, one GPU each: six steps with the fused peer-memory exchange, six with one NCCL
    # all-reduce per step, and six with the peer exchange in two buckets (eager and from a captured graph
    # with a forked side stream). With two ranks every sum is g0 + g1 (commutative), so the trajectories are
    # bit-identical, and both replicas of each run hold the same parameters.
    import torch.multiprocessing as mp
    mp.spawn(_two_process_worker, args=(2, 29541, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    assert list(r0["status"]) == [0, 0, 0] and list(r1["status"]) == [0, 0, 0]
    assert np.array_equal(r0["peer"], r1["peer"])
    assert np.array_equal(r0["nccl"], r1["nccl"])
    assert np.array_equal(r0["peer2"], r1["peer2"])
    assert np.array_equal(r0["peer"], r0["nccl"])
    assert np.array_equal(r0["peer"], r0["peer2"])
    assert r0["losses"][0] == r0["losses"][1] == r0["losses"][2] == r1["losses"][0] == r1["losses"][2]


# ---- tfb_peer_group: small all-reduce through peer memory, and the batch-sharded convolution ---------
def make_peer_groups(world, capacity):
    from tensors_b200.peer import PeerGroup
    gs = [PeerGroup(capacity) for _ in range(world)]
    regions = (ctypes.c_void_p * world)(*[g.region for g in gs])
    for r, g in enumerate(gs):
        capi.check(lib.tfb_peer_group_connect_ptrs(g.handle, r, world, regions))
    handles = (ctypes.c_void_p * world)(*[g.handle.value for g in gs])
    return gs, handles


@pytest.mark.parametrize("world,n", [(2, 1000), (3, 7), (4, 295040), (8, 1863690)])
def test_peer_allreduce_emulated_group_bit_exact(world, n):
    gs, handles = make_peer_groups(world, n)
    for rep in range(2):   # twice: the flags and the step counter carry over
        contrib = [refdata.normal(10 * rep + r, (n,)) for r in range(world)]
        for g, c in zip(gs, contrib):
            g.inp[:n].copy_(torch.from_numpy(c))
            g.out.fill_(float("nan"))
        capi.check(lib.tfb_peer_allreduce_sum_one_device(handles, world, n, stream_ptr()))
        assert_device_ok()
        want = contrib[0].copy()
        for c in contrib[1:]:
            want = (want + c).astype(np.float32)
        for r, g in enumerate(gs):
            assert np.array_equal(g.out[:n].cpu().numpy(), want), (rep, r)


def test_batch_sharded_conv_backward_sums_to_the_full_batch(oracle):
    # 4 ranks x 2 samples: each rank's weight / bias gradient share lands in its contribution buffer, the
    # peer all-reduce completes the sum over the batch (the sum nn/Conv2d.cpp:215-243 runs over samples)
    world, n_local = 4, 2
    N, Cin, H, W, Cout, k = world * n_local, 16, 12, 12, 32, 3
    x, w = refdata.normal(1, (N, Cin, H, W)), refdata.conv_weight(Cin, Cout, k)
    g = refdata.normal(3, (N, Cout, H, W))
    nw = Cout * Cin * k * k
    nw4 = (nw + 3) // 4 * 4
    gs, handles = make_peer_groups(world, nw4 + Cout)
    X, Wt, G = dev(x), dev(w), dev(g)
    gi = torch.full(x.shape, float("nan"), device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for r, grp in enumerate(gs):
        sl = slice(r * n_local, (r + 1) * n_local)
        capi.check(lib.tfb_conv2d_backward_sharded(grp.handle, p(X[sl]), p(Wt), p(G[sl]), p(gi[sl]), n_local, Cin, H, W, Cout,
                                                   k, k, 1, 1, 1, 1, 1, 1, 0, stream_ptr()))
    capi.check(lib.tfb_peer_allreduce_sum_one_device(handles, world, nw4 + Cout, stream_ptr()))
    assert_device_ok()
    oi, ow, ob = oracle.conv2d_backward(x, w, g, (1, 1), (1, 1), (1, 1))
    for grp in gs:
        out = grp.out.cpu().numpy()
        assert np.linalg.norm(out[:nw] - ow.ravel()) / np.linalg.norm(ow) < 1e-5
        assert np.linalg.norm(out[nw4:nw4 + Cout] - ob) / np.linalg.norm(ob) < 1e-5
        assert np.array_equal(out, gs[0].out.cpu().numpy())
    assert np.linalg.norm(gi.cpu().numpy() - oi) / np.linalg.norm(oi) < 1e-5


def _two_process_conv_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from tensors_b200.peer import PeerGroup
    N, Cin, H, W, Cout, k = 8, 64, 32, 32, 128, 3
    n_local = N // world
    x, w, g = refdata.normal(1, (N, Cin, H, W)), refdata.conv_weight(Cin, Cout, k), refdata.normal(3, (N, Cout, H, W))
    nw4 = Cout * Cin * k * k
    grp = PeerGroup(nw4 + Cout)
    grp.connect()
    sl = slice(rank * n_local, (rank + 1) * n_local)
    X, Wt, G = dev(x[sl]), dev(w), dev(g[sl])
    gi = torch.empty_like(X)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for _ in range(3):
        capi.check(lib.tfb_conv2d_backward_sharded(grp.handle, p(X), p(Wt), p(G), p(gi), n_local, Cin, H, W, Cout, k, k,
                                                   1, 1, 1, 1, 1, 1, 1, stream_ptr()))
    torch.cuda.synchronize()
    mine = grp.inp.clone()
    both = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    want = both[0].clone()
    for t in both[1:]:
        want += t
    np.savez(os.path.join(out_dir, f"conv{rank}.npz"), out=grp.out.cpu().numpy(), want=want.cpu().numpy(),
             status=np.array([capi.device_status()]))
    grp.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_process_batch_sharded_conv_backward(tmp_path):
    # the layer-2 convolution of the CIFAR-shaped configuration, batch split over two processes / GPUs
    import torch.multiprocessing as mp
    mp.spawn(_two_process_conv_worker, args=(2, 29543, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "conv0.npz"), np.load(tmp_path / "conv1.npz")
    assert r0["status"][0] == 0 and r1["status"][0] == 0
    assert np.array_equal(r0["out"], r1["out"])
    assert np.array_equal(r0["out"], r0["want"])   # g0 + g1 in rank order
