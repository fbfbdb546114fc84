"""Data-parallel host logic on CPU (gloo, world size 2): row sharding, the 1/global-batch loss scale and
the flat-buffer all-reduce must reproduce the single-process full-batch gradient. The arithmetic of each
rank comes from the oracle here (no GPU in this test); the same MLP class drives libtfb on the GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import refdata

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIMS = (20, 16, 12, 10)
BATCH = 37   # odd on purpose: ragged shards


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import Oracle
    from tensors_b200.mlp import MLP, shard_rows
    oracle = Oracle()
    ws = [refdata.linear_weight(DIMS[i], DIMS[i + 1]) for i in range(3)]
    x, lab = refdata.normal(1, (BATCH, DIMS[0])), refdata.labels(2, BATCH)
    b, e = shard_rows(BATCH, rank, world)
    m = MLP(DIMS, ws, device="cpu")
    loss, dws, dbs = oracle.mlp_grads(x[b:e], lab[b:e], ws, bs=[np.zeros(d, np.float32) for d in DIMS[1:]],
                                      global_rows=BATCH)
    for i in range(3):
        m.weight(i, m.grads).copy_(torch.from_numpy(dws[i]))
        m.bias(i, m.grads).copy_(torch.from_numpy(dbs[i]))
    m.grads_and_loss[m.numel] = loss   # the loss contribution rides in the slot behind the gradients
    m.allreduce_grads()                # one collective for both
    m.sgd_step(0.1, 0.9)               # host-logic mode: only moves the summed loss into m.loss
    np.save(os.path.join(out_dir, f"grads_{rank}.npy"), m.grads.numpy())
    np.save(os.path.join(out_dir, f"loss_{rank}.npy"), m.loss.numpy())
    dist.destroy_process_group()


def test_shard_rows_covers_the_batch():
    from tensors_b200.mlp import shard_rows
    for world in (1, 2, 3, 8):
        for n in (0, 1, 7, 8192):
            spans = [shard_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_allreduce_reproduces_full_batch_gradient(tmp_path, oracle):
    world = 2
    mp.spawn(_worker, args=(world, 29533, str(tmp_path)), nprocs=world, join=True)
    g0 = np.load(tmp_path / "grads_0.npy")
    g1 = np.load(tmp_path / "grads_1.npy")
    assert np.array_equal(g0, g1)
    ws = [refdata.linear_weight(DIMS[i], DIMS[i + 1]) for i in range(3)]
    x, lab = refdata.normal(1, (BATCH, DIMS[0])), refdata.labels(2, BATCH)
    loss, dws, dbs = oracle.mlp_grads(x, lab, ws, bs=[np.zeros(d, np.float32) for d in DIMS[1:]])
    from tensors_b200.mlp import MLP
    m = MLP(DIMS, ws, device="cpu")
    full = torch.from_numpy(g0)
    for i in range(3):
        got_w = m.weight(i, full).numpy()
        got_b = m.bias(i, full).numpy()
        assert np.linalg.norm(got_w - dws[i]) <= 2e-6 * np.linalg.norm(dws[i]) + 1e-9
        assert np.linalg.norm(got_b - dbs[i]) <= 2e-6 * np.linalg.norm(dbs[i]) + 1e-9
    assert abs(float(np.load(tmp_path / "loss_0.npy")[0]) - loss) < 1e-6
