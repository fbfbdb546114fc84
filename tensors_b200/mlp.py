"""Data-parallel MLP training step on libtfb (host side).

Mirrors the dataflow of the reference's training example (examples/train_mlp.cpp:161-183):
Linear -> ReLU -> Linear -> ReLU -> Linear -> log_softmax + mean NLL -> backward -> SGD, with the
documented momentum update (nn/optim/SGD.hpp:3-6). Every tensor operation is a libtfb call; torch
only supplies device memory, streams and — for more than one rank — the NCCL all-reduce of the flat
gradient buffer (one per step, a pure sum because each rank already divides by the global batch).
"""
import ctypes

import torch

from . import capi

lib = capi.lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def shard_rows(global_rows, rank, world):
    """Contiguous row range [begin, end) of the global batch that `rank` owns (sizes differ by at most 1)."""
    base, extra = divmod(int(global_rows), int(world))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class MLP:
    """dims = (d0, d1, ..., dL): L Linear layers, ReLU after all but the last."""

    def __init__(self, dims, weights, biases=None, device="cuda", process_group=None):
        self.dims = tuple(int(d) for d in dims)
        self.L = len(self.dims) - 1
        sizes = []
        for i in range(self.L):
            sizes += [self.dims[i + 1] * self.dims[i], self.dims[i + 1]]
        # 16-byte aligned segment starts keep every parameter usable as a TMA operand
        self.offsets = []
        off = 0
        for sz in sizes:
            self.offsets.append(off)
            off += (sz + 3) // 4 * 4
        self.numel = off
        self.params = torch.zeros(off, device=device, dtype=torch.float32)
        self.grads = torch.zeros(off, device=device, dtype=torch.float32)
        self.velocity = torch.zeros(off, device=device, dtype=torch.float32)
        self.group = process_group
        for i in range(self.L):
            self.weight(i).copy_(torch.as_tensor(weights[i], dtype=torch.float32).reshape(self.dims[i + 1], self.dims[i]))
            if biases is not None and biases[i] is not None:
                self.bias(i).copy_(torch.as_tensor(biases[i], dtype=torch.float32))
        self.loss = torch.zeros(1, device=device, dtype=torch.float32)
        self._acts = None
        self._plane_bufs = {}

    def _seg(self, buf, k, shape):
        n = 1
        for s in shape:
            n *= s
        return buf[self.offsets[k]:self.offsets[k] + n].view(*shape)

    def weight(self, i, buf=None):
        return self._seg(self.params if buf is None else buf, 2 * i, (self.dims[i + 1], self.dims[i]))

    def bias(self, i, buf=None):
        return self._seg(self.params if buf is None else buf, 2 * i + 1, (self.dims[i + 1],))

    def _planes(self, key, rows, cols, device):
        """Persistent hi / lo plane buffer [2, rows, ld] for a rows x cols FP32 operand."""
        ld = (cols + 3) // 4 * 4
        buf = self._plane_bufs.get(key)
        if buf is None or buf.shape != (2, rows, ld) or buf.device != device:
            buf = torch.empty((2, rows, ld), device=device, dtype=torch.float32)
            self._plane_bufs[key] = buf
        return buf, ld

    def _split(self, key, t):
        rows, cols = t.shape
        buf, ld = self._planes(key, rows, cols, t.device)
        capi.check(lib.tfb_split_tf32(_p(t), rows, cols, cols, _p(buf[0]), _p(buf[1]), ld, _stream()))
        return buf, ld

    def forward(self, X):
        """Each operand is split into its TF32 hi / lo planes once per step; the planes made for the
        forward products are kept for the backward ones."""
        batch = X.shape[0]
        acts = [X]
        self._xs, self._ws = [], []
        # All weights live in one flat buffer with 16-byte aligned segments, so one launch splits them
        # all; a weight whose row length is a multiple of 4 is then a view of the flat planes.
        flat, _ = self._split(("params",), self.params.view(1, -1))
        for i in range(self.L):
            xs, ldx = self._split(("x", i), acts[-1])
            if self.dims[i] % 4 == 0:
                n = self.dims[i + 1] * self.dims[i]
                ws = flat[:, 0, self.offsets[2 * i]:self.offsets[2 * i] + n].view(2, self.dims[i + 1], self.dims[i])
                ldw = self.dims[i]
            else:
                ws, ldw = self._split(("w", i), self.weight(i))
            Y = torch.empty((batch, self.dims[i + 1]), device=X.device, dtype=torch.float32)
            flags = capi.EPI_BIAS_COL | (capi.EPI_RELU if i < self.L - 1 else 0)
            capi.check(lib.tfb_gemm_presplit(_p(xs[0]), _p(xs[1]), _p(ws[0]), _p(ws[1]), _p(Y), batch,
                                             self.dims[i + 1], self.dims[i], ldx, ldw, self.dims[i + 1], 0, 1,
                                             _p(self.bias(i)), flags, _stream()))
            acts.append(Y)
            self._xs.append((xs, ldx))
            self._ws.append((ws, ldw))
        self._acts = acts
        return acts[-1]

    def forward_backward(self, X, labels, global_rows=None):
        """Fills self.grads (this rank's share of the full-batch gradient) and self.loss."""
        batch = X.shape[0]
        global_rows = int(global_rows or batch)
        logits = self.forward(X)
        acts = self._acts
        dz = torch.empty_like(logits)
        capi.check(lib.tfb_log_softmax_nll(_p(logits), _p(labels), _p(dz), _p(self.loss), batch, self.dims[-1],
                                           global_rows, _stream()))
        upstream = dz
        for i in reversed(range(self.L)):
            relu = i < self.L - 1
            dX = torch.empty_like(acts[i]) if i > 0 else None
            (xs, ldx), (ws, ldw) = self._xs[i], self._ws[i]
            capi.check(lib.tfb_linear_backward_presplit(
                _p(xs[0]), _p(xs[1]), ldx, _p(ws[0]), _p(ws[1]), ldw, _p(acts[i + 1]), _p(upstream), _p(dX),
                _p(self.weight(i, self.grads)), _p(self.bias(i, self.grads)), batch, self.dims[i],
                self.dims[i + 1], int(relu), _stream()))
            upstream = dX
        return self.loss

    def allreduce_grads(self):
        if self._distributed():
            torch.distributed.all_reduce(self.grads, group=self.group)
            torch.distributed.all_reduce(self.loss, group=self.group)

    def sgd_step(self, lr, momentum):
        capi.check(lib.tfb_sgd_momentum(_p(self.params), _p(self.velocity), _p(self.grads), self.numel,
                                        float(lr), float(momentum), 1.0, _stream()))

    def _distributed(self):
        return self.group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                          and torch.distributed.get_world_size() > 1)

    def capture_train_step(self, X, labels, lr=0.1, momentum=0.9, global_rows=None, warmup=2):
        """Records one training step into CUDA graphs and returns a callable that replays it: the
        step's ~40 launches then cost one or two graph launches on the host. Forward + backward and the
        SGD update are captured; with more than one rank the NCCL all-reduce stays an ordinary call
        between the two graphs (a collective is not recorded into a graph here). X and labels are
        captured by address — refill them in place for the next batch. The warm-up steps run eagerly
        first so that every scratch buffer exists before capture."""
        for _ in range(max(1, warmup)):
            self.train_step(X, labels, lr, momentum, global_rows)
        torch.cuda.synchronize()
        distributed = self._distributed()
        g_fb, g_sgd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_fb):
            self.forward_backward(X, labels, global_rows)
            if not distributed:
                self.sgd_step(lr, momentum)
        if distributed:
            with torch.cuda.graph(g_sgd):
                self.sgd_step(lr, momentum)

        def replay():
            g_fb.replay()
            if distributed:
                self.allreduce_grads()
                g_sgd.replay()
            return self.loss

        replay.graphs = (g_fb, g_sgd)
        return replay

    def train_step(self, X, labels, lr=0.1, momentum=0.9, global_rows=None):
        self.forward_backward(X, labels, global_rows)
        self.allreduce_grads()
        self.sgd_step(lr, momentum)
        return self.loss
