"""Data-parallel MLP training step: a thin ctypes caller of the tfb_mlp object of libtfb.

The step itself — Linear -> ReLU -> Linear -> ReLU -> Linear -> log_softmax + mean NLL -> backward ->
gradient exchange -> SGD with momentum (the dataflow of the reference's examples/train_mlp.cpp:161-183,
update as documented in nn/optim/SGD.hpp:3-6) — lives in C++ behind the C-ABI (csrc/mlp_step.cu) and
owns every device buffer. This module only maps those buffers as torch tensors for tests and
benchmarks and moves the ranks' IPC handles through torch.distributed, which is the host's job.

Two ways to exchange gradients between ranks:
  exchange="peer"  the fused reduce-scatter / SGD / all-gather kernel over NVLink peer memory
                   (tfb_mlp_exchange_update); the ranks' exchange regions are opened through CUDA IPC.
  exchange="nccl"  ONE torch.distributed all-reduce over the flat gradient buffer, whose last slot
                   carries the loss, followed by tfb_mlp_update.
With device="cpu" the class only keeps the flat layout and the all-reduce (host logic, for CPU tests).
"""
import ctypes

import torch


def shard_rows(global_rows, rank, world):
    """Contiguous row range [begin, end) of the global batch that `rank` owns (sizes differ by at most 1)."""
    base, extra = divmod(int(global_rows), int(world))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def flat_layout(dims):
    """Offsets of (weight 0, bias 0, weight 1, ...) in the flat buffers and their total length: every
    segment is padded to a multiple of 4 floats, the layout tfb_mlp_segment reports."""
    offsets, off = [], 0
    for i in range(len(dims) - 1):
        for sz in (dims[i + 1] * dims[i], dims[i + 1]):
            offsets.append(off)
            off += (sz + 3) // 4 * 4
    return offsets, off


class _DeviceArray:
    """Exposes library-owned device memory to torch through the CUDA array interface."""

    def __init__(self, ptr, n, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 2}


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class MLP:
    """dims = (d0, d1, ..., dL): L Linear layers, ReLU after all but the last."""

    P_PARAMS, P_GRADS, P_VELOCITY, P_LOSS, P_REDUCED, P_ACT, P_REGION = range(7)
    CAP_STEP, CAP_FB, CAP_UPDATE = range(3)
    OPT_WAIT_NS, OPT_CTAS, OPT_KEEP_REDUCED, OPT_TRACE, OPT_BUCKETS = range(5)

    def __init__(self, dims, weights, biases=None, device="cuda", process_group=None, max_rows=8192,
                 exchange="peer"):
        self.dims = tuple(int(d) for d in dims)
        self.L = len(self.dims) - 1
        self.offsets, self.numel = flat_layout(self.dims)
        self.group = process_group
        self.exchange = exchange
        self.handle = None
        self.max_rows = int(max_rows)
        self._rows = 0
        self._graph = None
        if device == "cpu":
            self.params = torch.zeros(self.numel)
            self.grads_and_loss = torch.zeros(self.numel + 4)
            self.velocity = torch.zeros(self.numel)
            self.loss = torch.zeros(1)
        else:
            from . import capi
            self.capi, self.lib = capi, capi.lib
            arr = (ctypes.c_int64 * (self.L + 1))(*self.dims)
            h = ctypes.c_void_p()
            capi.check(self.lib.tfb_mlp_create(self.L, arr, self.max_rows, ctypes.byref(h)))
            self.handle = h
            assert int(self.lib.tfb_mlp_numel(h)) == self.numel
            for i in range(self.L):
                wo, bo = ctypes.c_int64(), ctypes.c_int64()
                capi.check(self.lib.tfb_mlp_segment(h, i, ctypes.byref(wo), ctypes.byref(bo)))
                assert (wo.value, bo.value) == (self.offsets[2 * i], self.offsets[2 * i + 1])
            self.params = self._map(self.P_PARAMS, self.numel)
            self.grads_and_loss = self._map(self.P_GRADS, self.numel + 4)
            self.velocity = self._map(self.P_VELOCITY, self.numel)
            self.loss = self._map(self.P_LOSS, 1)
            self.reduced = self._map(self.P_REDUCED, self.numel)
        self.grads = self.grads_and_loss[:self.numel]
        for i in range(self.L):
            self.weight(i).copy_(torch.as_tensor(weights[i], dtype=torch.float32).reshape(self.dims[i + 1], self.dims[i]))
            if biases is not None and biases[i] is not None:
                self.bias(i).copy_(torch.as_tensor(biases[i], dtype=torch.float32))
        self._connected = False

    def __del__(self):
        try:
            if self.handle is not None:
                self.lib.tfb_mlp_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # ---- buffers ---------------------------------------------------------------------------------
    def _ptr(self, which, layer=0):
        p = ctypes.c_void_p()
        self.capi.check(self.lib.tfb_mlp_buffer(self.handle, which, layer, ctypes.byref(p)))
        return p.value

    def _map(self, which, n, layer=0):
        return torch.as_tensor(_DeviceArray(self._ptr(which, layer), n), device="cuda")

    def _seg(self, buf, k, shape):
        n = 1
        for s in shape:
            n *= s
        return buf[self.offsets[k]:self.offsets[k] + n].view(*shape)

    def weight(self, i, buf=None):
        return self._seg(self.params if buf is None else buf, 2 * i, (self.dims[i + 1], self.dims[i]))

    def bias(self, i, buf=None):
        return self._seg(self.params if buf is None else buf, 2 * i + 1, (self.dims[i + 1],))

    def activation(self, i):
        """Output of layer i of the last forward pass, [rows, dims[i + 1]] (a view of library memory)."""
        return self._map(self.P_ACT, self._rows * self.dims[i + 1], i).view(self._rows, self.dims[i + 1])

    @property
    def _acts(self):
        return [None] + [self.activation(i) for i in range(self.L)]

    def set_option(self, option, value):
        self.capi.check(self.lib.tfb_mlp_set_option(self.handle, option, int(value)))

    # ---- group -----------------------------------------------------------------------------------
    def _distributed(self):
        """exchange="local" keeps a handle out of the process group (a single-rank reference run next to
        a distributed one)."""
        if self.exchange == "local":
            return False
        return self.group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                          and torch.distributed.get_world_size() > 1)

    def connect(self):
        """Opens the other ranks' exchange regions (CUDA IPC handles gathered through the process group).
        Collective: every rank of the group calls it; raises on every rank if any rank could not map its
        peers (the group then stays unconnected and the NCCL exchange remains available)."""
        if self._connected or not self._distributed():
            return
        dist = torch.distributed
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        nbytes = int(self.lib.tfb_mlp_ipc_handle_bytes())
        mine = (ctypes.c_ubyte * nbytes)()
        rc = self.lib.tfb_mlp_ipc_handle(self.handle, mine)
        gathered = [None] * world
        dist.all_gather_object(gathered, bytes(mine) if rc == 0 else b"", group=self.group)
        err = ""
        if all(len(g) == nbytes for g in gathered):
            rc = self.lib.tfb_mlp_connect_ipc(self.handle, rank, world, b"".join(gathered))
        if rc != 0:
            err = self.capi.last_error()
        ok = torch.tensor([0.0 if rc != 0 else 1.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)   # also the barrier: all peers are mapped
        if ok.item() == 0:
            self.disconnect()
            raise RuntimeError("peer exchange unavailable: " + (err or "another rank could not map its peers"))
        self._connected = True

    def disconnect(self):
        """Unmaps the peers' regions. Collective when distributed: a region must not be freed while
        another process still maps it, so every rank unmaps first and then all meet at a barrier."""
        if self.handle is not None:
            self.lib.tfb_mlp_connect_ptrs(self.handle, 0, 1, None)
        if self._connected and self._distributed():
            torch.distributed.barrier(group=self.group)
        self._connected = False

    # ---- the step --------------------------------------------------------------------------------
    def forward_backward(self, X, labels, global_rows=None):
        """Fills self.grads (this rank's share of the full-batch gradient) and its loss contribution."""
        self._rows = int(X.shape[0])
        self.capi.check(self.lib.tfb_mlp_forward_backward(self.handle, _p(X), _p(labels), self._rows,
                                                          int(global_rows or self._rows), _stream()))
        return self.grads_and_loss[self.numel:self.numel + 1]

    def allreduce_grads(self):
        """One collective: the flat gradient buffer with the loss contribution in its last slot."""
        if self._distributed():
            torch.distributed.all_reduce(self.grads_and_loss, group=self.group)

    def sgd_step(self, lr, momentum):
        if self.handle is None:
            self.loss[0] = self.grads_and_loss[self.numel]
            return
        self.capi.check(self.lib.tfb_mlp_update(self.handle, float(lr), float(momentum), _stream()))

    def exchange_update(self, lr, momentum):
        self.capi.check(self.lib.tfb_mlp_exchange_update(self.handle, float(lr), float(momentum), _stream()))

    def _use_peer(self):
        return self.exchange == "peer" and self._distributed()

    def train_step(self, X, labels, lr=0.1, momentum=0.9, global_rows=None):
        if self._use_peer():
            # the whole step behind one call: with two exchange buckets (OPT_BUCKETS) the library overlaps
            # the first of them with the end of the backward pass
            self.connect()
            self._rows = int(X.shape[0])
            self.capi.check(self.lib.tfb_mlp_step(self.handle, _p(X), _p(labels), self._rows,
                                                  int(global_rows or self._rows), float(lr), float(momentum), _stream()))
        else:
            self.forward_backward(X, labels, global_rows)
            self.allreduce_grads()
            self.sgd_step(lr, momentum)
        return self.loss

    def capture_train_step(self, X, labels, lr=0.1, momentum=0.9, global_rows=None, warmup=2):
        """Records one training step into CUDA graphs held by the library and returns a callable that
        replays it. With the peer exchange (or a single rank) the whole step is one graph; with the NCCL
        exchange forward + backward is a graph, the all-reduce an ordinary call after it, and the update
        a second handle-free launch. X and labels are captured by address — refill them in place. The
        warm-up steps run eagerly first so that every scratch buffer exists before capture."""
        for _ in range(max(1, warmup)):
            self.train_step(X, labels, lr, momentum, global_rows)
        torch.cuda.synchronize()
        rows, g = int(X.shape[0]), int(global_rows or X.shape[0])
        self._rows = rows
        side = torch.cuda.Stream()
        whole = self._use_peer() or not self._distributed()
        what = self.CAP_STEP if whole else self.CAP_FB
        self.capi.check(self.lib.tfb_mlp_capture_step(self.handle, _p(X), _p(labels), rows, g, float(lr), float(momentum),
                                                      what, ctypes.c_void_p(side.cuda_stream)))
        torch.cuda.synchronize()

        def replay():
            self.capi.check(self.lib.tfb_mlp_replay(self.handle, _stream()))
            if not whole:
                self.allreduce_grads()
                self.sgd_step(lr, momentum)
            return self.loss

        return replay
