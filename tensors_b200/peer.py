"""Host-side helper around tfb_peer_group: maps a member's buffers as torch tensors and moves the ranks'
IPC handles through torch.distributed (the rendezvous is the host's job, not the library's)."""
import ctypes

import torch

from . import capi
from .mlp import _DeviceArray

lib = capi.lib


class PeerGroup:
    def __init__(self, capacity_floats, process_group=None):
        self.capacity = (int(capacity_floats) + 3) // 4 * 4
        self.group = process_group
        h = ctypes.c_void_p()
        capi.check(lib.tfb_peer_group_create(self.capacity, ctypes.byref(h)))
        self.handle = h
        i, o, r = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        capi.check(lib.tfb_peer_group_buffers(h, ctypes.byref(i), ctypes.byref(o), ctypes.byref(r)))
        self.region = r.value
        self.inp = torch.as_tensor(_DeviceArray(i.value, self.capacity), device="cuda")
        self.out = torch.as_tensor(_DeviceArray(o.value, self.capacity), device="cuda")
        self._connected = False

    def connect(self):
        """Collective over the process group: opens every other rank's region through CUDA IPC."""
        dist = torch.distributed
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        nbytes = int(lib.tfb_mlp_ipc_handle_bytes())
        mine = (ctypes.c_ubyte * nbytes)()
        capi.check(lib.tfb_peer_group_ipc_handle(self.handle, mine))
        gathered = [None] * world
        dist.all_gather_object(gathered, bytes(mine), group=self.group)
        capi.check(lib.tfb_peer_group_connect_ipc(self.handle, rank, world, b"".join(gathered)))
        dist.barrier(group=self.group)
        self._connected = True

    def allreduce(self, n):
        capi.check(lib.tfb_peer_allreduce_sum(self.handle, int(n), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.out[:n]

    def close(self):
        """Unmaps the peers (collective when connected: nobody frees a region another rank still maps)."""
        if self.handle is None:
            return
        lib.tfb_peer_group_connect_ptrs(self.handle, 0, 1, None)
        if self._connected:
            torch.distributed.barrier(group=self.group)
        lib.tfb_peer_group_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            if self.handle is not None:
                lib.tfb_peer_group_destroy(self.handle)
        except Exception:
            pass
