"""Peer-memory communicator for the fused all-reduce: one process per GPU, buffers exchanged as
CUDA IPC handles over ``torch.distributed`` (the reference exchanges raw addresses between its
per-GPU threads, tilert/models/deepseek_v3_2/modules/end2end.py:491-501)."""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

import tilert_b200 as _tb


class Comm:
    """Owns this rank's communication buffer and the mappings of the peers' buffers."""

    def __init__(self, max_rows: int, device: int):
        lib = _tb.lib()
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.device = device
        nbytes = lib.tilert_b200_comm_buffer_bytes(self.world, max_rows)
        own = ctypes.c_void_p()
        _tb.check(lib.tilert_b200_dev_alloc(nbytes, ctypes.byref(own)))
        self.own = own
        handle = (ctypes.c_uint8 * 64)()
        _tb.check(lib.tilert_b200_ipc_export(own, handle))
        mine = torch.tensor(list(handle), dtype=torch.uint8)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, mine.tolist())
        self.ptrs = (ctypes.c_void_p * self.world)()
        self.imported = []
        for r in range(self.world):
            if r == self.rank:
                self.ptrs[r] = own.value
            else:
                h = (ctypes.c_uint8 * 64)(*gathered[r])
                ptr = ctypes.c_void_p()
                _tb.check(lib.tilert_b200_ipc_import(h, ctypes.byref(ptr)))
                self.ptrs[r] = ptr.value
                self.imported.append(ptr)
        comm = ctypes.c_void_p()
        _tb.check(lib.tilert_b200_comm_create(ctypes.c_void_p(_tb.tilert_init(device)), self.world, self.rank,
                                              self.ptrs, max_rows, ctypes.byref(comm)))
        self.handle = comm.value
        dist.barrier()  # every buffer is mapped and zeroed before anyone's first call

    def close(self) -> None:
        lib = _tb.lib()
        torch.cuda.synchronize()
        dist.barrier()
        lib.tilert_b200_comm_destroy(ctypes.c_void_p(self.handle))
        for p in self.imported:
            lib.tilert_b200_ipc_close(p)
        dist.barrier()
        lib.tilert_b200_dev_free(self.own)
