"""Peer-mapped buffers for the in-kernel tensor-parallel all-reduce.

No counterpart in the reference (single GPU).  Every rank owns one block of
peer-visible device memory laid out as::

    [ residual stream [H/2] x {bf16x2, tag}           ]  written by chunk owners
    [ receive buffer  [tp, H/2] x {f32, tag, f32, tag} ]  written by every rank

and maps the blocks of all other ranks (CUDA IPC through ``libmkb200.so``;
handles travel by ``torch.distributed.all_gather_object``).  ``connect``
attaches the block to a ``Globals`` whose ``tp`` field the schedule builder
created.  Nothing in the block is ever reset: values carry tags (include/mkb200.h).
"""

from __future__ import annotations

import torch

from megakernels_b200.instructions import TensorParallelState


class _DeviceMemory:
    """Lets torch wrap a raw device allocation (CUDA array interface, version 2)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 2,
        }


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class PeerBlock:
    """One rank's peer-visible block plus the mapped blocks of the other ranks."""

    def __init__(self, hidden_size: int, num_layers: int, tp_size: int, tp_rank: int, device, group=None):
        import torch.distributed as dist

        from megakernels_b200.native import mk_llama as native

        self._native = native
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.hidden_off = 0
        hidden_bytes = hidden_size * 4  # every bf16 pair travels with a 4-byte tag
        self.recv_off = _round_up(hidden_bytes, 256)
        recv_bytes = tp_size * hidden_size * 8  # every fp32 pair travels with two 4-byte tags
        self.nbytes = self.recv_off + _round_up(recv_bytes, 256)

        torch.cuda.set_device(device)
        self.local_ptr, handle = native.peer_alloc(self.nbytes)
        handles: list = [None] * tp_size
        dist.all_gather_object(handles, handle, group=group)
        self.ptrs = [
            self.local_ptr if r == tp_rank else native.peer_open(handles[r]) for r in range(tp_size)
        ]
        self._raw = torch.as_tensor(_DeviceMemory(self.local_ptr, self.nbytes), device=device)
        self.hidden_tagged = self._raw[:hidden_bytes].view(torch.int32).view(hidden_size // 2, 2)
        self.recv = self._raw[self.recv_off : self.recv_off + recv_bytes].view(torch.int32).view(
            tp_size, hidden_size // 2, 4
        )
        # nobody may start storing into a block before every rank has mapped every block
        dist.barrier(group=group)

    def close(self):
        """Unmap the peers and free the local block (all ranks, after their last launch)."""
        if self.ptrs is None:
            return
        torch.cuda.synchronize()
        for r, ptr in enumerate(self.ptrs):
            if r != self.tp_rank:
                self._native.peer_close(ptr)
        self.hidden_tagged = self.recv = self._raw = None
        self._native.peer_free(self.local_ptr)
        self.ptrs = None


def connect(globs, group=None) -> PeerBlock:
    """Allocate and exchange the peer buffers for ``globs.tp`` (collective over ``group``)."""
    tp: TensorParallelState = globs.tp
    assert tp is not None, "build the schedule with LatencyScheduleOptions(tp_all_reduce_chunks=...)"
    H, L = globs.hidden_size, globs.num_hidden_layers
    block = PeerBlock(H, L, tp.size, tp.rank, globs.device, group)
    slices = max(globs.num_o_proj_col_splits(), globs.num_down_proj_col_splits())
    tp.partial = torch.zeros(slices, H, dtype=torch.float32, device=globs.device)
    tp.recv, tp.hidden_tagged = block.recv, block.hidden_tagged
    tp.epoch_device = torch.zeros(1, dtype=torch.int32, device=globs.device)
    tp.epoch = 0
    tp.hidden_ptrs = [p + block.hidden_off for p in block.ptrs]
    tp.recv_ptrs = [p + block.recv_off for p in block.ptrs]
    return block
