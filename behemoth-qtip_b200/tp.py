"""Tensor-parallel decode with the gather fused into the product kernel (qtip_multiply_push / qtip_gather_wait).

Every rank owns one exchange buffer that all ranks address directly; a rank's products go straight from the product
kernel into every rank's gathered buffer over NVLink. Takes the place of Rank::multiply + ncclAllGather of the
reference's tensor-parallel model (runtime/cuda/tensor_model.cpp:444-502). torch.distributed is used once, at set-up,
to exchange the inter-process handles.
"""
import ctypes as C

import torch

from ._lib import QtipTpExchange, lib
from .codec import _p, _stream, init


class Exchange:
    """One rank's view of the exchange: the local buffer (owned) and the peers' buffers (mapped)."""

    def __init__(self, rank, ranks, nbytes, local, bases, imported=()):
        self.rank, self.ranks, self.nbytes = rank, ranks, nbytes
        self._local, self._imported = local, list(imported)
        self.pod = QtipTpExchange()
        for p in range(ranks):
            self.pod.base[p] = bases[p]
        self.pod.bytes, self.pod.rank, self.pod.ranks = nbytes, rank, ranks
        self.uses = 0  # consecutive uses alternate the two slots

    @staticmethod
    def nbytes_for(out_full, max_tokens=1, max_splits=1):
        return int(lib().raw("qtip_tp_exchange_bytes")(out_full, max_tokens, max_splits))

    @staticmethod
    def alloc(nbytes):
        init()
        ptr = C.c_void_p()
        lib().call("qtip_tp_alloc", nbytes, C.byref(ptr))
        return ptr.value

    @classmethod
    def local_group(cls, ranks, out_full, max_tokens=1, max_splits=1):
        """All ranks of a group inside ONE process on the current device (their launches run one after another on one
        stream): the single-GPU stand-in for the multi-GPU exchange, used by tests."""
        nbytes = cls.nbytes_for(out_full, max_tokens, max_splits)
        bases = [cls.alloc(nbytes) for _ in range(ranks)]
        return [cls(r, ranks, nbytes, bases[r], bases) for r in range(ranks)]

    @classmethod
    def from_process_group(cls, out_full, max_tokens=1, max_splits=1, group=None):
        """One process per GPU: allocate the local buffer, trade inter-process handles through torch.distributed, map
        the peers' buffers. Collective over `group`."""
        import torch.distributed as dist
        rank, ranks = dist.get_rank(group), dist.get_world_size(group)
        nbytes = cls.nbytes_for(out_full, max_tokens, max_splits)
        local = cls.alloc(nbytes)
        handle = C.create_string_buffer(64)
        lib().call("qtip_tp_export", C.c_void_p(local), handle)
        handles = [None] * ranks
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        bases, imported = [], []
        for p in range(ranks):
            if p == rank:
                bases.append(local)
                continue
            ptr = C.c_void_p()
            lib().call("qtip_tp_import", C.create_string_buffer(handles[p], 64), C.byref(ptr))
            bases.append(ptr.value)
            imported.append(ptr.value)
        ex = cls(rank, ranks, nbytes, local, bases, imported)
        ex.reset()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        return ex

    def reset(self):
        lib().call("qtip_tp_reset", C.byref(self.pod), _stream())
        self.uses = 0

    def next_slot(self):
        slot = self.uses & 1
        self.uses += 1
        return slot

    def multiply_push(self, w_shard, rotated, slot, out_full, row0, splits=1, tokens=1, wait=False):
        """wait=True: the push kernel's last CTA also waits for the peers (every rank on a GPU of its own, only)."""
        lib().call("qtip_multiply_push", w_shard.pod, _p(rotated, torch.bfloat16), C.byref(self.pod), slot, out_full,
                   row0, splits, _stream(), tokens, int(wait))

    def gathered(self, slot):
        z = C.c_void_p()
        lib().call("qtip_gathered_products", C.byref(self.pod), slot, C.byref(z))
        return z.value

    def gather_wait(self, slot):
        """Enqueues the bounded wait for every rank's push of this slot; returns the device address of the gathered z."""
        z = C.c_void_p()
        lib().call("qtip_gather_wait", C.byref(self.pod), slot, C.byref(z), _stream())
        return z.value

    def check(self):
        """Synchronises the current stream; raises QtipError if a wait of this rank ran out."""
        lib().call("qtip_tp_status", C.byref(self.pod), _stream())

    def close(self, free_local=True):
        for ptr in self._imported:
            lib().call("qtip_tp_close", C.c_void_p(ptr))
        self._imported = []
        if free_local and self._local:
            lib().call("qtip_tp_free", C.c_void_p(self._local))
            self._local = None


def forward_tp(ex, w_full, w_shard, row0, x, y, scratch, rotated, round_z=False, splits=1, tokens=1, wait_inside=True):
    """One tensor-parallel projection on this rank: input transform, products pushed to every rank, bounded wait for
    the peers' products (inside the push kernel, or as a kernel of its own with wait_inside=False), output transform on
    the gathered z. Every rank ends with the full y. One process per GPU."""
    from . import linear
    slot = ex.next_slot()
    linear.qtip_prepare(w_shard, x, scratch, rotated, tokens)
    ex.multiply_push(w_shard, rotated, slot, w_full.n_out, row0, splits, tokens, wait_inside)
    z = ex.gathered(slot) if wait_inside else ex.gather_wait(slot)
    linear.qtip_finish(w_full, z, y, scratch, round_z, splits, tokens)
