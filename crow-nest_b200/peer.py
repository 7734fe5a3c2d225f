"""One device buffer per rank that every peer of the node has mapped over NVLink (CUDA IPC): the memory the
tensor-parallel and expert-parallel exchanges (`cn_tp_allgather`, `cn_ep_dispatch` / `cn_ep_return`) store into.
Setting one up is collective: all ranks of `group` call the constructor together, and either all succeed or all raise."""
import ctypes as C

import torch

from ._lib import CrownestError, check, lib


class PeerBuffer:
    def __init__(self, nbytes, rank, world, device, group=None):
        import torch.distributed as dist
        self.rank, self.world = rank, world
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        # a rank whose export or open fails still takes part in every step, and all ranks raise together
        handle, offset, err = C.create_string_buffer(64), C.c_size_t(0), None
        try:
            check(lib().cn_peer_export(self.buf.data_ptr(), handle, C.byref(offset)))
        except CrownestError as e:
            err = str(e)
        everyone = [None] * world
        dist.all_gather_object(everyone, (bytes(handle.raw), int(offset.value), err), group=group)
        self.bases = (C.c_void_p * world)()
        self.opened = []
        if not any(e for _, _, e in everyone):
            for r, (h, o, _) in enumerate(everyone):
                if r == rank:
                    self.bases[r] = self.buf.data_ptr()
                    continue
                p = C.c_void_p()
                try:
                    check(lib().cn_peer_open(h, o, C.byref(p)))
                except CrownestError as e:
                    err = str(e)
                    break
                self.bases[r] = p.value
                self.opened.append((p.value, o))
        errs = [None] * world
        dist.all_gather_object(errs, err, group=group)
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every buffer is zeroed and open before the first exchange
        bad = [e for e in errs if e] + [e for _, _, e in everyone if e]
        if bad:
            raise CrownestError("peer memory unavailable: " + bad[0])


def ep_layout(world, cap, hidden):
    """Byte offsets of the expert-parallel exchange buffer (see cn_ep_dispatch): inbox_x, inbox_meta, ret, flags, total."""
    up = lambda n: (n + 255) // 256 * 256
    inbox_x = 0
    inbox_meta = up(world * cap * hidden * 2)
    ret = inbox_meta + up(world * cap * 8)
    flags = ret + up(cap * hidden * 4)
    return inbox_x, inbox_meta, ret, flags, flags + up(int(lib().cn_ep_flag_bytes()))


def ep_owner(expert, experts, world):
    """Rank that holds `expert`: contiguous blocks of experts / world."""
    return expert // (experts // world)


def ep_slots(ids, experts, world):
    """The placement rule of cn_ep_dispatch, on the host (numpy ids [combos]): for every destination rank the combos
    sent to it in the order they land in its inbox (sorted by expert, stable). Returns a list of arrays."""
    import numpy as np
    ids = np.asarray(ids).reshape(-1)
    key = np.where((ids < 0) | (ids >= experts), experts, ids)
    order = np.argsort(key, kind="stable")
    epr = experts // world
    return [order[(key[order] // epr) == r] for r in range(world)]


class EpExchange:
    """The expert-parallel exchange buffer of one rank plus the per-slot arrays the routed kernels read."""

    def __init__(self, tokens, topk, hidden, experts, rank, world, device, group=None):
        self.rank, self.world, self.topk, self.hidden, self.experts = rank, world, topk, hidden, experts
        self.cap = tokens * topk
        self.off = ep_layout(world, self.cap, hidden)
        self.peer = PeerBuffer(self.off[4], rank, world, device, group)
        buf = self.peer.buf
        n = world * self.cap
        self.inbox_x = buf[self.off[0]:self.off[0] + n * hidden * 2].view(torch.bfloat16).view(n, hidden)
        self.ret = buf[self.off[2]:self.off[2] + self.cap * hidden * 4].view(torch.float32).view(self.cap, hidden)
        self.ids_in = torch.full((n,), -1, dtype=torch.int32, device=device)
        self.out_ptrs = torch.zeros(n, dtype=torch.int64, device=device)
        self.order = torch.empty(self.cap, dtype=torch.int32, device=device)
        self.slots = n

    def _args(self):
        return (self.peer.bases, self.rank, self.world, self.cap, self.hidden, self.off[0], self.off[1], self.off[2], self.off[3])

    def dispatch(self, ids, x):
        """ids [tokens][topk] int32, x [tokens][hidden] bf16 (this rank's); afterwards inbox_x / ids_in / out_ptrs are set."""
        st = torch.cuda.current_stream().cuda_stream
        combos = ids.numel()
        check(lib().cn_moe_sort(ids.data_ptr(), self.order.data_ptr(), combos, self.experts, st))
        check(lib().cn_ep_dispatch(*self._args(), ids.data_ptr(), self.order.data_ptr(), x.data_ptr(), combos, self.topk, self.experts,
                                   self.ids_in.data_ptr(), self.out_ptrs.data_ptr(), st))

    def finish(self, eo=None):
        """Return meeting; with `eo` [world * cap][hidden] f32 the rows are copied to their source ranks first."""
        check(lib().cn_ep_return(*self._args(), None if eo is None else eo.data_ptr(), self.ids_in.data_ptr(), self.out_ptrs.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream))
