"""The dense decode layer stack: the operator sequence the reference's ``Engine::decode_step`` runs
per layer (engine/src/gen.rs:6117-6190) reduced to its quantized projections - fused QKV, o_proj,
fused gate/up + SiLU, down - with everything that is not a GEMV left out (attention, norms and
residuals are other operators). One token (M = 1) or M <= 8 rows (``Engine::verify_rows``,
engine/src/gen.rs:5572).

Data flow per layer, chosen so that magnitudes stay bounded without the norms: the layer input x
feeds qkv, o_proj and gate/up; down reads the gate/up output h; the stack's output is the last
layer's down output. Every launch waits for its predecessor (programmatic dependent launch), as
the projections of a real decode step do.

Tensor parallelism (``world`` > 1): every matrix is split by output rows into contiguous ranges,
gate and up rows paired so the activation stays local; each rank's slice of every output is
all-gathered (NCCL) so that x and h are replicated again for the next projection.
"""
import numpy as np
import torch

from . import ops, synth
from ._lib import CrownestError


def _rand_nvfp4_device(rows, cols, gen, device, scale_sigma=0.05):
    """The benchmark's generator on the device: codes uniform over all 16 values, scale byte =
    E4M3(|N(0,1)| * sigma) (round to nearest even; never the NaN code at this magnitude)."""
    blocks = rows * cols // 64
    w = torch.randint(0, 256, (blocks, 36), dtype=torch.uint8, device=device, generator=gen)
    s = (torch.randn((blocks, 4), device=device, generator=gen).abs() * scale_sigma).to(torch.float8_e4m3fn)
    w[:, :4] = s.view(torch.uint8)
    return w.reshape(-1)


def tp_rows(n, rank, world):
    """Output rows [lo, hi) of an [n][k] matrix held by `rank`: contiguous, equal ranges."""
    if n % world:
        raise CrownestError(f"tensor parallel: {n} output rows do not split over {world} ranks")
    return rank * (n // world), (rank + 1) * (n // world)


def gather_rows(part, full, m, world, group=None):
    """All-gather the ranks' output slices part [m][n / world] into full [m][n] (rank r's columns at
    tp_rows(n, r, world)); works on any backend (NCCL on the device, gloo on the host)."""
    import torch.distributed as dist
    if m == 1:
        dist.all_gather_into_tensor(full[:1].view(-1), part.reshape(-1), group=group)
    else:
        # [world][m][n / world] -> [m][n]: gather into a staging buffer, then interleave
        tmp = torch.empty((world, m, part.shape[1]), dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(tmp.view(-1), part.reshape(-1), group=group)
        full[:m].copy_(tmp.permute(1, 0, 2).reshape(m, -1))


def line_buffer(epoch, occurrence, per_step):
    """Which of a vector's two line buffers the `occurrence`-th exchange of the vector in step `epoch` uses, as the kernels
    compute it: buf ^ (flip & epoch & 1) with buf = occurrence & 1 and flip = per_step & 1. Consecutive exchanges of a
    vector alternate, also from the last one of a step to the first of the next."""
    return (occurrence & 1) ^ ((per_step & 1) & epoch & 1)


def line_number(epoch, tag):
    """The number the lines of exchange `tag` (1..4095) of step `epoch` carry."""
    return (epoch * 4096 + tag) & 0xFFFFFFFF


def pack_lines(rows_bf16, number):
    """The 16-byte lines the GEMV's epilogue stores for output rows (uint16 bf16 bits, a multiple of four of them), as
    uint32 [lines][4] = {rows 0-1, number, rows 2-3, number}: the host twin of the kernel's packing, for tests."""
    import numpy as np
    r = np.asarray(rows_bf16, dtype=np.uint16).reshape(-1, 4).astype(np.uint32)
    out = np.empty((r.shape[0], 4), dtype=np.uint32)
    out[:, 0] = r[:, 0] | (r[:, 1] << 16)
    out[:, 2] = r[:, 2] | (r[:, 3] << 16)
    out[:, 1] = out[:, 3] = np.uint32(number)
    return out


def unpack_lines(lines, number):
    """What the receiver does with a slice's lines: None while a half of any line does not carry `number` yet, else the
    rows as uint16 bf16 bits."""
    import numpy as np
    lines = np.asarray(lines, dtype=np.uint32).reshape(-1, 4)
    if not (np.all(lines[:, 1] == np.uint32(number)) and np.all(lines[:, 3] == np.uint32(number))):
        return None
    w = np.stack([lines[:, 0], lines[:, 2]], axis=1).reshape(-1)
    return np.stack([w & 0xFFFF, w >> 16], axis=1).reshape(-1).astype(np.uint16)


class PeerExchange:
    """One buffer per rank, visible to every peer over NVLink (CUDA IPC), holding the replicated activation vectors
    of the tensor-parallel stack, plus the arrival counters of each exchange point (`cn_tp_allgather`)."""

    LINE_SLICE_MAX = 8192  # bytes: pushed by the exchange kernel, a 17 KB slice is faster as data + flag, 5 - 7 KB slices as lines (two GPUs)

    def __init__(self, vectors, rank, world, device, group=None, lines=True):
        """vectors: {name: elements}, bf16, one row; every vector's length divides by `world`. lines: slices up to
        LINE_SLICE_MAX bytes are exchanged as 16-byte lines that carry their sequence number (`cn_tp_allgather_ll`)
        instead of data followed by a flag."""
        from .peer import PeerBuffer
        self.rank, self.world, self.lines = rank, world, lines
        self.fused = lines == "fused"  # the producing GEMV stores the lines itself
        self._line_bases, self._tag, self._count, self._pending = {}, 0, {}, None
        self.per_step = {}  # exchanges of each vector per step (set by the owner of the step; odd counts alternate with the step counter)
        self.off, at = {}, 0
        for name, n in vectors.items():
            self.off[name] = (at, n * 2 // world)
            at += (n * 2 + 255) // 256 * 256
        self.flag_off = {}
        for name in vectors:
            self.flag_off[name] = at
            at += 64
        self.epoch_off = at  # the rank's step counter
        at += 64
        self.line_off = {}
        if lines:
            for name, n in vectors.items():
                if lines != "fused" and n * 2 // world > self.LINE_SLICE_MAX:
                    continue  # a long slice pushed by the exchange kernel goes as data followed by a flag: half the stores
                self.line_off[name] = at  # two line buffers (odd / even exchanges) of world slices, each twice the slice
                at += (2 * 2 * n * 2 + 255) // 256 * 256
        self.mem = PeerBuffer(at, rank, world, device, group)
        self.buf, self.bases = self.mem.buf, self.mem.bases

    def vector(self, name, n):
        """The local copy of a vector as a [1][n] bf16 tensor."""
        at, _ = self.off[name]
        return self.buf[at:at + 2 * n].view(torch.bfloat16).view(1, n)

    def begin_step(self):
        """Start of a step (fused line exchange): advance the rank's step counter, from which every exchange of the step
        takes its number, and restart the tags."""
        from ._lib import check, lib
        if not self.fused:
            return
        check(lib().cn_tp_epoch_advance(int(self.bases[self.rank]) + self.epoch_off, torch.cuda.current_stream().cuda_stream))
        self._tag = 0
        self._count = {n: 0 for n in self.line_off}

    def line_args(self, name):
        """What the producing GEMV needs to store its output rows as lines into the peers' buffers, or None when the vector
        is exchanged by a separate kernel: (addresses of the ranks' line buffers with 0 for this rank, ranks, global index
        of this rank's first row, bytes between the two line buffers, address of this rank's step counter, the exchange's
        tag within the step, its buffer, whether the buffer alternates with the step counter). exchange(name) must follow."""
        if name not in self.line_off or not self.fused:
            return None
        if name not in self._line_bases:
            import ctypes as C
            arr = (C.c_ulonglong * self.world)()
            for r in range(self.world):
                arr[r] = 0 if r == self.rank else int(self.bases[r]) + self.line_off[name]
            self._line_bases[name] = arr
        at, slice_bytes = self.off[name]
        self._tag += 1
        buf = self._count[name] & 1
        self._count[name] += 1
        self._pending = (name, self._tag, buf)
        return (self._line_bases[name], self.world, self.rank * (slice_bytes // 2), self.world * slice_bytes * 2,
                int(self.bases[self.rank]) + self.epoch_off, self._tag, buf, self.per_step.get(name, 0) & 1)

    def exchange(self, name):
        from ._lib import check, lib
        at, slice_bytes = self.off[name]
        if name in self.line_off and self.fused:
            # the lines were stored by the GEMV that produced the slice: only the receiving half is left
            pname, tag, buf = self._pending
            assert pname == name
            check(lib().cn_tp_recv_lines(int(self.bases[self.rank]), self.rank, self.world, at, slice_bytes, self.line_off[name],
                                         int(self.bases[self.rank]) + self.epoch_off, tag, buf, self.per_step.get(name, 0) & 1,
                                         torch.cuda.current_stream().cuda_stream))
        elif name in self.line_off:
            check(lib().cn_tp_allgather_ll(self.bases, self.rank, self.world, at, slice_bytes, self.line_off[name], self.flag_off[name],
                                           torch.cuda.current_stream().cuda_stream))
        else:
            check(lib().cn_tp_allgather(self.bases, self.rank, self.world, at, slice_bytes, self.flag_off[name],
                                        torch.cuda.current_stream().cuda_stream))


class DenseStack:
    def __init__(self, cfg=None, layers=None, device="cuda", seed=0, rank=0, world=1, group=None, max_m=1, dtype=torch.bfloat16,
                 exchange="nccl", gather_q=False):
        cfg = dict(cfg or synth.DENSE_27B)
        self.hidden, self.qkv, self.inter = cfg["hidden"], cfg["qkv"], cfg["inter"]
        self.layers = layers if layers is not None else cfg["layers"]
        self.rank, self.world, self.group, self.device, self.dtype = rank, world, group, device, dtype
        # Tensor parallel: the fused QKV output is split by heads and attention runs per head, so every rank keeps its own
        # slice and nothing is exchanged after that projection; o, gate/up and down outputs are needed whole by what follows
        # them. gather_q = True exchanges q as well (every projection followed by an all-gather).
        self.local_only = set() if gather_q or world == 1 else {"q"}
        for n in (self.qkv, self.hidden, self.inter):
            if n % world:
                raise CrownestError(f"tensor parallel: {n} output rows do not split over {world} ranks")
        gen = torch.Generator(device=device)
        self.w = []
        gs = torch.ones(1, dtype=torch.float32, device=device)
        for layer in range(self.layers):
            mats = {}
            for name, rows, k in synth.dense_layer_shapes(cfg):
                # every rank draws its own row range from a stream keyed by (seed, layer, matrix, rank)
                gen.manual_seed(((seed * 1000 + layer) * 8 + len(mats)) * 64 + rank)
                r = rows // world
                mats[name] = ops.Fp4(_rand_nvfp4_device(r, k, gen, device), gs, r, k)
            self.w.append(mats)
        self.max_m = max_m
        m = max_m
        self.x = torch.zeros((m, self.hidden), dtype=dtype, device=device)
        self.q = torch.empty((m, self.qkv), dtype=dtype, device=device)
        self.o = torch.empty((m, self.hidden), dtype=dtype, device=device)
        self.h = torch.empty((m, self.inter), dtype=dtype, device=device)
        self.y = torch.empty((m, self.hidden), dtype=dtype, device=device)
        self.peer = None
        if world > 1:
            # per-rank slices land here, then one all-gather per projection
            self.part = {n: torch.empty((m, r // world), dtype=dtype, device=device) for n, r in
                         (("q", self.qkv), ("o", self.hidden), ("h", self.inter), ("y", self.hidden))}
            if exchange in ("peer", "peer-lines", "peer-flags") and max_m == 1 and dtype == torch.bfloat16:
                # one activation row: the slices are written straight into a peer-visible buffer and pushed to the peers
                sizes = {"q": self.qkv, "o": self.hidden, "h": self.inter, "y": self.hidden}
                try:
                    self.peer = PeerExchange(sizes, rank, world, device, group, lines={"peer": "fused", "peer-lines": True, "peer-flags": False}[exchange])  # raises on every rank or on none
                    self.q, self.o, self.h, self.y = (self.peer.vector(n, r) for n, r in sizes.items())
                    self.peer.per_step = {n: self.layers for n in sizes if n not in self.local_only}  # once per layer each
                except CrownestError as e:  # no peer access between these GPUs: NCCL all-gather instead
                    self.peer, self.peer_error = None, str(e)
        # this library's kernels per step: four GEMVs per layer, plus one exchange kernel per exchanged vector and the step counter
        self.launches_per_step = 4 * self.layers
        if self.peer is not None:
            self.launches_per_step += (4 - len(self.local_only)) * self.layers + (1 if self.peer.fused else 0)
        self.graph = None
        self.chains = None

    def fuse(self, per_launch="token"):
        """Run the stack's projections through the balanced-share kernel (`ops.GemvSeq`): "gemv" = one launch per projection
        (every CTA an equal share of the matrix whatever its row count), "layer" = one persistent launch per layer, "token" =
        the whole stack in one. One activation row, one GPU. Every step waits for its predecessor, as the projections of a real
        decode step do."""
        if self.world != 1 or self.dtype != torch.bfloat16:
            raise CrownestError("the fused chain takes one bf16 row on one GPU")
        self.chains = []
        seq, prev = ops.GemvSeq(), None
        x = self.x[:1]
        for i, mats in enumerate(self.w):
            if per_launch == "gemv":
                for add in (lambda s: s.gemv(mats["qkv"], x, self.q[:1]), lambda s: s.gemv(mats["o"], x, self.o[:1]),
                            lambda s: s.gemv_gu(mats["gate"], mats["up"], x, self.h[:1]), lambda s: s.gemv(mats["down"], self.h[:1], self.y[:1])):
                    one = ops.GemvSeq()
                    add(one)
                    self.chains.append(one.build())
                continue
            prev = seq.gemv(mats["qkv"], x, self.q[:1], after=prev)
            prev = seq.gemv(mats["o"], x, self.o[:1], after=prev)
            prev = seq.gemv_gu(mats["gate"], mats["up"], x, self.h[:1], after=prev)
            prev = seq.gemv(mats["down"], self.h[:1], self.y[:1], after=prev)
            if per_launch == "layer" or i == len(self.w) - 1:
                self.chains.append(seq.build())
                seq, prev = ops.GemvSeq(), None
        self.launches_per_step = len(self.chains)
        return self

    # algorithmic bytes of one step over all ranks: every weight byte once, plus the tensor scale and the
    # activations in and out of each projection at the boundary dtype
    def bytes_per_step(self, m=1):
        es = 2 if self.dtype == torch.bfloat16 else 4
        per_layer_w = sum(r * k // 64 * 36 for _, r, k in synth.dense_layer_shapes(dict(hidden=self.hidden, qkv=self.qkv, inter=self.inter)))
        act = ((self.hidden + self.qkv) + 2 * self.hidden + (self.hidden + self.inter) + (self.inter + self.hidden)) * es * m
        return self.layers * (per_layer_w + act + 5 * 4)

    def weight_bytes_local(self):
        return sum(t.w.numel() for mats in self.w for t in mats.values())

    def _gather(self, name, full, m):
        gather_rows(self.part[name][:m], full, m, self.world, self.group)

    def _proj(self, w, x, name, full, m, gu=None):
        if name in self.local_only:
            lo, hi = tp_rows(full.shape[1], self.rank, self.world)
            ops.launch_gemv(w, x, full[:m, lo:hi])  # the rank's slice stays where it is: its consumer is local
            return
        if self.peer is not None:
            lo, hi = tp_rows(full.shape[1], self.rank, self.world)
            out = full[:, lo:hi]  # this rank's slice of the replicated vector, in place
        else:
            out = full[:m] if self.world == 1 else self.part[name][:m]
        lines = self.peer.line_args(name) if self.peer is not None and m == 1 else None
        if lines is not None:
            ops.launch_gemv_lines(w, x, out, lines, gu=gu)
        elif gu is None:
            ops.launch_gemv(w, x, out)
        else:
            ops.launch_gemv_gu(w, gu, x, out)
        if self.peer is not None:
            self.peer.exchange(name)
        elif self.world > 1:
            self._gather(name, full, m)

    def run_layers(self, m=1):
        """Enqueue the whole stack on the current stream (4 launches per layer, or the fused chains)."""
        if self.chains is not None and m == 1:
            for c in self.chains:
                c.run()
            return self.y[:1]
        x = self.x[:m]
        if self.peer is not None and m == 1:
            self.peer.begin_step()
        for mats in self.w:
            self._proj(mats["qkv"], x, "q", self.q, m)
            self._proj(mats["o"], x, "o", self.o, m)
            self._proj(mats["gate"], x, "h", self.h, m, gu=mats["up"])
            self._proj(mats["down"], self.h[:m], "y", self.y, m)
        return self.y[:m]

    def capture(self, m=1):
        """Record the stack into a CUDA graph (the reference captures its decode step the same way,
        engine/src/gen.rs:6100-6225)."""
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            self.run_layers(m)  # warm-up outside the capture: first-use set-up of every kernel and communicator
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                self.run_layers(m)
        self.graph, self.graph_m = g, m
        return g

    def decode_step(self, x_host, y_host):
        """Host-facing step: pinned host activations in, pinned host output back (the reference's
        embedding-row upload and result readback, engine/src/gen.rs:6071-6077, :6238-6242)."""
        m = x_host.shape[0]
        self.x[:m].copy_(x_host, non_blocking=True)
        if self.graph is not None and self.graph_m == m:
            self.graph.replay()
        else:
            self.run_layers(m)
        y_host.copy_(self.y[:m], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return y_host

    def host_copy(self, layer):
        """One layer's matrices as numpy bytes (for the CPU checker)."""
        return {n: (t.w.cpu().numpy(), t.rows, t.cols) for n, t in self.w[layer].items()}
