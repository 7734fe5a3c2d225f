"""Synthetic MoE decode workloads in the benchmark's shapes, on one GPU or expert-parallel over a
process group: the NVFP4 routed-expert step (hidden 2048, 512 experts, intermediate 512, one shared
expert, softmax top-10) and the MUL1 (EXL3, K = 3) routed step (hidden 4096, intermediate 1536, 64
experts, top-4).

Expert parallelism: expert e lives on rank e // (experts / world); the other entries of a rank's
pointer table are null, which the routed kernels skip (the reference's residency contract,
engine/src/kernels_mul1.cu:118-119). One step with B tokens per rank:
  dispatch  all-gather of the token rows and router logits (every rank sees all world * B tokens;
            the router is replicated and bit-identical on every rank),
  compute   routed experts of this rank over all tokens -> f32 partial sums,
  combine   reduce-scatter (sum) of the partial sums: each rank receives its own B rows,
  shared    the shared expert (replicated) on the rank's own rows, added after the combine.
"""
import torch

from . import moe, mul1, ops
from .dense import _rand_nvfp4_device


def ep_owner(expert, experts, world):
    """Rank that holds `expert`: contiguous blocks of experts / world."""
    return expert // (experts // world)


class MoeDecode:
    """NVFP4 routed-expert decode step (GpuMoePlan::run, engine/src/glm5_moe.rs:709)."""

    def __init__(self, tokens, device="cuda", rank=0, world=1, group=None, hidden=2048, inter=512, experts=512, topk=10, shared_inter=512,
                 seed=0):
        assert experts % world == 0
        self.tokens, self.rank, self.world, self.group, self.device = tokens, rank, world, group, device
        self.hidden, self.inter, self.experts, self.topk, self.shared_inter = hidden, inter, experts, topk, shared_inter
        gen = torch.Generator(device=device)
        gu, dn = [None] * experts, [None] * experts
        for e in range(experts):
            if ep_owner(e, experts, world) != rank:
                continue
            gen.manual_seed(seed * 100003 + e)  # an expert's bytes do not depend on the world size
            gu[e] = _rand_nvfp4_device(2 * inter, hidden, gen, device)
            dn[e] = _rand_nvfp4_device(hidden, inter, gen, device)
        gen.manual_seed(seed * 100003 + experts)
        sh = [_rand_nvfp4_device(shared_inter, hidden, gen, device), _rand_nvfp4_device(shared_inter, hidden, gen, device),
              _rand_nvfp4_device(hidden, shared_inter, gen, device)]
        one = torch.ones(1, dtype=torch.float32, device=device)
        self.shared_fp4 = [ops.Fp4(sh[0], one, shared_inter, hidden), ops.Fp4(sh[1], one, shared_inter, hidden), ops.Fp4(sh[2], one, hidden, shared_inter)]
        self.w = moe.GpuMoeWeights(hidden, inter, experts, 1.0, 1.0, gate_up=gu, down=dn, shared=sh if world == 1 else None,
                                   shared_gs=[1.0, 1.0, 1.0] if world == 1 else None, device=device)
        all_tokens = tokens * world
        self.plan = moe.GpuMoePlan(hidden, inter, experts, topk, max_tokens=all_tokens, shared_inter=shared_inter if world == 1 else 0)
        gen.manual_seed(seed * 100003 + experts + 1 + rank)
        self.x = torch.randn((tokens, hidden), device=device, generator=gen).to(torch.bfloat16)
        self.logits = torch.randn((tokens, experts), device=device, generator=gen)
        self.y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
        if world > 1:
            self.x_all = torch.empty((all_tokens, hidden), dtype=torch.bfloat16, device=device)
            self.logits_all = torch.empty((all_tokens, experts), dtype=torch.float32, device=device)
            self.part = torch.empty((all_tokens, hidden), dtype=torch.float32, device=device)
            self.own = torch.empty((tokens, hidden), dtype=torch.float32, device=device)
            self.hs = torch.empty((tokens, shared_inter), dtype=torch.bfloat16, device=device)
            self.ys = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
            self.side = torch.cuda.Stream(device=device)  # the shared expert runs beside dispatch, experts and combine
        self.launches_per_step = 5 + 2 * ((tokens + 7) // 8)  # router, sort, gate/up, down, combine, shared gate/up + down per 8 rows

    def step(self):
        """One decode step over this rank's tokens; returns y [tokens][hidden] bf16."""
        if self.world == 1:
            return self.plan.run(self.w, self.logits, self.x, self.y)
        import torch.distributed as dist
        # shared expert on the rank's own rows, 8 at a time (the kernels take up to 8 activation rows): it needs x only,
        # so it goes on a side stream that forks here and joins before the final sum (also under graph capture)
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            for t0 in range(0, self.tokens, 8):
                t1 = min(t0 + 8, self.tokens)
                ops.launch_gemv_gu(self.shared_fp4[0], self.shared_fp4[1], self.x[t0:t1], self.hs[t0:t1])
                ops.launch_gemv(self.shared_fp4[2], self.hs[t0:t1], self.ys[t0:t1])
        dist.all_gather_into_tensor(self.x_all, self.x, group=self.group)
        dist.all_gather_into_tensor(self.logits_all, self.logits, group=self.group)
        ids, wts = moe.route_softmax_topk(self.logits_all, self.topk)
        self.plan.experts_run(self.w, ids, wts, self.x_all, self.part, partial=True)
        dist.reduce_scatter_tensor(self.own, self.part, op=dist.ReduceOp.SUM, group=self.group)
        cur.wait_stream(self.side)
        torch.add(self.own, self.ys, out=self.y)  # f32 sum, rounded to bf16 once
        return self.y

    def bytes_per_step(self, ids=None):
        """Algorithmic bytes over all ranks: every distinct routed expert once, the shared expert once, activations."""
        if ids is None:
            ids, _ = moe.route_softmax_topk(self.logits, self.topk)
        distinct = int(torch.unique(ids).numel())
        per_expert = 3 * self.inter * self.hidden // 64 * 36
        shared = 3 * self.shared_inter * self.hidden // 64 * 36
        act = self.tokens * self.world * (2 * self.hidden * 2 + self.experts * 4)
        return distinct * per_expert + shared * self.world + act, distinct


def _rand_mul1_record(hidden, inter, K, gen, device):
    """One expert record in the container's layout (converter/src/mul1.rs:207-249): gate | up | down trellis from a
    uniform code stream, then six fp16 vectors (suh, svh per matrix) with |N(0,1)| * 0.02 magnitudes and random signs."""
    bits, half = mul1.bitrate(K)
    wpt = 16 * bits + (8 if half else 0)
    tb = (hidden // 16) * (inter // 16) * wpt * 2
    rec = torch.zeros(mul1.record_bytes(hidden, inter, K), dtype=torch.uint8, device=device)
    rec[:3 * tb] = torch.randint(0, 256, (3 * tb,), dtype=torch.uint8, device=device, generator=gen)
    at = 3 * tb
    for n in (hidden, inter, hidden, inter, inter, hidden):
        v = (torch.randn(n, device=device, generator=gen).abs() * 0.02 + 1e-3) * (torch.randint(0, 2, (n,), device=device, generator=gen) * 2 - 1)
        rec[at:at + 2 * n] = v.to(torch.float16).view(torch.uint8)
        at += 2 * n
    return rec


class Mul1MoeDecode:
    """MUL1 routed-expert decode step (GpuMoePlan::experts over mul1 records, engine/src/glm5_moe.rs:741-793)."""

    def __init__(self, tokens, device="cuda", rank=0, world=1, group=None, hidden=4096, inter=1536, experts=64, topk=4, K=3.0, seed=0):
        assert experts % world == 0
        self.tokens, self.rank, self.world, self.group, self.device = tokens, rank, world, group, device
        self.hidden, self.inter, self.experts, self.topk, self.K = hidden, inter, experts, topk, K
        gen = torch.Generator(device=device)
        self.recs = [None] * experts
        for e in range(experts):
            if ep_owner(e, experts, world) == rank:
                gen.manual_seed(seed * 100003 + 7 * e)
                self.recs[e] = _rand_mul1_record(hidden, inter, K, gen, device)
        self.table = torch.tensor([0 if r is None else r.data_ptr() for r in self.recs], dtype=torch.int64, device=device)
        all_tokens = tokens * world
        self.plan = mul1.Mul1Plan(hidden, inter, K, slots=all_tokens * topk, tokens=1)
        gen.manual_seed(seed * 100003 + 7 * experts + rank)
        self.x = (torch.randn((tokens, hidden), device=device, generator=gen) * 0.25).to(torch.bfloat16)
        self.logits = torch.randn((tokens, experts), device=device, generator=gen)
        self.y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
        if world > 1:
            self.x_all = torch.empty((all_tokens, hidden), dtype=torch.bfloat16, device=device)
            self.logits_all = torch.empty((all_tokens, experts), dtype=torch.float32, device=device)
            self.xf = torch.empty((all_tokens, hidden), dtype=torch.float32, device=device)
            self.part = torch.empty((all_tokens, hidden), dtype=torch.float32, device=device)
            self.own = torch.empty((tokens, hidden), dtype=torch.float32, device=device)

    def step(self):
        if self.world == 1:
            ids, wts = moe.route_softmax_topk(self.logits, self.topk)
            return self.plan.moe(self.table, ids, wts, self.x, y=self.y, limit=10.0)
        import torch.distributed as dist
        dist.all_gather_into_tensor(self.x_all, self.x, group=self.group)
        dist.all_gather_into_tensor(self.logits_all, self.logits, group=self.group)
        ids, wts = moe.route_softmax_topk(self.logits_all, self.topk)
        self.xf.copy_(self.x_all)  # f32 in, f32 partial sums out
        self.plan.moe(self.table, ids, wts, self.xf, y=self.part, limit=10.0)
        dist.reduce_scatter_tensor(self.own, self.part, op=dist.ReduceOp.SUM, group=self.group)
        self.y.copy_(self.own)
        return self.y

    def bytes_per_step(self):
        ids, _ = moe.route_softmax_topk(self.logits, self.topk)
        distinct = int(torch.unique(ids).numel())
        return distinct * mul1.record_bytes(self.hidden, self.inter, self.K) + self.tokens * self.world * (2 * self.hidden * 2 + self.experts * 4), distinct
