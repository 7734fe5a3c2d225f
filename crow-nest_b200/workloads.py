"""Synthetic MoE decode workloads in the benchmark's shapes, on one GPU or expert-parallel over a
process group: the NVFP4 routed-expert step (hidden 2048, 512 experts, intermediate 512, one shared
expert, softmax top-10) and the MUL1 (EXL3, K = 3) routed step (hidden 4096, intermediate 1536, 64
experts, top-4).

Expert parallelism: expert e lives on rank e // (experts / world); the other entries of a rank's
pointer table are null. One step with B tokens per rank (all-to-all over NVLink peer memory, `peer.EpExchange`):
  route     every rank routes its own B tokens,
  dispatch  the activation row of every (token, expert) combo goes to the rank that holds the expert, and only there,
  compute   a rank runs its experts over the rows it received (B * topk / world combos on average, whatever the
            world size), the down projection storing each result straight into the token's home rank,
  return    the ranks meet; every rank now holds the expert outputs of its own combos,
  combine   weighted sum in pick order plus the shared expert (replicated), on the token's home rank: the same sum,
            in the same order, as on one GPU.
"""
import torch

from . import moe, mul1, ops
from .dense import _rand_nvfp4_device
from .peer import EpExchange, ep_owner


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
        self.w = moe.GpuMoeWeights(hidden, inter, experts, 1.0, 1.0, gate_up=gu, down=dn, shared=sh, shared_gs=[1.0, 1.0, 1.0], device=device)
        self.plan = moe.GpuMoePlan(hidden, inter, experts, topk, max_tokens=tokens, shared_inter=shared_inter)
        gen.manual_seed(seed * 100003 + experts + 1 + rank)
        self.x = torch.randn((tokens, hidden), device=device, generator=gen).to(torch.bfloat16)
        self.logits = torch.randn((tokens, experts), device=device, generator=gen)
        self.y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
        if world > 1:
            self.ep = EpExchange(tokens, topk, hidden, experts, rank, world, device, group)
            # the rows a rank receives are one combo each: a second plan with top-1 geometry over all inbox slots
            self.plan_in = moe.GpuMoePlan(hidden, inter, experts, 1, max_tokens=self.ep.slots)
        self.launches_per_step = 5 + 2 * ((tokens + 7) // 8) + (5 if world > 1 else 0)

    def step(self):
        """One decode step over this rank's tokens; returns y [tokens][hidden] bf16."""
        if self.world == 1:
            return self.plan.run(self.w, self.logits, self.x, self.y)
        ids, wts = moe.route_softmax_topk(self.logits, self.topk)
        self.ids, self.wts = ids, wts
        self.plan.shared_begin(self.w, self.x)  # beside dispatch, experts and return
        self.ep.dispatch(ids, self.x)
        self.plan_in.experts_only(self.w, self.ep.ids_in, self.ep.inbox_x, eo_ptrs=self.ep.out_ptrs, x_div=1)
        self.ep.finish()
        return self.plan.finish(self.w, ids, wts, self.x, self.ep.ret, self.y)

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
        self.plan = mul1.Mul1Plan(hidden, inter, K, slots=tokens * topk * world, tokens=1)
        gen.manual_seed(seed * 100003 + 7 * experts + rank)
        self.x = (torch.randn((tokens, hidden), device=device, generator=gen) * 0.25).to(torch.bfloat16)
        self.logits = torch.randn((tokens, experts), device=device, generator=gen)
        self.y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
        if world > 1:
            self.ep = EpExchange(tokens, topk, hidden, experts, rank, world, device, group)
            self.eo = torch.empty((self.ep.slots, hidden), dtype=torch.float32, device=device)
        self.launches_per_step = 11 + (6 if world > 1 else 0)

    def step(self):
        ids, wts = moe.route_softmax_topk(self.logits, self.topk)
        if self.world == 1:
            return self.plan.moe(self.table, ids, wts, self.x, y=self.y, limit=10.0)
        from ._lib import CN_BF16, check, lib
        self.ids, self.wts = ids, wts
        self.ep.dispatch(ids, self.x)
        self.plan.experts_only(self.table, self.ep.ids_in, self.ep.inbox_x, self.eo, x_div=1, limit=10.0)
        self.ep.finish(self.eo)
        check(lib().cn_moe_combine(self.ep.ret.data_ptr(), wts.data_ptr(), ids.data_ptr(), None, None, None, self.y.data_ptr(), self.tokens,
                                   self.hidden, self.topk, self.experts, CN_BF16, torch.cuda.current_stream().cuda_stream))
        return self.y

    def bytes_per_step(self):
        ids, _ = moe.route_softmax_topk(self.logits, self.topk)
        distinct = int(torch.unique(ids).numel())
        return distinct * mul1.record_bytes(self.hidden, self.inter, self.K) + self.tokens * self.world * (2 * self.hidden * 2 + self.experts * 4), distinct
