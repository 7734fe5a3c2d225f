"""Host-side mirror of the reference's MoE operator over NVFP4 experts.

Names follow the reference: ``GpuMoeWeights`` (device pointer tables, engine/src/glm5_moe.rs:353-376,
residency tables engine/src/residency.rs:62), ``GpuMoePlan.new / route / experts / run / free``
(engine/src/glm5_moe.rs:605-793, :1116-1124). torch owns the device memory; the plan's scratch is
allocated once by the library and released by ``free()``.
"""
import ctypes as C

import numpy as np
import torch

from . import ops
from ._lib import CN_BF16, CN_BF16_IN_F32_OUT, CN_F32, CrownestError, check, lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None else None


def route_softmax_topk(logits, k):
    """ids, wts [T][k] in pick order - router_top10's selection (engine/src/kernels.rs:3109)."""
    t, e = logits.shape
    ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    check(lib().cn_route_softmax_topk(logits.data_ptr(), ids.data_ptr(), wts.data_ptr(), t, e, k, _stream()))
    return ids, wts


def route_sigmoid_topk(logits, bias, k, scale):
    """glm5_router_sig_topk / route_from_logits (engine/src/glm5_moe.rs:196)."""
    t, e = logits.shape
    ids = torch.empty((t, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    check(lib().cn_route_sigmoid_topk(logits.data_ptr(), _ptr(bias), ids.data_ptr(), wts.data_ptr(), t, e, k, float(scale), _stream()))
    return ids, wts


class GpuMoeWeights:
    """Expert matrices behind device pointer tables. ``gate_up`` [E] list of fused [2I][H] slabs (or
    ``gate`` + ``up`` lists), ``down`` [E]; an expert given as None is not resident (null entry)."""

    def __init__(self, hidden, inter, experts, gs_gu, gs_dn, gate_up=None, gate=None, up=None, down=None, gs_up=None, shared=None,
                 shared_gs=None, device="cuda"):
        self.hidden, self.inter, self.experts = hidden, inter, experts
        self.keep = [gate_up, gate, up, down, shared]

        def table(lst):
            if lst is None:
                return None
            assert len(lst) == experts
            return torch.tensor([0 if w is None else w.data_ptr() for w in lst], dtype=torch.int64, device=device)

        self.table_gu = table(gate_up if gate_up is not None else gate)
        self.table_up = table(up) if gate_up is None else None
        self.table_dn = table(down)
        f = lambda v: None if v is None else torch.tensor([v], dtype=torch.float32, device=device)
        self.gs_gu, self.gs_up, self.gs_dn = f(gs_gu), f(gs_up), f(gs_dn)
        self.shared = shared  # (gate, up, down) device byte tensors or None
        self.shared_inter = 0 if shared is None else shared[0].numel() // (hidden // 64 * 36)
        self.shared_gs = None if shared is None else torch.tensor(list(shared_gs), dtype=torch.float32, device=device)


class GpuMoePlan:
    def __init__(self, hidden, inter, experts, topk, max_tokens, shared_inter=0):
        self.hidden, self.inter, self.experts, self.topk, self.max_tokens = hidden, inter, experts, topk, max_tokens
        h = C.c_void_p()
        check(lib().cn_moe_nvfp4_plan_create(C.byref(h), hidden, inter, shared_inter, experts, topk, max_tokens))
        self.handle = h

    new = classmethod(lambda cls, *a, **k: cls(*a, **k))

    def experts_run(self, w: GpuMoeWeights, ids, wts, x, y=None, limit=0.0, sgate=None, partial=False):
        """`experts`: everything after the routing - routed experts, shared expert, combine.
        ``partial``: bf16 x in, f32 y out - the partial sums of a rank that holds part of the experts."""
        tokens = x.shape[0]
        if y is None:
            y = torch.empty(x.shape, dtype=torch.float32, device=x.device) if partial else torch.empty_like(x)
        dt = CN_BF16 if x.dtype == torch.bfloat16 else CN_F32
        if partial:
            if x.dtype != torch.bfloat16 or y.dtype != torch.float32:
                raise CrownestError("moe partial sums: x must be bf16 and y f32")
            dt = CN_BF16_IN_F32_OUT
        sh = w.shared or (None, None, None)
        check(lib().cn_moe_nvfp4_run(self.handle, _ptr(w.table_gu), _ptr(w.table_up), _ptr(w.table_dn), _ptr(w.gs_gu), _ptr(w.gs_up),
                                     _ptr(w.gs_dn), _ptr(sh[0]), _ptr(sh[1]), _ptr(sh[2]), _ptr(w.shared_gs), _ptr(sgate),
                                     ids.data_ptr(), wts.data_ptr(), x.data_ptr(), y.data_ptr(), tokens, float(limit), dt, _stream()))
        return y

    def experts_only(self, w: GpuMoeWeights, ids, x, eo=None, eo_ptrs=None, x_div=1, limit=0.0):
        """Routed gate|up and down over ids.numel() combos (cn_moe_nvfp4_experts): combo c reads row c // x_div of x and
        writes f32 row c of `eo`, or to the device address eo_ptrs[c]."""
        combos = ids.numel()
        dt = CN_BF16 if x.dtype == torch.bfloat16 else CN_F32
        check(lib().cn_moe_nvfp4_experts(self.handle, _ptr(w.table_gu), _ptr(w.table_up), _ptr(w.table_dn), _ptr(w.gs_gu), _ptr(w.gs_up),
                                         _ptr(w.gs_dn), ids.data_ptr(), x.data_ptr(), _ptr(eo), _ptr(eo_ptrs), combos, x_div, float(limit), dt,
                                         _stream()))
        return eo

    def shared_begin(self, w: GpuMoeWeights, x, limit=0.0):
        """Enqueue the shared expert now, beside what follows on the current stream; the next finish() joins it."""
        dt = CN_BF16 if x.dtype == torch.bfloat16 else CN_F32
        check(lib().cn_moe_nvfp4_shared_begin(self.handle, _ptr(w.shared[0]), _ptr(w.shared[1]), _ptr(w.shared[2]), _ptr(w.shared_gs), x.data_ptr(),
                                              x.shape[0], float(limit), dt, _stream()))

    def finish(self, w: GpuMoeWeights, ids, wts, x, eo, y=None, limit=0.0, sgate=None, table=None):
        """Shared expert on x and the weighted sum of the expert outputs `eo` [tokens * topk][hidden] f32 (cn_moe_nvfp4_finish)."""
        tokens = x.shape[0]
        if y is None:
            y = torch.empty_like(x)
        dt = CN_BF16 if x.dtype == torch.bfloat16 else CN_F32
        sh = w.shared or (None, None, None)
        check(lib().cn_moe_nvfp4_finish(self.handle, _ptr(sh[0]), _ptr(sh[1]), _ptr(sh[2]), _ptr(w.shared_gs), _ptr(sgate), ids.data_ptr(),
                                        wts.data_ptr(), _ptr(table), x.data_ptr(), eo.data_ptr(), y.data_ptr(), tokens, float(limit), dt, _stream()))
        return y

    def run(self, w: GpuMoeWeights, logits, x, y=None, router="softmax", bias=None, scale=1.0, limit=0.0, sgate=None):
        """route + experts (GpuMoePlan::run, engine/src/glm5_moe.rs:709)."""
        if router == "softmax":
            ids, wts = route_softmax_topk(logits, self.topk)
        else:
            ids, wts = route_sigmoid_topk(logits, bias, self.topk, scale)
        self.ids, self.wts = ids, wts
        return self.experts_run(w, ids, wts, x, y, limit, sgate)

    def read_routing(self):
        """Host copy of the last routing (GpuMoePlan::read_routing, engine/src/glm5_moe.rs:1116)."""
        return self.ids.cpu().numpy(), self.wts.cpu().numpy()

    def free(self):
        if self.handle:
            check(lib().cn_moe_nvfp4_plan_destroy(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
