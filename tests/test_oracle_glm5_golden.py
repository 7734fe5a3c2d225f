"""The CPU checker against the reference's HF-computed goldens on synthetic GLM-shaped weights
(engine/tests/fixtures/glm5/moe, checked there by engine/src/glm5_moe.rs:2546-2606): the sigmoid
router (id sets equal, weights <= 1e-6), the NVFP4 dense FFN and the MUL1 MoE layer (cosine >=
0.9999 per row). Inputs are regenerated from the seed and must hash to the golden's manifest."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN
from oracle import testkit as tk

MOE = os.path.join(GOLDEN, "glm5_moe")
COS_MIN = 0.9999
G = tk.GLM5


@pytest.fixture(scope="module")
def synth():
    s = tk.glm5_synth()
    man = json.load(open(os.path.join(MOE, "manifest.json")))
    for name, got in tk.input_shas(s).items():
        assert man["inputs_sha256"][name] == got, f"{name}: the golden was written from other inputs"
    return s, man


def raw(name, dtype, shape):
    return np.fromfile(os.path.join(MOE, name), dtype).reshape(shape)


def router_logits(s, x):
    # f64 accumulation, one rounding to f32 (engine/src/glm5_moe.rs:245-261)
    w = (s["router_w"].astype(np.uint32) << 16).view(np.float32).reshape(G["experts"], G["hidden"]).astype(np.float64)
    return (x.astype(np.float64) @ w.T).astype(np.float32)


def check_routing(ids, w, gold_ids, gold_w, tol=1e-6):
    for t in range(ids.shape[0]):
        order = np.argsort(ids[t], kind="stable")
        assert ids[t][order].tolist() == gold_ids[t].tolist(), f"row {t}: routed set differs from the oracle"
        assert np.max(np.abs(w[t][order].astype(np.float64) - gold_w[t])) <= tol


def cosine(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def test_router_matches_the_hf_golden(synth):
    s, _ = synth
    for x, ids_f, w_f, rows in ((s["x_route"], "router-ids.i32", "router-weights.f32", tk.TR), (s["x_moe"], "moe-ids.i32", "moe-weights.f32", tk.TM)):
        ids, w = oracle.route_sigmoid_topk(router_logits(s, x), s["bias"], G["topk"], G["routed_scaling"])
        check_routing(ids, w, raw(ids_f, "<i4", (rows, 8)), raw(w_f, "<f4", (rows, 8)))


def test_dense_nvfp4_ffn_matches_the_hf_golden(synth):
    s, _ = synth
    (g, i, h), (u, _, _), (d, _, _) = s["dense"]
    assert i == G["dense_inter"]
    y = oracle.nvfp4_ffn(g, u, d, h, i, [tk.NVFP4_GS] * 3, s["x_dense"], limit=G["swiglu_limit"], threads=8, path=1)
    gold = raw("dense-y.f32", "<f4", (tk.TD, h))
    for t in range(tk.TD):
        assert cosine(y[t], gold[t]) >= COS_MIN


def test_moe_layer_matches_the_hf_golden(synth):
    # engine/src/glm5_moe.rs:319-346 (`moe_cpu`): route, every needed expert once over the rows that chose
    # it, the shared expert, the combine
    s, man = synth
    h, k = G["hidden"], G["topk"]
    x = s["x_moe"]
    ids, w = oracle.route_sigmoid_topk(router_logits(s, x), s["bias"], k, G["routed_scaling"])
    check_routing(ids, w, raw("moe-ids.i32", "<i4", (tk.TM, 8)), raw("moe-weights.f32", "<f4", (tk.TM, 8)))
    (sg, si, _), (su, _, _), (sd, _, _) = s["shared"]
    ys = oracle.nvfp4_ffn(sg, su, sd, h, si, [tk.NVFP4_GS] * 3, x, limit=G["swiglu_limit"], threads=8, path=1)
    ye = np.zeros((tk.TM * k, h), np.float32)
    flat = ids.reshape(-1)
    for e in sorted(set(flat.tolist())):
        rec = tk.glm5_expert_record(e)
        assert man["records_sha256"][str(e)] == hashlib.sha256(rec.tobytes()).hexdigest(), f"expert {e}: the golden saw another record"
        combos = np.nonzero(flat == e)[0]
        out = oracle.mul1_expert_ffn(rec, h, G["expert_inter"], G["K"], x[combos // k], limit=G["swiglu_limit"], threads=8)
        ye[combos] = out
    y = oracle.moe_combine(ye, w, ys)
    gold = raw("moe-y.f32", "<f4", (tk.TM, h))
    for t in range(tk.TM):
        assert cosine(y[t], gold[t]) >= COS_MIN, t
