"""The CNQ container reader (crownest_b200/cnq.py) on the reference's own container fixture: index classification, tensor
table, raw bytes equal to what the reference's Python reader returned (tests/golden/nvfp4_dequant.npz holds its output),
and the refusals the reference makes by name (engine/src/cnq.rs:174-235, tests :1556-1700)."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

import oracle
from conftest import GOLDEN
from crownest_b200 import cnq

FIX = os.path.join(GOLDEN, "synthetic-v2.cnq")


def test_fixture_opens_as_index_v2_with_its_model_block():
    c = cnq.Cnq(FIX)
    assert c.family() == "Qwen35Dense" or isinstance(c.family(), str)
    assert json.loads(c.config_json())  # the checkpoint's config.json, verbatim and hash-checked
    assert c.blob_offset == 12 and len(c.tensors) == 15
    t = c.find("model.language_model.layers.0.linear_attn.in_proj_qkv.weight", "text")
    assert (t.dtype, t.shape, t.len) == ("nvfp4", [128, 64], 4608) and abs(t.global_scale - 9.300595411332324e-05) < 1e-12
    with pytest.raises(KeyError, match="tensor not found"):
        c.find("model.language_model.layers.0.linear_attn.in_proj_qkv.weight", "mtp")
    c.close()


def test_nvfp4_tensors_equal_the_reference_readers_bytes_and_values():
    g = np.load(os.path.join(GOLDEN, "nvfp4_dequant.npz"))
    c = cnq.Cnq(FIX)
    for i in range(int(g["cnq_count"])):
        t = c.find(str(g[f"cnq{i}_name"]), "text")
        raw = c.read_bytes(t)
        assert np.array_equal(raw, g[f"cnq{i}_raw"])
        rows, cols = t.shape
        deq = oracle.nvfp4_dequant(np.array(raw), rows, cols, np.float32(t.global_scale), rule=False)
        assert np.array_equal(deq.reshape(-1).view(np.uint32), g[f"cnq{i}_deq"].reshape(-1).view(np.uint32))
        # a row range is the matching slice of the bytes
        part, n, k = c.rows_nvfp4(t, 3, 10)
        assert (n, k) == (7, cols) and np.array_equal(part, raw[3 * cols // 64 * 36: 10 * cols // 64 * 36])
    c.close()


def _rewrite(tmp_path, edit):
    raw = open(FIX, "rb").read()
    (n,) = struct.unpack("<Q", raw[-8:])
    index = json.loads(raw[-8 - n:-8])
    edit(index)
    ib = json.dumps(index).encode()
    p = tmp_path / "edited.cnq"
    p.write_bytes(raw[:-8 - n] + ib + struct.pack("<Q", len(ib)))
    return str(p)


def test_refusals_are_named(tmp_path):
    with pytest.raises(cnq.CnqError, match="format_version 3 is not one this engine reads"):
        cnq.Cnq(_rewrite(tmp_path, lambda i: i.__setitem__("format_version", 3)))
    with pytest.raises(cnq.CnqError, match="only accepted for the Flash-Next CNQ4.5-M container of record"):
        cnq.Cnq(_rewrite(tmp_path, lambda i: i.pop("format_version")))

    def v2_without_fv(i):
        i.pop("format_version")
        i["version"] = 2
    with pytest.raises(cnq.CnqError, match="`version` 2 without a `format_version`"):
        cnq.Cnq(_rewrite(tmp_path, v2_without_fv))
    with pytest.raises(cnq.CnqError, match="the stored config was altered"):
        cnq.Cnq(_rewrite(tmp_path, lambda i: i["model"].__setitem__("config_json", i["model"]["config_json"] + " ")))
    with pytest.raises(cnq.CnqError, match="without a `model` block"):
        cnq.Cnq(_rewrite(tmp_path, lambda i: i.pop("model")))
    bad = tmp_path / "bad.cnq"
    bad.write_bytes(b"NOPE" + b"\0" * 40)
    with pytest.raises(cnq.CnqError, match="magic"):
        cnq.Cnq(str(bad))


def test_written_container_round_trips(tmp_path):
    from crownest_b200 import synth
    rng = np.random.default_rng(1)
    w = synth.nvfp4_matrix(96, 256, rng)
    norm = rng.standard_normal(256).astype(np.float32)
    p = str(tmp_path / "t.cnq")
    cnq.write_cnq(p, [("layers.0.mlp.down_proj.weight", "text", "nvfp4", (96, 256), w.tobytes(), 0.25),
                      ("layers.0.norm.weight", "text", "f32", (256,), norm.tobytes(), None)],
                  dict(family="Qwen35Dense", model_type="qwen3_5", config_json="{}", generation_config_json="{}", geo={}, source={}))
    c = cnq.Cnq(p)
    t = c.find("layers.0.mlp.down_proj.weight", "text")
    assert np.array_equal(c.read_bytes(t), w) and t.global_scale == 0.25
    assert np.array_equal(c.read_bytes(c.find("layers.0.norm.weight", "text")).view(np.float32), norm)
    c.close()
