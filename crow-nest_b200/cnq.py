"""Reader and loader of the CNQ container (magic ``CNQ1``, index as a trailer): the on-disk format the engine's weights
come in. Mirrors ``Cnq`` of the reference (engine/src/cnq.rs:23-120, :174-235, :946-1135): payload blob at
``blob_offset``, index JSON followed by its u64 LE length in the last 8 bytes, tensor offsets relative to the blob,
tensors looked up by (name, section). dtypes: ``nvfp4`` (36 B per 64 values + one f32 tensor scale), ``bf16``, ``f32``,
``i64`` raw little endian. Only an index v2 is read (its ``model`` block carries the checkpoint's config, each string
checked against the sha256 recorded beside it); a v1 index is refused by name as the reference refuses every v1
container but its one container of record.

The loader half puts NVFP4 tensors on the device in the layout the kernels consume (the container's own), optionally
only a contiguous row range (the tensor-parallel shard of an [out][in] matrix), and can hand a matrix straight to the
block-scaled GEMM's repack.
"""
import hashlib
import json
import mmap
import struct

import numpy as np

V1_REFUSAL = "CNQ index v1 is only accepted for the Flash-Next CNQ4.5-M container of record"


class CnqError(ValueError):
    pass


class TensorInfo:
    __slots__ = ("name", "section", "dtype", "offset", "n_values", "global_scale", "shape", "len")

    def __init__(self, t):
        self.name, self.section, self.dtype = t["name"], t.get("section", ""), t["dtype"]
        self.offset, self.n_values = int(t["offset"]), int(t["n_values"])
        self.global_scale = float(t.get("global_scale", 1.0))
        self.shape = [int(v) for v in t.get("shape", [self.n_values])]
        self.len = int(t["len"]) if "len" in t else self.byte_len()

    def byte_len(self):
        """engine/src/cnq.rs `byte_len`: nvfp4 = 36 B per started 64 values, bf16 2, f32 4, i64 8 bytes per value."""
        if self.dtype == "nvfp4":
            return (self.n_values + 63) // 64 * 36
        return self.n_values * {"bf16": 2, "f32": 4, "i64": 8}[self.dtype]


def _classify(index_bytes, index):
    """engine/src/cnq.rs:174-235: format_version 2 with a verified model block, anything else refused by name."""
    fv = index.get("format_version")
    if fv is None:
        v = index.get("version")
        if v is not None and v != 1:
            raise CnqError(f"CNQ index `version` {v} without a `format_version` - not an index this engine reads")
        raise CnqError(f"{V1_REFUSAL} (index sha256 {hashlib.sha256(index_bytes).hexdigest()}, {len(index_bytes)} B)")
    if fv != 2:
        raise CnqError(f"CNQ index format_version {fv} is not one this engine reads (it reads 2, and v1 only for the container of record)")
    m = index.get("model")
    if not isinstance(m, dict):
        raise CnqError("CNQ index v2 without a `model` block")
    for what in ("config_json", "generation_config_json"):
        text, want = m.get(what), m.get(what + "_sha256")
        if not isinstance(text, str) or not isinstance(want, str):
            raise CnqError(f"CNQ index v2: `model.{what}` missing or not a string")
        got = hashlib.sha256(text.encode()).hexdigest()
        if got != want:
            raise CnqError(f"CNQ index v2: model.{what} hashes to {got}, the index records {want} - the stored config was altered")
    for what in ("family", "model_type"):
        if not isinstance(m.get(what), str):
            raise CnqError(f"CNQ index v2: `model.{what}` missing or not a string")
    return m


class Cnq:
    def __init__(self, path):
        self.path = path
        self.file = open(path, "rb")
        self.file.seek(0, 2)
        size = self.file.tell()
        if size < 20:
            raise CnqError(f"{path}: too short for a CNQ container")
        self.file.seek(0)
        if self.file.read(4) != b"CNQ1":
            raise CnqError(f"{path}: not a CNQ container (magic)")
        self.file.seek(size - 8)
        (n,) = struct.unpack("<Q", self.file.read(8))
        if n + 8 > size:
            raise CnqError(f"{path}: index length {n} beyond the file")
        self.file.seek(size - 8 - n)
        raw = self.file.read(n)
        self.index = json.loads(raw)
        self.model = _classify(raw, self.index)
        self.blob_offset = int(self.index["blob_offset"])
        self.tensors = [TensorInfo(t) for t in self.index["tensors"] if "name" in t]
        self.map = mmap.mmap(self.file.fileno(), 0, access=mmap.ACCESS_READ)

    # -- the reference's accessors
    def config_json(self):
        return self.model["config_json"]

    def family(self):
        return self.model["family"]

    def find(self, name, section):
        for t in self.tensors:
            if t.name == name and t.section == section:
                return t
        raise KeyError(f"tensor not found: {name} [{section}]")

    def read_range(self, t, rel_off, length):
        if rel_off < 0 or rel_off + length > t.len:
            raise CnqError(f"{t.name}: range [{rel_off}, {rel_off + length}) beyond the tensor's {t.len} bytes")
        at = self.blob_offset + t.offset + rel_off
        return np.frombuffer(self.map, np.uint8, length, at)

    def read_bytes(self, t):
        return self.read_range(t, 0, t.len)

    # -- loader
    def rows_nvfp4(self, t, r0=0, r1=None):
        """Container bytes of rows [r0, r1) of a 2-D NVFP4 tensor (rows are whole blocks, contiguous, unpadded)."""
        if t.dtype != "nvfp4" or len(t.shape) != 2:
            raise CnqError(f"{t.name}: not a 2-D nvfp4 tensor")
        rows, cols = t.shape
        if cols % 64:
            raise CnqError(f"cpu_nvfp4: {cols} columns are not whole 64-value NVFP4 blocks")
        r1 = rows if r1 is None else r1
        if not 0 <= r0 <= r1 <= rows:
            raise CnqError(f"{t.name}: rows [{r0}, {r1}) of {rows}")
        rb = cols // 64 * 36
        return self.read_range(t, r0 * rb, (r1 - r0) * rb), r1 - r0, cols

    def load_fp4(self, name, section="text", device="cuda", rank=0, world=1):
        """An ``ops.Fp4`` on the device: the whole matrix, or this rank's contiguous share of its output rows."""
        import torch

        from . import dense, ops
        t = self.find(name, section)
        lo, hi = dense.tp_rows(t.shape[0], rank, world) if world > 1 else (0, t.shape[0])
        raw, rows, cols = self.rows_nvfp4(t, lo, hi)
        w = torch.from_numpy(raw.copy()).to(device)
        gs = torch.tensor([t.global_scale], dtype=torch.float32, device=device)
        return ops.Fp4(w, gs, rows, cols)

    def load_dense(self, name, section="text", device="cuda"):
        """bf16 / f32 / i64 tensors as torch tensors of their own dtype and shape."""
        import torch
        t = self.find(name, section)
        raw = self.read_bytes(t)
        if t.dtype == "bf16":
            return torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).reshape(t.shape).to(device)
        if t.dtype == "f32":
            return torch.from_numpy(raw.view("<f4").copy()).reshape(t.shape).to(device)
        if t.dtype == "i64":
            return torch.from_numpy(raw.view("<i8").copy()).reshape(t.shape).to(device)
        raise CnqError(f"{t.name}: dtype {t.dtype} is not a dense one")

    def close(self):
        try:
            self.map.close()
        except BufferError:  # views of the mapping are still alive: it goes when they do
            pass
        self.file.close()


def write_cnq(path, tensors, model, recipe="cnq4.5-qwen35-dense"):
    """A minimal index-v2 container (for tests and synthetic checkpoints): tensors = [(name, section, dtype, shape, bytes,
    global_scale or None)]; model = dict with family, model_type, config_json, generation_config_json."""
    blob, recs, at = [], [], 0
    for name, section, dtype, shape, raw, gs in tensors:
        raw = bytes(raw)
        rec = {"name": name, "section": section, "dtype": dtype, "shape": list(shape), "n_values": int(np.prod(shape)), "offset": at, "len": len(raw)}
        if gs is not None:
            rec["global_scale"] = float(gs)
        recs.append(rec)
        blob.append(raw)
        at += len(raw)
    m = dict(model)
    for what in ("config_json", "generation_config_json"):
        m[what + "_sha256"] = hashlib.sha256(m[what].encode()).hexdigest()
    index = json.dumps({"format": "crow-nest-quant", "format_version": 2, "blob_offset": 12, "recipe": recipe, "model": m, "tensors": recs}).encode()
    with open(path, "wb") as f:
        f.write(b"CNQ1" + b"\0" * 8)
        for b in blob:
            f.write(b)
        f.write(index)
        f.write(struct.pack("<Q", len(index)))
