"""Regenerates tests/golden/ from a checkout of the reference (needed only when the fixtures change).

    python tests/golden/make_golden.py /path/to/reference

What it writes, and where it comes from:
- nvfp4_dequant.npz: NVFP4 tensors dequantised by the reference's own Python block decoder
  (oracle/cnq_weights.py, imported and run): the six NVFP4 tensors of the reference's container
  fixture engine/tests/fixtures/synthetic-v2/synthetic-v2.cnq, plus one seeded matrix that holds
  every scale byte (0x7F and bit 7 among them) decoded with and without the 0x7F -> 0x7E rule.
- synthetic-v2.cnq: the reference's container fixture itself, byte for byte (data, not source), for the container reader.
- exl3-mul1-*.{tsv,bin}, fp8-*.tsv: the reference's golden vectors for the MUL1 codec and the
  FP8 codec, copied byte for byte (data, not source).
- glm5_moe/*: the HF-computed goldens of the sigmoid router, the NVFP4 dense FFN and the MUL1
  MoE layer, with their manifest, copied byte for byte.
"""
import os
import shutil
import sys

import numpy as np


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(ref, "oracle"))
    from cnq_weights import CnqReader  # the reference's decoder

    out = {}
    rd = CnqReader(os.path.join(ref, "engine/tests/fixtures/synthetic-v2/synthetic-v2.cnq"))
    names = [n for n, t in rd.tensors.items() if t["dtype"] == "nvfp4"]
    for i, n in enumerate(names):
        t = rd.tensors[n]
        out[f"cnq{i}_name"] = np.array(n)
        out[f"cnq{i}_shape"] = np.array(t["shape"], np.int64)
        out[f"cnq{i}_gs"] = np.array(t["global_scale"], np.float64)
        out[f"cnq{i}_raw"] = np.frombuffer(rd.raw_bytes(n), np.uint8).copy()
        out[f"cnq{i}_deq"] = rd.tensor_f32(n).numpy().astype(np.float32)
    out["cnq_count"] = np.array(len(names))

    # every scale byte x every code: 64 rows x 256 columns, scale byte = (4 * block + sub) % 256
    rng = np.random.default_rng(20261125)
    rows, cols = 64, 256
    blocks = rows * cols // 64
    raw = rng.integers(0, 256, size=(blocks, 36), dtype=np.uint8)
    raw[:, :4] = (np.arange(blocks * 4, dtype=np.int64) % 256).astype(np.uint8).reshape(blocks, 4)
    gs = np.float32(2.3e-4)
    for rule in (False, True):
        rd.sanitize_sf = rule
        deq = rd._deq_flat(raw.tobytes(), gs).astype(np.float32)
        out["all_deq_rule" if rule else "all_deq_raw"] = deq.reshape(rows, cols)
    out["all_raw"] = raw.reshape(-1)
    out["all_gs"] = np.array(gs, np.float32)
    np.savez_compressed(os.path.join(here, "nvfp4_dequant.npz"), **out)

    # the container fixture itself (data: 66 KB), for the container reader's test
    shutil.copyfile(os.path.join(ref, "engine/tests/fixtures/synthetic-v2/synthetic-v2.cnq"), os.path.join(here, "synthetic-v2.cnq"))

    fx = os.path.join(ref, "converter/tests/fixtures")
    for f in ("exl3-mul1-decode.tsv", "exl3-mul1-glm-sizes.tsv", "exl3-mul1-q-k2.bin", "exl3-mul1-q-k3.bin",
              "exl3-mul1-q-k3.5.bin", "exl3-mul1-q-k4.bin", "fp8-e4m3fn-lut.tsv", "fp8-dequant.tsv"):
        shutil.copyfile(os.path.join(fx, f), os.path.join(here, f))
    moe = os.path.join(here, "glm5_moe")
    os.makedirs(moe, exist_ok=True)
    src = os.path.join(ref, "engine/tests/fixtures/glm5/moe")
    for f in os.listdir(src):
        shutil.copyfile(os.path.join(src, f), os.path.join(moe, f))
    for root, _, files in os.walk(here):
        for f in files:
            os.chmod(os.path.join(root, f), 0o644)


if __name__ == "__main__":
    main(sys.argv[1])
