"""The operators around the GEMV chain, through the C ABI, against the CPU checker: residual add + RMSNorm (add_rms_1k),
the lm_head's argmax with the reference kernel's tie rule, the vocabulary GEMV + argmax, and loading NVFP4 tensors from a
CNQ container onto the device (whole and as a tensor-parallel row shard)."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from conftest import GOLDEN
from crownest_b200 import cnq, ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16


@pytest.mark.parametrize("rows,hidden", [(1, 5120), (4, 2560), (3, 1000)])
def test_add_rmsnorm_matches_the_cpu_reference(rows, hidden):
    rng = np.random.default_rng(hidden)
    h = rng.standard_normal((rows, hidden)).astype(np.float32)
    y = rng.standard_normal((rows, hidden)).astype(np.float32)
    w = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    for yy in (y, None):
        hd = torch.from_numpy(h.copy()).cuda()
        out = ops.add_norm(hd, None if yy is None else torch.from_numpy(yy).cuda(), torch.from_numpy(w).cuda())
        rh, ro = oracle.add_rmsnorm(h, yy, w)
        assert np.array_equal(hd.cpu().numpy().view(np.uint32), rh.view(np.uint32))  # the residual stream: bit-exact
        assert np.max(np.abs(out.cpu().numpy() - ro) / (np.abs(ro) + 1e-6)) <= 4e-7  # rsqrt approximation: 2 ulp


def test_argmax_breaks_ties_like_the_reference_kernel():
    rng = np.random.default_rng(0)
    n = 248320
    x = rng.standard_normal((4, n)).astype(np.float32)
    x[1, [7, 1029, 200000]] = 9.0      # ties across scanners: the tree keeps the lower scanner's, not the lowest index
    x[2, [5000, 5000 + 1024]] = 9.0    # ties inside one scanner: the first
    x[3, :] = np.nan
    x[3, 77] = -5.0
    got = ops.argmax(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, oracle.argmax(x))
    assert got[0] == int(np.argmax(x[0])) and got[2] == 5000 and got[3] == 77
    gb = ops.argmax(torch.from_numpy(x).cuda().to(torch.bfloat16)).cpu().numpy()
    xb = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(gb, oracle.argmax(xb))


def test_lm_head_and_argmax():
    vocab, k, m = 20000, 2048, 3
    rng = np.random.default_rng(2)
    w = synth.nvfp4_matrix(vocab, k, rng)
    xb, xf = synth.activations(m, k, rng)
    fw = ops.Fp4.from_host(w, vocab, k, 0.01)
    tok, logits = ops.lm_head_argmax(fw, to_dev_bf16(xb))
    ref = oracle.nvfp4_gemv(w, vocab, k, np.float32(0.01), xf, threads=8, path=1)
    check_close(from_dev_bf16(logits), ref, "lm_head")
    assert np.array_equal(tok.cpu().numpy(), oracle.argmax(from_dev_bf16(logits)))


def test_container_tensors_load_onto_the_device():
    c = cnq.Cnq(os.path.join(GOLDEN, "synthetic-v2.cnq"))
    g = np.load(os.path.join(GOLDEN, "nvfp4_dequant.npz"))
    for i in range(int(g["cnq_count"])):
        name = str(g[f"cnq{i}_name"])
        w = c.load_fp4(name)
        got = ops.dequant(w).cpu().numpy()
        assert np.array_equal(got.reshape(-1).view(np.uint32), g[f"cnq{i}_deq"].reshape(-1).view(np.uint32))
        half = c.load_fp4(name, rank=1, world=2)
        assert np.array_equal(ops.dequant(half).cpu().numpy(), got[got.shape[0] // 2:])
    emb = c.load_dense("model.language_model.embed_tokens.weight")
    assert emb.shape == (128, 64) and emb.dtype == torch.bfloat16
    c.close()
