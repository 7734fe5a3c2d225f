"""One GEMV shape launched a few times, for a profiler to capture: ``python -m crownest_b200.profile_case
--rows 34816 --k 5120 --m 1``. The launches rotate over several weight copies so that every launch
streams its bytes from HBM, not from L2. ``--op gu`` runs the fused gate/up form on rows / 2 indices, ``--op gemm`` the tcgen05 GEMM on ``--m`` rows."""
import argparse

import torch

from . import _lib, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=34816)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--op", default="gemv", choices=["gemv", "gu", "gemm"])
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--copies", type=int, default=3)
    args = ap.parse_args()
    _lib.lib()
    rows = args.rows // 2 if args.op == "gu" else args.rows
    nbytes = rows * args.k // 64 * 36
    gen = torch.Generator(device="cuda").manual_seed(0)
    ws = []
    for _ in range(args.copies * (2 if args.op == "gu" else 1)):
        w = torch.randint(0, 256, (nbytes // 36, 36), dtype=torch.uint8, device="cuda", generator=gen)
        w[:, :4] = torch.randint(0x20, 0x38, (nbytes // 36, 4), dtype=torch.uint8, device="cuda", generator=gen)
        ws.append(ops.Fp4(w.reshape(-1), torch.ones(1, device="cuda"), rows, args.k))
    x = torch.randn(args.m, args.k, device="cuda", generator=gen).to(torch.bfloat16)
    y = torch.empty(args.m, rows, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    scratch = torch.empty(ops.gemm_workspace_bytes(args.k, args.m), dtype=torch.uint8, device="cuda") if args.op == "gemm" else None
    for i in range(args.launches):
        if args.op == "gemm":
            ops.launch_gemm(ws[i % args.copies], x, y, workspace=scratch)
        elif args.op == "gu":
            ops.launch_gemv_gu(ws[2 * (i % args.copies)], ws[2 * (i % args.copies) + 1], x, y)
        else:
            ops.launch_gemv(ws[i % args.copies], x, y)
    torch.cuda.synchronize()
    print("device status", _lib.device_status())


if __name__ == "__main__":
    main()
