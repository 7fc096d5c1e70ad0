"""Runs the reference's own CUDA operators (built by ``oracle/build_ref_gpu.py``) in a process of their own.

TEST / BASELINE INFRASTRUCTURE ONLY.  The reference library registers the same ``torch.ops.approxtorch``
schemas as this repository's binding, so it cannot share a process with ``approxtorch_b200``; callers start
this file with ``python oracle/ref_gpu_worker.py <request.npz> <reply.npz>``.

Request keys: ``op`` (operator name) plus its tensor arguments ``arg0..argN`` (numpy arrays; int scalars as
0-d arrays).  ``time:<operator>`` times that operator instead of returning its outputs.  Special op ``bench_bgemm16``: times the raw LUT-BGEMM workload the reference way — 16 per-item
``gemm_fake_int8_forward_cuda_claude`` calls, 5 warm-up + 30 timed iterations between CUDA events
(approxtorch/backend/csrc/claude/bench.py:140-152).
"""

from __future__ import annotations

import glob
import os
import sys

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))


def main(req_path: str, reply_path: str) -> int:
    libs = sorted(glob.glob(os.path.join(_HERE, "_ref", "gpu", "ref_gpu_ops*.so")))
    if not libs:
        np.savez(reply_path, error=np.array("reference CUDA operators were not built (oracle/_ref/gpu is empty)"))
        return 0
    torch.ops.load_library(libs[0])
    dev = torch.device("cuda:0")
    req = np.load(req_path, allow_pickle=False)
    op = str(req["op"])
    args = []
    i = 0
    while f"arg{i}" in req:
        a = req[f"arg{i}"]
        args.append(int(a) if a.ndim == 0 and a.dtype.kind in "iu" else torch.from_numpy(a).to(dev))
        i += 1
    if op == "bench_bgemm16":
        a_idx, b_idx, lut = args          # [16,M,K] u8, [16,K,N] u8, [65536] f32
        fn = torch.ops.approxtorch.gemm_fake_int8_forward_cuda_claude
        def step():
            for b in range(a_idx.shape[0]):
                fn(a_idx[b], b_idx[b], lut)
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 30
        np.savez(reply_path, ms_per_step=np.array(ms))
        return 0
    if op.startswith("time:"):
        # any operator timed the reference's way: 5 warm-up + 30 iterations between CUDA events
        fn = getattr(torch.ops.approxtorch, op[5:])
        for _ in range(5):
            fn(*args)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            fn(*args)
        e1.record()
        torch.cuda.synchronize()
        np.savez(reply_path, ms_per_call=np.array(e0.elapsed_time(e1) / 30))
        return 0
    out = getattr(torch.ops.approxtorch, op)(*args)
    if isinstance(out, torch.Tensor):
        out = (out,)
    torch.cuda.synchronize()
    np.savez(reply_path, **{f"out{j}": t.detach().cpu().numpy() for j, t in enumerate(out)})
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2]))
