"""Rank program of the multi-GPU wire test: launched by torchrun, one process
per GPU.  Checks, per step, that the MXFP4 wire over NVLink peer stores gives
the bits of the CPU oracle on every rank, and that ranks agree (the reference's
tests/test_wire.py:43-67 does the same over gloo for its own wires)."""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from lockstep_b200 import wire          # noqa: E402
from oracle import cref                 # noqa: E402


def student_t(n, seed):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, generator=g)
    chi = (torch.randn(3, n, generator=g) ** 2).sum(0) / 3
    return (z / chi.sqrt() * 1e-3).float()


def main():
    rank, world, dev = wire.init()
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 1_000_003
    # the last entry of a tuple: groups handed out from a counter (True), fixed shares (False), the default (None)
    for method, mode, subs, stagger, dynamic in (("mxfp4", "launches", 0, False, None), ("mxfp4ef", "launches", 0, False, True),
                                                 ("mxfp4ef", "fused", 0, False, None), ("mxfp4ef", "fused", 8, True, False),
                                                 ("mxfp4", "fused", 2, False, None), ("mxfp4ef", "fused", 2, True, True)):
        w = wire.Wire(method, n, world, rank)
        w.set_mode(mode, subs, stagger, device=dev)
        if dynamic is not None:
            w.set_dynamic(dynamic, device=dev)
        ef = method == "mxfp4ef"
        res_c = [np.zeros(w._kpadded, np.float32) for _ in range(world)] if ef else None
        ores_c = [np.zeros(w._kpadded // world, np.float32) for _ in range(world)] if ef else None
        for step in range(3):
            grads = [student_t(n, 1000 * step + r).numpy() for r in range(world)]
            want, _, _ = cref.wire_step(grads, res_c, ores_c, unit=256)
            g = torch.from_numpy(grads[rank].copy()).to(dev)
            out = w(g)
            w.status()
            assert np.array_equal(out.cpu().numpy(), want), f"{method} {mode} step {step} rank {rank}: bits differ from the oracle"
            everyone = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(everyone, out)
            assert all(torch.equal(out, o) for o in everyone), f"{method}: ranks disagree"
            if ef:
                assert np.array_equal(w.res.cpu().numpy(), res_c[rank])
                assert np.array_equal(w.ores.cpu().numpy().reshape(-1), ores_c[rank])
        ref = torch.from_numpy(np.mean(np.stack(grads).astype(np.float64), 0))
        rel = ((out.cpu().double() - ref).norm() / ref.norm()).item()
        if not ef:                       # one-shot gate; with error feedback a step also carries old residuals
            assert rel <= 0.25, rel
        w.close()
    # the reference's own wires on the same transport API
    torch.manual_seed(rank)
    g = (torch.randn(5000) * (1 + rank)).to(dev)
    ref = g.double()
    dist.all_reduce(ref)
    ref /= world
    for method, tol in (("fp32", 1e-6), ("int16", 1e-3), ("int8", 5e-2)):
        w = wire.Wire(method, g.numel(), world, rank)
        out = w(g.clone())
        assert ((out.double() - ref).norm() / ref.norm()).item() < tol, method
        if w.dtype is not None:
            assert torch.equal(out, w(g.clone(), reverse=True)), f"{method}: order changed bits"
    if rank == 0:
        print(f"wire ranks ok: world {world}, n {n}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
