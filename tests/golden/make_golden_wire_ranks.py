"""Generates tests/golden/wire_int*_w{2,4}.npz by running the REAL reference
wire.Wire on several gloo ranks (CPU), three steps per method.

    python tests/golden/make_golden_wire_ranks.py /path/to/lockstep

Each archive holds the per-rank gradients `grads` [step, rank, n] and the
averaged output of every step `outs` [step, n] (identical on every rank: the
script checks that before writing).  The test-suite reads the archives only.
"""

import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

OUT = Path(__file__).resolve().parent
N = 5000


def _grads(world):
    g = torch.Generator().manual_seed(4242 + world)
    return [[torch.randn(N + 37 * world, generator=g) * (1 + r) * (1 + 0.5 * s) for r in range(world)] for s in range(3)]


def _rank(rank, world, port, ref):
    sys.path.insert(0, ref)
    import wire                                    # the reference's
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    grads = _grads(world)
    for method in ("int16", "int8", "int8ef"):
        w = wire.Wire(method, grads[0][0].numel(), world, rank)
        outs = []
        for s in range(3):
            out = w(grads[s][rank].clone())
            everyone = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(everyone, out)
            assert all(torch.equal(out, o) for o in everyone), f"{method}: ranks disagree"
            outs.append(out.numpy().copy())
        if rank == 0:
            np.savez_compressed(OUT / f"wire_{method}_w{world}.npz",
                                grads=np.stack([np.stack([t.numpy() for t in st]) for st in grads]),
                                outs=np.stack(outs))
    dist.destroy_process_group()


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_wire_ranks.py /path/to/lockstep")
    for world in (2, 4):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        mp.spawn(_rank, args=(world, port, sys.argv[1]), nprocs=world)
    print("multi-rank integer wire goldens written to", OUT)
