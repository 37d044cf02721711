"""CPU, world size 2 and 4 over gloo: the MXFP4 wire protocol run across real
process-group collectives (all_to_all for the reduce-scatter half, all_gather
for the gather half, as wire.py:53-74 moves its payloads) gives the same bits
as the one-process simulation the GPU tests are checked against, on every rank.
Also the host-side geometry (padding, shard bounds) used by the CUDA path."""

import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_port


def _grad(n, seed):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, generator=g)
    chi = (torch.randn(3, n, generator=g) ** 2).sum(0) / 3
    return (z / chi.sqrt() * 1e-3).float()


def _rank_main(rank, world, port, n):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    padded = ref_port.padded_len(n, world)
    shard = padded // world
    res, ores = torch.zeros(padded), torch.zeros(shard)
    sim_res = [torch.zeros(padded) for _ in range(world)]
    sim_ores = [torch.zeros(shard) for _ in range(world)]
    for step in range(3):
        grads = [_grad(n, 10 * step + r) for r in range(world)]
        want = ref_port.wire_mxfp4_step(grads, sim_res, sim_ores)[rank]
        # sender
        packed, e8 = ref_port.wire_mxfp4_encode(grads[rank], n, padded, res)
        recv_p, recv_e = torch.empty_like(packed), torch.empty_like(e8)
        dist.all_to_all_single(recv_p, packed)               # shard o of every sender lands on owner o
        dist.all_to_all_single(recv_e, e8)
        slots = [(recv_p[s * shard // 2:(s + 1) * shard // 2], recv_e[s * shard // 32:(s + 1) * shard // 32])
                 for s in range(world)]
        # owner
        op, oe = ref_port.wire_mxfp4_owner(slots, ores)
        all_p = [torch.empty_like(op) for _ in range(world)]
        all_e = [torch.empty_like(oe) for _ in range(world)]
        dist.all_gather(all_p, op)
        dist.all_gather(all_e, oe)
        out = ref_port.wire_mxfp4_decode(torch.cat(all_p), torch.cat(all_e))[:n] / world
        assert torch.equal(out, want), f"step {step} rank {rank}"
        assert torch.equal(res, sim_res[rank]) and torch.equal(ores, sim_ores[rank])
        everyone = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(everyone, out)
        assert all(torch.equal(out, o) for o in everyone), "ranks disagree"
        ref = torch.stack(grads).double().mean(0)
        assert ((out.double() - ref).norm() / ref.norm()).item() < 0.35
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_mxfp4_wire_over_gloo(world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(world, port, 5000 + 17 * world), nprocs=world)


def test_wire_geometry_without_gpu():
    from lockstep_b200 import wire
    for n, world in ((5000, 4), (64, 1), (1, 8), (124_000_000, 8)):
        w = wire.Wire("mxfp4ef", n, world, 0)
        assert w.padded == ref_port.padded_len(n, world) and w.padded % (world * 64) == 0
        assert w._kpadded % (world * 256) == 0 and 0 <= w._kpadded - n < world * 256
        assert w.bytes_per_el == 0.53125 and w.ef and w.res is None
    assert wire.Wire("int8ef", 10).lim == 127 and wire.Wire("int16", 10).dtype == torch.int16
    assert wire.METHODS[:4] == ("fp32", "bf16", "int16", "int8ef")
    with pytest.raises(RuntimeError, match="CUDA"):
        wire.Wire("mxfp4", 64)(torch.zeros(64))
