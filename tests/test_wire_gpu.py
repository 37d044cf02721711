"""GPU parity of the gradient wires.

MXFP4 wires: the three kernels (send / reduce / finish) against the CPU oracle
of the same protocol, bit for bit: outputs, residuals and the bytes that cross
the wire.  Several ranks are emulated on one GPU by running each phase rank
after rank (no kernel waits for another).  Integer wires: the reference's own
test thresholds (tests/test_wire.py:26-40) and golden outputs."""

import numpy as np
import pytest
import torch

from oracle import cref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wire():
    from lockstep_b200 import wire as m
    return m


def _student_t(n, seed):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, generator=g)
    chi = (torch.randn(3, n, generator=g) ** 2).sum(0) / 3
    return (z / chi.sqrt() * 1e-3).float()


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("ef", [False, True])
def test_mxfp4_wire_golden_outputs(wire, golden, world, ef):
    gd = golden(f"wire_mxfp4{'ef' if ef else ''}_w{world}")
    grads = gd["grads"]                                      # [step, rank, n]
    n = grads.shape[-1]
    grp = wire.LocalWireGroup(world, n, ef)
    for step in range(3):
        gs = [torch.from_numpy(grads[step, r].copy()).cuda() for r in range(world)]
        grp.step(gs)
        for r in range(world):
            assert np.array_equal(gs[r].cpu().numpy(), gd[f"out{step}"]), (step, r)
    grp.close()


@pytest.mark.parametrize("world,n", [(1, 1000), (2, 4096 + 13), (3, 70_001), (8, 100_003), (4, 1 << 20)])
def test_mxfp4_wire_bytes_and_residuals_vs_oracle(wire, world, n):
    grp = wire.LocalWireGroup(world, n, ef=True)
    padded, shard = grp.kpadded, grp.kpadded // world
    res_c = [np.zeros(padded, np.float32) for _ in range(world)]
    ores_c = [np.zeros(shard, np.float32) for _ in range(world)]
    for step in range(3):
        grads = [_student_t(n, 100 * step + r).numpy() for r in range(world)]
        want, sent, owned = cref.wire_step(grads, res_c, ores_c, unit=256)
        gs = [torch.from_numpy(g.copy()).cuda() for g in grads]
        grp.step(gs)
        for r in range(world):
            assert np.array_equal(gs[r].cpu().numpy(), want), (step, r)
            assert np.array_equal(grp.res[r].cpu().numpy(), res_c[r])
            assert np.array_equal(grp.ores[r].cpu().numpy(), ores_c[r])
            rs = grp.slots(r, 0).cpu().numpy()               # what rank r received as owner
            ag = grp.slots(r, 1).cpu().numpy()               # what rank r gathered
            for s in range(world):
                assert np.array_equal(rs[s, :shard // 2], sent[s][0][r * shard // 2:(r + 1) * shard // 2])
                assert np.array_equal(rs[s, shard // 2:shard // 2 + shard // 32],
                                      sent[s][1][r * shard // 32:(r + 1) * shard // 32])
                assert np.array_equal(ag[s, :shard // 2], owned[s][0])
                assert np.array_equal(ag[s, shard // 2:shard // 2 + shard // 32], owned[s][1])
    grp.close()


def test_mxfp4_wire_reverse_and_error(wire):
    world, n = 4, 50_000
    grads = [_student_t(n, 7 + r) for r in range(world)]
    ref = torch.stack(grads).double().mean(0)
    grp = wire.LocalWireGroup(world, n)
    gs = [g.clone().cuda() for g in grads]
    grp.step(gs, reverse=True)
    want, _, _ = cref.wire_step([g.numpy() for g in grads], reverse=True, unit=256)
    assert np.array_equal(gs[0].cpu().numpy(), want)
    rel = ((gs[0].cpu().double() - ref).norm() / ref.norm()).item()
    assert rel <= 0.25, rel                                   # one-shot error gate of the FP4 wire
    grp.close()


def test_wire_object_one_rank(wire):
    n = 10_000
    g = torch.randn(n, generator=torch.Generator().manual_seed(0))
    for method in ("mxfp4", "mxfp4ef"):
        w = wire.Wire(method, n)
        assert w.bytes_per_el == 0.53125 and w.padded == -(-n // 64) * 64
        x = g.clone().cuda()
        out = w(x)
        assert out.data_ptr() == x.data_ptr()                # in place, returns g
        want, _, _ = cref.wire_step([g.numpy()], [np.zeros(w._kpadded, np.float32)] if w.ef else None,
                                    [np.zeros(w._kpadded, np.float32)] if w.ef else None, unit=256)
        assert np.array_equal(out.cpu().numpy(), want)
        w.status()
        w.close()


@pytest.mark.parametrize("pieces", [4, 8, 3])
def test_pipelined_pieces_do_not_change_anything(wire, pieces):
    # the all-reduce cut into pieces over three streams: same g, residuals and wire bytes
    # as the single-piece call, step after step (one rank: the waits are met by this GPU's
    # own earlier kernels, so nothing waits for a later launch)
    from lockstep_b200 import _lib
    L = _lib.lib()
    n = (1 << 20) + 4096                   # shard = 262144 * 4 + 4096: divisible by 8 * 32 * 4 and * 8, not by 3
    gen = torch.Generator().manual_seed(5)
    steps = [torch.randn(n, generator=gen) * 1e-3 for _ in range(3)]
    outs = []
    for c in (1, pieces):
        w = wire.Wire("mxfp4ef", n)
        h = w._handle(torch.device("cuda", 0))
        assert L.ls_wire_set_chunks(h, c) == 0
        per = []
        for g in steps:
            x = g.clone().cuda()
            w(x)
            per.append((x.cpu(), w.res.cpu().clone(), w.ores.cpu().clone()))
        w.status()
        w.close()
        outs.append(per)
    for a, b in zip(*outs):
        assert all(torch.equal(x, y) for x, y in zip(a, b))
    w = wire.Wire("mxfp4ef", n)
    h = w._handle(torch.device("cuda", 0))
    assert L.ls_wire_set_chunks(h, 9) < 0 and L.ls_wire_set_chunks(h, -1) < 0
    w.close()


@pytest.mark.parametrize("method,tol", [("bf16", 1e-2), ("int16", 2e-4), ("int8", 3e-2), ("mxfp4", 0.2)])
def test_one_rank_error(wire, method, tol):
    # reference tests/test_wire.py:26-30
    g = torch.randn(10_000, device="cuda")
    out = wire.Wire(method, g.numel())(g.clone())
    assert ((out - g).norm() / g.norm()) < tol


def test_error_feedback_delivers_small_gradients(wire):
    # reference tests/test_wire.py:33-40, and the same property for the FP4 wire
    g = torch.full((64,), 1e-3, device="cuda")
    g[0] = 1.0
    plain, ef = wire.Wire("int8", 64), wire.Wire("int8ef", 64)
    sent_plain = sum(plain(g.clone()) for _ in range(100))
    sent_ef = sum(ef(g.clone()) for _ in range(100))
    assert (sent_plain[1:] == 0).all()
    assert torch.allclose(sent_ef[1:], 100 * g[1:], atol=2 / 127)
    g = torch.full((32,), 1e-3, device="cuda")
    g[0] = 1.0                                               # block scale 0.25: 1e-3 rounds to zero
    plain, ef = wire.Wire("mxfp4", 32), wire.Wire("mxfp4ef", 32)
    sent_plain = sum(plain(g.clone()) for _ in range(400))
    sent_ef = sum(ef(g.clone()) for _ in range(400))
    assert (sent_plain[1:] == 0).all()
    assert torch.allclose(sent_ef[1:], 400 * g[1:], atol=0.26)


@pytest.mark.parametrize("method", ["int16", "int8", "int8ef"])
def test_integer_wire_golden(wire, golden, method):
    # outputs of the real reference Wire over three steps: bit for bit
    gd = golden(f"wire_{method}_w1")
    g = torch.from_numpy(gd["g"]).cuda()
    w = wire.Wire(method, g.numel())
    for s in range(3):
        out = w(g.clone() * (1 + 0.5 * s))
        assert np.array_equal(out.cpu().numpy(), gd["outs"][s]), (method, s)
    w.status()
    w.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("bits,ef", [(16, False), (8, False), (8, True)])
def test_integer_wire_ranks_vs_oracle(wire, world, bits, ef):
    from oracle import ref_port
    n = 5000 + 333 * world
    lim = 2 ** (bits - 1) - 1
    grp = wire.LocalWireGroup(world, n, ef, bits=bits)
    padded = ref_port.padded_len(n, world)
    res = [torch.zeros(padded) for _ in range(world)] if ef else None
    ores = [torch.zeros(padded // 64 // world, 64) for _ in range(world)] if ef else None
    for step in range(3):
        grads = [torch.randn(n, generator=torch.Generator().manual_seed(17 * step + r)) * (1 + r) for r in range(world)]
        want = ref_port.wire_int_step(grads, lim, res, ores)[0]
        gs = [g.clone().cuda() for g in grads]
        grp.step(gs)
        for r in range(world):
            assert torch.equal(gs[r].cpu(), want), (step, r)
    grp.close()


def test_ranks_come_from_torchrun_then_slurm(wire, monkeypatch):
    # reference tests/test_wire.py:14-23
    names = ("RANK", "WORLD_SIZE", "LOCAL_RANK", "SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID",
             "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK")
    for k in names:
        monkeypatch.delenv(k, raising=False)
    assert wire.env_rank() == (0, 1, 0)
    for k, v in (("SLURM_PROCID", "5"), ("SLURM_NTASKS", "16"), ("SLURM_LOCALID", "1")):
        monkeypatch.setenv(k, v)
    assert wire.env_rank() == (5, 16, 1)
    for k, v in (("RANK", "3"), ("WORLD_SIZE", "8"), ("LOCAL_RANK", "3")):
        monkeypatch.setenv(k, v)
    assert wire.env_rank() == (3, 8, 3)


def test_missing_peer_is_reported_not_hung(wire):
    """Failure detection: rank 1 never sends.  Rank 0's owner kernel polls rank 1's
    flag a bounded number of times, records a time-out and returns; the host reads
    the status as an error, and the same handles work again afterwards."""
    import ctypes
    from lockstep_b200._lib import check, lib, ptr, stream
    L = lib()
    world, n = 2, 4096
    grp = wire.LocalWireGroup(world, n)
    for h in grp.handles:
        check(L.ls_wire_set_poll_limit(h, 2000))             # ~ a few ms
    g0 = torch.randn(n, device="cuda")
    check(L.ls_wire_send(grp.handles[0], ptr(g0), n, None, stream()))   # rank 1's send is "lost"
    check(L.ls_wire_reduce(grp.handles[0], None, 0, stream()))
    status = ctypes.c_int(0)
    rc = L.ls_wire_status(grp.handles[0], ctypes.byref(status))
    assert rc == -4 and status.value != 0                    # LS_ETIMEOUT
    assert b"gave up" in L.ls_last_error()
    assert L.ls_wire_status(grp.handles[0], None) == 0       # cleared; context still usable
    # bring rank 1 level with rank 0's epoch, then a complete step works
    g1 = torch.randn(n, device="cuda")
    check(L.ls_wire_send(grp.handles[1], ptr(g1), n, None, stream()))
    check(L.ls_wire_reduce(grp.handles[1], None, 0, stream()))
    gs = [torch.randn(n, device="cuda") for _ in range(world)]
    want, _, _ = cref.wire_step([g.cpu().numpy() for g in gs], unit=256)
    grp.step(gs)
    assert np.array_equal(gs[0].cpu().numpy(), want) and np.array_equal(gs[1].cpu().numpy(), want)
    grp.close()
