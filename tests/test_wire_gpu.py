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


@pytest.mark.parametrize("world,n,subs,stagger,dynamic", [(1, 70_001, 0, False, None), (2, 300_000, 4, False, None), (3, 70_001, 2, True, None),
                                                          (4, 1 << 20, 8, True, None), (8, 100_003, 0, False, None), (8, 3_000_000, 4, True, None),
                                                          (1, 1 << 20, 2, False, True), (2, 300_000, 3, True, True), (4, 3_000_000, 0, False, True),
                                                          (8, 3_000_000, 2, True, False)])
def test_cooperative_launch_bytes_and_residuals_vs_oracle(wire, world, n, subs, stagger, dynamic):
    # The pipelined kernel (send(t), reduce(t-1), finish(t-2) over sub-ranges, one flag per
    # sub-range) with every rank's CTAs inside ONE cooperative launch: the waits between ranks
    # are real.  Same bits as the oracle: g, both residuals and the bytes on the wire.
    # dynamic: the groups of a phase handed out from a counter (the default from eight ranks up) or as fixed shares
    grp = wire.LocalWireGroup(world, n, ef=True)
    if dynamic is not None:
        grp.set_dynamic(dynamic)
    padded, shard = grp.kpadded, grp.kpadded // world
    res_c = [np.zeros(padded, np.float32) for _ in range(world)]
    ores_c = [np.zeros(shard, np.float32) for _ in range(world)]
    for step in range(4 if dynamic else 3):
        grads = [_student_t(n, 100 * step + r).numpy() for r in range(world)]
        want, sent, owned = cref.wire_step(grads, res_c, ores_c, unit=256)
        gs = [torch.from_numpy(g.copy()).cuda() for g in grads]
        grp.step_fused(gs, subs=subs, stagger=stagger)
        for r in range(world):
            assert np.array_equal(gs[r].cpu().numpy(), want), (step, r)
            assert np.array_equal(grp.res[r].cpu().numpy(), res_c[r])
            assert np.array_equal(grp.ores[r].cpu().numpy(), ores_c[r])
            rs = grp.slots(r, 0).cpu().numpy()
            ag = grp.slots(r, 1).cpu().numpy()
            for s in range(world):
                assert np.array_equal(rs[s, :shard // 2], sent[s][0][r * shard // 2:(r + 1) * shard // 2])
                assert np.array_equal(rs[s, shard // 2:shard // 2 + shard // 32],
                                      sent[s][1][r * shard // 32:(r + 1) * shard // 32])
                assert np.array_equal(ag[s, :shard // 2], owned[s][0])
                assert np.array_equal(ag[s, shard // 2:shard // 2 + shard // 32], owned[s][1])
    grp.close()


def test_cooperative_launch_reverse_and_no_error_feedback(wire):
    world, n = 4, 50_000
    grads = [_student_t(n, 7 + r) for r in range(world)]
    grp = wire.LocalWireGroup(world, n)
    gs = [g.clone().cuda() for g in grads]
    grp.step_fused(gs, reverse=True, subs=2)
    want, _, _ = cref.wire_step([g.numpy() for g in grads], reverse=True, unit=256)
    for r in range(world):
        assert np.array_equal(gs[r].cpu().numpy(), want)
    grp.close()


@pytest.mark.parametrize("mode,subs", [("launches", 0), ("fused", 1), ("fused", 4), ("fused", 8), ("fused", 3)])
def test_wire_modes_give_the_same_bits(wire, mode, subs):
    # one rank, error feedback, three steps: g and both residuals against the oracle in every mode
    n = (1 << 20) + 4096
    gen = torch.Generator().manual_seed(5)
    w = wire.Wire("mxfp4ef", n)
    w.set_mode(mode, subs, stagger=subs == 4)
    if subs in (0, 3):
        w.set_dynamic(True)                                    # groups handed out from a counter, in both ways to run a step
    assert w.mode_name() == ("three launches" if mode == "launches" else "one cooperative launch")
    res_c, ores_c = [np.zeros(w._kpadded, np.float32)], [np.zeros(w._kpadded, np.float32)]
    for _ in range(3):
        g = torch.randn(n, generator=gen) * 1e-3
        want, _, _ = cref.wire_step([g.numpy()], res_c, ores_c, unit=256)
        x = g.clone().cuda()
        w(x)
        assert np.array_equal(x.cpu().numpy(), want)
        assert np.array_equal(w.res.cpu().numpy(), res_c[0])
        assert np.array_equal(w.ores.cpu().numpy().reshape(-1), ores_c[0])
    w.status()
    sd = w.state_dict()
    assert sd["res"].shape == (w.padded,) and sd["ores"].shape == (w._kpadded // 64, 64)
    w2 = wire.Wire("mxfp4ef", n)
    w2.load_state_dict({k: v.clone() for k, v in sd.items()})
    g = torch.randn(n, generator=gen) * 1e-3
    a, b = w(g.clone().cuda()), w2(g.clone().cuda())
    assert torch.equal(a, b) and torch.equal(w.res, w2.res) and torch.equal(w.ores, w2.ores)
    from lockstep_b200 import _lib
    assert _lib.lib().ls_wire_set_mode(w._h, 3, 0, 0) < 0 and _lib.lib().ls_wire_set_mode(w._h, 2, 9, 0) < 0
    w.close()
    w2.close()


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


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("method", ["int16", "int8", "int8ef"])
def test_integer_wire_golden_several_ranks(wire, golden, method, world):
    # outputs of the real reference Wire on 2 and 4 gloo ranks, three steps: bit for bit
    gd = golden(f"wire_{method}_w{world}")
    grads = gd["grads"]
    grp = wire.LocalWireGroup(world, grads.shape[-1], ef=method == "int8ef", bits=16 if method == "int16" else 8)
    for s in range(3):
        gs = [torch.from_numpy(grads[s, r].copy()).cuda() for r in range(world)]
        grp.step(gs)
        for r in range(world):
            assert np.array_equal(gs[r].cpu().numpy(), gd["outs"][s]), (method, world, s, r)
    grp.close()


def test_missing_peer_fails_the_step_everywhere_and_absorbs_nothing(wire):
    """Failure detection: rank 1 never takes part in the step.  Rank 0's owner kernel waits
    for rank 1's flag up to the time limit, records the time-out and returns WITHOUT
    storing: the owner residual and the gather slots (its own and the peer's) keep what
    they held, no gather flag is raised, so the decode kernel runs out as well and g is
    left alone.  The host reads the
    status as an error (also without synchronising, through the pinned copy); after a
    reset on every rank the same handles give the oracle's bits again."""
    import ctypes
    from lockstep_b200._lib import check, lib, ptr, stream
    L = lib()
    world, n = 2, 4096
    grp = wire.LocalWireGroup(world, n, ef=True)
    for h in grp.handles:
        check(L.ls_wire_set_timeout_us(h, 3000))
    g0 = torch.randn(n, device="cuda")
    keep0 = g0.clone()
    ag_before = grp.slots(0, 1).clone()
    check(L.ls_wire_send(grp.handles[0], ptr(g0), n, ptr(grp.res[0]), stream()))   # rank 1 never takes part
    check(L.ls_wire_reduce(grp.handles[0], ptr(grp.ores[0]), 0, stream()))
    check(L.ls_wire_finish(grp.handles[0], ptr(g0), n, stream()))
    torch.cuda.synchronize()
    assert L.ls_wire_poll_status(grp.handles[0], None) == -4         # seen without a synchronising call
    status = ctypes.c_int(0)
    rc = L.ls_wire_status(grp.handles[0], ctypes.byref(status))
    assert rc == -4 and status.value != 0                    # LS_ETIMEOUT
    assert b"gave up" in L.ls_last_error()
    assert L.ls_wire_status(grp.handles[0], None) == 0       # cleared; context still usable
    assert torch.equal(g0, keep0)                                                 # nothing decoded
    assert not grp.ores[0].any()                                                  # owner residual untouched
    assert torch.equal(grp.slots(0, 1), ag_before)                                # nothing gathered
    assert not grp.slots(1, 1).any()                                              # nothing pushed to the peer either
    for r in range(world):
        check(L.ls_wire_reset(grp.handles[r]))
        grp.res[r].zero_(), grp.ores[r].zero_()
        assert L.ls_wire_poll_status(grp.handles[r], None) == 0
    gs = [torch.randn(n, device="cuda") for _ in range(world)]
    res_c = [np.zeros(grp.kpadded, np.float32) for _ in range(world)]
    ores_c = [np.zeros(grp.kpadded // world, np.float32) for _ in range(world)]
    want, _, _ = cref.wire_step([g.cpu().numpy() for g in gs], res_c, ores_c, unit=256)
    grp.step(gs)
    assert np.array_equal(gs[0].cpu().numpy(), want) and np.array_equal(gs[1].cpu().numpy(), want)
    assert np.array_equal(grp.res[0].cpu().numpy(), res_c[0]) and np.array_equal(grp.ores[1].cpu().numpy(), ores_c[1])
    assert L.ls_wire_set_timeout_us(grp.handles[0], 0) < 0
    grp.close()


def test_wire_object_raises_on_the_call_after_a_time_out(wire):
    # Wire.__call__ reads the pinned status copy before it queues more work: a step that
    # timed out turns into an exception on the next call, without an extra synchronisation
    import ctypes
    from lockstep_b200._lib import check, lib
    L = lib()
    n = 4096
    grp = wire.LocalWireGroup(2, n)
    x = torch.randn(n, device="cuda")
    w = wire.Wire("mxfp4", n, world=2, rank=0, timeout=0.002)
    w._h = grp.handles[0]                                     # rank 0 of a two-rank wire whose peer never shows up
    check(L.ls_wire_set_timeout_us(w._h, 2000))
    w.send(x)
    w.reduce()
    w.finish(x)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="LS_ETIMEOUT"):
        w(x)
    w._h = None
    grp.close()


def test_phase_methods_equal_the_call(wire):
    # Wire.send / reduce / finish (what a training loop uses to send under backward) against Wire.__call__
    n = 300_000
    g = torch.randn(n, generator=torch.Generator().manual_seed(9)) * 1e-2
    a, b = wire.Wire("mxfp4ef", n), wire.Wire("mxfp4ef", n)
    for step in range(3):
        x, y = (g * (1 + step)).cuda(), (g * (1 + step)).cuda()
        a(x)
        b.send(y)
        b.reduce()
        b.finish(y)
        assert torch.equal(x, y) and torch.equal(a.res, b.res) and torch.equal(a.ores, b.ores)
    a.status(), b.status()
    a.close(), b.close()


@pytest.mark.parametrize("method", ["mxfp4ef", "int8ef"])
def test_a_wire_step_refuses_cuda_graph_capture(wire, method):
    # a step's epoch advances on the host and travels as a kernel argument: a replayed graph would wait on
    # flags of an old epoch.  The call is refused on a capturing stream, nothing is launched, and the wire
    # works as before afterwards.
    n = 100_000
    w = wire.Wire(method, n)
    g = (torch.randn(n, generator=torch.Generator().manual_seed(3)) * 1e-2).cuda()
    first = w(g.clone()).clone()
    graph = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="CUDA graph"):
        with torch.cuda.graph(graph):
            w(g.clone())
    torch.cuda.synchronize()
    w2 = wire.Wire(method, n)
    assert torch.equal(w2(g.clone()), first)                   # an untouched wire gives the first step's result
    w(g.clone())                                                # and the one that refused still runs
    w.status(), w2.status()
    w.close(), w2.close()
