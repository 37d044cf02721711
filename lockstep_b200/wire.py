"""Gradient all-reduce with the API of lockstep's wire.py, plus the FP4 wires.

  fp32     all_reduce in fp32                                  (wire.py:93-96)
  bf16     all_reduce in bf16                                  (wire.py:97-101)
  int16    integers on a shared per-64 grid, owner-reduced     (wire.py:104-138)
  int8     the same at 8 bits
  int8ef   8 bits with error feedback at sender and owner
  mxfp4    (new) MXFP4 payload: block-32 E2M1 + one UE8M0 byte, each block
           scaled by its own rank, so no MAX pre-collective; owner decodes and
           sums in fp32 in ascending sender order, re-encodes, gathers
  mxfp4ef  mxfp4 with error feedback at sender and owner

The MXFP4 and integer wires run as hand-written kernels that store the packed
bytes straight into the owner's / every rank's memory over NVLink
(`csrc/wire.cu`: one cooperative launch per MXFP4 step by default, or one
launch per phase); the process group only carries the IPC handles at set-up.
fp32 and bf16 are torch.distributed all-reduces, as in the reference.  `Wire(method, numel, world, rank)(g)` averages
the flat fp32 gradient `g` in place, as the reference does.
"""

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib, need_cuda, ptr, stream

CHUNK = 64                                     # elements per integer scale
METHODS = ("fp32", "bf16", "int16", "int8ef", "mxfp4", "mxfp4ef")
_KUNIT = 256                                   # the kernels pad to world * 256 elements


def env_rank():
    """(rank, world, local rank) from torchrun, SLURM or MPI variables; else one process (wire.py:30-36)."""
    def first(names, default):
        for n in names:
            if n in os.environ:
                return int(os.environ[n])
        return default
    return (first(("RANK", "SLURM_PROCID", "OMPI_COMM_WORLD_RANK"), 0),
            first(("WORLD_SIZE", "SLURM_NTASKS", "OMPI_COMM_WORLD_SIZE"), 1),
            first(("LOCAL_RANK", "SLURM_LOCALID", "OMPI_COMM_WORLD_LOCAL_RANK"), 0))


def init():
    """Join the process group if there is more than one rank; (rank, world, device) (wire.py:39-50)."""
    rank, world, local = env_rank()
    if not torch.cuda.is_available():
        raise RuntimeError("lockstep_b200.wire needs a CUDA device (there is no CPU path)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    return rank, world, device


class Wire:
    """Averages a flat fp32 gradient across ranks, in place, with one method.

    timeout: seconds a kernel of the peer-store transport waits for another rank
    before it gives up (then the step fails on every rank: see `status`)."""

    def __init__(self, method, numel, world=1, rank=0, timeout=20.0):
        bits = {"int16": 16, "int8": 8, "int8ef": 8}.get(method)
        self.method, self.world, self.rank, self.n = method, world, rank, numel
        self.fp4 = method in ("mxfp4", "mxfp4ef")
        self.ef = method in ("int8ef", "mxfp4ef")
        self.lim = 2 ** (bits - 1) - 1 if bits else None
        self.dtype = {16: torch.int16, 8: torch.int8}.get(bits)
        span = world * CHUNK
        self.padded = -(-numel // span) * span
        self.res = self.ores = None                # sender and owner residuals (EF)
        if self.fp4:
            self.bytes_per_el = 0.5 + 1 / 32       # 16 packed bytes + 1 exponent byte per 32
        else:
            self.bytes_per_el = {"fp32": 4.0, "bf16": 2.0}.get(method) or bits / 8 + 4 / CHUNK
        self.timeout = timeout
        self._h = None
        self._kpadded = -(-numel // (world * _KUNIT)) * world * _KUNIT

    # ---- peer-store transport (MXFP4 and integer payloads) ---------------------
    def _handle(self, device):
        if self._h is None:
            h = ctypes.c_void_p()
            if self.fp4:
                check(lib().ls_wire_create(self.rank, self.world, self._kpadded, ctypes.byref(h)))
            else:
                bits = 16 if self.dtype == torch.int16 else 8
                check(lib().ls_wire_create_int(self.rank, self.world, self._kpadded, bits, ctypes.byref(h)))
            self._h = h
            check(lib().ls_wire_set_timeout_us(h, max(1, int(self.timeout * 1e6))))
            if self.world > 1:
                nb = int(lib().ls_wire_handle_bytes())
                blob = (ctypes.c_uint8 * nb)()
                check(lib().ls_wire_local_handle(h, blob))
                mine = torch.tensor(list(blob), dtype=torch.uint8, device=device)
                everyone = torch.empty(self.world * nb, dtype=torch.uint8, device=device)
                dist.all_gather_into_tensor(everyone, mine)
                raw = bytes(everyone.cpu().tolist())
                check(lib().ls_wire_map_peers(h, raw))
                dist.barrier()
        return self._h

    def _residuals(self, device):
        """The kernels pad to world * 256 elements (the reference to world * 64): the
        residual buffers have the kernels' length.  `res` is flat [kpadded]; `ores` is
        [kpadded / world / 64, 64], the reference's owner-residual shape (wire.py:128-130)."""
        if self.ef and self.res is None:
            self.res = torch.zeros(self._kpadded, device=device)
            self.ores = torch.zeros(self._kpadded // self.world // CHUNK, CHUNK, device=device)

    def _check_args(self, g):
        need_cuda(g)
        assert g.dtype == torch.float32 and g.is_contiguous() and g.numel() == self.n
        h = self._handle(g.device)
        self._residuals(g.device)
        check(lib().ls_wire_poll_status(h, None))        # a time-out of an earlier call: raise before queueing more
        return h

    def _mxfp4(self, g, reverse):
        h = self._check_args(g)
        check(lib().ls_wire_allreduce(h, ptr(g), self.n, ptr(self.res), ptr(self.ores), int(bool(reverse)),
                                      stream()))
        return g

    # The three phases of an MXFP4 step as separate launches: send may be queued as soon as
    # the gradient is final (for instance under the rest of a backward pass, on a side
    # stream); reduce and finish follow in this order on every rank.
    def send(self, g):
        assert self.fp4
        h = self._check_args(g)
        check(lib().ls_wire_send(h, ptr(g), self.n, ptr(self.res), stream()))

    def reduce(self, reverse=False):
        assert self.fp4 and self._h is not None
        check(lib().ls_wire_reduce(self._h, ptr(self.ores), int(bool(reverse)), stream()))

    def finish(self, g):
        assert self.fp4 and self._h is not None
        check(lib().ls_wire_finish(self._h, ptr(g), self.n, stream()))
        return g

    def set_mode(self, mode="auto", subs=0, stagger=False, device=None):
        """How an MXFP4 step runs: "launches" (three kernels), "fused" (one cooperative
        launch that pipelines `subs` sub-ranges of every shard), or "auto"."""
        h = self._handle(device or torch.device("cuda", torch.cuda.current_device()))
        check(lib().ls_wire_set_mode(h, {"auto": 0, "launches": 1, "fused": 2}[mode], subs, int(bool(stagger))))

    def set_dynamic(self, on, device=None):
        """How a phase's groups are spread over the warps: handed out in chunks from a counter
        (True; the default from eight ranks up) or as fixed shares (False).  Results do not depend on it."""
        h = self._handle(device or torch.device("cuda", torch.cuda.current_device()))
        check(lib().ls_wire_set_dynamic(h, int(bool(on))))

    def mode_name(self):
        if self._h is None or not self.fp4:
            return "launches"
        return {1: "three launches", 2: "one cooperative launch"}[int(lib().ls_wire_mode(self._h))]

    def status(self):
        """Raises if a wire kernel gave up waiting for a peer (synchronises)."""
        if self._h is not None:
            check(lib().ls_wire_status(self._h, None))

    def reset(self):
        """After a time-out: clears flags and residuals and realigns the ranks.
        Collective when world > 1."""
        if self._h is None:
            return
        if self.world > 1 and dist.is_initialized():
            torch.cuda.synchronize()
            dist.barrier()
        check(lib().ls_wire_reset(self._h))
        if self.res is not None:
            self.res.zero_()
            self.ores.zero_()
        if self.world > 1 and dist.is_initialized():
            torch.cuda.synchronize()
            dist.barrier()

    def close(self):
        """Frees the receive arena.  Collective when world > 1: every rank must call
        it (it waits for all ranks first, because peers store into this memory)."""
        if self._h is not None:
            if self.world > 1 and dist.is_initialized():
                torch.cuda.synchronize()
                dist.barrier()
            lib().ls_wire_destroy(self._h)
            self._h = None

    def __del__(self):
        # With peers, memory they may still store into cannot be freed behind their back, and
        # a destructor cannot run a collective: an unclosed multi-rank wire keeps its arena
        # until the process ends.  Call close() on every rank to release it.
        try:
            if self.world == 1:
                self.close()
        except Exception:
            pass

    def state_dict(self):
        """Residuals carried across steps (what a checkpoint must hold).  `res` is cut to
        the reference's [padded] (the tail beyond it is padding and stays zero); `ores` is
        [own, 64].  The shapes equal the reference's whenever numel is a multiple of
        world * 256; otherwise this wire's shards are longer than the reference's
        (padded / world) and an owner residual cannot be exchanged with it."""
        if self.res is None:
            return {"res": None, "ores": None}
        return {"res": self.res[:self.padded], "ores": self.ores}

    def load_state_dict(self, sd):
        if sd["res"] is None:
            self.res = self.ores = None
            return
        dev = sd["res"].device
        if self.res is None:
            self._residuals(dev if dev.type == "cuda" else torch.device("cuda", torch.cuda.current_device()))
        assert sd["res"].numel() in (self.padded, self._kpadded) and sd["ores"].numel() == self.ores.numel(), \
            "residuals of another geometry"
        self.res.zero_()
        self.res[:sd["res"].numel()].copy_(sd["res"].reshape(-1))
        self.ores.copy_(sd["ores"].reshape(self.ores.shape))

    # ---- call ----------------------------------------------------------------
    def __call__(self, g, reverse=False):
        need_cuda(g)
        if self.method == "fp32":
            if self.world > 1:
                dist.all_reduce(g)
            return g.div_(self.world)
        if self.method == "bf16":
            h = g.to(torch.bfloat16)
            if self.world > 1:
                dist.all_reduce(h)
            return g.copy_(h).div_(self.world)
        if self.fp4:
            return self._mxfp4(g, reverse)
        return self._integer(g, reverse)

    def _integer(self, g, reverse):
        """The reference's integer wires (wire.py:104-138) as four kernels on the
        peer-store transport: shared grid from the maximum over ranks, exact
        int32 sum at the owner, owner grid, gather.  `reverse` has no effect:
        integer sums do not depend on the order (tests/test_wire.py:58-59)."""
        h = self._check_args(g)
        check(lib().ls_wire_int_allreduce(h, ptr(g), self.n, ptr(self.res), ptr(self.ores), stream()))
        return g


class LocalWireGroup:
    """All ranks of an MXFP4 wire inside ONE process on one GPU: handles are
    connected with plain pointers and the phases run rank after rank on one
    stream, so no kernel ever waits for another.  Exercises exactly the kernels,
    addressing and flags of the multi-GPU path; used by the single-GPU tests."""

    def __init__(self, world, numel, ef=False, bits=0):
        self.world, self.n, self.ef, self.bits = world, numel, ef, bits
        self.kpadded = -(-numel // (world * _KUNIT)) * world * _KUNIT
        self.handles = []
        for r in range(world):
            h = ctypes.c_void_p()
            if bits:
                check(lib().ls_wire_create_int(r, world, self.kpadded, bits, ctypes.byref(h)))
            else:
                check(lib().ls_wire_create(r, world, self.kpadded, ctypes.byref(h)))
            self.handles.append(h)
        arr = (ctypes.c_void_p * world)(*[h.value for h in self.handles])
        for h in self.handles:
            check(lib().ls_wire_map_local(h, arr))
        dev = torch.device("cuda")
        self.res = [torch.zeros(self.kpadded, device=dev) for _ in range(world)] if ef else [None] * world
        self.ores = [torch.zeros(self.kpadded // world, device=dev) for _ in range(world)] if ef else [None] * world

    def set_dynamic(self, on):
        """Groups handed out from a counter (True) or fixed shares per warp (False); see Wire.set_dynamic."""
        for h in self.handles:
            check(lib().ls_wire_set_dynamic(h, int(bool(on))))

    def step(self, gs, reverse=False):
        """One step with the phases as separate launches, rank after rank."""
        L = lib()
        if self.bits:
            for phase in range(4):
                for r, h in enumerate(self.handles):
                    check(L.ls_wire_int_phase(h, phase, ptr(gs[r]), self.n, ptr(self.res[r]), ptr(self.ores[r]), stream()))
            for h in self.handles:
                check(L.ls_wire_status(h, None))
            return gs
        for r, h in enumerate(self.handles):
            check(L.ls_wire_send(h, ptr(gs[r]), self.n, ptr(self.res[r]), stream()))
        for r, h in enumerate(self.handles):
            check(L.ls_wire_reduce(h, ptr(self.ores[r]), int(reverse), stream()))
        for r, h in enumerate(self.handles):
            check(L.ls_wire_finish(h, ptr(gs[r]), self.n, stream()))
        for h in self.handles:
            check(L.ls_wire_status(h, None))
        return gs

    def step_fused(self, gs, reverse=False, subs=0, stagger=False, check_status=True):
        """One step of every rank as ONE cooperative launch (the pipelined kernel): all
        ranks' CTAs are resident together, so the waits between ranks are real."""
        L = lib()
        assert not self.bits
        vp = ctypes.c_void_p
        for h in self.handles:
            check(L.ls_wire_set_mode(h, 2, subs, int(bool(stagger))))
        hs = (vp * self.world)(*[h.value for h in self.handles])
        g_arr = (vp * self.world)(*[g.data_ptr() for g in gs])
        r_arr = (vp * self.world)(*[None if r is None else r.data_ptr() for r in self.res])
        o_arr = (vp * self.world)(*[None if o is None else o.data_ptr() for o in self.ores])
        check(L.ls_wire_allreduce_group(hs, g_arr, self.n, r_arr, o_arr, int(reverse), stream()))
        if check_status:
            for h in self.handles:
                check(L.ls_wire_status(h, None))
        return gs

    def slots(self, rank, which):
        """Raw bytes this rank received: [world, slot_bytes] uint8."""
        sb = ctypes.c_int64()
        check(lib().ls_wire_debug_slots(self.handles[rank], which, None, ctypes.byref(sb), None))
        out = torch.empty(self.world, sb.value, dtype=torch.uint8, device="cuda")
        check(lib().ls_wire_debug_slots(self.handles[rank], which, ptr(out), ctypes.byref(sb), stream()))
        return out

    def close(self):
        torch.cuda.synchronize()
        for h in self.handles:
            lib().ls_wire_destroy(h)
        self.handles = []


def bench(out, numel, iters):
    """Microbenchmark in the manner of wire.py:141-185: every wire on one
    gradient-sized buffer, median time over `iters` calls and relative error
    against an fp64 all-reduce; rank 0 prints the rows and writes <out>/wire.csv."""
    import csv
    import statistics
    import time
    from pathlib import Path
    rank, world, dev = init()
    common = torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    noise = torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
    grad = common / world + 3 * noise / world ** 0.5            # shared signal + per-rank noise
    exact = grad.double()
    if world > 1:
        dist.all_reduce(exact)
    exact /= world
    table = []
    for method in ("fp32", "bf16", "int16", "int8", "int8ef", "mxfp4", "mxfp4ef"):
        began = time.perf_counter()
        w = Wire(method, numel, world, rank)
        first = w(grad.clone())
        err = ((first.double() - exact).norm() / exact.norm()).item()
        samples = []
        for _ in range(iters):
            buf = grad.clone()
            if world > 1:
                dist.barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            w(buf)
            t1.record()
            torch.cuda.synchronize()
            samples.append(t0.elapsed_time(t1))
        w.status()
        w.close()
        ms = statistics.median(samples)
        table.append({"method": method, "gpus": world, "B_per_el": round(w.bytes_per_el, 4), "ms": round(ms, 3),
                      "grad_GBps": round(numel * 4 / ms / 1e6, 1), "rel_err": f"{err:.3e}",
                      "seconds": round(time.perf_counter() - began, 1)})
        if rank == 0:
            print(table[-1], flush=True)
    if rank == 0:
        Path(out).mkdir(parents=True, exist_ok=True)
        with open(Path(out) / "wire.csv", "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(table[0]))
            wr.writeheader()
            wr.writerows(table)
    if world > 1:
        dist.destroy_process_group()
