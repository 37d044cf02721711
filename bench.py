"""Benchmark of the MXFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over one synthetic batch of the dual-batch
configuration: two activation batches of 4096 x 8192 bf16 are quantized to
MXFP4 on the fly and multiplied, in one launch, by one pre-quantized
8192 x 8192 MXFP4 weight (two 4096 x 8192 bf16 outputs, fp32 accumulation).
With N > 1 every rank runs this step on its own GPU (the GEMM path does not
shard: replicas only) and the line reports the aggregate.

Prints one JSON line (rank 0).  `value` is device-timed over exactly K steps
with inputs resident in HBM; every step carries three events (start, after the
quantizer, after the GEMM), so quantize_ms + gemm_ms = ms_per_step.  The same
loop then keeps running, still timed, until the GPU has been under this load
for about half a second: `value_sustained`, the roofline figures and the clock
record all come from that longer region.  `e2e` is the same step through the
public Python API with pinned HOST buffers, host<->device copies inside the
timed region.

`--impl reference` times the reference's own CPU path for the same step
(quantize both batches, dequantize, fp32 F.linear -> bf16: what lockstep's
fp4_linear.py runs anywhere but on an H100) on the host cores, on the full
configuration.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, N, K = 4096, 8192, 8192
METRIC = "dual MXFP4 GEMM TFLOPS/GPU (% FP4 peak); FP4 all-reduce algbw GB/s @1/2/4/8"
WORKLOAD = "dual-batch packed MXFP4 GEMM: 2 x [4096x8192 bf16, quantized on the fly] @ 8192x8192 MXFP4 W -> 2 x 4096x8192 bf16"
FP4_SPEC_TFLOPS = 9000.0
# DRAM bytes of one dual-GEMM launch on this workload (dram__bytes_read.sum + dram__bytes_write.sum of one
# ncu capture of mxfp4_gemm_pair_kernel).  Not measured by this script: carried with its source.
GEMM_DRAM_BYTES_PER_LAUNCH = 199.64e6
GEMM_DRAM_BYTES_SOURCE = ("one ncu capture (--set full, 1 launch) of mxfp4_gemm_pair_kernel on this workload; "
                          "carried as a constant, not re-measured in this run")
GEMM_ALGORITHMIC_BYTES = 2 * (M * K // 2 + M * K // 32) + (N * K // 2 + N * K // 32) + 2 * M * N * 2
SUSTAINED_SECONDS = 0.5                                 # length of the timed region the clock record covers


def env_int(name, default):
    return int(os.environ.get(name, default))


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.proc, self.path = None, None
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", uuid, f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
            t0 = time.time()                       # wait until the sampler is actually running
            while time.time() - t0 < 5.0 and os.path.getsize(self.path) == 0:
                time.sleep(0.02)
            self.skip = len(Path(self.path).read_text().splitlines())
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        rows = [r.split(",") for r in Path(self.path).read_text().splitlines()[self.skip:] if r.count(",") >= 6]
        os.unlink(self.path)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[0]) for r in rows]
        power = [float(r[2]) for r in rows if r[2].strip().replace(".", "").isdigit()]
        busy = [s for s, r in zip(sm, rows)] if not power else \
            [s for s, pw in zip(sm, power) if pw > 0.5 * max(power)] or sm
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any("Active" == r[3 + i].strip() for r in rows)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "samples": len(rows), "power_w_max": max(power) if power else None}


class CpuReference:
    """The reference's CPU path for the benchmark step (fp4_linear.py:33-40 on the
    non-H100 branch, with W quantized ahead of time as the workload states): per batch
    quantize x, dequantize x and W, fp32 F.linear, cast to bf16.  Uses the oracle port,
    which calls the same torch CPU kernels as the reference: this leg and the
    `cpu_baseline` figure are the places the benchmark may execute it."""

    def __init__(self, rows=M):
        from oracle import ref_port
        self.rp, self.rows = ref_port, rows
        g = torch.Generator().manual_seed(0)
        self.x = [torch.randn(rows, K, generator=g).bfloat16() for _ in range(2)]
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
        self.wc, self.ws = ref_port.quantize(w)                # W is pre-quantized in this configuration
        self.flops = 2 * 2 * rows * N * K

    def step(self):
        t0 = time.perf_counter()
        outs = []
        for x in self.x:
            xc, xs = self.rp.quantize(x)
            outs.append(torch.nn.functional.linear(self.rp.dequantize(xc, xs),
                                                   self.rp.dequantize(self.wc, self.ws)).to(torch.bfloat16))
        return time.perf_counter() - t0

    def sample(self):
        if self.rows == M:
            return (f"the full step: both {M}-row batches against the full {N}x{K} W, oracle port of "
                    "fp4.py / fp4_linear.py on torch CPU")
        return f"{self.rows} of {M} rows of each batch against the full W (not the full configuration)"


def host_threads():
    """Every host core this process may use (torchrun sets OMP_NUM_THREADS=1 for N > 1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(n)
    return torch.get_num_threads()


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = host_threads()
    ref = CpuReference(args.ref_rows)
    for _ in range(args.warmup):
        ref.step()
    times = [ref.step() for _ in range(args.steps)]
    t = sum(times) / len(times)
    val = ref.flops / t / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4 (e2m1 x ue8m0), fp32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sample": ref.sample(),
                                            "ms_per_step_median": statistics.median(times) * 1e3},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": ref.sample()},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_sweep(m_list=(1, 16, 128, 4096, 16384), nk_list=(4096, 8192, 16384)):
    """Shape sweep of the single MXFP4 GEMM: M in {1, 16, 128, 4096, 16384}, N = K in
    {4096, 8192, 16384}; weights N(0, 0.02), activations N(0, 1) with 1 % of the entries
    multiplied by 50.  One dict per shape: TFLOP/s, and for M <= 16 the fraction of
    the bytes roofline (packed W + scales + A + output over the measured HBM peak).
    Launches are replayed from a CUDA graph (device time, not launch overhead); successive
    launches walk through enough copies of the packed weight (> 256 MB together) that no
    launch finds its weight in the 126 MB L2."""
    from lockstep_b200 import fp4, mxfp4_gemm
    dev = torch.device("cuda", 0)
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    lines = []
    for nk in nk_list:
        w = (torch.randn(nk, nk, device=dev, generator=g) * 0.02).bfloat16()
        w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
        del w
        ncopies = max(2, -(-(256 << 20) // (w_pk.numel() + w_sf.numel())))
        w_pks = [w_pk] + [w_pk.clone() for _ in range(ncopies - 1)]
        w_sfs = [w_sf] + [w_sf.clone() for _ in range(ncopies - 1)]
        for m in m_list:
            a = torch.randn(m, nk, device=dev, generator=g)
            a = torch.where(torch.rand(m, nk, device=dev, generator=g) < 0.01, a * 50, a).bfloat16()
            a_pk, a_sf = fp4.quantize_mxfp4_packed(a)
            for i in range(3):
                mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pks[i % ncopies], a_sf, w_sfs[i % ncopies])
            reps = max(ncopies, 20) if m <= 4096 else 5
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                for i in range(reps):
                    c = mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pks[i % ncopies], a_sf, w_sfs[i % ncopies])
            graph.replay()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            graph.replay()
            t1.record()
            torch.cuda.synchronize()
            t_ms = t0.elapsed_time(t1) / reps
            del graph, c
            nbytes = nk * nk * 17 / 32 + m * nk * 17 / 32 + 2 * m * nk
            line = {"shape": [m, nk, nk], "us": t_ms * 1e3, "tflops": 2 * m * nk * nk / t_ms / 1e9,
                    "gbs": nbytes / t_ms / 1e6}
            if m <= 16:
                line["bytes_roofline_frac"] = nbytes / t_ms / 1e6 / pk["hbm"]
            lines.append(line)
        del w_pks, w_sfs
    mxfp4_gemm.gemm_status()
    return lines


def run_shape(m, n, k, out_f32, steps, fmt="mxfp4"):
    """One shape of the single FP4 GEMM: `steps` launches replayed from a CUDA graph
    (device time rather than launch overhead), timed with CUDA events after a 256 MiB
    write that flushes L2.  fmt: "mxfp4" (blocks of 32), "mxfp4-b16" (blocks of 16, UE8M0
    scales) or "nvfp4" (blocks of 16, E4M3 scales).  The quantizer of A (bf16 in) is timed too,
    one launch at a time after the same flush."""
    from lockstep_b200 import fp4, mxfp4_gemm, nvfp4
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    w = (torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16()
    a = torch.randn(m, k, device=dev, generator=g).bfloat16()
    dt = torch.float32 if out_f32 else torch.bfloat16
    if fmt == "nvfp4":
        quant = lambda t: nvfp4.quantize_nvfp4(t)[::2]
        gemm = lambda: nvfp4.nvfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf, dt)
        scale_bytes = 1 / 16 + 4 / 16                             # scale-factor bytes + the fp32 scales
    else:
        block = 16 if fmt == "mxfp4-b16" else 32
        quant = lambda t: fp4.quantize_mxfp4_packed(t, block=block)
        gemm = lambda: mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf, dt, block=block)
        scale_bytes = 1 / block
    w_pk, w_sf = quant(w)
    a_pk, a_sf = quant(a)
    for _ in range(3):
        gemm()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        for _ in range(steps):
            c = gemm()
    graph.replay()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    best, qbest = float("inf"), float("inf")
    for _ in range(3):
        flush.fill_(1)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        graph.replay()
        t1.record()
        flush.fill_(1)
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        quant(a)
        q1.record()
        torch.cuda.synchronize()
        best = min(best, t0.elapsed_time(t1) / steps)
        qbest = min(qbest, q0.elapsed_time(q1))
    del graph, c
    mxfp4_gemm.gemm_status()
    print(json.dumps({"shape": [m, n, k], "format": fmt, "out": "f32" if out_f32 else "bf16", "steps": steps, "us": best * 1e3,
                      "tflops": 2 * m * n * k / best / 1e9,
                      "out_gbs": m * n * (4 if out_f32 else 2) / best / 1e6,
                      "quantize_a_us": qbest * 1e3, "quantize_a_gbs": m * k * (2 + 0.5 + scale_bytes) / qbest / 1e6}), flush=True)


def wire_leg(args, dev, rank, world, barrier, pk):
    """FP4-compressed all-reduce of a 256 MiB fp32 gradient per rank, error feedback on.
    Returns (dict for the line, kernel launches, [ms, send, reduce, finish] for the max over ranks)."""
    import numpy as np
    import torch.distributed as dist
    from lockstep_b200 import wire
    from oracle import cref                                   # checker of the correctness bit only

    # ---- correctness bit, before and outside every timed region: two steps with error feedback on a
    # 1 Mi-element buffer per rank against the CPU oracle of the protocol, and rank against rank
    cn = 1 << 20
    grads = []
    for r in range(world):
        gg = torch.Generator().manual_seed(1000 + r)
        z = torch.randn(cn, generator=gg)
        chi = (torch.randn(3, cn, generator=gg) ** 2).sum(0) / 3
        grads.append((z / chi.sqrt() * 1e-3).float().numpy())
    wchk = wire.Wire("mxfp4ef", cn, world, rank)
    res_c = [np.zeros(wchk._kpadded, np.float32) for _ in range(world)]
    ores_c = [np.zeros(wchk._kpadded // world, np.float32) for _ in range(world)]
    exact = True
    for step in range(2):
        want, _, _ = cref.wire_step([g * (1 + step) for g in grads], res_c, ores_c, unit=256)
        out = wchk(torch.from_numpy(grads[rank] * (1 + step)).to(dev))
        exact = exact and bool(np.array_equal(out.cpu().numpy(), want))
        if world > 1:
            everyone = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(everyone, out)
            exact = exact and all(torch.equal(out, o) for o in everyone)
    wchk.status()
    wchk.close()
    flag = torch.tensor([1.0 if exact else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    exact = bool(flag.item() == 1.0)

    wn = args.wire_elements or ((8 << 20) if args.small else (64 << 20))
    wsteps = max(3, min(args.steps, 30))
    gw = torch.Generator(device=dev).manual_seed(100 + rank)
    z = torch.randn(wn, device=dev, generator=gw)
    chi = torch.zeros(wn, device=dev)
    for _ in range(3):
        chi += torch.randn(wn, device=dev, generator=gw) ** 2
    grad = z / (chi / 3).sqrt() * 1e-3                       # Student-t(3) * 1e-3
    del z, chi
    wobj = wire.Wire("mxfp4ef", wn, world, rank)
    for _ in range(3):
        wobj(grad)
    wobj.status()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(wsteps):
        wobj(grad)
    b.record()
    barrier()
    wobj.status()
    wire_ms = a.elapsed_time(b) / wsteps
    # ---- per phase (three launches with an event between them; ranks aligned by a barrier before each step)
    psteps = 10
    pev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(psteps)]
    for i in range(psteps):
        barrier()
        pev[i][0].record()
        wobj.send(grad)
        pev[i][1].record()
        wobj.reduce()
        pev[i][2].record()
        wobj.finish(grad)
        pev[i][3].record()
    barrier()
    wobj.status()
    phases = [statistics.median(e[j].elapsed_time(e[j + 1]) for e in pev) for j in range(3)]
    mode = wobj.mode_name()
    wobj.close()
    # ---- the reference's own default on the same buffer: Wire("fp32") is NCCL's all-reduce and a division (wire.py:93-95)
    nccl_ms = 0.0
    if world > 1:
        ref = grad.clone()
        for _ in range(3):
            dist.all_reduce(ref)
            ref.div_(world)
        barrier()
        a.record()
        for _ in range(wsteps):
            dist.all_reduce(ref)
            ref.div_(world)
        b.record()
        barrier()
        nccl_ms = a.elapsed_time(b) / wsteps
        del ref
    t = torch.tensor([wire_ms] + phases + [nccl_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    wire_ms, send_ms, reduce_ms, finish_ms, nccl_ms = t.tolist()
    comp = wn * 0.53125                                      # packed + exponent bytes of one buffer
    # per rank and step: send reads g, res and writes res, payload; reduce reads W payloads,
    # ores, writes ores and W payloads; finish reads the payload and writes g
    hbm = wn * (12 + 0.53125) + (wn / world) * (world * 0.53125 + 8 + world * 0.53125) + wn * (0.53125 + 4)
    out = {
        "method": "mxfp4ef", "world": world, "elements_per_rank": wn, "steps": wsteps, "mode": mode,
        "bit_exact": exact, "bit_exact_check": "2 steps, 1 Mi elements per rank, error feedback: every rank's result "
                                               "equals the CPU oracle of the protocol and every other rank's",
        "ms": wire_ms, "algbw_gbs": wn * 4 / (wire_ms * 1e-3) / 1e9,
        "link_busbw_gbs": 2 * (world - 1) / world * comp / (wire_ms * 1e-3) / 1e9,
        "link_peak_gbs": 900.0, "hbm_bytes_per_rank": hbm,
        "hbm_gbs": hbm / (wire_ms * 1e-3) / 1e9, "hbm_peak_gbs": pk["hbm"],
        "hbm_frac": hbm / (wire_ms * 1e-3) / 1e9 / pk["hbm"],
        "phases_ms": {"send": send_ms, "reduce_incl_wait": reduce_ms, "finish_incl_wait": finish_ms,
                      "how": f"three separate launches, median of {psteps} steps, barrier before each step, max over ranks"},
        "data": "Student-t(3) * 1e-3, seed 100 + rank"}
    if world > 1:
        out["nccl_fp32"] = {"ms": nccl_ms, "algbw_gbs": wn * 4 / (nccl_ms * 1e-3) / 1e9,
                            "what": "torch.distributed.all_reduce (NCCL) of the same fp32 buffer + division by the world size: "
                                    "the reference's Wire('fp32'), timed the same way"}
    if world == 1 and not args.no_cpu_baseline:
        cn = 8 << 20                                         # bounded sample of the 64 Mi buffer
        rng = np.random.default_rng(100)
        gc = (rng.standard_t(3, cn) * 1e-3).astype(np.float32)
        res_c, ores_c = [np.zeros(cn, np.float32)], [np.zeros(cn, np.float32)]
        cref.wire_step([gc], res_c, ores_c, unit=256)
        t0 = time.perf_counter()
        cref.wire_step([gc], res_c, ores_c, unit=256)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"algbw_gbs": cn * 4 / dt / 1e9, "cores": os.cpu_count(), "kind": "port",
                               "sample": "8 Mi of 64 Mi elements, one rank, C oracle (OpenMP)"}
    return out, 3 * (2 + 3 + wsteps + psteps)


def copy_bandwidth(dev, hx, hc):
    """Pinned-buffer copy rates of this rank alone in each direction, GB/s (context for `e2e`)."""
    d = torch.empty_like(hx, device=dev)
    out = {}
    for name, fn, nbytes in (("h2d_gbs", lambda: d.copy_(hx, non_blocking=True), hx.numel() * 2),
                             ("d2h_gbs", lambda: hc.view(-1)[:hx.numel()].copy_(d.view(-1), non_blocking=True), hx.numel() * 2)):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            fn()
        b.record()
        torch.cuda.synchronize()
        out[name] = 3 * nbytes / (a.elapsed_time(b) * 1e-3) / 1e9
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-rows", type=int, default=M, help="rows per batch of the CPU reference step (default: all)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--e2e-chunks", type=int, default=2, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--no-wire", action="store_true", help="skip the all-reduce leg")
    ap.add_argument("--no-train", action="store_true", help="skip the FP4-linear training-step leg")
    ap.add_argument("--wire-elements", type=int, default=0, help="elements per rank of the all-reduce leg (profiling runs)")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M <= 16 rows of the shape sweep")
    ap.add_argument("--no-sustained", action="store_true", help="time only the K steps (profiling runs)")
    ap.add_argument("--small", action="store_true", help="1024-row batches (profiling under ncu)")
    ap.add_argument("--sweep", action="store_true", help="shape sweep of the single GEMM instead of the benchmark step")
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), help="time one shape of the single GEMM instead")
    ap.add_argument("--out-f32", action="store_true", help="with --shape: fp32 output instead of bf16")
    ap.add_argument("--format", default="mxfp4", choices=["mxfp4", "mxfp4-b16", "nvfp4"],
                    help="with --shape: operand format (scale blocks of 32, of 16 with UE8M0 scales, of 16 with E4M3 scales)")
    args = ap.parse_args()
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.sweep or args.shape:
        if rank == 0:
            if args.shape:
                run_shape(*args.shape, args.out_f32, min(args.steps, 50), args.format)
            else:
                for line in run_sweep():
                    print(json.dumps(line), flush=True)
        return

    import torch.distributed as dist
    from lockstep_b200 import dual_gemm, fp4, mxfp4_gemm

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    m = 1024 if args.small else M
    flops_step = 2 * 2 * m * N * K
    warmup = max(args.warmup, 3)
    g = torch.Generator(device=dev).manual_seed(rank)
    xs = torch.randn(2, m, K, device=dev, generator=g).bfloat16()        # the two microbatches, one allocation
    x1, x2 = xs[0], xs[1]
    both = xs.view(2 * m, K)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
    w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
    del w
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)        # > 126 MB L2

    class Ev:                                              # start / after the quantizer / after the GEMM
        def __init__(self):
            self.e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def step(ev=None):
        """What dual_gemm.dual_mxfp4(x1, x2, w_pk, w_sf) runs for two adjacent microbatches: one
        quantizer launch over both, one dual-GEMM launch; written out so that an event can sit between."""
        if ev:
            ev.e[0].record()
        p, sf = fp4.quantize_mxfp4_packed(both)
        if ev:
            ev.e[1].record()
        half = sf.numel() // 2
        out = dual_gemm.dual_mxfp4_packed(p[:m], p[m:], w_pk, sf[:half], sf[half:], w_sf)
        if ev:
            ev.e[2].record()
        return out

    for _ in range(warmup):
        c1, c2 = step()
    ref1, ref2 = dual_gemm.dual_mxfp4(x1, x2, w_pk, w_sf)                # the one-call form gives the same bits
    assert torch.equal(ref1, c1) and torch.equal(ref2, c2)
    mxfp4_gemm.gemm_status()

    # ---- device-timed: inputs resident in HBM, L2 flushed between steps.  Exactly K steps between
    # two barriers; then the same loop goes on (timed the same way) until the load has lasted
    # SUSTAINED_SECONDS, so that the clock sampler sees the region the roofline numbers come from.
    evs = [Ev() for _ in range(args.steps)]
    barrier()
    sampler = ClockSampler(dev) if rank == 0 else None
    for _ in range(warmup):                                  # the GPU idled while the sampler started: warm up again
        step()
    barrier()
    for ev in evs:
        flush.zero_()
        step(ev)
    barrier()
    step_ms = sum(ev.e[0].elapsed_time(ev.e[2]) for ev in evs)
    quant_ms_k = sum(ev.e[0].elapsed_time(ev.e[1]) for ev in evs) / args.steps
    gemm_ms_k = sum(ev.e[1].elapsed_time(ev.e[2]) for ev in evs) / args.steps
    # Ceilings measured inside the same region, so that they see the same power state as the step:
    # every 8th step is followed by (1) the MMA-only kernel (the pair kernel's instruction stream of
    # block-scaled FP4 MMAs on operands resident in shared memory: no loads, no scale copies, no
    # epilogue) and (2) cuBLASLt's block-scaled FP4 GEMM as torch exposes it (NVFP4: block 16, E4M3
    # scales; this torch build has no MXFP4 recipe) on 8192^3, the same FLOPs as one dual launch.
    import ctypes
    from lockstep_b200 import _lib
    sus, ceil, trip = [], {}, {"mma_only": [], "cublaslt": [], "own_nvfp4": []}
    if not args.no_sustained:
        L = _lib.lib()
        flop = ctypes.c_double()
        lib_args = None
        if rank == 0 and not args.small:
            try:
                la = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
                lb = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
                lsa = torch.randint(0x30, 0x40, (N * (K // 16),), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
                lsb = torch.randint(0x30, 0x40, (N * (K // 16),), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
                torch._scaled_mm(la, lb.t(), lsa, lsb, out_dtype=torch.bfloat16)
                lib_args = (la, lb.t(), lsa, lsb)
            except Exception as e:                           # not offered by this build / device
                ceil["cublaslt_nvfp4_error"] = repr(e)[:200]
            # this library's NVFP4 GEMM on the shape and operand format of the cuBLASLt call
            from lockstep_b200 import nvfp4
            own = (torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev),
                   torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev),
                   torch.randint(0x30, 0x40, (fp4.sf_bytes(N, K, 16),), dtype=torch.uint8, device=dev),
                   torch.randint(0x30, 0x40, (fp4.sf_bytes(N, K, 16),), dtype=torch.uint8, device=dev))
            nvfp4.nvfp4_gemm_packed(*own)
            _lib.check(L.ls_fp4_mma_peak(600, ctypes.byref(flop), _lib.stream()))
            torch.cuda.synchronize()

        def time_one(fn, key):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            trip[key].append((a, b))
        n_sus = int(min(4000, max(args.steps, SUSTAINED_SECONDS / max(step_ms / args.steps * 1e-3 + 80e-6, 1e-5))))
        sus = [Ev() for _ in range(n_sus)]
        for i, ev in enumerate(sus):
            flush.zero_()
            step(ev)
            if rank == 0 and not args.small and i % 8 == 4:
                time_one(lambda: _lib.check(L.ls_fp4_mma_peak(600, ctypes.byref(flop), _lib.stream())), "mma_only")
                if lib_args:
                    time_one(lambda: torch._scaled_mm(*lib_args, out_dtype=torch.bfloat16), "cublaslt")
                time_one(lambda: nvfp4.nvfp4_gemm_packed(*own), "own_nvfp4")
        barrier()
        med = {k: sorted(a.elapsed_time(b) for a, b in v)[len(v) // 2] for k, v in trip.items() if v}
        if "mma_only" in med:
            ceil["mma_only_tflops"] = flop.value / med["mma_only"] / 1e9
            ceil["how"] = (f"inside the sustained region: after every 8th step one MMA-only launch ({len(trip['mma_only'])} in all) "
                           "one cuBLASLt NVFP4 8192^3 GEMM and this library's NVFP4 GEMM of the same shape, each after an L2 flush; medians")
        if "cublaslt" in med:
            ceil["cublaslt_nvfp4_tflops"] = 2 * N * N * K / med["cublaslt"] / 1e9
        if "own_nvfp4" in med:
            ceil["own_nvfp4_tflops"] = 2 * N * N * K / med["own_nvfp4"] / 1e9
        del lib_args
    clocks = sampler.stop() if sampler else None
    mxfp4_gemm.gemm_status()
    timed = sus if sus else evs
    gemm_all = sorted(ev.e[1].elapsed_time(ev.e[2]) for ev in timed)
    quant_all = sorted(ev.e[0].elapsed_time(ev.e[1]) for ev in timed)
    gemm_ms = gemm_all[len(gemm_all) // 2]                    # median over the region the clocks were sampled on
    quant_ms = quant_all[len(quant_all) // 2]
    sus_ms = sum(ev.e[0].elapsed_time(ev.e[2]) for ev in timed) / len(timed)
    if clocks is not None:
        clocks["region"] = (f"{args.steps} + {len(sus)} timed steps (about {SUSTAINED_SECONDS} s of this load); "
                            "median SM clock over the samples under load")

    # ---- end to end: pinned host buffers in, pinned host buffers out, every step.
    # Row chunks of both batches flow through three streams (copy in, compute, copy out)
    # so that the two PCIe directions and the kernels overlap.
    hx = xs.cpu().pin_memory()
    hc = torch.empty((2, m, N), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    chunks = args.e2e_chunks if m % (args.e2e_chunks * 128) == 0 else 1
    cm = m // chunks
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dx = [torch.empty((2, cm, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dc = [torch.empty((2, cm, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_free_x = [torch.cuda.Event() for _ in range(2)]
    ev_free_c = [torch.cuda.Event() for _ in range(2)]

    def e2e_step():
        main = torch.cuda.current_stream()
        for c in range(chunks):
            b = c & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free_x[b])
                dx[b][0].copy_(hx[0, c * cm:(c + 1) * cm], non_blocking=True)
                dx[b][1].copy_(hx[1, c * cm:(c + 1) * cm], non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            main.wait_event(ev_free_c[b])
            o1, o2 = dual_gemm.dual_mxfp4(dx[b][0], dx[b][1], w_pk, w_sf)
            dc[b][0].copy_(o1)
            dc[b][1].copy_(o2)
            ev_cmp[b].record(main)
            ev_free_x[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                hc[0, c * cm:(c + 1) * cm].copy_(dc[b][0], non_blocking=True)
                hc[1, c * cm:(c + 1) * cm].copy_(dc[b][1], non_blocking=True)
                ev_free_c[b].record(s_out)

    e2e_ms = float("nan")
    copies = {}
    if not args.no_e2e:
        e2e_step()
        torch.cuda.current_stream().wait_stream(s_out)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()                        # steps follow each other without draining the copy streams
        torch.cuda.current_stream().wait_stream(s_out)
        b.record()
        barrier()
        e2e_ms = a.elapsed_time(b) / e2e_steps
        assert torch.equal(hc[0], ref1.cpu()) and torch.equal(hc[1], ref2.cpu()), "host-buffer path disagrees"
        barrier()
        copies = copy_bandwidth(dev, hx, hc)                  # all ranks at once: what the host gives N GPUs together
        barrier()
    del dx, dc, flush

    pk = peaks()
    allreduce, wire_launches = None, 0
    if not args.no_wire:
        allreduce, wire_launches = wire_leg(args, dev, rank, world, barrier, pk)

    train = None
    if not args.no_train and not args.small:                 # every rank takes part (the sync is a collective)
        import train_bench
        torch.cuda.empty_cache()
        train = train_bench.report(dev, world=world, rank=rank)
        tt = torch.tensor([train["sync"]["after_backward_ms"], train["sync"]["sent_under_backward_ms"]], device=dev,
                          dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            train["sync"]["after_backward_ms"], train["sync"]["sent_under_backward_ms"] = tt.tolist()
            train["block_linears"]["mxfp4"]["ms_per_step"] = tt[0].item()
            train["block_linears"]["mxfp4"]["tokens_per_s"] = world * 16 * 1024 / (tt[0].item() * 1e-3)

    t = torch.tensor([step_ms, e2e_ms, sus_ms, copies.get("h2d_gbs", 0.0), copies.get("d2h_gbs", 0.0)],
                     device=dev, dtype=torch.float64)
    if world > 1:                                             # times: max over ranks; copy rates: sum over ranks
        tsum = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    else:
        tsum = t
    step_ms_max, e2e_ms_max, sus_ms_max = t.tolist()[:3]
    h2d_sum, d2h_sum = tsum.tolist()[3:]

    if rank == 0:
        value = world * flops_step * args.steps / (step_ms_max * 1e-3) / 1e12
        gemm_tflops = flops_step / (gemm_ms * 1e-3) / 1e12
        bf16x4 = 4 * pk["bf16"]
        fp4_peak = ceil.get("mma_only_tflops") or bf16x4
        mhz = clocks.get("sm_mhz") if clocks else None
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": step_ms_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4 (e2m1 x ue8m0), fp32 accumulate",
            "data": "synthetic",
            "value_sustained": world * flops_step / (sus_ms_max * 1e-3) / 1e12,
            "config": {"workload": WORKLOAD if not args.small else WORKLOAD.replace("4096x8192 bf16", "1024x8192 bf16"),
                       "step": "dual_gemm.dual_mxfp4: quantize A1 and A2 (1 launch over both microbatches) + dual GEMM "
                               "(1 launch); W pre-quantized",
                       "parallelism": f"replicas x{world}", "l2": "256 MiB buffer written between timed steps",
                       "quantize_ms": quant_ms_k, "gemm_ms": gemm_ms_k,
                       "timing": "three events per step: quantize_ms + gemm_ms = ms_per_step (means over the K steps, rank 0)",
                       "sustained": {"steps": len(timed), "ms_per_step": sus_ms_max, "quantize_ms_median": quant_ms,
                                     "gemm_ms_median": gemm_ms,
                                     "gemm_us_x_ghz": None if not mhz else gemm_ms * 1e3 * mhz / 1e3}},
            "e2e": {"value": world * flops_step / (e2e_ms_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": hx.numel() * 2, "d2h_bytes_per_step": hc.numel() * 2,
                    "pipeline": f"{chunks} row chunks over copy-in / compute / copy-out streams",
                    "ms_per_step": e2e_ms_max,
                    "copy_only": {"h2d_gbs_all_ranks": h2d_sum, "d2h_gbs_all_ranks": d2h_sum,
                                  "how": "every rank copies its own 134 MB pinned buffer at the same time, one direction "
                                         "at a time; sum over ranks"}},
            "gpu_launches": 2 * (2 * warmup + 1 + args.steps + len(sus)) + len(trip["mma_only"]) + 2 * chunks * (e2e_steps + 2) + wire_launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "mxfp4_gemm_pair_kernel (cta_group::2, dual batch)",
                         "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                         "timed": f"median launch duration over the {len(timed)} steps of the sustained region (events "
                                  "around the launch, on its stream)",
                         "peak_source": ("block-scaled FP4 MMA-only kernel measured in this run inside the same timed region "
                                         "(ls_fp4_mma_peak: the pair kernel's MMA stream on operands resident in shared memory)"
                                         if ceil.get("mma_only_tflops") else
                                         f"4 x {pk['source']} bf16 burst {pk['bf16']} (small run: no FP4 figure measured)"),
                         "ceilings": ceil or None,
                         "frac_of_4x_bf16_burst": gemm_tflops / bf16x4,
                         "bf16_peaks": f"{pk['source']}: burst {pk['bf16']}, sustained {pk['bf16_sustained']} TFLOP/s",
                         "frac_of_spec": gemm_tflops / FP4_SPEC_TFLOPS, "spec_tflops": FP4_SPEC_TFLOPS,
                         "flop_per_launch": flops_step,
                         "traffic": None if args.small else GEMM_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": None if args.small else GEMM_DRAM_BYTES_SOURCE,
                         "algorithmic_bytes": None if args.small else GEMM_ALGORITHMIC_BYTES},
        }
        if allreduce:
            line["allreduce"] = allreduce
        if train is not None:
            line["train_step"] = train
        if world == 1 and not args.no_sweep and not args.small:
            torch.cuda.empty_cache()
            line["sweep_skinny"] = {"lines": run_sweep(m_list=(1, 16)),
                                    "what": "single MXFP4 GEMM, M <= 16, N = K in {4096, 8192, 16384}: us per launch "
                                            "(CUDA graph, weights not in L2) and fraction of the bytes roofline"}
        if world == 1 and not args.no_cpu_baseline:
            cores = host_threads()
            ref = CpuReference(M)
            dts = [ref.step() for _ in range(2)]
            line["cpu_baseline"] = {"value": ref.flops / min(dts) / 1e12, "unit": "TFLOP/s", "cores": cores,
                                    "kind": "port", "sample": ref.sample() + ", best of 2"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
