"""Benchmark of the MXFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over one synthetic batch of the dual-batch
configuration: two activation batches of 4096 x 8192 bf16 are quantized to
MXFP4 on the fly and multiplied, in one launch, by one pre-quantized
8192 x 8192 MXFP4 weight (two 4096 x 8192 bf16 outputs, fp32 accumulation).
With N > 1 every rank runs this step on its own GPU (the GEMM path does not
shard: replicas only) and the line reports the aggregate.

Prints one JSON line (rank 0).  `value` is device-timed with inputs resident
in HBM; `e2e` is the same step through the public Python API with pinned HOST
buffers, host<->device copies inside the timed region.

`--impl reference` times the reference's own CPU path for the same step
(quantize both batches, dequantize, fp32 F.linear: what lockstep's
fp4_linear.py runs anywhere but on an H100) on the host cores, on a bounded
row sample of the batch.
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
FLOPS_PER_STEP = 2 * 2 * M * N * K                      # two batches
METRIC = "dual MXFP4 GEMM TFLOPS/GPU (% FP4 peak); FP4 all-reduce algbw GB/s @1/2/4/8"
WORKLOAD = "dual-batch packed MXFP4 GEMM: 2 x [4096x8192 bf16, quantized on the fly] @ 8192x8192 MXFP4 W -> 2 x 4096x8192 bf16"
FP4_SPEC_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one dual-GEMM launch on this workload, from the
# ncu capture summarised in profiles/mxfp4_gemm_pair_dual_4096x8192x8192.md
GEMM_DRAM_BYTES_PER_LAUNCH = 197.87e6
GEMM_ALGORITHMIC_BYTES = 2 * (M * K // 2 + M * K // 32) + (N * K // 2 + N * K // 32) + 2 * M * N * 2
CPU_SAMPLE_ROWS = 256                                   # rows per batch in the CPU-baseline sample


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


def cpu_reference_step(rows, threads=None):
    """The reference's CPU path for `rows` rows of each batch; returns
    (seconds, flops).  Uses the oracle port: this leg is the one place the
    benchmark may execute it."""
    from oracle import ref_port
    if threads:
        torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    x1 = torch.randn(rows, K, generator=g).bfloat16()
    x2 = torch.randn(rows, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    wc, ws = ref_port.quantize(w)                          # W is pre-quantized in this configuration
    t0 = time.perf_counter()
    outs = []
    for x in (x1, x2):
        xc, xs = ref_port.quantize(x)
        outs.append(torch.nn.functional.linear(ref_port.dequantize(xc, xs),
                                               ref_port.dequantize(wc, ws)).to(torch.bfloat16))
    dt = time.perf_counter() - t0
    return dt, 2 * 2 * rows * N * K


def run_reference(args, rank, world):
    if rank != 0:
        return
    args.steps = min(args.steps, 5)          # each step is seconds of CPU work
    # every host core this process may use (torchrun sets OMP_NUM_THREADS=1 for N > 1)
    torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = torch.get_num_threads()
    for _ in range(min(args.warmup, 1)):
        cpu_reference_step(CPU_SAMPLE_ROWS)
    times = []
    flops = 0
    for _ in range(args.steps):
        dt, flops = cpu_reference_step(CPU_SAMPLE_ROWS)
        times.append(dt)
    t = sum(times) / len(times)
    val = flops / t / 1e12
    sample = f"{CPU_SAMPLE_ROWS} of {M} rows of each batch, full 8192x8192 W, oracle port of fp4.py/fp4_linear.py on torch CPU"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3 * (M / CPU_SAMPLE_ROWS),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4 (e2m1 x ue8m0), fp32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_sweep(args):
    """Shape sweep of the single MXFP4 GEMM: M in {1, 16, 128, 4096, 16384}, N = K in
    {4096, 8192, 16384}; weights N(0, 0.02), activations N(0, 1) with 1 % of the entries
    multiplied by 50.  One JSON line per shape: TFLOP/s, and for M <= 16 the fraction of
    the bytes roofline (packed W + scales + A + output over the measured HBM peak)."""
    from lockstep_b200 import fp4, mxfp4_gemm
    dev = torch.device("cuda", 0)
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    for nk in (4096, 8192, 16384):
        w = (torch.randn(nk, nk, device=dev, generator=g) * 0.02).bfloat16()
        w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
        del w
        for m in (1, 16, 128, 4096, 16384):
            a = torch.randn(m, nk, device=dev, generator=g)
            a = torch.where(torch.rand(m, nk, device=dev, generator=g) < 0.01, a * 50, a).bfloat16()
            a_pk, a_sf = fp4.quantize_mxfp4_packed(a)
            for _ in range(3):
                mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf)
            reps = 20 if m <= 4096 else 5
            # replayed as a CUDA graph so that small shapes show device time, not launch overhead
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                for _ in range(reps):
                    c = mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf)
            graph.replay()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            graph.replay()
            t1.record()
            torch.cuda.synchronize()
            ms = t0.elapsed_time(t1) / reps
            del graph, c
            nbytes = nk * nk * 17 / 32 + m * nk * 17 / 32 + 2 * m * nk
            line = {"shape": [m, nk, nk], "us": ms * 1e3, "tflops": 2 * m * nk * nk / ms / 1e9,
                    "gbs": nbytes / ms / 1e6}
            if m <= 16:
                line["bytes_roofline_frac"] = nbytes / ms / 1e6 / pk["hbm"]
            print(json.dumps(line), flush=True)
    mxfp4_gemm.gemm_status()


def run_shape(m, n, k, out_f32, steps):
    """One shape of the single MXFP4 GEMM: `steps` launches replayed from a CUDA graph
    (device time rather than launch overhead), timed with CUDA events after a 256 MiB
    write that flushes L2."""
    from lockstep_b200 import fp4, mxfp4_gemm
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    w = (torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16()
    a = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
    a_pk, a_sf = fp4.quantize_mxfp4_packed(a)
    dt = torch.float32 if out_f32 else torch.bfloat16
    for _ in range(3):
        mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf, dt)
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        for _ in range(steps):
            c = mxfp4_gemm.mxfp4_gemm_packed(a_pk, w_pk, a_sf, w_sf, dt)
    graph.replay()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    best = float("inf")
    for _ in range(3):
        flush.fill_(1)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        graph.replay()
        t1.record()
        torch.cuda.synchronize()
        best = min(best, t0.elapsed_time(t1) / steps)
    del graph, c
    mxfp4_gemm.gemm_status()
    print(json.dumps({"shape": [m, n, k], "out": "f32" if out_f32 else "bf16", "steps": steps, "us": best * 1e3,
                      "tflops": 2 * m * n * k / best / 1e9,
                      "out_gbs": m * n * (4 if out_f32 else 2) / best / 1e6}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--e2e-chunks", type=int, default=2, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--no-wire", action="store_true", help="skip the all-reduce leg")
    ap.add_argument("--no-train", action="store_true", help="skip the FP4-linear training-step leg")
    ap.add_argument("--small", action="store_true", help="1024-row batches (profiling under ncu)")
    ap.add_argument("--sweep", action="store_true", help="shape sweep of the single GEMM instead of the benchmark step")
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), help="time one shape of the single GEMM instead")
    ap.add_argument("--out-f32", action="store_true", help="with --shape: fp32 output instead of bf16")
    args = ap.parse_args()
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.sweep or args.shape:
        if rank == 0:
            if args.shape:
                run_shape(*args.shape, args.out_f32, min(args.steps, 50))
            else:
                run_sweep(args)
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
    g = torch.Generator(device=dev).manual_seed(rank)
    xs = torch.randn(2, m, K, device=dev, generator=g).bfloat16()        # the two microbatches, one allocation
    x1, x2 = xs[0], xs[1]
    w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
    w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
    del w
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)        # > 126 MB L2

    def step():                                            # the public call: quantize both batches + dual GEMM
        return dual_gemm.dual_mxfp4(x1, x2, w_pk, w_sf)

    for _ in range(max(args.warmup, 3)):
        c1, c2 = step()
    mxfp4_gemm.gemm_status()

    # ---- device-timed: inputs resident in HBM, L2 flushed between steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
    barrier()
    sampler = ClockSampler(dev) if rank == 0 else None
    t_start = time.time()
    for i in range(args.steps):
        flush.zero_()
        ev[i][0].record()
        c1, c2 = step()
        ev[i][1].record()
    barrier()
    extra = 0
    if sampler:
        # nvidia-smi samples every 20 ms: a short timed region is followed by more (untimed)
        # steps of the same load until the sampler has seen at least 0.3 s of it
        while time.time() - t_start < 0.3:
            for _ in range(20):
                step()
            torch.cuda.synchronize()
            extra += 20
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["extra_untimed_steps"] = extra
    mxfp4_gemm.gemm_status()
    step_ms = sum(e[0].elapsed_time(e[1]) for e in ev)

    # ---- the dominant kernel alone (roofline): one dual-GEMM launch over both full batches
    pk, sf = fp4.quantize_mxfp4_packed(xs.view(2 * m, K))
    half = sf.numel() // 2
    gsteps = max(3, min(args.steps, 200))
    gev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(gsteps)]
    for i in range(gsteps):
        flush.zero_()
        gev[i][0].record()
        dual_gemm.dual_mxfp4_packed(pk[:m], pk[m:], w_pk, sf[:half], sf[half:], w_sf)
        gev[i][1].record()
    torch.cuda.synchronize()
    gemm_ms = sum(e[0].elapsed_time(e[1]) for e in gev) / gsteps
    qev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    flush.zero_()
    qev[0].record()
    for _ in range(10):
        fp4.quantize_mxfp4_packed(xs.view(2 * m, K))
    qev[1].record()
    torch.cuda.synchronize()
    quant_ms = qev[0].elapsed_time(qev[1]) / 10
    del pk, sf

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
        ref1, ref2 = dual_gemm.dual_mxfp4(x1, x2, w_pk, w_sf)
        assert torch.equal(hc[0], ref1.cpu()) and torch.equal(hc[1], ref2.cpu()), "host-buffer path disagrees"

    # ---- FP4-compressed all-reduce of a 256 MiB fp32 gradient per rank (error feedback on)
    from lockstep_b200 import wire
    wn = (8 << 20) if args.small else (64 << 20)
    wsteps = 0 if args.no_wire else max(3, min(args.steps, 30))
    wire_ms = float("nan")
    if wsteps:
        del flush
        gw = torch.Generator(device=dev).manual_seed(100 + rank)
        z = torch.randn(wn, device=dev, generator=gw)
        chi = torch.zeros(wn, device=dev)
        for _ in range(3):
            chi += torch.randn(wn, device=dev, generator=gw) ** 2
        grad = z / (chi / 3).sqrt() * 1e-3                   # Student-t(3) * 1e-3
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
        wobj.close()

    t = torch.tensor([step_ms, e2e_ms, gemm_ms, wire_ms], device=dev, dtype=torch.float64)  # max over ranks below
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms_max, e2e_ms_max, gemm_ms_max, wire_ms_max = t.tolist()

    if rank == 0:
        pk = peaks()
        value = world * flops_step * args.steps / (step_ms_max * 1e-3) / 1e12
        gemm_tflops = flops_step / (gemm_ms * 1e-3) / 1e12
        fp4_peak = 4 * pk["bf16"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "mxfp4 (e2m1 x ue8m0), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": WORKLOAD if not args.small else WORKLOAD.replace("4096x8192 bf16", "1024x8192 bf16"),
                       "step": "dual_gemm.dual_mxfp4: quantize A1 and A2 (1 launch over both microbatches) + dual GEMM "
                               "(1 launch); W pre-quantized",
                       "parallelism": f"replicas x{world}", "l2": "256 MiB buffer written between timed steps",
                       "quantize_ms": quant_ms, "gemm_ms": gemm_ms},
            "e2e": {"value": world * flops_step / (e2e_ms_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": hx.numel() * 2, "d2h_bytes_per_step": hc.numel() * 2,
                    "pipeline": f"{chunks} row chunks over copy-in / compute / copy-out streams",
                    "ms_per_step": e2e_ms_max},
            "gpu_launches": 2 * args.steps + gsteps + 10 + 3 * wsteps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "mxfp4_gemm_pair_kernel (cta_group::2, dual batch)",
                         "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                         "peak_source": f"4 x {pk['source']} bf16 burst {pk['bf16']} (no FP4 figure is measured); "
                                        f"spec dense FP4 {FP4_SPEC_TFLOPS}",
                         "frac_of_spec": gemm_tflops / FP4_SPEC_TFLOPS,
                         "flop_per_launch": flops_step,
                         "traffic": None if args.small else GEMM_DRAM_BYTES_PER_LAUNCH,
                         "algorithmic_bytes": None if args.small else GEMM_ALGORITHMIC_BYTES},
        }
        if wsteps:
            comp = wn * 0.53125                              # packed + exponent bytes of one buffer
            # per rank and step: send reads g, res and writes res, payload; reduce reads W payloads,
            # ores, writes ores and W payloads; finish reads the payload and writes g
            hbm = wn * (12 + 0.53125) + (wn / world) * (world * 0.53125 + 8 + world * 0.53125) + wn * (0.53125 + 4)
            line["allreduce"] = {
                "method": "mxfp4ef", "world": world, "elements_per_rank": wn, "steps": wsteps,
                "ms": wire_ms_max, "algbw_gbs": wn * 4 / (wire_ms_max * 1e-3) / 1e9,
                "link_busbw_gbs": 2 * (world - 1) / world * comp / (wire_ms_max * 1e-3) / 1e9,
                "link_peak_gbs": 900.0, "hbm_bytes_per_rank": hbm,
                "hbm_gbs": hbm / (wire_ms_max * 1e-3) / 1e9, "hbm_peak_gbs": pk["hbm"],
                "hbm_frac": hbm / (wire_ms_max * 1e-3) / 1e9 / pk["hbm"], "data": "Student-t(3) * 1e-3, seed 100 + rank"}
        if wsteps and world == 1 and not args.no_cpu_baseline:
            import numpy as np
            from oracle import cref
            cn = 8 << 20                                     # bounded sample of the 64 Mi buffer
            rng = np.random.default_rng(100)
            gc = (rng.standard_t(3, cn) * 1e-3).astype(np.float32)
            res_c, ores_c = [np.zeros(cn, np.float32)], [np.zeros(cn, np.float32)]
            cref.wire_step([gc], res_c, ores_c, unit=256)
            t0 = time.perf_counter()
            cref.wire_step([gc], res_c, ores_c, unit=256)
            dt = time.perf_counter() - t0
            line["allreduce"]["cpu_baseline"] = {"algbw_gbs": cn * 4 / dt / 1e9, "cores": os.cpu_count(), "kind": "port",
                                                 "sample": "8 Mi of 64 Mi elements, one rank, C oracle (OpenMP)"}
        if world == 1 and not args.no_train and not args.small:
            from lockstep_b200 import gpt
            torch.cuda.empty_cache()
            tr = {}
            for mode in ("ste", "mxfp4"):
                sec, loss = gpt.training_step_time(backward=mode, steps=5, warmup=2, device=dev)
                tr[mode] = {"tokens_per_s": 16 * 1024 / sec, "ms_per_step": sec * 1e3, "loss": loss}
            line["train_step"] = {"model": "decoder-only 12L d1024 h16 ffn4096 seq1024 batch16 vocab32000, every block "
                                           "linear MXFP4Linear, bf16 autocast, fused AdamW, synthetic ids seed 0",
                                  "backward": tr}
        if world == 1 and not args.no_cpu_baseline:
            dt, fl = cpu_reference_step(CPU_SAMPLE_ROWS)
            dt2, fl = cpu_reference_step(CPU_SAMPLE_ROWS)
            line["cpu_baseline"] = {"value": fl / min(dt, dt2) / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                    "kind": "port",
                                    "sample": f"{CPU_SAMPLE_ROWS} of {M} rows of each batch against the full W, best of 2"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
