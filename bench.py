#!/usr/bin/env python
"""Benchmark of the EXL3 streamed GEMV (batch-1 decode) on B200.

Workload (the batch-1..16 GEMV sweep configuration the headline metric is quoted on): the three
27B-class decode shapes 5120->17408 (gate/up), 17408->5120 (down) and 5120->5120
(o_proj) at K = 4 bits/weight, 3INST codebook, one activation row, random packed
trellis words and random +-1 sign vectors (seeded synthetic data; decode cost is
value-independent).  One STEP is one pass over a ring of `--ring` such layer sets
with distinct weights (default 16 sets = 1.6 GB of packed weights, far larger than
the 126 MB L2, so every step streams from HBM).  The step is captured in a CUDA
graph; `value` = packed weight bytes of the step / device time.

    python bench.py                      # 1 GPU
    torchrun ... bench.py --gpus N       # tensor-parallel by output tile + all-gather
    python bench.py --impl reference     # the CPU oracle port on all host cores
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [(5120, 17408), (17408, 5120), (5120, 5120)]
WORKLOAD = ("configs[1]: batch-1 GEMV, K=4, 3INST, shapes 5120x17408 + 17408x5120 + 5120x5120")
K_BITS, CB, ROWS = 4, 0, 1
CB_NAMES = {0: "3INST", 1: "MCG", 2: "MUL1"}
METRIC = "exl3_gemv_packed_weight_bandwidth"
UNIT = "GB/s"
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum over packed weight bytes, from the ncu capture of
# the K=4 batch-1 GEMV 5120 -> 17408
DRAM_TRAFFIC_RATIO = 1.0028
# dram read + write per tile of the encoder workload (592 tiles, K=4), from its ncu capture
ENCODE_DRAM_BYTES_PER_TILE = (97.128867e9 + 159.096134e9) / 592


def packed_bytes(shape, k=K_BITS):
    return shape[0] * shape[1] * k // 8


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------ clocks -----

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------------ reference arm -----

def cpu_pass(oracle, np, layers, x_by_in, budget_s: float):
    """Times the oracle's forward (decode + rotations + GEMV) over `layers`; returns
    (packed bytes done, seconds).  Stops after `budget_s` seconds at a layer boundary."""
    done, t0 = 0, time.perf_counter()
    for (inf, outf, tr, suh, svh) in layers:
        oracle.linear_forward(x_by_in[inf], tr, K_BITS, CB, suh, svh)
        done += inf * outf * K_BITS // 8
        if time.perf_counter() - t0 > budget_s:
            break
    return done, time.perf_counter() - t0


def make_cpu_layers(np, seed: int):
    layers, xs = [], {}
    for i, (inf, outf) in enumerate(SHAPES):
        rng = np.random.default_rng(seed + i)
        tr = rng.integers(0, 65536, size=(inf // 16, outf // 16, 16 * K_BITS), dtype=np.uint16)
        suh = np.where(rng.random(inf) > 0.5, -1.0, 1.0).astype(np.float16)
        svh = np.where(rng.random(outf) > 0.5, -1.0, 1.0).astype(np.float16)
        layers.append((inf, outf, tr, suh, svh))
        xs.setdefault(inf, rng.standard_normal((ROWS, inf)).astype(np.float16))
    return layers, xs


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path.  The reference is
    pure Python/numpy and does not travel to the GPU box, so this arm times its C
    restatement (oracle/, pinned bit-exact to the reference's decoded weights) with all
    host threads, on the same workload; each step is one layer set (three layers)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import exl3_oracle as oracle

    oracle.lib()
    cores = oracle.host_cores()
    oracle.set_threads(cores)
    layers, xs = make_cpu_layers(np, 1000)
    for _ in range(min(args.warmup, 1)):
        cpu_pass(oracle, np, layers[:1], xs, 1e9)
    steps = max(1, min(args.steps, 5))
    total, t = 0, 0.0
    for _ in range(steps):
        b, dt = cpu_pass(oracle, np, layers, xs, 1e9)
        total += b
        t += dt
    value = total / t / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * t / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": ROWS, "k": K_BITS, "codebook": "3INST",
                   "step": "one layer set per step (GB/s does not depend on the step size)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{steps} x one layer set ({len(SHAPES)} layer(s), "
                                   f"{sum(packed_bytes(s) for s in SHAPES) / 1e6:.1f} MB packed)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------ GPU arm -----

_RESULT_FD = None


def quiet_stdout():
    """Libraries print banners on stdout (NCCL's version line, for one); the result line must be
    the only thing there.  Everything written to fd 1 from here on goes to stderr; `emit` writes
    the result to the real stdout."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def finish_ranks(dist):
    """End of a multi-rank run (the caller has dropped its CUDA graph: captured NCCL kernels
    must be gone before the communicator).  If tearing the process group down still does not
    return promptly, the ranks leave without it — their results are already printed."""
    import gc
    import torch
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    done = threading.Event()

    def teardown():
        try:
            dist.destroy_process_group()
        finally:
            done.set()

    threading.Thread(target=teardown, daemon=True).start()
    if not done.wait(20.0):
        os._exit(0)


def shard_cols(outf: int, world: int, rank: int):
    """Column range owned by `rank` (tensor parallel by output tile, whole 128-column blocks)."""
    from ponyexl3_b200.parallel import shard_columns
    return shard_columns(outf, world, rank)


def run_gpu(args):
    import numpy as np
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))

    from ponyexl3_b200 import EXL3Layer, _lib, ops
    from ponyexl3_b200.linear import EXL3Linear

    lib = _lib.load()
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000)

    # ---- layers: ring of sets, each rank holding its column slice -------------------
    class DevLayer:
        pass

    layers = []
    step_bytes_global = 0
    for s in range(args.ring):
        for (inf, outf) in SHAPES:
            c0, c1 = shard_cols(outf, world, rank)
            L = DevLayer()
            L.inf, L.outf, L.c0, L.c1 = inf, outf, c0, c1
            L.trellis = torch.randint(-32768, 32767, (inf // 16, (c1 - c0) // 16, 16 * K_BITS),
                                      dtype=torch.int16, device=dev, generator=gen)
            L.suh = (torch.randint(0, 2, (inf,), device=dev, generator=gen) * 2 - 1).to(torch.float16)
            L.svh = (torch.randint(0, 2, (c1 - c0,), device=dev, generator=gen) * 2 - 1).to(torch.float16)
            L.y_full = torch.empty((ROWS, outf), dtype=torch.float16, device=dev)
            L.y = torch.empty((ROWS, c1 - c0), dtype=torch.float16, device=dev)
            layers.append(L)
            step_bytes_global += packed_bytes((inf, outf))
    xs = {inf: torch.randn((ROWS, inf), device=dev, generator=gen).to(torch.float16)
          for inf in {s[0] for s in SHAPES}}
    from ponyexl3_b200.parallel import all_gather_columns

    # N > 1: every layer's output row is completed on every rank.  Default: the GEMV epilogue
    # stores its blocks into all ranks' rows over peer memory (exl3_gemv_peers) and the NEXT layer's
    # kernel waits for the arrivals (a one-thread wait kernel after the last layer of the step);
    # --nccl-gather uses an NCCL all-gather per layer instead.
    peer = None
    if dist is not None and not args.nccl_gather:
        from ponyexl3_b200.parallel import PeerExchange
        # one (row buffer, counter) pair per layer of the step: the step's result is the ring itself
        peer = PeerExchange(ROWS, max(s[1] for s in SHAPES), ring=len(layers))

    def one_layer(L, x):
        if dist is None:
            ops.gemv(x, L.trellis, K_BITS, CB, L.suh, L.svh, None, pdl=True, out=L.y, fast_accum=args.fast_accum)
        elif peer is not None:
            # the wait for a layer's arrivals is folded into the next layer's kernel
            L.y_full = ops.gemv_peers(x, L.trellis, K_BITS, CB, L.suh, L.svh, None, exchange=peer,
                                      out_features_total=L.outf, col0=L.c0, pdl=True, defer_wait=True)
        else:
            # between NCCL kernels plain stream order is kept (no programmatic launch)
            ops.gemv(x, L.trellis, K_BITS, CB, L.suh, L.svh, None, pdl=False, out=L.y)
            if ROWS == 1 and (L.outf // 128) % world == 0:
                # one row, even split: the gathered chunks ARE the full row, no reshuffle
                dist.all_gather_into_tensor(L.y_full.view(-1), L.y.view(-1))
            else:
                L.y_full = all_gather_columns(L.y, L.outf)

    def step_body():
        if peer is not None:
            peer.restart()
        for L in layers:
            one_layer(L, xs[L.inf])
        if peer is not None:
            peer.settle(pdl=True)          # the last layer's arrivals

    stream = torch.cuda.Stream(device=dev)
    # NCCL all-gathers are captured with the kernels; every rank captures the same sequence
    use_graph = not args.no_graph
    graph = None
    with torch.cuda.stream(stream):
        step_body()  # allocates the workspace outside capture
        stream.synchronize()
        if use_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step_body()
            except Exception as e:  # capture not possible: run the launches eagerly
                if dist is not None:
                    raise       # ranks must not diverge (graph on one, eager on another)
                graph = None
                torch.cuda.synchronize()
                if rank == 0:
                    print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); eager launches",
                          file=sys.stderr)

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step_body()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run_step()
        barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        # keep the GPU under the same load a little longer so the clock sampler sees it; a
        # fixed step count, because every rank must issue the same number of collectives
        extra = max(args.steps, int(250.0 / max(ms / args.steps, 1e-3))) if dist is None else args.steps
        for _ in range(min(extra, 2000)):
            run_step()
        torch.cuda.synchronize()
        clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = ops.Workspace.get(dev, ROWS, max(s[0] for s in SHAPES)).status()

    # ---- end to end through the module API with host buffers --------------------------------
    mods = []
    for L in layers:
        m = EXL3Linear.from_device_tensors(trellis=L.trellis, k=K_BITS, cb=CB, suh=L.suh, svh=L.svh,
                                           key="bench")
        m.pdl = dist is None
        m.full_out = L.outf
        mods.append(m)
    h_in = {inf: torch.randn((ROWS, inf)).to(torch.float16).pin_memory() for inf in xs}
    d_in = {inf: torch.empty_like(xs[inf]) for inf in xs}
    h2d = sum(v.numel() * 2 for v in h_in.values())
    e2e_graph = None
    if dist is None or peer is None:
        # the step's result: every layer's output row, side by side in one device buffer that goes
        # back to pinned host memory in one copy at the end of the step
        widths = [m.full_out if dist is not None else m.out_features for m in mods]
        d_out = torch.empty((ROWS, sum(widths)), dtype=torch.float16, device=dev)
        h_out = torch.empty((ROWS, sum(widths)), dtype=torch.float16).pin_memory()
        offs = [0]
        for wd in widths:
            offs.append(offs[-1] + wd)
        d_views = [d_out[:, a:b] for a, b in zip(offs[:-1], offs[1:])]

        def e2e_step():
            for inf in h_in:
                d_in[inf].copy_(h_in[inf], non_blocking=True)
            if dist is None:
                for m, dv in zip(mods, d_views):
                    m(d_in[m.in_features], out=dv)
            else:
                for L, dv in zip(layers, d_views):
                    one_layer(L, d_in[L.inf])
                    dv.copy_(L.y_full)
            h_out.copy_(d_out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e2e_api = "EXL3Linear.forward per layer, pinned host x and y"
    else:
        # N > 1 over peer memory: every layer's completed row lands in its own slot of the exchange
        # ring, so the whole ring goes back to the host in one copy; H2D, the layers and D2H are
        # one CUDA graph (one launch per step instead of ~150 host calls)
        d_out = peer.buf[:peer.ring * peer.slot_elems * 2].view(torch.float16)
        h_out = torch.empty(d_out.shape, dtype=torch.float16).pin_memory()

        def e2e_body():
            for inf in h_in:
                d_in[inf].copy_(h_in[inf], non_blocking=True)
            peer.restart()
            for L in layers:
                one_layer(L, d_in[L.inf])
            peer.settle(pdl=True)
            h_out.copy_(d_out, non_blocking=True)

        with torch.cuda.stream(stream):
            e2e_body()
            stream.synchronize()
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph, stream=stream):
                e2e_body()

        def e2e_step():
            e2e_graph.replay()
            stream.synchronize()
        e2e_api = ("ops.gemv_peers per layer (output rows completed on every rank over peer memory), pinned "
                   "host x and y, the step captured in one CUDA graph")
    d2h = h_out.numel() * 2

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # ---- N > 1: is the gathered row right?  One 5120 -> 17408 layer whose FULL trellis every rank draws
    # from the same seed: each rank runs its column shard through the exchange, rank 0 also runs the
    # unsharded layer on its own GPU and compares the two rows (outside every timed region).
    tp_check = None
    if dist is not None:
        cg = torch.Generator(device=dev)
        cg.manual_seed(4242)
        inf, outf = SHAPES[0]
        full = torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * K_BITS), dtype=torch.int16, device=dev,
                             generator=cg)
        c_suh = (torch.randint(0, 2, (inf,), device=dev, generator=cg) * 2 - 1).to(torch.float16)
        c_svh = (torch.randint(0, 2, (outf,), device=dev, generator=cg) * 2 - 1).to(torch.float16)
        c_x = torch.randn((ROWS, inf), device=dev, generator=cg).to(torch.float16)
        c0, c1 = shard_cols(outf, world, rank)
        shard = full[:, c0 // 16:c1 // 16].contiguous()
        with torch.cuda.stream(stream):
            if peer is not None:
                peer.restart()
                got = ops.gemv_peers(c_x, shard, K_BITS, CB, c_suh, c_svh[c0:c1].contiguous(), None, exchange=peer,
                                     out_features_total=outf, col0=c0, pdl=False).clone()
            else:
                yl = ops.gemv(c_x, shard, K_BITS, CB, c_suh, c_svh[c0:c1].contiguous(), None)
                got = all_gather_columns(yl, outf)
            want = ops.gemv(c_x, full, K_BITS, CB, c_suh, c_svh, None)
            stream.synchronize()
        rel = float((got.float() - want.float()).norm() / want.float().norm())
        t = torch.tensor([rel], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # every rank holds a gathered row: the worst one counts
        tp_check = {"max_rel": float(t.item()), "ok": bool(float(t.item()) <= 1e-3),
                    "what": "5120x17408 layer, gathered row of every rank vs the unsharded layer on the same GPU"}
        del full, shard

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import exl3_oracle as oracle

        oracle.lib()
        cores = oracle.host_cores()
        oracle.set_threads(cores)
        cl, cx = make_cpu_layers(np, 1000)
        b, dt, passes = 0, 0.0, 0
        while dt < 10.0:
            pb, pt = cpu_pass(oracle, np, cl, cx, 25.0)
            b, dt, passes = b + pb, dt + pt, passes + 1
        cpu = {"value": b / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{passes} passes over one layer set ({len(SHAPES)} layer(s), {b / passes / 1e6:.1f} MB packed "
                         f"each) through the C oracle with OpenMP, {dt:.1f} s"}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        n_gemv = len(layers)
        value = step_bytes_global * args.steps / (ms * 1e-3) / 1e9
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "rows": ROWS, "k": K_BITS, "codebook": "3INST", "ring_sets": args.ring,
                "accumulate": "fast" if args.fast_accum else "exact",
                "step_packed_bytes": step_bytes_global,
                "l2": f"inputs larger than L2: {step_bytes_global / world / 1e6:.0f} MB of distinct "
                      f"weights per GPU per step vs 126 MB L2",
                "launch": "cuda_graph" if graph is not None else "eager",
                "parallelism": (f"tp{world} by output tile, output rows completed over peer memory in the "
                                f"GEMV epilogue" if peer is not None else
                                f"tp{world} by output tile + NCCL all-gather") if world > 1 else "single GPU",
            },
            "roofline": {
                "bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                "frac": per_gpu / peak, "traffic": DRAM_TRAFFIC_RATIO * step_bytes_global / world / n_gemv,
                "traffic_unit": "bytes per launch (dram read + write)",
                "traffic_note": "ncu capture of the 5120x17408 launch: 44.69 MB read + 2.6-8.4 KB written for "
                                "44.56 MB of packed weights (ratio 1.0028); scaled by packed bytes to the "
                                "average launch of this step",
                "peak_kind": f"of {peak_kind}",
                "kernel": "exl3::gemv_kernel<4,0,1,0,1>",
                "note": "achieved = packed bytes per launch / (step time / GEMV launches); both "
                        "rotations run inside the GEMV kernel",
                "avg_launch_us": 1e3 * ms / args.steps / n_gemv,
            },
            "cpu_baseline": cpu,
            "e2e": {"value": step_bytes_global / e2e_s / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1e3 * e2e_s, "api": e2e_api},
            # one fused kernel per layer (rotation inside); over peer memory one wait kernel per step
            "gpu_launches": (n_gemv + (1 if peer is not None else 0)) * args.steps,
            "clocks": clocks,
            "kernel_status": status,
        }
        if tp_check is not None:
            line["tp_check"] = tp_check
        emit(line)
    if dist is not None:
        graph = None          # the captured NCCL kernels go before the communicator does
        e2e_graph = None
        finish_ranks(dist)
        if tp_check is not None and not tp_check["ok"]:
            raise SystemExit(f"tensor-parallel result differs from the unsharded layer: {tp_check}")


def run_decode(args):
    """The dense-transformer decode configuration: one greedy decode step of the synthetic 64-layer dense model
    (all linears EXL3, K in {4,5}, KV context 8192) at --rows new positions, tensor parallel by
    output tile over the launched ranks.  A step = one forward + arg-max, captured in a CUDA
    graph; value = rows / step time."""
    import numpy as np
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    from ponyexl3_b200 import ops
    from ponyexl3_b200.dense_step import DenseConfig, SyntheticDenseDecoder

    cfg = DenseConfig(layers=args.layers, max_rows=max(16, args.rows))
    dec = SyntheticDenseDecoder(cfg, dev, seed=5000, peer_exchange=not args.nccl_gather)
    rows = args.rows
    tok_in = torch.randint(0, cfg.vocab, (rows,), device=dev, generator=torch.Generator(device=dev).manual_seed(5))
    stream = torch.cuda.Stream(device=dev)
    graph = None
    with torch.cuda.stream(stream):
        tok_out = dec.step(tok_in)
        stream.synchronize()
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                tok_out = dec.step(tok_in)

    def run_step():
        if graph is not None:
            graph.replay()
            return tok_out
        return dec.step(tok_in)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run_step()
        barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        # end to end: token ids come from pinned host memory, the chosen tokens go back to it
        h_tok = tok_in.cpu().pin_memory()
        h_out = torch.empty((rows,), dtype=torch.int64).pin_memory()
        e2e_steps = max(3, min(args.steps, 20))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            tok_in.copy_(h_tok, non_blocking=True)
            out = run_step()
            h_out.copy_(out, non_blocking=True)
            stream.synchronize()
            h_tok.copy_(h_out % cfg.vocab)
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0].item()), float(t[1].item())
    status = ops.Workspace.get(dev, 1, 128).status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import exl3_oracle as oracle
        oracle.lib()
        cores = oracle.host_cores()
        oracle.set_threads(cores)
        rng = np.random.default_rng(5000)
        d, i = cfg.hidden, cfg.intermediate
        slots = [(d, (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim), (d, d), (d, 2 * i), (i, d)]
        t_layer = 0.0
        for (inf, outf) in slots:
            tr = rng.integers(0, 65536, size=(inf // 16, outf // 16, 64), dtype=np.uint16)
            sg = np.ones(inf, dtype=np.float16)
            sv = np.ones(outf, dtype=np.float16)
            x = rng.standard_normal((rows, inf)).astype(np.float16)
            t0 = time.perf_counter()
            oracle.linear_forward(x, tr, 4, 0, sg, sv)
            t_layer += time.perf_counter() - t0
        weights_layer = sum(a * b for a, b in slots)
        est = t_layer * (cfg.layers * weights_layer + d * cfg.vocab) / weights_layer
        cpu = {"value": rows / est, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": f"the four linear slots of ONE layer at K=4 through the C oracle ({t_layer:.2f} s), "
                         f"scaled by weight count to {cfg.layers} layers + head; attention and norms not "
                         f"included (they favour the CPU figure)"}
    if rank == 0:
        peak, peak_kind = measured_peaks()
        step_s = ms * 1e-3 / args.steps
        bytes_gpu = dec.packed_local + dec.kv_bytes_local
        line = {
            "metric": "decode_tokens_per_s", "value": rows / step_s, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * step_s,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": f"configs[4]: greedy decode step, {cfg.layers} layers, hidden {cfg.hidden}, "
                            f"MLP {cfg.intermediate}, {cfg.q_heads}q/{cfg.kv_heads}kv heads x {cfg.head_dim}, "
                            f"vocab {cfg.vocab}, KV context {cfg.context}, rows {rows}",
                "rows": rows, "bits": "K in {4,5}, mean %.3f bpw" % (sum(dec.ks) / len(dec.ks)),
                "packed_bytes_per_gpu": dec.packed_local, "kv_bytes_per_gpu": dec.kv_bytes_local,
                "l2": "weights + KV per GPU per step far larger than the 126 MB L2",
                "launch": "cuda_graph" if graph is not None else "eager",
                "parallelism": (f"tp{world} by output tile, heads sharded, 4 exchanges per layer over "
                                + ("peer memory" if dec.peer is not None else "NCCL all-gather"))
                               if world > 1 else "single GPU",
                "glue": "residual+RMSNorm, rotary+cache append, split-context GQA attention, SwiGLU: library "
                        "kernels; embedding gather and arg-max: PyTorch",
            },
            "roofline": {"bound": "hbm", "achieved": bytes_gpu / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": bytes_gpu / step_s / 1e9 / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "note": "whole step: packed weights + KV cache bytes per GPU over the step time"},
            "cpu_baseline": cpu,
            "e2e": {"value": rows / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8 * rows,
                    "d2h_bytes_per_step": 8 * rows, "ms_per_step": 1e3 * e2e_s,
                    "api": "SyntheticDenseDecoder.step, token ids from and to pinned host memory"},
            # per layer: 2 norms, 4 GEMVs (rotations inside for up to 8 rows, else 4 rotation kernels),
            # rotary, 2 attention, SwiGLU (+ 2 copies and 4 waits with the peer exchange); then the
            # final norm and the head
            "gpu_launches": (cfg.layers * (10 + (4 if rows > 8 else 0) + (6 if dec.peer is not None else 0)) + 2
                             + (1 if rows > 8 else 0)) * args.steps,
            "clocks": clocks, "kernel_status": status,
        }
        emit(line)
    if dist is not None:
        graph = None          # the captured NCCL kernels go before the communicator does
        finish_ranks(dist)


def run_gemm(args):
    """The prefill configuration: M = 8192 tokens x 5120 -> 5120 at K = 4, 3INST, bf16 activations
    N(0,1).  A step = one prefill call (input rotation kernel + tcgen05 GEMM) on the next layer of a
    ring of distinct layers; x (84 MB), the rotated copy (84 MB) and y (84 MB) of one call are
    already larger than the 126 MB L2.  value = 2*M*in*out FLOP / step time."""
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the product path)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    from ponyexl3_b200 import ops
    from ponyexl3_b200.linear import EXL3Linear

    M, inf, outf, k, cb = args.gemm_rows, 5120, 5120, 4, 0
    g = torch.Generator(device=dev).manual_seed(3000)
    ring = max(2, args.ring // 2)
    trs = [torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * k), dtype=torch.int16, device=dev, generator=g)
           for _ in range(ring)]
    suh = (torch.randint(0, 2, (inf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (outf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    x = torch.randn((M, inf), device=dev, generator=g).to(torch.bfloat16)
    y = torch.empty((M, outf), dtype=torch.float16, device=dev)
    flops = 2.0 * M * inf * outf
    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream(dev))

    def timed(fn, steps, warm):
        with torch.cuda.stream(stream):
            for i in range(warm):
                fn(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            e0.record(stream)
            for i in range(steps):
                fn(i)
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) / steps

    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(lambda i: ops.gemm(x, trs[i % ring], k, cb, suh, svh, None, out=y), args.steps, max(args.warmup, 3))
    # keep the load up for the sampler
    timed(lambda i: ops.gemm(x, trs[i % ring], k, cb, suh, svh, None, out=y), max(args.steps, int(250 / max(ms, 1e-3))), 0)
    clocks = sampler.stop()
    # the rotation kernel alone (same kernel, same x, fp16 output): its share of a call
    rot_ms = timed(lambda i: ops.had_r_128(x, pre_scale=suh), args.steps, 3)
    status = ops.Workspace.get(dev, 1, 128).status()

    # end to end through the module with pinned host buffers
    mod = EXL3Linear.from_device_tensors(trellis=trs[0], k=k, cb=cb, suh=suh, svh=svh, key="bench")
    h_x = x.cpu().pin_memory()
    h_y = torch.empty((M, outf), dtype=torch.float16).pin_memory()
    d_x = torch.empty_like(x)

    def e2e_step():
        d_x.copy_(h_x, non_blocking=True)
        h_y.copy_(mod(d_x), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        e2e_step()
    n_e2e = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = (time.perf_counter() - t0) / n_e2e

    cpu = None
    if not args.no_cpu:
        from oracle import exl3_oracle as oracle
        oracle.lib()
        cores = oracle.host_cores()
        oracle.set_threads(cores)
        rows_s = 256
        xs_np = x[:rows_s].float().cpu().numpy().astype(np.float16)
        tr_np = trs[0].cpu().numpy().view(np.uint16)
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < 10.0:
            oracle.linear_forward(xs_np, tr_np, k, cb, suh.cpu().numpy(), svh.cpu().numpy())
            n += 1
        dt = time.perf_counter() - t0
        cpu = {"value": 2.0 * rows_s * inf * outf * n / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"{n} forwards of {rows_s} of the {M} rows (decode of the whole layer each time) through "
                         f"the C oracle with OpenMP, {dt:.1f} s"}
    line = {
        "metric": "exl3_prefill_gemm_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"configs[2]: prefill GEMM, M={M} tokens x {inf}->{outf}, K={k}, 3INST, bf16 "
                               f"activations", "rows": M, "k": k, "codebook": "3INST", "ring_layers": ring,
                   "flops": flops, "l2": "x, its rotated copy and y of one call (3 x 84 MB) exceed the 126 MB L2; "
                                         "weights rotate over a ring of layers",
                   "operands": "fp16 x fp16 -> fp32 (decoded weights are exact in fp16; the reference rounds "
                               "the rotated activations to fp16)"},
        "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": 1657.8, "unit": "TFLOP/s",
                     "frac": flops / (ms * 1e-3) / 1e12 / 1657.8, "traffic": None,
                     "peak_kind": "of measured (burst bf16 GEMM); sustained 1408.3",
                     "frac_of_sustained": flops / (ms * 1e-3) / 1e12 / 1408.3,
                     "kernel": "exl3::gemm_kernel (tcgen05) + exl3::hadamard_mma_kernel",
                     "rotation_ms": rot_ms, "gemm_kernel_ms_est": ms - rot_ms,
                     "gemm_kernel_tflops_est": flops / ((ms - rot_ms) * 1e-3) / 1e12,
                     "note": "achieved = FLOPs of the call / time of the call (rotation kernel included); the "
                             "rotation kernel timed alone on the same x gives the split"},
        "cpu_baseline": cpu,
        "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * inf * 2,
                "d2h_bytes_per_step": M * outf * 2, "ms_per_step": 1e3 * e2e_s,
                "api": "EXL3Linear.forward, pinned host x (bf16) and y"},
        "gpu_launches": 2 * args.steps, "clocks": clocks, "kernel_status": status,
    }
    emit(line)


def run_encode(args):
    """The converter's tile search: exact Viterbi encoding of 16x16 tiles of N(0,1) weights at K = 4,
    3INST (one whole wave of tiles per SM and then some).  A step = one exl3_encode_tiles call over
    592 tiles; value = tiles per second.  The float64 costs of the 148 tiles in flight (1 MiB each)
    exceed the L2, so the search streams them through DRAM every step: the roofline line reports that
    traffic against the HBM peak.  The CPU baseline is the C oracle's search on all host cores."""
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the product path)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    from ponyexl3_b200 import ops

    n, k, cb = 592, 4, 0
    g = torch.Generator(device=dev).manual_seed(5000)
    w = torch.randn((n, 256), device=dev, generator=g)
    for _ in range(max(args.warmup, 3)):
        ops.quantize_tiles(w, k, cb)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = max(1, min(args.steps, 20))
    e0.record()
    for _ in range(steps):
        states, packed = ops.quantize_tiles(w, k, cb)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    clocks = sampler.stop()
    # end to end: weights from pinned host memory, packed tiles back
    h_w = w.cpu().pin_memory()
    h_p = torch.empty((n, 16 * k), dtype=torch.int16).pin_memory()
    d_w = torch.empty_like(w)
    t0 = time.perf_counter()
    for _ in range(3):
        d_w.copy_(h_w, non_blocking=True)
        h_p.copy_(ops.quantize_tiles(d_w, k, cb)[1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_s = (time.perf_counter() - t0) / 3
    cpu = None
    if not args.no_cpu:
        from oracle import exl3_oracle as oracle
        oracle.lib()
        cores = oracle.host_cores()
        oracle.set_threads(cores)
        wn = w.cpu().numpy()
        t0 = time.perf_counter()
        m = 0
        while time.perf_counter() - t0 < 10.0 and m < n:
            st, _ = oracle.quantize_tile(wn[m], k, cb)
            assert (st == states[m].cpu().numpy().view(np.uint16)).all(), "encoder differs from the oracle"
            m += 1
        dt = time.perf_counter() - t0
        cpu = {"value": m / dt, "unit": "tiles/s", "cores": cores, "kind": "port",
               "sample": f"the first {m} of the {n} tiles through the C oracle's search (each checked against the GPU's "
                         f"states), {dt:.1f} s"}
    # per pass and step: 65,536 float64 costs read and written, 4,096 back-pointer bytes
    step_bytes = 2 * 65536 * 8 + (65536 >> k)
    emit({
        "metric": "exl3_trellis_encode_tiles_per_s", "value": n / (ms * 1e-3), "unit": "tiles/s", "n_gpus": 1,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"trellis encoder: exact Viterbi search of {n} tiles (16x16, N(0,1)), K={k}, 3INST, "
                               "up to 4 pinned passes", "tiles": n, "k": k, "codebook": "3INST",
                   "l2": "the cost arrays of the 148 tiles in flight (148 MiB) exceed the 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": n * 256 * step_bytes / (ms * 1e-3) / 1e9, "peak": 6551.4,
                     "unit": "GB/s", "frac": n * 256 * step_bytes / (ms * 1e-3) / 1e9 / 6551.4,
                     "traffic": ENCODE_DRAM_BYTES_PER_TILE * n,
                     "traffic_unit": "bytes per launch (dram read + write)",
                     "traffic_note": "ncu capture of this launch: 97.1 GB read + 159.1 GB written for 592 tiles; the "
                                     "cost arrays of the 148 tiles in flight (148 MiB) do not fit the 126 MB L2, so "
                                     "every step's costs go through DRAM",
                     "peak_kind": "of measured",
                     "kernel": "exl3::encode_kernel",
                     "note": "achieved counts ONE pass per tile (costs read and written, back-pointers written, "
                             "per step); tiles take 1-5 passes, which is why the DRAM traffic is higher"},
        "cpu_baseline": cpu,
        "e2e": {"value": n / e2e_s, "unit": "tiles/s", "h2d_bytes_per_step": n * 256 * 4,
                "d2h_bytes_per_step": n * 16 * k * 2, "ms_per_step": 1e3 * e2e_s,
                "api": "ops.quantize_tiles, pinned host weights in, packed tiles out"},
        "gpu_launches": steps, "clocks": clocks, "kernel_status": 0,
    })


def run_moe(args):
    """The MoE expert-layer configuration: stacked-expert SwitchGLU, 256 experts, top-8, hidden 2048, expert
    intermediate 512, K=4, router logits N(0,1) -> softmax top-8, for --tokens 1, 16 or 4096.
    N > 1: experts partitioned by expert; few tokens are replicated and the partial outputs summed
    (all-reduce), many tokens are partitioned, gathered, and every output row is stored into the memory
    of the rank that owns its token.
    A step = one SwitchGLU forward (expert outputs before the router-weighted sum)."""
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    from ponyexl3_b200 import ops
    from ponyexl3_b200.moe import EXL3SwitchGLU, route_topk
    from ponyexl3_b200.parallel import EPSwitchGLU, shard_expert_weights

    E, D, H, kk, k, T = 256, 2048, 512, 8, 4, args.tokens
    g = torch.Generator(device=dev)
    g.manual_seed(4000)                                   # the same experts and tokens on every rank
    ri = lambda *sh: torch.randint(-32768, 32767, sh, dtype=torch.int16, device=dev, generator=g)
    sg = lambda *sh: (torch.randint(0, 2, sh, device=dev, generator=g) * 2 - 1).to(torch.float16)
    w = dict(gu_trellis=ri(D // 16, E * 2 * H // 16, 16 * k), gu_suh=sg(E, 2, D), gu_svh=sg(E, 2 * H),
             dn_trellis=ri(H // 16, E * D // 16, 16 * k), dn_suh=sg(E, H), dn_svh=sg(E, D))
    x = (torch.randn((T, D), device=dev, generator=g) * 0.02).to(torch.float16)
    inds, _ = route_topk(torch.randn((1, T, E), device=dev, generator=g), kk)
    inds = inds.reshape(T, kk)
    if world == 1:
        switch = EXL3SwitchGLU(**w, k=k, cb=0)
        step = lambda: switch(x.view(1, T, D), inds.view(1, T, kk))
        mode = "single GPU"
    else:
        local_sw = EXL3SwitchGLU(**shard_expert_weights(w, E, world, rank), k=k, cb=0)
        del w
        if T <= 16:
            ep = EPSwitchGLU(local_sw, E)
            step = lambda: ep(x.view(1, T, D), inds.view(1, T, kk))
            mode = f"ep{world}: tokens replicated, pairs picked on the device, all-reduce of partial outputs, one CUDA graph"
        else:
            if T % world:
                raise SystemExit("--tokens must be a multiple of the number of GPUs")
            t0, t1 = T * rank // world, T * (rank + 1) // world
            xl, il = x[t0:t1].contiguous(), inds[t0:t1].contiguous()
            ep = EPSwitchGLU(local_sw, E)
            step = lambda: ep.forward_partitioned(xl, il)
            mode = (f"ep{world}: tokens partitioned; all-gather of tokens and routing, every rank computes the pairs of "
                    "its experts (picked on the device) and stores the outputs into the owners' memory over NVLink; "
                    "two CUDA graphs replayed in turn")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        # No host round trip anywhere: the call is captured, the collectives included.  Expert
        # parallelism over many tokens rotates its exchange buffers per call, so two graphs (two
        # consecutive calls) are captured and replayed in turn.
        graphs = []
        if not args.no_graph:
            for _ in range(2 if (world > 1 and T > 16) else 1):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=stream):
                    step()
                graphs.append(gr)
        turn = [0]

        def run():
            if not graphs:
                return step()
            graphs[turn[0] % len(graphs)].replay()
            turn[0] += 1
        for _ in range(3):
            run()
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = ops.Workspace.get(dev, 1, 128).status()

    # end to end (1 GPU): tokens and routing come from pinned host memory, the expert outputs go back
    e2e = None
    if world == 1:
        h_x, h_i = x.cpu().pin_memory(), inds.cpu().pin_memory()
        h_y = torch.empty((T, kk, D), dtype=torch.float16).pin_memory()
        d_x, d_i = torch.empty_like(x), torch.empty_like(inds)

        def e2e_step():
            d_x.copy_(h_x, non_blocking=True)
            d_i.copy_(h_i, non_blocking=True)
            h_y.copy_(switch(d_x.view(1, T, D), d_i.view(1, T, kk)).view(T, kk, D), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(2):
            e2e_step()
        n_e2e = max(3, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        e2e_s = (time.perf_counter() - t0) / n_e2e
        e2e = {"ms_per_step": 1e3 * e2e_s, "h2d_bytes_per_step": h_x.numel() * 2 + h_i.numel() * h_i.element_size(),
               "d2h_bytes_per_step": h_y.numel() * 2, "api": "EXL3SwitchGLU.__call__, pinned host x, indices and y"}

    # CPU baseline: the oracle's SwitchGLU on a bounded sample of (token, slot) pairs
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import numpy as np
        from oracle import exl3_oracle as oracle
        oracle.lib()
        cores = oracle.host_cores()
        oracle.set_threads(cores)
        wn = {n: (t.cpu().numpy().view(np.uint16) if t.dtype == torch.int16 else t.cpu().numpy()) for n, t in w.items()}
        n_pairs = min(T * kk, 64)
        toks = np.arange(n_pairs) // kk if T * kk <= 64 else np.arange(n_pairs) * (T // n_pairs)
        slots = np.arange(n_pairs) % kk
        xi = x.cpu().numpy()[toks]
        ii = inds.cpu().numpy()[toks, slots][:, None]
        t0 = time.perf_counter()
        oracle.switch_glu(xi, ii, **wn, k=k, cb=0)
        dt = time.perf_counter() - t0
        cpu = {"pairs": int(n_pairs), "seconds": dt, "cores": cores, "kind": "port",
               "sample": f"{n_pairs} (token, slot) pairs of the same call through the C oracle "
                         f"(decode of each distinct expert once, then three forwards per pair), {dt:.1f} s"}
    if rank == 0:
        touched = int(torch.unique(inds).numel())
        packed = touched * 3 * D * H * k // 8
        flops = 2.0 * T * kk * 3 * D * H
        hbm_peak, kind = measured_peaks()
        few = T <= 16
        line = {
            "metric": "moe_expert_weight_bandwidth" if few else "moe_expert_tflops",
            "value": packed / (ms * 1e-3) / 1e9 if few else flops / (ms * 1e-3) / 1e12,
            "unit": "GB/s" if few else "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"configs[3]: SwitchGLU, {E} experts, top-{kk}, hidden {D}, intermediate {H}, "
                                   f"K={k}, {T} tokens", "tokens": T, "experts_touched": touched,
                       "packed_bytes_touched": packed, "flops": flops, "parallelism": mode,
                       "launch": "cuda_graph" if graphs else "eager"},
            "roofline": ({"bound": "hbm", "achieved": packed / (ms * 1e-3) / 1e9 / world, "peak": hbm_peak,
                          "unit": "GB/s", "frac": packed / (ms * 1e-3) / 1e9 / world / hbm_peak, "traffic": None,
                          "peak_kind": f"of {kind}"} if few else
                         {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12 / world, "peak": 1657.8,
                          "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / world / 1657.8, "traffic": None,
                          "peak_kind": "of measured (burst)"}),
            "cpu_baseline": None, "e2e": None, "clocks": clocks, "kernel_status": status,
            "gpu_launches": 5 * args.steps if world == 1 else None,
        }
        unit_work = packed if few else flops        # what `value` counts per step
        scale = 1e9 if few else 1e12
        if e2e is not None:
            e2e.update(value=unit_work / (e2e["ms_per_step"] * 1e-3) / scale, unit=line["unit"])
            line["e2e"] = e2e
        if cpu is not None:
            # the sample's share of the step's work, over its time
            share = cpu["pairs"] / float(T * kk)
            cpu.update(value=unit_work * share / cpu["seconds"] / scale, unit=line["unit"])
            line["cpu_baseline"] = cpu
        emit(line)
    if dist is not None:
        graph = None
        finish_ranks(dist)


def run_sweep(args):
    """The GEMV sweep configuration in full: rows x K x codebook x shape, one graph-captured train
    of launches over distinct layers (more packed bytes than L2) per case.  Prints one JSON
    line per case and, with --sweep-out, writes a markdown table."""
    import torch
    from ponyexl3_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peak, peak_kind = measured_peaks()
    gen = torch.Generator(device=dev)
    gen.manual_seed(2000)
    rows_list = [int(r) for r in args.sweep_rows.split(",")]
    ks = [int(k) for k in args.sweep_k.split(",")]
    cbs = [int(c) for c in args.sweep_cb.split(",")]
    stream = torch.cuda.Stream(device=dev)
    results = []
    for (inf, outf) in SHAPES:
        suh = (torch.randint(0, 2, (inf,), device=dev, generator=gen) * 2 - 1).to(torch.float16)
        svh = (torch.randint(0, 2, (outf,), device=dev, generator=gen) * 2 - 1).to(torch.float16)
        for k in ks:
            per = inf * outf * k // 8
            n = max(3, min(96, int(2.5 * L2_BYTES // per) + 1))       # distinct layers per train
            trs = [torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * k), dtype=torch.int16,
                                 device=dev, generator=gen) for _ in range(n)]
            for rows in rows_list:
                x = torch.randn((rows, inf), device=dev, generator=gen).to(torch.float16)
                y = torch.empty((rows, outf), dtype=torch.float16, device=dev)
                stream.wait_stream(torch.cuda.current_stream(dev))     # inputs are written before use
                for cb in cbs:
                    with torch.cuda.stream(stream):
                        ops.gemv(x, trs[0], k, cb, suh, svh, None, pdl=True, out=y)
                        stream.synchronize()
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=stream):
                            for t in trs:
                                ops.gemv(x, t, k, cb, suh, svh, None, pdl=True, out=y)
                        for _ in range(3):
                            g.replay()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        stream.synchronize()
                        e0.record(stream)
                        for _ in range(args.sweep_iters):
                            g.replay()
                        e1.record(stream)
                        stream.synchronize()
                    status = ops.Workspace.get(dev, rows, inf).status()
                    if status:
                        raise SystemExit(f"kernel status {status} at {inf}x{outf} K={k} cb={cb} rows={rows}")
                    us = 1e3 * e0.elapsed_time(e1) / args.sweep_iters / n
                    gbs = per / (us * 1e-6) / 1e9
                    r = {"shape": f"{inf}x{outf}", "k": k, "cb": CB_NAMES[cb], "rows": rows,
                         "us_per_launch": round(us, 2), "packed_gbs": round(gbs, 1),
                         "frac_hbm": round(gbs / peak, 4), "gweights_s": round(inf * outf / us / 1e3, 1),
                         "other_bytes": 2 * rows * (inf + outf) + 2 * (inf + outf), "layers_in_train": n}
                    print(json.dumps(r), flush=True)
                    results.append(r)
                    del g
            del trs
            torch.cuda.empty_cache()
    if args.sweep_out:
        lines = [f"Peak: {peak:.1f} GB/s ({peak_kind}).  Cells: packed-weight GB/s (fraction of peak), "
                 f"3INST / MCG / MUL1.", ""]
        for (inf, outf) in SHAPES:
            lines += [f"### {inf} -> {outf}", "", "| K | " + " | ".join(f"rows={r}" for r in rows_list) + " |",
                      "|---|" + "---|" * len(rows_list)]
            for k in ks:
                cells = []
                for rows in rows_list:
                    v = [r for r in results if r["shape"] == f"{inf}x{outf}" and r["k"] == k and r["rows"] == rows]
                    cells.append(" / ".join(f"{r['packed_gbs']:.0f} ({r['frac_hbm']:.2f})" for r in v))
                lines.append(f"| {k} | " + " | ".join(cells) + " |")
            lines.append("")
        Path(args.sweep_out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.sweep_out).write_text("\n".join(lines))


def run_profile_case(case: str):
    """Small fixed cases for `ncu` captures (a few launches, a few GB at most on the device):
    gemv = four batch-1 GEMVs 5120->17408 K=4 on distinct layers; gemm = three prefill GEMMs
    8192 x 5120 -> 5120 K=4 with bf16 activations."""
    import torch
    from ponyexl3_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    if case == "gemv":
        inf, outf, rows, n = 5120, 17408, 1, 4
    else:
        inf, outf, rows, n = 5120, 5120, 8192, 1
    trs = [torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * K_BITS), dtype=torch.int16,
                         device=dev, generator=g) for _ in range(n)]
    suh = (torch.randint(0, 2, (inf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (outf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    x = torch.randn((rows, inf), device=dev, generator=g)
    x = x.to(torch.float16) if case == "gemv" else x.to(torch.bfloat16)
    for i in range(4 if case == "gemv" else 3):
        fn = ops.gemv if case == "gemv" else ops.gemm
        y = fn(x, trs[i % n], K_BITS, CB, suh, svh, None)
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": case, "mean_abs_y": float(y.float().abs().mean())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ring", type=int, default=16, help="layer sets per step")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: NCCL all-gather per layer instead of the peer-memory epilogue")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--fast-accum", action="store_true",
                    help="gemv workload, 1 GPU: EXL3_FLAG_FAST_ACCUM (the two fp16 halves of a codebook value "
                         "are added inside the fp32 accumulation; outputs move by about 4e-4 relative)")
    ap.add_argument("--profile-case", choices=["gemv", "gemm"], default=None,
                    help="run one small case for an ncu capture and exit")
    ap.add_argument("--sweep", action="store_true",
                    help="rows x K x codebook x shape GEMV sweep (one JSON line per case) and exit")
    ap.add_argument("--sweep-rows", default="1,2,4,8,16")
    ap.add_argument("--sweep-k", default="1,2,3,4,5,6,7,8")
    ap.add_argument("--sweep-cb", default="0,1,2")
    ap.add_argument("--sweep-iters", type=int, default=5)
    ap.add_argument("--sweep-out", default=None, help="write a markdown table of the sweep here")
    ap.add_argument("--workload", choices=["gemv", "single", "gemm", "decode", "moe", "encode"], default="gemv",
                    help="gemv = the headline batch-1 GEMV ring; single = one 4096x4096 layer (ring of copies); "
                         "gemm = the 8192-token prefill GEMM; decode = the 64-layer decode step; "
                         "moe = the 256-expert SwitchGLU layer; encode = the converter's exact tile search")
    ap.add_argument("--gemm-rows", type=int, default=8192, help="gemm workload: tokens per call")
    ap.add_argument("--tokens", type=int, default=1, help="moe workload: tokens per step (1, 16, 4096)")
    ap.add_argument("--rows", type=int, default=1, help="decode workload: new positions per step (1 or 16)")
    ap.add_argument("--layers", type=int, default=64, help="decode workload: transformer layers")
    args = ap.parse_args()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        quiet_stdout()
    if args.sweep:
        run_sweep(args)
        return
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    if args.workload == "single":
        # the single-layer configuration: in = out = 4096, K = 4, 3INST, x [1, 4096]; 8 MiB of packed
        # weights per layer, so the ring holds 32 distinct layers (268 MB) to stay out of the L2
        global SHAPES, WORKLOAD
        SHAPES = [(4096, 4096)]
        WORKLOAD = "configs[0]: single layer, in=out=4096, K=4, 3INST, x [1,4096]"
        args.ring = max(args.ring, 32)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "gemm":
        run_gemm(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "encode":
        run_encode(args)
    elif args.workload == "moe":
        run_moe(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
