#!/usr/bin/env python3
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (all synthetic, seed 0, shapes and distributions of the reference's
benchmark configurations):
  prefill_gemm  BitLinear prefill, M=2048: up/gate [8640,3200] and down [3200,8640]
                projections (one step = both, 226.5 GOP); value in TOPS.
  decode_gemv   BitLinear decode, x fp32 [1,3200], W ternary [8640,3200]; one step =
                64 calls over 64 distinct weights (442 MB > L2); value in GB/s of
                algorithmic bytes (packed W + x + y per call).
  w4a16         W4A16, N=11008, K=4096, group 128, M in {1,16}; one step = 24 calls
                over 24 distinct weights (563 MB > L2); value in GB/s.
One JSON line is printed by rank 0.  With --gpus N > 1 (launched by torchrun) the
weights are column-sharded over the ranks, x is replicated and each output is
all-gathered with NCCL: total work is fixed ("strong" scaling).

--impl reference times the reference's CPU arithmetic for the same workload (the C
restatement under oracle/, all host threads) on a bounded sample and prints the same
line with "impl": "reference".
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode GEMV HBM GB/s & prefill TOPS (% roofline); BitNet-3B decode tok/s"
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    """Measured peaks of this pool (driver-written file), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # the busiest half of the samples: the idle ones before/after the region say nothing
        busy = sm[len(sm) // 2:] if sm else []
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- inputs
def ternary_packed(rng, n, k):
    import numpy as np
    trits = rng.integers(-1, 2, size=(n, k), dtype=np.int8)
    c = (trits + 1).astype(np.uint8).reshape(n, k // 4, 4)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).astype(np.uint8)


def device_ternary(torch, n, k, gen):
    """Packed ternary weight generated on the device: every 2-bit field uniform over {0,1,2}."""
    c = torch.randint(0, 3, (n, k // 4, 4), device="cuda", dtype=torch.uint8, generator=gen)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).contiguous()


# ----------------------------------------------------------------------------- workloads
class Workload:
    name = ""
    unit = ""
    dtype = ""

    def units_per_step(self):
        raise NotImplementedError


class DecodeGemv(Workload):
    """BitLinear decode GEMV (configs[0] shape), 64 distinct weights per step."""
    name, unit, dtype = "bitlinear_decode_gemv_m1_n8640_k3200", "GB/s", "int8xint2->int32"
    N, K, M, LAYERS = 8640, 3200, 1, 64

    def __init__(self, torch, ops, rank, world, streams=1):
        self.torch, self.ops, self.rank, self.world = torch, ops, rank, world
        self.streams = max(1, streams)
        self.side = [torch.cuda.Stream() for _ in range(self.streams)] if self.streams > 1 else []
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        r0, rows = ops.shard_rows(self.N, world, rank)
        self.rows = rows
        self.layers = []
        for _ in range(self.LAYERS):
            full = device_ternary(torch, self.N, self.K, gen)          # same on every rank (seed 0)
            self.layers.append(ops.BitLinear(full[r0:r0 + rows].contiguous(), 0.02))
            del full
        self.x = torch.randn(self.M, self.K, device="cuda", generator=gen)
        self.x_host = self.x.cpu().pin_memory()
        self.x_stage = torch.empty_like(self.x)
        self.y_local = torch.empty(self.M, rows, device="cuda")
        self.y_side = [torch.empty(self.M, rows, device="cuda") for _ in self.side]
        self.y_full = torch.empty(world, self.M, rows, device="cuda") if world > 1 else None
        self.y_host = torch.empty(self.M, self.N, dtype=torch.float32).pin_memory()
        self.ws = torch.empty(int(ops.lib().nslq_bitlinear_workspace_bytes(self.M, self.K)), dtype=torch.uint8,
                              device="cuda")
        self.qa = ops.act_quant_i8(self.x, plain=False, perm=True)
        self.bytes_per_call = self.N * self.K // 4 + self.M * self.K * 4 + self.M * self.N * 4
        self.launches_per_step = self.LAYERS          # M <= 4: quantisation is fused into the GEMV kernel
        self.h2d, self.d2h = self.M * self.K * 4, self.M * self.N * 4

    def units_per_step(self):
        return self.LAYERS * self.bytes_per_call / 1e9            # GB of algorithmic bytes (whole job)

    def one_call(self, layer, x):
        layer.forward(x, out=self.y_local, workspace=self.ws)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.y_full, self.y_local)

    def step(self):
        if self.streams > 1 and self.world == 1:
            # the calls are independent (same x, distinct weights): issue them round-robin on
            # several streams so that one call's weight stream overlaps another's tail
            cur = self.torch.cuda.current_stream()
            for st in self.side:
                st.wait_stream(cur)
            for i, layer in enumerate(self.layers):
                j = i % self.streams
                with self.torch.cuda.stream(self.side[j]):
                    layer.forward(self.x, out=self.y_side[j], workspace=self.ws)   # M <= 4: workspace unused
            for st in self.side:
                cur.wait_stream(st)
            return
        for layer in self.layers:
            self.one_call(layer, self.x)

    kernel_name = "ternary_gemv_fused_kernel"

    def kernel_only(self):
        if self.world == 1:
            return self.step()                        # the step is that kernel and nothing else
        for layer in self.layers:                     # the GEMV launches without the all-gather
            layer.forward(self.x, out=self.y_local, workspace=self.ws)

    def kernel_bytes(self):
        # per launch, this rank's shard: packed W + x (fp32) + y (fp32)
        return self.rows * self.K // 4 + self.M * self.K * 4 + self.M * self.rows * 4

    def e2e_step(self, i):
        layer = self.layers[i % self.LAYERS]
        self.x_stage.copy_(self.x_host, non_blocking=True)
        self.one_call(layer, self.x_stage)
        out = self.y_full if self.world > 1 else self.y_local
        self.y_host.view(-1)[:out.numel()].copy_(out.view(-1), non_blocking=True)

    e2e_units = property(lambda self: self.bytes_per_call / 1e9)

    def roofline(self, peaks, kernel_ms):
        ach = self.kernel_bytes() / (kernel_ms * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": self.kernel_name, "achieved": round(ach, 1), "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4), "traffic": None,
                "peak_source": peaks["source"] + " (burst copy)", "kernel_us": round(kernel_ms * 1e3, 3)}

    def cpu_baseline(self, threads, budget_s=12.0):
        import numpy as np
        from oracle import oracle as o
        rng = np.random.default_rng(0)
        packed = ternary_packed(rng, self.N, self.K)
        x = rng.standard_normal((self.M, self.K)).astype(np.float32)
        o.bitlinear_forward_packed(x, packed, self.N, 0.02, threads=threads)
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and n < 400:
            o.bitlinear_forward_packed(x, packed, self.N, 0.02, threads=threads)
            n += 1
        dt = (time.perf_counter() - t0) / n
        return {"value": round(self.bytes_per_call / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": "%d full [1,3200]x[8640,3200] calls, %.2f ms each" % (n, dt * 1e3)}, dt


class PrefillGemm(Workload):
    """BitLinear prefill GEMM (configs[1]): up/gate then down projection, M=2048."""
    name, unit, dtype = "bitlinear_prefill_gemm_m2048_up8640x3200_down3200x8640", "TOPS", "int8xint2->int32"
    M, H, F = 2048, 3200, 8640

    def __init__(self, torch, ops, rank, world):
        self.torch, self.ops, self.rank, self.world = torch, ops, rank, world
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        self.shapes = [(self.F, self.H), (self.H, self.F)]      # (N, K) up/gate, down
        self.layers, self.xs, self.ys, self.ygs, self.qas, self.xh, self.xst = [], [], [], [], [], [], []
        for n, k in self.shapes:
            r0, rows = ops.shard_rows(n, world, rank)
            full = device_ternary(torch, n, k, gen)
            self.layers.append(ops.BitLinear(full[r0:r0 + rows].contiguous(), 0.02))
            x = torch.randn(self.M, k, device="cuda", generator=gen)
            self.xs.append(x)
            self.xh.append(x.cpu().pin_memory())
            self.xst.append(torch.empty_like(x))
            self.ys.append(torch.empty(self.M, rows, device="cuda"))
            self.ygs.append(torch.empty(world, self.M, rows, device="cuda") if world > 1 else None)
            self.qas.append(ops.act_quant_i8(x, plain=False, perm=True))
        self.ws = torch.empty(int(ops.lib().nslq_bitlinear_workspace_bytes(self.M, self.F)), dtype=torch.uint8,
                              device="cuda")
        self.y_host = torch.empty(self.M * self.F, dtype=torch.float32).pin_memory()
        self.ops_per_proj = 2 * self.M * self.H * self.F
        self.launches_per_step = 4
        self.h2d = self.M * (self.H + self.F) * 4
        self.d2h = self.M * (self.H + self.F) * 4
        # L2 flush buffer: written between timed steps is not needed (the two projections
        # stream 26+71 MB of x, 14 MB of W and 97 MB of y per step, > L2 in total)

    def units_per_step(self):
        return 2 * self.ops_per_proj / 1e12                       # tera-ops per step (whole job)

    def one_call(self, i, x):
        self.layers[i].forward(x, out=self.ys[i], workspace=self.ws)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(self.ygs[i], self.ys[i])

    def step(self):
        for i in range(2):
            self.one_call(i, self.xs[i])

    def kernel_only(self):
        for i in range(2):
            self.layers[i].forward_quantized(self.qas[i], out=self.ys[i])

    kernel_name = "ternary_gemm_kernel"

    def e2e_step(self, it):
        for i in range(2):
            self.xst[i].copy_(self.xh[i], non_blocking=True)
            self.one_call(i, self.xst[i])
            out = self.ygs[i] if self.world > 1 else self.ys[i]
            self.y_host[:out.numel()].copy_(out.view(-1), non_blocking=True)

    e2e_units = property(lambda self: 2 * self.ops_per_proj / 1e12)

    def roofline(self, peaks, kernel_ms):
        # kernel_ms = average duration of one GEMM launch (two launches per kernel_only pass)
        ops_launch = self.ops_per_proj / self.world
        ach = ops_launch / (kernel_ms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        return {"bound": "tensor", "kernel": self.kernel_name, "achieved": round(ach, 1), "peak": round(peak, 1),
                "unit": "TOPS", "frac": round(ach / peak, 4), "traffic": None,
                "peak_source": "2 x %s bf16 burst (no int8 figure is measured on this pool; datasheet int8 dense = 4500)"
                               % peaks["source"], "kernel_us": round(kernel_ms * 1e3, 2)}

    def cpu_baseline(self, threads, budget_s=15.0):
        import numpy as np
        from oracle import oracle as o
        rng = np.random.default_rng(0)
        rows = 16
        dt_tot = 0.0
        for n, k in self.shapes:
            packed = ternary_packed(rng, n, k)
            x = rng.standard_normal((rows, k)).astype(np.float32)
            t0, reps = time.perf_counter(), 0
            while True:
                o.bitlinear_forward_packed(x, packed, n, 0.02, threads=threads)
                reps += 1
                if time.perf_counter() - t0 > budget_s / 2 or reps >= 50:
                    break
            dt_tot += (time.perf_counter() - t0) / reps * (self.M / rows)
        return {"value": round(2 * self.ops_per_proj / dt_tot / 1e12, 6), "unit": "TOPS", "cores": threads,
                "kind": "port", "sample": "16 of 2048 token rows per projection, extrapolated linearly "
                                          "(%.1f s per full step)" % dt_tot}, dt_tot


WORKLOADS = {"decode_gemv": DecodeGemv, "prefill_gemm": PrefillGemm}
DEFAULT_WORKLOAD = "decode_gemv"


# ----------------------------------------------------------------------------- timing
def timed(torch, fn, iters, dist=None):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def capture(torch, fn):
    """Captures fn() into a CUDA graph (launch-bound inner loops are replayed, not re-issued)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from nsl_b200 import lib, ops
    if args.no_pdl:
        lib().nslq_set_dependent_launch(0)
    peaks = load_peaks()
    if args.workload == "decode_gemv":
        wl = DecodeGemv(torch, ops, rank, world, streams=args.streams)
    else:
        wl = WORKLOADS[args.workload](torch, ops, rank, world)

    use_graph = world == 1 and not args.no_graph
    step = wl.step
    graph = None
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if use_graph:
        graph = capture(torch, step)
        for _ in range(2):
            graph.replay()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ms = timed(torch, (lambda i: graph.replay()) if graph else (lambda i: step()), args.steps, dist)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = wl.units_per_step() / (ms_per_step * 1e-3)

    # dominant kernel alone (pre-quantised activations), same buffers, live CUDA-event timing
    kgraph = capture(torch, wl.kernel_only) if use_graph else None
    n_launch = len(wl.layers)
    reps = max(args.steps, 5)
    for _ in range(3):
        kgraph.replay() if kgraph else wl.kernel_only()
    kms = timed(torch, (lambda i: kgraph.replay()) if kgraph else (lambda i: wl.kernel_only()), reps, dist)
    kernel_ms = kms / reps / n_launch
    roof = wl.roofline(peaks, kernel_ms)

    # end to end through the host-facing call: pinned host input -> device -> op -> host result
    for i in range(3):
        wl.e2e_step(i)
    e2e_iters = max(args.steps, 10)
    ems = timed(torch, wl.e2e_step, e2e_iters, dist)
    e2e_val = wl.e2e_units / (ems / e2e_iters * 1e-3)

    if rank == 0:
        cpu, _ = wl.cpu_baseline(1)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seed 0)",
            "config": {"workload": wl.name, "cuda_graph": bool(graph), "dependent_launch": not args.no_pdl, "streams": getattr(wl, "streams", 1), "l2": "inputs larger than L2 per step",
                       "parallelism": "column-sharded x%d + NCCL all-gather" % world if world > 1 else "single GPU"},
            "e2e": {"value": round(e2e_val, 3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d,
                    "d2h_bytes_per_step": wl.d2h},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof, "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU arithmetic for the same workload, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as o
    o.build()
    threads = o.max_threads()

    class _NoGpu:
        pass

    cls = WORKLOADS[args.workload]
    wl = cls.__new__(cls)
    if isinstance(wl, DecodeGemv):
        wl.bytes_per_call = wl.N * wl.K // 4 + wl.M * wl.K * 4 + wl.M * wl.N * 4
    else:
        wl.shapes = [(wl.F, wl.H), (wl.H, wl.F)]
        wl.ops_per_proj = 2 * wl.M * wl.H * wl.F
    vals, per = [], []
    total = max(args.warmup, 0) + args.steps
    budget = min(8.0, 150.0 / max(total, 1))
    for i in range(total):
        cpu, dt = wl.cpu_baseline(threads, budget_s=budget)
        if i >= args.warmup:
            vals.append(cpu["value"])
            per.append(dt)
    v = sum(vals) / len(vals)
    cpu["value"] = round(v, 6)
    line = {"impl": "reference", "metric": METRIC, "value": round(v, 6), "unit": cls.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sum(per) / len(per) * 1e3, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": cls.dtype,
            "data": "synthetic (seed 0)", "config": {"workload": cls.name, "host_threads": threads},
            "cpu_baseline": cpu,
            "e2e": {"value": round(v, 6), "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true", help="issue launches directly instead of replaying a CUDA graph")
    ap.add_argument("--streams", type=int, default=1,
                    help="decode_gemv: issue the independent calls of a step round-robin on this many streams")
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels without the programmatic-dependent-launch attribute")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
