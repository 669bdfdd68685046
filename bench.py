#!/usr/bin/env python3
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (all synthetic, seed 0, shapes and distributions of the reference's benchmark
configurations):
  prefill_gemm  (default) BitLinear prefill, M=2048: up/gate [8640,3200] and down [3200,8640]
                projections (one step = both, 226.5 GOP); value in TOPS.  The two projections are
                independent calls and are issued on two streams (--streams 1: on one), so the second
                one's CTAs fill the SMs that the first one's last round of tiles leaves idle.
  decode_gemv   BitLinear decode, x fp32 [1,3200], W ternary [8640,3200]; one step = 64 calls
                over 64 distinct weights (442 MB > L2); value in GB/s of algorithmic bytes
                (packed W + x + y per call).  --streams S issues the (independent) calls
                round-robin on S streams.
  w4a16_m1 / w4a16_m16 / w4a16_m256
                W4A16, N=11008, K=4096, group 128; one step = 24 (M=1,16) or 8 (M=256) calls over
                distinct weights (> L2); GB/s for M=1,16, TFLOPS for M=256.
  bitnet3b_b1 / _b8 / _b64
                BitNet b1.58-3B-shaped decoder (26 layers, hidden 3200, FFN 8640, vocab 32002), random
                ternary weights, 512-token prompt, 256 greedy decode steps in one CUDA graph; every
                projection (and, per decode step, norms, attention and SwiGLU) through the C ABI; value in decode tok/s.
One JSON line is printed by rank 0; at N=1 the default run appends the other workloads' figures
under "also" and the decoder's under "decoder".  With --gpus N > 1 (launched by torchrun) the weights are column-sharded over the
ranks, x is replicated and each output is all-gathered (by peer stores from the GEMM epilogue, or with NCCL:
--gather): total work is fixed ("strong").
"e2e" is the same step fed from pinned host memory and read back to pinned host memory inside the
timed region; the prefill step keeps the copies in and out on streams of their own (PCIe is full duplex).
Sharded, every byte still crosses PCIe once for the whole job: each rank uploads its block of x's rows, the
rows are all-gathered over NVLink, and each rank reads back its block of rows of the gathered result.

--impl reference times the reference's CPU arithmetic for the same workload (the C restatement
under oracle/, all host threads) on a bounded sample and prints the same line with
"impl": "reference".
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

# DRAM bytes per launch of the dominant kernels, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum, one launch, single GPU, full-size shard).
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (the GEMM's 71 MB output is still in the 126 MB L2 when the kernel ends, hence less than algorithmic)
NCU_TRAFFIC = {"ternary_gemv_bulk_dp4a_kernel": 6.95e6, "ternary_gemm_kernel": 28.4e6, "ternary_decode_kernel": 25.7e6,
               "w4a16_decode_kernel": 25.5e6}


def load_peaks():
    """Measured peaks of the machine (MEASURED_PEAKS.json beside this file), else the stated fallback."""
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
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
        time.sleep(0.12)
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
        busy = sm[len(sm) // 2:] if sm else []     # the busier half: idle samples before/after say nothing
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- inputs
def host_ternary(rng, n, k):
    import numpy as np
    c = rng.integers(0, 3, size=(n, k // 4, 4), dtype=np.uint8)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).astype(np.uint8)


def device_ternary(torch, n, k, gen):
    """Packed ternary weight generated on the device: every 2-bit field uniform over {0,1,2}."""
    c = torch.randint(0, 3, (n, k // 4, 4), device="cuda", dtype=torch.uint8, generator=gen)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).contiguous()


def timed(torch, fn, iters, dist=None):
    """CUDA-event time of iters calls of fn(i), barrier + synchronize on both sides, max over ranks."""
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


# ----------------------------------------------------------------------------- workloads
class Workload:
    """One benchmark workload.  Class constants describe the shapes so that the CPU arm can be
    timed without a GPU; instances hold the device buffers of this rank's shard."""
    key = name = unit = dtype = kernel_name = ""
    bound = "hbm"

    comm = None

    def gather(self, y_local, gathered):
        if self.world > 1:
            self.comm.allgather_cols(y_local, gathered=gathered)     # ncclAllGather, called by the library

    def roofline(self, peaks, kernel_ms):
        per_launch = self.kernel_work()                      # this rank's shard, one launch
        if self.bound == "hbm":
            ach, peak, unit = per_launch / (kernel_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
            src = peaks["source"] + " copy bandwidth (burst)"
        else:
            ach, unit = per_launch / (kernel_ms * 1e-3) / 1e12, self.unit
            peak = peaks["bf16_tflops"] * (2.0 if self.int8 else 1.0)
            src = ("2 x " if self.int8 else "") + peaks["source"] + " bf16 burst" + \
                  (" (the line's library_int8_gemm gives a measured int8 figure; datasheet int8 dense = 4500)" if self.int8 else "")
        out = {"bound": self.bound, "kernel": self.kernel_name, "achieved": round(ach, 1), "peak": round(peak, 1),
               "unit": unit, "frac": round(ach / peak, 4),
               "traffic": NCU_TRAFFIC.get(self.kernel_name) if self.world == 1 else None,
               "peak_source": src, "kernel_us": round(kernel_ms * 1e3, 3),
               "algorithmic_per_launch": per_launch}
        if self.bound == "tensor" and self.int8:
            # the second denominator: the datasheet's dense int8 rate (ncu's sm__pipe_tensor_cycles_active, summarised
            # under profiles/, is the direct hardware figure)
            out["peak_datasheet"], out["frac_datasheet"] = 4500.0, round(ach / 4500.0, 4)
        if self.kernel_name == "ternary_gemm_kernel" and out["traffic"]:
            out["traffic_note"] = ("DRAM bytes of one launch from ncu; below the algorithmic bytes because the output of a "
                                   "launch is still in the 126 MB L2 when the kernel ends -- no re-reads")
        return out


class PrefillGemm(Workload):
    """BitLinear prefill GEMM (configs[1]): up/gate then down projection, M=2048.

    x is fp32 as the configuration states; y is bf16, the output type of the reference's own GPU
    kernel (crates/nsl-codegen/src/bitnet/mod.rs:133-307 emits f16/bf16 stores) -- the fp32 values
    are bit-equal to the CPU path and rounded once (out_dtype="f32" runs the fp32-output variant).

    N > 1: the weight rows are sharded over the ranks and x is replicated.  gather="peer" (default):
    the GEMM epilogue stores every finished tile into all ranks' copies of the [M, N] result over
    NVLink (nslq_bitlinear_forward_gathered), the two projections run on two streams, and a flag
    barrier closes the step.  gather="nccl": each rank writes its [M, N/G] block and the library
    calls ncclAllGather (nslq_allgather_cols), the first projection's gather overlapping the second
    projection."""
    key, name = "prefill_gemm", "bitlinear_prefill_gemm_m2048_up8640x3200_down3200x8640"
    unit, dtype, bound, int8 = "TOPS", "int8 x int2 -> int32", "tensor", True
    kernel_name = "ternary_gemm_kernel"
    M, H, F = 2048, 3200, 8640
    SHAPES = [(8640, 3200), (3200, 8640)]                      # (N, K): up/gate, down
    OPS_PER_PROJ = 2 * 2048 * 3200 * 8640

    def __init__(self, torch, ops, rank, world, comm=None, gather="peer", out_dtype="bf16", streams=1, **_):
        self.torch, self.ops, self.rank, self.world = torch, ops, rank, world
        self.streams = 2 if (world == 1 and streams >= 2) else 1
        self.comm, self.mode = comm, (gather if world > 1 else "none")
        self.ydt = torch.bfloat16 if out_dtype == "bf16" else torch.float32
        self.out_dtype = out_dtype
        es = 2 if out_dtype == "bf16" else 4
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        self.layers, self.xs, self.ys, self.ygs, self.qas, self.xh, self.xst, self.wss = [], [], [], [], [], [], [], []
        self.full_w = []
        for n, k in self.SHAPES:
            r0, rows = ops.shard_rows(n, world, rank)
            full = device_ternary(torch, n, k, gen)            # same bytes on every rank (seed 0)
            self.layers.append(ops.BitLinear(full[r0:r0 + rows].contiguous(), 0.02))
            self.full_w.append(full if (world > 1 and rank == 0) else None)
            x = torch.randn(self.M, k, device="cuda", generator=gen)
            self.xs.append(x)
            self.xh.append(x.cpu().pin_memory())
            self.xst.append(torch.empty_like(x))
            self.ys.append(torch.empty(self.M, rows, device="cuda", dtype=self.ydt))
            if world > 1 and self.mode in ("peer", "ce"):
                self.ygs.append(comm.symm_empty((self.M, n), self.ydt))        # [M, N], every rank stores into it
            elif world > 1:
                self.ygs.append(torch.empty(world, self.M, rows, device="cuda", dtype=self.ydt))
            else:
                self.ygs.append(None)
            self.qas.append(ops.act_quant_i8(x, plain=False, perm=True))
            self.wss.append(torch.empty(int(ops.lib().nslq_bitlinear_workspace_bytes(self.M, k)), dtype=torch.uint8,
                                        device="cuda"))
        self.y_host = torch.empty(self.M * self.F, dtype=self.ydt).pin_memory()
        self.side = torch.cuda.Stream() if (world > 1 or self.streams == 2) else None
        self.e2e_streams = None
        self.kernel_launches = 2                               # per kernel_only() pass
        # 2 x (act quant + GEMM); sharded: + 2 flag barriers (peer) or 2 NCCL all-gathers, not counted as ours
        self.launches_per_step = 4 + (2 if self.mode in ("peer", "ce") else 0)
        # bytes over PCIe per step for the whole job (sharded with peer memory: every rank moves 1/G of them)
        whole_job_once = world == 1 or (self.mode == "peer" and self.M % world == 0)
        self.h2d = self.M * (self.H + self.F) * 4 * (1 if whole_job_once else world)
        self.d2h = self.M * (self.H + self.F) * es * (1 if whole_job_once else world)
        self.e2e_io = ("x from pinned host memory, y to pinned host memory" if world == 1 else
                       "each rank uploads M/G rows of x (all-gathered over NVLink) and reads back M/G rows of the gathered y"
                       if whole_job_once else "every rank uploads all of x and reads back all of the gathered y")
        self.l2_note = "inputs larger than L2 (26+71 MB of x, 14 MB of W, %d MB of y per step)" % (self.d2h // 1000000)

    def units_per_step(self):
        return 2 * self.OPS_PER_PROJ / 1e12

    e2e_units = property(lambda self: 2 * self.OPS_PER_PROJ / 1e12)

    def kernel_work(self):
        return self.OPS_PER_PROJ / self.world

    def one_call(self, i, x):
        if self.mode == "peer":
            self.layers[i].forward_gathered(self.comm, x, self.ygs[i], workspace=self.wss[i])
        elif self.mode == "ce":
            # the product goes into this rank's own copy of the [M, N] result (column block, row stride N)
            self.layers[i].forward_cols(x, [self.ygs[i]], self.rank * self.layers[i].N, workspace=self.wss[i])
        else:
            self.layers[i].forward(x, out=self.ys[i], workspace=self.wss[i])
            if self.mode == "nccl":
                self.comm.allgather_cols(self.ys[i], gathered=self.ygs[i])

    def step(self, xs=None):
        xs = xs or self.xs
        torch = self.torch
        cur = torch.cuda.current_stream()
        if self.world == 1:
            if self.streams == 2:
                # the two projections are independent: on two streams the second one's CTAs take the SMs that the
                # first one's last, partial round of tiles leaves idle
                fork = torch.cuda.Event()
                fork.record(cur)
                self.side.wait_event(fork)
                with torch.cuda.stream(self.side):
                    self.one_call(1, xs[1])
                    join = torch.cuda.Event()
                    join.record(self.side)
                self.one_call(0, xs[0])
                cur.wait_event(join)
                return
            for i in range(2):
                self.one_call(i, xs[i])
            return
        if self.mode == "peer":
            # The peers may still be reading the previous step's result: nobody stores before everybody
            # has arrived.  Then the two projections (independent calls) run side by side on two streams,
            # their tiles going out over NVLink as they finish, and a second barrier says "all landed".
            self.comm.barrier()
            fork = torch.cuda.Event()
            fork.record(cur)
            self.side.wait_event(fork)
            with torch.cuda.stream(self.side):
                self.one_call(1, xs[1])
                join = torch.cuda.Event()
                join.record(self.side)
            self.one_call(0, xs[0])
            cur.wait_event(join)
            self.comm.barrier()
            return
        if self.mode == "ce":
            # Copy-engine plane: each projection writes its block into this rank's own copy; the copy engines
            # then push the block to the peers on a second stream, under the next projection's kernels.
            self.comm.barrier()
            for i in range(2):
                self.one_call(i, xs[i])
                ready = torch.cuda.Event()
                ready.record(cur)
                self.side.wait_event(ready)
                with torch.cuda.stream(self.side):
                    self.comm.push_cols_async(self.ygs[i], self.layers[i].N)
            done = torch.cuda.Event()
            done.record(self.side)
            cur.wait_event(done)
            self.comm.barrier()
            return
        # NCCL plane: the all-gather of the first projection's shards runs on a second stream under the
        # second projection's quantisation and GEMM (both captured in the graph).
        for i in range(2):
            self.layers[i].forward(xs[i], out=self.ys[i], workspace=self.wss[i])
            ready = torch.cuda.Event()
            ready.record(cur)
            self.side.wait_event(ready)
            with torch.cuda.stream(self.side):
                self.comm.allgather_cols(self.ys[i], gathered=self.ygs[i])
        done = torch.cuda.Event()
        done.record(self.side)
        cur.wait_event(done)

    def kernel_only(self):
        for i in range(2):
            if self.mode == "peer":
                self.layers[i].forward_quantized_gathered(self.comm, self.qas[i], self.ygs[i])
            elif self.mode == "ce":
                self.layers[i].forward_quantized_cols(self.qas[i], [self.ygs[i]], self.rank * self.layers[i].N)
            else:
                self.layers[i].forward_quantized(self.qas[i], out=self.ys[i])

    def gather_check(self):
        """Rank 0: the gathered [M, N] of both projections against the unsharded kernel on a row sample
        (the unsharded kernel is what the parity tests hold against the CPU path)."""
        if self.world == 1 or self.rank != 0:
            return None
        torch, ok = self.torch, True
        rows = torch.arange(0, self.M, 16, device="cuda")
        for i, (n, k) in enumerate(self.SHAPES):
            ref = self.ops.BitLinear(self.full_w[i], 0.02).forward(self.xs[i][rows].contiguous(), out_dtype=self.ydt)
            got = self.ygs[i] if self.mode in ("peer", "ce") else self.ygs[i].permute(1, 0, 2).reshape(self.M, n)
            ok = ok and bool(torch.equal(got[rows], ref))
        return "gathered [M,N] of both projections bit-equal to the unsharded kernel on %d sampled rows: %s" % (
            rows.numel(), "yes" if ok else "NO")

    def e2e_step(self, it):
        """Pinned host x -> device -> quantise + GEMM -> pinned host y, both projections.  Single GPU: the
        copies in and out run on their own streams, so the result of the first projection leaves while the
        input of the second arrives (PCIe is full duplex); every buffer is single and guarded by events, and
        the step ends only when its last result is on the host.  Sharded: the inputs arrive (a row block per
        rank, all-gathered over NVLink), the sharded step runs, the gathered results leave (a row block per rank)."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        if self.world > 1 and self.mode == "peer" and self.M % self.world == 0:
            # Every byte crosses PCIe once for the whole job: rank r uploads rows r*M/G.. of each x and the ranks
            # all-gather the rows over NVLink (ncclAllGather called by the library); after a projection rank r reads
            # rows r*M/G.. of its gathered result -- columns computed by every rank -- back to its host.  Copies in
            # and out run on their own streams as on one GPU; a projection stands between two flag barriers, and a
            # rank arrives at the first one only when its own read-back of that buffer's previous content is over.
            rows = self.M // self.world
            r0 = self.rank * rows
            if not hasattr(self, "xsl"):
                self.xsl = [torch.empty(rows, k, device="cuda") for _, k in self.SHAPES]
                self.e2e_streams = (torch.cuda.Stream(), torch.cuda.Stream())
                self.e2e_consumed = [None, None]             # row block i gathered, its staging buffer free again
                self.e2e_out_done = [None, None]             # rows of result i copied to the host
            s_in, s_out = self.e2e_streams
            for i in range(2):
                if self.e2e_consumed[i] is not None:
                    s_in.wait_event(self.e2e_consumed[i])
                with torch.cuda.stream(s_in):
                    self.xsl[i].copy_(self.xh[i][r0:r0 + rows], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(s_in)
                cur.wait_event(arrived)
                self.comm.allgather_cols(self.xsl[i], gathered=self.xst[i].view(self.world, rows, -1))
                gathered = torch.cuda.Event()
                gathered.record(cur)
                self.e2e_consumed[i] = gathered
                if self.e2e_out_done[i] is not None:
                    cur.wait_event(self.e2e_out_done[i])
                self.comm.barrier()
                self.one_call(i, self.xst[i])
                self.comm.barrier()
                computed = torch.cuda.Event()
                computed.record(cur)
                s_out.wait_event(computed)
                out = self.ygs[i][r0:r0 + rows]
                with torch.cuda.stream(s_out):
                    self.y_host[:out.numel()].copy_(out.reshape(-1), non_blocking=True)   # the host buffer holds one result at a time
                    left = torch.cuda.Event()
                    left.record(s_out)
                self.e2e_out_done[i] = left
            cur.wait_event(self.e2e_out_done[1])              # the timed stream sees the last byte reach the host
            return
        if self.world > 1:
            for i in range(2):
                self.xst[i].copy_(self.xh[i], non_blocking=True)
            self.step(self.xst)
            for i in range(2):
                out = self.ygs[i]
                self.y_host[:out.numel()].copy_(out.view(-1), non_blocking=True)    # the host buffer holds one result at a time
            return
        if self.e2e_streams is None:
            self.e2e_streams = (torch.cuda.Stream(), torch.cuda.Stream())
            self.e2e_consumed = [None, None]                 # x staging buffer i read by its projection
            self.e2e_out_done = [None, None]                 # y buffer i copied to the host
        s_in, s_out = self.e2e_streams
        for i in range(2):
            if self.e2e_consumed[i] is not None:
                s_in.wait_event(self.e2e_consumed[i])
            with torch.cuda.stream(s_in):
                self.xst[i].copy_(self.xh[i], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            cur.wait_event(arrived)
            if self.e2e_out_done[i] is not None:
                cur.wait_event(self.e2e_out_done[i])
            self.one_call(i, self.xst[i])
            computed = torch.cuda.Event()
            computed.record(cur)
            self.e2e_consumed[i] = computed
            s_out.wait_event(computed)
            out = self.ys[i]
            with torch.cuda.stream(s_out):
                self.y_host[:out.numel()].copy_(out.view(-1), non_blocking=True)
                left = torch.cuda.Event()
                left.record(s_out)
            self.e2e_out_done[i] = left
        cur.wait_event(self.e2e_out_done[1])                  # the timed stream sees the last byte reach the host

    @classmethod
    def cpu_baseline(cls, threads, budget_s=15.0):
        import numpy as np
        from oracle import oracle as o
        rng = np.random.default_rng(0)
        rows, dt_tot = 16, 0.0
        for n, k in cls.SHAPES:
            packed = host_ternary(rng, n, k)
            x = rng.standard_normal((rows, k)).astype(np.float32)
            t0, reps = time.perf_counter(), 0
            while True:
                o.bitlinear_forward_packed(x, packed, n, 0.02, threads=threads)
                reps += 1
                if time.perf_counter() - t0 > budget_s / 2 or reps >= 50:
                    break
            dt_tot += (time.perf_counter() - t0) / reps
        # the rate on the sample is the rate on the whole workload (rows are independent): ops of the sample / its time
        val = 2 * cls.OPS_PER_PROJ * (rows / cls.M) / dt_tot / 1e12
        return {"value": round(val, 6), "unit": "TOPS", "cores": threads, "kind": "port",
                "sample": "%d of %d token rows of both projections per step (%.3f s); a full step at this rate: %.1f s"
                          % (rows, cls.M, dt_tot, dt_tot * cls.M / rows)}, dt_tot


class DecodeGemv(Workload):
    """BitLinear decode GEMV (configs[0] shape), 64 distinct weights per step."""
    key, name = "decode_gemv", "bitlinear_decode_gemv_m1_n8640_k3200"
    unit, dtype, bound, int8 = "GB/s", "int8 x int2 -> int32", "hbm", True
    kernel_name = "ternary_gemv_bulk_dp4a_kernel"
    N, K, M, LAYERS = 8640, 3200, 1, 64
    BYTES_PER_CALL = 8640 * 3200 // 4 + 3200 * 4 + 8640 * 4    # packed W + x fp32 + y fp32

    def __init__(self, torch, ops, rank, world, streams=1, comm=None, **_):
        self.torch, self.ops, self.rank, self.world, self.comm = torch, ops, rank, world, comm
        self.streams = max(1, streams) if world == 1 else 1
        self.side = [torch.cuda.Stream() for _ in range(self.streams)] if self.streams > 1 else []
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        r0, rows = ops.shard_rows(self.N, world, rank)
        self.rows = rows
        self.layers = []
        for _ in range(self.LAYERS):
            full = device_ternary(torch, self.N, self.K, gen)
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
        self.kernel_launches = self.LAYERS
        # one row: the quantisation is fused into the decode kernel
        self.launches_per_step = self.LAYERS * (1 if self.M == 1 else 2)
        self.h2d, self.d2h = self.M * self.K * 4, self.M * self.N * 4
        mb = self.N * self.K / 4e6
        self.l2_note = "%d distinct %.1f MB weights per step (%.0f MB > L2)" % (self.LAYERS, mb, self.LAYERS * mb)

    def units_per_step(self):
        return self.LAYERS * self.BYTES_PER_CALL / 1e9

    e2e_units = property(lambda self: self.BYTES_PER_CALL / 1e9)

    def kernel_work(self):
        return self.rows * self.K // 4 + self.M * self.K * 4 + self.M * self.rows * 4

    def step(self):
        if self.streams > 1:
            # the calls are independent (same x, distinct weights): issue them round-robin on several
            # streams so that one call's weight stream overlaps another's arithmetic
            cur = self.torch.cuda.current_stream()
            for st in self.side:
                st.wait_stream(cur)
            for i, layer in enumerate(self.layers):
                j = i % self.streams
                with self.torch.cuda.stream(self.side[j]):
                    layer.forward(self.x, out=self.y_side[j], workspace=self.ws)   # one row: workspace unused
            for st in self.side:
                cur.wait_stream(st)
            return
        for layer in self.layers:
            layer.forward(self.x, out=self.y_local, workspace=self.ws)
            self.gather(self.y_local, self.y_full)

    def kernel_only(self):
        if self.world == 1:
            return self.step()                                 # the step is that kernel and nothing else
        for layer in self.layers:
            layer.forward(self.x, out=self.y_local, workspace=self.ws)

    def e2e_step(self, i):
        layer = self.layers[i % self.LAYERS]
        self.x_stage.copy_(self.x_host, non_blocking=True)
        layer.forward(self.x_stage, out=self.y_local, workspace=self.ws)
        self.gather(self.y_local, self.y_full)
        out = self.y_full if self.world > 1 else self.y_local
        self.y_host.view(-1)[:out.numel()].copy_(out.view(-1), non_blocking=True)

    @classmethod
    def cpu_baseline(cls, threads, budget_s=12.0):
        import numpy as np
        from oracle import oracle as o
        rng = np.random.default_rng(0)
        packed = host_ternary(rng, cls.N, cls.K)
        x = rng.standard_normal((cls.M, cls.K)).astype(np.float32)
        o.bitlinear_forward_packed(x, packed, cls.N, 0.02, threads=threads)
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and n < 400:
            o.bitlinear_forward_packed(x, packed, cls.N, 0.02, threads=threads)
            n += 1
        dt = (time.perf_counter() - t0) / n
        return {"value": round(cls.BYTES_PER_CALL / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": "%d full [%d,%d]x[%d,%d] calls, %.2f ms each" % (n, cls.M, cls.K, cls.N, cls.K, dt * 1e3)}, dt


class DecodeGemvVocab(DecodeGemv):
    """The same decode call on the decoder's largest matrix shape (vocabulary projection, 25.6 MB
    packed)."""
    key, name = "decode_gemv_vocab", "bitlinear_decode_gemv_m1_n32002_k3200"
    kernel_name = "ternary_gemv_bulk_dp4a_kernel"
    N, K, M, LAYERS = 32002, 3200, 1, 16
    BYTES_PER_CALL = 32002 * 3200 // 4 + 3200 * 4 + 32002 * 4


class DecodeGemvVocabM16(DecodeGemv):
    """Sixteen tokens against the same matrix (batched decode): act_quant + the streaming kernel."""
    key, name = "decode_gemv_vocab_m16", "bitlinear_decode_m16_n32002_k3200"
    kernel_name = "ternary_decode_kernel"
    N, K, M, LAYERS = 32002, 3200, 16, 16
    BYTES_PER_CALL = 32002 * 3200 // 4 + 16 * 3200 * 4 + 16 * 32002 * 4


class W4A16(Workload):
    """AWQ-style W4A16 (configs[2]): N=11008, K=4096, group 128, M tokens of bf16 activations."""
    N, K, GS = 11008, 4096, 128
    dtype, int8 = "bf16 x uint4 -> fp32", False

    def __init__(self, torch, ops, rank, world, M=1, comm=None, **_):
        self.torch, self.ops, self.rank, self.world, self.M, self.comm = torch, ops, rank, world, M, comm
        self.key = "w4a16_m%d" % M
        self.name = "w4a16_m%d_n11008_k4096_g128" % M
        gemm = M > 16
        self.bound, self.unit = ("tensor", "TFLOPS") if gemm else ("hbm", "GB/s")
        self.kernel_name = "w4a16_gemm_kernel" if gemm else ("w4a16_decode_kernel" if M >= 4 else "w4a16_gemv_persistent_kernel")
        self.LAYERS = 8 if gemm else 24
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        G = self.K // self.GS
        r0, rows = ops.shard_rows(self.N, world, rank)
        self.rows = rows
        self.layers = []
        for _ in range(self.LAYERS):
            codes = torch.randint(0, 256, (self.N, self.K // 2), device="cuda", dtype=torch.uint8, generator=gen)
            scale = (torch.randn(self.N, G, device="cuda", generator=gen).abs() * (0.02 / 7)).to(torch.bfloat16)
            zp = torch.randint(0, 16, (self.N, G), device="cuda", dtype=torch.uint8, generator=gen)
            self.layers.append(ops.W4A16.from_nk(codes[r0:r0 + rows].contiguous(), scale[r0:r0 + rows].contiguous(),
                                                 zp[r0:r0 + rows].contiguous(), self.GS))
            del codes, scale, zp
        self.x = torch.randn(M, self.K, device="cuda", generator=gen).to(torch.bfloat16)
        self.x_host = self.x.cpu().pin_memory()
        self.x_stage = torch.empty_like(self.x)
        self.y_local = torch.empty(M, rows, device="cuda", dtype=torch.bfloat16)
        self.y_full = torch.empty(world, M, rows, device="cuda", dtype=torch.bfloat16) if world > 1 else None
        self.y_host = torch.empty(M * self.N, dtype=torch.bfloat16).pin_memory()
        self.kernel_launches = self.LAYERS * ((M + 15) // 16 if not gemm else 1)
        self.launches_per_step = self.kernel_launches
        self.h2d, self.d2h = M * self.K * 2, M * self.N * 2
        self.l2_note = "%d distinct 22.5 MB weights per step (> L2)" % self.LAYERS

    def bytes_per_call(self, rows):
        G = self.K // self.GS
        return rows * self.K // 2 + rows * G * 2 + rows * G // 2 + self.M * self.K * 2 + self.M * rows * 2

    def flops_per_call(self, rows):
        return 2 * self.M * rows * self.K

    def units_per_step(self):
        per = self.flops_per_call(self.N) / 1e12 if self.bound == "tensor" else self.bytes_per_call(self.N) / 1e9
        return self.LAYERS * per

    @property
    def e2e_units(self):
        return self.units_per_step() / self.LAYERS

    def kernel_work(self):
        return self.flops_per_call(self.rows) if self.bound == "tensor" else self.bytes_per_call(self.rows)

    def step(self):
        for layer in self.layers:
            layer.forward(self.x, out=self.y_local)
            self.gather(self.y_local, self.y_full)

    def kernel_only(self):
        for layer in self.layers:
            layer.forward(self.x, out=self.y_local)

    def e2e_step(self, i):
        self.x_stage.copy_(self.x_host, non_blocking=True)
        self.layers[i % self.LAYERS].forward(self.x_stage, out=self.y_local)
        self.gather(self.y_local, self.y_full)
        out = self.y_full if self.world > 1 else self.y_local
        self.y_host[:out.numel()].copy_(out.view(-1), non_blocking=True)

    @classmethod
    def cpu_baseline_m(cls, M, threads, budget_s=12.0):
        import numpy as np
        from oracle import oracle as o
        rng = np.random.default_rng(0)
        G = cls.K // cls.GS
        codes = rng.integers(0, 256, size=(cls.N, cls.K // 2), dtype=np.uint8)
        scale = (np.abs(rng.standard_normal((cls.N, G))) * 0.02 / 7).astype(np.float32)
        zp = rng.integers(0, 16, size=(cls.N, G), dtype=np.uint8)
        rows = min(M, 4)
        x = rng.standard_normal((rows, cls.K)).astype(np.float32)
        t0, n = time.perf_counter(), 0
        while True:
            o.w4a16_matmul_nk(x, codes, scale, zp, cls.N, cls.K, cls.GS, threads=threads)
            n += 1
            if time.perf_counter() - t0 > budget_s or n >= 50:
                break
        dt = (time.perf_counter() - t0) / n * (M / rows)
        if M > 16:
            val, unit = 2 * M * cls.N * cls.K / dt / 1e12, "TFLOPS"
        else:
            val = (cls.N * cls.K // 2 + cls.N * G * 2 + cls.N * G // 2 + M * cls.K * 2 + M * cls.N * 2) / dt / 1e9
            unit = "GB/s"
        return {"value": round(val, 6), "unit": unit, "cores": threads, "kind": "port",
                "sample": "%d of %d token rows, extrapolated linearly (%.2f s per call)" % (rows, M, dt)}, dt


def make_workload(key, torch, ops, rank, world, streams=1, comm=None, gather="peer", out_dtype="bf16"):
    if key == "prefill_gemm":
        return PrefillGemm(torch, ops, rank, world, comm=comm, gather=gather, out_dtype=out_dtype, streams=streams)
    if key in DECODE_CLASSES:
        return DECODE_CLASSES[key](torch, ops, rank, world, streams=streams, comm=comm)
    if key.startswith("w4a16_m"):
        return W4A16(torch, ops, rank, world, M=int(key[7:]), comm=comm)
    raise SystemExit("unknown workload %s" % key)


def library_int8_yardstick(torch, ours_kernel_us):
    """A measured int8 yardstick for the tensor roofline: the BLAS library's dense int8 x int8 -> int32 GEMM
    (torch._int_mm, cuBLASLt) timed here on the two projection shapes of the prefill workload -- plain int8 operands,
    nothing to unpack, int32 results left as they are -- and on a large cube for its peak rate.  Never on the
    product path."""
    if not hasattr(torch, "_int_mm"):
        return None
    g = torch.Generator(device="cuda")
    g.manual_seed(2)

    def timed_call(M, N, K, reps):
        a = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8, generator=g)
        b = torch.randint(-1, 2, (N, K), device="cuda", dtype=torch.int8, generator=g).t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    try:
        same = [timed_call(PrefillGemm.M, n, k, 20) for n, k in PrefillGemm.SHAPES]
        cube = timed_call(8192, 8192, 8192, 5)
    except RuntimeError as e:                 # a build of the framework without this routine for the device
        return {"unavailable": str(e)[:120]}
    mean = sum(same) / len(same)
    return {"routine": "torch._int_mm (cuBLASLt int8 x int8 -> int32), dense int8 weights, no epilogue",
            "same_shapes_us": [round(v, 2) for v in same], "same_shapes_mean_us": round(mean, 2),
            "same_shapes_TOPS": round(PrefillGemm.OPS_PER_PROJ / 1e12 / (mean * 1e-6), 1),
            "ours_kernel_us": ours_kernel_us, "ours_over_library": round(mean / ours_kernel_us, 3) if ours_kernel_us else None,
            "peak_TOPS_8192_cube": round(2.0 * 8192 ** 3 / 1e12 / (cube * 1e-6), 1)}


def gpu_prior_art(torch, ours_prefill_ms, ours_decode_us, ours_w4_us=None):
    """The design of the one GPU kernel NSL emits for BitLinear (one thread per output column, scalar loop over
    packed bytes read straight from HBM, every CTA re-quantising its activation row), restated in
    oracle/gpu_prior_art.cu and timed on this GPU on the two BitLinear configurations: a baseline leg beside the
    CPU one, never part of the product.  Its results are checked bit for bit in tests/test_gpu_prior_art.py."""
    from oracle import oracle as o
    g = torch.Generator(device="cuda")
    g.manual_seed(1)

    def timed_call(M, N, K, iters):
        x = torch.randn(M, K, device="cuda", generator=g)
        w = torch.randint(0, 256, (N, K // 4), device="cuda", dtype=torch.uint8, generator=g) & 0xA5   # codes 0..2 only
        o.gpu_prior_art_bitlinear(x, w, 0.02)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            o.gpu_prior_art_bitlinear(x, w, 0.02)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def timed_w4(Mt, iters):
        N, K, GS = W4A16.N, W4A16.K, W4A16.GS
        codes = torch.randint(0, 256, (N, K // 2), device="cuda", dtype=torch.uint8, generator=g)
        scale = torch.rand(N, K // GS, device="cuda", generator=g) * 0.003
        zp = torch.randint(0, 16, (N, K // GS), device="cuda", dtype=torch.uint8, generator=g)
        x = torch.randn(Mt, K, device="cuda", generator=g).to(torch.bfloat16)
        o.gpu_prior_art_w4_matmul(x, codes, scale, zp, GS)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            o.gpu_prior_art_w4_matmul(x, codes, scale, zp, GS)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    M = PrefillGemm.M
    pre = sum(timed_call(M, n, k, 3) for n, k in PrefillGemm.SHAPES)
    dec = timed_call(1, 8640, 3200, 20) * 1e3
    w4 = {m: timed_w4(m, 10) for m in (1, 16, 256)}
    return {"kernel": "oracle/gpu_prior_art.cu: structure of NSL's emitted BitLinear kernel (crates/nsl-codegen/src/bitnet/mod.rs:133-236), "
                      "block_n 128, fp32 in and out, quantisation inside as in the reference",
            "prefill_m2048_both_projections": {"ms": round(pre, 3), "TOPS": round(2 * PrefillGemm.OPS_PER_PROJ / 1e12 / (pre * 1e-3), 2),
                                               "ours_ms": round(ours_prefill_ms, 5), "speedup_of_ours": round(pre / ours_prefill_ms, 1)},
            "decode_m1_8640x3200": {"us": round(dec, 2), "ours_us": ours_decode_us,
                                    "speedup_of_ours": round(dec / ours_decode_us, 1) if ours_decode_us else None},
            "w4a16_n11008_k4096_g128": {
                "route": "the reference's nsl_qtensor_matmul_mixed (crates/nsl-runtime/src/quantize.rs:547-585): dequantise the whole "
                         "weight to f32 on every call (here on the GPU, oracle/gpu_prior_art.cu; the reference does it on the CPU), "
                         "then the BLAS library's f32 tensor-core (TF32) matmul",
                "us": {"m%d" % m: round(v, 1) for m, v in w4.items()},
                "ours_us": ours_w4_us,
                "speedup_of_ours": {k: round(w4[int(k[1:])] / v, 1) for k, v in (ours_w4_us or {}).items() if v}}}


def cpu_arm(key, threads, budget_s):
    if key == "prefill_gemm":
        return PrefillGemm.cpu_baseline(threads, budget_s)
    if key in DECODE_CLASSES:
        return DECODE_CLASSES[key].cpu_baseline(threads, budget_s)
    return W4A16.cpu_baseline_m(int(key[7:]), threads, budget_s)


DECODE_CLASSES = {c.key: c for c in (DecodeGemv, DecodeGemvVocab, DecodeGemvVocabM16)}
WORKLOAD_KEYS = ["prefill_gemm", "decode_gemv", "decode_gemv_vocab", "decode_gemv_vocab_m16", "w4a16_m1", "w4a16_m4", "w4a16_m8", "w4a16_m16", "w4a16_m256",
                 "bitnet3b_b1", "bitnet3b_b8", "bitnet3b_b64"]
DEFAULT_WORKLOAD = "prefill_gemm"
META = {"prefill_gemm": PrefillGemm, **DECODE_CLASSES}


# ----------------------------------------------------------------------------- decoder workload
def run_decoder(torch, batch, peaks, prompt=512, steps=256, warm=8, layers=None):
    """BitNet b1.58-3B-shaped decoder (configs[3]): random ternary weights, uniform-random prompt ids,
    greedy decode.  Returns decode / prefill tokens per second and the HBM figures of a decode step.
    `layers` / `steps` below the model's own are for profiler captures only (a few launches of each kernel)."""
    from nsl_b200 import decoder
    cfg = decoder.BitNetConfig() if not layers else decoder.BitNetConfig(layers=layers)
    model = decoder.BitNetDecoder(cfg, batch, prompt + steps + warm + 8)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    ids_host = torch.randint(0, cfg.vocab, (batch, prompt), generator=torch.Generator().manual_seed(0)).pin_memory()
    ids = ids_host.cuda()
    model.prefill(ids)                                   # warm-up (lazy initialisation, workspaces)
    torch.cuda.synchronize()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    model.prefill(ids)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    model.capture()
    model.decode(warm)
    torch.cuda.synchronize()
    e1.record()
    model.decode(steps)
    e2.record()
    torch.cuda.synchronize()
    dec_ms = e1.elapsed_time(e2)
    step_ms = dec_ms / steps
    ctx_mid = prompt + warm + steps // 2
    step_bytes = model.step_bytes(ctx_mid)
    ach = step_bytes / (step_ms * 1e-3) / 1e9
    # host to host: prompt ids from pinned memory, prefill, then every step's tokens read back
    tok_host = torch.empty(batch, dtype=torch.long).pin_memory()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ids2 = ids_host.cuda(non_blocking=True)
    model.prefill(ids2)
    for _ in range(steps):
        model.graph.replay()
        tok_host.copy_(model.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_s = time.perf_counter() - t0
    out = {"workload": "bitnet_b158_3b_decoder_b%d_prompt%d_decode%d" % (batch, prompt, steps),
           "decode_tok_s": round(batch * steps / (dec_ms * 1e-3), 1), "ms_per_decode_step": round(step_ms, 4),
           "prefill_tok_s": round(batch * prompt / (prefill_ms * 1e-3), 1), "prefill_ms": round(prefill_ms, 2),
           "e2e_tok_s": round(batch * (steps) / e2e_s, 1),
           "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": round(ach / peaks["hbm_gbs"], 4), "bytes_per_step": step_bytes,
                        "note": "ternary weights + bf16 lm_head + KV read at mid-run context; a decode step is library launches "
                                "(embedding rows, RMSNorm and SiLU*up inside the projections' launches at one token per sequence batch of one, RoPE + KV "
                                "append + attention, final norm, argmax) except the lm_head's bf16 GEMM (cuBLAS); at prefill the attention "
                                "over the prompt (SDPA) and the lm_head are PyTorch, RoPE + cache writes are one library launch"},
           "ceiling_tok_s": round(batch / (step_bytes / (peaks["hbm_gbs"] * 1e9)), 1)}
    del model
    torch.cuda.empty_cache()
    return out


def decoder_cpu_baseline(budget_s=6.0):
    """The reference's CPU arithmetic for the linears of ONE decoder layer at one token (BitNet-3B shapes), one
    host thread; decode tokens per second = 1 / (26 layers x that time), the glue between the linears not counted."""
    import numpy as np
    from oracle import oracle as o
    rng = np.random.default_rng(0)
    h, f = 3200, 8640
    shapes = [(h, h)] * 4 + [(f, h)] * 2 + [(h, f)]
    ws = [host_ternary(rng, n, k) for n, k in shapes]
    xs = {h: rng.standard_normal((1, h)).astype(np.float32), f: rng.standard_normal((1, f)).astype(np.float32)}
    t0, reps = time.perf_counter(), 0
    while True:
        for (n, k), w in zip(shapes, ws):
            o.bitlinear_forward_packed(xs[k], w, n, 0.02, threads=1)
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 20:
            break
    t_layer = (time.perf_counter() - t0) / reps
    return {"value": round(1.0 / (26 * t_layer), 3), "unit": "tok/s", "cores": 1, "kind": "port",
            "sample": "the seven BitLinear calls of one layer at one token, %d times (%.3f s per layer); x 26 layers, "
                      "norms, attention and lm_head not counted; per token, so the same for every batch size" % (reps, t_layer)}


# ----------------------------------------------------------------------------- sharded decoder workload
def run_sharded_decoder(torch, comm, dist, peaks, batch=256, context=2048, n_layers=4, reps=10):
    """configs[4]: 7B-class ternary decoder, batch 256 decode at context 2048, weights column-sharded over
    the ranks.  n_layers distinct layers are built and timed (all 32 have the same shapes; the whole model's
    KV cache is 275 GB); tok/s is batch / (32 x time per layer)."""
    from nsl_b200 import ops, sharded_decoder
    m = sharded_decoder.ShardedDecodeLayers(comm, batch, context, n_layers)
    cfg = m.cfg

    def graph_us(fn, per=1):
        for _ in range(2):
            fn()
        g = capture(torch, fn)
        g.replay()
        ms = timed(torch, lambda i: g.replay(), reps, dist)
        return ms * 1e3 / reps / per

    layer_us = graph_us(m.step, n_layers)
    # the pieces, each over the n_layers distinct layers (weights and caches larger than L2 in total)
    x = m.x
    qa_h = ops.rmsnorm_act_quant_i8(x, m.layers[0]["n1"], cfg.eps, plain=False, perm=True)
    q0, k0, v0 = m.qkv(m.layers[0], qa_h)
    a0 = m.attention(m.layers[0], q0, k0, v0)
    qa_f = ops.act_quant_i8(m.h_full, plain=False, perm=True)
    g0 = m.layers[0]["gate"].forward_quantized(qa_h, out_dtype=torch.bfloat16)
    parts = {
        "rmsnorm_quant": graph_us(lambda: [ops.rmsnorm_act_quant_i8(x, L["n1"], cfg.eps, plain=False, perm=True) for L in m.layers], n_layers),
        "qkv_linears": graph_us(lambda: [m.qkv(L, qa_h) for L in m.layers], n_layers),
        "attention": graph_us(lambda: [m.attention(L, q0, k0, v0) for L in m.layers], n_layers),
        "attn_out_gather": graph_us(lambda: [m.gather_act(a0, m.a_full) for _ in m.layers], n_layers),
        "o_linear_local": graph_us(lambda: [L["o"].forward_quantized(qa_h, out_dtype=torch.bfloat16) for L in m.layers], n_layers),
        "o_linear_gathered": graph_us(lambda: [m.linear_gathered(L["o"], qa_h, m.o_full) for L in m.layers], n_layers),
        "gate_up_linears": graph_us(lambda: [(L["gate"].forward_quantized(qa_h, out_dtype=torch.bfloat16),
                                              L["up"].forward_quantized(qa_h, out_dtype=torch.bfloat16)) for L in m.layers], n_layers),
        "swiglu_gather": graph_us(lambda: [m.gather_act(g0, m.h_full) for _ in m.layers], n_layers),
        "down_linear_local": graph_us(lambda: [L["down"].forward_quantized(qa_f, out_dtype=torch.bfloat16) for L in m.layers], n_layers),
        "down_linear_gathered": graph_us(lambda: [m.linear_gathered(L["down"], qa_f, m.d_full) for L in m.layers], n_layers),
    }
    parts = {k: round(v, 2) for k, v in parts.items()}
    G = comm.world
    comm_us = parts["attn_out_gather"] + parts["swiglu_gather"] + (parts["o_linear_gathered"] - parts["o_linear_local"]) + \
        (parts["down_linear_gathered"] - parts["down_linear_local"])
    kv_floor_us = m.kv_bytes_per_layer / (peaks["hbm_gbs"] * 1e9) * 1e6
    out = {"workload": "ternary_7b_decoder_b%d_ctx%d_column_sharded_x%d" % (batch, context, G),
           "decode_tok_s": round(batch / (cfg.layers * layer_us * 1e-6), 1), "us_per_layer": round(layer_us, 1),
           "layers_timed": n_layers, "layers_model": cfg.layers,
           "per_layer_us": parts, "communication_us_per_layer": round(comm_us, 1),
           "exchange_bytes_per_layer_per_rank": int((3 * cfg.hidden + cfg.ffn) * batch * 2 * (G - 1) / G),
           "kv_read_floor_us_per_layer": round(kv_floor_us, 1),
           "note": "one CUDA graph per step over the timed layers; q/k/v stay local, attention is head-sharded, four "
                   "all-gathers per layer (attention output, o_proj output, SiLU(gate)*up, down output) by peer stores + "
                   "flag barrier; embedding, final norm and lm_head not included; one GPU cannot hold this workload "
                   "(KV cache 275 GB)"}
    st = comm.status()
    if st:
        out["status"] = st
    del m
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- measurement
def measure(torch, wl, steps, warmup, use_graph, dist, sampler=None, want_e2e=True):
    """value (whole job), the dominant kernel alone, and the host-to-host number of one workload."""
    for _ in range(max(warmup, 3)):
        wl.step()
    torch.cuda.synchronize()
    graph = capture(torch, wl.step) if use_graph else None
    if graph:
        for _ in range(2):
            graph.replay()
    if sampler:
        sampler.start()
        time.sleep(0.2)
    ms = timed(torch, (lambda i: graph.replay()) if graph else (lambda i: wl.step()), steps, dist)
    clocks = sampler.stop() if sampler else None
    ms_per_step = ms / steps
    out = {"value": wl.units_per_step() / (ms_per_step * 1e-3), "ms_per_step": ms_per_step, "clocks": clocks,
           "graph": bool(graph)}

    # dominant kernel alone (pre-quantised activations, no collective), same buffers
    kgraph = capture(torch, wl.kernel_only) if use_graph else None
    reps = max(steps, 5)
    for _ in range(3):
        kgraph.replay() if kgraph else wl.kernel_only()
    kms = timed(torch, (lambda i: kgraph.replay()) if kgraph else (lambda i: wl.kernel_only()), reps, dist)
    out["kernel_ms"] = kms / reps / wl.kernel_launches

    if want_e2e:
        # through the host-facing call: pinned host input -> device -> op -> pinned host result
        for i in range(3):
            wl.e2e_step(i)
        iters = max(steps, 10)
        ems = timed(torch, wl.e2e_step, iters, dist)
        out["e2e"] = wl.e2e_units / (ems / iters * 1e-3)
    return out


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from nsl_b200 import lib, ops
    comm = None
    if world > 1:
        from nsl_b200 import sharding
        # NCCL may print its version banner on stdout when a communicator is created; stdout carries the one
        # JSON line, so the banner is sent to stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            comm = sharding.Comm.from_torch()      # the library's own communicator (NCCL + peer memory)
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    if args.no_pdl:
        lib().nslq_set_dependent_launch(0)
    peaks = load_peaks()
    use_graph = not args.no_graph            # NCCL collectives are captured into the graph as well

    if args.workload.startswith("bitnet3b_b"):
        out = run_decoder(torch, int(args.workload[10:]), peaks, steps=args.decode_steps, layers=args.decoder_layers)
        if args.decoder_layers or args.decode_steps != 256:
            out["workload"] += "_REDUCED_layers%s_not_a_benchmark" % (args.decoder_layers or 26)
        out.update({"metric": METRIC, "value": out["decode_tok_s"], "unit": "tok/s", "n_gpus": 1,
                    "higher_is_better": True, "data": "synthetic (seed 0)", "dtype": "int8 x int2 -> int32"})
        print(json.dumps(out))
        return
    wl = make_workload(args.workload, torch, ops, rank, world, streams=args.streams, comm=comm, gather=args.gather,
                       out_dtype=args.out_dtype)
    sampler = ClockSampler(local) if rank == 0 else None
    m = measure(torch, wl, args.steps, args.warmup, use_graph, dist, sampler)
    roof = wl.roofline(peaks, m["kernel_ms"])
    check = wl.gather_check() if hasattr(wl, "gather_check") else None
    if world == 1:
        par = "single GPU"
    elif getattr(wl, "mode", "nccl") == "ce":
        par = ("weight rows sharded x%d, x replicated; each GEMM writes its block into this rank's copy of the result and "
               "the copy engines push it to every peer on a second stream (under the next projection), flag barriers "
               "before and after" % world)
    elif getattr(wl, "mode", "nccl") == "peer":
        par = ("weight rows sharded x%d, x replicated; all-gather fused into the GEMM epilogue (tiles stored into every "
               "rank's copy over NVLink), two projections on two streams, flag barriers before and after" % world)
    else:
        par = "weight rows sharded x%d, x replicated; ncclAllGather of the output shards called by the library" % world
    line = None
    if rank == 0:
        cpu, _ = cpu_arm(args.workload, 1, 12.0)
        line = {
            "metric": METRIC, "value": round(m["value"], 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(m["ms_per_step"], 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seed 0)",
            "config": {"workload": wl.name, "cuda_graph": m["graph"], "dependent_launch": not args.no_pdl,
                       "streams": getattr(wl, "streams", 1), "l2": wl.l2_note,
                       "x_dtype": "f32", "y_dtype": getattr(wl, "out_dtype", "f32"), "parallelism": par,
                       "e2e_io": getattr(wl, "e2e_io", None)},
            "e2e": {"value": round(m["e2e"], 3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d,
                    "d2h_bytes_per_step": wl.d2h},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof, "cpu_baseline": cpu, "clocks": m["clocks"],
        }
        if check:
            line["gather_check"] = check
    status = ops.device_status()
    if comm is not None:
        status = status or comm.status()
    del wl
    torch.cuda.empty_cache()

    # the other configurations of the metric, shorter runs, single GPU only
    if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_also:
        also, cpu_cache = [], {}
        for key, streams in (("w4a16_m256", 1), ("w4a16_m16", 1), ("w4a16_m1", 1), ("decode_gemv_vocab_m16", 1),
                             ("decode_gemv_vocab", 1), ("decode_gemv_vocab", 4), ("decode_gemv", 1), ("decode_gemv", 4)):
            w2 = make_workload(key, torch, ops, rank, world, streams=streams)
            m2 = measure(torch, w2, max(10, args.steps // 3), 3, use_graph, None, None, want_e2e=True)
            r2 = w2.roofline(peaks, m2["kernel_ms"])
            if key not in cpu_cache:
                cpu_cache[key] = cpu_arm(key, 1, 3.0)[0]
            entry = {"workload": w2.name, "streams": streams, "value": round(m2["value"], 2), "unit": w2.unit,
                     "ms_per_step": round(m2["ms_per_step"], 5), "e2e": round(m2["e2e"], 3),
                     "roofline": {k: r2[k] for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "kernel_us")},
                     "cpu_baseline": cpu_cache[key]}
            also.append(entry)
            status = status or ops.device_status()
            del w2
            torch.cuda.empty_cache()
        dec_cpu = decoder_cpu_baseline()
        line["decoder"] = [dict(run_decoder(torch, b, peaks), cpu_baseline=dec_cpu) for b in (64, 8, 1)]
        line["also"] = also                 # the decode GEMV of configs[0] comes last: the end of a long line is what survives a cut
        g1 = [a for a in also if a["workload"].startswith("bitlinear_decode_gemv_m1_n8640")]
        chain = [a for a in g1 if a["streams"] == 1]
        w4_us = {"m" + a["workload"].split("_")[1][1:]: a["roofline"]["kernel_us"] for a in also if a["workload"].startswith("w4a16_m")}
        line["gpu_prior_art"] = gpu_prior_art(torch, m["ms_per_step"], chain[0]["roofline"]["kernel_us"] if chain else None, w4_us)
        line["library_int8_gemm"] = library_int8_yardstick(torch, roof.get("kernel_us"))
        line["targets"] = {
            "decode_gemv_m1_8640x3200": {("independent_calls_%d_streams" % a["streams"]) if a["streams"] > 1 else "dependent_chain":
                                         {"us_per_call": a["roofline"]["kernel_us"], "GBps": a["roofline"]["achieved"],
                                          "frac_of_measured_hbm": a["roofline"]["frac"]} for a in g1},
            "decode_gemv_floor_us": {"dependent_chain": 2.9, "independent_calls_4_streams": 1.0,
                                     "what": "a kernel that only streams the 6.9 MB matrix into registers, launched the same two ways "
                                             "(measured once with a load-only probe, not per run): what launch, latency and HBM leave"},
            "prefill_gemm_m2048": {"TOPS_kernel": roof["achieved"], "frac_of_2x_measured_bf16": roof["frac"],
                                   "frac_of_datasheet_int8": roof.get("frac_datasheet")},
            "bitnet3b_decode_tok_s": {d["workload"].split("_")[4]: d["decode_tok_s"] for d in line["decoder"]},
        }
    if world > 1 and args.workload == DEFAULT_WORKLOAD and not args.no_also:
        sd = run_sharded_decoder(torch, comm, dist, peaks)
        if rank == 0:
            line["sharded_decoder"] = sd
    elif world == 1 and rank == 0 and args.workload == DEFAULT_WORKLOAD and not args.no_also:
        line["sharded_decoder"] = {"workload": "ternary_7b_decoder_b256_ctx2048_column_sharded",
                                   "unavailable": "needs 2, 4 or 8 GPUs: the KV cache of batch 256 at context 2048 is 275 GB "
                                                  "(8.6 GB per layer), more than one GPU holds; run with --gpus N"}
    if rank == 0:
        line["device_status"] = status
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        if comm is not None:
            comm.close()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU arithmetic for the same workload, all host threads, bounded sample per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import oracle as o
    o.build()
    threads = o.max_threads()
    total = max(args.warmup, 0) + args.steps
    budget = min(8.0, 150.0 / max(total, 1))
    vals, per, cpu = [], [], None
    for i in range(total):
        cpu, dt = cpu_arm(args.workload, threads, budget)
        if i >= args.warmup:
            vals.append(cpu["value"])
            per.append(dt)
    v = sum(vals) / len(vals)
    cpu["value"] = round(v, 6)
    name = META[args.workload].name if args.workload in META else "w4a16_m%s_n11008_k4096_g128" % args.workload[7:]
    dtype = META[args.workload].dtype if args.workload in META else W4A16.dtype
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(v, 6), "unit": cpu["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sum(per) / len(per) * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic (seed 0)", "config": {"workload": name, "host_threads": threads},
        "cpu_baseline": cpu,
        "e2e": {"value": round(v, 6), "unit": cpu["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=WORKLOAD_KEYS)
    ap.add_argument("--streams", type=int, default=None,
                    help="decode_gemv: issue the independent calls of a step round-robin on this many streams (default 1: a "
                         "dependent chain); prefill_gemm: 2 (default) runs the step's two independent projections on two "
                         "streams, 1 on one")
    ap.add_argument("--gather", default="peer", choices=["peer", "ce", "nccl"],
                    help="N > 1, prefill: shards stored into every rank's copy by the GEMM epilogue, or ncclAllGather")
    ap.add_argument("--out-dtype", default="bf16", choices=["bf16", "f32"], help="prefill: dtype of y")
    ap.add_argument("--no-graph", action="store_true", help="issue launches directly instead of replaying a CUDA graph")
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels without the programmatic-dependent-launch attribute")
    ap.add_argument("--no-also", action="store_true", help="skip the secondary workloads of the default run")
    ap.add_argument("--decoder-layers", type=int, default=0, help="bitnet3b_*: build this many layers only (profiler captures; the result is not a benchmark figure)")
    ap.add_argument("--decode-steps", type=int, default=256, help="bitnet3b_*: decode steps timed (256 is the workload's own)")
    args = ap.parse_args()
    if args.streams is None:
        args.streams = 2 if args.workload == "prefill_gemm" else 1
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
