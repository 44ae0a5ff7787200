"""Benchmark of the int64 fixed-point hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the hot path over one batch of
seeded synthetic input.  `value` is measured with the inputs resident in HBM; `e2e` is
the same metric through the drop-in kernel module with host buffers (pinned host ->
device copy of the step's input and device -> host copy of its result inside the timed
region).  `roofline` describes the dominant kernel, timed live with CUDA events on its
own stream; `cpu_baseline` is the CPU oracle (an OpenMP int128 restatement of the
reference's CUDA kernels, which have no CPU implementation of their own) timed on the
host cores on a bounded sample of the same workload.

--impl reference runs that CPU restatement alone, on all host threads, and prints the
same line shape with "impl": "reference".
"""
import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "zk-deepseek_b200"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
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
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------

class PipelinedIO:
    """End-to-end steps with host buffers: every step copies its input from pinned host memory to the device
    and its result back, but on copy streams of their own, so the input copy of step k + 1 and the result
    copy of step k - 1 overlap the kernels of step k (two device input buffers, two pinned result buffers).
    All of it lies inside the timed region; the timed loop ends with a device-wide synchronisation."""

    def __init__(self, torch, x_dev, out_shape):
        self.torch = torch
        self.x_host = x_dev.cpu().pin_memory()
        self.x_in = [torch.empty_like(x_dev) for _ in range(2)]
        self.out_host = [torch.empty(out_shape, dtype=torch.int64).pin_memory() for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.ready = [None, None]          # input buffer b holds step data (event of its copy)
        self.free = [None, None]           # the kernels that read input buffer b have finished
        self.drained = [None, None]        # result buffer b has been copied out
        self.k = 0

    def _load(self, b):
        torch = self.torch
        with torch.cuda.stream(self.s_in):
            if self.free[b] is not None:
                self.s_in.wait_event(self.free[b])
            self.x_in[b].copy_(self.x_host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.s_in)
        self.ready[b] = ev

    INLINE = False      # True: both copies on the compute stream, before and after the step's kernels

    def step(self, fn):
        torch = self.torch
        b = self.k & 1
        main = torch.cuda.current_stream()
        if self.INLINE:
            self.x_in[0].copy_(self.x_host, non_blocking=True)
            out = fn(self.x_in[0])
            self.out_host[0].copy_(out, non_blocking=True)
            return out
        if self.ready[b] is None:
            self._load(b)                  # first step: nothing was prefetched
        self._load(b ^ 1)                  # the next step's input, while this step computes
        main.wait_event(self.ready[b])
        self.ready[b] = None
        out = fn(self.x_in[b])
        done = torch.cuda.Event()
        done.record(main)
        self.free[b] = done
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            self.out_host[b].copy_(out, non_blocking=True)
        out.record_stream(self.s_out)
        self.k += 1
        return out


class GemmWorkload:
    """One bit-exact int64 GEMM of a large dense projection (the `wo` shape of the MLA block,
    inference/model.py:722): X int64 [4096, 16384] uniform in +-2^20, W int32 [7168, 16384]
    uniform in +-2^15, Y = (X W^T) >> 16 with a 128-bit sum.  Each rank runs its own batch of
    4096 tokens (weak scaling, no collective on the path)."""
    name = "gemm_wo_4096x16384x7168"
    metric = "int64_gemm_gops"
    unit = "Gop/s"
    M, K, N, SHIFT = 4096, 16384, 7168, 16
    A_BITS, W_BITS, A_LIMBS = 20, 15, 3

    def __init__(self, torch, k, dev, rank):
        import numpy as np
        self.torch, self.k, self.dev, self.np = torch, k, dev, np
        g = torch.Generator().manual_seed(1000 + rank)
        self.X_host = torch.randint(-2**self.A_BITS, 2**self.A_BITS, (1, self.M, self.K),
                                    generator=g, dtype=torch.int64).pin_memory()
        gw = torch.Generator().manual_seed(7)
        self.W_host = torch.randint(-2**self.W_BITS, 2**self.W_BITS, (self.N, self.K), generator=gw,
                                    dtype=torch.int32)
        self.X = self.X_host.to(dev)
        self.W = self.W_host.to(dev)
        self.planes = k.WeightPlanes(self.W)          # static weights: split once
        self.a_limbs = self.A_LIMBS                    # |x| < 2^20 fits three signed 8-bit limbs
        self.C_host = torch.empty((1, self.M, self.N), dtype=torch.int64).pin_memory()
        self.X_dev2 = torch.empty_like(self.X)
        self.ops = 2.0 * self.M * self.N * self.K
        self.launches_per_step = 2                     # limb split of X + tensor-core kernel
        self.units = self.ops

    def config(self):
        return {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shift": self.SHIFT,
                "x_range": "+-2^%d" % self.A_BITS, "w_range": "+-2^%d int32" % self.W_BITS, "a_limbs": self.a_limbs,
                "w_limbs": self.planes.limbs, "weights": "limb planes prepared once",
                "l2": "inputs larger than L2 (X 537 MB, W planes %d MB)"
                      % (self.planes.limbs * self.N * self.K >> 20)}

    def step(self):
        return self.k.linear_prepared(self.X, self.planes, self.SHIFT, a_limbs=self.a_limbs)

    def step_e2e(self):
        self.X_dev2.copy_(self.X_host, non_blocking=True)
        C = self.k.linear_prepared(self.X_dev2, self.planes, self.SHIFT, a_limbs=self.a_limbs)
        self.C_host.copy_(C, non_blocking=True)
        return C

    def e2e_bytes(self):
        return self.X_host.numel() * 8, self.C_host.numel() * 8

    def value(self, seconds_per_step, world):
        return self.ops * world / seconds_per_step / 1e9

    def roofline(self, peaks):
        k = self.k
        k.kernel_timing(True)
        times = []
        for _ in range(8):
            self.step()
            times.append(k.last_kernel_ms())
        k.kernel_timing(False)
        kernel_ms = statistics.mean(times)
        int8_peak = 2.0 * peaks["bf16_tflops"]         # int8 tcgen05 rate is twice the bf16 rate
        pairs = self.a_limbs * self.planes.limbs
        achieved = pairs * self.ops / (kernel_ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "limb_gemm_kernel", "achieved": round(achieved, 1),
                "peak": round(int8_peak, 1), "unit": "TFLOP/s", "frac": round(achieved / int8_peak, 4),
                "traffic": None, "kernel_ms": round(kernel_ms, 4), "limb_pairs": pairs,
                "note": "int8 tensor ops = limb pairs x 2MNK; peak = 2 x cuBLAS bf16 burst (%s)"
                        % peaks["source"]}

    def check(self, orc):
        """bit-exact against the CPU oracle on a row sample"""
        C = self.step()[0, :8].cpu().numpy()
        want, _ = orc.gemm(self.X_host[:, :8].numpy(), self.W_host.numpy(), 1, 1, self.SHIFT)
        return int((C != want[0]).sum())

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """the same GEMM on a bounded row sample; returns (Gop/s, description)"""
        K, N = GemmWorkload.K, GemmWorkload.N
        rng = np.random.default_rng(7)
        W = rng.integers(-2**15, 2**15, (N, K), dtype=np.int64).astype(np.int32)
        X = rng.integers(-2**20, 2**20, (1, 4, K), dtype=np.int64)
        t0 = time.time()
        orc.gemm(X, W, 1, 1, 16)
        per_row = (time.time() - t0) / 4
        rows = int(max(4, min(4096, seconds / max(per_row, 1e-6))))
        X = rng.integers(-2**20, 2**20, (1, rows, K), dtype=np.int64)
        t0 = time.time()
        orc.gemm(X, W, 1, 1, 16)
        dt = time.time() - t0
        return 2.0 * rows * N * K / dt / 1e9, "%d of 4096 rows of X against the full W" % rows, dt


def graph_call_us(torch, fn, calls, reps=10):
    """GPU time of one call of `fn` in microseconds with no host in the way: `calls` consecutive calls are
    captured in a CUDA graph on a side stream and the graph is replayed `reps` times between two events."""
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            fn()
        st.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=st):
            for _ in range(calls):
                fn()
        gr.replay()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(reps):
            gr.replay()
        e1.record(st)
        st.synchronize()
    return e0.elapsed_time(e1) / (calls * reps) * 1e3


class GemmSmallMWorkload:
    """BASELINE's first configuration, the one the reference can run on a CPU: one bit-exact int64 GEMM of
    the wkv_a projection shape, X int64 [32, 7168] uniform in +-2^20, W [576, 7168] uniform in +-2^15 (held as
    int64 and as int32), Y = (X W^T) >> 16, seed 0.  HBM bound: the weight is read once per call, so the
    workload rotates over COPIES of W (together larger than L2) and every call streams its weight from HBM.
    A step is COPIES calls through prepared limb planes (the product path of Linear_int)."""
    name = "gemm_32x7168x576_small_m"
    metric = "int64_gemm_gops"
    unit = "Gop/s"
    M, K, N, SHIFT, COPIES = 32, 7168, 576, 16, 16

    def __init__(self, torch, k, dev, rank):
        import numpy as np
        self.torch, self.k, self.dev, self.np = torch, k, dev, np
        rng = np.random.default_rng(0)
        self.X_np = rng.integers(-2**20, 2**20, (1, self.M, self.K), dtype=np.int64)
        self.W_np = rng.integers(-2**15, 2**15, (self.N, self.K), dtype=np.int64)
        self.X = torch.from_numpy(self.X_np).to(dev)
        w64 = torch.from_numpy(self.W_np).to(dev)
        # the copies differ (rolled rows) so that nothing can be reused between calls
        self.W64 = [torch.roll(w64, i, 0).contiguous() for i in range(self.COPIES)]
        self.W32 = [w.to(torch.int32) for w in self.W64]
        self.planes = [k.WeightPlanes(w) for w in self.W32]
        self.a_limbs = 3
        self.i = 0
        self.ops = 2.0 * self.M * self.N * self.K
        self.launches_per_step = 2 * self.COPIES
        self.units = self.ops * self.COPIES
        self.X_host = self.X.cpu().pin_memory()
        self.X_in = torch.empty_like(self.X)
        self.C_host = torch.empty((1, self.M, self.N), dtype=torch.int64).pin_memory()

    def config(self):
        return {"workload": self.name, "M": self.M, "K": self.K, "N": self.N, "shift": self.SHIFT,
                "x_range": "+-2^20", "w_range": "+-2^15", "a_limbs": self.a_limbs, "w_limbs": self.planes[0].limbs,
                "calls_per_step": self.COPIES,
                "l2": "%d copies of W (%d MB of int64, %d MB of limb planes) rotate, more than L2 holds"
                      % (self.COPIES, self.COPIES * self.N * self.K * 8 >> 20,
                         self.COPIES * self.N * self.K * self.planes[0].limbs >> 20)}

    def _prepared(self):
        self.i = (self.i + 1) % self.COPIES
        return self.k.linear_prepared(self.X, self.planes[self.i], self.SHIFT, a_limbs=self.a_limbs, dynamic=True)

    def _legacy(self, ws):
        self.i = (self.i + 1) % self.COPIES
        return self.k.int64_bmm_broadcast(self.X, ws[self.i], 1, 1, self.SHIFT)

    def step(self):
        for _ in range(self.COPIES):
            out = self._prepared()
        return out

    def step_e2e(self):
        for _ in range(self.COPIES):
            self.X_in.copy_(self.X_host, non_blocking=True)
            self.i = (self.i + 1) % self.COPIES
            C = self.k.linear_prepared(self.X_in, self.planes[self.i], self.SHIFT, a_limbs=self.a_limbs, dynamic=True)
            self.C_host.copy_(C, non_blocking=True)

    def e2e_bytes(self):
        return self.COPIES * self.X_host.numel() * 8, self.COPIES * self.C_host.numel() * 8

    def value(self, seconds_per_step, world):
        return self.units * world / seconds_per_step / 1e9

    def paths(self, peaks):
        """GPU microseconds per call of the three ways this GEMM is reached, and what that is of the HBM
        roofline on the algorithmic bytes 8MK + wNK + 16MN (C and R written)"""
        torch, k = self.torch, self.k
        out = {}
        M, K, N = self.M, self.K, self.N

        def alg(w):
            return 8 * M * K + w * N * K + 16 * M * N

        us = graph_call_us(torch, self._prepared, self.COPIES)
        L = self.planes[0].limbs
        out["prepared_planes"] = {"us": round(us, 2), "bytes_read_by_the_kernels": 8 * M * K + (3 * M + L * N) * K,
                                  "GB/s_algorithmic_int32_W": round(alg(4) / us / 1e3, 1),
                                  "frac_of_hbm_algorithmic_int32_W": round(alg(4) / us / 1e3 / peaks["hbm_gbs"], 3)}
        for name, ws, w in (("legacy_symbol_int32_W", self.W32, 4), ("legacy_symbol_int64_W", self.W64, 8)):
            for _ in range(3):
                self._legacy(ws)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(2 * self.COPIES):
                self._legacy(ws)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / (2 * self.COPIES) * 1e3
            out[name] = {"us": round(us, 2), "GB/s_algorithmic": round(alg(w) / us / 1e3, 1),
                         "frac_of_hbm_algorithmic": round(alg(w) / us / 1e3 / peaks["hbm_gbs"], 3),
                         "note": "measures both operand ranges (a host synchronisation) and splits W on every call"}
        return out

    def roofline(self, peaks):
        paths = self.paths(peaks)
        pp = paths["prepared_planes"]
        alg = 8 * self.M * self.K + 4 * self.N * self.K + 16 * self.M * self.N
        gbs = alg / pp["us"] / 1e3
        return {"bound": "hbm", "kernel": "split_rows_kernel + limb_gemm_kernel (split over K)",
                "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": 15200000, "kernel_us": pp["us"],
                "traffic_note": "ncu dram__bytes_read + dram__bytes_write of one call: 13.3 MB tensor-core kernel "
                                "(weight and activation planes) + 1.9 MB activation split; the outputs stay in L2",
                "algorithmic_bytes": alg, "paths": paths,
                "note": "algorithmic bytes = 8MK + 4NK + 16MN (int32 W) / GPU time of one call replayed from a CUDA "
                        "graph (activation split + tensor-core kernel); the kernels read %d-limb planes of W, "
                        "fewer bytes than the int32 weight; peak = STREAM-style copy (%s)"
                        % (self.planes[0].limbs, peaks["source"])}

    def check(self, orc):
        C, R = self.k.linear_prepared(self.X, self.planes[0], self.SHIFT, a_limbs=self.a_limbs, want_remainder=True,
                                      dynamic=True)
        Co, Ro = orc.gemm(self.X_np, self.W_np, 1, 1, self.SHIFT, orc.R_LEGACY)
        bad = int((C.cpu().numpy() != Co).sum()) + int((R.cpu().numpy() != Ro).sum())
        C, R = self.k.int64_bmm_broadcast(self.X, self.W64[0], 1, 1, self.SHIFT)
        return bad + int((C.cpu().numpy() != Co).sum()) + int((R.cpu().numpy() != Ro).sum())

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """the whole GEMM (it is small) on the int128 oracle, repeated"""
        rng = np.random.default_rng(0)
        X = rng.integers(-2**20, 2**20, (1, 32, 7168), dtype=np.int64)
        W = rng.integers(-2**15, 2**15, (576, 7168), dtype=np.int64)
        orc.gemm(X, W, 1, 1, 16)
        n, t0 = 0, time.time()
        while time.time() - t0 < min(seconds, 3.0):
            orc.gemm(X, W, 1, 1, 16)
            n += 1
        dt = (time.time() - t0) / n
        return 2.0 * 32 * 576 * 7168 / dt / 1e9, "the full 32 x 7168 x 576 GEMM, %d repetitions" % n, dt * n


def torch_cpu_baseline(torch, np, seconds=3.0):
    """The reference's own CPU path for a Linear: torch.nn.functional.linear on int64 tensors (linear() takes
    that branch for every non-fp8 weight, inference/model.py:179-181) followed by >> s, on BASELINE's first
    configuration, where it is valid because |sum| < 2^42 stays inside the wrapping int64."""
    rng = np.random.default_rng(0)
    X = torch.from_numpy(rng.integers(-2**20, 2**20, (1, 32, 7168), dtype=np.int64))
    W = torch.from_numpy(rng.integers(-2**15, 2**15, (576, 7168), dtype=np.int64))
    torch.nn.functional.linear(X, W)
    n, t0 = 0, time.time()
    while time.time() - t0 < seconds:
        Y = torch.nn.functional.linear(X, W) >> 16
        n += 1
    dt = (time.time() - t0) / n
    return {"value": round(2.0 * 32 * 576 * 7168 / dt / 1e9, 3), "unit": "Gop/s", "ms_per_call": round(dt * 1e3, 3),
            "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(), "kind": "reference",
            "sample": "torch.nn.functional.linear(X, W) >> 16 on int64 CPU tensors, 32 x 7168 x 576, %d calls" % n,
            "checksum": int(Y.sum().item())}


class ChainWorkload:
    """Fixed-point nonlinearity chain on one MLA block's activations (T = 2048 tokens):
    RMSNorm over x int64 [T, 7168] ~ N(0, 2^16) with int32 weight near 2^16; RoPE on q_pe
    [1, T, 128, 64] with a 2^42-scaled cos/sin table (base 10000); Q19 softmax over scores
    [1, T, 128, T] ~ N(0, 4*2^16) with the causal mask -(64<<36) added; Q23 SiLU over
    [1, T, 18432] ~ N(0, 2^16).  Four kernel launches per step, each an HBM stream."""
    name = "fixedpoint_chain_T2048"
    metric = "fixedpoint_chain_tokens_per_s"
    unit = "tokens/s"
    T, DIM, H, ROPE, INTER = 2048, 7168, 128, 64, 18432

    def __init__(self, torch, k, dev, rank, T=None):
        import numpy as np
        if T:
            self.T = T
        self.torch, self.k, self.dev, self.np = torch, k, dev, np
        T = self.T
        g = torch.Generator(device=dev).manual_seed(2000 + rank)

        def normal(shape, scale):
            return torch.round(torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
                               * scale).to(torch.int64)

        self.x = normal((T, self.DIM), 2.0**16)
        self.w = (2**16 + normal((self.DIM,), 2.0**8)).to(torch.int32)
        self.q_pe = normal((1, T, self.H, self.ROPE // 2, 2), 2.0**16)
        freqs = 1.0 / (10000.0 ** (np.arange(0, self.ROPE, 2, dtype=np.float64) / self.ROPE))
        ang = np.outer(np.arange(T), freqs)
        tab = np.stack([np.rint(np.cos(ang) * 2.0**42), np.rint(np.sin(ang) * 2.0**42)], -1)
        self.table = torch.from_numpy(tab.astype(np.int64)).to(dev).view(1, T, 1, self.ROPE // 2, 2)
        self.scores = normal((1, T, self.H, T), 4 * 2.0**16)
        self.scores += torch.full((T, T), -(64 << 36), dtype=torch.int64, device=dev).triu_(1)[:, None, :]
        self.act = normal((1, T, self.INTER), 2.0**16)
        self.probs = torch.empty_like(self.scores)
        self.act_out = torch.empty_like(self.act)
        k.softmax_init_q19()
        k.silu_init_q23()
        k.SOFTMAX_WRITES_WEIGHTS = False      # keep the scores intact from step to step
        self.bytes = {"rmsnorm": 16 * self.x.numel() + 4 * self.DIM,
                      "rope": 16 * self.q_pe.numel() + 8 * self.table.numel(),
                      "softmax": 16 * self.scores.numel(), "silu": 16 * self.act.numel()}
        self.launches_per_step = 4
        self.host = None

    def config(self):
        return {"workload": self.name, "tokens": self.T, "rmsnorm": [self.T, self.DIM],
                "rope": [1, self.T, self.H, self.ROPE], "softmax": [1, self.T, self.H, self.T],
                "silu": [1, self.T, self.INTER], "rope_shift": 42, "softmax_frac": 19, "silu_frac": 23,
                "l2": "every tensor is larger than L2 (117 MB to 4.3 GB)"}

    def step(self):
        k = self.k
        n, _ = k.rms_norm_int64_device(self.x, self.w, 1, self.DIM)
        r = k.complex_int64_mul_broadcast(self.q_pe, self.table)
        k.softmax_q19(self.scores, self.probs)
        k.silu_q23(self.act, self.act_out)
        return n, r

    def time_parts(self, reps=5):
        """CUDA-event duration of each kernel on the launching stream (average of reps)"""
        torch, k = self.torch, self.k
        out = {}
        calls = {"rmsnorm": lambda: k.rms_norm_int64_device(self.x, self.w, 1, self.DIM),
                 "rope": lambda: k.complex_int64_mul_broadcast(self.q_pe, self.table),
                 "softmax": lambda: k.softmax_q19(self.scores, self.probs),
                 "silu": lambda: k.silu_q23(self.act, self.act_out)}
        for name, fn in calls.items():
            fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            out[name] = e0.elapsed_time(e1) / reps
        return out

    def step_e2e(self):
        torch = self.torch
        if self.host is None:
            self.host = {n: getattr(self, n).cpu().pin_memory() for n in ("x", "q_pe", "scores", "act")}
            self.dev_in = {n: torch.empty_like(getattr(self, n)) for n in self.host}
            self.host_out = {n: torch.empty_like(t).pin_memory() for n, t in self.host.items()}
        for n, h in self.host.items():
            self.dev_in[n].copy_(h, non_blocking=True)
        k = self.k
        nrm, _ = k.rms_norm_int64_device(self.dev_in["x"], self.w, 1, self.DIM)
        rot = k.complex_int64_mul_broadcast(self.dev_in["q_pe"], self.table)
        k.softmax_q19(self.dev_in["scores"], self.probs)
        k.silu_q23(self.dev_in["act"], self.act_out)
        self.host_out["x"].copy_(nrm, non_blocking=True)
        self.host_out["q_pe"].copy_(rot, non_blocking=True)
        self.host_out["scores"].copy_(self.probs, non_blocking=True)
        self.host_out["act"].copy_(self.act_out, non_blocking=True)

    def e2e_bytes(self):
        n = 8 * (self.x.numel() + self.q_pe.numel() + self.scores.numel() + self.act.numel())
        return n, n

    def value(self, seconds_per_step, world):
        return self.T * world / seconds_per_step

    def roofline(self, peaks):
        parts = self.time_parts()
        gbs = {n: self.bytes[n] / (ms * 1e-3) / 1e9 for n, ms in parts.items()}
        dom = "softmax"
        return {"bound": "hbm", "kernel": "softmax_kernel<19>", "achieved": round(gbs[dom], 1),
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs[dom] / peaks["hbm_gbs"], 4),
                "traffic": None, "kernel_ms": round(parts[dom], 4),
                "parts": {n: {"ms": round(parts[n], 4), "GB/s": round(gbs[n], 1),
                              "frac": round(gbs[n] / peaks["hbm_gbs"], 4),
                              "algorithmic_bytes": self.bytes[n]} for n in parts},
                "note": "algorithmic bytes = 8 B read + 8 B written per element (+ weights/table); "
                        "peak = STREAM-style copy (%s)" % peaks["source"]}

    def check(self, orc):
        """bit-exact against the CPU oracle on slices of every tensor"""
        k, bad = self.k, 0
        nrm, rot = self.step()
        want, _ = orc.rms_norm(self.x[:16].cpu().numpy(), self.w.cpu().numpy(), 1, self.DIM)
        bad += int((nrm[:16].cpu().numpy() != want).sum())
        want = orc.rope(self.q_pe[:, :8].cpu().numpy(), self.table.view(self.T, -1, 2)[:8].cpu().numpy(), 42)
        bad += int((rot[:, :8].cpu().numpy() != want).sum())
        sl = slice(self.T - 2, self.T)
        bad += int((self.probs[:, sl].cpu().numpy() != orc.softmax(self.scores[:, sl].cpu().numpy(), 19)).sum())
        bad += int((self.act_out[:, :4].cpu().numpy() != orc.act(self.act[:, :4].cpu().numpy(), "silu", 23)).sum())
        return bad

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """the chain on a bounded token sample (softmax rows stay 2048 long)"""
        T, rows = ChainWorkload.T, 8
        rng = np.random.default_rng(3)
        while True:
            x = np.rint(rng.standard_normal((rows, 7168)) * 2**16).astype(np.int64)
            w = (2**16 + np.rint(rng.standard_normal(7168) * 2**8)).astype(np.int32)
            q = np.rint(rng.standard_normal((1, rows, 128, 32, 2)) * 2**16).astype(np.int64)
            tab = np.rint(rng.uniform(-1, 1, (rows, 32, 2)) * 2**42).astype(np.int64)
            sc = np.rint(rng.standard_normal((1, rows, 128, T)) * 4 * 2**16).astype(np.int64)
            a = np.rint(rng.standard_normal((1, rows, 18432)) * 2**16).astype(np.int64)
            t0 = time.time()
            orc.rms_norm(x, w, 1, 7168)
            orc.rope(q, tab, 42)
            orc.softmax(sc, 19)
            orc.act(a, "silu", 23)
            dt = time.time() - t0
            if dt > seconds / 4 or rows >= 256:
                return rows / dt, "%d of %d tokens through all four kernels" % (rows, T), dt
            rows = min(256, int(rows * max(2.0, 0.8 * seconds / max(dt, 1e-3))))


def _normal_i(torch, gen, shape, scale, dev, dtype):
    """round(N(0,1) * scale) generated on the device in chunks (seeded generator)"""
    out = torch.empty(shape, dtype=dtype, device=dev)
    flat = out.view(-1)
    step = 1 << 26
    for i in range(0, flat.numel(), step):
        n = min(step, flat.numel() - i)
        flat[i:i + n] = torch.round(torch.randn(n, generator=gen, device=dev) * scale).to(dtype)
    return out


class MlaWorkload:
    """One DeepSeek-V3 MLA attention layer in int64 fixed point, prefill of 4096 tokens
    (dim 7168, q_lora 1536, kv_lora 512, 128 heads, nope 128, rope 64, v 128; MLA.forward of
    inference/model.py:747-957).  Hidden states ~ N(0, 2^16), int32 weights ~ N(0, 2^16/sqrt(fan_in)),
    norm weights near 2^16, every runtime shift 16 (the layer's fixed-point scale); the shifts the
    reference hard-codes stay (scores 23 / 21, RoPE 42, softmax Q19).  `scales="reference"` uses the
    reference's magnitudes instead (activations 2^21, weights 2^30/sqrt(fan_in), shifts 29-31).
    With N GPUs every rank holds 4096 / N consecutive tokens: the down projections, norms and wo run on the
    local tokens, the attention core on all tokens for 128 / N heads, with one all-gather of the normed
    latents and one all-to-all of the attention output between the two layouts (MLA.seq_parallel): strong
    scaling of the same 4096 tokens, input and output distributed over the ranks."""
    name = "mla_layer_prefill_4096"
    metric = "int64_mla_layer_tokens_per_s"
    e2e_note = ("pinned host -> device copy of every step's input and device -> host copy of its result on copy "
                "streams: they overlap the kernels of the neighbouring steps (two buffers each way)")
    unit = "tokens/s"
    scaling = "strong"
    collective_check = True
    T = 4096
    SCALES = "baseline"

    def __init__(self, torch, k, dev, rank, T=None, scales="baseline"):
        import numpy as np
        self.torch, self.k, self.dev, self.np, self.rank = torch, k, dev, np, rank
        if T:
            self.T = T
        M = importlib.import_module(PKG + ".model")
        self.M = M
        import torch.distributed as dist
        M.world_size = dist.get_world_size() if dist.is_initialized() else 1
        M.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = M.world_size
        a = M.ModelArgs(max_seq_len=self.T, vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048,
                        n_layers=61, n_dense_layers=3, n_heads=128, n_routed_experts=256, n_shared_experts=1,
                        n_activated_experts=8, n_expert_groups=8, n_limited_groups=4, score_func="sigmoid",
                        route_scale=2.5, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                        qk_rope_head_dim=64, v_head_dim=128)
        self.args = a
        self.scales = scales
        if scales == "baseline":
            xs, wb, nb, shift, self.act_limbs, self.score_limbs = 16, 16, 16, 16, 3, (3, 3)
        else:
            # |q| and |kv| stay below 2^31 at these magnitudes (2^19 and 2^23 fixed-point scales): four limbs each,
            # promised; the split passes verify it on the device and k.device_status() would report a miss
            xs, wb, nb, shift, self.act_limbs, self.score_limbs = 21, 30, 19, 30, 4, (4, 4)
        self.shift = shift
        with torch.device(dev):
            attn = M.MLA(0, a, seq_parallel=self.world > 1)
        g = torch.Generator(device=dev).manual_seed(5)          # same weights on every rank
        H, Hl = a.n_heads, a.n_heads // self.world
        r = M.rank

        def weight(out_f, in_f, rows=None):
            w = _normal_i(torch, g, (out_f, in_f), 2.0**wb / math.sqrt(in_f), dev, torch.int32)
            return w if rows is None else w[rows[0]:rows[1]].contiguous()

        def norm_weight(n):
            return (2**nb + _normal_i(torch, g, (n,), 2.0**(nb - 8), dev, torch.int64)).to(torch.int32)

        heads = lambda d: (r * Hl * d, (r + 1) * Hl * d)
        attn.wq_a.weight = weight(a.q_lora_rank, a.dim)
        attn.q_norm.weight = norm_weight(a.q_lora_rank)
        attn.wq_b1.weight = weight(H * a.qk_nope_head_dim, a.q_lora_rank, heads(a.qk_nope_head_dim))
        attn.wq_b2.weight = weight(H * a.qk_rope_head_dim, a.q_lora_rank, heads(a.qk_rope_head_dim))
        attn.wkv_a1.weight = weight(a.kv_lora_rank, a.dim)
        attn.wkv_a2.weight = weight(a.qk_rope_head_dim, a.dim)
        attn.kv_norm.weight = norm_weight(a.kv_lora_rank)
        attn.wkv_b_1.weight = weight(H * a.qk_nope_head_dim, a.kv_lora_rank, heads(a.qk_nope_head_dim))
        attn.wkv_b_2.weight = weight(H * a.v_head_dim, a.kv_lora_rank, heads(a.v_head_dim))
        attn.wo.weight = weight(a.dim, H * a.v_head_dim)        # whole on every rank: wo runs on the rank's tokens
        for lin in (attn.wq_a, attn.wq_b1, attn.wq_b2, attn.wkv_a1, attn.wkv_a2):
            lin.res_rescale = shift if scales == "baseline" else lin.res_rescale
        for lin in (attn.wkv_b_1, attn.wkv_b_2, attn.wo):
            lin.scale = torch.tensor(shift, dtype=torch.int32, device=dev)
        attn.score_limbs = self.score_limbs
        self.attn = attn
        gx = torch.Generator(device=dev).manual_seed(55)
        x_all = _normal_i(torch, gx, (1, self.T, a.dim), 2.0**xs, dev, torch.int64)
        # N > 1: every rank holds T / N consecutive tokens (input and output), see MLA.seq_parallel
        self.T_local = self.T // self.world
        self.x = x_all[:, r * self.T_local:(r + 1) * self.T_local].contiguous() if self.world > 1 else x_all
        del x_all
        self.freqs = M.precompute_freqs_cis(a).to(dev)
        self.mask = torch.full((self.T, self.T), -(64 << 36), dtype=torch.int64, device=dev).triu_(1)
        self.mask._zkds_causal = True
        M.ACT_LIMBS = self.act_limbs
        k.softmax_init_q19()
        k.SOFTMAX_WRITES_WEIGHTS = False
        self.x_host = None
        T, D, C, R = self.T, a.dim, a.kv_lora_rank, a.qk_rope_head_dim
        nope, v, q = a.qk_nope_head_dim, a.v_head_dim, a.q_lora_rank
        self.ops = 2.0 * T * (D * q + q * H * (nope + R) + D * (C + R) + H * nope * C + H * T * (C + R)
                              + H * T * C + H * C * v + H * v * D)
        self.launches_per_step = 0

    @classmethod
    def static_config(cls, world, scales=None, T=None):
        """the configuration record of this workload; needs no GPU (the reference arm prints the same one)"""
        T = T or cls.T
        scales = scales or cls.SCALES
        D, q, C, R, H, nope, v = 7168, 1536, 512, 64, 128, 128, 128
        ops = 2.0 * T * (D * q + q * H * (nope + R) + D * (C + R) + H * nope * C + H * T * (C + R)
                         + H * T * C + H * C * v + H * v * D)
        base = scales == "baseline"
        return {"workload": cls.name, "tokens": T, "dim": D, "heads": H, "q_lora": q, "kv_lora": C, "scales": scales,
                "shift": 16 if base else 30, "act_limbs_bound": 3 if base else 4,
                "score_limbs_bound": [3, 3] if base else [4, 4], "heads_per_gpu": H // world,
                "useful_ops_per_step": ops, "l2": "activations and score tensors (up to 17 GB) far exceed L2"}

    def config(self):
        return self.static_config(self.world, self.scales, self.T)

    def step(self):
        return self.attn(self.x, 0, self.freqs, self.mask)

    def step_e2e(self):
        torch = self.torch
        if self.x_host is None:
            self.x_host = PipelinedIO(torch, self.x, (1, self.T_local, self.args.dim))
        self.x_host.step(lambda x: self.attn(x, 0, self.freqs, self.mask))

    def e2e_bytes(self):
        n = 8 * self.T * self.args.dim            # over all ranks: each copies its T / N tokens in and out
        return n, n

    def value(self, seconds_per_step, world):
        return self.T / seconds_per_step          # the same 4096 tokens on every N

    def roofline(self, peaks):
        k = self.k
        k.kernel_timing(2)
        self.step()
        self.torch.cuda.synchronize()
        ms, ops, n = k.kernel_timing_totals()
        k.kernel_timing(False)
        # per step: n tensor-core launches, a limb split of A for each, a split of the three
        # un-prepared B operands (kv / pe caches), 2 RMSNorm, 2 RoPE, 1 softmax
        self.launches_per_step = 2 * n + 3 + 5
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        achieved = ops / (ms * 1e-3) / 1e12
        # DRAM bytes of the step's largest launch, the fused score kernel: dram__bytes_read + dram__bytes_write of
        # one ncu capture of the 1024-token case (1.413 GB per launch), scaled by (T / 1024)^2 like its output
        H = self.args.n_heads // self.world
        traffic = 1.4128e9 * (self.T / 1024.0) ** 2 * (H / 128.0)
        alg = 8.0 * self.T * H * self.T + 3.0 * 576 * (self.T * H + self.T)
        return {"bound": "tensor", "kernel": "limb_gemm_kernel (%d launches per step)" % n,
                "achieved": round(achieved, 1), "peak": round(int8_peak, 1), "unit": "TFLOP/s",
                "frac": round(achieved / int8_peak, 4), "traffic": round(traffic), "kernel_ms": round(ms, 3),
                "traffic_note": "fused score launch, DRAM read + write scaled from an ncu capture at 1024 tokens; its "
                                "algorithmic bytes (scores written once, limb planes read once) are %d" % round(alg),
                "int8_ops_per_step": ops,
                "note": "sum over the step's tensor-core launches of limb pairs x 2MNK / sum of their CUDA-event "
                        "durations; peak = 2 x sustained cuBLAS bf16 (%s)" % peaks["source"]}

    def check(self, orc):
        """Rows of the ACTUAL T-token pass against the numpy restatement of MLA.forward: three groups of four
        consecutive query tokens (first, middle, last) x every head, each against the whole cache before it.
        The oracle takes the cache rows before a group from the GPU (it recomputes and compares the group's
        own rows and 16 rows elsewhere), so every contraction of the full-extent run is covered: the 2^31-word
        score tensor, the last column tiles, K = T in P.KV."""
        np, torch, a = self.np, self.torch, self.args
        at, T = self.attn, self.T
        got = self.step()                       # with N > 1 every rank joins the collectives here
        x_all = self.x
        if self.world > 1:                      # token blocks of the ranks -> the whole input and output
            import torch.distributed as dist
            full = torch.empty((T, a.dim), dtype=torch.int64, device=self.dev)
            dist.all_gather_into_tensor(full, got[0].contiguous())
            got = full[None]
            x_all = torch.empty((1, T, a.dim), dtype=torch.int64, device=self.dev)
            dist.all_gather_into_tensor(x_all[0], self.x[0].contiguous())
        kv_gpu = at.kv_cache[0, :T].cpu().numpy()
        pe_gpu = at.pe_cache[0, :T].cpu().numpy()

        def full(name):          # head / column slices of the ranks -> the whole weight
            w = getattr(at, name).weight
            if self.world == 1 or name in ("wq_a", "wkv_a1", "wkv_a2", "q_norm", "kv_norm", "wo"):
                return w.cpu().numpy()
            import torch.distributed as dist
            parts = [torch.empty_like(w) for _ in range(self.world)]
            dist.all_gather(parts, w.contiguous())
            return torch.cat(parts, 0).cpu().numpy()

        p = {n: full(n) for n in
             ("wq_a", "wq_b1", "wq_b2", "wkv_a1", "wkv_a2", "wkv_b_1", "wkv_b_2", "wo", "q_norm", "kv_norm")}
        if orc is None:
            return None
        from oracle import model_oracle as mo
        p.update(wkv_b_1_scale=self.shift, wkv_b_2_scale=self.shift, wo_scale=self.shift)
        sq, skv = (self.shift, self.shift) if self.scales == "baseline" else (30, 29)
        freqs = self.freqs.cpu().numpy()
        S = 4
        bad = 0
        for st in sorted({0, max(0, T // 2 - 2), max(0, T - S)}):
            end = st + S
            kv = np.zeros((1, end, a.kv_lora_rank), np.int64)
            pe = np.zeros((1, end, a.qk_rope_head_dim), np.int64)
            kv[0, :st], pe[0, :st] = kv_gpu[:st], pe_gpu[:st]
            mask = np.where(np.arange(end)[None, :] > (st + np.arange(S))[:, None], mo.MASK_VALUE, 0).astype(np.int64)
            x = x_all[:, st:end].cpu().numpy()
            want = mo.mla_forward(p, x, st, freqs[st:end], mask, kv, pe, a.n_heads, s_q=sq, s_kv=skv)
            bad += int((got[:, st:end].cpu().numpy() != want).sum())
            bad += int((kv[0, st:end] != kv_gpu[st:end]).sum()) + int((pe[0, st:end] != pe_gpu[st:end]).sum())
        rows = np.random.default_rng(9).choice(T, 16, replace=False)
        for r in rows:
            x = x_all[:, r:r + 1].cpu().numpy()
            kvr = mo.rms_norm(mo.linear(x, p["wkv_a1"], skv)[0], p["kv_norm"])[0]
            per = mo.rotary(mo.linear(x, p["wkv_a2"], skv)[0][:, :, None, :], freqs[r:r + 1])[:, :, 0]
            bad += int((kvr[0, 0] != kv_gpu[r]).sum()) + int((per[0, 0] != pe_gpu[r]).sum())
        return bad

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """the layer's contractions and softmax for a sample of query tokens (full K and T extents, operands at
        the workload's magnitudes).  The sample grows until it uses about `seconds`; tokens/s of the sample is
        what a full 4096-token pass would give, since every query token costs the same."""
        T, H = 4096, 128
        rng = np.random.default_rng(5)
        ri = lambda shape, b: np.rint(rng.standard_normal(shape) * 2.0**b).astype(np.int64)
        wi = lambda n, kk: np.rint(rng.standard_normal((n, kk)) * 2.0**16 / math.sqrt(kk)).astype(np.int32)
        ws = [wi(n, kk) for (n, kk) in ((1536, 7168), (24576, 1536), (576, 7168), (7168, 16384))]
        wh = [np.rint(rng.standard_normal((H, 128, 512)) * 2.0**16 / math.sqrt(512)).astype(np.int32) for _ in range(2)]
        kv, pe = ri((1, T, 512), 16), ri((1, T, 64), 16)

        def run(S):
            t0 = time.time()
            for w in ws:
                orc.gemm(ri((1, S, w.shape[1]), 16), w, 1, 1, 16)
            sc = orc.einsum_bshc_btc_bsht(ri((1, S, H, 512), 16), kv, 23) + \
                orc.einsum_bshc_btc_bsht(ri((1, S, H, 64), 16), pe, 21)
            pr = orc.softmax(sc * 94 // 695, 19)
            ctx = orc.einsum_bsht_btc_bshc(pr, kv, 23)
            orc.einsum_bshc_hdc_bshd(ctx, wh[0], 16)
            orc.einsum_bshd_hdc_bshc(ri((1, S, H, 128), 16), wh[1], 16)
            return time.time() - t0

        dt = run(4)
        S = int(max(4, min(64, 4 * 0.8 * seconds / max(dt, 1e-3))))
        if S > 4:
            dt = run(S)
        else:
            S = 4
        return S / dt, ("%d of 4096 query tokens against the full 4096-token cache and the full weights; "
                        "tokens/s of the sample (a 4096-token pass was not run on the CPU)" % S), dt


class MoeWorkload:
    """One DeepSeek-V3 MoE layer in int64 fixed point (MoE.forward, inference/model.py:1325-1383):
    dim 7168, 256 routed experts + 1 shared expert, moe_inter_dim 2048, sigmoid gate with top-8
    routing over 8 groups / 4 kept, route scale 2.5.  8192 tokens ~ N(0, 2^16); int32 gate,
    shared and expert weights ~ N(0, 2^16/sqrt(fan_in)); every shift 16 except the gate's, which is 9 so
    that its logits have a standard deviation of about 1.0 in Q23 (what the sigmoid reads); int32 gate bias
    >= 0 of about 0.004.  Like the trained model's balancing bias this leaves the expert load even (a bias
    that outweighs the spread of the scores would send every token to the same eight experts); the load the
    gate actually produced is reported in config.routing.
    With N GPUs the experts are split 256/N per GPU and the 8192 tokens N ways; rows travel to the
    experts' owners and back with NCCL all-to-all (strong scaling)."""
    name = "moe_layer_8192_tokens"
    metric = "int64_moe_layer_tokens_per_s"
    e2e_note = ("pinned host -> device copy of every step's input and device -> host copy of its result on copy "
                "streams: they overlap the kernels of the neighbouring steps (two buffers each way)")
    unit = "tokens/s"
    scaling = "strong"
    collective_check = True
    T, E, SHIFT, GATE_SHIFT = 8192, 256, 16, 9

    def __init__(self, torch, k, dev, rank, T=None, E=None):
        import numpy as np
        import torch.distributed as dist
        self.torch, self.k, self.dev, self.np, self.rank = torch, k, dev, np, rank
        if T:
            self.T = T
        if E:
            self.E = E
        M = importlib.import_module(PKG + ".model")
        self.M = M
        M.world_size = dist.get_world_size() if dist.is_initialized() else 1
        M.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = M.world_size
        a = M.ModelArgs(max_seq_len=64, vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048,
                        n_layers=61, n_dense_layers=3, n_heads=128, n_routed_experts=self.E,
                        n_shared_experts=1, n_activated_experts=8, n_expert_groups=8, n_limited_groups=4,
                        score_func="sigmoid", route_scale=2.5, q_lora_rank=1536, kv_lora_rank=512,
                        qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
        self.args = a
        D, I = a.dim, a.moe_inter_dim
        with torch.device(dev):
            moe = M.MoE(3, a, token_parallel=True)
        g = torch.Generator(device=dev).manual_seed(6)
        sh = self.SHIFT

        def weight(gen, out_f, in_f):
            return _normal_i(torch, gen, (out_f, in_f), 2.0**16 / math.sqrt(in_f), dev, torch.int32)

        moe.gate.weight = weight(g, self.E, D)
        moe.gate.scale = torch.tensor(self.GATE_SHIFT, dtype=torch.int32, device=dev)
        moe.gate.bias = torch.abs(_normal_i(torch, g, (self.E,), 2.0**15, dev, torch.int64)).to(torch.int32)
        for name, (o, i) in (("w1", (I, D)), ("w3", (I, D)), ("w2", (D, I))):
            lin = getattr(moe.shared_experts, name)
            lin.weight = weight(g, o, i)
            lin.scale = torch.tensor(sh, dtype=torch.int32, device=dev)
        self._weight = weight
        for j in range(moe.n_local_experts):
            w1, w3, w2 = self.expert_weights(moe.experts_start_idx + j)
            moe.experts_w13[j, :I] = w1
            moe.experts_w13[j, I:] = w3
            moe.experts_w2[j] = w2
        moe.experts_shift.fill_(sh)
        self.moe = moe
        gx = torch.Generator(device=dev).manual_seed(66)
        x_all = _normal_i(torch, gx, (self.T, D), 2.0**16, dev, torch.int64)
        self.T_local = self.T // self.world
        self.x = x_all[M.rank * self.T_local:(M.rank + 1) * self.T_local].contiguous()[None]
        del x_all
        M.ACT_LIMBS = 3
        k.silu_init_q23()
        self.x_host = None
        pairs = self.T * a.n_activated_experts
        self.ops = 2.0 * 3 * D * I * (pairs + self.T) + 2.0 * self.T * D * self.E
        self.launches_per_step = 0
        self.routing = self._expert_load()

    def _peer(self):
        """the peer-memory exchange is switched on and available to this process group"""
        par = importlib.import_module(PKG + ".parallel")
        return bool(self.world > 1 and self.M.PEER_EXPERTS and par.peer_available())

    def _expert_load(self):
        """rows per expert and per GPU that the gate produces for the whole batch (every rank's tokens)"""
        import torch.distributed as dist
        idx = self.moe.gate(0, self.x.view(-1, self.args.dim))[1]
        rows = self.torch.bincount(idx.flatten(), minlength=self.E)
        if self.world > 1:
            dist.all_reduce(rows)
        per_gpu = rows.view(self.world, -1).sum(1)
        mean_e = float(rows.sum().item()) / self.E
        return {"experts_hit": int((rows > 0).sum().item()),
                "rows_per_expert_max_over_mean": round(float(rows.max().item()) / mean_e, 3),
                "rows_per_expert_min": int(rows.min().item()),
                "rows_per_gpu_max_over_mean": round(float(per_gpu.max().item()) * self.world / float(rows.sum().item()), 3)}

    def expert_weights(self, global_id):
        """(w1, w3, w2) of one routed expert, seeded by its global id (same on every rank)"""
        D, I = self.args.dim, self.args.moe_inter_dim
        ge = self.torch.Generator(device=self.dev).manual_seed(10000 + global_id)
        return self._weight(ge, I, D), self._weight(ge, I, D), self._weight(ge, D, I)

    def config(self):
        a = self.args
        return {"workload": self.name, "tokens": self.T, "tokens_per_gpu": self.T_local, "dim": a.dim,
                "routed_experts": self.E, "experts_per_gpu": self.E // self.world, "top_k": 8,
                "moe_inter_dim": a.moe_inter_dim, "shift": self.SHIFT, "gate_shift": self.GATE_SHIFT,
                "act_limbs_bound": 3, "routing": self.routing, "useful_ops_per_step": self.ops,
                "exchange": ("none (one GPU)" if self.world == 1 else
                             "peer memory: rows read in place by the owner's limb split, results stored into the "
                             "home GPU's slots, flag barriers" if self._peer() else
                             "NCCL all-to-all of packed rows"),
                "exchange_check": getattr(self, "paths_compared", None), "weights": "resident limb planes, all experts",
                "l2": "expert weights (45 GB int32) and token rows far exceed L2"}

    def step(self):
        return self.moe(0, self.x)

    def step_e2e(self):
        torch = self.torch
        if self.x_host is None:
            self.x_host = PipelinedIO(torch, self.x, tuple(self.x.shape))
        self.x_host.step(lambda x: self.moe(0, x))

    def e2e_bytes(self):
        n = 8 * self.T_local * self.args.dim
        return n, n

    def value(self, seconds_per_step, world):
        return self.T / seconds_per_step

    def roofline(self, peaks):
        k = self.k
        k.kernel_timing(2)
        self.step()
        self.torch.cuda.synchronize()
        recs = k.kernel_timing_records()
        k.kernel_timing(False)
        pairs_local = self.T_local * 8
        if self.world > 1:
            # (token, expert) pairs whose expert this rank owns: counted over every rank's routing
            import torch.distributed as dist
            idx = self.moe.gate(0, self.x.view(-1, self.args.dim))[1]
            owners = self.torch.bincount((idx // (self.E // self.world)).flatten(), minlength=self.world)
            dist.all_reduce(owners)
            pairs_local = int(owners[self.M.rank].item())
        ms = sum(r["ms"] for r in recs)
        ops = 0.0
        for r in recs:
            rows = r["batches"] * r["M"]
            if r["grouped"] and pairs_local:
                rows = pairs_local                      # padded tiles carry no useful work
            ops += 2.0 * r["la"] * r["lb"] * rows * r["N"] * r["K"]
        self.launches_per_step = 2 * len(recs) + 3 + 12   # + gather, GLU x2, combine, sigmoid, routing ops
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        achieved = ops / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "limb_gemm_kernel (%d launches per step)" % len(recs),
                "achieved": round(achieved, 1), "peak": round(int8_peak, 1), "unit": "TFLOP/s",
                "frac": round(achieved / int8_peak, 4), "traffic": None, "kernel_ms": round(ms, 3),
                "launches": [{kk: (round(v, 3) if kk == "ms" else v) for kk, v in r.items()} for r in recs],
                "note": "limb pairs x 2 x rows x N x K of every tensor-core launch (grouped launches count the "
                        "routed rows, not the padding) / sum of CUDA-event durations; peak = 2 x sustained "
                        "cuBLAS bf16 (%s)" % peaks["source"]}

    def check(self, orc):
        """Tokens of the ACTUAL pass (all T tokens routed, so experts receive several 128-row tiles each) against
        the numpy restatement of MoE.forward: eight tokens spread over the batch, each through the gate, the
        shared expert and its eight routed experts.  The GPU's expert choice is passed on so that a score tie
        cannot make the two differ."""
        np, a, moe = self.np, self.args, self.moe
        got_all = self.step()                   # with N > 1 every rank joins the exchange here
        extra_bad = 0
        if self.world > 1 and self._peer():
            # the two exchanges must agree on every word of every rank's output
            import torch.distributed as dist
            self.M.PEER_EXPERTS = False
            try:
                other = self.step()
            finally:
                self.M.PEER_EXPERTS = True
            bad = (other != got_all).sum().to(self.torch.int64).reshape(1)
            dist.all_reduce(bad)
            extra_bad = int(bad.item())
            self.paths_compared = ("outputs of the peer-memory and the NCCL all-to-all exchange compared word for "
                                   "word on every rank: %d differ" % extra_bad)
            del other
        if orc is None:
            return None
        from oracle import model_oracle as mo
        Tl = self.T_local
        sample = sorted({0, 1, Tl // 3, Tl // 2, Tl // 2 + 1, (2 * Tl) // 3, Tl - 2, Tl - 1})
        idx_all = moe.gate(0, self.x.view(-1, a.dim))[1]
        counts = self.torch.bincount(idx_all.flatten(), minlength=self.E)
        self.max_rows_per_expert = int(counts.max().item())
        xs = self.x[:, sample].contiguous()
        got = got_all[:, sample].cpu().numpy()
        idx = idx_all[sample].cpu().numpy()
        sh = self.SHIFT
        mlp = lambda m: {"w1": m.w1.weight.cpu().numpy(), "w3": m.w3.weight.cpu().numpy(),
                         "w2": m.w2.weight.cpu().numpy(), "w1_scale": sh, "w3_scale": sh, "w2_scale": sh}
        experts = [None] * self.E
        for e in np.unique(idx):          # regenerated from the expert's seed: any rank's expert
            w1, w3, w2 = self.expert_weights(int(e))
            experts[e] = {"w1": w1.cpu().numpy(), "w3": w3.cpu().numpy(), "w2": w2.cpu().numpy(),
                          "w1_scale": sh, "w3_scale": sh, "w2_scale": sh}
        p = {"gate": {"weight": moe.gate.weight.cpu().numpy(), "scale": self.GATE_SHIFT,
                      "bias": moe.gate.bias.cpu().numpy()},
             "shared": mlp(moe.shared_experts), "experts": experts}
        want, _, _ = mo.moe_forward(p, xs.cpu().numpy(), 8, 4, 8, indices=idx)
        return int((got != want).sum()) + extra_bad

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """per-token work of the layer on a token sample: gate, shared expert and 8 routed experts"""
        D, I, S = 7168, 2048, 8
        rng = np.random.default_rng(6)
        ri = lambda shape, b: np.rint(rng.standard_normal(shape) * 2.0**b).astype(np.int64)
        w13 = ri((2 * I, D), 9).astype(np.int32)
        w2 = ri((D, I), 10).astype(np.int32)
        wg = ri((256, D), 9).astype(np.int32)
        x = ri((1, S, D), 16)
        t0 = time.time()
        orc.act(orc.gemm(x, wg, 1, 1, 9)[0], "sigmoid", 23)
        for _ in range(9):                       # shared + 8 routed experts per token
            r = orc.gemm(x, w13, 1, 1, 16)[0]
            h = (orc.act(np.ascontiguousarray(r[..., :I]), "silu", 23) * r[..., I:]) >> 23
            orc.gemm(h, w2, 1, 1, 16)
        dt = time.time() - t0
        return S / dt, "%d of 8192 tokens through gate, shared expert and 8 routed experts" % S, dt


class MoeSmallWorkload(MoeWorkload):
    """The MoE layer with 2048 tokens and 64 experts (quick checks, profiler captures)."""
    name = "moe_layer_2048_tokens_64_experts"
    T, E = 2048, 64

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return MoeWorkload.cpu_sample(orc, np, seconds, rank)


class DecodeWorkload:
    """Reduced-depth int64 DeepSeek-V3 decode at full width: 3 dense layers (inter_dim 18432) and
    one MoE layer (256 routed experts + shared, top-8), int64 embedding and head over a vocabulary of
    129280, every weight random-init at scale 2^16 (int32 layer weights ~ N(0, 2^16/sqrt(fan_in)),
    int64 head), every shift 16.  64 sequences decode greedily, one token per step, against
    latent caches of 2048 positions that were filled with seeded random normalised latents
    (~ N(0, 2^16)) instead of by running a prefill.  One step = one token for each of the 64
    sequences (embedding, 4 blocks, final norm, head, argmax)."""
    name = "decode_4_layers_batch64_cache2048"
    metric = "int64_decode_tokens_per_s"
    unit = "tokens/s"
    scaling = "weak"
    BATCH, CACHE, LAYERS, DENSE = 64, 2048, 4, 3
    SHARDED = False      # True: the N GPUs share ONE model and ONE batch (see DecodeShardedWorkload)

    def __init__(self, torch, k, dev, rank, experts=256, vocab=129280, inter=18432):
        import numpy as np
        import torch.distributed as dist
        self.torch, self.k, self.dev, self.np, self.rank = torch, k, dev, np, rank
        M = importlib.import_module(PKG + ".model")
        self.M = M
        if self.SHARDED and dist.is_initialized():
            M.world_size, M.rank = dist.get_world_size(), dist.get_rank()
        else:
            M.world_size, M.rank = 1, 0           # every GPU decodes its own 64 sequences
        W, R = M.world_size, M.rank
        self.world = W

        def part(n):                               # this rank's slice of n rows
            return (R * (n // W), (R + 1) * (n // W))
        a = M.ModelArgs(max_seq_len=self.CACHE + 512, vocab_size=vocab, dim=7168, inter_dim=inter,
                        moe_inter_dim=2048, n_layers=self.LAYERS, n_dense_layers=self.DENSE, n_heads=128,
                        n_routed_experts=experts, n_shared_experts=1, n_activated_experts=8, n_expert_groups=8,
                        n_limited_groups=4, score_func="sigmoid", route_scale=2.5, q_lora_rank=1536,
                        kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
        self.args = a
        sh = 16
        g = torch.Generator(device=dev).manual_seed(7)

        def weight(out_f, in_f, gen=g, rows=None):
            # every rank draws the whole tensor from the same generator state and keeps its rows
            w = _normal_i(torch, gen, (out_f, in_f), 2.0**16 / math.sqrt(in_f), dev, torch.int32)
            return w if rows is None or W == 1 else w[rows[0]:rows[1]].contiguous()

        def norm_weight(n, dtype=torch.int32):
            return (2**16 + _normal_i(torch, g, (n,), 2.0**8, dev, torch.int64)).to(dtype)

        def scale():
            return torch.tensor(sh, dtype=torch.int32, device=dev)

        with torch.device(dev):
            model = M.Transformer(a)
        M.world_size, M.rank = W, R               # Transformer() reads them from torch.distributed
        vlo, vhi = part(vocab)
        model.embed.weight = _normal_i(torch, g, (vocab, a.dim), 2.0**16, dev, torch.int64)[vlo:vhi].contiguous()
        model.norm.weight = norm_weight(a.dim, torch.int64)
        model.head.weight = _normal_i(torch, g, (vocab, a.dim), 2.0**16 / math.sqrt(a.dim), dev,
                                      torch.int64)[vlo:vhi].contiguous()
        model.head.weight_rescale = 1
        model.head.res_rescale = sh
        D, I = a.dim, a.moe_inter_dim
        for i in range(a.n_layers):
            with torch.device(dev):
                blk = M.Block(i, a, cache_batch=self.BATCH)
            at = blk.attn
            H = a.n_heads
            at.wq_a.weight = weight(a.q_lora_rank, D)
            at.q_norm.weight = norm_weight(a.q_lora_rank)
            at.wq_b1.weight = weight(H * a.qk_nope_head_dim, a.q_lora_rank, rows=part(H * a.qk_nope_head_dim))
            at.wq_b2.weight = weight(H * a.qk_rope_head_dim, a.q_lora_rank, rows=part(H * a.qk_rope_head_dim))
            at.wkv_a1.weight = weight(a.kv_lora_rank, D)
            at.wkv_a2.weight = weight(a.qk_rope_head_dim, D)
            at.kv_norm.weight = norm_weight(a.kv_lora_rank)
            at.wkv_b_1.weight = weight(H * a.qk_nope_head_dim, a.kv_lora_rank, rows=part(H * a.qk_nope_head_dim))
            at.wkv_b_2.weight = weight(H * a.v_head_dim, a.kv_lora_rank, rows=part(H * a.v_head_dim))
            at.wo.weight = weight(D, H * a.v_head_dim, rows=part(D))       # output columns split, full K
            for lin in (at.wq_a, at.wq_b1, at.wq_b2, at.wkv_a1, at.wkv_a2):
                lin.res_rescale = sh
            for lin in (at.wkv_b_1, at.wkv_b_2, at.wo):
                lin.scale = scale()
            at.score_limbs = (3, 3)
            at.kv_cache[:, :self.CACHE] = _normal_i(torch, g, (self.BATCH, self.CACHE, a.kv_lora_rank), 2.0**16, dev,
                                                    torch.int64)
            at.pe_cache[:, :self.CACHE] = _normal_i(torch, g, (self.BATCH, self.CACHE, a.qk_rope_head_dim),
                                                    2.0**16, dev, torch.int64)
            blk.attn_norm.weight = norm_weight(D)
            blk.ffn_norm.weight = norm_weight(D)
            if i < a.n_dense_layers:
                for name, (o, n_in) in (("w1", (inter, D)), ("w3", (inter, D)), ("w2", (D, inter))):
                    lin = getattr(blk.ffn, name)
                    lin.weight = weight(o, n_in, rows=part(o))
                    lin.scale = scale()
            else:
                moe = blk.ffn
                moe.gate.weight = weight(experts, D)
                # shift 9: logits with a standard deviation near 1.0 in Q23 and a small bias, so that the 64
                # tokens spread over the experts as they do in the trained model (see config.experts_hit)
                moe.gate.scale = torch.tensor(9, dtype=torch.int32, device=dev)
                moe.gate.bias = torch.abs(_normal_i(torch, g, (experts,), 2.0**15, dev, torch.int64)).to(torch.int32)
                for name, (o, n_in) in (("w1", (I, D)), ("w3", (I, D)), ("w2", (D, I))):
                    lin = getattr(moe.shared_experts, name)
                    lin.weight = weight(o, n_in, rows=part(o))
                    lin.scale = scale()
                for j in range(moe.n_local_experts):          # each expert from its own seed: any rank can make it
                    ge = torch.Generator(device=dev).manual_seed(7000 + moe.experts_start_idx + j)
                    moe.experts_w13[j, :I] = weight(I, D, gen=ge)
                    moe.experts_w13[j, I:] = weight(I, D, gen=ge)
                    moe.experts_w2[j] = weight(D, I, gen=ge)
                moe.experts_shift.fill_(sh)
            model.layers[i] = blk
        self.model = model
        gt = torch.Generator(device=dev).manual_seed(70 + (0 if self.SHARDED else rank))
        self.tokens = torch.randint(0, vocab, (self.BATCH, 1), generator=gt, device=dev)
        self.pos = self.CACHE
        M.ACT_LIMBS = 3
        self.launches_per_step = 0
        self.tok_host = None
        # bytes the step must stream from HBM (limb planes of every weight it touches + caches)
        self.bytes_fixed = None

    def config(self):
        a = self.args
        return {"workload": self.name, "batch": self.BATCH, "cache_positions": self.CACHE, "layers": a.n_layers,
                "dense_layers": a.n_dense_layers, "dim": a.dim, "vocab": a.vocab_size, "experts": a.n_routed_experts,
                "shift": 16, "act_limbs_bound": 3, "cache_fill": "seeded random latents, no prefill pass",
                "l2": "weights streamed per step (tens of GB) far exceed L2"}

    def _decode(self, tokens):
        m = self.model
        if self.pos >= self.args.max_seq_len:          # wrap: keep the cache length bounded in long runs
            self.pos = self.CACHE
        h, pos, S = m.prep_inference(tokens, self.pos)
        for i in range(self.args.n_layers):
            h = m.layer_inference(i, h, pos, S)
        logits = m.finish_inference(h)                 # [1, B, vocab]
        self.pos += 1
        return logits[0].argmax(dim=-1, keepdim=True)  # greedy, first maximum

    def step(self):
        self.tokens = self._decode(self.tokens)
        return self.tokens

    def step_e2e(self):
        torch = self.torch
        if self.tok_host is None:
            self.tok_host = self.tokens.cpu().pin_memory()
            self.tok_in = torch.empty_like(self.tokens)
        self.tok_in.copy_(self.tok_host, non_blocking=True)
        nxt = self._decode(self.tok_in)
        self.tok_host.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the next step's input is this step's output

    def e2e_bytes(self):
        return self.BATCH * 8, self.BATCH * 8

    def value(self, seconds_per_step, world):
        return self.BATCH * (1 if self.SHARDED else world) / seconds_per_step

    def roofline(self, peaks):
        k = self.k
        k.kernel_timing(2)
        self.step()
        self.torch.cuda.synchronize()
        recs = k.kernel_timing_records()
        k.kernel_timing(False)
        ms = sum(r["ms"] for r in recs)
        # weight bytes each tensor-core launch streams: its B limb planes (N x K x limbs)
        wbytes = 0.0
        hit = [int((blk.ffn.last_counts > 0).sum().item()) for blk in self.model.layers
               if getattr(blk.ffn, "last_counts", None) is not None]
        self.experts_hit = hit
        grouped = [r for r in recs if r["grouped"]]
        for r in recs:
            # a grouped launch reads the planes of the experts that received a row (two launches per MoE layer)
            nb = (hit[grouped.index(r) // 2] if r["grouped"] and len(grouped) == 2 * len(hit) else
                  (self.args.n_routed_experts // self.world) if r["grouped"] else
                  (r["batches"] if r["b_batched"] else 1))
            wbytes += float(nb) * r["N"] * r["K"] * r["lb"]
        self.launches_per_step = 2 * len(recs) + 40
        gbs = wbytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": "limb_gemm kernels of one decode step (%d launches)" % len(recs),
                "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": None, "kernel_ms": round(ms, 3),
                "weight_plane_bytes_per_step": wbytes, "experts_hit_per_moe_layer": hit,
                "launches": [{kk: (round(v, 4) if kk == "ms" else v) for kk, v in r.items()} for r in recs],
                "note": "algorithmic bytes = limb planes of the B operand of every tensor-core launch (weights, "
                        "for the grouped launches the planes of the experts that received at least one row, latent caches); peak = "
                        "STREAM-style copy (%s)" % peaks["source"]}

    def check(self, orc):
        """block 0 (attention over the 2048-position cache + dense MLP) for the first two sequences
        against the numpy restatement of Block.forward, then the head on the same hidden state"""
        from oracle import model_oracle as mo
        np, torch, a, m = self.np, self.torch, self.args, self.model
        blk = m.layers[0]
        pos = self.pos if self.pos < a.max_seq_len else self.CACHE
        h = m.embed(self.tokens)
        freqs = m.freqs_cis[pos:pos + 1]
        kv_before = blk.attn.kv_cache[:2, :pos].cpu().numpy()
        pe_before = blk.attn.pe_cache[:2, :pos].cpu().numpy()
        got = blk(h, pos, freqs, None)[:2].cpu().numpy()
        at = blk.attn
        n = lambda t: t.cpu().numpy()
        pa = {k2: n(getattr(at, k2).weight) for k2 in ("wq_a", "wq_b1", "wq_b2", "wkv_a1", "wkv_a2", "wkv_b_1", "wkv_b_2",
                                                       "wo", "q_norm", "kv_norm")}
        pa.update(wkv_b_1_scale=16, wkv_b_2_scale=16, wo_scale=16)
        p = {"attn_norm": n(blk.attn_norm.weight), "ffn_norm": n(blk.ffn_norm.weight)}
        pf = {"w1": n(blk.ffn.w1.weight), "w3": n(blk.ffn.w3.weight), "w2": n(blk.ffn.w2.weight),
              "w1_scale": 16, "w3_scale": 16, "w2_scale": 16}
        bad = 0
        for b in range(2):
            kv = np.zeros((1, pos + 1, a.kv_lora_rank), np.int64)
            pe = np.zeros((1, pos + 1, a.qk_rope_head_dim), np.int64)
            kv[0, :pos], pe[0, :pos] = kv_before[b], pe_before[b]
            x = n(h[b:b + 1])
            normed, _ = mo.rms_norm(x, p["attn_norm"])
            attned = mo.mla_forward(pa, normed, pos, n(freqs), None, kv, pe, a.n_heads, s_q=16, s_kv=16)
            x1 = x + attned * (2 ** 12)
            f, _ = mo.rms_norm(x1, p["ffn_norm"])
            want = x1 + mo.mlp_forward(pf, f) * (2 ** 8)
            bad += int((got[b:b + 1] != want).sum())
        hn = n(m.norm(h[:2])[0][:, -1])
        logits = n(m.head(m.norm(h[:2])[0][:, -1][None, :]))
        want_l, _ = orc.gemm(hn[None], n(m.head.weight[:4096]), 1, 1, 16)
        bad += int((logits[:, :, :4096] != want_l).sum())
        return bad

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        """one token of one sequence through the GEMVs of one dense layer + head (weights at full width)"""
        rng = np.random.default_rng(7)
        ri = lambda shape, b: np.rint(rng.standard_normal(shape) * 2.0**b).astype(np.int64)
        x = ri((1, 1, 7168), 16)
        shapes = ((1536, 7168), (24576, 1536), (576, 7168), (7168, 16384), (36864, 7168), (7168, 18432))
        ws = [ri(sh, 9).astype(np.int32) for sh in shapes]
        t0 = time.time()
        for w in ws:
            orc.gemm(ri((1, 1, w.shape[1]), 16), w, 1, 1, 16)
        dt = time.time() - t0
        # one dense layer per token; the 4-layer model + head costs about 5.3x that
        return 1.0 / (dt * 5.3), "GEMVs of one dense layer for one token, scaled to 4 layers + head", dt


class DecodeShardedWorkload(DecodeWorkload):
    """The same decode with ONE model and ONE batch of 64 sequences spread over the N GPUs (strong scaling):
    attention heads, the dense MLPs' and the shared expert's hidden and output columns, the routed experts
    (256 / N per GPU, integer all-reduce of their weighted sums as in model.py:1381-1382) and the vocabulary
    rows of embedding and head are split; every output column keeps its full K, so the tokens are those of one
    GPU.  Collectives per step: all-reduce of the embedding, all-gathers of attention output / MLP hidden /
    projection outputs, all-reduce of the routed sums, all-gather of the logits."""
    name = "decode_sharded_4_layers_batch64_cache2048"
    scaling = "strong"
    SHARDED = True
    collective_check = True

    def check(self, orc):
        """the logits of this rank's vocabulary slice against the oracle's head GEMM on the step's final hidden
        state, and every rank's next tokens identical (they all hold the gathered logits)"""
        import torch.distributed as dist
        torch, m = self.torch, self.model
        pos = self.pos if self.pos < self.args.max_seq_len else self.CACHE
        h, p, S = m.prep_inference(self.tokens, pos)
        for i in range(self.args.n_layers):
            h = m.layer_inference(i, h, p, S)
        logits = m.finish_inference(h)                       # gathered over the ranks
        self.pos += 1
        tok = logits[0].argmax(-1)
        if self.world > 1:
            both = [torch.empty_like(tok) for _ in range(self.world)]
            dist.all_gather(both, tok)
            same = all(bool(torch.equal(both[0], t)) for t in both)
        else:
            same = True
        if orc is None:
            return None
        hn = m.norm(h)[0][:, -1].contiguous()
        n = m.head.weight.shape[0]
        want, _ = orc.gemm(hn[None].cpu().numpy(), m.head.weight[:2048].cpu().numpy(), 1, 1, 16)
        lo = self.M.rank * n
        bad = int((logits[:, :, lo:lo + 2048].cpu().numpy() != want).sum())
        return bad + (0 if same else 1)


class GemmWideRangeWorkload(GemmWorkload):
    """The same `wo`-shaped GEMM with wide operands: X uniform in +-2^36, W over the whole int32 range,
    shift 30.  Sums reach 2^81, so the accumulation must be wider than int64; five activation limbs against
    five weight limbs (25 limb pairs instead of 9)."""
    name = "gemm_wo_4096x16384x7168_wide_operands"
    A_BITS, W_BITS, A_LIMBS, SHIFT = 36, 31, 5, 30

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return GemmWorkload.cpu_sample(orc, np, seconds, rank)


class GemmProfWorkload(GemmWorkload):
    """Smaller GEMM of the same kernel for profiler captures (inputs still exceed L2)."""
    name = "gemm_4096x8192x4096"
    M, K, N = 4096, 8192, 4096

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return GemmWorkload.cpu_sample(orc, np, seconds, rank)


class ChainProfWorkload(ChainWorkload):
    """The chain at T = 1024 for profiler captures (softmax tensor 1 GB, still far beyond L2)."""
    name = "fixedpoint_chain_T1024"
    T = 1024

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return ChainWorkload.cpu_sample(orc, np, seconds, rank)


class MlaRefScaleWorkload(MlaWorkload):
    """The MLA layer at the reference's fixed-point magnitudes (activations 2^21, int32 weights
    2^30/sqrt(fan_in), shifts 29-31): more limbs per operand than the 2^16 configuration."""
    name = "mla_layer_prefill_4096_reference_scales"
    SCALES = "reference"

    def __init__(self, torch, k, dev, rank):
        super().__init__(torch, k, dev, rank, scales="reference")

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return MlaWorkload.cpu_sample(orc, np, seconds, rank)


class MlaCausalSkipWorkload(MlaWorkload):
    """The MLA layer with the masked half of the causal score and probability tensors neither
    computed, written nor read (same layer output; reported beside the full computation)."""
    name = "mla_layer_prefill_4096_masked_tiles_skipped"

    def __init__(self, torch, k, dev, rank):
        super().__init__(torch, k, dev, rank)
        self.attn.causal_skip = True

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return MlaWorkload.cpu_sample(orc, np, seconds, rank)


class MlaSmallWorkload(MlaWorkload):
    """The MLA layer at 1024 tokens (profiler captures, quick checks)."""
    name = "mla_layer_prefill_1024"
    T = 1024

    @staticmethod
    def cpu_sample(orc, np, seconds, rank=0):
        return MlaWorkload.cpu_sample(orc, np, seconds, rank)


WORKLOADS = {"gemm": GemmWorkload, "gemm_prof": GemmProfWorkload, "gemm_cfg1": GemmSmallMWorkload,
             "gemm_wide": GemmWideRangeWorkload, "chain": ChainWorkload,
             "chain_prof": ChainProfWorkload, "mla": MlaWorkload, "mla_ref": MlaRefScaleWorkload,
             "mla_small": MlaSmallWorkload, "mla_causal": MlaCausalSkipWorkload, "moe": MoeWorkload,
             "moe_small": MoeSmallWorkload, "decode": DecodeWorkload, "decode_sharded": DecodeShardedWorkload}
DEFAULT_WORKLOAD = "mla"


# --------------------------------------------------------------------------------------------

def _timed_steps(torch, w, n):
    for _ in range(3):
        w.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        w.step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / n


def reference_kernels_on_this_gpu(torch, np):
    """The reference's own CUDA kernels (its unmodified int64_gemm.cu compiled for this GPU by oracle/Makefile,
    otherwise only a checker) timed with CUDA events inside the limits they work in: BASELINE's first
    configuration, and the two score contractions + Q19 softmax of 16 heads at T = 1024."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libint64gemm_ref.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libint64gemm_ref.so was not built where this repository was packed"}
    L = ctypes.CDLL(path)
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    L.int64_64_bmm_broadcast_launcher.argtypes = [vp, vp, vp, vp, ll, ll, ll, ci, ci, ci, ci]
    L.int64_32_bmm_broadcast_launcher.argtypes = [vp, vp, vp, vp, ll, ll, ll, ci, ci, ci, ci]
    L.einsum_bshc_btc_bsht.argtypes = [vp, vp, vp, ll, ci, ci, ci, ci, ci]
    L.softmax_q19.argtypes = [vp, vp, vp, ci, ci, ci, ci]
    L.softmax_init_q19.argtypes = [vp]
    dev = torch.device("cuda", torch.cuda.current_device())

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()                      # the reference launches on the legacy default stream
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    rng = np.random.default_rng(0)
    X = torch.from_numpy(rng.integers(-2**20, 2**20, (1, 32, 7168), dtype=np.int64)).to(dev)
    W = torch.from_numpy(rng.integers(-2**15, 2**15, (576, 7168), dtype=np.int64)).to(dev)
    W32 = W.to(torch.int32)
    C, R = torch.empty((1, 32, 576), dtype=torch.int64, device=dev), torch.empty((1, 32, 576), dtype=torch.int64, device=dev)
    out = {"kind": "reference_cuda", "library": "oracle/_ref/libint64gemm_ref.so (the reference's int64_gemm.cu, nvcc -arch=sm_100)"}
    with torch.cuda.stream(torch.cuda.default_stream()):
        for name, fn, w in (("gemm_32x7168x576_int64_W", L.int64_64_bmm_broadcast_launcher, W),
                            ("gemm_32x7168x576_int32_W", L.int64_32_bmm_broadcast_launcher, W32)):
            ms = timed(lambda: fn(X.data_ptr(), w.data_ptr(), C.data_ptr(), R.data_ptr(), 1, 1, 16, 1, 32, 7168, 576), 5)
            out[name] = {"ms": round(ms, 4), "Gop/s": round(2.0 * 32 * 576 * 7168 / ms / 1e6, 1)}
        S, H, T = 64, 16, 1024
        q = torch.from_numpy(rng.integers(-2**16, 2**16, (1, S, H, 512), dtype=np.int64)).to(dev)
        kv = torch.from_numpy(rng.integers(-2**16, 2**16, (1, T, 512), dtype=np.int64)).to(dev)
        qp = torch.from_numpy(rng.integers(-2**16, 2**16, (1, S, H, 64), dtype=np.int64)).to(dev)
        pe = torch.from_numpy(rng.integers(-2**16, 2**16, (1, T, 64), dtype=np.int64)).to(dev)
        s1, s2 = torch.empty((1, S, H, T), dtype=torch.int64, device=dev), torch.empty((1, S, H, T), dtype=torch.int64, device=dev)
        probs = torch.empty_like(s1)
        lut = torch.zeros(256, dtype=torch.int64)
        L.softmax_init_q19(lut.data_ptr())
        lut = lut.to(dev)

        def scores():
            L.einsum_bshc_btc_bsht(q.data_ptr(), kv.data_ptr(), s1.data_ptr(), 23, 1, S, H, T, 512)
            L.einsum_bshc_btc_bsht(qp.data_ptr(), pe.data_ptr(), s2.data_ptr(), 21, 1, S, H, T, 64)
            sc = (s1 + s2) * 94 // 695
            L.softmax_q19(sc.data_ptr(), probs.data_ptr(), lut.data_ptr(), 1, S, H, T)

        ms = timed(scores, 3)
        out["scores_softmax_64q_16h_T1024"] = {"ms": round(ms, 4),
                                               "Gop/s": round(2.0 * S * H * T * 576 / ms / 1e6, 1),
                                               "note": "two score einsums, torch glue (s1+s2)*94//695, softmax_q19"}
    return out


def default_line_extras(torch, k, dev, rank, peaks, np, wl):
    """Parts of the default line beside the MLA layer: the int64 GEMM at a tensor-bound projection shape in
    two operand ranges, BASELINE's first (small-M, HBM-bound) configuration, the layer at the reference's own
    magnitudes, and the reference's CUDA kernels on this GPU."""
    out = {}
    torch.cuda.empty_cache()
    for key, cls in (("int64_gemm", GemmWorkload), ("int64_gemm_wide_operands", GemmWideRangeWorkload)):
        gw = cls(torch, k, dev, rank)
        sec = _timed_steps(torch, gw, 10)
        out[key] = {"metric": gw.metric, "value": round(gw.value(sec, 1), 1), "unit": gw.unit, "workload": gw.name,
                    "config": gw.config(), "ms": round(sec * 1e3, 4), "roofline": gw.roofline(peaks)}
        k.device_status(sync=True)
        del gw
        torch.cuda.empty_cache()
    sw = GemmSmallMWorkload(torch, k, dev, rank)
    sec = _timed_steps(torch, sw, 10)
    out["int64_gemm_small_m"] = {"metric": sw.metric, "value": round(sw.value(sec, 1), 1), "unit": sw.unit,
                                 "workload": sw.name, "config": sw.config(),
                                 "us_per_call_host_launched": round(sec * 1e6 / sw.COPIES, 2),
                                 "roofline": sw.roofline(peaks)}
    k.device_status(sync=True)
    del sw
    torch.cuda.empty_cache()
    # the same layer at the reference's fixed-point magnitudes (more limbs per operand)
    old_limbs = wl.M.ACT_LIMBS
    wl.attn = None
    torch.cuda.empty_cache()
    rw = MlaRefScaleWorkload(torch, k, dev, rank)
    sec = _timed_steps(torch, rw, 3)
    out["value_reference_scales"] = {"metric": rw.metric, "value": round(rw.value(sec, 1), 2), "unit": rw.unit,
                                     "workload": rw.name, "config": rw.config(), "ms_per_step": round(sec * 1e3, 3),
                                     "roofline": rw.roofline(peaks)}
    k.device_status(sync=True)
    del rw
    wl.M.ACT_LIMBS = old_limbs
    torch.cuda.empty_cache()
    try:
        out["reference_kernels_b200"] = reference_kernels_on_this_gpu(torch, np)
    except Exception as err:  # noqa: BLE001 - a baseline, never fatal
        out["reference_kernels_b200"] = {"unavailable": repr(err)}
    return out


def run_reference(args, rank, world):
    """The reference has no CPU implementation of this path beyond torch's int64 `F.linear` (its kernels are
    CUDA only, its library is built as a checker under oracle/_ref).  The CPU arm is the OpenMP int128 oracle
    (`kind: "port"`), the same arithmetic the reference's kernels perform, on every host thread, on a bounded
    sample of the workload per step; the torch `F.linear` path is timed beside it on BASELINE's first
    configuration, the only one where wrapping int64 is exact."""
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as orc
    orc.build()
    # torch.distributed.run exports OMP_NUM_THREADS=1: use every core for every N all the same
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    wl = WORKLOADS[args.workload]
    vals = []
    budget = 60.0 / max(1, args.steps + args.warmup)
    desc = ""
    for i in range(args.warmup + args.steps):
        v, desc, dt = wl.cpu_sample(orc, np, min(budget, 10.0))
        if i >= args.warmup:
            vals.append((v, dt))
    value = statistics.mean(v for v, _ in vals)
    config = wl.static_config(world) if hasattr(wl, "static_config") else {"workload": wl.name}
    line = {"impl": "reference", "metric": wl.metric, "value": round(value, 3), "unit": wl.unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(1e3 * statistics.mean(d for _, d in vals), 3),
            "higher_is_better": True, "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None,
            "dtype": "int64", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": round(value, 3), "unit": wl.unit, "cores": orc.num_threads(),
                             "kind": "port", "sample": desc},
            "e2e": {"value": round(value, 3), "unit": wl.unit, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    try:
        import torch
        torch.set_num_threads(cores)
        line["cpu_baseline_torch"] = torch_cpu_baseline(torch, np, 2.0)
    except Exception as err:  # noqa: BLE001 - the arm must still print its line
        line["cpu_baseline_torch"] = {"unavailable": repr(err)}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--moe-exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel MoE on N > 1 GPUs: rows and results over peer memory inside the expert "
                         "kernels (default) or NCCL all-to-all of packed rows")
    ap.add_argument("--e2e-copies", default="pipelined", choices=["pipelined", "inline"],
                    help="end-to-end steps of the layer workloads: host copies on copy streams that overlap the "
                         "neighbouring steps' kernels (default) or on the compute stream around each step")
    ap.add_argument("--op-profile", default=None, metavar="FILE",
                    help="after the timed steps, run three more under torch.profiler and write rank 0's table of "
                         "CUDA time per operator and kernel to FILE (where a multi-rank step's time goes; the "
                         "timed numbers are taken before it)")
    ap.add_argument("--no-extras", action="store_true",
                    help="default workload only: leave out the GEMM, small-M, reference-scale and reference-kernel parts")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    k = importlib.import_module(PKG + ".kernel")
    peaks = measured_peaks()
    importlib.import_module(PKG + ".model").PEER_EXPERTS = args.moe_exchange == "peer"
    PipelinedIO.INLINE = args.e2e_copies == "inline"
    wl = WORKLOADS[args.workload](torch, k, dev, rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------
    for _ in range(args.warmup):
        wl.step()
    k.device_status()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        wl.step()
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed = ev0.elapsed_time(ev1) * 1e-3
    k.device_status()
    # duration of the dominant kernel, CUDA events recorded around it on its own stream
    roof = wl.roofline(peaks)
    t = torch.tensor([elapsed], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec_per_step = float(t.item()) / args.steps

    if args.op_profile:
        from torch.profiler import profile, ProfilerActivity
        barrier()
        from torch.profiler import schedule
        # two steps with the profiler attached but not recording (its start-up differs per rank and would
        # show up as waiting inside the first collective), then three recorded ones
        tables = []
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                     schedule=schedule(wait=0, warmup=2, active=3, repeat=1),
                     on_trace_ready=lambda p_: tables.append(p_.key_averages().table(
                         sort_by="cuda_time_total", row_limit=30, max_name_column_width=70))) as prof:
            for i in range(5):
                if i == 2:
                    torch.cuda.synchronize()
                    barrier()
                wl.step()
                if i == 4:
                    torch.cuda.synchronize()
                prof.step()
        if rank == 0:
            with open(args.op_profile, "w") as f:
                f.write("three steps of %s on %d GPU(s), rank 0\n" % (wl.name, world))
                f.write(tables[0] if tables else "the profiler recorded nothing\n")
        barrier()

    # ---- end to end through the drop-in module with host buffers -------------------------------
    for _ in range(3):
        wl.step_e2e()
    barrier()
    ev0.record()
    for _ in range(args.steps):
        wl.step_e2e()
    ev1.record()
    barrier()
    t = torch.tensor([ev0.elapsed_time(ev1) * 1e-3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_sec = float(t.item()) / args.steps
    h2d, d2h = wl.e2e_bytes()

    mismatches = None
    if world > 1 and getattr(wl, "collective_check", False):
        orc = None
        if rank == 0:
            from oracle import oracle as orc
            orc.build()
        mismatches = wl.check(orc)          # every rank takes part in the collectives
        barrier()
    extras = {}
    if rank == 0:
        from oracle import oracle as orc
        orc.build()
        orc.set_threads(os.cpu_count() or 1)      # torch.distributed.run exports OMP_NUM_THREADS=1
        if world == 1 or not getattr(wl, "collective_check", False):
            mismatches = wl.check(orc)
    if args.workload == DEFAULT_WORKLOAD and world == 1 and not args.no_extras:
        # the rest of the headline metric and the configurations the default workload does not cover
        wl.x_host = None
        extras = default_line_extras(torch, k, dev, rank, peaks, np, wl)
        extras["cpu_baseline_torch"] = torch_cpu_baseline(torch, np, 2.0)
    if rank == 0:
        cpu_v, cpu_desc, _ = (wl.cpu_sample(orc, np, args.cpu_seconds)
                                if world == 1 and args.cpu_seconds > 0 else (None, None, 0))
        launches = wl.launches_per_step * args.steps
        line = {"metric": wl.metric, "value": round(wl.value(sec_per_step, world), 2), "unit": wl.unit,
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(sec_per_step * 1e3, 4), "higher_is_better": True,
                "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": "int64",
                "data": "synthetic", "config": wl.config(),
                "e2e": {"value": round(wl.value(e2e_sec, world), 2), "unit": wl.unit,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": round(e2e_sec * 1e3, 4),
                        "copies": getattr(wl, "e2e_note", "on the compute stream, before and after the step's kernels")},
                "gpu_launches": launches,
                "roofline": roof,
                "clocks": clocks, "mismatched_words_vs_oracle": mismatches}
        line.update(extras)
        if cpu_v is not None:
            line["cpu_baseline"] = {"value": round(cpu_v, 3), "unit": wl.unit,
                                    "cores": orc.num_threads(), "kind": "port", "sample": cpu_desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
