#!/usr/bin/env python
"""Benchmark of the tensor hot path: `python bench.py --gpus N --steps K --warmup W`.

With no --workload the headline is the MLP forward (BASELINE configs[1]); the same run then
measures, a few steps each, every other configuration and kernel family and attaches them to the
one JSON line under "extras" (so that every quoted number has a line in a driver-run record).

Workloads (seeded synthetic inputs with the shapes and distributions of the reference
configurations; no dataset is used):
  mlp    3-layer MLP forward, batch 4096, 784->1024->1024->10, relu/relu/softmax+argmax
         (metric: samples/s) - the headline
  gemm   one fp32 GEMM M=N=K (default 16384, --size), 3xTF32 (or --precision bf16)
  gemm_sharded  the same product with the rows of A split over the ranks and C all-gathered in
         row panels on a side stream while the next panel computes (strong scaling)
  conv   conv2d 256x64x56x56 * 128x64x3x3, pad 1, + bias + relu
  cnn    conv32-conv64-pool-dense128-dense10 forward on 1x28x28 images, batch 8192
  add, mul, scale, relu, gt, exp, log, sum, softmax   2^28 float32 (HBM-bound)
  sum_axis0, sum_axis1, argmax_rows, transpose, maxpool, fill, split_rows   the remaining
         HBM-bound kernel families (axis reductions, movement, pooling, constructors, GEMM pre-pass)
  mma_peak   the tensor pipe's ceiling: back-to-back tcgen05.mma on resident operands

Under torchrun every rank runs the same per-GPU workload on its own shard (weak scaling, no
data-path collective: samples / row blocks are independent; gemm_sharded is the exception);
rank 0 prints ONE JSON line.
`--impl reference` times the reference's own CPU operators (oracle/_ref) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (every 100 ms) for the whole run;
    `window(t0, t1)` summarises the samples that fell inside a timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0, t1):
        """Clocks seen between host times t0 and t1 (a sample describes the 100 ms before it, so
        the window is widened by that much; a region shorter than the sampling period takes the
        nearest sample)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        deadline = time.time() + 0.25
        while time.time() < deadline and not any(t >= t1 for t, _ in self.rows):
            time.sleep(0.02)
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.12]
        if not rows and self.rows:
            rows = [min(self.rows, key=lambda tr: abs(tr[0] - t1))[1]]
        sm, mx, power, reasons = [], None, [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for n, v in zip(self.NAMES, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
                power.append(float(r[6]))
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w": float(np.median(power)) if power else None}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


# ---------------------------------------------------------------------------------------
# seeded inputs (numpy PCG64; identical on every rank and on the CPU baseline)
# ---------------------------------------------------------------------------------------

def mlp_inputs(batch):
    rng = np.random.default_rng(1)

    def kaiming(fi, fo):
        lim = np.sqrt(6.0 / fi)
        return rng.uniform(-lim, lim, (fi, fo)).astype(np.float32)

    w = [kaiming(784, 1024), kaiming(1024, 1024), kaiming(1024, 10)]
    b = [np.zeros(1024, np.float32), np.zeros(1024, np.float32), np.zeros(10, np.float32)]
    x = np.random.default_rng(2).uniform(0, 1, (batch, 784)).astype(np.float32)
    return x, w, b


MLP_FLOP_PER_SAMPLE = 2 * (784 * 1024 + 1024 * 1024 + 1024 * 10)


def gemm_inputs(m, k, n, seed=5):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    return a, b


def conv_inputs(batch):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((batch, 64, 56, 56), dtype=np.float32)
    w = (rng.standard_normal((128, 64, 3, 3)) * np.sqrt(2.0 / (64 * 9))).astype(np.float32)
    b = np.zeros(128, np.float32)
    return x, w, b


# ---------------------------------------------------------------------------------------
# reference arm: the reference's own CPU operators on a bounded sample
# ---------------------------------------------------------------------------------------

def _reference_worker(workload, size, steps, warmup):
    """One host process: builds its own inputs, runs `steps` bounded samples on the reference's
    compiled operators (oracle/_ref), or on the C restatement when that library is absent.
    Returns (kind, units per step, mean seconds per step, description of the sample)."""
    import oracle
    from oracle import IntArray

    be = oracle.ref() if oracle.Reference.available() else None
    p = oracle.port()
    if workload == "mlp":
        sample = 16  # the reference loop runs at ~0.2 GFLOP/s per thread
        x, w, b = mlp_inputs(sample)

        def step():
            h = x
            for i in range(3):
                if be is not None:
                    xb = be.call("concat", h, be.call("ones", IntArray([h.shape[0], 1])), 1)
                    wb = be.call("concat", w[i], b[i].reshape(1, -1), 0)
                    h = be.call("matmul", xb, wb)
                    if i < 2:
                        h = be.call("multiply", h, be.call("gt", h, 0))
                else:
                    h = p.dense(h, w[i], b[i], 1 if i < 2 else 0)
            p.softmax_rows(h)
            p.argmax_axis(h, 1)

        units = sample
        desc = f"{sample} of 4096 samples per step and process, full layer widths"
    elif workload == "gemm":
        n, cols = size, min(size, 512)
        rows = max(1, int(1.0e9 / (2.0 * n * cols)))
        a, bm = gemm_inputs(rows, n, cols)

        def step():
            be.call("matmul", a, bm) if be is not None else p.matmul(a, bm)

        units = 2.0 * rows * n * cols / 1e12
        desc = f"{rows} rows of A x {cols} columns of B (k = {n}) per step and process"
    else:
        return None
    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return ("reference" if be is not None else "port", units, float(np.mean(times)), desc)


def run_reference(args, rank):
    """The reference arm: the reference's own CPU operators.  Its kernels are single-threaded, so
    the host's cores are used the only way the reference could use them: independent shards of
    the batch (samples / row blocks) in parallel, one process per core."""
    if rank != 0:
        return
    if args.workload == "default":
        args.workload = "mlp"  # the headline
    metric, unit = {"mlp": ("mlp_forward_samples_per_s", "samples/s"),
                    "gemm": ("gemm_fp32_tflops", "TFLOP/s")}.get(args.workload, (None, None))
    if metric is None:
        print(json.dumps({"impl": "reference", "unavailable": f"workload {args.workload} has no reference arm"}))
        return
    import multiprocessing as mp
    from concurrent.futures import ProcessPoolExecutor

    cores = os.cpu_count() or 1
    workers = 1 if args.ref_workers == 1 else max(1, min(cores, args.ref_workers or 32))
    steps, warmup = max(1, min(args.steps, 3)), max(0, min(args.warmup, 1))
    if workers == 1:
        results = [_reference_worker(args.workload, args.size, steps, warmup)]
    else:
        with ProcessPoolExecutor(max_workers=workers, mp_context=mp.get_context("spawn")) as ex:
            futs = [ex.submit(_reference_worker, args.workload, args.size, steps, warmup) for _ in range(workers)]
            results = [f.result() for f in futs]
    kind, units, _, desc = results[0]
    t = max(r[2] for r in results)  # the slowest shard bounds the step
    value = units * workers / t
    # the same workload description as the GPU arm prints for this --workload
    workload = {"mlp": "mlp_forward 784-1024-1024-10 relu,relu,softmax+argmax (BASELINE configs[1])",
                "gemm": f"gemm fp32 M=N=K={args.size} U(-1,1) (BASELINE configs[4] per-GPU problem)"}[args.workload]
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (float64 accumulate, the reference's arithmetic)", "data": "synthetic",
            "config": {"workload": workload, "batch_per_gpu": 4096 if args.workload == "mlp" else None,
                       "note": "the reference's CPU operators on the host cores, a bounded sample per step and process"},
            "cpu_baseline": {"value": value, "unit": unit, "cores": workers, "kind": kind,
                             "sample": desc + f"; {workers} processes (the kernels themselves are single-threaded)",
                             "host_cores_available": cores},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

class Workload:
    """One step = one pass of the hot path over one batch.  `step()` runs with inputs resident
    in HBM; `e2e_step()` goes through host buffers (pinned) with the copies inside."""

    name = ""
    metric = ""
    unit = ""
    dominant = "gemm_tc"
    bound = "tensor"
    scaling = "weak"

    def units_per_step(self):  # in the metric's unit numerator
        raise NotImplementedError

    def algorithmic_per_step(self):  # flops (tensor) or bytes (hbm) of the dominant kernel
        raise NotImplementedError

    def ncu_traffic(self):
        """(DRAM bytes per launch of the dominant kernel from an ncu capture, where it came from).
        The figures are constants copied from the summaries under profiles/: a profiler never runs
        inside the bench."""
        return None, "no ncu capture of this shape"


class _Pinned:
    """Page-locked host buffer from the library's own allocator (ct_host_alloc)."""

    def __init__(self, shape, dtype):
        from camel_b200 import pipeline
        self.buf = pipeline.pinned_array(shape, dtype)

    def data_ptr(self):
        return self.buf.ptr

    def numpy(self):
        return self.buf.array

    def numel(self):
        return int(self.buf.array.size)


def _pin_empty(shape, dtype):
    return _Pinned(shape, dtype)


def _pin(torch, a):
    a = np.asarray(a)
    t = _Pinned(a.shape, a.dtype)
    t.numpy()[...] = a
    return t


class MlpWorkload(Workload):
    name, metric, unit = "mlp", "mlp_forward_samples_per_s", "samples/s"

    def __init__(self, torch, T, batch, use_graph=True):
        self.T, self.torch, self.batch = T, torch, batch
        x, w, b = mlp_inputs(batch)
        self.w = [T.from_numpy(v) for v in w]
        self.b = [T.from_numpy(v) for v in b]
        self.x = T.from_numpy(x)
        self.x_host = _pin(torch, x)
        self.x_stage = T.Tensor(0, x.shape)
        self.probs_host = _pin_empty((batch, 10), np.float32)
        self.arg_host = _pin_empty((batch,), np.int64)
        self.h2d = x.nbytes
        self.d2h = batch * 10 * 4 + batch * 8
        self.graph = None
        if use_graph:
            # the forward pass is seven launches of 5-50 us: record it once, replay per step
            from camel_b200._lib import check, lib
            check(lib.ct_d2d(self.x_stage.ptr, self.x.ptr, self.h2d))
            warm = [self.forward(self.x_stage) for _ in range(2)]
            T.check_async()
            with T.Graph() as g:
                g.keep = self.forward(self.x_stage)
            self.graph = g
            del warm

    def forward(self, x):
        T = self.T
        h = T.dense(x, self.w[0], self.b[0], "relu")
        h = T.dense(h, self.w[1], self.b[1], "relu")
        return T.dense(h, self.w[2], self.b[2], "softmax", with_argmax=True)

    def step(self):
        if self.graph is not None:
            self.graph.launch()
        else:
            self.out = self.forward(self.x)

    def eager_step(self):
        self.out = self.forward(self.x)

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(self.x_stage.ptr, self.x_host.data_ptr(), self.h2d))
        if self.graph is not None:
            self.graph.launch()
            probs, arg = self.graph.keep
        else:
            probs, arg = self.forward(self.x_stage)
        check(lib.ct_d2h(self.probs_host.data_ptr(), probs.ptr, self.batch * 40))
        check(lib.ct_d2h(self.arg_host.data_ptr(), arg.ptr, self.batch * 8))

    def e2e_run(self, steps, flush):
        """Every step copies its batch from pinned host memory, runs the recorded forward pass
        and reads probabilities and argmax back; the three stages of consecutive steps overlap
        (camel_b200.pipeline.HostPipeline).  The L2 flush sits on the compute stream in front
        of every step's kernels, inside the timed region.  Returns device ms for all steps."""
        from camel_b200 import pipeline
        from camel_b200._lib import F32, check, lib
        if getattr(self, "pipe", None) is None:
            pre = None
            if flush is not None:
                pre = lambda: check(lib.ct_fill(F32, 1.0, flush.numel() // 4, flush.data_ptr()))  # noqa: E731
            self.pipe = pipeline.HostPipeline(self.forward, F32, (self.batch, 784), depth=2, pre_compute=pre)
            self.host_in = [self.x_host, _pin(self.torch, self.x_host.numpy()[::-1])]
            self.host_out = [(_pin_empty((self.batch, 10), np.float32), _pin_empty((self.batch,), np.int64))
                             for _ in range(2)]
        ins = [self.host_in[i % 2].data_ptr() for i in range(steps)]
        outs = [tuple(t.data_ptr() for t in self.host_out[i % 2]) for i in range(steps)]
        return self.pipe.run(ins, outs)

    def units_per_step(self):
        return self.batch

    def algorithmic_per_step(self):
        return 2.0 * self.batch * (784 * 1024 + 1024 * 1024)  # the two tensor-core layers

    def ncu_traffic(self):
        if self.batch != 4096:
            return None, "captured at batch 4096 only"
        return 38.1e6, ("ncu capture of this workload: 43.4 MB (k=1024) and 32.9 MB (k=784) per launch = the "
                        "operand planes read once; the result stays in L2")

    def resident_bytes(self):
        return self.x.nbytes + sum(t.nbytes for t in self.w) + 2 * self.batch * 1024 * 4

    def config(self):
        return {"workload": "mlp_forward 784-1024-1024-10 relu,relu,softmax+argmax (BASELINE configs[1])",
                "batch_per_gpu": self.batch, "precision": "3xtf32",
                "weights": "tensor-core layout kept with each weight tensor (built at first use)"
                if self.T._weight_cache else "transposed and split at every call"}


class GemmWorkload(Workload):
    name, metric, unit = "gemm", "gemm_fp32_tflops", "TFLOP/s"

    def __init__(self, torch, T, n, precision, e2e=True):
        self.T, self.n, self.precision = T, n, precision
        dev = torch.device("cuda")
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        # U(-1,1) generated on the device: 2 GiB of host RNG per rank would dominate start-up
        self.a_t = torch.rand((n, n), generator=g, device=dev, dtype=torch.float32) * 2 - 1
        self.b_t = torch.rand((n, n), generator=g, device=dev, dtype=torch.float32) * 2 - 1
        self.c_t = torch.empty((n, n), device=dev, dtype=torch.float32)
        torch.cuda.synchronize()
        self.a = T.wrap_device(self.a_t.data_ptr(), 0, (n, n), keep=self.a_t)
        self.b = T.wrap_device(self.b_t.data_ptr(), 0, (n, n), keep=self.b_t)
        self.e2e_rows = min(n, 2048)
        self.h2d = self.e2e_rows * n * 4
        self.d2h = self.e2e_rows * n * 4
        if e2e:
            self.a_host = _pin(torch, self.a_t[: self.e2e_rows].cpu().numpy())
            self.c_host = _pin_empty((self.e2e_rows, n), np.float32)

    def step(self):
        from camel_b200._lib import check, lib
        n = self.n
        check(lib.ct_matmul(0, self.a.ptr, 0, self.b.ptr, n, n, n, self.c_t.data_ptr()))

    def e2e_step(self):
        # B is the replicated operand (resident); a row block of A comes from the host and the
        # matching block of C goes back: what a row-sharded caller does per block.
        from camel_b200._lib import check, lib
        n, r = self.n, self.e2e_rows
        check(lib.ct_h2d(self.a_t.data_ptr(), self.a_host.data_ptr(), self.h2d))
        check(lib.ct_matmul(0, self.a.ptr, 0, self.b.ptr, r, n, n, self.c_t.data_ptr()))
        check(lib.ct_d2h(self.c_host.data_ptr(), self.c_t.data_ptr(), self.d2h))

    def units_per_step(self):
        return 2.0 * self.n ** 3 / 1e12

    def e2e_units_per_step(self):
        return 2.0 * self.e2e_rows * self.n * self.n / 1e12

    def algorithmic_per_step(self):
        return 2.0 * self.n ** 3

    def ncu_traffic(self):
        if self.n == 4096:
            return 690.7e6, "ncu capture at 4096^3 (335 MB algorithmic: operand tiles re-read 2.1x)"
        return None, ("captured at 4096^3 only: the re-read factor depends on how the raster groups fit in L2 "
                      "and does not scale with the flops")

    def resident_bytes(self):
        return 3 * self.n * self.n * 4

    def config(self):
        return {"workload": f"gemm fp32 M=N=K={self.n} U(-1,1) (BASELINE configs[4] per-GPU problem)",
                "precision": self.precision}


class ShardedGemmWorkload(Workload):
    """BASELINE configs[4] as one job: C = A.B with M=N=K=n, A split by rows over the ranks, B
    replicated (placed once, outside the timed region), every rank ends up with all of C.  The
    only exchange is the all-gather of C row blocks (NCCL over NVLink); it is issued per row panel
    on a side stream so that panel j travels while panel j+1 is computed.  Strong scaling."""

    name, metric, unit, scaling = "gemm_sharded", "gemm_fp32_tflops", "TFLOP/s", "strong"

    def __init__(self, torch, dist, T, n, world, rank):
        self.torch, self.dist, self.T, self.n, self.world, self.rank = torch, dist, T, n, world, rank
        dev = torch.device("cuda")
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        a_full = torch.rand((n, n), generator=g, device=dev, dtype=torch.float32) * 2 - 1
        self.b_t = torch.rand((n, n), generator=g, device=dev, dtype=torch.float32) * 2 - 1
        from camel_b200 import sharding
        self.sharding = sharding
        _, self.rows = sharding.row_shard(n, world, rank)
        # panel j travels while panel j+1 is computed, so only the last gather is exposed: the panels
        # halve down to 256 rows (two row tiles; the early ones stay large enough to fill the GPU).
        # Rows are dealt out band by band (band j = panel j of every rank), so that a gathered panel
        # is one contiguous piece of C and its all-gather runs in place, without a staging copy.
        plan = sharding.tapered_panel_plan(self.rows) if world > 1 else [(0, self.rows)]
        self.bands = sharding.banded_rows(plan, world, rank)
        self.panels = len(plan)
        self.a_t = torch.cat([a_full[g0:g0 + cnt] for _, cnt, g0, _ in self.bands]).contiguous()
        # a few rows of A from all over the matrix, to check the gathered product once (first warm-up step)
        self.check_rows = torch.arange(7, n, n // 24, device=dev)[:24]
        self.check_a = a_full[self.check_rows].double()
        self.checked = False
        del a_full
        self.c_t = torch.empty((n, n), device=dev, dtype=torch.float32)  # the gathered product
        # B is placed once: so is its tensor-core layout (transposed hi/lo planes), outside the timed region
        import ctypes as C
        from camel_b200._lib import check, lib
        self.b_packed = C.c_void_p()
        check(lib.ct_weights_pack(self.b_t.data_ptr(), n, n, C.byref(self.b_packed)))
        self.a_packed = C.c_void_p()  # planes of this rank's rows of A: refilled every step, allocated once
        self.side = torch.cuda.Stream()
        # all bands in one launch: per-band counters of finished tiles, which the side stream waits on
        self.band_done = torch.zeros(8, dtype=torch.int32, device=dev)
        self.band_rows = (C.c_int64 * len(self.bands))(*[cnt for _, cnt, _, _ in self.bands])
        self.band_out = (C.c_void_p * len(self.bands))(*[self.c_t.data_ptr() + g0 * n * 4 for _, _, g0, _ in self.bands])
        self.band_tiles = (C.c_uint32 * len(self.bands))()
        torch.cuda.synchronize()
        self.h2d = self.d2h = 0

    def step(self):
        import ctypes as C
        from camel_b200._lib import check, lib
        torch, n = self.torch, self.n
        check(lib.ct_rows_pack(self.a_t.data_ptr(), self.rows, n, C.byref(self.a_packed)))
        # One launch computes the bands in order and counts finished tiles per band; the side stream
        # waits for a band's count and all-gathers it while the same launch works on the next band.
        self.band_done.zero_()
        cleared = torch.cuda.Event()
        cleared.record()
        check(lib.ct_matmul_packed_bands(self.a_packed, self.b_packed, len(self.bands), self.band_rows, self.band_out,
                                         self.band_done.data_ptr(), self.band_tiles))
        if self.world > 1:
            with torch.cuda.stream(self.side):
                self.side.wait_event(cleared)  # not before the counters of the previous step were cleared
                for j, (off, cnt, g0, band0) in enumerate(self.bands):
                    check(lib.ct_set_stream(self.side.cuda_stream))
                    check(lib.ct_stream_wait_value(self.band_done.data_ptr() + 4 * j, self.band_tiles[j]))
                    check(lib.ct_set_stream(None))
                    self.sharding.gather_band(self.dist, self.c_t, band0, cnt, self.rank, self.world)
            torch.cuda.current_stream().wait_stream(self.side)
        if not self.checked:  # untimed: the first warm-up step
            self.checked = True
            torch.cuda.synchronize()
            ref = self.check_a @ self.b_t.double()
            err = float((self.c_t[self.check_rows].double() - ref).abs().max() / ref.abs().max())
            if not err <= 1e-5:
                raise RuntimeError(f"gemm_sharded: gathered product is off by {err:.3e} of its largest entry on rank {self.rank}")
            del ref, self.check_a

    def e2e_step(self):
        self.step()

    def units_per_step(self):
        return 2.0 * self.n ** 3 / self.world / 1e12

    def algorithmic_per_step(self):
        return 2.0 * self.n ** 3 / self.world

    def resident_bytes(self):
        return 3 * self.n * self.n * 4

    def config(self):
        return {"workload": f"gemm fp32 M=N=K={self.n}, A row-sharded over {self.world} ranks, C all-gathered "
                            f"in place in {self.panels} bands of halving size (one launch, a band travels as soon as its tiles are done), B and its tensor-core layout "
                            f"placed once (BASELINE configs[4])",
                "precision": "3xtf32", "e2e": "same as value: operands are resident by construction",
                "parallelism": f"{self.world} ranks, rows of A and C sharded, NCCL all-gather of C on a side stream"}


class ConvWorkload(Workload):
    name, metric, unit = "conv", "conv2d_fp32_tflops", "TFLOP/s"

    def __init__(self, torch, T, batch, e2e=True):
        self.T, self.batch = T, batch
        x, w, b = conv_inputs(batch)
        self.x, self.w, self.b = T.from_numpy(x), T.from_numpy(w), T.from_numpy(b)
        if e2e:
            self.x_host = _pin(torch, x)
            self.out_host = _pin_empty((batch, 128, 56, 56), np.float32)
        self.h2d, self.d2h = x.nbytes, batch * 128 * 56 * 56 * 4
        self.flops = 2.0 * batch * 128 * 56 * 56 * 64 * 9

    def step(self):
        self.out = self.T.conv2d(self.x, self.w, self.b, 1, 1, "relu")

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(self.x.ptr, self.x_host.data_ptr(), self.h2d))
        out = self.T.conv2d(self.x, self.w, self.b, 1, 1, "relu")
        check(lib.ct_d2h(self.out_host.data_ptr(), out.ptr, self.d2h))

    def units_per_step(self):
        return self.flops / 1e12

    def algorithmic_per_step(self):
        return self.flops

    def ncu_traffic(self):
        # batch-32 capture: 52.1 MB read = the NHWC and weight planes once; reads scale with the batch,
        # and at full size the whole result goes to DRAM (at batch 32 most of it was still in L2)
        reads = 52.1e6 * self.batch / 32.0
        writes = self.batch * 128 * 56 * 56 * 4.0
        return reads + writes, ("ncu capture at batch 32: reads scaled by the batch (planes are read once), "
                                "writes = the size of the result")

    def resident_bytes(self):
        return self.h2d + self.d2h

    def config(self):
        return {"workload": "conv2d 64->128 56x56 3x3 pad1 +bias +relu (BASELINE configs[2])",
                "batch_per_gpu": self.batch, "precision": "3xtf32"}


class AddWorkload(Workload):
    name, metric, unit = "add", "elementwise_add_gbs", "GB/s"
    dominant, bound = "elementwise", "hbm"

    def __init__(self, torch, T, n):
        self.T, self.n = T, n
        rng = np.random.default_rng(6)
        x = rng.uniform(-1, 1, n).astype(np.float32)
        y = rng.uniform(-1, 1, n).astype(np.float32)
        self.x, self.y = T.from_numpy(x), T.from_numpy(y)
        self.out = T.Tensor(0, (n,))
        self.e2e_n = min(n, 1 << 24)
        self.x_host, self.y_host = _pin(torch, x[: self.e2e_n]), _pin(torch, y[: self.e2e_n])
        self.o_host = _pin_empty((self.e2e_n,), np.float32)
        self.h2d, self.d2h = 8 * self.e2e_n, 4 * self.e2e_n

    def step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_binary(0, 0, self.x.ptr, 0, self.y.ptr, self.n, self.out.ptr))

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_binary_host(0, self.x_host.data_ptr(), self.y_host.data_ptr(), self.e2e_n, self.o_host.data_ptr()))

    def units_per_step(self):
        return 12.0 * self.n / 1e9

    def e2e_units_per_step(self):
        return 12.0 * self.e2e_n / 1e9

    def algorithmic_per_step(self):
        return 12.0 * self.n

    def ncu_traffic(self):
        return 12.0 * self.n, ("ncu capture at 2^26 elements moved its algorithmic 12 B/element (reads exact, the "
                               "tail of the writes still in L2); scaled by n")

    def resident_bytes(self):
        return 12 * self.n

    def config(self):
        return {"workload": f"elementwise add of {self.n} float32 (12 B/element)"}


class HbmWorkload(Workload):
    """One memory-bound operator over 2^28 float32 (or 8192 x 8192 for softmax)."""

    bound = "hbm"
    unit = "GB/s"
    #        op: (bytes per element, profile family)
    OPS = {"add": (12, "elementwise"), "relu": (8, "elementwise"), "exp": (8, "elementwise"), "log": (8, "elementwise"),
           "mul": (12, "elementwise"), "scale": (8, "elementwise"), "gt": (5, "elementwise"),
           "sum": (4, "reduce"), "softmax": (8, "softmax")}

    def __init__(self, torch, T, op, n, on_device=False):
        if op == "softmax":
            n = min(n, 1 << 26)  # 8192 rows of 8192: a row stays in the registers of one block
        self.T, self.op, self.n = T, op, n
        self.bpe, self.dominant = self.OPS[op]
        self.name, self.metric = op, f"elementwise_{op}_gbs"
        self.e2e_n = min(n, 1 << 24)
        if on_device:
            # the same distribution drawn on the device (seeded): a gigabyte of host RNG per operator
            # would dominate a run that measures many of them
            g = torch.Generator(device="cuda")
            g.manual_seed(6)
            xt = torch.rand(n, generator=g, device="cuda", dtype=torch.float32) * 2 - 1
            if op == "log":
                xt += 1.0001
            self.x = T.wrap_device(xt.data_ptr(), 0, (8192, n // 8192) if op == "softmax" else (n,), keep=xt)
            self.y = None
            if op in ("mul", "add"):
                yt = torch.rand(n, generator=g, device="cuda", dtype=torch.float32) * 2 - 1
                self.y = T.wrap_device(yt.data_ptr(), 0, (n,), keep=yt)
            x = xt[: self.e2e_n].cpu().numpy()
        else:
            rng = np.random.default_rng(6)
            x = rng.uniform(-1, 1, n).astype(np.float32)
            if op == "log":
                x = x + np.float32(1.0001)  # shifted to (0, 2): log throws on values <= 0
            self.x = T.from_numpy(x.reshape(8192, -1) if op == "softmax" else x)
            self.y = T.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)) if op in ("mul", "add") else None
        self.x_host = _pin(torch, x[: self.e2e_n])
        self.o_host = _pin_empty((self.e2e_n,), np.float32)
        self.h2d, self.d2h = 4 * self.e2e_n, 4 * self.e2e_n
        self.x_small = T.Tensor(0, (8192, self.e2e_n // 8192) if op == "softmax" else (self.e2e_n,))

    def _run(self, x):
        T = self.T
        if self.op == "relu":
            return T.relu(x)
        if self.op == "exp":
            return T.exp(x)
        if self.op == "log":
            return T.log(x)
        if self.op == "mul":
            return T.multiply(x, self.y)
        if self.op == "add":
            return T.add(x, self.y)
        if self.op == "scale":
            return T.multiply(x, 0.5)
        if self.op == "gt":
            return T.gt(x, 0.0)
        if self.op == "sum":
            return T.sum(x)
        return T.softmax(x)

    def step(self):
        self.out = self._run(self.x)

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(self.x_small.ptr, self.x_host.data_ptr(), self.h2d))
        if self.op in ("mul", "add"):
            out = (self.T.multiply if self.op == "mul" else self.T.add)(self.x_small, self.x_small)
        else:
            out = self._run(self.x_small)
        if isinstance(out, float):
            self.d2h = 8
            return
        self.d2h = out.nbytes
        check(lib.ct_d2h(self.o_host.data_ptr(), out.ptr, min(out.nbytes, self.o_host.numel() * 4)))

    def units_per_step(self):
        return self.bpe * self.n / 1e9

    def e2e_units_per_step(self):
        return self.bpe * self.e2e_n / 1e9

    def algorithmic_per_step(self):
        return float(self.bpe) * self.n

    def ncu_traffic(self):
        if self.op in ("exp", "softmax"):
            return float(self.bpe) * self.n, ("ncu capture at 2^26 elements read and wrote every element once "
                                               "(8 B/element); scaled by n")
        return None, "no ncu capture of this operator"

    def resident_bytes(self):
        return self.bpe * self.n

    def config(self):
        return {"workload": f"{self.op} over {self.n} float32 ({self.bpe} B/element)"}


class KernelFamilyWorkload(Workload):
    """The HBM-bound kernel families that are not elementwise maps: axis reductions, transpose,
    max-pool, constructors and the GEMM operand pre-pass.  Inputs are drawn on the device (seeded).
    `bytes` is the algorithmic traffic of one call: what must be read plus what must be written."""

    bound, unit = "hbm", "GB/s"

    def __init__(self, torch, T, kind):
        from camel_b200._lib import check, lib
        self.T, self.kind, self.lib, self.check = T, kind, lib, check
        self.name, self.metric = kind, f"{kind}_gbs"
        g = torch.Generator(device="cuda")
        g.manual_seed(7)
        rand = lambda *shape: torch.rand(shape, generator=g, device="cuda", dtype=torch.float32) * 2 - 1  # noqa: E731
        wrap = lambda t: T.wrap_device(t.data_ptr(), 0, tuple(t.shape), keep=t)  # noqa: E731
        self.h2d = self.d2h = 0
        if kind in ("sum_axis0", "sum_axis1", "max_axis1", "argmax_axis1"):
            r = c = 8192
            self.x = wrap(rand(r, c))
            out = c if kind == "sum_axis0" else r
            self.bytes = 4.0 * r * c + (8.0 if kind.startswith("argmax") else 4.0) * out
            self.dominant = "reduce"
            self.desc = f"{kind} of {r} x {c} float32"
        elif kind == "argmax_rows":
            r, c = 1 << 22, 10  # the classifier's shape (4096 x 10) is 160 KB: far below anything measurable
            self.x = wrap(rand(r, c))
            self.bytes = 4.0 * r * c + 8.0 * r
            self.dominant = "reduce"
            self.desc = f"argmax over the 10 columns of {r} rows (the classifier's row shape, many rows)"
        elif kind == "transpose":
            r = c = 8192
            self.x = wrap(rand(r, c))
            self.bytes = 8.0 * r * c
            self.dominant = "transpose"
            self.desc = f"transpose of {r} x {c} float32"
        elif kind == "maxpool":
            self.x = wrap(rand(2048, 64, 28, 28))
            self.bytes = 5.0 * self.x.numel
            self.dominant = "maxpool"
            self.desc = "maxpool2d 2x2 of 2048 x 64 x 28 x 28 (BASELINE configs[3] layer shape, a quarter of its batch)"
        elif kind == "fill":
            self.n = 1 << 28
            self.out = T.Tensor(0, (self.n,))
            self.bytes = 4.0 * self.n
            self.dominant = "elementwise"
            self.desc = f"full([{self.n}], 1.5): 4 B/element written"
        elif kind == "split_rows":
            import ctypes as C
            self.rows, self.k = 16384, 8192
            self.x = wrap(rand(self.rows, self.k))
            self.packed = C.c_void_p()
            self.bytes = 12.0 * self.rows * self.k
            self.dominant = "gemm_prepass"
            self.desc = f"operand pre-pass of the 3xTF32 GEMM over {self.rows} x {self.k} float32 (4 B read, 8 B written per element)"
        else:
            raise ValueError(kind)

    def step(self):
        T, k = self.T, self.kind
        if k == "sum_axis0":
            self.out = T.sum(self.x, 0)
        elif k == "sum_axis1":
            self.out = T.sum(self.x, 1)
        elif k == "max_axis1":
            self.out = T.max(self.x, 1)
        elif k in ("argmax_axis1", "argmax_rows"):
            self.out = T.argmax(self.x, 1)
        elif k == "transpose":
            self.out = T.transpose(self.x)
        elif k == "maxpool":
            self.out = T.maxpool2d(self.x, 2)
        elif k == "fill":
            self.check(self.lib.ct_fill(0, 1.5, self.n, self.out.ptr))
        else:
            import ctypes as C
            self.check(self.lib.ct_rows_pack(self.x.ptr, self.rows, self.k, C.byref(self.packed)))

    def units_per_step(self):
        return self.bytes / 1e9

    def algorithmic_per_step(self):
        return self.bytes

    def resident_bytes(self):
        return self.bytes

    def config(self):
        return {"workload": self.desc}

    def close(self):
        if getattr(self, "packed", None):
            self.lib.ct_rows_free(self.packed)
            self.packed = None


class Gemm512Workload(Workload):
    """BASELINE configs[0]: fp32 GEMM M=N=K=512, U(-1,1), seed 0, through the matmul operator.
    0.27 GFLOP: launch- and latency-bound, reported without a roofline expectation."""

    name, metric, unit = "gemm512", "gemm_fp32_tflops", "TFLOP/s"

    def __init__(self, torch, T):
        rng = np.random.default_rng(0)
        self.T = T
        self.a = T.from_numpy(rng.uniform(-1, 1, (512, 512)).astype(np.float32))
        self.b = T.from_numpy(rng.uniform(-1, 1, (512, 512)).astype(np.float32))
        self.h2d = self.d2h = 0

    def step(self):
        self.out = self.T.matmul(self.a, self.b)

    def units_per_step(self):
        return 2.0 * 512 ** 3 / 1e12

    def algorithmic_per_step(self):
        return 2.0 * 512 ** 3

    def resident_bytes(self):
        return 3 * 512 * 512 * 4

    def config(self):
        return {"workload": "gemm fp32 M=N=K=512 U(-1,1) seed 0 (BASELINE configs[0]): latency-bound",
                "precision": "3xtf32"}


class CnnWorkload(Workload):
    """BASELINE configs[3]: conv 1->32 +relu, conv 32->64 +relu, 2x2 maxpool, flatten,
    dense 12544->128 +relu, dense 128->10 +softmax, on 1x28x28 Uniform(0,1) images."""

    name, metric, unit = "cnn", "cnn_forward_samples_per_s", "samples/s"

    def __init__(self, torch, T, batch, fuse_pool=True, use_graph=True):
        self.T, self.batch = T, batch
        rng = np.random.default_rng(4)

        def kaiming(shape, fan_in):
            lim = np.sqrt(6.0 / fan_in)
            return rng.uniform(-lim, lim, shape).astype(np.float32)

        self.w = [T.from_numpy(kaiming((32, 1, 3, 3), 9)), T.from_numpy(kaiming((64, 32, 3, 3), 288)),
                  T.from_numpy(kaiming((12544, 128), 12544)), T.from_numpy(kaiming((128, 10), 128))]
        self.b = [T.from_numpy(np.zeros(n, np.float32)) for n in (32, 64, 128, 10)]
        x = rng.uniform(0, 1, (batch, 1, 28, 28)).astype(np.float32)
        self.x = T.from_numpy(x)
        self.x_host = _pin(torch, x)
        self.probs_host = _pin_empty((batch, 10), np.float32)
        self.arg_host = _pin_empty((batch,), np.int64)
        self.h2d, self.d2h = x.nbytes, batch * 48
        self.flops = 2.0 * batch * (28 * 28 * (32 * 9 + 64 * 288) + 12544 * 128 + 1280)
        self.fuse_pool = fuse_pool
        # the forward pass is eight launches and as many allocations: record it once, replay per step
        # (launched call by call, the host falls behind the GPU once the memory pool has served other
        # workloads: 2.43 instead of 2.05 ms per step with the same kernel times)
        self.graph = None
        if use_graph:
            warm = [self.forward(self.x) for _ in range(2)]
            T.check_async()
            with T.Graph() as g:
                g.keep = self.forward(self.x)
            self.graph = g
            del warm

    def forward(self, x):
        T = self.T
        h = T.conv2d(x, self.w[0], self.b[0], 1, 1, "relu")
        if self.fuse_pool:  # conv + relu + 2x2 max-pool as one call (the pool in the conv's epilogue)
            h = T.flatten(T.conv2d(h, self.w[1], self.b[1], 1, 1, "relu", pool=2))
        else:
            h = T.conv2d(h, self.w[1], self.b[1], 1, 1, "relu")
            h = T.flatten(T.maxpool2d(h, 2))
        h = T.dense(h, self.w[2], self.b[2], "relu")
        return T.dense(h, self.w[3], self.b[3], "softmax", with_argmax=True)

    def step(self):
        if self.graph is not None:
            self.graph.launch()
        else:
            self.out = self.forward(self.x)

    def eager_step(self):
        self.out = self.forward(self.x)

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(self.x.ptr, self.x_host.data_ptr(), self.h2d))
        if self.graph is not None:
            self.graph.launch()
            probs, arg = self.graph.keep
        else:
            probs, arg = self.forward(self.x)
        check(lib.ct_d2h(self.probs_host.data_ptr(), probs.ptr, self.batch * 40))
        check(lib.ct_d2h(self.arg_host.data_ptr(), arg.ptr, self.batch * 8))

    def units_per_step(self):
        return self.batch

    def algorithmic_per_step(self):
        # the tensor-core launches: conv2 and dense1 (conv1 with 9 taps of one channel and the
        # 10-column classifier run on CUDA cores)
        return 2.0 * self.batch * (28 * 28 * 64 * 288 + 12544 * 128)

    def resident_bytes(self):
        return self.batch * 64 * 28 * 28 * 4

    def config(self):
        return {"workload": "cnn_forward conv32-conv64-pool-dense128-dense10 on 1x28x28 (BASELINE configs[3])",
                "batch_per_gpu": self.batch, "precision": "3xtf32",
                "weights": "tensor-core layout kept with each weight tensor (built at first use)"
                if self.T._weight_cache else "transposed and split at every call"}


class Bench:
    """Timing harness shared by the headline and the extras: CUDA events on the launching stream
    around every step, L2 flushed between steps when the working set is smaller than L2, a barrier
    and a device synchronisation on both sides, the slowest rank's time."""

    def __init__(self, torch, dist, lib, check, T, rank, world, sampler):
        self.torch, self.dist, self.lib, self.check, self.T = torch, dist, lib, check, T
        self.rank, self.world, self.sampler = rank, world, sampler
        self.flush_buf = None

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def flush_for(self, wl):
        if wl.resident_bytes() >= 2 * L2_BYTES:
            return None
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(L2_BYTES * 2, dtype=self.torch.uint8, device="cuda")
        return self.flush_buf

    def reduce_max(self, v):
        from camel_b200 import sharding
        return sharding.reduce_max(self.dist, self.torch, v, "cuda")

    def timed(self, fn, steps, flush):
        torch = self.torch
        evs = []
        self.barrier()
        for _ in range(steps):
            if flush is not None:
                flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        self.barrier()
        return sum(a.elapsed_time(b) for a, b in evs)

    def measure(self, wl, steps, warmup, min_gpu_s=0.0, max_blocks=2000, min_blocks=1):
        """Resident throughput of `wl`: `warmup` untimed steps, then blocks of exactly `steps`
        timed steps, repeated until `min_gpu_s` seconds of device time have been timed and at
        least `min_blocks` blocks; the reported time per step is the median block's (a host that is
        descheduled between two launches of a short block would otherwise show up as GPU time).  Then the dominant kernel's own
        launch durations from the library's event brackets on the same inputs."""
        lib, check, T = self.lib, self.check, self.T
        flush = self.flush_for(wl)
        for _ in range(max(warmup, 3)):
            wl.step()
        T.check_async()
        replayed = getattr(wl, "graph", None) is not None
        launches0 = lib.ct_launch_count()
        t0 = time.time()
        blocks = [self.reduce_max(self.timed(wl.step, steps, flush))]
        launches = lib.ct_launch_count() - launches0
        # every rank must run the same number of blocks: the count comes from the first block's
        # (already max-reduced) time
        extra_blocks = min_blocks - 1
        if min_gpu_s > 0 and blocks[0] > 0:
            extra_blocks = max(extra_blocks, min(max_blocks, int(np.ceil(min_gpu_s * 1e3 / blocks[0]))))
        for _ in range(extra_blocks):
            blocks.append(self.reduce_max(self.timed(wl.step, steps, flush)))
        t1 = time.time()
        clocks = self.sampler.window(t0, t1) if self.sampler is not None else None
        # The dominant kernel's own launch durations: a second pass over the same inputs with the
        # library's event brackets on (they switch programmatic dependent launch off, so that a
        # bracket times one kernel alone; the timed region above ran without them).  A replayed
        # graph bypasses the brackets, so that pass runs call by call.
        prof_steps = min(steps, 10)
        check(lib.ct_profile_enable(1))
        self.timed(wl.eager_step if replayed else wl.step, prof_steps, flush)
        tot, cnt = ctypes_double(), ctypes_u64()
        check(lib.ct_profile_read(wl.dominant.encode(), tot, cnt))
        # every kernel family's share of a step (the library's own brackets, this pass)
        scopes = {}
        for name in PROFILE_SCOPES:
            t_s, n_s = ctypes_double(), ctypes_u64()
            check(lib.ct_profile_read(name.encode(), t_s, n_s))
            if n_s.value:
                scopes[name] = {"ms_per_step": t_s.value / prof_steps, "launches_per_step": n_s.value / prof_steps}
        check(lib.ct_profile_read(None, None, None))
        check(lib.ct_profile_enable(0))
        T.check_async()
        ms_block = float(np.median(blocks))
        return {"ms_per_step": ms_block / steps, "blocks": len(blocks), "gpu_s": float(sum(blocks)) / 1e3,
                "launches": int(launches), "dom_ms": tot.value / max(1, cnt.value),
                "launches_per_step": cnt.value / prof_steps, "clocks": clocks,
                "flush": flush is not None, "scopes": scopes}


def measured_mma_peaks(lib, check, sampler):
    """The tensor pipe's ceiling on this GPU, now: tcgen05.mma back to back on resident operands
    (ct_measure_mma_peak).  Burst = the rate between two short launches of 70 and 240 us (what a
    short kernel can be held against); sustained = a run of about two seconds (what a kernel
    inside a long, power-capped step can be held against)."""
    import ctypes as C
    from camel_b200._lib import PREC_3XTF32, PREC_BF16

    out = {}
    tf, ms = C.c_double(), C.c_double()
    for name, kind in (("tf32", PREC_3XTF32), ("bf16", PREC_BF16)):
        # a launch pays ~15 us of set-up besides its MMAs: the pipe's own rate is the difference
        # quotient of two launch sizes (best of five each), 200 and 800 groups of four MMAs per SM
        best = {}
        for groups in (200, 800):
            t_best, f_best = None, None
            for _ in range(5):
                check(lib.ct_measure_mma_peak(kind, groups, 1, C.byref(tf), C.byref(ms)))
                if t_best is None or ms.value < t_best:
                    t_best, f_best = ms.value, tf.value * ms.value  # tflops * ms = Gflop
            best[groups] = (t_best, f_best)
        burst = (best[800][1] - best[200][1]) / (best[800][0] - best[200][0])
        check(lib.ct_measure_mma_peak(kind, 800, 20, C.byref(tf), C.byref(ms)))
        n = max(20, min(20000, int(2000.0 / max(ms.value / 20, 1e-3))))
        t0 = time.time()
        check(lib.ct_measure_mma_peak(kind, 800, n, C.byref(tf), C.byref(ms)))
        clocks = sampler.window(t0, time.time()) if sampler is not None else None
        out[name] = {"burst_tflops": burst, "burst_launch_us": [best[200][0] * 1e3, best[800][0] * 1e3],
                     "sustained_tflops": tf.value, "sustained_s": ms.value / 1e3, "sustained_clocks": clocks}
        # the same pipe in its own clock domain (stamps inside the kernel): SM cycles per 128 x 256 MMA
        # and the SM clock the measuring loop really ran at
        cpm, mhz = C.c_double(), C.c_double()
        check(lib.ct_measure_mma_clocks(kind, 128, 256, C.byref(cpm), C.byref(mhz)))
        k = 8 if name == "tf32" else 16
        out[name].update({"clocks_per_mma_128x256": cpm.value, "sm_mhz_in_kernel": mhz.value,
                          "flop_per_clk_per_sm": 2.0 * 128 * 256 * k / cpm.value if cpm.value > 0 else None})
    return out


def roofline_of(wl, m, pk, mma, precision):
    """roofline object of one measured workload.  Tensor-bound kernels are held against the measured
    MMA rate of this run (tf32 / 3 for the 3xTF32 scheme): the burst figure for launches shorter
    than 5 ms, the sustained one for longer launches; the figure derived from the driver-written
    bf16 GEMM peak is kept beside it.  `frac_at_clock` holds the kernel against the pipe's rate per SM cycle
    (cycle stamps inside the measuring kernel) times the median SM clock sampled during this workload."""
    dom_ms = m["dom_ms"]
    alg = wl.algorithmic_per_step() / max(1.0, m["launches_per_step"])
    out = {"bound": wl.bound, "kernel": wl.dominant, "launches_per_step": m["launches_per_step"],
           "avg_launch_ms": dom_ms}
    if wl.bound == "tensor":
        achieved = alg / (dom_ms / 1e3) / 1e12 if dom_ms > 0 else 0.0
        kind = "bf16" if precision == "bf16" else "tf32"
        div = 1.0 if precision == "bf16" else 3.0
        derived = pk["bf16_tflops"] / (1.0 if precision == "bf16" else 6.0)
        if mma is not None:
            which = "burst" if dom_ms < 5.0 else "sustained"

            def pipe(w):
                # a tf32 MMA moves the bytes of a bf16 MMA with half the k: the pipe gives tf32 half the
                # bf16 rate.  On some GPUs of the pool the tf32 measuring loop itself reads a quarter
                # lower than that (while the GEMM kernels run as fast as elsewhere), so the ceiling is
                # the larger of the two readings: never flatter the kernel with a slow measurement.
                if kind == "bf16":
                    return mma["bf16"][f"{w}_tflops"]
                return max(mma["tf32"][f"{w}_tflops"], mma["bf16"][f"{w}_tflops"] / 2.0)

            peak = pipe(which) / div
            note = (f"measured in this run: tcgen05.mma back to back on resident operands, {which} figure"
                    + ("" if precision == "bf16" else ", the larger of kind::tf32 and kind::f16 / 2, / 3 (three MMAs per product)"))
            out["peak_burst"] = pipe("burst") / div
            out["peak_sustained"] = pipe("sustained") / div
        else:
            peak, note = derived, "derived (no MMA measurement on this rank)"
        out.update({"achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                    "peak_note": note, "peak_derived_from_bf16_gemm": derived,
                    "frac_of_derived": achieved / derived if derived else None})
        c = m.get("clocks") or {}
        fpc = None
        if mma is not None and mma[kind].get("flop_per_clk_per_sm"):
            fpc = mma[kind]["flop_per_clk_per_sm"]
            if kind == "tf32" and mma["bf16"].get("flop_per_clk_per_sm"):
                fpc = max(fpc, mma["bf16"]["flop_per_clk_per_sm"] / 2.0)
        if fpc and c.get("sm_mhz"):
            # the pipe's rate per SM clock (cycle stamps inside the measuring kernel) x SMs x the clock
            # sampled during this workload: what the MMAs alone would reach at the clock the power
            # cap left this kernel
            at_clock = fpc * SM_COUNT * c["sm_mhz"] * 1e6 / 1e12 / div
            out["peak_at_clock"] = at_clock
            out["frac_at_clock"] = achieved / at_clock
            out["time_x_mhz"] = dom_ms * c["sm_mhz"]
            if achieved > 1.02 * at_clock:
                out["clock_note"] = ("the sampled clock understates the clock this kernel ran at (nvidia-smi samples every "
                                     "200 ms; the measuring loop's own cycle/ns stamps read "
                                     f"{mma[kind]['sm_mhz_in_kernel']:.0f} MHz while the sampler read "
                                     f"{(mma[kind]['sustained_clocks'] or {}).get('sm_mhz')} MHz): read `frac` instead")
    else:
        achieved = alg / (dom_ms / 1e3) / 1e9 if dom_ms > 0 else 0.0
        out.update({"achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "peak_note": f"{pk['source']} STREAM-style copy"})
    traffic, traffic_note = wl.ncu_traffic() if precision != "bf16" else (None, "no ncu capture in bf16 mode")
    out.update({"traffic": traffic, "traffic_unit": "bytes per launch", "traffic_note": traffic_note})
    return out


SM_COUNT = 148  # B200
# the kernel families the library brackets with events when profiling is on (ct_profile_enable)
PROFILE_SCOPES = ["gemm_tc", "gemm_prepass", "gemm_skinny", "gemm_splitk_reduce", "conv_prepass", "conv_small_c",
                  "im2col", "maxpool", "elementwise", "reduce", "softmax", "transpose", "concat", "weights_pack"]

EXTRA_STEPS = {"gemm": 5, "gemm_bf16": 5, "gemm512": 50, "conv": 10, "cnn": 5, "gemm_sharded": 3}


def run_extras(bench, args, pk, mma):
    """Every other configuration and kernel family, a few steps each, for the `extras` list."""
    import gc

    torch, T, lib, check = bench.torch, bench.T, bench.lib, bench.check
    from camel_b200 import _lib

    names = ["gemm512", "gemm", "gemm_bf16", "conv", "cnn"]
    if bench.world > 1:
        names.append("gemm_sharded")
    else:
        names += ["add", "mul", "scale", "relu", "gt", "sum", "exp", "log", "softmax", "sum_axis0", "sum_axis1",
                  "max_axis1", "argmax_axis1", "argmax_rows", "transpose", "maxpool", "fill", "split_rows"]
    out = []
    for name in names:
        precision = "bf16" if name == "gemm_bf16" else "3xtf32"
        if precision == "bf16":
            check(lib.ct_set_precision(_lib.PREC_BF16))
        try:
            if name == "gemm512":
                wl = Gemm512Workload(torch, T)
            elif name in ("gemm", "gemm_bf16"):
                wl = GemmWorkload(torch, T, 16384, precision, e2e=False)
            elif name == "gemm_sharded":
                wl = ShardedGemmWorkload(torch, bench.dist, T, 16384, bench.world, bench.rank)
            elif name == "conv":
                wl = ConvWorkload(torch, T, 256, e2e=False)
            elif name == "cnn":
                wl = CnnWorkload(torch, T, 8192)
            elif name in HbmWorkload.OPS:
                wl = HbmWorkload(torch, T, name, 1 << 28, on_device=True)
            else:
                wl = KernelFamilyWorkload(torch, T, name)
            steps = EXTRA_STEPS.get(name, 10)
            m = bench.measure(wl, steps, 3, min_blocks=3)
            # whole-job aggregate: a rank's units per step (its share, for a strong-scaling job) x ranks
            value = wl.units_per_step() * bench.world / (m["ms_per_step"] / 1e3)
            rec = {"workload": name, "metric": wl.metric, "value": value, "unit": wl.unit,
                   "ms_per_step": m["ms_per_step"], "steps": steps, "scaling": wl.scaling,
                   "config": wl.config(), "gpu_launches": m["launches"], "clocks": m["clocks"],
                   "l2": "flushed between steps" if m["flush"] else "inputs larger than L2",
                   "kernel_families_per_step": m["scopes"]}
            if name != "gemm512":
                rec["roofline"] = roofline_of(wl, m, pk, mma, precision)
            out.append(rec)
        finally:
            if precision == "bf16":
                check(lib.ct_set_precision(_lib.PREC_3XTF32))
        if hasattr(wl, "close"):
            wl.close()
        del wl
        gc.collect()
        torch.cuda.empty_cache()
    return out


def plugin_leg(args, batch, world_reduce):
    """The headline's end-to-end number through the plugin's operator bodies, driven the way a
    scheduler drives them (src/passes/sched/nodevm/nodevm.cpp:557-591): per step a host batch
    becomes a tensor (host-to-device copy), the operators are called through operator_t, and the
    host reads probabilities and arg-max back; wall clock in C++ around each step.  mode 0: the
    fused operators; mode 1: the module's small operators (deferred-expression path)."""
    import ctypes as C

    harness = ROOT / "camel_b200" / "host" / "_build" / "libcamel_tensor_host_test.so"
    if not harness.exists():
        return None
    h = C.CDLL(str(harness))
    x, w, b = mlp_inputs(batch)
    xs = np.ascontiguousarray(np.stack([x, x[::-1]]))
    # the same two batches in page-locked memory (a host that page-locks its input buffers) and in
    # ordinary memory (where the reference's allocator puts large tensors: gen.h:259-271)
    locked = _Pinned(xs.shape, np.float32)
    locked.numpy()[...] = xs
    probs, arg = np.zeros((batch, 10), np.float32), np.zeros(batch, np.int64)
    steps = max(20, args.steps)
    out = {}
    for mode, key, src in ((0, "fused_operators", locked.data_ptr()), (0, "fused_operators_pageable", xs.ctypes.data),
                           (1, "small_operators", locked.data_ptr())):
        secs = (C.c_double * steps)()
        launches, err = C.c_uint64(), C.create_string_buffer(512)
        P = lambda a: C.c_void_p(a.ctypes.data)  # noqa: E731
        rc = h.camel_host_mlp_forward(
            C.c_int(mode), C.c_void_p(src), C.c_int(2), C.c_int64(batch), C.c_int64(784), C.c_int64(1024), C.c_int64(1024),
            C.c_int64(10), P(w[0]), P(b[0]), P(w[1]), P(b[1]), P(w[2]), P(b[2]), C.c_int(steps), P(probs), P(arg),
            secs, C.byref(launches), err, C.c_int(512))
        if rc != 0:
            raise RuntimeError("plugin leg: " + err.value.decode())
        t = np.array(list(secs))[3:]  # the first steps build the weights' tensor-core layout
        med = world_reduce(float(np.median(t)))
        out[key] = {"seconds_per_step": med, "launches_per_step": launches.value / steps,
                    "argmax_checksum": int(arg.sum()), "probs_row_sums_ok": bool(np.all(np.abs(probs.sum(1) - 1) < 1e-4))}
    return out


def training_leg(lib):
    """One update step of the reference's MNIST program (test/run/nn/mnist.cml:27-41) at its own
    sizes, 60000 x 785 features (bias column included) x 10 classes, operator by operator through
    the plugin's operator_t bodies with tensors resident: matmul, the ten-operator softmax,
    subtract, transpose, matmul, multiply, subtract.  Deferred (the module recognises the idioms
    and launches fused kernels) and eager (every operator launches), wall clock in C++ around the
    loop including the final read-back of the weights; launches counted by the library."""
    import ctypes as C

    harness = ROOT / "camel_b200" / "host" / "_build" / "libcamel_tensor_host_test.so"
    if not harness.exists():
        return None
    h = C.CDLL(str(harness))
    n, d, classes, steps = 60000, 785, 10, 20
    rng = np.random.default_rng(11)
    x = rng.uniform(0, 1, (n, d)).astype(np.float32)
    x[:, -1] = 1.0
    y = np.zeros((n, classes), np.float32)
    y[np.arange(n), rng.integers(0, classes, n)] = 1.0
    out = {"workload": "one update step of test/run/nn/mnist.cml:27-41, 60000 x 785 x 10, through operator_t"}
    P = lambda a: C.c_void_p(a.ctypes.data)  # noqa: E731
    lib.ct_launch_count.restype = C.c_uint64
    for key, lazy in (("deferred", 1), ("eager", 0)):
        best, launches = None, 0
        for rep in range(3):  # the first repetition also builds what is built once
            w = np.zeros((d, classes), np.float32)
            secs, err = C.c_double(), C.create_string_buffer(512)
            h.camel_host_session_begin(C.c_int(lazy))
            l0 = lib.ct_launch_count()
            rc = h.camel_host_sgd_loop(P(x), P(y), P(w), C.c_int64(n), C.c_int64(d), C.c_int64(classes), C.c_double(0.5),
                                       C.c_int(steps), C.c_int(1), None, C.byref(secs), err, C.c_int(512))
            if rc != 0:
                raise RuntimeError("training leg: " + err.value.decode())
            launches = lib.ct_launch_count() - l0
            best = secs.value if best is None else min(best, secs.value)
        out[key] = {"us_per_step": best / steps * 1e6, "launches_per_step": launches / steps,
                    "weights_checksum": float(np.abs(w).sum())}
    h.camel_host_session_begin(C.c_int(1))
    return out


def h2d_ceiling(bench, nbytes, copies=40):
    """Bare host-to-device bandwidth of this rank while every rank copies at once: `copies`
    cudaMemcpyAsync of the step's input size from page-locked memory, no kernels."""
    import ctypes as C

    lib, check = bench.lib, bench.check
    src = _Pinned((nbytes,), np.uint8)
    dst = bench.T.Tensor(2, (nbytes,))
    e0, e1 = C.c_void_p(), C.c_void_p()
    check(lib.ct_event_create(C.byref(e0)))
    check(lib.ct_event_create(C.byref(e1)))
    for _ in range(3):
        check(lib.ct_h2d_async(dst.ptr, src.data_ptr(), nbytes))
    bench.barrier()
    check(lib.ct_event_record(e0))
    for _ in range(copies):
        check(lib.ct_h2d_async(dst.ptr, src.data_ptr(), nbytes))
    check(lib.ct_event_record(e1))
    bench.barrier()
    ms = C.c_float()
    check(lib.ct_event_elapsed_ms(e0, e1, C.byref(ms)))
    check(lib.ct_event_destroy(e0))
    check(lib.ct_event_destroy(e1))
    ms_max = bench.reduce_max(float(ms.value))
    return nbytes * copies / (ms_max / 1e3) / 1e9


def run_gpu(args, rank, world):
    import torch

    global SM_COUNT
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    SM_COUNT = torch.cuda.get_device_properties(local).multi_processor_count
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import camel_b200  # noqa: F401
    from camel_b200 import _lib, tensor as T
    from camel_b200._lib import check, lib

    check(lib.ct_set_device(local))
    check(lib.ct_set_stream(None))  # legacy default stream: ordered with torch's default stream
    if args.precision == "bf16":
        check(lib.ct_set_precision(_lib.PREC_BF16))
    T.set_weight_cache(not args.no_weight_cache)

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    bench = Bench(torch, dist, lib, check, T, rank, world, sampler)
    pk = peaks()
    headline = args.workload == "default"
    name = "mlp" if headline else args.workload

    if name == "mma_peak":
        mma = measured_mma_peaks(lib, check, sampler) if rank == 0 else None
        if rank == 0:
            print(json.dumps({"metric": "tensor_pipe_peak_tflops", "unit": "TFLOP/s", "n_gpus": 1,
                              "value": mma["tf32"]["burst_tflops"], "mma_peak": mma,
                              "config": {"workload": "tcgen05.mma 128x256 back to back on resident operands, one CTA per SM"}}))
        if sampler is not None:
            sampler.stop()
        if dist is not None:
            dist.destroy_process_group()
        return

    if name == "mlp":
        wl = MlpWorkload(torch, T, args.batch or 4096, use_graph=not args.eager)
    elif name == "gemm":
        wl = GemmWorkload(torch, T, args.size, args.precision)
    elif name == "gemm512":
        wl = Gemm512Workload(torch, T)
    elif name == "gemm_sharded":
        wl = ShardedGemmWorkload(torch, dist, T, args.size, world, rank)
    elif name == "conv":
        wl = ConvWorkload(torch, T, args.batch or 256)
    elif name == "cnn":
        wl = CnnWorkload(torch, T, args.batch or 8192, fuse_pool=not args.unfused_pool, use_graph=not args.eager)
    elif name == "add":
        wl = AddWorkload(torch, T, args.size if args.size != 16384 else 1 << 28)
    elif name in HbmWorkload.OPS:
        wl = HbmWorkload(torch, T, name, args.size if args.size != 16384 else 1 << 28)
    else:
        wl = KernelFamilyWorkload(torch, T, name)

    # the tensor pipe's ceiling, measured first on rank 0 (the other ranks wait at the next barrier)
    mma = None
    if rank == 0 and (wl.bound == "tensor" or headline) and not args.no_peak:
        mma = measured_mma_peaks(lib, check, sampler)

    m = bench.measure(wl, args.steps, args.warmup, min_gpu_s=1.0 if headline else 0.0, min_blocks=3)
    ms_per_step = m["ms_per_step"]
    # whole-job aggregate: a rank's units per step (its share, for a strong-scaling job) x ranks
    value = wl.units_per_step() * world / (ms_per_step / 1e3)

    # end to end through host buffers
    flush = bench.flush_for(wl)
    e2e = None
    if hasattr(wl, "e2e_step") or hasattr(wl, "e2e_run"):
        streamed = hasattr(wl, "e2e_run") and not args.eager
        if streamed:
            wl.e2e_run(3, flush)
            e2e_steps = max(1, args.steps)
            bench.barrier()
            t0 = time.perf_counter()
            e2e_ms_dev = wl.e2e_run(e2e_steps, flush)
            bench.barrier()
        else:
            for _ in range(2):
                wl.e2e_step()
            e2e_steps = max(1, min(args.steps, 10))
            bench.barrier()
            t0 = time.perf_counter()
            e2e_ms_dev = bench.timed(wl.e2e_step, e2e_steps, flush)
        e2e_wall = time.perf_counter() - t0
        T.check_async()
        e2e_ms = bench.reduce_max(max(e2e_ms_dev, 0.0))
        e2e_units = getattr(wl, "e2e_units_per_step", wl.units_per_step)()
        e2e = {"value": e2e_units * e2e_steps * world / (e2e_ms / 1e3), "unit": wl.unit,
               "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "steps": e2e_steps, "wall_s": e2e_wall,
               "mode": "copy in / kernels / copy out of consecutive steps overlapped on three streams"
               if streamed else "copy in, kernels, copy out one after the other, each step"}
        if wl.h2d:
            e2e["h2d_ceiling_gbs_per_gpu"] = h2d_ceiling(bench, wl.h2d)
            e2e["h2d_gbs_per_gpu_achieved"] = wl.h2d * e2e_steps / (e2e_ms / 1e3) / 1e9

    plugin = None
    if name == "mlp" and not args.eager:
        if hasattr(wl, "pipe") and wl.pipe is not None:
            wl.pipe.close()
            wl.pipe = None
        plugin = plugin_leg(args, wl.batch, bench.reduce_max)

    extras = run_extras(bench, args, pk, mma) if headline and not args.no_extras else None
    training = training_leg(lib) if headline and not args.no_extras and rank == 0 else None

    if rank == 0:
        roofline = roofline_of(wl, m, pk, mma, args.precision)
        cpu = cpu_baseline(args) if world == 1 and not args.no_cpu_baseline else None
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, f32 accumulate)"
                if args.precision != "bf16" else "bf16 in / f32 accumulate", "data": "synthetic",
                "config": {"parallelism": f"{world} ranks, independent shards, no data-path collective",
                           **wl.config(), "l2": "flushed between steps" if m["flush"] else "inputs larger than L2"},
                "timed_region": {"blocks_of_steps": m["blocks"], "gpu_s": m["gpu_s"],
                                 "rule": "blocks of exactly `steps` timed steps; ms_per_step is the median block's"},
                "gpu_launches": m["launches"], "roofline": roofline, "clocks": m["clocks"],
                "kernel_families_per_step": m["scopes"]}
        if plugin is not None:
            # the headline end-to-end figure: through the plugin's operator bodies, host buffers in and out
            fused = plugin["fused_operators"]
            line["e2e"] = {"value": wl.batch * world / fused["seconds_per_step"], "unit": wl.unit,
                           "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                           "seconds_per_step": fused["seconds_per_step"], "launches_per_step": fused["launches_per_step"],
                           "mode": "per step: host batch in page-locked memory -> tensor (one synchronous copy), dense_relu, "
                                   "dense_relu, dense_softmax, argmax through operator_t, host read-back of both results; "
                                   "wall clock in C++ around the step, median step, slowest rank"}
            pageable = plugin["fused_operators_pageable"]
            line["e2e_plugin_pageable_host"] = {
                "value": wl.batch * world / pageable["seconds_per_step"], "unit": wl.unit,
                "seconds_per_step": pageable["seconds_per_step"],
                "mode": "the same step with the host batch in ordinary (pageable) memory, where the reference's "
                        "allocator keeps large tensors: the copy is staged by the driver"}
            small = plugin["small_operators"]
            line["e2e_plugin_small_operators"] = {
                "value": wl.batch * world / small["seconds_per_step"], "unit": wl.unit,
                "seconds_per_step": small["seconds_per_step"], "launches_per_step": small["launches_per_step"],
                "mode": "the same step written with the module's small operators (x @ w, h * (h > 0), the softmax "
                        "function of mnist.cml:13-25): deferred expressions recognised and fused by the plugin"}
            if e2e is not None:
                line["e2e_pipelined"] = e2e
        elif e2e is not None:
            line["e2e"] = e2e
        if mma is not None:
            line["mma_peak"] = mma
        if extras is not None:
            line["extras"] = extras
        if training is not None:
            line["plugin_training_step"] = training
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if sampler is not None:
        sampler.stop()
    if dist is not None:
        dist.destroy_process_group()


def ctypes_double():
    import ctypes
    return ctypes.c_double()


def ctypes_u64():
    import ctypes
    return ctypes.c_uint64()


def cpu_baseline(args):
    """Rank 0, N=1: the reference CPU operators on a bounded sample of the same workload."""
    import contextlib
    import io

    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        run_reference(args, 0)
    try:
        ref = json.loads(buf.getvalue().strip().splitlines()[-1])
    except (ValueError, IndexError):
        return None
    return ref.get("cpu_baseline")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="default",
                    choices=["default", "mlp", "gemm", "gemm512", "gemm_sharded", "conv", "cnn", "add", "relu", "exp", "log",
                             "mul", "scale", "gt", "sum", "softmax", "sum_axis0", "sum_axis1", "max_axis1",
                             "argmax_axis1", "argmax_rows", "transpose", "maxpool", "fill", "split_rows", "mma_peak"],
                    help="default: the MLP forward as the headline plus every other workload under `extras`")
    ap.add_argument("--no-extras", action="store_true", help="the headline only")
    ap.add_argument("--no-peak", action="store_true",
                    help="skip the tensor-pipe measurement (thousands of launches: unwanted under a profiler); the "
                         "roofline then falls back to the figure derived from the driver-written bf16 GEMM peak")
    ap.add_argument("--unfused-pool", action="store_true", help="cnn: conv2d then maxpool2d instead of the fused call")
    ap.add_argument("--size", type=int, default=16384)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "bf16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-workers", type=int, default=0, help="processes of the reference arm (0: one per core, max 32)")
    ap.add_argument("--eager", action="store_true", help="do not replay the forward pass as a CUDA graph")
    ap.add_argument("--no-weight-cache", action="store_true",
                    help="transpose and split the weights of every dense layer at every call instead of once per tensor")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_gpu(args, rank, world)


if __name__ == "__main__":
    main()
