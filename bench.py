#!/usr/bin/env python
"""Benchmark of the tensor hot path: `python bench.py --gpus N --steps K --warmup W`.

Workloads (seeded synthetic inputs with the shapes and distributions of the reference
configurations; no dataset is used):
  mlp    3-layer MLP forward, batch 4096, 784->1024->1024->10, relu/relu/softmax+argmax
         (metric: samples/s) - the default
  gemm   one fp32 GEMM M=N=K (default 16384, --size), 3xTF32 (or --precision bf16)
  gemm_sharded  the same product with the rows of A split over the ranks and C all-gathered in
         row panels on a side stream while the next panel computes (strong scaling)
  conv   conv2d 256x64x56x56 * 128x64x3x3, pad 1, + bias + relu
  cnn    conv32-conv64-pool-dense128-dense10 forward on 1x28x28 images, batch 8192
  add, mul, scale, relu, gt, exp, log, sum, softmax   2^28 float32 (HBM-bound)

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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


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
        return 38.1e6, ("profiles/mlp_forward_launch_list_and_gemm.md: 43.4 MB (k=1024) and 32.9 MB (k=784) per "
                        "launch = the operand planes read once; the result stays in L2")

    def resident_bytes(self):
        return self.x.nbytes + sum(t.nbytes for t in self.w) + 2 * self.batch * 1024 * 4

    def config(self):
        return {"workload": "mlp_forward 784-1024-1024-10 relu,relu,softmax+argmax (BASELINE configs[1])",
                "batch_per_gpu": self.batch, "precision": "3xtf32",
                "weights": "tensor-core layout kept with each weight tensor (built at first use)"
                if self.T._weight_cache else "transposed and split at every call"}


class GemmWorkload(Workload):
    name, metric, unit = "gemm", "gemm_fp32_tflops", "TFLOP/s"

    def __init__(self, torch, T, n, precision):
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
        self.a_host = _pin(torch, self.a_t[: self.e2e_rows].cpu().numpy())
        self.c_host = _pin_empty((self.e2e_rows, n), np.float32)
        self.h2d = self.e2e_rows * n * 4
        self.d2h = self.e2e_rows * n * 4

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
            return 690.7e6, "profiles/gemm_tc_kernel_gemm4096.md (335 MB algorithmic: operand tiles re-read 2.1x)"
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
        torch.cuda.synchronize()
        self.h2d = self.d2h = 0

    def step(self):
        import ctypes as C
        from camel_b200._lib import check, lib
        torch, n = self.torch, self.n
        check(lib.ct_rows_pack(self.a_t.data_ptr(), self.rows, n, C.byref(self.a_packed)))
        for off, cnt, g0, band0 in self.bands:
            check(lib.ct_matmul_packed_rows(self.a_packed, off, cnt, self.b_packed, self.c_t.data_ptr() + g0 * n * 4))
            if self.world > 1:
                done = torch.cuda.Event()
                done.record()
                with torch.cuda.stream(self.side):
                    self.side.wait_event(done)
                    self.sharding.gather_band(self.dist, self.c_t, band0, cnt, self.rank, self.world)
        if self.world > 1:
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
                            f"in place in {self.panels} bands of halving size overlapped with compute, B and its tensor-core layout "
                            f"placed once (BASELINE configs[4])",
                "precision": "3xtf32", "e2e": "same as value: operands are resident by construction",
                "parallelism": f"{self.world} ranks, rows of A and C sharded, NCCL all-gather of C on a side stream"}


class ConvWorkload(Workload):
    name, metric, unit = "conv", "conv2d_fp32_tflops", "TFLOP/s"

    def __init__(self, torch, T, batch):
        self.T, self.batch = T, batch
        x, w, b = conv_inputs(batch)
        self.x, self.w, self.b = T.from_numpy(x), T.from_numpy(w), T.from_numpy(b)
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
        return reads + writes, ("profiles/conv2d_and_elementwise_kernels.md: reads scaled from the batch-32 capture "
                                "by the batch, writes = the size of the result")

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
        return 12.0 * self.n, ("profiles/conv2d_and_elementwise_kernels.md: the 2^26 capture moved its algorithmic "
                               "12 B/element (reads exact, the tail of the writes still in L2); scaled by n")

    def resident_bytes(self):
        return 12 * self.n

    def config(self):
        return {"workload": f"elementwise add of {self.n} float32 (12 B/element)"}


class HbmWorkload(Workload):
    """One memory-bound operator over 2^28 float32 (or 8192 x 8192 for softmax)."""

    bound = "hbm"
    unit = "GB/s"
    #        op: (bytes per element, profile family)
    OPS = {"relu": (8, "elementwise"), "exp": (8, "elementwise"), "log": (8, "elementwise"),
           "mul": (12, "elementwise"), "scale": (8, "elementwise"), "gt": (5, "elementwise"),
           "sum": (4, "reduce"), "softmax": (8, "softmax")}

    def __init__(self, torch, T, op, n):
        if op == "softmax":
            n = min(n, 1 << 26)  # 8192 rows of 8192: a row stays in the registers of one block
        self.T, self.op, self.n = T, op, n
        self.bpe, self.dominant = self.OPS[op]
        self.name, self.metric = op, f"elementwise_{op}_gbs"
        rng = np.random.default_rng(6)
        x = rng.uniform(-1, 1, n).astype(np.float32)
        if op == "log":
            x = x + np.float32(1.0001)  # shifted to (0, 2): log throws on values <= 0
        self.x = T.from_numpy(x.reshape(8192, -1) if op == "softmax" else x)
        self.y = T.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)) if op == "mul" else None
        self.e2e_n = min(n, 1 << 24)
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
        if self.op == "mul":
            out = self.T.multiply(self.x_small, self.x_small)
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
            return float(self.bpe) * self.n, ("profiles/conv2d_and_elementwise_kernels.md: the 2^26 capture read and "
                                               "wrote every element once (8 B/element); scaled by n")
        return None, "no ncu capture of this operator"

    def resident_bytes(self):
        return self.bpe * self.n

    def config(self):
        return {"workload": f"{self.op} over {self.n} float32 ({self.bpe} B/element)"}


class CnnWorkload(Workload):
    """BASELINE configs[3]: conv 1->32 +relu, conv 32->64 +relu, 2x2 maxpool, flatten,
    dense 12544->128 +relu, dense 128->10 +softmax, on 1x28x28 Uniform(0,1) images."""

    name, metric, unit = "cnn", "cnn_forward_samples_per_s", "samples/s"

    def __init__(self, torch, T, batch):
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
        self.fuse_pool = not os.environ.get("CAMEL_BENCH_UNFUSED_POOL")

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
        self.out = self.forward(self.x)

    def e2e_step(self):
        from camel_b200._lib import check, lib
        check(lib.ct_h2d(self.x.ptr, self.x_host.data_ptr(), self.h2d))
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


def run_gpu(args, rank, world):
    import torch

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import camel_b200
    from camel_b200 import _lib, tensor as T
    from camel_b200._lib import check, lib

    check(lib.ct_set_device(local))
    check(lib.ct_set_stream(None))  # legacy default stream: ordered with torch's default stream
    if args.precision == "bf16":
        check(lib.ct_set_precision(_lib.PREC_BF16))
    T.set_weight_cache(not args.no_weight_cache)

    if args.workload == "mlp":
        wl = MlpWorkload(torch, T, args.batch or 4096, use_graph=not args.eager)
    elif args.workload == "gemm":
        wl = GemmWorkload(torch, T, args.size, args.precision)
    elif args.workload == "gemm_sharded":
        wl = ShardedGemmWorkload(torch, dist, T, args.size, world, rank)
    elif args.workload == "conv":
        wl = ConvWorkload(torch, T, args.batch or 256)
    elif args.workload == "cnn":
        wl = CnnWorkload(torch, T, args.batch or 8192)
    elif args.workload in HbmWorkload.OPS:
        wl = HbmWorkload(torch, T, args.workload, args.size if args.size != 16384 else 1 << 28)
    else:
        wl = AddWorkload(torch, T, args.size if args.size != 16384 else 1 << 28)

    flush = torch.empty(L2_BYTES * 2, dtype=torch.uint8, device="cuda") if wl.resident_bytes() < 2 * L2_BYTES else None

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps, CUDA events around each step on the launching stream, L2 flushed between
        steps when the working set is smaller than L2; returns total device ms."""
        evs = []
        barrier()
        for _ in range(steps):
            if flush is not None:
                flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        barrier()
        return sum(a.elapsed_time(b) for a, b in evs)

    for _ in range(max(args.warmup, 3)):
        wl.step()
    T.check_async()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    replayed = getattr(wl, "graph", None) is not None
    if not replayed:
        check(lib.ct_profile_enable(1))
    launches0 = lib.ct_launch_count()
    ms = timed(wl.step, args.steps)
    launches = lib.ct_launch_count() - launches0
    prof_steps = args.steps
    if replayed:
        # a replayed graph bypasses the per-launch event brackets: time the dominant kernel on
        # the same inputs, call by call, right after the timed region
        prof_steps = min(args.steps, 10)
        check(lib.ct_profile_enable(1))
        timed(wl.eager_step, prof_steps)
    tot, cnt = ctypes_double(), ctypes_u64()
    check(lib.ct_profile_read(wl.dominant.encode(), tot, cnt))
    check(lib.ct_profile_read(None, None, None))
    check(lib.ct_profile_enable(0))
    clocks = sampler.stop() if rank == 0 else None
    T.check_async()

    # end to end through host buffers
    streamed = hasattr(wl, "e2e_run") and not args.eager
    if streamed:
        wl.e2e_run(3, flush)
        e2e_steps = max(1, args.steps)
        barrier()
        t0 = time.perf_counter()
        e2e_ms_dev = wl.e2e_run(e2e_steps, flush)
        barrier()
    else:
        for _ in range(2):
            wl.e2e_step()
        e2e_steps = max(1, min(args.steps, 10))
        barrier()
        t0 = time.perf_counter()
        e2e_ms_dev = timed(wl.e2e_step, e2e_steps)
    e2e_wall = time.perf_counter() - t0
    T.check_async()

    def reduce_max(v):
        from camel_b200 import sharding
        return sharding.reduce_max(dist, torch, v, "cuda")

    ms = reduce_max(ms)
    e2e_ms = reduce_max(max(e2e_ms_dev, 0.0))
    value = wl.units_per_step() * args.steps * world / (ms / 1e3)
    e2e_units = getattr(wl, "e2e_units_per_step", wl.units_per_step)()
    e2e_value = e2e_units * e2e_steps * world / (e2e_ms / 1e3)

    if rank == 0:
        pk = peaks()
        dom_ms = tot.value / max(1, cnt.value)
        launches_per_step = cnt.value / prof_steps
        alg = wl.algorithmic_per_step() / max(1.0, launches_per_step)
        if wl.bound == "tensor":
            if args.precision == "bf16":
                peak, peak_note = pk["bf16_tflops"], f"{pk['source']} bf16 dense burst"
            else:
                peak = pk["bf16_tflops"] / 6.0
                peak_note = (f"{pk['source']} bf16 dense burst / 2 (tf32 rate) / 3 (three MMAs per product); "
                             f"sustained variant {pk['bf16_tflops_sustained'] / 6.0:.1f}")
            achieved = alg / (dom_ms / 1e3) / 1e12 if dom_ms > 0 else 0.0
            runit = "TFLOP/s"
        else:
            peak, peak_note = pk["hbm_gbs"], f"{pk['source']} STREAM-style copy"
            achieved = alg / (dom_ms / 1e3) / 1e9 if dom_ms > 0 else 0.0
            runit = "GB/s"
        traffic, traffic_note = wl.ncu_traffic() if args.precision != "bf16" else (None, "no ncu capture in bf16 mode")
        roofline = {"bound": wl.bound, "kernel": wl.dominant, "achieved": achieved, "peak": peak, "unit": runit,
                    "frac": achieved / peak if peak else None, "traffic": traffic, "traffic_unit": "bytes per launch",
                    "traffic_note": traffic_note, "peak_note": peak_note,
                    "launches_per_step": launches_per_step, "avg_launch_ms": dom_ms}
        cpu = cpu_baseline(args) if world == 1 and not args.no_cpu_baseline else None
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, f32 accumulate)"
                if args.precision != "bf16" else "bf16 in / f32 accumulate", "data": "synthetic",
                "config": {"parallelism": f"{world} ranks, independent shards, no data-path collective",
                           **wl.config(), "l2": "flushed between steps" if flush is not None else "inputs larger than L2"},
                "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                        "steps": e2e_steps, "wall_s": e2e_wall,
                        "mode": "copy in / kernels / copy out of consecutive steps overlapped on three streams"
                        if streamed else "copy in, kernels, copy out one after the other, each step"},
                "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks}
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
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
    ap.add_argument("--workload", default="mlp", choices=["mlp", "gemm", "gemm_sharded", "conv", "cnn", "add", "relu", "exp", "log", "mul", "scale", "gt", "sum",
                             "softmax"])
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
