#!/usr/bin/env python
"""Headline benchmark: square GEMM C = A·B at M=N=K=8192 through the C-ABI of libtfb.so.

One "step" is one FP32 product (error-compensated 3xTF32 on the tcgen05 tensor cores: one launch that
splits both operands plus the GEMM launch). Every timed loop runs after a pre-heat of at least one
second of the same work, so all figures of a line are taken in the same (power-capped) clock state,
and every loop carries its own clock samples. The same line also holds:

  roofline      the GEMM kernel alone (operands pre-split), timed right before and right after the
                headline loop, against the measured BF16 peak / 6
  timing        the headline is the mean over back-to-back K-step blocks covering at least two seconds
                (under the power cap one K-step block is only a sample of a wandering clock state)
  bf16          the BF16-input / FP32-accumulate product
  e2e           the product through tfb_matmul_host: pinned host buffers in and out, copies inside the
                timed region
  sweep         the five sizes of the square sweep, FP32 and BF16
  strong_16384  one 16384^3 product split into N row panels (B staged per GPU beforehand): the one
                point of the curve that is not embarrassingly parallel in its size
  mlp_dp        the data-parallel MLP training step (784-1024-1024-10, global batch 8192 sharded over
                the ranks, SGD lr 0.1 momentum 0.9): step time with the fused peer-memory exchange and
                with one NCCL all-reduce, the exchange alone, and loss + gradient norm after exactly one
                step from identical parameters next to the single-rank values
  cpu_baseline  the reference's own CPU Tensor::matmul on a bounded sample (rank 0, N = 1 only)

N GPUs (one process per GPU under torch.distributed.run): weak scaling by M row-panels — every rank
multiplies its own 8192-row panel of A by a replicated B; there is no data-path collective in the
headline. `--impl reference` times the reference's own CPU Tensor::matmul (the unmodified reference
compiled into oracle/_ref, else the C restatement in oracle/) on row panels of the same product.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "GEMM TFLOPS (3xTF32-FP32 & BF16) and % tensor-pipe peak at 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MLP_DIMS, MLP_BATCH, MLP_FLOP = (784, 1024, 1024, 10), 8192, 78.35e9


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons through NVML while a timed region runs.
    Read-only: no clock, power or mode setting is touched."""

    REASONS = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
               ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.sm_max = None
        self._stop = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber devices; resolve through the CUDA device's UUID.
            import torch
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            return

        def pump():
            while not self._stop.is_set():
                try:
                    mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                    try:
                        mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception:
                        mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                    self.samples.append((time.time(), mhz, mask))
                except Exception:
                    pass
                self._stop.wait(0.002)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self, t0, t1, ms=None):
        sm, reasons = [], set()
        for ts, mhz, mask in self.samples:
            if ts < t0 or ts > t1:
                continue
            sm.append(mhz)
            for name, bit in self.REASONS:
                if mask & bit:
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": self.sm_max, "reasons": sorted(reasons),
               "samples": len(sm)}
        if ms is not None:
            out["ms_x_mhz"] = ms * out["sm_mhz"]   # clock-normalised time: compare these between loops
        return out


# ------------------------------------------------------------------------------------------
def reference_arm(args, rank):
    """The reference's own CPU matmul on row panels of the 8192^3 product, all host threads."""
    if rank != 0:
        return
    import refdata
    from oracle_lib import Oracle, Reference, have_reference

    n = args.n
    threads = max(1, min(os.cpu_count() or 1, args.cpu_threads or (os.cpu_count() or 1)))
    rows_per_thread = args.cpu_rows
    B = refdata.uniform(1, (n, n))
    A = refdata.uniform(0, (threads * rows_per_thread, n))
    if have_reference():
        ref = Reference()
        held = ref.hold_matrix(B)
        kind = "reference"

        def panel(i):
            ref.matmul_held(A[i * rows_per_thread:(i + 1) * rows_per_thread], held)
    else:
        orc = Oracle()
        orc.lib.orc_set_threads(1)
        kind = "port"

        def panel(i):
            orc.matmul(A[i * rows_per_thread:(i + 1) * rows_per_thread], B, mt=False)

    def step():
        ts = [threading.Thread(target=panel, args=(i,)) for i in range(threads)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * threads * rows_per_thread * n * n
    value = flops / dt / 1e12
    sample = (f"{threads} concurrent Tensor::matmul calls per step, each a {rows_per_thread}-row panel of A "
              f"times the full {n}x{n} B ({threads * rows_per_thread} of {n} rows; rate extrapolates linearly)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"square GEMM M=N=K={n}, FP32, CPU Tensor::matmul on row panels", "n": n},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
class Harness:
    """Timing plumbing shared by the sections: CUDA events on the launching stream, barrier +
    synchronize on both sides, maximum over ranks, a pre-heat of the same work, clock samples."""

    def __init__(self, rank, world, local_rank, sampler):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local_rank, self.sampler = rank, world, local_rank, sampler

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def preheat(self, fn, seconds, min_steps):
        """At least min_steps calls of fn and about `seconds` of device time. Every rank runs the SAME
        number of calls (fn may contain a collective): the count comes from a first timed batch whose
        duration is the maximum over ranks."""
        torch = self.torch
        first = max(4, int(min_steps))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(first):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = self.max_over_ranks(e0.elapsed_time(e1) / first)
        extra = int(max(0.0, seconds * 1e3 - ms * first) / max(ms, 1e-3))
        for _ in range(min(extra, 200000)):
            fn()
        torch.cuda.synchronize()

    def timed(self, fn, steps, warmup, preheat_s=1.0):
        torch = self.torch
        self.preheat(fn, preheat_s, warmup)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        t1 = time.time()
        ms = self.max_over_ranks(e0.elapsed_time(e1) / steps)
        clocks = self.sampler.summary(t0, t1, ms) if self.rank == 0 else None
        return ms, clocks

    def timed_blocks(self, fn, steps, warmup, seconds, preheat_s=1.0):
        """The K-step measurement repeated back to back until at least `seconds` of device time are
        covered: under the power cap the clock state of a B200 wanders on a scale of hundreds of
        milliseconds, so one K-step block is a sample of it and the mean over blocks is the figure that
        repeats. Every block is exactly `steps` calls bracketed by CUDA events; nothing synchronises
        between blocks. Returns (mean, fastest, slowest) ms per step, maximum over ranks, the clock
        summary and the number of blocks."""
        torch = self.torch
        self.preheat(fn, preheat_s, warmup)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        hint = self.max_over_ranks(e0.elapsed_time(e1))          # ms of one block, the same on every rank
        blocks = max(1, int(seconds * 1e3 / max(hint, 1e-3)) + 1)
        self.barrier()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
        t0 = time.time()
        marks[0].record()
        for b in range(blocks):
            for _ in range(steps):
                fn()
            marks[b + 1].record()
        self.barrier()
        t1 = time.time()
        per = [marks[b].elapsed_time(marks[b + 1]) / steps for b in range(blocks)]
        mean = self.max_over_ranks(sum(per) / blocks)
        lo, hi = self.max_over_ranks(min(per)), self.max_over_ranks(max(per))
        clocks = self.sampler.summary(t0, t1, mean) if self.rank == 0 else None
        return {"ms": mean, "ms_fastest_block": lo, "ms_slowest_block": hi, "blocks": blocks,
                "steps_per_block": steps, "seconds": mean * steps * blocks / 1e3, "clocks": clocks}


def section_gemm(h, args, capi, lib, peaks, peak_src):
    import refdata
    torch = h.torch
    n = args.n

    def stream():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    # Inputs: uniform[-1,1); B is replicated, each rank owns its own row panel of A.
    A_h = torch.from_numpy(refdata.uniform(1000 + h.rank, (n, n))).pin_memory()
    B_h = torch.from_numpy(refdata.uniform(1, (n, n))).pin_memory()
    C_h = torch.empty((n, n), dtype=torch.float32).pin_memory()
    A = A_h.cuda(non_blocking=True)
    B = B_h.cuda(non_blocking=True)
    C = torch.empty((n, n), device="cuda", dtype=torch.float32)
    A16, B16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
    torch.cuda.synchronize()

    def step_fp32():
        capi.check(lib.tfb_matmul(p(A), p(B), p(C), n, n, n, capi.DTYPE_F32, capi.DTYPE_F32, stream()))

    def step_bf16():
        capi.check(lib.tfb_matmul(p(A16), p(B16), p(C), n, n, n, capi.DTYPE_BF16, capi.DTYPE_F32, stream()))

    # With several ranks B is the same matrix everywhere: every rank uploads rows [k0, k1) of it, the
    # slices are exchanged over NVLink (one NCCL all-gather) and B crosses the host link once in total.
    if h.world > 1:
        assert n % h.world == 0
        kb = n // h.world
        B_slice_h = B_h[h.rank * kb:(h.rank + 1) * kb]
        B_stage = torch.empty((n, n), device="cuda", dtype=torch.float32)

    def step_e2e():
        # host buffers in, host buffer out: uploads, product and download pipelined inside the call
        if h.world == 1:
            capi.check(lib.tfb_matmul_host(ctypes.c_void_p(A_h.data_ptr()), ctypes.c_void_p(B_h.data_ptr()),
                                           ctypes.c_void_p(C_h.data_ptr()), n, n, n, capi.DTYPE_F32, stream()))
            return
        mine = B_stage[h.rank * kb:(h.rank + 1) * kb]
        mine.copy_(B_slice_h, non_blocking=True)
        h.dist.all_gather_into_tensor(B_stage, mine)
        capi.check(lib.tfb_matmul_host_b_resident(ctypes.c_void_p(A_h.data_ptr()), p(B_stage),
                                                  ctypes.c_void_p(C_h.data_ptr()), n, n, n, capi.DTYPE_F32, stream()))

    flops = 2.0 * n * n * n
    # GEMM kernel alone (operands split beforehand): the roofline numerator. The split pass alone too.
    hi_lo = torch.empty((4, n, n), device="cuda", dtype=torch.float32)
    capi.check(lib.tfb_split_tf32(p(A), n, n, n, p(hi_lo[0]), p(hi_lo[1]), n, stream()))
    capi.check(lib.tfb_split_tf32(p(B), n, n, n, p(hi_lo[2]), p(hi_lo[3]), n, stream()))

    def step_kernel():
        capi.check(lib.tfb_gemm_presplit(p(hi_lo[0]), p(hi_lo[1]), p(hi_lo[2]), p(hi_lo[3]), p(C), n, n, n, n, n, n,
                                         0, 0, None, 0, stream()))

    def step_split():
        capi.check(lib.tfb_split_tf32(p(A), n, n, n, p(hi_lo[0]), p(hi_lo[1]), n, stream()))
        capi.check(lib.tfb_split_tf32(p(B), n, n, n, p(hi_lo[2]), p(hi_lo[3]), n, stream()))

    # kernel alone -> full step -> kernel alone; each figure is the mean over back-to-back K-step blocks
    # that cover >= 1 s (kernel alone) or >= 2 s (the step), after a pre-heat of the same work
    k0 = h.timed_blocks(step_kernel, args.steps, args.warmup, 1.0)
    full = h.timed_blocks(step_fp32, args.steps, args.warmup, 2.0)
    k1 = h.timed_blocks(step_kernel, args.steps, args.warmup, 1.0, preheat_s=0.2)
    split = h.timed_blocks(step_split, args.steps, args.warmup, 0.3, preheat_s=0.2)
    half = h.timed_blocks(step_bf16, args.steps, args.warmup, 2.0)
    del hi_lo
    mse, clocks_e = h.timed(step_e2e, max(2, args.steps // 2), 3, preheat_s=0.0)
    ms32, ms16 = full["ms"], half["ms"]

    parity = None
    cpu = None
    if h.rank == 0 and h.world == 1 and not args.no_cpu_baseline:
        import numpy as np
        from oracle_lib import Oracle, Reference, have_reference
        rows = args.cpu_rows * 4
        a_rows = A_h[:rows].numpy()
        b_np = B_h.numpy()
        t0c = time.perf_counter()
        if have_reference():
            ref = Reference()
            held = ref.hold_matrix(b_np)
            t0c = time.perf_counter()
            want = ref.matmul_held(a_rows, held)
            kind = "reference"
        else:
            orc = Oracle()
            want = orc.matmul(a_rows, b_np, mt=False)
            kind = "port"
        dtc = time.perf_counter() - t0c
        cpu = {"value": 2.0 * rows * n * n / dtc / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
               "sample": f"Tensor::matmul on the first {rows} rows of A times the full {n}x{n} B, one thread "
                         f"({dtc:.1f} s); the rate extrapolates linearly to all {n} rows"}
        step_fp32()
        torch.cuda.synchronize()
        got = C[:rows].cpu().numpy().astype(np.float64)
        parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))

    if h.rank != 0:
        return None
    w = h.world
    msk = 0.5 * (k0["ms"] + k1["ms"])
    tf32_peak, tf32_peak_sus = peaks["bf16_tflops"] / 6.0, peaks["bf16_tflops_sustained"] / 6.0
    ach = flops / (msk * 1e-3) / 1e12
    tf = lambda ms: flops / (ms * 1e-3) / 1e12
    out = {
        "value": w * tf(ms32), "ms_per_step": ms32, "clocks": full["clocks"],
        "timing": {"blocks": full["blocks"], "steps_per_block": full["steps_per_block"], "seconds": full["seconds"],
                   "fastest_block_tflops": w * tf(full["ms_fastest_block"]),
                   "slowest_block_tflops": w * tf(full["ms_slowest_block"]),
                   "note": "value = mean over back-to-back K-step blocks (>= 2 s); the fastest block is the burst figure"},
        "roofline": {"bound": "tensor", "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s", "frac": ach / tf32_peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch at n = 8192 from a one-pass
                     # ncu capture of this command (algorithmic bytes: 1.34e9); other sizes: not captured
                     "traffic": (7.78e9 + 0.274e9) if n == 8192 else None,
                     "kernel": "gemm_tcgen05_kernel<TF32x3,BN=256,CTA pair> alone, operands pre-split",
                     "peak_source": f"{peak_src} bf16_tflops {peaks['bf16_tflops']} (burst) / 6: TF32 issues at half the "
                                    f"BF16 rate and three products make one FP32 product",
                     "frac_of_sustained_peak": ach / tf32_peak_sus,
                     "burst_achieved": tf(min(k0["ms_fastest_block"], k1["ms_fastest_block"])),
                     "kernel_ms": msk, "kernel_ms_before_step": k0["ms"], "kernel_ms_after_step": k1["ms"],
                     "split_ms": split["ms"], "clocks_before": k0["clocks"], "clocks_after": k1["clocks"],
                     "step_minus_kernel_minus_split_ms": ms32 - msk - split["ms"],
                     "consistent": bool(ms32 >= msk)},
        "bf16": {"value": w * tf(ms16), "unit": "TFLOP/s", "ms_per_step": ms16,
                 "dtype": "bf16 in, f32 accumulate and out",
                 "fastest_block_tflops": w * tf(half["ms_fastest_block"]), "blocks": half["blocks"],
                 "roofline": {"bound": "tensor", "achieved": tf(ms16),
                              "traffic": (1.10e9 + 0.252e9) if n == 8192 else None,
                              "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                              "frac": tf(ms16) / peaks["bf16_tflops"],
                              "peak_source": f"{peak_src} bf16_tflops (burst); the loop itself runs for seconds under "
                                             f"the power cap, where the same library GEMM sustains "
                                             f"{peaks['bf16_tflops_sustained']}",
                              "frac_of_sustained_peak": tf(ms16) / peaks["bf16_tflops_sustained"],
                              "burst_frac": tf(half["ms_fastest_block"]) / peaks["bf16_tflops"]},
                 "clocks": half["clocks"]},
        "e2e": {"value": w * flops / (mse * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": mse,
                "h2d_bytes_per_step": n * n * 4 + n * n * 4 // w, "d2h_bytes_per_step": n * n * 4, "clocks": clocks_e,
                "note": "per rank: its panel of A, and 1/N of the shared B (the rest arrives over NVLink by one "
                        "all-gather)" if w > 1 else "A and B uploaded, C downloaded, inside the call"},
    }
    if cpu is not None:
        out["cpu_baseline"] = cpu
        out["parity_rel_err_vs_cpu_rows"] = parity
    return out


def section_sweep(h, args, capi, lib):
    """The five square sizes, FP32 (3xTF32) and BF16 inputs, per GPU (every rank runs it; rank 0 reports
    the maximum time over ranks)."""
    import refdata
    torch = h.torch
    rows = []
    for n in (1024, 2048, 4096, 8192, 16384):
        if n == 16384 and args.skip_16384:
            continue
        src = torch.from_numpy(refdata.uniform(5, (min(n, 4096), n))).cuda()
        A = src.repeat((n + src.shape[0] - 1) // src.shape[0], 1)[:n].contiguous()
        B = A.flip(0).contiguous()
        C = torch.empty((n, n), device="cuda")
        st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        steps = 20 if n <= 8192 else 5
        f32 = lambda: capi.check(lib.tfb_matmul(p(A), p(B), p(C), n, n, n, 0, 0, st()))
        ms, _ = h.timed(f32, steps, 3, preheat_s=0.3)
        A16, B16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
        del A, B
        b16 = lambda: capi.check(lib.tfb_matmul(p(A16), p(B16), p(C), n, n, n, 2, 0, st()))
        ms16, _ = h.timed(b16, steps, 3, preheat_s=0.3)
        rows.append({"n": n, "fp32_ms": ms, "fp32_tflops": 2.0 * n ** 3 / ms / 1e9, "bf16_ms": ms16,
                     "bf16_tflops": 2.0 * n ** 3 / ms16 / 1e9})
        del A16, B16, C, src
        torch.cuda.empty_cache()
    return rows


def section_strong(h, args, capi, lib):
    """One 16384^3 FP32 product split into `world` row panels; B is staged on every GPU before timing."""
    import refdata
    torch = h.torch
    n = 16384
    from tensors_b200.mlp import shard_rows
    b, e = shard_rows(n, h.rank, h.world)
    src = torch.from_numpy(refdata.uniform(6, (2048, n))).cuda()
    B = src.repeat(n // 2048, 1).contiguous()
    A = src.flip(1).repeat((e - b + 2047) // 2048, 1)[:e - b].contiguous()
    C = torch.empty((e - b, n), device="cuda")
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = lambda: capi.check(lib.tfb_matmul(p(A), p(B), p(C), e - b, n, n, 0, 0, st()))
    ms, clocks = h.timed(fn, 6, 2, preheat_s=0.5)
    out = {"ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9, "rows_per_gpu": e - b, "scaling": "strong",
           "what": "16384^3 FP32 (3xTF32) split into row panels, B resident on every GPU, no communication",
           "clocks": clocks}
    del A, B, C, src
    torch.cuda.empty_cache()
    return out


def section_mlp(h, args, capi, lib):
    """The data-parallel MLP step (see the module docstring)."""
    import numpy as np
    import refdata
    from tensors_b200.mlp import MLP, shard_rows
    torch, dist = h.torch, h.dist
    dims, batch = MLP_DIMS, MLP_BATCH
    ws = [refdata.linear_weight(dims[i], dims[i + 1]) for i in range(3)]
    x_all, l_all = refdata.mnist_like(7, (batch, 784)), refdata.labels(8, batch)
    b, e = shard_rows(batch, h.rank, h.world)
    X_h = torch.from_numpy(x_all[b:e]).pin_memory()
    L_h = torch.from_numpy(l_all[b:e]).pin_memory()
    X, L = X_h.cuda(), L_h.cuda()
    out = {"config": "MLP 784-1024-1024-10, ReLU, log_softmax + NLL, SGD lr 0.1 momentum 0.9, global batch 8192 "
                     f"sharded over {h.world} rank(s) ({e - b} rows each)", "flop_per_step": MLP_FLOP}

    def one_step(m, Xs, Ls):
        m.set_option(MLP.OPT_KEEP_REDUCED, 1)
        m.train_step(Xs, Ls, lr=0.1, momentum=0.9, global_rows=batch)
        torch.cuda.synchronize()
        lo, hi = (0, m.numel) if not m._use_peer() else (4 * ((m.numel // 4) * h.rank // h.world),
                                                         4 * ((m.numel // 4) * (h.rank + 1) // h.world))
        g2 = (m.reduced[lo:hi].double() ** 2).sum()
        if m._use_peer():
            dist.all_reduce(g2)
        m.set_option(MLP.OPT_KEEP_REDUCED, 0)
        return float(m.loss.item()), float(g2.sqrt().item()), float(m.params.double().norm().item())

    # ---- exactly one step from identical parameters: N ranks next to one rank -------------------
    peer_ok = True
    m = MLP(dims, ws, max_rows=e - b, exchange="peer")
    if h.world > 1:
        try:
            m.connect()
        except Exception as ex:   # CUDA IPC unavailable in this container: report it, keep the NCCL path
            peer_ok = False
            out["peer_exchange_unavailable"] = str(ex)[:200]
        flag = torch.tensor([1.0 if peer_ok else 0.0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        peer_ok = bool(flag.item() > 0)
        if not peer_ok:
            m.exchange = "nccl"
    loss, gnorm, pnorm = one_step(m, X, L)
    out["one_step"] = {"loss": loss, "grad_norm": gnorm, "param_norm_after": pnorm}
    if h.world > 1 and h.rank == 0:
        m1 = MLP(dims, ws, max_rows=batch, exchange="local")
        X1, L1 = torch.from_numpy(x_all).cuda(), torch.from_numpy(l_all).cuda()
        loss1, gnorm1, pnorm1 = one_step(m1, X1, L1)
        out["one_step"].update({"loss_1rank": loss1, "grad_norm_1rank": gnorm1, "param_norm_after_1rank": pnorm1,
                                "loss_rel_diff": abs(loss - loss1) / abs(loss1),
                                "grad_norm_rel_diff": abs(gnorm - gnorm1) / gnorm1,
                                "params_rel_diff": float((m.params - m1.params).double().norm().item() / pnorm1)})
        del m1, X1, L1
    h.barrier()

    # ---- step time: whole step as one CUDA graph (peer exchange inside) ---------------------------
    def h2d():
        X.copy_(X_h, non_blocking=True)
        L.copy_(L_h, non_blocking=True)

    replay = m.capture_train_step(X, L, lr=0.1, momentum=0.9, global_rows=batch, warmup=2)
    us, clocks = h.timed(replay, 50, 5, preheat_s=0.5)
    out.update({"step_us": us * 1e3, "tflops": MLP_FLOP / (us * 1e-3) / 1e12, "exchange": m.exchange if h.world > 1 else "none",
                "clocks": clocks})

    # End to end as a training loop feeds it: every step's batch crosses the host link inside the timed region,
    # but one step ahead — batch i + 1 is uploaded on a copy stream into the other of two device buffers while
    # step i computes — and every step ends with the device -> host read of its loss.
    copy_stream = torch.cuda.Stream()
    bufs = [(X, L), (torch.empty_like(X), torch.empty_like(L))]
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    state = {"i": 0}

    def upload(i):
        Xd, Ld = bufs[i & 1]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i & 1])    # the step that last read this buffer has finished with it
            Xd.copy_(X_h, non_blocking=True)
            Ld.copy_(L_h, non_blocking=True)
            copied[i & 1].record(copy_stream)

    for ev in consumed:
        ev.record()
    upload(0)

    def e2e_step():
        i = state["i"]
        state["i"] = i + 1
        upload(i + 1)
        Xd, Ld = bufs[i & 1]
        torch.cuda.current_stream().wait_event(copied[i & 1])
        m.train_step(Xd, Ld, lr=0.1, momentum=0.9, global_rows=batch)
        consumed[i & 1].record()
        return m.loss.item()   # the device -> host read of the step's result

    us_e, _ = h.timed(e2e_step, 30, 3, preheat_s=0.2)
    torch.cuda.synchronize()
    out["e2e_step_us"] = us_e * 1e3
    out["e2e_h2d_bytes_per_step"] = int(X_h.numel() * 4 + L_h.numel() * 8)
    out["e2e_note"] = "eager steps; the next batch is uploaded on a copy stream while the current step computes"
    del bufs

    # ---- forward + backward alone, and the exchange alone ---------------------------------------
    fb = lambda: m.forward_backward(X, L, batch)
    us_fb, _ = h.timed(fb, 30, 3, preheat_s=0.2)
    out["forward_backward_us_eager"] = us_fb * 1e3
    if h.world > 1:
        if peer_ok:
            ex = lambda: m.exchange_update(0.0, 0.9)   # lr 0: parameters stay put while the traffic is the real one
            us_x, _ = h.timed(ex, 50, 5, preheat_s=0.2)
            out["peer_exchange_us"] = us_x * 1e3
        scratch = torch.zeros(m.numel + 4, device="cuda")
        ar = lambda: dist.all_reduce(scratch)
        us_ar, _ = h.timed(ar, 50, 5, preheat_s=0.2)
        out["nccl_allreduce_us"] = us_ar * 1e3
        # the same step with ONE NCCL all-reduce per step (loss in the last slot) and the update kernel
        m.disconnect()
        del m
        m2 = MLP(dims, ws, max_rows=e - b, exchange="nccl")
        replay2 = m2.capture_train_step(X, L, lr=0.1, momentum=0.9, global_rows=batch, warmup=2)
        us2, _ = h.timed(replay2, 50, 5, preheat_s=0.3)
        out["step_us_nccl"] = us2 * 1e3
        out["exchange_share_of_step"] = (out.get("peer_exchange_us") or out["nccl_allreduce_us"]) / out["step_us"]
        del m2
    return out


def ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import tensors_b200.capi as capi

    lib = capi.lib
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL announces its version on stdout at this level; stdout carries the one JSON line only.
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    capi.check(lib.tfb_init())
    peaks, peak_src = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    h = Harness(rank, world, local_rank, sampler)

    gemm = section_gemm(h, args, capi, lib, peaks, peak_src)
    torch.cuda.empty_cache()
    sections, errors = {}, {}
    for name, fn in (("sweep", section_sweep), ("strong_16384", section_strong), ("mlp_dp", section_mlp)):
        if name in args.skip.split(","):
            continue
        try:
            sections[name] = fn(h, args, capi, lib)
        except Exception as ex:   # a failing side section must not lose the headline; it is reported in the line
            errors[name] = f"{type(ex).__name__}: {ex}"[:300]
            if world > 1:
                raise
        torch.cuda.empty_cache()
    if rank == 0:
        sampler.stop()
    status = capi.device_status()

    if rank == 0:
        n = args.n
        line = {
            "metric": METRIC, "value": gemm["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": gemm["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"square GEMM M=N=K={n} per GPU (FP32 in/out, 3xTF32 on tcgen05), uniform[-1,1) seeded; "
                                   f"N GPUs: M row-panels of {n} rows each, B replicated, no communication",
                       "n": n, "l2": "operands and output (268 MB each) exceed the 126 MB L2; no flush needed",
                       "preheat": "every timed loop follows >= 1 s of the same work (>= the warm-up steps)",
                       "parallelism": f"row-panels x{world}"},
            "roofline": gemm["roofline"], "timing": gemm["timing"], "bf16": gemm["bf16"], "e2e": gemm["e2e"],
            # per step: split_tf32_pair_kernel + gemm_tcgen05_kernel (the launch list under profiles/)
            "gpu_launches": 2 * args.steps,
            "clocks": gemm["clocks"], "device_status": status,
        }
        for k in ("cpu_baseline", "parity_rel_err_vs_cpu_rows"):
            if k in gemm:
                line[k] = gemm[k]
        line.update(sections)
        if errors:
            line["section_errors"] = errors
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if status != 0:
        sys.exit(f"a kernel recorded device error {status}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--cpu-rows", type=int, default=8, help="rows of A per CPU-baseline panel")
    ap.add_argument("--cpu-threads", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip", default="", help="comma-separated sections to leave out: sweep,strong_16384,mlp_dp")
    ap.add_argument("--skip-16384", action="store_true", help="leave the largest size out of the sweep")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if world == 1 and args.gpus > 1:
        # Launched without torchrun: re-launch as one process per GPU on this node.
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511"] + sys.argv
        sys.exit(subprocess.call(cmd))
    ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
