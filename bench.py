#!/usr/bin/env python
"""Headline benchmark: square GEMM C = A·B at M=N=K=8192 through the C-ABI of libtfb.so.

One "step" is one FP32 product (error-compensated 3xTF32 on the tcgen05 tensor cores: one
launch that splits both operands plus the GEMM launch). The same run also measures the BF16-input /
FP32-accumulate product, the GEMM kernel alone for the roofline, and the end-to-end path with
host buffers (pinned host -> device copies, product, device -> host copy inside the timed region).

N GPUs (one process per GPU under torch.distributed.run): weak scaling by M row-panels — every rank
multiplies its own 8192-row panel of A by a replicated B; there is no data-path collective.

`--impl reference` times the reference's own CPU Tensor::matmul (the unmodified reference compiled
into oracle/_ref, else the C restatement in oracle/) on row panels of the same product.
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

    def summary(self, t0, t1):
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
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": self.sm_max, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
def reference_arm(args, rank):
    """The reference's own CPU matmul on row panels of the 8192^3 product, all host threads."""
    if rank != 0:
        return
    import numpy as np
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
def ours(args, rank, world, local_rank):
    import numpy as np
    import torch
    import torch.distributed as dist

    import refdata
    import tensors_b200.capi as capi

    lib = capi.lib
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL announces its version on stdout at this level; stdout carries the one JSON line only.
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    capi.check(lib.tfb_init())
    n = args.n
    peaks, peak_src = load_peaks()

    def stream():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    # Inputs: uniform[-1,1); B is replicated, each rank owns its own row panel of A.
    A_h = torch.from_numpy(refdata.uniform(1000 + rank, (n, n))).pin_memory()
    B_h = torch.from_numpy(refdata.uniform(1, (n, n))).pin_memory()
    C_h = torch.empty((n, n), dtype=torch.float32).pin_memory()
    A = A_h.cuda(non_blocking=True)
    B = B_h.cuda(non_blocking=True)
    C = torch.empty((n, n), device="cuda", dtype=torch.float32)
    A16, B16 = A.to(torch.bfloat16), B.to(torch.bfloat16)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t1 = time.time()
        return max_over_ranks(e0.elapsed_time(e1) / steps), t0, t1

    def step_fp32():
        capi.check(lib.tfb_matmul(p(A), p(B), p(C), n, n, n, capi.DTYPE_F32, capi.DTYPE_F32, stream()))

    def step_bf16():
        capi.check(lib.tfb_matmul(p(A16), p(B16), p(C), n, n, n, capi.DTYPE_BF16, capi.DTYPE_F32, stream()))

    def step_e2e():
        # host buffers in, host buffer out: uploads, product and download pipelined inside the call
        capi.check(lib.tfb_matmul_host(ctypes.c_void_p(A_h.data_ptr()), ctypes.c_void_p(B_h.data_ptr()),
                                       ctypes.c_void_p(C_h.data_ptr()), n, n, n, capi.DTYPE_F32, stream()))

    flops = 2.0 * n * n * n
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    # GEMM kernel alone (operands split beforehand): the roofline numerator.
    hi_lo = torch.empty((4, n, n), device="cuda", dtype=torch.float32)
    capi.check(lib.tfb_split_tf32(p(A), n, n, n, p(hi_lo[0]), p(hi_lo[1]), n, stream()))
    capi.check(lib.tfb_split_tf32(p(B), n, n, n, p(hi_lo[2]), p(hi_lo[3]), n, stream()))

    def step_kernel():
        capi.check(lib.tfb_gemm_presplit(p(hi_lo[0]), p(hi_lo[1]), p(hi_lo[2]), p(hi_lo[3]), p(C), n, n, n, n, n, n,
                                         0, 0, None, 0, stream()))

    ms32, t0, t1 = timed(step_fp32, args.steps, args.warmup)
    clocks = sampler.summary(t0, t1) if rank == 0 else None
    msk, _, _ = timed(step_kernel, args.steps, args.warmup)
    ms16, t0b, t1b = timed(step_bf16, args.steps, args.warmup)
    clocks16 = sampler.summary(t0b, t1b) if rank == 0 else None
    del hi_lo
    mse, _, _ = timed(step_e2e, max(2, args.steps // 2), 3)
    if rank == 0:
        sampler.stop()
    status = capi.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # CPU baseline on a bounded sample, and a parity spot check of the rows it produced.
    cpu = None
    parity = None
    if world == 1 and not args.no_cpu_baseline:
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

    tf32_peak = peaks["bf16_tflops"] / 6.0
    value = world * flops / (ms32 * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms32, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"square GEMM M=N=K={n} per GPU (FP32 in/out, 3xTF32 on tcgen05), uniform[-1,1) seeded; "
                               f"N GPUs: M row-panels of {n} rows each, B replicated, no communication",
                   "n": n, "l2": "operands and output (268 MB each) exceed the 126 MB L2; no flush needed",
                   "parallelism": f"row-panels x{world}"},
        "roofline": {"bound": "tensor", "achieved": flops / (msk * 1e-3) / 1e12, "peak": tf32_peak, "unit": "TFLOP/s",
                     "frac": flops / (msk * 1e-3) / 1e12 / tf32_peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch at n = 8192, from the ncu
                     # capture summarised in profiles/bench_8192_launch_list_and_dram.md (algorithmic: 1.34e9)
                     "traffic": (7.36e9 + 0.268e9) if n == 8192 else None,
                     "kernel": "gemm_tcgen05_kernel<TF32x3,BN=256,CTA pair> alone, operands pre-split",
                     "peak_source": f"{peak_src} bf16_tflops {peaks['bf16_tflops']} / 6 (TF32 issues at half the BF16 "
                                    f"rate and three products make one FP32 product)",
                     "kernel_ms": msk},
        "bf16": {"value": world * flops / (ms16 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms16,
                 "dtype": "bf16 in, f32 accumulate and out",
                 "roofline": {"bound": "tensor", "achieved": flops / (ms16 * 1e-3) / 1e12,
                              "traffic": (1.10e9 + 0.252e9) if n == 8192 else None,
                              "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                              "frac": flops / (ms16 * 1e-3) / 1e12 / peaks["bf16_tflops"],
                              "peak_source": f"{peak_src} bf16_tflops (burst)"},
                 "clocks": clocks16},
        "e2e": {"value": world * flops / (mse * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": mse,
                "h2d_bytes_per_step": 2 * n * n * 4, "d2h_bytes_per_step": n * n * 4},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
        "device_status": status,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
        line["parity_rel_err_vs_cpu_rows"] = parity
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
