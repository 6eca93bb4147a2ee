#!/usr/bin/env python
"""Benchmark of the sm_100a gemm path through the library's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-also]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload ("c5", the largest configured single-GPU workload and the one defined at 1/2/4/8 GPUs): the
LLM MLP projection
    C[16384, 14336] (bf16) = X[16384, 4096] (bf16) . W[4096, 14336] (fp8 E4M3, per-column fp32 scale)
with W and C partitioned by columns over the N ranks (X replicated, no data-path collective, outputs
left sharded).  One step = one call of skl_gemm_ex_sm100a per rank: the exact fp8->bf16 widening of the
rank's W slice followed by the tcgen05 bf16 GEMM with the per-column scale and the bf16 narrowing fused
into its epilogue.  `value` is whole-job TFLOP/s (2*M*N*K per step over the slowest rank's device time)
with operands resident in HBM; `e2e` is the same call handed pinned HOST buffers, so the host->device
copies of X, W, scales and the device->host copy of C are inside the timed region.  The total work is
fixed as N grows ("strong" scaling).  Inputs are seeded synthetic tensors of the configured
shapes and distributions; every operand set is larger than the 126 MB L2.

At N = 1 the line also carries, under "also", short measurements of the other configured workloads
(int8 8192^3, bf16/fp16 4096^3, fp8 8192^3, the decode GEMV at M = 1/4/16) and a `cpu_baseline`:
the reference's scalar routines (oracle/_ref when built, else the oracle port) timed on the host cores
on a bounded row sample of the same workload.

--impl reference times only that CPU path (rank 0; other ranks exit at once).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_C5, K_C5, N_C5 = 16384, 4096, 14336
C5_DRAM_BYTES_PER_LAUNCH_1GPU = 804.4e6 + 453.8e6  # dram__bytes_read + dram__bytes_write, one launch of this build


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"],
                "bf16_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks (read-only NVML)
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU from a background thread while a region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.power_w = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        self._stop.wait(self.period)  # the first sample is taken once the region is under way, not at its first instant
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        pw = sorted(self.power_w)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s),
                "power_w": (round(pw[len(pw) // 2], 1) if pw else None)}


def bind_to_gpu_cpus(index: int):
    """Restricts this process to the CPUs NVML lists as local to GPU `index` (a CPU affinity of this process, not a
    GPU setting), so that pinned host buffers are first touched on the GPU's own NUMA node.  Returns the CPU
    count, or None when NVML or the affinity call is unavailable."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, bits in enumerate(words) for b in range(64) if (int(bits) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


# ----------------------------------------------------------------------------- CPU baseline (checker only)
def cpu_reference_sample(rows_per_thread: int | None, budget_s: float, threads: int):
    """Times the reference's scalar path on a row sample of the c5 workload.

    The sample is `threads * rows_per_thread` rows of C at full N and K: widening of W with
    skl_cvt_f8e4m3_bf16_ref, then skl_gemm_bf16rc_bf16rc_f32rc_ref on each thread's row slab (rows are
    independent, arithmetic unchanged; W is handed over k-contiguous, which is bit-identical and faster
    for the scalar loop).  Returns (tflops, seconds, rows, kind)."""
    import numpy as np

    from oracle import pyoracle as orc

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import helpers as H

    ref = orc.ref()
    kind = "reference" if ref is not None else "port"
    g = H.rng(5)
    n, k = N_C5, K_C5
    w8 = H.random_operand(H.F8E4M3, (n, k), g)  # [N][K], k contiguous
    wide = np.zeros((n, k), np.uint16)

    def widen(i0, rows):
        if ref is not None:
            ref.skl_cvt_f8e4m3_bf16_ref(orc._p(wide[i0:]), orc._p(w8[i0:]), rows * k)
        else:
            orc.port().orc_cvt_f8_bf16(orc._p(wide[i0:]), orc._p(w8[i0:]), rows * k, H.F8E4M3)

    def run(rows_per_thread):
        rows = rows_per_thread * threads
        x = H.random_operand(H.BF16, (rows, k), g)
        c = np.zeros((rows, n), np.float32)

        def slab(i0, r):
            if ref is not None:
                orc.ref_gemm_rc(H.BF16, r, n, k, 1.0, x[i0:], k, 1, wide, 1, k, 0.0, c[i0:], n, 1)
            else:
                orc.port_gemm_rc(H.BF16, H.BF16, r, n, k, 1.0, x[i0:], k, 1, wide, 1, k, 0.0, c[i0:], n, 1)

        t0 = time.perf_counter()
        orc.rows_in_parallel(widen, n, threads)
        orc.rows_in_parallel(slab, rows, threads)
        return time.perf_counter() - t0, rows

    if rows_per_thread is None:
        t1, _ = run(1)  # calibration pass: one row per thread
        rows_per_thread = max(1, min(64, int(budget_s / max(t1, 1e-3))))
        if rows_per_thread == 1:
            return 2.0 * threads * n * k / t1 / 1e12, t1, threads, kind, 1
    t, rows = run(rows_per_thread)
    return 2.0 * rows * n * k / t / 1e12, t, rows, kind, rows_per_thread


def reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    total_budget = 150.0
    per_step = max(0.5, min(4.0, total_budget / max(1, args.steps + args.warmup + 1)))
    tf, t, rows, kind, rpt = cpu_reference_sample(None, per_step, threads)  # calibration + first sample
    for _ in range(max(0, args.warmup - 1)):
        cpu_reference_sample(rpt, per_step, threads)
    times = []
    for _ in range(args.steps):
        tf_i, t_i, rows, kind, _ = cpu_reference_sample(rpt, per_step, threads)
        times.append(t_i)
    ms = 1e3 * sum(times) / len(times)
    value = 2.0 * rows * N_C5 * K_C5 / (ms * 1e-3) / 1e12
    sample = (f"{rows} of {M_C5} rows of C at full N={N_C5}, K={K_C5} per step ({rpt} rows per thread), "
              "fp8->bf16 widening of W included; rate is independent of the row count")
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {"workload": "c5: bf16 X[16384x4096] . fp8-E4M3 W[4096x14336] with per-column fp32 scales -> bf16 C, "
                        "W and C column-sharded over the ranks, X replicated",
            "m": M_C5, "k": K_C5, "n": N_C5, "n_per_gpu": N_C5 // max(1, n_gpus),
            "l2": "operands larger than L2 (X 128 MiB + W slice + C slice)", "parallelism": f"n-shard x{n_gpus}"}


# ----------------------------------------------------------------------------- device helpers
def time_steps(torch, fn, steps: int, barrier=None):
    """K back-to-back calls between two events on the current stream, synchronised on both sides."""
    torch.cuda.synchronize()
    if barrier:
        barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1)  # ms


def make_workloads(torch, S, lib):
    """Named device-resident workloads besides c5: name -> builder returning (call, work, kind, reps).

    kind "tflops" / "tflops8" (8-bit operands) / "tflops4" (4-bit operands): work = operations per call; kind "gbs": work = algorithmic
    bytes per call."""
    dev = "cuda"
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    W = {}

    def gemm_ex(m, n, k, ta, tb, tc, a, b, c, alpha=1.0):
        def call():
            lib.skl_gemm_ex_sm100a(m, n, k, ta, a.data_ptr(), k, 1, tb, b.data_ptr(), n, 1, alpha, None, None, 0.0, tc,
                                   c.data_ptr(), n, 1)
        return call

    def int8_8192():
        # the perf companion of config 1 (whose own 0.5 GOP cannot load the machine): SKL entry, int32 out
        m = n = k = 8192
        a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device=dev, generator=g)
        b = torch.randint(-128, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
        c = torch.empty((m, n), dtype=torch.int32, device=dev)

        def call():
            lib.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, a.data_ptr(), k, b.data_ptr(), n, 0, c.data_ptr(), n)
        return call, 2.0 * m * n * k, "tflops8", 20

    def c5_like(parts, static):
        def build():
            # the headline shape and operand distributions (X ~ N(0,1); W ~ N(0, 0.02) quantised per column with scale
            # amax/448); static: the weights are declared static, so W is widened by the first call only
            m, k, n = M_C5, K_C5, N_C5 // parts  # one rank's column shard when parts > 1
            x = (torch.randn((m, k), device=dev, generator=g)).to(torch.bfloat16)
            w32 = torch.randn((k, n), device=dev, generator=g) * 0.02
            sc = (w32.abs().amax(dim=0) / 448.0).clamp_min(1e-30).contiguous()
            w32 /= sc[None, :]
            w = torch.empty((k, n), dtype=torch.uint8, device=dev)
            lib.skl_cvt_sat_f32_f8e4m3_sm100a(w.data_ptr(), w32.data_ptr(), 1.0, k * n)
            del w32
            c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

            def call():
                lib.skl_b200_set_static_weights(1 if static else 0)
                lib.skl_gemm_ex_sm100a(m, n, k, S.BF16, x.data_ptr(), k, 1, S.F8E4M3, w.data_ptr(), n, 1, 1.0, None,
                                       sc.data_ptr(), 0.0, S.BF16, c.data_ptr(), n, 1)
                lib.skl_b200_set_static_weights(0)
            return call, 2.0 * m * n * k, "tflops", 20
        return build

    def int8_packed(force_simt):
        def build():
            # SKL's packed entry point on an mmt4d-style layout: A [m1][k1][16][8], B [n1][k1][16][8], C [m1][n1][16][16]
            m = n = k = 4096 if not force_simt else 1024
            m0, n0, k0 = 16, 16, 8
            m1, n1, k1 = m // m0, n // n0, k // k0
            a = torch.randint(-128, 128, (m * k,), dtype=torch.int8, device=dev, generator=g)
            b = torch.randint(-128, 128, (k * n,), dtype=torch.int8, device=dev, generator=g)
            c = torch.empty((m * n,), dtype=torch.int32, device=dev)

            def call():
                if force_simt:
                    lib.skl_b200_force_path(S.PATH_GENERIC)
                lib.skl_gemm_i8rcprc_i8rcprc_i32rcprc_sm100a(
                    m0, n0, k0, m1, n1, k1, 1, a.data_ptr(), k0, 1, k1 * m0 * k0, m0 * k0, b.data_ptr(), 1, k0, n0 * k0,
                    k1 * n0 * k0, 0, c.data_ptr(), n0, 1, n1 * m0 * n0, m0 * n0)
                if force_simt:
                    lib.skl_b200_force_path(0)
            return call, 2.0 * m * n * k, "tflops8", 10
        return build

    def int8_packed_te(out_blocked):
        def build():
            # the matrix-engine packed entry point on operands packed ahead of time: A in TE x 1 panels (element (i, kk)
            # at (i / TE) * TE * K + kk * TE + i % TE), B in 1 x TE panels, C in TE x TE blocks (or row-major when
            # not out_blocked: rsc0 = N, csc0 = 1, blocks side by side); the kernel reads the panels in place
            m = n = k = 4096
            te = int(lib.skl_b200_te())
            m1, n1 = m // te, n // te
            a = torch.randint(-128, 128, (m * k,), dtype=torch.int8, device=dev, generator=g)
            b = torch.randint(-128, 128, (k * n,), dtype=torch.int8, device=dev, generator=g)
            c = torch.empty((m * n,), dtype=torch.int32, device=dev)
            cstr = (te, 1, n1 * te * te, te * te) if out_blocked else (n, 1, te * n, te)

            def call():
                lib.skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a(m1, n1, k, 1, a.data_ptr(), te * k, te, b.data_ptr(),
                                                                       te, te * k, 0, c.data_ptr(), *cstr)
            return call, 2.0 * m * n * k, "tflops8", 20
        return build

    def mxf4():
        # block-scaled E2M1 operands (one E8M0 scale per 32 k), uniform random codes, scales 2^-4 .. 2^4; one call =
        # one launch of the kernel on the block-scaled tensor-core instruction
        m = n = k = 8192
        a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=dev, generator=g)
        b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
        sa = torch.randint(123, 132, (m, k // 32), dtype=torch.uint8, device=dev, generator=g)
        sb = torch.randint(123, 132, (n, k // 32), dtype=torch.uint8, device=dev, generator=g)
        c = torch.empty((m, n), dtype=torch.float32, device=dev)

        def call():
            lib.skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a(m, n, k, 1.0, a.data_ptr(), k // 2, sa.data_ptr(), k // 32, b.data_ptr(),
                                                      k // 2, sb.data_ptr(), k // 32, 0.0, c.data_ptr(), n)
        return call, 2.0 * m * n * k, "tflops4", 10

    def fp8(ta):
        def build():
            # config 3 as configured: fp32 N(0,1) operands narrowed by the library's saturating cvt with the
            # per-tensor scale (largest finite value of the format) / amax; alpha = s_a * s_b; bf16 output
            m = n = k = 8192
            fmax_a = 448.0 if ta == S.F8E4M3 else 57344.0
            cvt_a = lib.skl_cvt_sat_f32_f8e4m3_sm100a if ta == S.F8E4M3 else lib.skl_cvt_sat_f32_f8e5m2_sm100a
            a = torch.empty((m, k), dtype=torch.uint8, device=dev)
            b = torch.empty((k, n), dtype=torch.uint8, device=dev)
            src = torch.randn((m, k), device=dev, generator=g)
            s_a = float(src.abs().max()) / fmax_a
            cvt_a(a.data_ptr(), src.data_ptr(), 1.0 / s_a, m * k)
            src = torch.randn((k, n), device=dev, generator=g)
            s_b = float(src.abs().max()) / 448.0
            lib.skl_cvt_sat_f32_f8e4m3_sm100a(b.data_ptr(), src.data_ptr(), 1.0 / s_b, k * n)
            lib.skl_b200_synchronize()
            del src
            c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            return gemm_ex(m, n, k, ta, S.F8E4M3, S.BF16, a, b, c, s_a * s_b), 2.0 * m * n * k, "tflops8", 20
        return build

    def half(tdt, code):
        def build():
            m = n = k = 4096  # config 2
            a = (torch.randn((m, k), device=dev, generator=g) / 64.0).to(tdt)
            b = (torch.randn((k, n), device=dev, generator=g) / 64.0).to(tdt)
            c = torch.empty((m, n), dtype=tdt, device=dev)
            return gemm_ex(m, n, k, code, code, code, a, b, c), 2.0 * m * n * k, "tflops", 40
        return build

    def bf16_pair(m, n, k, comparator):
        def build():
            # bf16 x bf16 on N(0,1)/64 operands (B as [N][K], k contiguous), bf16 out; with comparator=True the
            # same tensors go through torch.matmul (cuBLAS) instead -- a yardstick only, never used by the library
            a = (torch.randn((m, k), device=dev, generator=g) / 64.0).to(torch.bfloat16)
            b = (torch.randn((n, k), device=dev, generator=g) / 64.0).to(torch.bfloat16)
            c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            if comparator:
                bt = b.t()

                def call():
                    torch.matmul(a, bt, out=c)
            else:
                def call():
                    lib.skl_gemm_ex_sm100a(m, n, k, S.BF16, a.data_ptr(), k, 1, S.BF16, b.data_ptr(), 1, k, 1.0, None,
                                           None, 0.0, S.BF16, c.data_ptr(), n, 1)
            return call, 2.0 * m * n * k, "tflops", 30
        return build

    def gemv(mm, n=14336, static=False):
        def build():
            # config 4; rotate over weight copies totalling > 2x L2 so every pass streams from HBM
            k = 4096
            copies = max(2, min(8, (360 << 20) // (n * k) + 1))
            w = torch.randint(-127, 128, (copies, n, k), dtype=torch.int8, device=dev, generator=g)
            sw = torch.rand((n,), device=dev, generator=g) * 1e-2 + 5e-3
            x = torch.randint(-127, 128, (mm, k), dtype=torch.int8, device=dev, generator=g)
            sx = torch.rand((mm,), device=dev, generator=g) + 0.5
            y = torch.empty((mm, n), dtype=torch.float32, device=dev)
            idx = [0]

            def call():
                wi = w[idx[0] % copies]
                idx[0] += 1
                if static:  # weights declared static: consecutive launches overlap drain and weight prefetch
                    lib.skl_b200_set_static_weights(1)
                lib.skl_gemm_ex_sm100a(mm, n, k, S.I8, x.data_ptr(), k, 1, S.I8, wi.data_ptr(), 1, k, 1.0, sx.data_ptr(),
                                       sw.data_ptr(), 0.0, S.F32, y.data_ptr(), n, 1)
                if static:
                    lib.skl_b200_set_static_weights(0)
            return call, float(n * k + mm * k + 4 * (n + mm) + 4 * mm * n), "gbs", 60
        return build

    def cvt_f32_e4m3():
        n = 1 << 27  # 512 MiB in, 128 MiB out: config 3's operand preparation at twice the size
        src = torch.randn((n,), device=dev, generator=g)
        dst = torch.empty((n,), dtype=torch.uint8, device=dev)

        def call():
            lib.skl_cvt_sat_f32_f8e4m3_sm100a(dst.data_ptr(), src.data_ptr(), 0.37, n)
        return call, 5.0 * n, "gbs", 10

    def cvt_e4m3_bf16():
        n = 1 << 28
        src = torch.randint(0, 256, (n,), dtype=torch.uint8, device=dev, generator=g)
        dst = torch.empty((n,), dtype=torch.bfloat16, device=dev)

        def call():
            lib.skl_cvt_f8e4m3_bf16_sm100a(dst.data_ptr(), src.data_ptr(), n)
        return call, 3.0 * n, "gbs", 10

    def transpose(e, m):
        def make():
            n = m
            dt = {8: torch.uint8, 16: torch.int16, 32: torch.int32}[e]
            a = torch.randint(0, 127, (m, n), dtype=dt, device=dev, generator=g)
            at = torch.empty((n, m), dtype=dt, device=dev)
            fn = getattr(lib, f"skl_transpose_e{e}_sm100a")

            def call():
                fn(m, n, a.data_ptr(), n, at.data_ptr(), m)
            return call, 2.0 * m * n * (e // 8), "gbs", 10
        return make

    def pack_e16():
        m, n, m0, n0 = 16384, 8192, 128, 64  # row-major bf16 matrix into 128 x 64 row-major blocks
        a = torch.randint(0, 30000, (m, n), dtype=torch.int16, device=dev, generator=g)
        out = torch.empty((m * n,), dtype=torch.int16, device=dev)
        n1 = n // n0

        def call():
            lib.skl_pack_e16rc_e16rcprc_sm100a(m, n, a.data_ptr(), n, 1, m0, n0, out.data_ptr(), n0, 1, n1 * m0 * n0,
                                               m0 * n0, 0)
        return call, 4.0 * m * n, "gbs", 10

    W["int8_8192_i32out"] = int8_8192
    W["c5_static_weights"] = c5_like(1, True)
    # one rank's share of the 2- / 4- / 8-GPU runs on this GPU alone (widening pass included, nothing static)
    W["c5_shard_of_2"], W["c5_shard_of_4"], W["c5_shard_of_8"] = c5_like(2, False), c5_like(4, False), c5_like(8, False)
    W["int8_4096_packed_i32out"] = int8_packed_te(True)
    W["int8_4096_packed_rowmajor_i32out"] = int8_packed_te(False)
    W["int8_4096_packed_16x16x8_i32out"] = int8_packed(False)
    W["int8_1024_packed_i32out_simt_kernel"] = int8_packed(True)
    W["fp8_e4m3xe4m3_8192_bf16out"] = fp8(S.F8E4M3)
    W["fp8_e5m2xe4m3_8192_bf16out"] = fp8(S.F8E5M2)
    W["mxf4_8192_f32out"] = mxf4
    W["bf16_4096_bf16out"] = half(torch.bfloat16, S.BF16)
    W["fp16_4096_fp16out"] = half(torch.float16, S.F16)
    W["bf16_4096_kmajor_randn"] = bf16_pair(4096, 4096, 4096, False)
    W["comparator_torch_matmul_bf16_4096_kmajor_randn"] = bf16_pair(4096, 4096, 4096, True)
    W["bf16_c5shape_kmajor_randn"] = bf16_pair(M_C5, N_C5, K_C5, False)
    W["comparator_torch_matmul_bf16_c5shape_kmajor_randn"] = bf16_pair(M_C5, N_C5, K_C5, True)
    W["gemv_i8_m1"], W["gemv_i8_m4"], W["gemv_i8_m16"] = gemv(1), gemv(4), gemv(16)
    W["gemv_i8_m1_static_weights"], W["gemv_i8_m2_static_weights"] = gemv(1, static=True), gemv(2, static=True)
    W["gemv_i8_m2"] = gemv(2)
    # the same kernels at other row counts: separates the fixed cost of a launch from the streaming rate
    for rows in (1184, 4736, 28672, 57344):
        W[f"gemv_i8_m1_n{rows}"] = gemv(1, rows)
        W[f"gemv_i8_m16_n{rows}"] = gemv(16, rows)
    W["cvt_sat_f32_f8e4m3_128M"] = cvt_f32_e4m3
    W["cvt_f8e4m3_bf16_256M"] = cvt_e4m3_bf16
    W["transpose_e8_16384"] = transpose(8, 16384)
    W["transpose_e16_16384"] = transpose(16, 16384)
    W["transpose_e32_8192"] = transpose(32, 8192)
    W["transpose_e16_8192"] = transpose(16, 8192)
    W["transpose_e32_16384"] = transpose(32, 16384)
    W["pack_e16_16384x8192"] = pack_e16
    return W


def time_graph(torch, lib, call, reps, replays=5):
    """Device time per call with the host out of the picture: `reps` calls captured into one CUDA graph
    (the library only enqueues when its operands are device memory), the graph replayed between two events."""
    prev = lib.skl_b200_get_stream()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    lib.skl_b200_set_stream(side.cuda_stream)
    try:
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                call()
    finally:
        lib.skl_b200_set_stream(prev)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * reps)


def run_workload(torch, S, lib, peaks, build, warmup=3, reps=None):
    call, work, kind, default_reps = build()
    reps = reps or default_reps
    for _ in range(warmup):
        call()
    S.check()
    ms = time_steps(torch, call, reps) / reps
    lib.skl_b200_synchronize()
    S.check()
    if kind in ("tflops", "tflops8", "tflops4"):
        tf = work / (ms * 1e-3) / 1e12
        out = {"tflops": round(tf, 1), "ms": round(ms, 4)}
        if kind == "tflops8":  # 8-bit operands: against the datasheet's dense peak and against twice the measured bf16 rate
            out["frac_of_4500_datasheet"] = round(tf / 4500.0, 3)
            out["frac_of_2x_measured_bf16_burst"] = round(tf / (2.0 * peaks["bf16_burst"]), 3)
        elif kind == "tflops4":  # 4-bit operands: datasheet dense peak 9 P; four times the measured bf16 rate
            out["frac_of_9000_datasheet"] = round(tf / 9000.0, 3)
            out["frac_of_4x_measured_bf16_burst"] = round(tf / (4.0 * peaks["bf16_burst"]), 3)
        else:
            out["frac_of_measured_bf16_burst"] = round(tf / peaks["bf16_burst"], 3)
        return out
    # bandwidth-bound kernels last microseconds: time them inside a CUDA graph so that the figure is the
    # device's, and keep the back-to-back API figure (host launch cost included) beside it
    out = {"us_api_back_to_back": round(ms * 1e3, 2)}
    try:
        ms = time_graph(torch, lib, call, reps)
        out["timing"] = "cuda graph replay"
    except Exception as exc:  # pragma: no cover - capture refused: keep the API timing
        out["timing"] = f"api calls (graph capture failed: {type(exc).__name__})"
    lib.skl_b200_synchronize()
    S.check()
    gbs = work / (ms * 1e-3) / 1e9
    out.update({"gbs": round(gbs, 1), "us": round(ms * 1e3, 2), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)})
    return out


def also_configs(torch, S, lib, peaks):
    """Short device-resident measurements of the other configured workloads and companions (1 GPU)."""
    out = {}
    for name, build in make_workloads(torch, S, lib).items():
        if "_n" in name.rsplit("_m", 1)[-1]:
            continue  # row-count sweeps are for --only
        out[name] = run_workload(torch, S, lib, peaks, build)
        torch.cuda.empty_cache()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-also", action="store_true", help="skip the other configs and the CPU baseline")
    ap.add_argument("--only", default=None, help="run one named side workload (see make_workloads) and print "
                                                 "its own small JSON line; used for profiler captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import numpy as np
    import torch

    import skl_b200 as S

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    all_cpus = os.sched_getaffinity(0)
    local_cpus = bind_to_gpu_cpus(local_rank)  # pinned buffers get first-touched on the GPU's NUMA node
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    barrier = (lambda: dist.barrier()) if dist else None

    lib = S.lib()  # raises if the CUDA library is not built: no fallback
    lib.skl_b200_set_stream(torch.cuda.current_stream().cuda_stream)
    peaks = measured_peaks()

    if args.only:
        lib.skl_b200_set_async(1)
        res = run_workload(torch, S, lib, peaks, make_workloads(torch, S, lib)[args.only], warmup=args.warmup,
                           reps=args.steps)
        print(json.dumps({"workload": args.only, **res, "steps": args.steps, "warmup": args.warmup}), flush=True)
        return

    # ---------------- inputs (seed 5): X ~ N(0,1) bf16; W ~ N(0, 0.02), per-column scale amax/448, E4M3
    m, k, n_total = M_C5, K_C5, N_C5
    col0, ncols = S.shard_columns(n_total, world, rank, 256)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    x = torch.randn((m, k), device="cuda", generator=gen).to(torch.bfloat16)
    w32_full = torch.randn((k, n_total), device="cuda", generator=gen) * 0.02
    w32 = w32_full[:, col0:col0 + ncols].contiguous()
    del w32_full
    scale = (w32.abs().amax(dim=0) / 448.0).clamp_min(1e-30).contiguous()
    wq_in = (w32 / scale[None, :]).contiguous()
    w8 = torch.empty((k, ncols), dtype=torch.uint8, device="cuda")
    lib.skl_cvt_sat_f32_f8e4m3_sm100a(w8.data_ptr(), wq_in.data_ptr(), 1.0, k * ncols)
    S.check()
    del w32, wq_in
    c = torch.empty((m, ncols), dtype=torch.bfloat16, device="cuda")

    def step():
        lib.skl_gemm_ex_sm100a(m, ncols, k, S.BF16, x.data_ptr(), k, 1, S.F8E4M3, w8.data_ptr(), ncols, 1, 1.0, None,
                               scale.data_ptr(), 0.0, S.BF16, c.data_ptr(), ncols, 1)

    lib.skl_b200_set_async(0)
    step()
    S.check()
    assert lib.skl_b200_last_path() == S.PATH_TCGEN05, "workload did not run on the tcgen05 kernel"
    launches_per_step = lib.skl_b200_last_launch_count()
    lib.skl_b200_set_async(1)
    for _ in range(args.warmup):
        step()
    lib.skl_b200_synchronize()
    S.check()

    # ---------------- timed region, device-resident operands
    lib.skl_b200_profile_begin(args.steps)
    with ClockSampler(local_rank) as clk:
        ms_total = time_steps(torch, step, args.steps, barrier)
    kernel_ms = S.C.c_double(0.0)
    recorded = lib.skl_b200_profile_end(S.C.byref(kernel_ms))
    lib.skl_b200_synchronize()
    S.check()
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    flops_step = 2.0 * m * n_total * k
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---------------- the same step looped for at least two seconds: the rate the power cap sustains
    sus_steps = max(args.steps, int(2.2e3 / max(ms_step, 1e-3)) + 1)
    lib.skl_b200_profile_begin(0)
    with ClockSampler(local_rank, period_s=0.02) as sus_clk:
        sus_ms = time_steps(torch, step, sus_steps, barrier)
    lib.skl_b200_synchronize()
    S.check()
    t = torch.tensor([sus_ms], device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sus_ms = float(t.item())
    sus_value = flops_step * sus_steps / (sus_ms * 1e-3) / 1e12
    sc = sus_clk.summary()
    sustained = {"value": sus_value, "unit": "TFLOP/s", "steps": sus_steps, "seconds": round(sus_ms * 1e-3, 3),
                 "ms_per_step": sus_ms / sus_steps,
                 "frac_of_sustained_peak": sus_value / (world * peaks["bf16_sustained"]),
                 "peak": f"{peaks['bf16_sustained']} TFLOP/s per GPU (sustained bf16, of {peaks['source']})",
                 "sm_mhz": sc["sm_mhz"], "power_w": sc["power_w"], "reasons": sc["reasons"]}

    # ---------------- optional final all-gather of C (outside `value`): NCCL all-gather of the shards into
    # [G][M][N/G], then the library's local re-layout to the row-major M x N matrix
    gather = None
    if dist and n_total % (world * 256) == 0:
        gathered = torch.empty((world, m, ncols), dtype=torch.bfloat16, device="cuda")
        c_full = torch.empty((m, n_total), dtype=torch.bfloat16, device="cuda")

        def gather_step(ev):
            ev[0].record()
            dist.all_gather_into_tensor(gathered, c)
            ev[1].record()
            lib.skl_b200_unshard_columns_sm100a(2, m, n_total, world, 256, gathered.data_ptr(), m * ncols,
                                                c_full.data_ptr(), n_total)
            ev[2].record()

        lib.skl_b200_set_async(1)
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(6)]
        for ev in evs:
            if barrier:
                barrier()
            gather_step(ev)
        torch.cuda.synchronize()
        S.check()
        ag = sorted(ev[0].elapsed_time(ev[1]) for ev in evs[2:])
        rl = sorted(ev[1].elapsed_time(ev[2]) for ev in evs[2:])
        t = torch.tensor([ag[len(ag) // 2], rl[len(rl) // 2]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ag_ms, rl_ms = float(t[0].item()), float(t[1].item())
        # every rank ends with the whole C: compare with the unsharded product computed here
        c_ref = torch.empty((m, n_total), dtype=torch.bfloat16, device="cuda")
        w_all = [torch.empty_like(w8) for _ in range(world)]
        s_all = [torch.empty_like(scale) for _ in range(world)]
        dist.all_gather(w_all, w8)
        dist.all_gather(s_all, scale)
        w_full, s_full = torch.cat(w_all, dim=1).contiguous(), torch.cat(s_all).contiguous()
        lib.skl_gemm_ex_sm100a(m, n_total, k, S.BF16, x.data_ptr(), k, 1, S.F8E4M3, w_full.data_ptr(), n_total, 1, 1.0,
                               None, s_full.data_ptr(), 0.0, S.BF16, c_ref.data_ptr(), n_total, 1)
        lib.skl_b200_synchronize()
        S.check()
        recv = (world - 1) * m * ncols * 2
        gather = {"allgather_ms": ag_ms, "relayout_ms": rl_ms, "bytes_received_per_gpu": recv,
                  "allgather_gbs_per_gpu": recv / (ag_ms * 1e-3) / 1e9, "nvlink_peer_copy_gbs_measured": 770.0,
                  "relayout_gbs": 2.0 * m * n_total * 2 / (rl_ms * 1e-3) / 1e9,
                  "equals_unsharded_product": bool(torch.equal(c_full, c_ref)),
                  "note": "NCCL all-gather of the bf16 C shards into [G][M][N/G] + skl_b200_unshard_columns_sm100a; "
                          "median of 4, max over ranks; not part of `value`"}
        del gathered, c_full, c_ref, w_all, s_all, w_full, s_full
        torch.cuda.empty_cache()

    # ---------------- end to end: pinned host buffers through the same call
    lib.skl_b200_set_async(0)
    w8h = w8.cpu().pin_memory()
    sh = scale.cpu().pin_memory()
    ch = torch.empty((m, ncols), dtype=torch.bfloat16).pin_memory()
    gather_x = bool(dist) and world > 1 and m % world == 0
    if gather_x:
        # X is replicated on the devices but need not cross PCIe N times: each rank uploads its own m/N rows and
        # the ranks all-gather them over NVLink (NCCL); W, the scales and C stay host buffers of the library call.
        rows = m // world
        xh = x[rank * rows:(rank + 1) * rows].cpu().pin_memory()
        x_part = torch.empty((rows, k), dtype=torch.bfloat16, device="cuda")
        x_all = torch.empty((m, k), dtype=torch.bfloat16, device="cuda")

        phase_ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

        def step_host():
            phase_ev[0].record()
            x_part.copy_(xh, non_blocking=True)
            phase_ev[1].record()
            dist.all_gather_into_tensor(x_all, x_part)
            phase_ev[2].record()
            lib.skl_gemm_ex_sm100a(m, ncols, k, S.BF16, x_all.data_ptr(), k, 1, S.F8E4M3, w8h.data_ptr(), ncols, 1, 1.0,
                                   None, sh.data_ptr(), 0.0, S.BF16, ch.data_ptr(), ncols, 1)
            phase_ev[3].record()
    else:
        xh = x.cpu().pin_memory()

        def step_host():
            lib.skl_gemm_ex_sm100a(m, ncols, k, S.BF16, xh.data_ptr(), k, 1, S.F8E4M3, w8h.data_ptr(), ncols, 1, 1.0,
                                   None, sh.data_ptr(), 0.0, S.BF16, ch.data_ptr(), ncols, 1)

    e2e_steps = max(3, min(args.steps, 8))
    for _ in range(2):
        step_host()
    S.check()
    ms_e2e_total = time_steps(torch, step_host, e2e_steps, barrier)
    S.check()
    t = torch.tensor([ms_e2e_total], device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item()) / e2e_steps
    e2e_value = flops_step / (ms_e2e * 1e-3) / 1e12
    same = bool(torch.equal(ch.cuda(), c))
    phases = {"cpus_bound_to": local_cpus} if local_cpus else None
    if gather_x:
        # device time of the last step's phases on this rank (max over ranks): upload of the rank's rows of X, the
        # all-gather of X over NVLink, the library call (upload of the W shard and scales, widening, row-chunk GEMM
        # overlapped with the download of the C shard)
        torch.cuda.synchronize()
        t = torch.tensor([phase_ev[i].elapsed_time(phase_ev[i + 1]) for i in range(3)], device="cuda",
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases = {"x_rows_h2d_ms": float(t[0].item()), "x_allgather_ms": float(t[1].item()),
                  "library_call_ms": float(t[2].item()), "cpus_bound_to": local_cpus}
    h2d = xh.numel() * 2 + w8h.numel() + sh.numel() * 4
    d2h = ch.numel() * 2
    del xh, w8h, sh, ch

    # ---------------- roofline of the dominant kernel (the tcgen05 GEMM), from the library's event pairs
    kern_ms = kernel_ms.value / max(1, recorded)
    achieved = 2.0 * m * ncols * k / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None
    region_s = ms_total * 1e-3
    peak_kind = "sustained" if region_s >= 2.0 else "burst"
    peak = peaks["bf16_sustained"] if peak_kind == "sustained" else peaks["bf16_burst"]
    roofline = {"bound": "tensor", "kernel": "gemm_tc2_kernel<256, f16> (CTA pair; bf16 x bf16 -> fp32 in TMEM -> bf16)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": (achieved / peak if achieved else None),
                "peak_kind": f"{peak_kind}, of {peaks['source']}", "kernel_ms": kern_ms,
                # dram__bytes_read + dram__bytes_write of one launch at the 1-GPU shape, from a profiler capture of
                # this kernel on this workload (algorithmic: 0.70e9); not captured per shard
                "traffic": (C5_DRAM_BYTES_PER_LAUNCH_1GPU if world == 1 else None)}

    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "steps": e2e_steps, "matches_device_run": same,
                "bytes_are": "per rank",
                "x_distribution": ("each rank uploads m/N rows, all-gather over NVLink (NCCL)" if gather_x
                                   else "uploaded whole by the library call"),
                "phases": phases},
        "sustained": sustained,
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "clocks": clk.summary(),
        "roofline": roofline,
    }

    if gather is not None:
        line["gather"] = gather
    if world == 1 and not args.no_also:
        lib.skl_b200_set_async(1)
        del x, w8, c
        torch.cuda.empty_cache()
        line["also"] = also_configs(torch, S, lib, peaks)
        lib.skl_b200_synchronize()
        lib.skl_b200_set_async(0)
        os.sched_setaffinity(0, all_cpus)  # the CPU baseline uses every host core again
        threads = os.cpu_count() or 1
        tf, secs, rows, kind, rpt = cpu_reference_sample(None, 3.0, threads)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                                "sample": f"{rows} of {M_C5} rows of C at full N and K ({rpt} per thread, {secs:.1f} s), "
                                          "widening of W included; rate is independent of the row count"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
