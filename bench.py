"""Benchmark of the scaled_mm hot path: bit-exact emulated FP8 GEMM throughput, 2*M*N*K / t.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config 2 of the headline metric): profile 'hopper', M = N = K = 4096 per GPU, e4m3 x e4m3 operands from
N(0, 1) * 4, tensor-wise fp32 scales 2^U(-4, 4), bf16 output, split-K 1, torch's default slow accumulation. With N > 1
GPUs every rank computes its own 4096-row slab of a (4096 * N) x 4096 x 4096 call (weak scaling; the second operand is
replicated) and the output slabs are assembled with one NCCL all-gather inside the timed step.

One JSON line is printed by rank 0; see the keys below. `--impl reference` times the CPU restatement of the
reference's model (the oracle) on the host's cores instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_PER_GPU, N_, K_ = 4096, 4096, 4096
PROFILE, NFMA, FAST = "hopper", 32, False
L2_FLUSH_BYTES = 512 << 20
METRIC = "bit-exact emulated FP8 GEMM TFLOP/s (2MNK/t)"

# Executed warp-instruction lanes per emulated multiply-accumulate of each kernel family, from the ncu captures
# summarised under profiles/ (smsp__inst_executed.sum * 32 / (M*N*K) on the same workload).
INST_PER_MAC = {"integer": None, "fast": 3.78, "staged": 2.78}
# DRAM bytes per launch of the main kernel on the workload above, from a one-pass capture at full size
# (dram__bytes_read.sum + dram__bytes_write.sum = 1,170,526,464 + 32,845,568); None where no capture exists.
DRAM_TRAFFIC = {"integer": None, "fast": None, "staged": 1203372032}


def make_operands(rank: int):
    """Seeded synthetic operands of the workload, as uint8 code tensors on the CPU, and the two scales."""
    import torch
    g = lambda s: torch.Generator().manual_seed(s)  # noqa: E731
    a = (torch.randn(M_PER_GPU, K_, generator=g(2 + 1000 * rank)) * 4).clamp(-448, 448).to(torch.float8_e4m3fn)
    bt = (torch.randn(N_, K_, generator=g(3)) * 4).clamp(-448, 448).to(torch.float8_e4m3fn)
    sa = (2.0 ** (torch.rand((), generator=g(4)) * 8 - 4)).to(torch.float32)
    sb = (2.0 ** (torch.rand((), generator=g(5)) * 8 - 4)).to(torch.float32)
    return a, bt, sa, sb


class ClockSampler(threading.Thread):
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs: NVML every 5 ms when the
    pynvml module is present, else one nvidia-smi query per 100 ms. Read-only; nothing on the GPU is changed."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag = index, threading.Event()
        self.sm, self.max_sm, self.power, self.seen = [], None, [], set()

    def _nvml(self) -> bool:
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.index
            if visible:
                entry = visible.split(",")[self.index].strip()
                if not entry.isdigit():
                    return False
                index = int(entry)
            h = nv.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                    "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                    "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag.is_set():
                self.sm.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = int(reasons(h))
                self.seen.update(n for n, b in bits.items() if mask & int(b))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                except Exception:  # noqa: BLE001
                    pass
                self.stop_flag.wait(0.005)
            return True
        except Exception:  # noqa: BLE001
            return bool(self.sm)

    def _smi(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                r = [x.strip() for x in out.strip().split(",")]
                if len(r) >= 7 and r[0].isdigit():
                    self.sm.append(int(r[0]))
                    self.max_sm = int(r[1]) if r[1].isdigit() else self.max_sm
                    self.seen.update(n for i, n in enumerate(self.NAMES) if r[3 + i] == "Active")
            except Exception:  # noqa: BLE001
                return
            self.stop_flag.wait(0.1)

    def run(self):
        if not self._nvml():
            self._smi()

    def summary(self) -> dict:
        self.stop_flag.set()
        self.join(3)
        sm = sorted(self.sm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"]}
        out = {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.max_sm,
               "reasons": [n for n in self.NAMES if n in self.seen], "samples": len(sm)}
        if self.power:
            out["power_w_median"] = sorted(self.power)[len(self.power) // 2]
        return out


def cpu_baseline(a_u8, bt_u8, sa: float, sb: float, seconds: float = 12.0) -> dict:
    """The oracle timed on the host's cores on a row subset of the workload sized for about `seconds` of CPU work."""
    from oracle import oracle
    threads = oracle.num_threads()
    rows = 8
    t0 = time.perf_counter()
    oracle.scaled_mm(a_u8[:rows], bt_u8, sa, sb, out="bfloat16", preset=NFMA, fast=FAST)
    probe = time.perf_counter() - t0
    rows = int(max(8, min(a_u8.shape[0], rows * seconds / max(probe, 1e-3))))
    t0 = time.perf_counter()
    oracle.scaled_mm(a_u8[:rows], bt_u8, sa, sb, out="bfloat16", preset=NFMA, fast=FAST)
    dt = time.perf_counter() - t0
    return {"value": 2.0 * rows * N_ * K_ / dt / 1e12, "unit": "TFLOP/s (emulated, 2MNK/t)", "cores": threads,
            "kind": "port", "sample": f"first {rows} of {a_u8.shape[0]} rows x all {N_} columns x K={K_}, {dt:.1f} s",
            "seconds": dt}


def run_reference(args) -> int:
    """The reference arm: the CPU restatement of the reference's model, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    a, bt, sa, sb = make_operands(0)
    a_u8, bt_u8 = a.view(__import__("torch").uint8).numpy(), bt.view(__import__("torch").uint8).numpy()
    from oracle import oracle
    oracle.build()
    rows = 16
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        oracle.scaled_mm(a_u8[:rows], bt_u8, float(sa), float(sb), out="bfloat16", preset=NFMA, fast=FAST)
        dt = time.perf_counter() - t0
        if i < args.warmup:
            rows = int(max(16, min(M_PER_GPU, rows * 4.0 / max(dt, 1e-3))))     # about 4 s per step
        else:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = 2.0 * rows * N_ * K_ / (ms / 1e3) / 1e12
    base = {"value": value, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{rows} of {M_PER_GPU} rows x {N_} columns x K={K_} per step"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32/fp32 (CPU integer model)", "data": "synthetic",
        "config": {"workload": f"hopper e4m3xe4m3 {M_PER_GPU}x{N_}x{K_} bf16 slow-accum split-K 1, CPU row sample"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0


def run_ours(args) -> int:
    import torch
    import torch.distributed as dist
    import mmaemu_b200 as mm
    from mmaemu_b200 import _lib
    from mmaemu_b200.sharding import sharded_scaled_mm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus):
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch N > 1 with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: mmaemu_b200 has no CPU fallback")
    _lib.load()                                                # fails loudly if the CUDA library was never built
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    kernel = args.kernel
    backend = "cuda:b200" if kernel == "auto" else f"cuda:b200-{kernel}"
    M_total = M_PER_GPU * world

    a, bt, sa, sb = make_operands(rank)
    a_pin, bt_pin = a.view(torch.uint8).pin_memory(), bt.view(torch.uint8).pin_memory()
    a_dev, bt_dev = a.to(dev), bt.to(dev)
    sa_dev, sb_dev = sa.to(dev), sb.to(dev)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    kw = dict(out_dtype=torch.bfloat16, use_fast_accum=FAST, profile=PROFILE, backend=backend, splitk=1)

    def step_resident():
        if world == 1:
            return mm.scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, **kw)
        return sharded_scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, input_is_local=True, full_rows=M_total, **kw)

    out_pin = torch.empty((M_PER_GPU, N_), dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        ad = a_pin.to(dev, non_blocking=True).view(torch.float8_e4m3fn)
        bd = bt_pin.to(dev, non_blocking=True).view(torch.float8_e4m3fn)
        y = mm.scaled_mm(ad, bd.t(), sa_dev, sb_dev, **kw)
        out_pin.copy_(y, non_blocking=True)
        return y

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed(fn, steps):
        """Sum of per-step device times (CUDA events on the launch stream); L2 is flushed between steps, outside the
        event pairs."""
        pairs = []
        for _ in range(steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            pairs.append((e0, e1))
        torch.cuda.synchronize(dev)
        return sum(e0.elapsed_time(e1) for e0, e1 in pairs)

    # exactness gate before timing: sampled rows and columns of the full output against the oracle
    if rank == 0 and not args.skip_gate:
        import numpy as np
        from oracle import oracle
        oracle.build()
        y = mm.scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, **kw)      # this rank's slab; no collective in the gate
        torch.cuda.synchronize(dev)
        rows = torch.arange(0, M_PER_GPU, max(1, M_PER_GPU // 12 - 1))[:12]
        cols = torch.arange(0, N_, max(1, N_ // 40 - 1))[:40]
        got = y[rows][:, cols].cpu().view(torch.int16).numpy().view(np.uint16)
        want = oracle.scaled_mm(a.view(torch.uint8).numpy()[rows.numpy()], bt.view(torch.uint8).numpy()[cols.numpy()],
                                float(sa), float(sb), out="bfloat16", preset=NFMA, fast=FAST)
        if not np.array_equal(got, want):
            raise SystemExit("exactness gate failed: the kernel's output differs from the oracle; not timing")

    for _ in range(max(3, args.warmup)):
        step_resident()
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    sync_all()
    total_ms = timed(step_resident, args.steps)
    sync_all()
    launches = _lib.launch_count() - launches0
    clocks = sampler.summary() if rank == 0 else None

    for _ in range(2):
        step_e2e()
    sync_all()
    e2e_ms = timed(step_e2e, args.steps)
    sync_all()

    # the same through the C ABI's host-buffer entry point (pinned host operands in, pinned host result out; the call
    # stages, computes and synchronises its stream itself, so it is timed on the host clock)
    L = _lib.load()
    host_args = (a_pin.data_ptr(), K_, 0, bt_pin.data_ptr(), K_, 0, out_pin.data_ptr(), N_, 1, M_PER_GPU, N_, K_, NFMA,
                 int(FAST), 1, 0, ctypes.c_float(float(sa)), ctypes.c_float(float(sb)), None, 0,
                 ctypes.c_void_p(stream.cuda_stream))
    for _ in range(2):
        _lib.check("mmb200_scaled_mm_host", L.mmb200_scaled_mm_host(*host_args))
    sync_all()
    t_host = time.perf_counter()
    for _ in range(args.steps):
        _lib.check("mmb200_scaled_mm_host", L.mmb200_scaled_mm_host(*host_args))
    host_ms = (time.perf_counter() - t_host) * 1e3
    sync_all()

    t = torch.tensor([total_ms, e2e_ms, host_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, host_ms = (float(x) for x in t.cpu())
    ms = total_ms / args.steps
    macs = float(M_total) * N_ * K_
    value = 2.0 * macs / (ms / 1e3) / 1e12
    e2e_value = 2.0 * macs / (e2e_ms / args.steps / 1e3) / 1e12

    if rank == 0:
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except Exception:  # noqa: BLE001
            pass
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        auto = _lib.load().mmb200_kernel_for(a_dev.data_ptr(), K_, bt_dev.data_ptr(), K_, K_, NFMA, 1)
        used = kernel if kernel != "auto" else ("fast" if auto == _lib.KERNEL_CODES["fast"] else "integer")
        if used == "fast" and os.environ.get("MMAEMU_B200_WORKSPACE", "1") != "0":
            used = "staged"                                        # operands decoded once into scratch memory
        clk_mhz = (clocks or {}).get("sm_mhz") or float(peaks.get("sm_max_mhz", 1965.0))
        issue_peak = 148 * 128 * clk_mhz * 1e6 / 1e12                 # T lane-instructions / s at the sampled SM clock
        per_gpu_macs = float(M_PER_GPU) * N_ * K_
        kernel_s = ms / 1e3
        ipm = INST_PER_MAC[used]
        achieved_issue = per_gpu_macs * ipm / kernel_s / 1e12 if ipm else None
        algo_bytes = M_PER_GPU * K_ + N_ * K_ + M_PER_GPU * N_ * 2 + 12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32 round-toward-zero FMA + int32 (exact emulation of fp8 x fp8 blocks)"
            if used != "integer" else "int32", "data": "synthetic",
            "config": {"workload": f"profile {PROFILE}, e4m3xe4m3, M={M_total} N={N_} K={K_} ({M_PER_GPU} rows per GPU), "
                                   f"bf16 out, split-K 1, use_fast_accum={FAST}, kernel {used}",
                       "profile": PROFILE,
                       "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB write)",
                       "multi_gpu": "row slabs + one NCCL all-gather per step" if world > 1 else "single GPU"},
            "roofline": {"bound": "alu-issue", "achieved": achieved_issue, "peak": issue_peak,
                         "unit": "T lane-instructions/s",
                         "frac": achieved_issue / issue_peak if achieved_issue else None,
                         "traffic": DRAM_TRAFFIC[used],
                         "peak_basis": f"148 SMs x 128 lanes x {clk_mhz:.0f} MHz sampled under load (measured issue "
                                       f"rate of FFMA on this pool: 128 lanes/clk/SM; INT32 ALU pipe 64)",
                         "inst_per_mac": INST_PER_MAC[used],
                         "algorithmic_ops_per_mac": 4 + 12 / NFMA,
                         "algorithmic_achieved": per_gpu_macs * (4 + 12 / NFMA) / kernel_s / 1e12,
                         "hbm": {"achieved_gbs": algo_bytes / kernel_s / 1e9, "peak_gbs": hbm_peak,
                                 "frac": algo_bytes / kernel_s / 1e9 / hbm_peak, "of": "measured"
                                 if "hbm_gbs" in peaks else "fallback"}},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": (M_PER_GPU + N_) * K_,
                    "d2h_bytes_per_step": M_PER_GPU * N_ * 2, "ms_per_step": e2e_ms / args.steps,
                    "call": "mmaemu_b200.scaled_mm on operands copied from pinned host memory each step, result "
                            "copied back to pinned host memory",
                    "c_abi_host_call": {"value": 2.0 * macs / (host_ms / args.steps / 1e3) / 1e12, "unit": "TFLOP/s",
                                        "ms_per_step": host_ms / args.steps,
                                        "call": "mmb200_scaled_mm_host: pinned host operands in, pinned host result "
                                                "out, device staging inside the call, host clock"}},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a.view(torch.uint8).numpy(), bt.view(torch.uint8).numpy(), float(sa),
                                                float(sb))
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--kernel", choices=("auto", "integer", "fast"), default="auto")
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), default=None,
                    help="per-GPU problem size instead of the headline 4096 4096 4096 (profiling runs)")
    ap.add_argument("--fast-accum", action="store_true", help="use_fast_accum=True instead of torch's default")
    ap.add_argument("--profile", default=None, help="emulated platform profile (default hopper)")
    ap.add_argument("--skip-gate", action="store_true", help="skip the exactness gate before timing")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    global M_PER_GPU, N_, K_, FAST, PROFILE, NFMA
    if args.shape:
        M_PER_GPU, N_, K_ = args.shape
    if args.fast_accum:
        FAST = True
    if args.profile:
        PROFILE, NFMA = args.profile, (16 if args.profile.startswith("ada") else 32)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
