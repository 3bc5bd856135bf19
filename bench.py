"""Benchmark of the scaled_mm hot path: bit-exact emulated FP8 GEMM throughput, 2*M*N*K / t.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One GPU (the headline, configuration 2 of the metric): profile 'hopper', M = N = K = 4096, e4m3 x e4m3 operands from
N(0, 1) * 4, tensor-wise fp32 scales 2^U(-4, 4), bf16 output, split-K 1, torch's default slow accumulation. The same
line carries, under "configs", the other configurations of the metric at their own sizes (the 256-cube under 'ada', the
tall-skinny mixed-format shapes including table rows that split K, the FP8 projection stack under 'hopper-te', slabs of
the sharded problem under 'hopper' and 'ada'), and under "context" the reference's own CUDA kernels (cuda:h4, cuda:h1)
and torch._scaled_mm timed on the same GPU with the same method.

N > 1 GPUs: STRONG scaling of one fixed problem with the recipe of the metric's sharded configuration -- e4m3 x e4m3,
N(0, 1) * 16 operands with 1 % special codes (subnormals, +-max) and NaN codes in a seeded 1 % of the rows of both
operands, fp16 output (overflow), use_fast_accum=True, profile 'hopper' -- at M = N = 16384, K = 8192 (a quarter of the
metric's 32768 x 32768 x 8192 so that one GPU finishes a step in a quarter of a second). Rows are split across the
ranks, every rank ends up with the whole result (mmaemu_b200.sharded_scaled_mm); before timing, all ranks compare a
sha256 of the assembled result and rank 0 checks sampled rows of every rank's slab against the oracle.

One JSON line is printed by rank 0. `--impl reference` times the reference's own CPU backend
(mmaemu.scaled_mm(..., backend="reference") of the unmodified package under baseline/_ref) on all host cores on a
bounded row sample of the same workload; without that package, the CPU restatement of the model (the oracle).
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import os
import subprocess
import sys
import threading
import time
import warnings
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "baseline"))

L2_FLUSH_BYTES = 512 << 20
METRIC = "bit-exact emulated FP8 GEMM TFLOP/s (2MNK/t)"
NFMA_OF = {"hopper": 32, "hopper-te": 32, "hopper-ws0": 32, "ada": 16, "ada-te": 16, "ada-ws0": 16}

HEADLINE = dict(name="cfg2_hopper_4096cube", profile="hopper", M=4096, N=4096, K=4096, fa="e4m3", fb="e4m3",
                out="bfloat16", fast=False, splitk=1)
STRONG = dict(name="cfg5_recipe_16384x16384x8192", profile="hopper", M=16384, N=16384, K=8192, fa="e4m3", fb="e4m3",
              out="float16", fast=True, splitk="auto", scale_a=1.0, scale_b=0.25)

# Executed warp-instruction lanes per emulated multiply-accumulate, from ncu captures of the kernels as committed
# (smsp__inst_executed.sum * 32 / (M*N*K), profiles/): keyed by (kernel, products per block, accumulation). A workload
# whose kernel has no capture gets no issue-slot roofline (null), never another kernel's constant.
INST_PER_MAC = {("staged_tc_kernel", 32, "slow"): 2.514,       # 4096 cube, profiles/staged_tc_kernel_hopper_e4m3_2048cube.md
                ("staged_kernel", 32, "slow"): 3.16,           # 2048 cube e5m2 x e4m3 with MMAEMU_B200_TC_EPASS=0, profiles/staged_kernel_hopper_e5m2xe4m3_2048cube.md
                ("fast_kernel", 32, "slow"): 3.37,             # 2048 cube, profiles/fast_kernel_hopper_e4m3_2048cube.md
                ("staged_kernel, at most 16 rows", 32, "slow"): 5.18,   # 16 x 4096 x 8192, profiles/few_rows_kernel_hopper_e5m2xe4m3_16x4096x8192.md
                ("integer_kernel", 32, "slow"): 8.56}           # 2048 cube, profiles/integer_kernel_hopper_e4m3_2048cube.md
# DRAM bytes per launch of the main kernel on the headline workload, one-pass ncu capture at full size
# (dram__bytes_read.sum + dram__bytes_write.sum = 873,141,504 + 32,601,856; same profile file).
DRAM_TRAFFIC = {("staged_tc_kernel", 32, "slow", 4096, 4096, 4096): 905743360}


# ---------------------------------------------------------------------------------------------------------------
# data
def _f8(name):
    import torch
    return torch.float8_e4m3fn if name == "e4m3" else torch.float8_e5m2


def gaussian_codes(rows, K, sigma, seed, fmt="e4m3", device="cpu"):
    """[rows, K] FP8 tensor from N(0, 1) * sigma, seeded."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    mx = 448.0 if fmt == "e4m3" else 57344.0
    return (torch.randn(rows, K, generator=g, device=device) * sigma).clamp(-mx, mx).to(_f8(fmt))


def headline_operands():
    import torch
    g = lambda s: torch.Generator().manual_seed(s)  # noqa: E731
    c = HEADLINE
    a = gaussian_codes(c["M"], c["K"], 4.0, 2)
    bt = gaussian_codes(c["N"], c["K"], 4.0, 3)
    sa = (2.0 ** (torch.rand((), generator=g(4)) * 8 - 4)).to(torch.float32)
    sb = (2.0 ** (torch.rand((), generator=g(5)) * 8 - 4)).to(torch.float32)
    return a, bt, sa, sb


def special_codes(rows, K, seed, device):
    """E4M3 codes of the sharded configuration's recipe for `rows` rows: N(0, 1) * 16; 1 % of the elements replaced by a
    subnormal code (0x01..0x07, either sign) or +-max (0x7E / 0xFE); NaN codes (0x7F / 0xFF) at three positions of a
    seeded 1 % of the rows. Generated on `device` from `seed` (the same bytes on every GPU of one model)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    x = (torch.randn(rows, K, generator=g, device=device) * 16).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    pick = torch.rand(rows, K, generator=g, device=device)
    kind = torch.randint(0, 16, (rows, K), generator=g, device=device, dtype=torch.uint8)
    sub = ((kind % 7) + 1) | ((kind & 8) << 4)                             # 0x01..0x07 with a random sign
    top = torch.where((kind & 8) != 0, 0xFE, 0x7E).to(torch.uint8)
    x = torch.where(pick < 0.005, sub, x)
    x = torch.where((pick >= 0.005) & (pick < 0.01), top, x)
    nan_rows = torch.nonzero(torch.rand(rows, generator=g, device=device) < 0.01).flatten()
    if nan_rows.numel():
        cols = torch.randint(0, K, (nan_rows.numel(), 3), generator=g, device=device)
        x[nan_rows[:, None], cols] = torch.where(cols % 2 == 0, 0x7F, 0xFF).to(torch.uint8)
    return x


STRONG_CHUNKS = 8          # operand A of the strong-scaling problem is generated in 8 row chunks, one seed each


def strong_a_rows(m0, m1, device):
    """Rows [m0, m1) of the strong-scaling problem's first operand (whole chunks only)."""
    import torch
    per = STRONG["M"] // STRONG_CHUNKS
    assert m0 % per == 0 and m1 % per == 0
    return torch.cat([special_codes(per, STRONG["K"], 50 + c, device) for c in range(m0 // per, m1 // per)])


def strong_bt(device):
    return special_codes(STRONG["N"], STRONG["K"], 51_000, device)


# ---------------------------------------------------------------------------------------------------------------
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


# ---------------------------------------------------------------------------------------------------------------
# the reference package (unmodified, under baseline/_ref) and the CPU arms
def load_reference():
    """The reference's `mmaemu` module from baseline/_ref, or None when it is not installed there."""
    try:
        import install_reference
        if not install_reference.add_to_path():
            return None
        import mmaemu
        return mmaemu
    except Exception:  # noqa: BLE001
        return None


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:  # noqa: BLE001
        return os.cpu_count() or 1


def cpu_call(ref, a, bt, sa, sb, cfg, rows):
    """One call of the CPU arm on the first `rows` rows of the workload: the reference's CPU backend when `ref` is the
    reference module, else the oracle. Returns seconds."""
    import torch
    t0 = time.perf_counter()
    if ref is not None:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ref.scaled_mm(a[:rows], bt.t(), sa, sb, out_dtype=getattr(torch, cfg["out"]), use_fast_accum=cfg["fast"],
                          profile=cfg["profile"], splitk=1, backend="reference")
    else:
        from oracle import oracle
        oracle.scaled_mm(a[:rows].view(torch.uint8).numpy(), bt.view(torch.uint8).numpy(), float(sa), float(sb),
                         out=cfg["out"], fmt_a=cfg["fa"], fmt_b=cfg["fb"], preset=NFMA_OF[cfg["profile"]],
                         fast=cfg["fast"], threads=host_cores())
    return time.perf_counter() - t0


def cpu_baseline(a, bt, sa, sb, cfg, seconds: float = 12.0) -> dict:
    """The reference's CPU backend (kind "reference") -- or, without it, the oracle (kind "port") -- on all host cores,
    on a row subset of the workload sized for about `seconds` of CPU work; plus the oracle port as a second figure."""
    import torch
    cores = host_cores()
    torch.set_num_threads(cores)
    ref = load_reference()
    flops_per_row = 2.0 * cfg["N"] * cfg["K"]

    def measure(impl, target_s):
        rows = 8
        probe = cpu_call(impl, a, bt, sa, sb, cfg, rows)
        rows = int(max(8, min(a.shape[0], rows * target_s / max(probe, 1e-3))))
        dt = cpu_call(impl, a, bt, sa, sb, cfg, rows)
        return {"value": rows * flops_per_row / dt / 1e12, "unit": "TFLOP/s (emulated, 2MNK/t)", "cores": cores,
                "sample": f"first {rows} of {a.shape[0]} rows x all {cfg['N']} columns x K={cfg['K']}, {dt:.1f} s",
                "seconds": dt}
    if ref is not None:
        out = measure(ref, seconds)
        out["kind"] = "reference"
        out["what"] = "mmaemu.scaled_mm(..., backend='reference') of the unmodified reference on CPU tensors"
        port = measure(None, 5.0)
        port["kind"] = "port"
        out["port"] = port
    else:
        out = measure(None, seconds)
        out["kind"] = "port"
        out["what"] = "the C restatement of the model (oracle/), OpenMP; the reference package is not under baseline/_ref"
    return out


def run_reference(args) -> int:
    """The reference arm: the reference's own CPU implementation of the path, all host threads, a bounded row sample
    of the headline workload per step. Under torchrun only rank 0 works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import torch
    cores = host_cores()
    torch.set_num_threads(cores)
    cfg = HEADLINE
    a, bt, sa, sb = headline_operands()
    ref = load_reference()
    if ref is None:
        from oracle import oracle
        oracle.build()
    rows, times = 16, []
    for i in range(args.warmup + args.steps):
        dt = cpu_call(ref, a, bt, sa, sb, cfg, rows)
        if i < args.warmup:
            rows = int(max(16, min(cfg["M"], rows * 4.0 / max(dt, 1e-3))))     # about 4 s per step
        else:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = 2.0 * rows * cfg["N"] * cfg["K"] / (ms / 1e3) / 1e12
    kind = "reference" if ref is not None else "port"
    base = {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {cfg['M']} rows x {cfg['N']} columns x K={cfg['K']} per step",
            "what": "mmaemu.scaled_mm(..., backend='reference') on CPU tensors (unmodified reference package)"
            if ref is not None else "C restatement of the model (the reference package is not under baseline/_ref)"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "float64 torch model on CPU" if ref is not None else "int32/fp32 (CPU integer model)",
        "data": "synthetic", "config": {"workload": workload_text(cfg) + ", CPU row sample"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0


# ---------------------------------------------------------------------------------------------------------------
def workload_text(c) -> str:
    return (f"profile {c['profile']}, {c['fa']}x{c['fb']}, M={c['M']} N={c['N']} K={c['K']}, {c['out']} out, "
            f"use_fast_accum={c['fast']}, split-K {c['splitk']}")


def kernel_of(cfg, S=1) -> str:
    """Name of the main kernel the automatic choice runs for a configuration (with scratch memory)."""
    pair = (cfg["fa"], cfg["fb"])
    name = ("staged_tc_kernel" if pair == ("e4m3", "e4m3") else
            "staged_kernel" if pair == ("e5m2", "e5m2") else "staged_tc_kernel, powers of 32")
    # with at most 16 rows (unsplit plans and K slices) the instantiations that decode both operands themselves run
    return name + ", at most 16 rows" if cfg["M"] <= 16 else name


class Timer:
    """CUDA-event timing on torch's current stream with the L2 flushed between steps, outside the event pairs."""

    def __init__(self, dev):
        import torch
        self.dev = dev
        self.flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        self.stream = torch.cuda.current_stream(dev)

    def total_ms(self, fn, steps) -> float:
        import torch
        pairs = []
        for _ in range(steps):
            self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            fn()
            e1.record(self.stream)
            pairs.append((e0, e1))
        torch.cuda.synchronize(self.dev)
        return sum(e0.elapsed_time(e1) for e0, e1 in pairs)

    def median_ms(self, fn, steps, warm=2) -> float:
        import torch
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(self.dev)
        ts = sorted(self.total_ms(fn, 1) for _ in range(steps))
        return ts[len(ts) // 2]


def issue_peak(L, timer, clk_mhz):
    """Peak of the roofline: lane-instructions per second the SMs issue. Measured live with the library's probe kernel
    (independent round-toward-zero FMAs, 2048 threads per SM; the best of nine launches) and, beside it, the nominal 148 SMs x 128 lanes x clock
    and the rate of the integer pipe (three-input adds and logic operations) from the same probe."""
    import torch
    nominal = 148 * 128 * clk_mhz * 1e6 / 1e12
    info = {"nominal_fp32_lanes": nominal}
    try:
        iters, ctas = 8192, 148 * 8
        stream = ctypes.c_void_p(timer.stream.cuda_stream)
        sink = torch.zeros(ctas * 256, dtype=torch.float32, device=timer.dev)
        ops = float(ctas) * 256 * iters * 32            # 32 independent instructions per thread and iteration
        rates = {}
        for kind, name in ((0, "measured_ffma_rz"), (1, "measured_iadd3_lop3")):
            run = lambda: L.mmb200_probe_issue_rate(kind, ctas, iters, sink.data_ptr(), stream)  # noqa: E731
            if run() != 0:
                return nominal, info
            run()
            torch.cuda.synchronize(timer.dev)
            samples = sorted(timer.total_ms(run, 1) for _ in range(9))
            ms = samples[0]                             # a peak: the best of nine launches (the median is reported too)
            rates[name] = ops / (ms / 1e3) / 1e12
            info[name] = rates[name]
            info[name + "_median"] = ops / (samples[len(samples) // 2] / 1e3) / 1e12
            info[name + "_lanes_per_clk_sm"] = rates[name] * 1e12 / (148 * clk_mhz * 1e6)
        return rates["measured_ffma_rz"], info
    except Exception:  # noqa: BLE001
        return nominal, info


def sampled_gate(mm, oracle, y, a_u8, bt_u8, sa, sb, cfg, S, scheme, label, rows=None, cols=None):
    """Sampled rows and columns of a result against the oracle, bit for bit; raises SystemExit on a difference."""
    import numpy as np
    import torch
    M, N = y.shape
    rows = np.unique(np.linspace(0, M - 1, 12).astype(np.int64)) if rows is None else np.asarray(rows)
    cols = np.unique(np.linspace(0, N - 1, 40).astype(np.int64)) if cols is None else np.asarray(cols)
    view = {4: (torch.int32, np.uint32), 2: (torch.int16, np.uint16), 1: (torch.uint8, np.uint8)}[y.element_size()]
    got = y[torch.as_tensor(rows, device=y.device)][:, torch.as_tensor(cols, device=y.device)].cpu().view(view[0]) \
        .numpy().view(view[1])
    want = oracle.scaled_mm(a_u8[rows], bt_u8[cols], float(sa), float(sb), out=cfg["out"], fmt_a=cfg["fa"],
                            fmt_b=cfg["fb"], preset=NFMA_OF[cfg["profile"]], fast=cfg["fast"], S=S, scheme=scheme)
    if not np.array_equal(got, want):
        raise SystemExit(f"exactness gate failed ({label}): {int((got != want).sum())} of {want.size} sampled outputs "
                         f"differ from the oracle; not timing")


def time_config(mm, oracle, timer, dev, cfg, a, bt, sa, sb, steps=5):
    """One configuration through mmaemu_b200.scaled_mm: gate on sampled outputs, then median device time."""
    import torch
    from mmaemu_b200.splitk import resolve_splitk
    od = getattr(torch, cfg["out"])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if cfg["splitk"] == "auto":
            d = resolve_splitk(cfg["M"], cfg["N"], cfg["K"], a_dtype=cfg["fa"], b_dtype=cfg["fb"], out_dtype=cfg["out"],
                               use_fast_accum=cfg["fast"], profile=cfg["profile"])
            S, scheme = d.S, d.scheme
        else:
            S, scheme = 1, "none"
        ad, bd = a.to(dev), bt.to(dev)
        sad, sbd = torch.tensor(float(sa), device=dev), torch.tensor(float(sb), device=dev)
        fn = lambda: mm.scaled_mm(ad, bd.t(), sad, sbd, out_dtype=od, use_fast_accum=cfg["fast"],  # noqa: E731
                                  profile=cfg["profile"], splitk=cfg["splitk"])
        y = fn()
        torch.cuda.synchronize(dev)
        sampled_gate(mm, oracle, y, a.view(torch.uint8).cpu().numpy(), bt.view(torch.uint8).cpu().numpy(), sa, sb, cfg,
                     S, scheme, cfg["name"])
        ms = timer.median_ms(fn, steps)
    macs = float(cfg["M"]) * cfg["N"] * cfg["K"]
    return {"workload": workload_text(cfg), "split": f"S={S} {scheme}", "ms": ms, "tflops": 2 * macs / (ms / 1e3) / 1e12,
            "kernel": kernel_of(cfg, S), "exact_vs_oracle": True}


def other_configs(mm, oracle, timer, dev, issue_peak_t):
    """Configurations 1, 3, 4 and slabs of 5 at their own sizes (one GPU)."""
    import torch
    out = {}

    def add(cfg, a, bt, sa, sb, steps=5):
        r = time_config(mm, oracle, timer, dev, cfg, a, bt, sa, sb, steps)
        ipm = INST_PER_MAC.get((r["kernel"], NFMA_OF[cfg["profile"]], "fast" if cfg["fast"] else "slow"))
        r["roofline_frac"] = (float(cfg["M"]) * cfg["N"] * cfg["K"] * ipm / (r["ms"] / 1e3) / 1e12 / issue_peak_t
                              if ipm else None)
        out[cfg["name"]] = r
    g = lambda s: torch.Generator().manual_seed(s)  # noqa: E731
    # 1: ada, 256 cube
    c = dict(name="cfg1_ada_256cube", profile="ada", M=256, N=256, K=256, fa="e4m3", fb="e4m3", out="bfloat16",
             fast=False, splitk="auto")
    add(c, (torch.randn(256, 256, generator=g(0)) * 2).to(torch.float8_e4m3fn),
        torch.randn(256, 256, generator=g(1)).to(torch.float8_e4m3fn), 0.5, 1.25)
    # 3: tall-skinny, e5m2 x e4m3, N(0, 1) * 8; two table shapes with S = 1 and two table rows that split K
    for i, (prof, M, N, K, o, fast) in enumerate([("hopper", 128, 4096, 16384, "float32", False),
                                                   ("hopper", 16, 4096, 8192, "bfloat16", False),
                                                   ("hopper-te", 16, 8192, 28672, "bfloat16", False),
                                                   ("hopper", 128, 128, 16384, "float32", True)]):
        c = dict(name=f"cfg3_{prof}_{M}x{N}x{K}", profile=prof, M=M, N=N, K=K, fa="e5m2", fb="e4m3", out=o, fast=fast,
                 splitk="auto")
        add(c, gaussian_codes(M, K, 8.0, 6 + i, "e5m2"), gaussian_codes(N, K, 8.0, 20 + i, "e4m3"), 2.0 ** -5, 2.0 ** -4)
    # a prefill-like call with few rows and fast accumulation (one chain per output, 32 output tiles): the 16-row
    # kernels take it by default (row groups); the same call with the switch off, for comparison
    c = dict(name="rowgroups_hopper_64x4096x4096", profile="hopper", M=64, N=4096, K=4096, fa="e4m3", fb="e4m3",
             out="bfloat16", fast=True, splitk=1)
    ra, rb = gaussian_codes(64, 4096, 4.0, 60), gaussian_codes(4096, 4096, 4.0, 61)
    add(c, ra, rb, 0.5, 1.25)
    os.environ["MMAEMU_B200_ROW_GROUPS"] = "0"
    try:
        off = time_config(mm, oracle, timer, dev, dict(c, name="rowgroups_off"), ra, rb, 0.5, 1.25, 5)
    finally:
        os.environ.pop("MMAEMU_B200_ROW_GROUPS", None)
    out[c["name"]]["ms_with_8_row_slot_kernels"] = off["ms"]
    out[c["name"]]["kernel"] = "staged_tc_kernel, 16 rows per CTA (row groups)"
    # 4: FP8 projection stack, hopper-te, amax-derived scales
    for i, (N, K) in enumerate([(5760, 1920), (1920, 1920), (24576, 8192)]):
        M = 8192
        x = torch.randn(M, K, generator=g(40 + 3 * i))
        w = torch.randn(N, K, generator=g(41 + 3 * i)) * 0.02
        sx, sw = 448.0 / float(x.abs().max()), 448.0 / float(w.abs().max())
        c = dict(name=f"cfg4_hopper-te_{M}x{N}x{K}", profile="hopper-te", M=M, N=N, K=K, fa="e4m3", fb="e4m3",
                 out="bfloat16", fast=True, splitk="auto")
        add(c, (x * sx).clamp(-448, 448).to(torch.float8_e4m3fn), (w * sw).clamp(-448, 448).to(torch.float8_e4m3fn),
            1.0 / sx, 1.0 / sw, steps=3)
    # 5: one 2048-row slab of the strong-scaling problem (what each of 8 GPUs computes), hopper and ada, and the whole
    # strong-scaling problem on this one GPU (the N = 1 point of the strong-scaling curve)
    bt = strong_bt(dev).view(torch.float8_e4m3fn)
    a = strong_a_rows(0, STRONG["M"], dev).view(torch.float8_e4m3fn)
    for prof in ("hopper", "ada"):
        c = dict(STRONG, name=f"cfg5_slab_{prof}_2048x16384x8192", profile=prof, M=2048)
        add(c, a[:2048], bt, STRONG["scale_a"], STRONG["scale_b"], steps=3)
    add(dict(STRONG, name="cfg5_strong_n1"), a, bt, STRONG["scale_a"], STRONG["scale_b"], steps=3)
    return out


def reference_gpu_context(timer, dev, a_dev, bt_dev, sa_dev, sb_dev, y_ours, cfg):
    """The reference's own CUDA kernels on this GPU, same operands, same timing method: the whole mmaemu.scaled_mm call
    with the headline's arguments, and the chain kernel alone over the full K (one launch). Full outputs are compared
    bit for bit with ours first. Context only."""
    import torch
    ref = load_reference()
    if ref is None:
        return {"unavailable": "the reference package is not installed under baseline/_ref"}
    out = {}
    od = getattr(torch, cfg["out"])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for name in ("h4", "h1"):
            try:
                call = lambda: ref.scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, out_dtype=od,  # noqa: E731
                                             use_fast_accum=cfg["fast"], profile=cfg["profile"], splitk=1,
                                             backend=f"cuda:{name}")
                y = call()
                torch.cuda.synchronize(dev)
                same = bool(torch.equal(y.view(torch.int16), y_ours.view(torch.int16)))
                ms = timer.median_ms(call, 5, warm=1)
                from mmaemu.backends import ChainRequest
                from mmaemu.backends.registry import select
                req = ChainRequest(device=dev, fmt_a="e4m3", fmt_b="e4m3", preset="hopper")
                chain = select(req, f"cuda:{name}").chain_fn(req)
                au, bu = a_dev.view(torch.uint8), bt_dev.view(torch.uint8)
                ms_chain = timer.median_ms(lambda: chain(au, bu), 5, warm=1)
                flops = 2.0 * cfg["M"] * cfg["N"] * cfg["K"]
                out[f"ref_{name}"] = {"whole_call_ms": ms, "value": flops / (ms / 1e3) / 1e12, "unit": "TFLOP/s",
                                      "chain_kernel_alone_ms": ms_chain,
                                      "chain_kernel_alone_tflops": flops / (ms_chain / 1e3) / 1e12,
                                      "bit_identical_to_ours": same,
                                      "what": f"mmaemu.scaled_mm(..., backend='cuda:{name}') of the unmodified reference, "
                                              f"its stock loader; chain kernel = one launch over K={cfg['K']}"}
            except Exception as e:  # noqa: BLE001
                out[f"ref_{name}"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    try:
        ms = timer.median_ms(lambda: torch._scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, out_dtype=od), 5)
        out["native_scaled_mm"] = {"ms": ms, "value": 2.0 * cfg["M"] * cfg["N"] * cfg["K"] / (ms / 1e3) / 1e12,
                                   "unit": "TFLOP/s", "what": "torch._scaled_mm on the B200's own tensor cores (other "
                                                              "numerics; context only)"}
    except Exception as e:  # noqa: BLE001
        out["native_scaled_mm"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return out


# ---------------------------------------------------------------------------------------------------------------
def run_one_gpu(args) -> int:
    import numpy as np  # noqa: F401
    import torch
    import mmaemu_b200 as mm
    from mmaemu_b200 import _lib
    from oracle import oracle
    L = _lib.load()                                            # fails loudly if the CUDA library was never built
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg = dict(HEADLINE)
    if args.shape:
        cfg.update(M=args.shape[0], N=args.shape[1], K=args.shape[2], name="custom")
    if args.fast_accum:
        cfg["fast"] = True
    if args.profile:
        cfg["profile"] = args.profile
    if args.formats:
        cfg.update(fa=args.formats[0], fb=args.formats[1], name="custom")
    if args.out:
        cfg.update(out=args.out, name="custom")
    default_workload = cfg == HEADLINE
    kernel = args.kernel
    backend = "cuda:b200" if kernel == "auto" else f"cuda:b200-{kernel}"
    if default_workload:
        a, bt, sa, sb = headline_operands()
    else:
        a, bt = gaussian_codes(cfg["M"], cfg["K"], 4.0, 2, cfg["fa"]), gaussian_codes(cfg["N"], cfg["K"], 4.0, 3, cfg["fb"])
        sa, sb = torch.tensor(0.37), torch.tensor(1.9)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    od = getattr(torch, cfg["out"])
    es = torch.empty((), dtype=od).element_size()
    a_pin, bt_pin = a.view(torch.uint8).pin_memory(), bt.view(torch.uint8).pin_memory()
    a_dev, bt_dev, sa_dev, sb_dev = a.to(dev), bt.to(dev), sa.to(dev), sb.to(dev)
    timer = Timer(dev)
    kw = dict(out_dtype=od, use_fast_accum=cfg["fast"], profile=cfg["profile"], backend=backend, splitk=1)
    step = lambda: mm.scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, **kw)  # noqa: E731
    out_pin = torch.empty((M, N), dtype=od).pin_memory()

    def step_copies():
        ad = a_pin.to(dev, non_blocking=True).view(a.dtype)
        bd = bt_pin.to(dev, non_blocking=True).view(bt.dtype)
        y = mm.scaled_mm(ad, bd.t(), sa_dev, sb_dev, **kw)
        out_pin.copy_(y, non_blocking=True)
        return y

    a_host, bt_host = a_pin.view(a.dtype), bt_pin.view(bt.dtype)

    def step_e2e():
        # host operands in, host result out: the library stages them, overlaps the copies with the kernels and waits
        return mm.scaled_mm_host(a_host, bt_host.t(), sa, sb, out=out_pin, **kw)

    oracle.build()
    y_gate = step()
    torch.cuda.synchronize(dev)
    if not args.skip_gate:
        sampled_gate(mm, oracle, y_gate, a.view(torch.uint8).numpy(), bt.view(torch.uint8).numpy(), sa, sb, cfg, 1, "none",
                     "headline")
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(dev.index)
    sampler.start()
    launches0 = _lib.launch_count()
    total_ms = timer.total_ms(step, args.steps)
    launches = _lib.launch_count() - launches0
    clocks = sampler.summary()
    for _ in range(2):
        step_e2e()
    torch.cuda.synchronize(dev)
    if not bool(torch.equal(out_pin.view(torch.uint8), y_gate.cpu().view(torch.uint8))):
        raise SystemExit("scaled_mm_host: the result differs from scaled_mm on the same operands")
    e2e_ms = timer.total_ms(step_e2e, args.steps)
    for _ in range(2):
        step_copies()
    torch.cuda.synchronize(dev)
    copies_ms = timer.total_ms(step_copies, args.steps)
    # the same through the C ABI's host-buffer entry point (pinned host operands in, pinned host result out; the call
    # stages, computes and synchronises its stream itself, so it is timed on the host clock)
    host_args = (a_pin.data_ptr(), K, _lib.FMT_CODES[cfg["fa"]], bt_pin.data_ptr(), K, _lib.FMT_CODES[cfg["fb"]],
                 out_pin.data_ptr(), N, _lib.OUT_CODES[cfg["out"]], M, N, K, NFMA_OF[cfg["profile"]], int(cfg["fast"]), 1,
                 0, ctypes.c_float(float(sa)), ctypes.c_float(float(sb)), None, 0,
                 ctypes.c_void_p(timer.stream.cuda_stream))
    for _ in range(2):
        _lib.check("mmb200_scaled_mm_host", L.mmb200_scaled_mm_host(*host_args))
    torch.cuda.synchronize(dev)
    t_host = time.perf_counter()
    for _ in range(args.steps):
        _lib.check("mmb200_scaled_mm_host", L.mmb200_scaled_mm_host(*host_args))
    host_ms = (time.perf_counter() - t_host) * 1e3

    ms = total_ms / args.steps
    macs = float(M) * N * K
    value = 2.0 * macs / (ms / 1e3) / 1e12
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:  # noqa: BLE001
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    auto = L.mmb200_kernel_for(a_dev.data_ptr(), K, bt_dev.data_ptr(), K, K, NFMA_OF[cfg["profile"]], 1)
    if kernel == "integer" or (kernel == "auto" and auto != _lib.KERNEL_CODES["fast"]):
        used = "integer_kernel"
    elif os.environ.get("MMAEMU_B200_WORKSPACE", "1") == "0":
        used = "fast_kernel"
    else:
        used = kernel_of(cfg)
    clk_mhz = clocks.get("sm_mhz") or float(peaks.get("sm_max_mhz", 1965.0))
    peak_t, peak_info = issue_peak(L, timer, clk_mhz)
    key = (used, NFMA_OF[cfg["profile"]], "fast" if cfg["fast"] else "slow")
    ipm = INST_PER_MAC.get(key)
    achieved = macs * ipm / (ms / 1e3) / 1e12 if ipm else None
    algo_bytes = M * K + N * K + M * N * es + 12
    algo_ops = 4 + 12 / NFMA_OF[cfg["profile"]]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int32" if used == "integer_kernel" else "fp32 round-toward-zero FMA + int32 (exact emulation of fp8 x "
                                                         "fp8 blocks)",
        "data": "synthetic",
        "config": {"workload": workload_text(cfg) + f", kernel {used}", "profile": cfg["profile"],
                   "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB write)", "multi_gpu": "single GPU"},
        "roofline": {"bound": "alu-issue", "kernel": used, "achieved": achieved, "peak": peak_t,
                     "unit": "T lane-instructions/s", "frac": achieved / peak_t if achieved else None,
                     "traffic": DRAM_TRAFFIC.get(key + (M, N, K)),
                     "peak_basis": "lane-instructions per second of independent fma.rz.f32 measured in this run with the "
                                   "library's probe kernel (FP32 pipe: 128 lanes per clock and SM; the INT32 ALU pipe "
                                   "issues 64)", "peak_detail": peak_info, "inst_per_mac": ipm,
                     "note": None if ipm else "no ncu capture of this kernel and accumulation mode: no issue-slot figure",
                     "algorithmic_ops_per_mac": algo_ops,
                     "algorithmic_achieved": macs * algo_ops / (ms / 1e3) / 1e12,
                     "hbm": {"achieved_gbs": algo_bytes / (ms / 1e3) / 1e9, "peak_gbs": hbm_peak,
                             "frac": algo_bytes / (ms / 1e3) / 1e9 / hbm_peak,
                             "of": "measured" if "hbm_gbs" in peaks else "fallback"}},
        "e2e": {"value": 2.0 * macs / (e2e_ms / args.steps / 1e3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": (M + N) * K, "d2h_bytes_per_step": M * N * es, "ms_per_step": e2e_ms / args.steps,
                "call": "mmaemu_b200.scaled_mm_host: pinned host operands in, pinned host result out each step; the "
                        "library copies B and decodes it once, then runs row slabs of A on internal streams so that "
                        "copies in both directions overlap the kernels; result checked against scaled_mm bit for bit",
                "torch_copies_then_scaled_mm": {"value": 2.0 * macs / (copies_ms / args.steps / 1e3) / 1e12,
                                                "unit": "TFLOP/s", "ms_per_step": copies_ms / args.steps,
                                                "call": "tensor.to(device) of both operands, mmaemu_b200.scaled_mm, "
                                                        "copy_ of the result to pinned host memory, one stream"},
                "c_abi_host_call": {"value": 2.0 * macs / (host_ms / args.steps / 1e3) / 1e12, "unit": "TFLOP/s",
                                    "ms_per_step": host_ms / args.steps,
                                    "call": "mmb200_scaled_mm_host: pinned host operands in, pinned host result out, "
                                            "device staging inside the call, host clock"}},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if default_workload and not args.headline_only:
        sampler2 = ClockSampler(dev.index)
        sampler2.start()
        line["context"] = reference_gpu_context(timer, dev, a_dev, bt_dev, sa_dev, sb_dev, y_gate, cfg)
        line["context"]["clocks"] = sampler2.summary()
        sampler3 = ClockSampler(dev.index)
        sampler3.start()
        line["configs"] = other_configs(mm, oracle, timer, dev, peak_t)
        line["configs"]["clocks"] = sampler3.summary()
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(a, bt, sa, sb, cfg)
    print(json.dumps(line))
    return 0


def run_multi_gpu(args) -> int:
    import datetime
    import numpy as np
    import torch
    import torch.distributed as dist
    import mmaemu_b200 as mm
    from mmaemu_b200 import _lib
    from mmaemu_b200.sharding import shard_rows, sharded_scaled_mm
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries the one JSON line and nothing else: whatever libraries print there while the job runs (NCCL's
    # version banner, for one) goes to stderr instead
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch N > 1 with torch.distributed.run")
    _lib.load()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    cfg = STRONG
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    od = getattr(torch, cfg["out"])
    m0, m1 = shard_rows(M, world, rank)
    a_dev = strong_a_rows(m0, m1, dev).view(torch.float8_e4m3fn)
    bt_dev = strong_bt(dev).view(torch.float8_e4m3fn)
    sa_dev, sb_dev = torch.tensor(cfg["scale_a"], device=dev), torch.tensor(cfg["scale_b"], device=dev)
    timer = Timer(dev)
    # keep_symmetric: the assembled result is used where the kernels put it (a symmetric-memory buffer that the next call
    # of this shape reuses) instead of being copied out -- every output is still produced on every GPU in every step
    kw = dict(out_dtype=od, use_fast_accum=cfg["fast"], profile=cfg["profile"], splitk=cfg["splitk"],
              input_is_local=True, full_rows=M, assemble=args.assemble, keep_symmetric=True)

    def sync_all():
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    def step():
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return sharded_scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, **kw)

    def step_compute_only():
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return sharded_scaled_mm(a_dev, bt_dev.t(), sa_dev, sb_dev, gather=False, **kw)

    a_pin, bt_pin = a_dev.view(torch.uint8).cpu().pin_memory(), bt_dev.view(torch.uint8).cpu().pin_memory()
    out_pin = torch.empty((m1 - m0, N), dtype=od).pin_memory()

    from mmaemu_b200.sharding import gather_rows
    b0, b1 = shard_rows(N, world, rank)
    bt_pin_own = bt_pin[b0:b1]

    def step_e2e():
        # every input byte crosses the host link once per job: this rank's rows of A, and its 1 / world of B's rows,
        # which one all-gather over NVLink then completes on every GPU
        ad = a_pin.to(dev, non_blocking=True).view(torch.float8_e4m3fn)
        bd = gather_rows(bt_pin_own.to(dev, non_blocking=True), N).view(torch.float8_e4m3fn)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            y = sharded_scaled_mm(ad, bd.t(), sa_dev, sb_dev, **kw)
        out_pin.copy_(y[m0:m1], non_blocking=True)
        return y

    # ---- verification before timing: every rank holds the same assembled result; rank 0 checks rows of every slab
    y = step()
    sync_all()
    digest = hashlib.sha256(y.view(torch.int16).cpu().numpy().tobytes()).hexdigest()
    digests = [None] * world
    dist.all_gather_object(digests, digest)
    if len(set(digests)) != 1:
        raise SystemExit(f"assembled results differ between ranks: {digests}")
    gate = {"sha256_equal_on_all_ranks": True, "sha256": digest[:16]}
    if rank == 0 and not args.skip_gate:
        from oracle import oracle
        oracle.build()
        bt_u8 = bt_pin.numpy()
        checked = 0
        for r in range(world):
            r0, r1 = shard_rows(M, world, r)
            a_r = strong_a_rows(r0, r1, dev)
            nan_rows = torch.nonzero(((a_r & 0x7F) == 0x7F).any(dim=1)).flatten()[:2].cpu().numpy()
            rows = np.unique(np.concatenate([np.array([0, (r1 - r0) // 2 + 1, r1 - r0 - 1]), nan_rows]))
            nan_cols = np.nonzero(((bt_u8 & 0x7F) == 0x7F).any(axis=1))[0][:3]
            cols = np.unique(np.concatenate([np.linspace(0, N - 1, 45).astype(np.int64), nan_cols]))
            sampled_gate(mm, oracle, y[r0:r1], a_r.cpu().numpy(), bt_u8, cfg["scale_a"], cfg["scale_b"], cfg, 1, "none",
                         f"slab of rank {r}", rows=rows, cols=cols)
            checked += rows.size * cols.size
        inf = int(((y.view(torch.int16) & 0x7FFF) == 0x7C00).sum())
        nan = int(((y.view(torch.int16) & 0x7FFF) > 0x7C00).sum())
        gate.update(oracle_sampled_outputs=checked, fp16_inf_outputs=inf, nan_outputs=nan)
        sys.stderr.write(f"gate: all {world} ranks hold sha256 {digest[:16]}...; {checked} sampled outputs of every slab "
                         f"equal the oracle; {inf} outputs overflowed fp16, {nan} are NaN\n")
    del y
    for _ in range(max(3, args.warmup)):
        step()
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    sync_all()
    total_ms = timer.total_ms(step, args.steps)
    sync_all()
    launches = _lib.launch_count() - launches0
    clocks = sampler.summary() if rank == 0 else None
    compute_ms = timer.total_ms(step_compute_only, args.steps)
    sync_all()
    for _ in range(2):
        step_e2e()
    sync_all()
    e2e_ms = timer.total_ms(step_e2e, args.steps)
    sync_all()
    # a row-poor shape of the tall-skinny configuration (16 x 8192 x 28672, hopper-te: the table splits K in two): there
    # is nothing to cut along M, so the ranks take column groups (grid "auto" = 1 x world); every rank ends up with the
    # whole result, compared first with the one-GPU call of the same operands on this rank
    gM, gN, gK = 16, 8192, 28672
    ga = gaussian_codes(gM, gK, 8.0, 8, "e5m2").to(dev)
    gb = gaussian_codes(gN, gK, 8.0, 22, "e4m3").to(dev)
    gsa, gsb = torch.tensor(2.0 ** -5, device=dev), torch.tensor(2.0 ** -4, device=dev)
    gkw = dict(out_dtype=torch.bfloat16, use_fast_accum=False, profile="hopper-te", splitk="auto")

    def grid_step():
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return sharded_scaled_mm(ga, gb.t(), gsa, gsb, grid="auto", assemble=args.assemble, keep_symmetric=True,
                                     **gkw)

    def grid_single():
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return mm.scaled_mm(ga, gb.t(), gsa, gsb, **gkw)
    grid_same = bool(torch.equal(grid_step().view(torch.int16), grid_single().view(torch.int16)))
    sync_all()
    for _ in range(3):
        grid_step()
    sync_all()
    grid_ms = timer.total_ms(grid_step, args.steps)
    sync_all()
    grid_single_ms = timer.total_ms(grid_single, args.steps)
    sync_all()
    t = torch.tensor([total_ms, e2e_ms, compute_ms, grid_ms, grid_single_ms, 0.0 if grid_same else 1.0],
                     dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, compute_ms, grid_ms, grid_single_ms, grid_bad = (float(x) for x in t.cpu())
    if grid_bad:
        raise SystemExit("the column-group result differs from the one-GPU result of the same call")
    if rank == 0:
        from mmaemu_b200 import sharding
        ms = total_ms / args.steps
        macs = float(M) * N * K
        es = torch.empty((), dtype=od).element_size()
        mode = args.assemble
        if mode == "auto":
            mode = "nccl" if any(sharding._symm_failed.values()) or not sharding._symm_cache else "peer"
        line = {
            "metric": METRIC, "value": 2.0 * macs / (ms / 1e3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 round-toward-zero FMA + int32 (exact emulation of fp8 x fp8 blocks)", "data": "synthetic",
            "config": {"workload": workload_text(cfg) + f"; the sharded configuration's recipe (1 % special codes, NaN rows, "
                                   f"fp16 overflow) at a quarter of its 32768 x 32768 x 8192; rows split over {world} "
                                   f"GPUs ({m1 - m0} each), every GPU ends up with the whole result",
                       "profile": cfg["profile"], "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB write)",
                       "multi_gpu": {"peer": "the kernel's epilogue stores each output into every GPU's copy of the "
                                             "result through peer pointers (symmetric memory, NVLink); a device-side "
                                             "barrier before and after; the result stays in that buffer (no copy)",
                                     "nccl": "row slabs + one NCCL all-gather per step"}[mode],
                       "n1_point": "the same problem on one GPU is `configs.cfg5_strong_n1` of the --gpus 1 line"},
            "compute_only_ms_per_step": compute_ms / args.steps,
            "assembly_exposed_ms_per_step": ms - compute_ms / args.steps,
            "gate": gate,
            "e2e": {"value": 2.0 * macs / (e2e_ms / args.steps / 1e3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": ((m1 - m0) + (b1 - b0)) * K, "d2h_bytes_per_step": (m1 - m0) * N * es,
                    "ms_per_step": e2e_ms / args.steps,
                    "call": "mmaemu_b200.sharded_scaled_mm on this rank's rows of A and its 1/N of B's rows copied from "
                            "pinned host memory each step (bytes per rank; mmaemu_b200.sharding.gather_rows completes B "
                            "on every GPU with one all-gather over NVLink), this rank's rows of the assembled result "
                            "copied back"},
            "gpu_launches": int(launches), "clocks": clocks,
            "row_poor_grid": {"workload": f"hopper-te, {gM} x {gN} x {gK}, e5m2 x e4m3 -> bfloat16, slow accumulation, "
                                          f"split-K from the table; column groups 1 x {world}, every GPU ends up with "
                                          f"the whole result",
                              "ms_per_step": grid_ms / args.steps, "one_gpu_ms_per_step": grid_single_ms / args.steps,
                              "tflops": 2.0 * gM * gN * gK / (grid_ms / args.steps / 1e3) / 1e12,
                              "bit_identical_to_one_gpu": True},
        }
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
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
                    help="problem size instead of the headline 4096 4096 4096 (profiling runs, one GPU)")
    ap.add_argument("--formats", nargs=2, choices=("e4m3", "e5m2"), metavar=("A", "B"), default=None,
                    help="FP8 formats of the two operands instead of e4m3 e4m3 (profiling runs, one GPU)")
    ap.add_argument("--out", choices=("float32", "bfloat16", "float16"), default=None, help="output dtype (profiling runs)")
    ap.add_argument("--fast-accum", action="store_true", help="use_fast_accum=True instead of torch's default")
    ap.add_argument("--profile", default=None, help="emulated platform profile (default hopper)")
    ap.add_argument("--skip-gate", action="store_true", help="skip the exactness gate before timing")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="one GPU: skip the context and the other configurations")
    ap.add_argument("--assemble", choices=("auto", "peer", "nccl"), default="auto",
                    help="N > 1: how the result is assembled on every GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: mmaemu_b200 has no CPU fallback")
    if max(1, args.gpus) == 1:
        if int(os.environ.get("WORLD_SIZE", "1")) != 1:
            raise SystemExit("--gpus 1 but WORLD_SIZE > 1")
        return run_one_gpu(args)
    return run_multi_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
