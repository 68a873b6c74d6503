"""Benchmark of the quantised matrix-product path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extra]

Headline workload (`config.workload`): the decode configuration of the int8
weight-only product, `aten::_weight_int8pack_mm` with bf16 A[M, 8192] for M in
{1, 4, 16} against int8 W[28672, 8192] and bf16 per-channel scales. One step is
the three products (one per M). The metric is weight-streaming bandwidth: the
algorithmic bytes of the three launches (weights + scales + A + C) per second.
With N GPUs the weight rows (output columns) are sharded N ways; every rank's
kernel stores its columns straight into every rank's output buffer (peer stores
over NVLink) and counts their arrival, so the product is its own all-gather
(strong scaling). Every rank then rotates through enough distinct copies of its
weight slice that each launch streams from HBM, and the gathered outputs are
checked against the CPU product before and after the timed loops.

One JSON line is printed by rank 0. `value` is timed on the device with the
inputs resident in HBM; `e2e` runs the same step through the public API from
pinned host memory (copy of A up, copy of C down, every call); `roofline` is the
decode kernel against the measured HBM copy bandwidth; `cpu_baseline` is
PyTorch's CPU kernel for the same op (the kernel the reference falls back to and
is validated against) timed on this host's cores; `extra` holds the other
benchmark configurations, each with its own roofline and CPU baseline.

`--impl reference` times that CPU kernel alone, on the same workload and metric.
"""

import argparse
import datetime
import json
import math
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_OUT, K_IN = 28672, 8192
MS = (1, 4, 16)
METRIC = "int8_weight_only_decode_weight_bandwidth"
UNIT = "GB/s"
WORKLOAD = "config2: _weight_int8pack_mm bf16 A[M,8192] M in {1,4,16} x int8 W[28672,8192] + bf16 scales[28672]"
L2_BYTES = 126e6
DTYPE_NOTE = "bf16 activations, int8 weights, float32 accumulation"


def algorithmic_bytes(m, n, k, act_bytes=2):
    """Weights + scales + A + C of one int8 weight-only product."""
    return n * k + act_bytes * n + act_bytes * m * k + act_bytes * m * n


def gen(seed):
    return torch.Generator().manual_seed(seed)


def make_inputs(n_rows, rank_seed=0):
    w = torch.randint(-127, 128, (n_rows, K_IN), dtype=torch.int8, generator=gen(2 + rank_seed))
    s = (torch.rand(n_rows, generator=gen(3 + rank_seed)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16)
    a = {m: torch.randn(m, K_IN, generator=gen(1 + m)).to(torch.bfloat16) for m in MS}
    return a, w, s


def int8_expected(a, w, s, chunk=4096):
    """The reference test's expected value and error bound for _weight_int8pack_mm (tests/python/test_quant.py:31-37):
    the float32 product rounded to A's dtype, and eps * |want| + 2^-20 * (|A| @ |W * s|). Row chunks bound the memory."""
    af = a.float()
    wants, mags = [], []
    for r0 in range(0, w.shape[0], chunk):
        ws = w[r0:r0 + chunk].float() * s[r0:r0 + chunk].float()[:, None]
        wants.append(af @ ws.t())
        mags.append(af.abs() @ ws.abs().t())
    want = torch.cat(wants, 1).to(a.dtype)
    tol = torch.finfo(a.dtype).eps * want.float().abs() + 2.0 ** -20 * torch.cat(mags, 1)
    return want, tol


def config_fp8(m, k, n, rowwise):
    """float8 config: values ~ N(0,1)*64 clamped to +-448; scales 1/64 or uniform in [1/128, 1/32]."""
    a = (torch.randn(m, k, generator=gen(1)) * 64).clamp(-448, 448).to(torch.float8_e4m3fn)
    b = (torch.randn(n, k, generator=gen(2)) * 64).clamp(-448, 448).to(torch.float8_e4m3fn).t()
    if rowwise:
        sa = torch.rand(m, 1, generator=gen(3)) * (1 / 32 - 1 / 128) + 1 / 128
        sb = torch.rand(1, n, generator=gen(4)) * (1 / 32 - 1 / 128) + 1 / 128
    else:
        sa, sb = torch.tensor(1 / 64), torch.tensor(1 / 64)
    return a, b, sa, sb


def config_dyn4_weights(k=4096, n=14336, bs=32):
    """dyn-int4 config: uniform nibbles; bf16 group scales uniform in [5e-3, 5e-2]; bias ~ N(0, 0.1)."""
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=gen(7))
    sc = (torch.rand(n, k // bs, generator=gen(8)) * (5e-2 - 5e-3) + 5e-3).to(torch.bfloat16)
    bias = torch.randn(n, generator=gen(9)) * 0.1
    return w, sc, bias


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def profiled_traffic(grouped=False):
    """DRAM bytes per decode launch (one product, or a grouped launch of the step's three) from the committed ncu summary
    (its `roofline.traffic` lines), or None."""
    path = os.path.join(ROOT, "profiles", "qmm8_skinny_config2.md")
    try:
        with open(path) as f:
            found = re.search(r"([0-9.]+) MB \(the figure `bench\.py` reports as `roofline\.traffic`" + (" for a grouped step" if grouped else "") + r"\)",
                              f.read())
        return float(found.group(1)) * 1e6 if found else None
    except OSError:
        return None


def mark(what):
    """Progress on stderr when TVB200_BENCH_TRACE is set (where a run that got stuck was)."""
    if os.environ.get("TVB200_BENCH_TRACE"):
        print(f"[bench {time.strftime('%H:%M:%S')}] {what}", file=sys.stderr, flush=True)


def roof(bound, achieved, peak, unit, kernel, peak_note):
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "kernel": kernel,
            "peak_source": peak_note}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.proc, self.path = None, None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(device_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 7 and parts[0].replace(".", "").isdigit():
                    rows.append(parts)
        os.unlink(self.path)
        if not rows:
            return out
        busiest = sorted(float(r[2]) if r[2].replace(".", "").isdigit() else 0.0 for r in rows)
        load_cut = busiest[len(busiest) // 2]
        under_load = [r for r in rows if (float(r[2]) if r[2].replace(".", "").isdigit() else 0.0) >= load_cut] or rows
        out["sm_mhz"] = statistics.median(float(r[0]) for r in under_load)
        out["sm_max_mhz"] = float(rows[0][1])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        out["reasons"] = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        out["samples"] = len(rows)
        return out


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_time(fn, budget_s, min_reps=3, max_reps=50):
    """Median seconds of fn() on the host after one warm call, repeated within a time budget."""
    fn()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_reps or (time.perf_counter() < t_end and len(times) < max_reps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def run_reference(args, rank):
    """The reference arm: the CPU kernel the reference falls back to (crates/pyvk/csrc/quant.cpp:77), all host threads."""
    if rank != 0:
        return
    # torchrun gives every rank OMP_NUM_THREADS=1; this arm is rank 0 alone and takes the host's cores
    if torch.get_num_threads() < host_threads():
        torch.set_num_threads(host_threads())
    a, w, s = make_inputs(N_OUT)
    step_bytes = sum(algorithmic_bytes(m, N_OUT, K_IN) for m in MS)
    for _ in range(max(args.warmup, 1)):
        for m in MS:
            torch._weight_int8pack_mm(a[m], w, s)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for m in MS:
            torch._weight_int8pack_mm(a[m], w, s)
    dt = (time.perf_counter() - t0) / args.steps
    value = step_bytes / dt / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": DTYPE_NOTE, "data": "synthetic", "config": {"workload": WORKLOAD},
        "details": {"device": "host CPU", "torch": torch.__version__, "os_cpu_count": os.cpu_count()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": "the full workload, every step: torch._weight_int8pack_mm on CPU tensors, the kernel the "
                                   "reference hands this op to without a GPU and checks its shader against"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Timer:
    """CUDA-event timing on the backend's stream."""

    def __init__(self, tv, stream, device_index):
        self.tv, self.stream, self.dev = tv, stream, device_index

    def region(self, fn, iters):
        """Milliseconds of `iters` calls of fn(i) queued back to back between two events."""
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(self.stream)
        for i in range(iters):
            fn(i)
        e.record(self.stream)
        self.tv.synchronize(self.dev)
        return s.elapsed_time(e)

    def median(self, fn, iters, warm=3):
        """Median milliseconds of one fn(), an event pair per call."""
        for _ in range(warm):
            fn()
        self.tv.synchronize(self.dev)
        evs = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(self.stream)
            fn()
            e.record(self.stream)
            evs.append((s, e))
        self.tv.synchronize(self.dev)
        return statistics.median(s.elapsed_time(e) for s, e in evs)


# ---------------------------------------------------------------------------------------------- extras, one GPU

def extra_config1(tv, timer, peaks, cpu):
    """Config 1: _weight_int8pack_mm, float32 A[32,4096] x int8 W[4096,4096] + float32 scales. The 17 MB of weights fit the
    L2, so twelve distinct weight copies are used in turn for the HBM figure (201 MB, more than the L2 holds) and one copy for
    the L2-resident figure; both replay a graph of twelve products."""
    from torch_vulkan_b200 import shard

    m, k, n = 32, 4096, 4096
    a = torch.randn(m, k, generator=gen(1))
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(2))
    s = torch.rand(n, generator=gen(3)) * (2e-2 - 1e-3) + 1e-3
    av, sv = a.to("vk"), s.to("vk")
    copies = [torch.roll(w, 16 * i, 0).to("vk") for i in range(12)]
    scales = [torch.roll(s, 16 * i, 0).to("vk") for i in range(12)]
    got = torch._weight_int8pack_mm(av, copies[0], sv).cpu()
    want, tol = int8_expected(a, w, s)
    if not ((got - want).abs() <= tol).all():
        raise SystemExit("bench.py: config 1 product outside the reference's bound")
    nbytes = algorithmic_bytes(m, n, k, act_bytes=4)
    out = {}
    for label, pick in (("hbm_streaming", lambda i: i), ("l2_resident", lambda i: 0)):
        graph = shard.StepGraph(lambda: [torch._weight_int8pack_mm(av, copies[pick(i)], scales[pick(i)]) for i in range(12)])
        us = timer.median(graph.replay, 7) / 12 * 1e3
        out[label] = {"us_per_product": us, "weight_gbs": nbytes / us / 1e3}
        del graph
    res = {"workload": "config1: _weight_int8pack_mm f32 A[32,4096] x int8 W[4096,4096] + f32 scales[4096]", **out,
           "roofline": roof("hbm", out["hbm_streaming"]["weight_gbs"], peaks["hbm_gbs"], "GB/s", "qmm8_f32_tc_kernel",
                            peaks["source"] + " HBM copy bandwidth; 17.84 MB per product, twelve weight copies in turn")}
    if cpu:
        sec, reps = cpu_time(lambda: torch._weight_int8pack_mm(a, w, s), 2.0)
        res["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "ms": sec * 1e3, "cores": torch.get_num_threads(),
                               "kind": "reference", "sample": f"{reps} full products (median), torch._weight_int8pack_mm on CPU"}
    del copies, scales
    return {"config1_int8_f32": res}


def extra_fp8(tv, timer, peaks, cpu, quick):
    """Config 4: float8 _scaled_mm 8192^3, tensor-wise and row-wise scales, bf16 output."""
    out = {}
    m = n = k = 8192
    peak = 2 * peaks["bf16_tflops"]
    for rowwise in (False, True):
        a, b, sa, sb = config_fp8(m, k, n, rowwise)
        av, bv, sav, sbv = a.to("vk"), b.t().to("vk").t(), sa.to("vk"), sb.to("vk")
        ms = timer.median(lambda: torch._scaled_mm(av, bv, sav, sbv, out_dtype=torch.bfloat16), 5 if quick else 10)
        tf = 2.0 * m * n * k / ms / 1e9
        key = "fp8_scaled_mm_8192_" + ("rowwise" if rowwise else "tensorwise")
        out[key] = {"tflops": tf, "ms": ms, "frac_of_2x_measured_bf16": tf / peak, "frac_of_nominal_fp8": tf / 4500.0,
                    "roofline": roof("tensor", tf, peak, "TFLOP/s", "gemm_tc_kernel<kind::f8f6f4>",
                                     "2 x the " + peaks["source"] + " bf16 GEMM figure (no float8 peak was measured)")}
        if cpu:
            # the reference's emulated formula (crates/pyvk/csrc/quant.cpp:283-299) with the host's sgemm, on a 2048^3 corner
            c = 2048
            ac, bc = a[:c, :c], b[:c, :c]
            sac = sa[:c] if rowwise else sa
            sbc = sb[:, :c] if rowwise else sb
            sec, reps = cpu_time(lambda: ((ac.float() * sac) @ (bc.float() * sbc)).to(torch.bfloat16), 1.5)
            out[key]["cpu_baseline"] = {"value": 2.0 * c ** 3 / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                        "kind": "reference", "ms_extrapolated_to_8192": sec * 64 * 1e3,
                                        "sample": f"{reps} runs (median) of the emulated formula on a 2048^3 corner of the operands; "
                                                  "the 8192^3 time is 64 times that, extrapolated"}
        del av, bv
    return out


def extra_mm(tv, timer, peaks, quick):
    """The unquantised products either side of the path: aten::mm bf16 8192^3 and int8 weight-only at prefill sizes."""
    out = {}
    m = n = k = 8192
    a16 = torch.randn(m, k, generator=gen(21)).to(torch.bfloat16).to("vk")
    w16 = torch.randn(n, k, generator=gen(22)).to(torch.bfloat16).to("vk")
    ms = timer.median(lambda: torch.mm(a16, w16.t()), 5 if quick else 10)
    tf = 2.0 * m * n * k / ms / 1e9
    out["bf16_mm_8192"] = {"tflops": tf, "ms": ms, "frac_of_measured_bf16": tf / peaks["bf16_tflops"]}
    del a16, w16
    for mm, nn_, kk in ((2048, 14336, 4096),) if quick else ((2048, 14336, 4096), (8192, 8192, 8192)):
        a8 = torch.randn(mm, kk, generator=gen(31)).to(torch.bfloat16).to("vk")
        w8 = torch.randint(-127, 128, (nn_, kk), dtype=torch.int8, generator=gen(32)).to("vk")
        s8 = (torch.rand(nn_, generator=gen(33)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16).to("vk")
        ms = timer.median(lambda: torch._weight_int8pack_mm(a8, w8, s8), 5)
        tf = 2.0 * mm * nn_ * kk / ms / 1e9
        out[f"int8_weight_only_m{mm}_n{nn_}_k{kk}"] = {"tflops": tf, "ms": ms, "frac_of_measured_bf16": tf / peaks["bf16_tflops"]}
        del a8, w8, s8
    return out


def extra_dyn4(tv, timer, peaks, cpu, quick):
    """Config 3: _dyn_quant_matmul_4bit, float32 [M,4096] x int4 [14336,4096], block 32, bias; plus its decoding shapes."""
    from torch_vulkan_b200 import shard

    out = {}
    n, k, bs = 14336, 4096, 32
    w, sc, bias = config_dyn4_weights()
    packed = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bias.to("vk"), bs, k, n)
    peak = 2 * peaks["bf16_tflops"]
    cpu_row_s = None
    if cpu:
        # PyTorch's CPU kernel runs at about 1 GOP/s: a 16-row slice is timed and scaled by rows (rows are independent,
        # crates/vkcore/shaders/qmm4.slang:134)
        packed_cpu = torch._dyn_quant_pack_4bit_weight(w, sc, bias, bs, k, n)
        x16 = torch.randn(16, k, generator=gen(11))
        sec, _ = cpu_time(lambda: torch._dyn_quant_matmul_4bit(x16, packed_cpu, bs, k, n), 3.0, min_reps=1, max_reps=3)
        cpu_row_s = sec / 16
        del packed_cpu
    for mm in ((128,) if quick else (128, 512, 2048)):
        xv = torch.randn(mm, k, generator=gen(11)).to("vk")
        for mode in ("exact", "fast"):  # exact: bit for bit (the default); fast: TORCH_VK_QMM4=fast, rtol 1e-5
            before = os.environ.get("TORCH_VK_QMM4")
            if mode == "fast":
                os.environ["TORCH_VK_QMM4"] = "fast"
            ms = timer.median(lambda: torch._dyn_quant_matmul_4bit(xv, packed, bs, k, n), 5)
            if mode == "fast":
                os.environ.pop("TORCH_VK_QMM4", None)
                if before is not None:
                    os.environ["TORCH_VK_QMM4"] = before
            tops = 2.0 * mm * n * k / ms / 1e9
            entry = {"tops": tops, "ms": ms, "frac_of_2x_measured_bf16": tops / peak,
                     "roofline": roof("tensor", tops, peak, "TOP/s",
                                      "qmm4_tc_kernel<kind::i8>" if mode == "exact" else "gemm_tc_kernel<kind::f16> (fast route)",
                                      "2 x the " + peaks["source"] + " bf16 GEMM figure (no int8 peak was measured)")}
            if cpu_row_s is not None and mode == "exact":
                entry["cpu_baseline"] = {"value": 2.0 * n * k / cpu_row_s / 1e12, "unit": "TOP/s", "cores": torch.get_num_threads(),
                                         "kind": "reference", "ms_extrapolated": cpu_row_s * mm * 1e3,
                                         "sample": "torch._dyn_quant_matmul_4bit on CPU, a 16-row slice timed and scaled by rows: extrapolated"}
            out[f"dyn_int4_m{mm}_{mode}"] = entry
    # decoding (at most 16 rows): twelve products replayed as one graph, against the bytes of the real int4 data
    # (29.36 MB of nibbles + 3.67 MB of block scales + bias, activations and outputs)
    packs = [packed] + [torch._dyn_quant_pack_4bit_weight(torch.roll(w, i, 0).to("vk"), sc.to("vk"), bias.to("vk"), bs, k, n)
                        for i in (1, 2, 3)]  # four weight sets in turn: 147 MB in their decode form, more than the L2 holds
    for mm in (1, 16):
        xv = torch.randn(mm, k, generator=gen(12)).to("vk")
        graph = shard.StepGraph(lambda: [torch._dyn_quant_matmul_4bit(xv, packs[i % 4], bs, k, n) for i in range(12)])
        ms = timer.median(graph.replay, 5) / 12
        nbytes = n * k // 2 + n * (k // bs) * 2 + n * 4 + mm * k * 4 + mm * n * 4
        gbs = nbytes / ms / 1e6
        entry = {"us": ms * 1e3, "weight_gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                 "roofline": roof("hbm", gbs, peaks["hbm_gbs"], "GB/s", "qmm4_decode_kernel", peaks["source"] + " HBM copy bandwidth")}
        if cpu_row_s is not None:
            entry["cpu_baseline"] = {"value": nbytes / (cpu_row_s * mm) / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
                                     "kind": "reference", "sample": "the 16-row CPU timing above scaled by rows: extrapolated"}
        out[f"dyn_int4_decode_m{mm}"] = entry
        del graph
    del packs
    tv.empty_cache()
    return out


STACK_SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]  # qkv, o, gate_up, down: (n, k)


def stack_host_weights():
    """The four weight matrices of a layer: uniform int8, and per-channel scales uniform in [0.5, 1.5] / (73.6 sqrt(k)) (73.6:
    the root mean square of the weights), so that every product keeps the magnitude of its input and the activations of a
    128-product chain stay finite and away from zero: the chain's outputs can be checked."""
    host = []
    for i, (n, k) in enumerate(STACK_SHAPES):
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(40 + i))
        sc = ((torch.rand(n, generator=gen(50 + i)) + 0.5) / (73.6 * math.sqrt(k))).to(torch.bfloat16)
        host.append((w, sc))
    return host


def check_last_layer(host, qkv, o, gu, h, what):
    """The last layer's o, gate_up and down products (device results, already on the host) against the CPU product of their
    own inputs, within the reference's bound."""
    for got, a_in, (w, sc), name in ((o, qkv[:, :4096], host[1], "o"), (gu, o, host[2], "gate_up"), (h, gu[:, :14336], host[3], "down")):
        want, tol = int8_expected(a_in.contiguous(), w, sc)
        if not ((got.float() - want.float()).abs() <= tol).all():
            raise SystemExit(f"bench.py: {what}: last layer's {name} product outside the reference's bound")


def stack_chain(shard, weights, x, m, device_index, channel=None, gathered=None):
    """The stack's 128 products as one chain (tvb_qmm8_chain_*): every product takes the previous one's output (its first 4096
    or 14336 columns) as its A. Returns the chain and the last layer's four output buffers."""
    prods, h, last = [], x, None
    for layer in weights:
        if channel is None:
            bufs = [torch.empty(m, n, dtype=torch.bfloat16, device=x.device) for n, _ in STACK_SHAPES]
            outs = bufs
        else:
            bufs, outs = [g.bufs[0] for g in gathered], [(g, 0) for g in gathered]
        (wq, sq), (wo, so), (wg, sg), (wd, sd) = layer
        prods += [(h, wq, sq, outs[0]), (bufs[0][:, :4096], wo, so, outs[1]), (bufs[1], wg, sg, outs[2]), (bufs[2][:, :14336], wd, sd, outs[3])]
        h, last = bufs[3], bufs
    return shard.ProductChain(prods, device_index, channel), last


def int8_stack(tv, timer, peaks, cpu, ms_list=(1, 8, 64), layers=32):
    """Config 5 on one GPU: the int8 weight-only Linears of a 32-layer decoder (hidden 4096: qkv 6144, o 4096, gate_up 28672,
    down from 14336; 7 GB of weights, every layer its own buffers), decoded as one replayed graph of 128 products per step.
    Between the products stands the stack's glue only (the first 4096 columns of qkv feed o, the first 14336 of gate_up feed
    down)."""
    from torch_vulkan_b200 import _native, shard

    host = stack_host_weights()
    weights = [[(w.to("vk"), sc.to("vk")) for w, sc in host] for _ in range(layers)]
    wbytes = layers * sum(n * k for n, k in STACK_SHAPES)
    out = {}
    for m in ms_list:
        x_host = torch.randn(m, 4096, generator=gen(60)).to(torch.bfloat16)
        x = x_host.to("vk")

        def step():
            keep, h = [], x
            for (wq, sq), (wo, so), (wg, sg), (wd, sd) in weights:
                qkv = torch._weight_int8pack_mm(h, wq, sq)
                o = torch._weight_int8pack_mm(qkv[:, :4096], wo, so)
                gu = torch._weight_int8pack_mm(o, wg, sg)
                h = torch._weight_int8pack_mm(gu[:, :14336], wd, sd)
                keep += [qkv, o, gu, h]
            return keep

        graph = shard.StepGraph(step)
        for _ in range(3):
            graph.replay()
        iters = 10
        ms_ops = timer.region(lambda i: graph.replay(), iters) / iters
        del graph
        # the same step as one launch of the persistent decode kernel (m > 16: one pass per 16 rows)
        mark(f"int8 stack m={m}: per-product graph {ms_ops:.3f} ms; chain")
        chain, last = stack_chain(shard, weights, x, m, timer.dev)
        for _ in range(3):
            chain.run()
        ms_chain = timer.region(lambda i: chain.run(), iters) / iters
        check_last_layer(host, *[t.cpu() for t in last], f"int8 stack as a chain (m={m})")
        del chain, last
        ms = min(ms_ops, ms_chain)
        gbs = wbytes / ms / 1e6
        entry = {"ms_per_token_step": ms, "weight_gbs": gbs, "products": 4 * layers, "weight_bytes": wbytes,
                 "one_launch_per_product_ms": ms_ops, "chain_ms": ms_chain,
                 "roofline": roof("hbm", gbs, peaks["hbm_gbs"], "GB/s",
                                  "qmm8_chain_kernel" if ms_chain <= ms_ops else ("qmm8_skinny_kernel" if m <= 32 else "qmm8 tcgen05 kernels"),
                                  peaks["source"] + " HBM copy bandwidth, weight bytes only")}
        if m == 1 or m == 16:
            # The same stack with its two residual additions (after o and after down): in the decode kernel's epilogue
            # (tvb_qmm8_linear, 128 launches per step) against a product and an add each (192 launches).
            def step_residual(fused):
                def run():
                    keep, h = [], x
                    for (wq, sq), (wo, so), (wg, sg), (wd, sd) in weights:
                        qkv = torch._weight_int8pack_mm(h, wq, sq)
                        if fused:
                            o = _native.int8_linear(qkv[:, :4096], wo, so, None, h)
                        else:
                            o = torch._weight_int8pack_mm(qkv[:, :4096], wo, so)
                            o += h
                        gu = torch._weight_int8pack_mm(o, wg, sg)
                        if fused:
                            h = _native.int8_linear(gu[:, :14336], wd, sd, None, o)
                        else:
                            h = torch._weight_int8pack_mm(gu[:, :14336], wd, sd)
                            h += o
                        keep += [qkv, o, gu, h]
                    return keep

                return run

            for label, fused in (("residual_in_epilogue", True), ("residual_as_own_launch", False)):
                graph = shard.StepGraph(step_residual(fused))
                for _ in range(3):
                    graph.replay()
                entry[label + "_ms"] = timer.region(lambda i: graph.replay(), iters) / iters
                del graph
        if cpu:
            def cpu_pass():
                h = x_host
                for _ in range(layers):
                    qkv = torch._weight_int8pack_mm(h, *host[0])
                    o = torch._weight_int8pack_mm(qkv[:, :4096].contiguous(), *host[1])
                    gu = torch._weight_int8pack_mm(o, *host[2])
                    h = torch._weight_int8pack_mm(gu[:, :14336].contiguous(), *host[3])
                return h

            sec, reps = cpu_time(cpu_pass, 2.0, min_reps=1, max_reps=5)
            entry["cpu_baseline"] = {"value": wbytes / sec / 1e9, "unit": "GB/s", "ms_per_token_step": sec * 1e3,
                                     "cores": torch.get_num_threads(), "kind": "reference",
                                     "sample": f"{reps} passes (median) of the 128 products with torch._weight_int8pack_mm on CPU "
                                               "(one set of the four weight matrices reused by every layer)"}
        out[f"int8_stack_32layers_m{m}"] = entry
    del weights
    tv.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------- extras, N GPUs

def int8_stack_sharded(tv, timer, peaks, channel, rank, world, dev, ms_list=(1, 8, 64), layers=32):
    """Config 5 with every Linear's weight rows sharded `world` ways: 128 fused sharded products per step, each kernel
    storing its columns into every rank's buffer and waiting by itself for the previous product's columns from all ranks (no
    call between the products), one wait at the end of the step; the whole step is one replayed graph. The last layer's
    products are checked on every rank against the CPU product of the gathered inputs."""
    from torch_vulkan_b200 import shard

    host = stack_host_weights()
    weights = [[(shard.shard_rows(w, rank, world).to(dev), shard.shard_rows(sc, rank, world).to(dev)) for w, sc in host]
               for _ in range(layers)]
    wbytes = layers * sum(n * k for n, k in STACK_SHAPES)
    out = {}
    for m in ms_list:
        x = torch.randn(m, 4096, generator=gen(60)).to(torch.bfloat16).to(dev)
        outs = [shard.GatheredOutputs(m, n, torch.bfloat16, channel, depth=1) for n, _ in STACK_SHAPES]
        iters = 10
        chain, last = stack_chain(shard, weights, x, m, channel.dev, channel, outs)
        for _ in range(3):
            chain.run()
        tv.synchronize(channel.dev)
        shard.barrier()
        ms = timer.region(lambda i: chain.run(), iters) / iters
        check_last_layer(host, *[t.cpu() for t in last], f"rank {rank}: sharded int8 stack as a chain (m={m})")
        shard.barrier()
        ms_ops = None
        if True:
            # the other way: one launch per product (tvb_qmm8_gather; a pass per 16 rows), each kernel waiting for the previous
            # product's columns
            def step():
                h = x
                for (wq, sq), (wo, so), (wg, sg), (wd, sd) in weights:
                    qkv = outs[0].weight_int8pack_mm(h, wq, sq)
                    o = outs[1].weight_int8pack_mm(qkv[:, :4096], wo, so)
                    gu = outs[2].weight_int8pack_mm(o, wg, sg)
                    h = outs[3].weight_int8pack_mm(gu[:, :14336], wd, sd)
                channel.wait()
                return qkv, o, gu, h

            graph = shard.StepGraph(step, channel.dev)
            for _ in range(3):
                graph.replay()
            tv.synchronize(channel.dev)
            shard.barrier()
            ms_ops = timer.region(lambda i: graph.replay(), iters) / iters
            check_last_layer(host, *[t.cpu() for t in graph.outputs], f"rank {rank}: sharded int8 stack, one launch per product (m={m})")
            del graph
            shard.barrier()
        t = torch.tensor([ms, ms_ops if ms_ops is not None else 0.0], dtype=torch.float64, device=torch.device("cuda", channel.dev))
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_chain, ms_ops = t[0].item(), (t[1].item() if ms_ops is not None else None)
        ms = ms_chain if ms_ops is None else min(ms_chain, ms_ops)
        gbs = wbytes / ms / 1e6
        out[f"int8_stack_32layers_m{m}_sharded"] = {
            "ms_per_token_step": ms, "weight_gbs": gbs, "products": 4 * layers, "weight_bytes": wbytes, "n_gpus": world,
            "chain_ms": ms_chain, "one_launch_per_product_ms": ms_ops,
            "checked": "last layer's o, gate_up and down products on every rank",
            "roofline": roof("hbm", gbs / world, peaks["hbm_gbs"], "GB/s",
                             ("qmm8_chain_kernel" if ms == ms_chain else "qmm8_skinny_kernel") + " (sharded, fused gather)",
                             peaks["source"] + " HBM copy bandwidth per GPU, weight bytes only")}
        del chain, last, outs
    del weights
    tv.empty_cache()
    return out


def fp8_sharded(tv, timer, peaks, channel, rank, world, dev):
    """Config 4 with B's columns sharded `world` ways: every rank multiplies A by its [8192, 8192 / world] slice and the
    [8192, 8192] output is assembled on every rank, either by the kernel's own epilogue (tvb_scaled_mm_gather: every tile
    stored into every rank's buffer over NVLink while the other tiles are multiplied) or by an NCCL all-gather after the
    product. Each rank checks 64 rows of the assembled output against the reference's formula."""
    from torch_vulkan_b200 import shard

    out = {}
    m = n = k = 8192
    fused_out = shard.GatheredOutputs(m, n, torch.bfloat16, channel) if channel is not None else None
    for rowwise in (False, True):
        a, b, sa, sb = config_fp8(m, k, n, rowwise)
        b_sh, sb_sh = shard.shard_scaled_mm_b(b, sb, rank, world)
        av, bv = a.to(dev), b_sh.t().contiguous().to(dev).t()
        sav, sbv = sa.to(dev), sb_sh.to(dev)
        r0 = 64 * rank
        af, bf = a[r0:r0 + 64].float() * (sa[r0:r0 + 64] if rowwise else sa), b.float() * sb
        want = (af @ bf).to(torch.bfloat16)
        tol = torch.finfo(torch.bfloat16).eps * want.float().abs() + 2.0 ** -20 * (af.abs() @ bf.abs())

        def fused(buf=None):
            c = fused_out.scaled_mm(av, bv, sav, sbv, buf=buf)
            channel.wait()
            return c

        ways = [("NCCL all-gather of the column slices", lambda: shard.scaled_mm(av, bv, sav, sbv, out_dtype=torch.bfloat16))]
        if fused_out is not None:
            ways.insert(0, ("fused into the tcgen05 epilogue (peer stores over NVLink)", fused))
        results = {}
        for label, fn in ways:
            got = fn()
            if not ((got[r0:r0 + 64].cpu().float() - want.float()).abs() <= tol).all():
                raise SystemExit(f"bench.py: rank {rank}: sharded float8 product ({label}) outside the reference's bound")
            shard.barrier()
            if fn is fused:  # (replayed as a graph: the product and the wait kernel without the host's launch calls between them)
                graph = shard.StepGraph(lambda: fused(0), channel.dev, warm=False)
                ms = timer.median(graph.replay, 5)
                del graph
            else:
                ms = timer.median(fn, 5)
            t = torch.tensor([ms], dtype=torch.float64, device=torch.device("cuda", torch.cuda.current_device()))
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            results[label] = t.item()
        label = min(results, key=results.get)
        ms = results[label]
        tf = 2.0 * m * n * k / ms / 1e9
        out["fp8_scaled_mm_8192_" + ("rowwise" if rowwise else "tensorwise") + "_sharded"] = {
            "tflops": tf, "ms": ms, "n_gpus": world, "gather": label, "ms_by_gather": results,
            "checked": "64 rows of the assembled output on every rank",
            "roofline": roof("tensor", tf / world, 2 * peaks["bf16_tflops"], "TFLOP/s", "gemm_tc_kernel<kind::f8f6f4> (sharded)",
                             "2 x the " + peaks["source"] + " bf16 GEMM figure per GPU")}
        del av, bv
    del fused_out
    tv.empty_cache()
    return out


def run_only(tv, timer, which, iters, slice_world):
    """One configuration, `iters` launches after one warm-up (small enough to sit under a profiler)."""
    stream = timer.stream
    if which in ("fp8", "fp8_big"):
        m = n = k = 4096 if which == "fp8" else 8192
        a, b, sa, sb = config_fp8(m, k, n, True)
        av, bv, sav, sbv = a.to("vk"), b.t().to("vk").t(), sa.to("vk"), sb.to("vk")
        fn = lambda: torch._scaled_mm(av, bv, sav, sbv, out_dtype=torch.bfloat16)  # noqa: E731
        flops = 2.0 * m * n * k
    elif which == "bf16_mm":
        m = n = k = 4096
        a16 = torch.randn(m, k, generator=gen(21)).to(torch.bfloat16).to("vk")
        w16 = torch.randn(n, k, generator=gen(22)).to(torch.bfloat16).to("vk")
        fn = lambda: torch.mm(a16, w16.t())  # noqa: E731
        flops = 2.0 * m * n * k
    elif which == "config1":
        m, k, n = 32, 4096, 4096
        av = torch.randn(m, k, generator=gen(1)).to("vk")
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(2))
        sv = (torch.rand(n, generator=gen(3)) * (2e-2 - 1e-3) + 1e-3).to("vk")
        copies = [torch.roll(w, 16 * i, 0).to("vk") for i in range(12)]
        from torch_vulkan_b200 import shard

        graph = shard.StepGraph(lambda: [torch._weight_int8pack_mm(av, copies[i], sv) for i in range(12)])
        us = timer.median(graph.replay, max(iters, 5)) / 12 * 1e3
        graph1 = shard.StepGraph(lambda: [torch._weight_int8pack_mm(av, copies[0], sv) for i in range(12)])
        us1 = timer.median(graph1.replay, max(iters, 5)) / 12 * 1e3
        single = timer.median(lambda: torch._weight_int8pack_mm(av, copies[0], sv), 10) * 1e3
        return {"only": which, "us_per_product_hbm_streaming": us, "weight_gbs": algorithmic_bytes(m, n, k, 4) / us / 1e3,
                "us_per_product_l2_resident": us1, "us_single_eager_launch": single}
    elif which == "int8_slice":
        # the weight slice one rank of `slice_world` owns in config 2, on one GPU: enough copies in turn to stream from HBM
        rows = N_OUT // slice_world
        nsets = weight_sets(rows * K_IN, slice_world)
        w = torch.randint(-127, 128, (rows, K_IN), dtype=torch.int8, generator=gen(2))
        sv = (torch.rand(rows, generator=gen(3)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16).to("vk")
        copies = [torch.roll(w, 16 * i, 0).to("vk") for i in range(nsets)]
        a = {m: torch.randn(m, K_IN, generator=gen(1 + m)).to(torch.bfloat16).to("vk") for m in MS}
        from torch_vulkan_b200 import shard

        res = {"only": which, "rows": rows, "weight_sets": nsets, "us_per_launch_by_m": {}}
        for m in MS:
            graph = shard.StepGraph(lambda: [torch._weight_int8pack_mm(a[m], copies[i % nsets], sv) for i in range(4 * nsets)])
            res["us_per_launch_by_m"][str(m)] = timer.median(graph.replay, max(iters, 3)) / (4 * nsets) * 1e3
            del graph
        res["hbm_floor_us"] = rows * K_IN / 6543.1e3
        return res
    elif which == "chain_probe":
        # the persistent decode kernel on config 2's weights: one product, three independent ones, three that wait for one
        # another, against one launch per product
        from torch_vulkan_b200 import shard

        w = torch.randint(-127, 128, (N_OUT, K_IN), dtype=torch.int8, generator=gen(2)).to("vk")
        sv = (torch.rand(N_OUT, generator=gen(3)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16).to("vk")
        a = {m: torch.randn(m, K_IN, generator=gen(1 + m)).to(torch.bfloat16).to("vk") for m in MS}
        outs = {m: torch.empty(m, N_OUT, dtype=torch.bfloat16, device="vk") for m in MS}
        res = {"only": which}
        for label, prods in (("one_product_m16", [(a[16], w, sv, outs[16])]),
                             ("three_independent", [(a[m], w, sv, outs[m], i) for i, m in enumerate(MS)]),
                             ("three_in_sequence", [(a[m], w, sv, outs[m], 0) for m in MS])):
            chain = shard.ProductChain(prods, timer.dev)
            res[label + "_us"] = timer.median(chain.run, max(iters, 5)) * 1e3
            del chain
        res["one_launch_m16_us"] = timer.median(lambda: torch._weight_int8pack_mm(a[16], w, sv), max(iters, 5)) * 1e3
        return res
    elif which == "dyn4_decode":
        # four weight sets in turn (147 MB of int4 data and scales in their decode form, more than the L2 holds)
        mm = 16
        w, sc, bias = config_dyn4_weights()
        packs = [torch._dyn_quant_pack_4bit_weight(torch.roll(w, i, 0).to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
                 for i in range(4)]
        xv = torch.randn(mm, 4096, generator=gen(11)).to("vk")
        state = {"i": 0}

        def fn():
            state["i"] += 1
            return torch._dyn_quant_matmul_4bit(xv, packs[state["i"] % 4], 32, 4096, 14336)

        for _ in range(4):
            fn()
        flops = 2.0 * mm * 14336 * 4096
    elif which == "dyn4":
        mm = 512
        w, sc, bias = config_dyn4_weights()
        packed = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
        xv = torch.randn(mm, 4096, generator=gen(11)).to("vk")
        fn = lambda: torch._dyn_quant_matmul_4bit(xv, packed, 32, 4096, 14336)  # noqa: E731
        flops = 2.0 * mm * 14336 * 4096
    else:
        # int8_large_m: the 16-bit GEMM over (cached) widened weights; int8_mid_m: the kernel that widens in its main loop,
        # which needs no copy of the weights
        m, n, k = (2048 if which == "int8_large_m" else 256), 14336, 4096
        a = torch.randn(m, k, generator=gen(1)).to(torch.bfloat16).to("vk")
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(2)).to("vk")
        s = (torch.rand(n, generator=gen(3)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16).to("vk")
        if which == "int8_large_m":
            fn = lambda: torch._weight_int8pack_mm(a, w, s)  # noqa: E731
        else:
            # straight through the C ABI, variant 3: the kernel the op falls back to when its budget for widened copies is spent
            from torch_vulkan_b200 import cabi

            ac, wc, sc_ = tv.as_cuda(a), tv.as_cuda(w), tv.as_cuda(s)
            fn = lambda: cabi.qmm8(ac, wc, sc_, variant=3)  # noqa: E731
        flops = 2.0 * m * n * k
    fn()
    tv.synchronize()
    ms = timer.region(lambda i: fn(), iters) / iters
    return {"only": which, "ms": ms, "tflops": flops / ms / 1e9, "iters": iters}


def weight_sets(set_bytes, world):
    """Distinct copies of a rank's weight slice used in turn, so that a copy is read again only after more than twice the
    L2's capacity of other weights has streamed through: one when the slice alone is that large, else a multiple of the
    three products of a step."""
    if world == 1 and set_bytes > 1.5 * L2_BYTES:
        return 1
    return len(MS) * max(1, math.ceil(2 * L2_BYTES / (len(MS) * set_bytes)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baselines")
    ap.add_argument("--only", default=None,
                    choices=["fp8", "fp8_big", "dyn4", "dyn4_decode", "int8_large_m", "int8_mid_m", "int8_stack", "bf16_mm", "config1",
                             "int8_slice", "chain_probe", "dyn4_all"],
                    help="run one configuration a few times and exit (for profilers); prints its own JSON line")
    ap.add_argument("--slice-world", type=int, default=8, help="--only int8_slice: the rank count whose weight slice is timed")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch_vulkan_b200 as tv  # raises if the extension is missing: there is no fallback

    if not tv.is_available():
        raise SystemExit("bench.py: no B200 available to torch_vulkan_b200 (and there is no CPU path)")
    torch.cuda.set_device(local_rank)
    tv.set_device(local_rank)
    dev = f"vk:{local_rank}"
    stream = tv.cuda_stream(local_rank)
    timer = Timer(tv, stream, local_rank)
    peaks = measured_peaks()
    if world > 1 or torch.get_num_threads() < 2:
        torch.set_num_threads(max(1, host_threads() // world))  # (torchrun gives every rank one thread; the checks use more)
    if args.only == "dyn4_all":
        res = extra_dyn4(tv, timer, peaks, cpu=False, quick=False)
        print(json.dumps({"only": "dyn4_all", **{k: {a: b for a, b in v.items() if a in ("tops", "ms", "us", "weight_gbs")} for k, v in res.items()}}), flush=True)
        return
    if args.only == "int8_stack":
        print(json.dumps({"only": "int8_stack", **int8_stack(tv, timer, peaks, cpu=False)}), flush=True)
        return
    if args.only is not None:
        print(json.dumps(run_only(tv, timer, args.only, max(args.steps, 1) if args.steps != 200 else 3, args.slice_world)), flush=True)
        return
    from torch_vulkan_b200 import shard

    channel = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # (no device_id: with "vk" registered, torch takes that for the accelerator; a short timeout: a rank that fell out must
        # not hold the others for ten minutes)
        dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=180))
        objects = dist.new_group(backend="gloo")
        if os.environ.get("TVB200_GATHER", "fused") == "fused":
            channel = shard.PeerChannel(local_rank, objects)

    # ---- inputs: this rank's slice of the weight rows (output columns), in `nsets` rotated copies; A replicated
    rows = N_OUT // world
    nsets = weight_sets(rows * K_IN, world)
    a_host, w_full, s_full = make_inputs(N_OUT)
    w_slice, s_slice = w_full[rank * rows:(rank + 1) * rows], s_full[rank * rows:(rank + 1) * rows]
    shift = 16  # copy j holds the slice's rows rolled by 16 j: its output columns are rolled likewise
    w_sets = [torch.roll(w_slice, shift * j, 0).contiguous().to(dev) for j in range(nsets)]
    s_sets = [torch.roll(s_slice, shift * j, 0).contiguous().to(dev) for j in range(nsets)]
    # the step's activations lie one after the other in one device buffer and in one page-locked host buffer (a caller
    # that knows the step's products in advance lays them out so): one copy takes all of them up
    a_all_pinned = torch.cat([a_host[m] for m in MS]).pin_memory()
    a_all_dev = a_all_pinned.to(dev)
    a_dev, row = {}, 0
    for m in MS:
        a_dev[m] = a_all_dev[row:row + m]
        row += m
    mark("expected values on the CPU")
    expected = {m: int8_expected(a_host[m], w_full, s_full) for m in MS}
    mark("inputs ready")

    def check(m, got, j, what):
        """`got` [m, N] against the CPU product for weight copy j (every rank's slice of columns rolled by 16 j)."""
        want, tol = expected[m]
        want = torch.roll(want.view(m, world, rows), shift * j, 2).reshape(m, N_OUT)
        tol = torch.roll(tol.view(m, world, rows), shift * j, 2).reshape(m, N_OUT)
        if not ((got.float() - want.float()).abs() <= tol).all():
            bad = int(((got.float() - want.float()).abs() > tol).sum())
            raise SystemExit(f"bench.py: rank {rank}: {what}: {bad} outputs of the M={m} product outside the reference's bound")

    fused = None
    if channel is not None:
        fused = {m: shard.GatheredOutputs(m, N_OUT, torch.bfloat16, channel) for m in MS}
    plain_out = {m: [torch.empty(m, N_OUT, dtype=torch.bfloat16, device=dev) for _ in range(2)] for m in MS} if world == 1 else None

    def product(m, a, j, buf, pos=None):
        if world == 1:
            return torch._weight_int8pack_mm(a, w_sets[j], s_sets[j])
        if fused is not None:
            # every rank's kernel stores its column slice into every rank's [m, N] buffer (peer stores over NVLink); the
            # three products of a step have nothing to do with each other: none waits for the ones before it in the step
            return fused[m].weight_int8pack_mm(a, w_sets[j], s_sets[j], buf=buf, independent=MS.index(m) if pos is None else pos)
        # every rank's column slice, then the NCCL all-gather into [m, N] (queued on the backend's stream)
        return shard.weight_int8pack_mm(a, w_sets[j], s_sets[j])

    # Step g of a cycle of `ngraphs` uses weight copies 3g .. 3g+2 (mod nsets) and output buffer set g % 2: a buffer is
    # written again only a whole step after the step whose outputs it held.
    ngraphs = 1 if world == 1 else (nsets // len(MS)) * (2 if (nsets // len(MS)) % 2 else 1)

    def step_sets(g):
        return [(len(MS) * g + i) % nsets for i in range(len(MS))]

    def barrier():
        tv.synchronize(local_rank)
        torch.cuda.synchronize()
        if world > 1:
            shard.barrier()

    # Two ways to queue a step. "chain": the three products as one launch of the persistent decode kernel
    # (tvb_qmm8_chain_*), which streams the next product's weights while the current one is finished and, sharded, ends when
    # every rank's columns have arrived. "per_product": one launch per product through aten::_weight_int8pack_mm (sharded:
    # tvb_qmm8_gather, then one wait kernel per step).
    use_chain = os.environ.get("TVB200_CHAIN", "1") != "0" and (world == 1 or fused is not None)
    chains = None
    if use_chain:
        chains = []
        for g in range(ngraphs):
            outs = [plain_out[m][g % 2] if world == 1 else (fused[m], g % 2) for m in MS]
            chains.append(shard.ProductChain([(a_dev[m], w_sets[j], s_sets[j], out, i)
                                              for i, (m, j, out) in enumerate(zip(MS, step_sets(g), outs))], local_rank, channel))

    def step_fn(mode, g):
        if mode == "chain":
            return chains[g].run()
        if mode == "group":
            # the step's three products in ONE launch of the decode kernel (tvb_qmm8_group / tvb_qmm8_group_gather): its
            # (tile, chunk) units run through all three products and are cut into one range per SM
            sets = step_sets(g)
            acts, ws, ss = [a_dev[m] for m in MS], [w_sets[j] for j in sets], [s_sets[j] for j in sets]
            if world == 1:
                return shard.weight_int8pack_mm_group(acts, ws, ss, outs=[plain_out[m][g % 2] for m in MS], device_index=local_rank)
            outs = shard.weight_int8pack_mm_group(acts, ws, ss, outs=[fused[m] for m in MS], bufs=[g % 2] * len(MS))
            channel.wait()
            return outs
        outs = [product(m, a_dev[m], j, g % 2) for m, j in zip(MS, step_sets(g))]
        if channel is not None:
            channel.wait()  # the step ends when every rank holds every column
        return outs

    def time_mode(mode, steps, warmup):
        """Parity before, `steps` timed steps after `warmup`, parity after. Returns (ms of the timed region, replayable steps)."""
        mark(f"{mode}: parity before timing")
        for g in range(ngraphs):
            for m, j, out in zip(MS, step_sets(g), step_fn(mode, g)):
                check(m, out.cpu(), j, f"{mode}, before timing")
        barrier()
        # The step is captured into CUDA graphs and replayed: at 4 and 8 GPUs it is shorter than the host's launch calls.
        graphs = None
        mark(f"{mode}: capture")
        if os.environ.get("TVB200_GRAPH", "1") != "0" and (world == 1 or fused is not None):
            try:
                graphs = [shard.StepGraph(lambda g=g: step_fn(mode, g), local_rank, warm=False) for g in range(ngraphs)]
            except Exception as exc:  # noqa: BLE001
                if rank == 0:
                    print(f"bench.py: graph capture failed ({exc}); launching eagerly", file=sys.stderr)
                try:
                    tv.synchronize(local_rank)
                except Exception:  # noqa: BLE001
                    pass
                graphs = None

        def step(i):
            if graphs is not None:
                graphs[i % ngraphs].replay()
            else:
                step_fn(mode, i % ngraphs)

        mark(f"{mode}: warm-up and timed steps")
        for i in range(warmup):
            step(i)
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(steps):
            step(warmup + i)
        end.record(stream)
        barrier()
        ms = start.elapsed_time(end)
        for g in range(ngraphs):  # what a further run of every recorded step leaves in the output buffers
            if graphs is not None:
                graphs[g].replay()
                outs = graphs[g].outputs
            else:
                outs = step_fn(mode, g)
            tv.synchronize(local_rank)
            for m, j, out in zip(MS, step_sets(g), outs):
                check(m, out.cpu(), j, f"{mode}, after the timed steps")
        barrier()
        return ms, step, graphs is not None

    # ---- device-resident timing
    sampler = ClockSampler(local_rank) if rank == 0 else None
    sampler_t0 = time.perf_counter()
    # both ways of queueing a step are timed; the faster one is the headline (and the end-to-end path), the other is reported
    # beside it. (Every rank must pick the same one: the choice is made on the slowest rank's times.)
    MODES = ("per_product", "group", "chain")
    timed = {"per_product": time_mode("per_product", args.steps, args.warmup)}
    if os.environ.get("TVB200_GROUP", "1") != "0" and (world == 1 or fused is not None):
        timed["group"] = time_mode("group", args.steps, args.warmup)
    if use_chain:
        timed["chain"] = time_mode("chain", args.steps, args.warmup)
    times = torch.tensor([timed[k][0] if k in timed else float("inf") for k in MODES], dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist

        t = times.to(torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.cpu()
    mode = MODES[int(torch.argmin(times))]
    use_chain = mode == "chain"
    total_ms, step_plain, replayed = timed[mode]
    total_ms = float(times[MODES.index(mode)])
    other_ms = {k: float(times[MODES.index(k)]) for k in MODES if k != mode and k in timed}
    STEP_TEXT = {"per_product": "one launch per product (aten::_weight_int8pack_mm)" + (" and a wait kernel" if channel is not None else ""),
                 "group": "one launch of the decode kernel over the step's three products (tvb_qmm8_group" + ("_gather) and a wait kernel" if channel is not None else ")"),
                 "chain": "one launch of the persistent decode kernel over the step's three products (tvb_qmm8_chain_run)"}
    per_step_launches = {"per_product": len(MS) + (1 if channel is not None else 0), "group": 1 + (1 if channel is not None else 0), "chain": 1}[mode]
    launches = args.steps * per_step_launches

    # ---- the decode kernel alone on this rank's slice (no exchange), one launch per product, per M
    mark("isolated launches")
    isolated_ms = {}
    for m in MS:
        reps = 4 * max(nsets, 3)
        g_iso = shard.StepGraph(lambda: [torch._weight_int8pack_mm(a_dev[m], w_sets[i % nsets], s_sets[i % nsets]) for i in range(reps)],
                                local_rank)
        isolated_ms[m] = timer.median(g_iso.replay, 5) / reps
        del g_iso
    barrier()
    # nvidia-smi needs a second or so of load to return samples: when the timed region was shorter than that, the
    # same steps keep running (untimed) until the sampling window is filled
    while world == 1 and time.perf_counter() - sampler_t0 < 1.5:
        for i in range(20):
            step_plain(i)
        barrier()
    # average duration per product over the timed region: the region holds nothing but the steps, queued back to back
    avg_launch_ms = total_ms / (args.steps * len(MS))

    # ---- end to end through the C ABI / the ops: A from pinned host memory, C back to the host, every step
    out_pinned = {m: torch.empty(m, N_OUT, dtype=torch.bfloat16).pin_memory() for m in MS}
    host_gathered = None
    if fused is not None and "group" in timed and os.environ.get("TVB200_HOST_GATHER", "1") != "0":
        try:  # (every rank raises or none does: see HostGathered)
            host_gathered = {m: shard.HostGathered(m, N_OUT, torch.bfloat16, channel) for m in MS}
        except RuntimeError as exc:
            host_gathered = None
            if rank == 0:
                print(f"bench.py: no shared host buffer ({exc}); every rank copies the results down", file=sys.stderr)

    def e2e_body(g, mode):
        # every product's A goes up from page-locked memory (into the buffers the step reads) and its C comes back into
        # page-locked memory
        a_all_dev.copy_(a_all_pinned, non_blocking=True)
        if mode == "group" and world == 1:
            # the grouped launch stores its results straight into the page-locked host buffers: the kernel's stores are
            # the copy down
            sets = step_sets(g)
            return shard.weight_int8pack_mm_group([a_dev[m] for m in MS], [w_sets[j] for j in sets], [s_sets[j] for j in sets],
                                                  outs=[out_pinned[m] for m in MS], device_index=local_rank)
        if mode == "group" and host_gathered is not None:
            # sharded: every rank's kernel also stores its columns into page-locked host memory that all ranks of the node
            # map (one shared segment): the whole result is on the host, once, when every rank's columns have arrived
            sets = step_sets(g)
            outs = shard.weight_int8pack_mm_group([a_dev[m] for m in MS], [w_sets[j] for j in sets], [s_sets[j] for j in sets],
                                                  outs=[fused[m] for m in MS], bufs=[g % 2] * len(MS), host_outs=[host_gathered[m] for m in MS])
            channel.wait()
            return outs
        if mode in ("chain", "group"):
            outs = step_fn(mode, g)
            for m, c in zip(MS, outs):
                out_pinned[m].copy_(c, non_blocking=True)
            return outs
        # one launch per product: each result leaves on the runtime's second stream as soon as it is complete, under the
        # products that follow (largest first, so that the copy left over at the end of the step is the smallest)
        sets = dict(zip(MS, step_sets(g)))
        outs = {}
        for pos, m in enumerate(sorted(MS, reverse=True)):
            c = product(m, a_dev[m], sets[m], g % 2, pos)
            if channel is not None:
                channel.wait()  # every rank's columns of this product have arrived
            tv.copy_to_host_overlapped(out_pinned[m], c)
            outs[m] = c
        return [outs[m] for m in MS]

    e2e_steps = max(5, min(args.steps, 30))

    def time_e2e(step):
        for i in range(3):
            step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            step(3 + i)
        barrier()
        return (time.perf_counter() - t0) / e2e_steps

    # End to end the step is timed both with one launch per product (each result leaves under the following products) and,
    # where the device-resident headline is another way of queueing it, that way too; the faster is reported.
    e2e_modes = ["per_product"] + ([mode] if mode != "per_product" else [])
    e2e_s = e2e_eager_s = float("inf")
    e2e_how = e2e_mode = None
    last_g = (3 + e2e_steps - 1) % ngraphs
    for em in e2e_modes:
        def step_e2e_eager(i, em=em):
            e2e_body(i % ngraphs, em)
            tv.synchronize(local_rank)  # the step ends when all three results are on the host

        mark(f"end to end, eager, {em}")
        eager_s = time_e2e(step_e2e_eager)
        best_s, how = eager_s, "eager: every copy and product queued by its own call"
        if replayed:
            # the same copies and products recorded once per buffer set (the host buffers are fixed; a caller rewrites A in place)
            mark(f"end to end, replayed, {em}")
            e2e_graphs = [shard.StepGraph(lambda g=g, em=em: e2e_body(g, em), local_rank, warm=False) for g in range(ngraphs)]

            def step_e2e_graph(i, graphs=e2e_graphs):
                graphs[i % ngraphs].replay()
                tv.synchronize(local_rank)

            best_s = time_e2e(step_e2e_graph)
            how = ("CUDA graph replay of the step's copies and products" +
                   (" (results copied out beside the following products)" if em == "per_product" else
                    " (the kernel stores its results into the page-locked host buffers)" if em == "group" and world == 1 else
                    " (every rank's kernel stores its columns into one page-locked host buffer that all ranks map)" if em == "group" and host_gathered is not None else "") +
                   ", then a stream synchronize")
            del e2e_graphs
        if world > 1:
            shard.barrier()  # (a shared host buffer is complete for everyone when every rank's step has ended)
        for m, j in zip(MS, step_sets(last_g)):  # what came back to the host from the last end-to-end step
            on_host = host_gathered[m].tensors[last_g % 2] if em == "group" and host_gathered is not None else out_pinned[m]
            check(m, on_host, j, f"end-to-end outputs on the host ({em})")
        if world > 1:  # (every rank must pick the same way: the slowest rank's times decide)
            import torch.distributed as dist

            t = torch.tensor([best_s, eager_s], dtype=torch.float64, device=torch.device("cuda", local_rank))
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            best_s, eager_s = t.tolist()
        if best_s < e2e_s:
            e2e_s, e2e_eager_s, e2e_how, e2e_mode = best_s, eager_s, how + "; " + STEP_TEXT[em], em

    # ---- max over ranks
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([e2e_s, e2e_eager_s] + [isolated_ms[m] for m in MS], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_eager_s, *iso = t.tolist()
        isolated_ms = dict(zip(MS, iso))

    # ---- the other configurations (every rank takes part in the sharded ones)
    extra = {}
    mark("other configurations")
    if not args.no_extra:
        del w_sets, s_sets
        tv.empty_cache()
        cpu = not args.no_cpu and rank == 0
        if world == 1:
            extra.update(extra_config1(tv, timer, peaks, cpu))
            extra.update(extra_fp8(tv, timer, peaks, cpu, quick=False))
            extra.update(extra_mm(tv, timer, peaks, quick=False))
            extra.update(extra_dyn4(tv, timer, peaks, cpu, quick=False))
            extra.update(int8_stack(tv, timer, peaks, cpu))
        else:
            if channel is not None:
                extra.update(int8_stack_sharded(tv, timer, peaks, channel, rank, world, dev))
            extra.update(fp8_sharded(tv, timer, peaks, channel, rank, world, dev))
    clocks = sampler.stop() if sampler is not None else None
    if clocks is not None:
        clocks["window"] = "warm-up, timed region, per-launch pass, end-to-end steps and the other configurations"

    if rank == 0:
        step_bytes = sum(algorithmic_bytes(m, N_OUT, K_IN) for m in MS)  # whole job, all ranks
        ms_per_step = total_ms / args.steps
        value = step_bytes / (ms_per_step * 1e-3) / 1e9
        launch_bytes = statistics.mean(algorithmic_bytes(m, rows, K_IN) for m in MS)  # one launch, this rank's slice
        achieved = launch_bytes / (avg_launch_ms * 1e-3) / 1e9
        iso_mean = statistics.mean(isolated_ms.values())
        streams = "each launch streams %.0f MB of weights" % (rows * K_IN / 1e6)
        l2_note = ("no flush: " + streams + ", larger than the 126 MB L2") if nsets == 1 else \
            ("no flush: %d distinct copies of the rank's weight slice are used in turn (%.0f MB, twice the 126 MB L2, between two "
             "uses of a copy): %s from HBM" % (nsets, nsets * rows * K_IN / 1e6, streams))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE_NOTE, "data": "synthetic", "config": {"workload": WORKLOAD},
            "details": {"sharding": f"weight rows / {world}" + ((" + fused peer-store gather of C (arrival counted per CTA and source rank)" if fused is not None else " + NCCL all-gather of C") if world > 1 else ""),
                        "l2": l2_note, "weight_copies_per_rank": nsets, "launches_per_step": per_step_launches,
                        "step": STEP_TEXT[mode],
                        "launch": f"CUDA graph replay, {ngraphs} recorded step(s) in turn" if replayed else "eager",
                        "parity": "every rank's assembled outputs checked against the CPU product (the reference's bound) for every weight "
                                  "copy before timing, after the timed replays and after the end-to-end steps"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "kernel": "qmm8_chain_kernel" if use_chain else "qmm8_skinny_kernel", "avg_launch_us": avg_launch_ms * 1e3,
                         "avg_launch_how": "timed region / products (steps queued back to back, as in decoding; a launch that holds a "
                                           "step's three products takes three times this and moves three times the bytes; with "
                                           "sharding the region includes the exchange)",
                         "isolated_launch_us_by_m": {str(m): isolated_ms[m] * 1e3 for m in MS},
                         "isolated_how": "the kernel alone on this rank's weight slice (no exchange), a replayed graph of launches over "
                                         "the weight copies in turn",
                         "isolated_frac": launch_bytes / (iso_mean * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "e2e": {"value": step_bytes / e2e_s / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": sum(2 * m * K_IN for m in MS), "d2h_bytes_per_step": sum(2 * m * N_OUT for m in MS),
                    "d2h_how": ("every rank stores its own columns into one host buffer shared by the node's ranks: the figure is the whole node's"
                                if e2e_mode == "group" and host_gathered is not None else "every rank brings the whole result down"),
                    "ms_per_step": e2e_s * 1e3, "how": e2e_how, "eager_value": step_bytes / e2e_eager_s / 1e9},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        line["details"]["other_ways"] = [{"step": STEP_TEXT[k], "value": step_bytes / (v / args.steps * 1e-3) / 1e9, "ms_per_step": v / args.steps}
                                         for k, v in other_ms.items()]
        if world > 1:
            line["roofline"]["exchange_us_per_product"] = (avg_launch_ms - iso_mean) * 1e3
        if world == 1:
            traffic = profiled_traffic(grouped=mode == "group")
            line["roofline"]["traffic"] = traffic
            line["roofline"]["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum per launch (" +
                                                  ("a grouped launch holds the step's three products: compare with three times the bytes of a product" if mode == "group"
                                                   else "mean of the M = 1, 4, 16 launches") + "), read from profiles/qmm8_skinny_config2.md")
            line["roofline"]["bytes_per_launch"] = step_bytes if mode != "per_product" else step_bytes / len(MS)
            line["roofline"]["launch_us"] = avg_launch_ms * 1e3 * (len(MS) if mode != "per_product" else 1)
        if not args.no_cpu and world == 1:
            if torch.get_num_threads() < host_threads():
                torch.set_num_threads(host_threads())

            def cpu_step():
                for m in MS:
                    torch._weight_int8pack_mm(a_host[m], w_full, s_full)

            cpu_s, reps = cpu_time(cpu_step, 8.0)
            line["cpu_baseline"] = {"value": step_bytes / cpu_s / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
                                    "kind": "reference",
                                    "sample": f"{reps} full steps (median): torch._weight_int8pack_mm on CPU tensors, the kernel "
                                              "the reference hands this op to without a GPU and checks its shader against",
                                    "ms_per_step": cpu_s * 1e3}
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        shard.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
