"""Benchmark of the quantised matrix-product path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extra]

Headline workload (`config.workload`): the decode configuration of the int8
weight-only product, `aten::_weight_int8pack_mm` with bf16 A[M, 8192] for M in
{1, 4, 16} against int8 W[28672, 8192] and bf16 per-channel scales. One step is
the three products (one per M). The metric is weight-streaming bandwidth: the
algorithmic bytes of the three launches (weights + scales + A + C) per second.
With N GPUs the weight rows (output columns) are sharded N ways, every rank runs
its slice and the outputs are assembled with an NCCL all-gather (strong scaling).

One JSON line is printed by rank 0. `value` is timed on the device with the
inputs resident in HBM; `e2e` runs the same step through the public API from
pinned host memory (copy of A up, copy of C down, every call); `roofline` is the
decode kernel against the measured HBM copy bandwidth; `cpu_baseline` is
PyTorch's CPU kernel for the same op (the kernel the reference falls back to and
is validated against) timed on this host's cores; `extra` holds the large-m
configurations (dyn-int4 and float8) in TFLOP/s.

`--impl reference` times that CPU kernel alone, on the same workload and metric.
"""

import argparse
import json
import os
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


NCU_DRAM_BYTES_PER_LAUNCH = 241.64e6  # one decode launch of this workload on one GPU, from the committed ncu capture


def algorithmic_bytes(m, n, k):
    """Weights + scales + A + C of one product (bf16 activations, int8 weights)."""
    return n * k + 2 * n + 2 * m * k + 2 * m * n


def gen(seed):
    return torch.Generator().manual_seed(seed)


def make_inputs(n_rows, rank_seed=0):
    w = torch.randint(-127, 128, (n_rows, K_IN), dtype=torch.int8, generator=gen(2 + rank_seed))
    s = (torch.rand(n_rows, generator=gen(3 + rank_seed)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16)
    a = {m: torch.randn(m, K_IN, generator=gen(1 + m)).to(torch.bfloat16) for m in MS}
    return a, w, s


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


def cpu_reference_time(a, w, s, budget_s):
    """Seconds per step of PyTorch's CPU _weight_int8pack_mm on the full workload (all host threads)."""
    for m in MS:
        torch._weight_int8pack_mm(a[m], w, s)  # warm call
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        for m in MS:
            torch._weight_int8pack_mm(a[m], w, s)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def run_reference(args, rank):
    """The reference arm: the CPU kernel the reference falls back to (crates/pyvk/csrc/quant.cpp:77), all host threads."""
    if rank != 0:
        return
    # torchrun gives every rank OMP_NUM_THREADS=1; this arm is rank 0 alone and takes the host's cores
    host_threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < host_threads:
        torch.set_num_threads(host_threads)
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
        "dtype": "bf16 activations, int8 weights, float32 accumulation", "data": "synthetic",
        "config": {"workload": WORKLOAD, "device": "host CPU", "torch": torch.__version__, "os_cpu_count": os.cpu_count()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": "the full workload, every step: torch._weight_int8pack_mm on CPU tensors, the kernel the "
                                   "reference hands this op to without a GPU and checks its shader against"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_steps(fn, steps, stream):
    """Runs fn(step) `steps` times between two events on `stream`; returns the events."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for i in range(steps):
        fn(i)
    end.record(stream)
    return start, end


def extra_configs(tv, stream, peaks, quick):
    """Large-m configurations, one GPU: float8 _scaled_mm 8192^3 and dyn-int4 [M,4096]x[14336,4096]."""
    out = {}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        tv.synchronize()
        evs = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            fn()
            e.record(stream)
            evs.append((s, e))
        tv.synchronize()
        return statistics.median(s.elapsed_time(e) for s, e in evs)

    m = n = k = 8192
    for rowwise in (False, True):
        a, b, sa, sb = config_fp8(m, k, n, rowwise)
        av, bv, sav, sbv = a.to("vk"), b.t().to("vk").t(), sa.to("vk"), sb.to("vk")
        ms = timed(lambda: torch._scaled_mm(av, bv, sav, sbv, out_dtype=torch.bfloat16), 5 if quick else 10)
        tf = 2.0 * m * n * k / ms / 1e9
        out["fp8_scaled_mm_8192_" + ("rowwise" if rowwise else "tensorwise")] = {
            "tflops": tf, "ms": ms, "frac_of_2x_measured_bf16": tf / (2 * peaks["bf16_tflops"]), "frac_of_nominal_fp8": tf / 4500.0}
        del av, bv
    # the unquantised product on the same main loop (aten::mm, bfloat16), against the library GEMM the peak was measured with
    a16 = torch.randn(m, k, generator=gen(21)).to(torch.bfloat16).to("vk")
    w16 = torch.randn(n, k, generator=gen(22)).to(torch.bfloat16).to("vk")
    ms = timed(lambda: torch.mm(a16, w16.t()), 5 if quick else 10)
    tf = 2.0 * m * n * k / ms / 1e9
    out["bf16_mm_8192"] = {"tflops": tf, "ms": ms, "frac_of_measured_bf16": tf / peaks["bf16_tflops"]}
    del a16, w16
    # int8 weight-only at prefill sizes (weights widened once per call into scratch, then the same 16-bit main loop)
    for mm, nn_, kk in ((2048, 14336, 4096),) if quick else ((2048, 14336, 4096), (8192, 8192, 8192)):
        a8 = torch.randn(mm, kk, generator=gen(31)).to(torch.bfloat16).to("vk")
        w8 = torch.randint(-127, 128, (nn_, kk), dtype=torch.int8, generator=gen(32)).to("vk")
        s8 = (torch.rand(nn_, generator=gen(33)) * (2e-2 - 1e-3) + 1e-3).to(torch.bfloat16).to("vk")
        ms = timed(lambda: torch._weight_int8pack_mm(a8, w8, s8), 5)
        tf = 2.0 * mm * nn_ * kk / ms / 1e9
        out[f"int8_weight_only_m{mm}_n{nn_}_k{kk}"] = {"tflops": tf, "ms": ms, "frac_of_measured_bf16": tf / peaks["bf16_tflops"]}
        del a8, w8, s8
    w, sc, bias = config_dyn4_weights()
    packed = torch._dyn_quant_pack_4bit_weight(w.to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
    for mm in ((128,) if quick else (128, 512, 2048)):
        xv = torch.randn(mm, 4096, generator=gen(11)).to("vk")
        for mode in ("exact", "fast"):  # exact: bit for bit (the default); fast: TORCH_VK_QMM4=fast, rtol 1e-5
            if mode == "fast":
                os.environ["TORCH_VK_QMM4"] = "fast"
            ms = timed(lambda: torch._dyn_quant_matmul_4bit(xv, packed, 32, 4096, 14336), 3)
            os.environ.pop("TORCH_VK_QMM4", None)
            tops = 2.0 * mm * 14336 * 4096 / ms / 1e9
            out[f"dyn_int4_m{mm}_{mode}"] = {"tops": tops, "ms": ms, "frac_of_2x_measured_bf16": tops / (2 * peaks["bf16_tflops"])}
    # dyn-int4 decoding (at most 16 rows): twelve products replayed as one graph, against the bytes of the real int4 data
    # (29.36 MB of nibbles + 3.67 MB of block scales + bias, activations and outputs)
    from torch_vulkan_b200 import shard

    packs = [packed] + [torch._dyn_quant_pack_4bit_weight(torch.roll(w, i, 0).to("vk"), sc.to("vk"), bias.to("vk"), 32, 4096, 14336)
                        for i in (1, 2, 3)]  # four weight sets in turn: 147 MB in their decode form, more than the L2 holds
    for mm in (1, 16):
        xv = torch.randn(mm, 4096, generator=gen(12)).to("vk")
        graph = shard.StepGraph(lambda: [torch._dyn_quant_matmul_4bit(xv, packs[i % 4], 32, 4096, 14336) for i in range(12)])
        ms = timed(graph.replay, 5) / 12
        nbytes = 14336 * 4096 // 2 + 14336 * 128 * 2 + 14336 * 4 + mm * 4096 * 4 + mm * 14336 * 4
        out[f"dyn_int4_decode_m{mm}"] = {"us": ms * 1e3, "weight_gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
        del graph
    del packs
    tv.empty_cache()
    if not quick:
        out.update(int8_stack(tv, stream))
    return out


def int8_stack(tv, stream, layers=32):
    """The int8 weight-only Linears of a 32-layer decoder (hidden 4096: qkv 6144, o 4096, gate_up 28672, down from 14336;
    7 GB of weights, every layer its own buffers), decoded as one replayed graph of 128 products per step. Between the
    products stands the stack's glue only (the first 4096 columns of qkv feed o, the first 14336 of gate_up feed down)."""
    from torch_vulkan_b200 import shard

    shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
    host = []
    for i, (n, k) in enumerate(shapes):
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen(40 + i))
        sc = (torch.rand(n, generator=gen(50 + i)) * 2e-3 + 1e-4).to(torch.bfloat16)
        host.append((w, sc))
    weights = [[(w.to("vk"), sc.to("vk")) for w, sc in host] for _ in range(layers)]
    wbytes = layers * sum(n * k for n, k in shapes)
    out = {}
    for m in (1, 16):
        x = torch.randn(m, 4096, generator=gen(60)).to(torch.bfloat16).to("vk")

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
        tv.synchronize()
        iters = 20
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in range(iters):
            graph.replay()
        e0.record(stream)
        tv.synchronize()
        ms = s0.elapsed_time(e0) / iters
        out[f"int8_stack_32layers_m{m}"] = {"ms_per_token_step": ms, "weight_gbs": wbytes / ms / 1e6, "products": 4 * layers,
                                             "weight_bytes": wbytes}
        del graph

        # The same stack with its two residual additions (after o and after down): in the decode kernel's epilogue
        # (tvb_qmm8_linear, 128 launches per step) against a product and an add each (192 launches).
        def step_residual(fused):
            from torch_vulkan_b200 import _native

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
            tv.synchronize()
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            for _ in range(iters):
                graph.replay()
            e0.record(stream)
            tv.synchronize()
            out[f"int8_stack_32layers_m{m}"][label + "_ms"] = s0.elapsed_time(e0) / iters
            del graph
    del weights
    tv.empty_cache()
    return out


def run_only(tv, stream, which, iters):
    """One large-m configuration, `iters` launches after one warm-up (small enough to sit under a profiler)."""
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
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for _ in range(iters):
        fn()
    e0.record(stream)
    tv.synchronize()
    ms = s0.elapsed_time(e0) / iters
    return {"only": which, "ms": ms, "tflops": flops / ms / 1e9, "iters": iters}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the large-m configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--only", default=None, choices=["fp8", "fp8_big", "dyn4", "dyn4_decode", "int8_large_m", "int8_mid_m", "int8_stack", "bf16_mm"],
                    help="run one large-m configuration a few times and exit (for profilers); prints its own JSON line")
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
    if args.only == "int8_stack":
        print(json.dumps({"only": "int8_stack", **int8_stack(tv, stream)}), flush=True)
        return
    if args.only is not None:
        print(json.dumps(run_only(tv, stream, args.only, max(args.steps, 1) if args.steps != 200 else 3)), flush=True)
        return
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")  # (no device_id: with "vk" registered, torch takes that for the accelerator)
    peaks = measured_peaks()

    # ---- inputs: this rank's slice of the weight rows (output columns); A replicated
    rows = N_OUT // world
    a_host, w_full, s_full = make_inputs(N_OUT)
    w = w_full[rank * rows:(rank + 1) * rows].contiguous().to(dev)
    s = s_full[rank * rows:(rank + 1) * rows].contiguous().to(dev)
    a_dev = {m: a_host[m].to(dev) for m in MS}
    a_pinned = {m: a_host[m].pin_memory() for m in MS}
    from torch_vulkan_b200 import shard

    fused = None
    if world > 1 and os.environ.get("TVB200_GATHER", "fused") == "fused":
        import torch.distributed as dist

        objects = dist.new_group(backend="gloo")
        fused = {m: shard.GatheredOutputs(m, N_OUT, torch.bfloat16, local_rank, objects) for m in MS}

    def product(m, a):
        if world == 1:
            return torch._weight_int8pack_mm(a, w, s)
        if fused is not None:
            # every rank's kernel stores its column slice into every rank's [m, N] buffer (peer stores over NVLink)
            return fused[m].weight_int8pack_mm(a, w, s)
        # every rank's column slice, then the NCCL all-gather into [m, N] (queued on the backend's stream)
        return shard.weight_int8pack_mm(a, w, s)

    def step_eager():
        return [product(m, a_dev[m]) for m in MS]

    # The step (three short kernels, plus the flag waits when sharded) is captured once into a CUDA graph and replayed:
    # at 4 and 8 GPUs the kernels are shorter than the host's launch calls.
    graph = None
    if os.environ.get("TVB200_GRAPH", "1") != "0":
        try:
            graph = shard.StepGraph(step_eager, local_rank)
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(f"bench.py: graph capture failed ({exc}); launching eagerly", file=sys.stderr)
            graph = None

    def step_plain(i):
        if graph is not None:
            graph.replay()
        else:
            step_eager()

    def barrier():
        tv.synchronize(local_rank)
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist

            shard.barrier()

    # ---- device-resident timing
    sampler = ClockSampler(local_rank) if rank == 0 else None
    sampler_t0 = time.perf_counter()
    for i in range(args.warmup):
        step_plain(i)
    barrier()
    launches_before = tv.dispatch_count()
    start, end = time_steps(step_plain, args.steps, stream)
    barrier()
    launches = tv.dispatch_count() - launches_before
    if graph is not None:
        launches = args.steps * len(MS) * (2 if fused is not None else 1)  # replayed kernels are not re-counted by the runtime
    total_ms = start.elapsed_time(end)

    # ---- per-launch duration of the decode kernel (the roofline's numerator), same loop with an event pair per launch
    pairs = []
    for i in range(args.steps):
        for m in MS:
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            torch._weight_int8pack_mm(a_dev[m], w, s)
            e0.record(stream)
            pairs.append((m, s0, e0))
    barrier()
    # nvidia-smi needs a second or so of load to return samples: when the timed region was shorter than that, the
    # same steps keep running (untimed) until the sampling window is filled
    while world == 1 and time.perf_counter() - sampler_t0 < 1.5:
        for i in range(20):
            step_plain(i)
        barrier()
    clocks = sampler.stop() if sampler is not None else None
    if clocks is not None:
        clocks["window"] = "warm-up, timed region and per-launch pass, plus identical untimed steps up to 1.5 s"
    isolated_ms = {m: statistics.median(s0.elapsed_time(e0) for mm, s0, e0 in pairs if mm == m) for m in MS}
    # average launch duration over the timed region: the region holds nothing but these launches, queued back to back
    avg_launch_ms = total_ms / (args.steps * len(MS)) if world == 1 else statistics.mean(isolated_ms.values())

    # ---- end to end through the public API: A from pinned host memory, C back to the host, every call
    out_pinned = {m: torch.empty(m, N_OUT, dtype=torch.bfloat16).pin_memory() for m in MS}

    def e2e_body():
        # every product's A goes up from page-locked memory and its C comes back into page-locked memory; the three
        # products of a step are queued back to back
        ups = [a_pinned[m].to(dev, non_blocking=True) for m in MS]
        outs = [product(m, a) for m, a in zip(MS, ups)]
        for m, c in zip(MS, outs):
            out_pinned[m].copy_(c, non_blocking=True)
        return ups, outs

    def time_e2e(step):
        for _ in range(3):
            step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step()
        barrier()
        return (time.perf_counter() - t0) / e2e_steps

    def step_e2e_eager():
        e2e_body()
        tv.synchronize(local_rank)  # the step ends when all three results are on the host

    e2e_steps = max(5, min(args.steps, 30))
    e2e_eager_s = time_e2e(step_e2e_eager)
    e2e_s, e2e_how = e2e_eager_s, "eager: every copy and product queued by its own call"
    if graph is not None:
        # the same copies and products recorded once (the host buffers are fixed; a caller rewrites A in place) and replayed
        e2e_graph = shard.StepGraph(e2e_body, local_rank)

        def step_e2e_graph():
            e2e_graph.replay()
            tv.synchronize(local_rank)

        e2e_s, e2e_how = time_e2e(step_e2e_graph), "CUDA graph replay of the step's copies and products, then a stream synchronize"
        for m in MS:  # what came back through the replayed copies is what the eager calls deliver
            want = product(m, a_dev[m]).cpu() if world == 1 else None
            if want is not None and not torch.equal(want.view(torch.int16), out_pinned[m].view(torch.int16)):
                raise SystemExit("bench.py: the replayed end-to-end step returned different results")

    # ---- max over ranks
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([total_ms, e2e_s, avg_launch_ms, e2e_eager_s], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_s, avg_launch_ms, e2e_eager_s = t.tolist()

    if rank == 0:
        step_bytes = sum(algorithmic_bytes(m, N_OUT, K_IN) for m in MS)  # whole job, all ranks
        ms_per_step = total_ms / args.steps
        value = step_bytes / (ms_per_step * 1e-3) / 1e9
        launch_bytes = statistics.mean(algorithmic_bytes(m, rows, K_IN) for m in MS)  # one launch, this rank's slice
        achieved = launch_bytes / (avg_launch_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 activations, int8 weights, float32 accumulation", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": f"weight rows / {world}" + ((" + fused peer-store gather of C" if fused is not None else " + NCCL all-gather of C") if world > 1 else ""),
                       "l2": "no flush: each launch streams %.0f MB of weights, larger than the 126 MB L2" % (rows * K_IN / 1e6)
                       if rows * K_IN > 126e6 else "weight slice of %.0f MB fits the 126 MB L2: launches after the first read it from L2" % (rows * K_IN / 1e6),
                       "launches_per_step": len(MS), "launch": "CUDA graph replay of one step" if graph is not None else "eager"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "kernel": "qmm8_skinny_kernel", "avg_launch_us": avg_launch_ms * 1e3,
                         "avg_launch_how": "timed region / launches (launches queued back to back, as in decoding)",
                         "isolated_launch_us_by_m": {str(m): isolated_ms[m] * 1e3 for m in MS}},
            "e2e": {"value": step_bytes / e2e_s / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": sum(2 * m * K_IN for m in MS), "d2h_bytes_per_step": sum(2 * m * N_OUT for m in MS),
                    "ms_per_step": e2e_s * 1e3, "how": e2e_how, "eager_value": step_bytes / e2e_eager_s / 1e9},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world == 1:
            line["roofline"]["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH
            line["roofline"]["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean of the M = 1, 4, 16 launches (profiles/qmm8_skinny_config2.md)"
        if not args.no_cpu and world == 1:
            cpu_s, reps = cpu_reference_time(a_host, w_full, s_full, 8.0)
            line["cpu_baseline"] = {"value": step_bytes / cpu_s / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
                                    "kind": "reference",
                                    "sample": f"{reps} full steps (median): torch._weight_int8pack_mm on CPU tensors, the kernel "
                                              "the reference hands this op to without a GPU and checks its shader against",
                                    "ms_per_step": cpu_s * 1e3}
        if not args.no_extra and world == 1:
            del w_full
            line["extra"] = extra_configs(tv, stream, peaks, quick=False)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        shard.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
