#!/usr/bin/env python
"""Benchmark of the Linear-DiT block hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload stack|seqpar|nvfp4|dit]

Default workload ("stack"): the Sana-1.6B transformer stack - 20 SanaMSBlocks, hidden 2240,
70 linear-attention heads x 32, FFN hidden 5600, bf16, 128x128 latent grid = 16 384 tokens,
300 text tokens - at global batch 8, batch-data-parallel over N GPUs (8/N images per GPU, no
collective in the forward; "strong" scaling).  One step = one forward of the stack over this
rank's images.  value = block-tokens/s of the whole job = 8 * 16384 * 20 / step time.

"dit": the same stack inside the whole DiT forward (latents in, latents out: patch embedding,
embedders, final layer, unpatchify), same unit.  "nvfp4": one block with FP4 projections.

"seqpar": one block on a 21x45x80 = 75 600-token grid, rows sharded over the N GPUs
(linear-attention state all-reduce + one-row conv halos); value = tokens/s of the block.
The default line carries the same measurement as the sub-record "seqpar" at every N (graph
replay and eager launches, the NCCL exchanges beside the fused peer-memory ones, a per-kernel
breakdown, and the error of this rank's rows against the unsharded block run on the same GPU).

Timing: W >= 3 warm-up steps, then K steps between barrier + synchronize, CUDA events on the
compute stream, max over ranks.  Every step reads > 3 GB of weights and activations (inputs
larger than the 126 MB L2), so no explicit L2 flush is needed.

--impl reference times the CPU restatement of upstream's block (oracle/) on the host cores
(upstream is pure PyTorch; its own modules cannot travel to a box without a checkout, the
restatement is pinned bit-for-bit to them by the golden fixtures).  Both arms also report
"gpu_eager_baseline": the same restatement - plain torch ops, i.e. cuBLAS / cuDNN kernels - run
on the GPU in bf16 on one block of 16 384 tokens, outside every timed region of the product.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "Linear-DiT block tokens/s, Sana-1.6B width, 16K tokens"
UNIT = "block-tokens/s"
C, HEADS, HID, DEPTH, GRID, TEXT = 2240, 20, 5600, 20, (128, 128), 300
GLOBAL_BATCH = 8
SEQPAR_GRID = (21, 45, 80)

# dram__bytes_read.sum + dram__bytes_write.sum of the tensor-core GEMM, averaged over the seven
# launches of one block at batch 1 (one ncu capture: 1.958 GB / 7).  The bench's launches carry
# `per-GPU batch` times the rows, and activations dominate the bytes, so the figure is scaled by
# the per-GPU batch.  A profiler figure cannot be taken inside a timed run; "traffic_algorithmic"
# next to it is computed from the shapes of the launches this run timed.
NCU_TRAFFIC_BYTES_PER_LAUNCH_BATCH1 = 279.7e6


def block_roofline_seconds(T: int, B: int, peaks: dict, C: int = C) -> float:
    """Serial sum of per-kernel bounds for one block: tensor time of the GEMM FLOPs plus HBM
    time of the bandwidth-bound kernels (linear-attention core 4*T*C*e + depthwise-GLU 3*T*hid*e)."""
    f_gemm = 27.0 * T * C * C + 4.0 * B * TEXT * C * C + 4.0 * T * TEXT * C
    bytes_bw = 11.5 * T * C * 2
    return f_gemm / (peaks["tflops"] * 1e12) + bytes_bw / (peaks["hbm_gbs"] * 1e9)


def load_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "tflops_burst": float(d["bf16_tflops"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period: float = 0.05):
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake": 0x80, "sync_boost": 0x10}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                r = get(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_block_tokens_per_s(tokens_grid=(32, 32), budget_s: float = 12.0, max_runs: int = 20):
    """Times the oracle's SanaMSBlock forward (fp32, all host threads) on a bounded sample."""
    from oracle import sana_oracle as O
    from sana_b200 import synthetic

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    shp = synthetic.BlockShape("cpu", C, HEADS, 1, tuple(tokens_grid))
    params = synthetic.make_block_params(C, HID, seed=0)
    x, y, t = synthetic.make_block_inputs(shp, seed=0)
    with torch.no_grad():
        O.sana_ms_block_forward(x, y, t, params, HEADS, shp.grid)  # warm-up
        times = []
        t_begin = time.perf_counter()
        while len(times) < max_runs and (time.perf_counter() - t_begin < budget_s or len(times) < 2):
            t0 = time.perf_counter()
            O.sana_ms_block_forward(x, y, t, params, HEADS, shp.grid)
            times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return shp.tokens / med, threads, f"1 block, fp32, {shp.tokens} tokens ({tokens_grid[0]}x{tokens_grid[1]} grid) at 1.6B width, median of {len(times)} runs"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import sana_oracle as O
    from sana_b200 import synthetic

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    grid = (64, 64)  # 4096 tokens per step: a bounded sample of the 16 384-token workload
    shp = synthetic.BlockShape("cpu", C, HEADS, 1, grid)
    params = synthetic.make_block_params(C, HID, seed=0)
    x, y, t = synthetic.make_block_inputs(shp, seed=0)
    with torch.no_grad():
        for _ in range(max(1, min(args.warmup, 2))):
            O.sana_ms_block_forward(x, y, t, params, HEADS, grid)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            O.sana_ms_block_forward(x, y, t, params, HEADS, grid)
        dt = time.perf_counter() - t0
    val = shp.tokens * args.steps / dt
    sample = f"1 block x {shp.tokens} tokens (64x64 grid) per step, fp32, CPU restatement of upstream's block"
    gpu_eager = None
    if torch.cuda.is_available():  # the practical bar, reported beside the CPU figure (not the arm's value)
        torch.cuda.set_device(0)
        gpu_eager = gpu_eager_block_tokens_per_s(torch.device("cuda", 0))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg3: Sana-1.6B stack (20 blocks, hidden 2240, 16384 tokens, batch 8)", "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_eager_baseline": gpu_eager,
    }))


def fp4_library_rate(M: int, N: int, K: int, iters: int = 20) -> dict:
    """The measured FP4 peak: torch._scaled_mm on float4_e2m1fn_x2 operands with E4M3 scales per 16
    elements (the vendor library's block-scaled FP4 GEMM), same shape, random codes and scales.  Reported
    beside our kernels as the denominator of their roofline; never on the product's path."""
    if not hasattr(torch, "float4_e2m1fn_x2"):
        return {"fp4_library": "unavailable: this torch has no float4_e2m1fn_x2"}
    dev = torch.device("cuda", 0)
    try:
        a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
        sf = lambda rows: (torch.rand(((rows + 127) // 128) * (((K // 16) + 3) // 4) * 512, device=dev) * 2).to(  # noqa: E731
            torch.float8_e4m3fn)
        sa, sb = sf(M), sf(N)
        fn = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)  # noqa: E731
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        return {"fp4_library_ms": ms, "fp4_library_tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    except Exception as e:  # noqa: BLE001 - the probe must not take the measurement down
        return {"fp4_library": f"unavailable: {type(e).__name__}: {str(e)[:160]}"}


def run_gemm_rates(tokens: int, iters: int = 20) -> None:
    """Device-timed rate of each projection shape of a 1.6B-width block, bf16 and NVFP4
    (one JSON line; quantisation of the operands is outside the timed region)."""
    from sana_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(0)
    shapes = [("qkv", 3 * C, C), ("proj", C, C), ("expand", 2 * HID, C), ("point", C, HID)]
    out = {"workload": f"projection rates, {tokens} tokens, hidden {C}", "rows": []}
    for name, n, k in shapes:
        a = torch.randn(tokens, k, generator=g, device=dev).bfloat16()
        w = (torch.randn(n, k, generator=g, device=dev) * 0.02).bfloat16()
        qa, qw = ops.nvfp4_quantize(a), ops.nvfp4_quantize(w)
        o = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
        row = {"name": name, "M": tokens, "N": n, "K": k}
        for kind, variant, fn in (("bf16_1cta", 1, lambda: ops.gemm(a, w, out=o)),
                                  ("bf16_2cta", 2, lambda: ops.gemm(a, w, out=o)),
                                  ("nvfp4_1cta", 1, lambda: ops.gemm_nvfp4(qa, qw, out=o)),
                                  ("nvfp4_2cta", 2, lambda: ops.gemm_nvfp4(qa, qw, out=o))):
            ops.set_gemm_variant(variant)
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            row[kind + "_ms"] = ms
            row[kind + "_tflops"] = 2.0 * tokens * n * k / (ms * 1e-3) / 1e12
        ops.set_gemm_variant(0)
        # the vendor library on the same operands (torch.matmul = cuBLASLt), for comparison only
        wt = w.t()
        for _ in range(3):
            torch.matmul(a, wt, out=o)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            torch.matmul(a, wt, out=o)
        e1.record()
        torch.cuda.synchronize()
        row["bf16_library_ms"] = e0.elapsed_time(e1) / iters
        row["bf16_library_tflops"] = 2.0 * tokens * n * k / (row["bf16_library_ms"] * 1e-3) / 1e12
        row.update(fp4_library_rate(tokens, n, k, iters))
        out["rows"].append(row)
    print(json.dumps(out))


def run_gemm_sustained(tokens: int, seconds: float = 2.0) -> None:
    """The bf16 projections of a block run back to back for `seconds` each way - our kernels, then the vendor
    library (torch.matmul) on the same operands - so that both are measured under the power cap, the regime of
    the stack (one JSON line).  Epilogues: plain for the library; ours also with the bias + gate + residual
    epilogue of the attention projection."""
    from sana_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(0)
    shapes = [("qkv", 3 * C, C), ("proj", C, C), ("expand", 2 * HID, C), ("point", C, HID)]
    ops_ = []
    for name, n, k in shapes:
        a = torch.randn(tokens, k, generator=g, device=dev).bfloat16()
        w = (torch.randn(n, k, generator=g, device=dev) * 0.02).bfloat16()
        o = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
        ops_.append((name, a, w, o, 2.0 * tokens * n * k))
    flops = sum(f for *_, f in ops_)

    def ours():
        for _, a, w, o, _f in ops_:
            ops.gemm(a, w, out=o)

    def library():
        for _, a, w, o, _f in ops_:
            torch.matmul(a, w.t(), out=o)

    out = {"workload": f"the four projection shapes back to back for {seconds} s each way, {tokens} tokens, hidden {C}"}
    for tag, fn in (("ours", ours), ("library", library), ("ours_again", ours)):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        n = max(int(seconds * 1e3 / e0.elapsed_time(e1)), 1)
        with ClockSampler(0) as clk:
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
        c = clk.summary()
        ms = e0.elapsed_time(e1) / n
        out[tag] = {"ms_per_round": ms, "tflops": flops / (ms * 1e-3) / 1e12, "rounds": n, "clocks": c}
    print(json.dumps(out))


def run_kernel_rates(tokens_side: int, batch: int, iters: int = 20) -> None:
    """Device-timed rate of each HBM-bound kernel of a 1.6B-width block on `batch` samples of
    tokens_side x tokens_side tokens (one JSON line).  Bytes are the algorithmic ones: every
    input element read once, every output element written once; the fraction is of the measured
    copy bandwidth.  Inputs are far larger than L2 at the default batch."""
    from sana_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(0)
    Wd = Hh = tokens_side
    N = Wd * Hh
    rows = batch * N
    peaks = load_peaks()
    peak = peaks["hbm_gbs"]
    LH = C // 32  # linear-attention heads
    x = torch.randn(rows, C, generator=g, device=dev).bfloat16()
    table = (torch.randn(6, C, generator=g, device=dev) * 0.1).bfloat16()
    t = (torch.randn(batch, 6 * C, generator=g, device=dev) * 0.1).bfloat16()
    qkv = torch.randn(rows, 3 * C, generator=g, device=dev).bfloat16()
    u = torch.randn(rows, 2 * HID, generator=g, device=dev).bfloat16()
    dw_w = (torch.randn(2 * HID, 1, 3, 3, generator=g, device=dev) * 0.2).bfloat16()
    dw_b = (torch.randn(2 * HID, generator=g, device=dev) * 0.1).bfloat16()
    rms_w = torch.ones(C, device=dev, dtype=torch.bfloat16)
    state = ops.la_state(qkv[:, C:2 * C], qkv[:, 2 * C:], batch, N, LH)
    o = torch.empty(rows, C, dtype=torch.bfloat16, device=dev)
    # the video model's self-attention at the same width: 20 heads of 112 channels, rotation after the ReLU
    VH, VD = C // 112, 112
    ang = torch.randn(N, VD // 2, generator=g, device=dev)
    rcos, rsin = ang.cos().contiguous(), ang.sin().contiguous()
    rstate = ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], rcos, rsin, batch, N, VH, VD)
    cases = [
        ("ln_modulate", lambda: ops.ln_modulate(x.view(batch, N, C), table, t, 0, 1), 2 * rows * C * 2),
        ("la_state", lambda: ops.la_state(qkv[:, C:2 * C], qkv[:, 2 * C:], batch, N, LH), 2 * rows * C * 2),
        ("la_apply", lambda: ops.la_apply(qkv[:, :C], state, batch, N, LH, 1e-8, out=o), 2 * rows * C * 2),
        ("dwconv_glu", lambda: ops.dwconv_glu(u, dw_w, dw_b, Wd, Hh), rows * 3 * HID * 2),
        ("rmsnorm", lambda: ops.rmsnorm_(qkv[:, :C], rms_w, 1e-5), 2 * rows * C * 2),
        ("la_rope_state", lambda: ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], rcos, rsin, batch, N, VH, VD),
         2 * rows * C * 2),
        ("la_rope_apply", lambda: ops.la_rope_apply(qkv[:, :C], rcos, rsin, rstate, batch, N, VH, VD, 1e-8, out=o),
         2 * rows * C * 2),
    ]
    # softmax core of the cross-attention: 20 heads x 112 over 300 text tokens (tensor / MUFU-bound, not HBM-bound;
    # "bytes" are q + out, the time per image is what is compared with torch's SDPA = the vendor flash kernel)
    import torch.nn.functional as F

    CH, CD = HEADS, C // HEADS
    kv = torch.randn(batch * TEXT, 2 * C, generator=g, device=dev).bfloat16()
    qc = qkv[:, :C]

    def ca(variant):
        ops.set_cross_attention_variant(variant)
        r = ops.cross_attention(qc, kv[:, :C], kv[:, C:], None, batch, N, TEXT, CH, CD)
        ops.set_cross_attention_variant(0)
        return r

    kvv = kv.view(batch, TEXT, 2, CH, CD)
    sdpa = lambda: F.scaled_dot_product_attention(qc.reshape(batch, N, CH, CD).transpose(1, 2), kvv[:, :, 0].transpose(1, 2),  # noqa: E731
                                                  kvv[:, :, 1].transpose(1, 2))
    cases += [("cross_attention (tcgen05 kernel)", lambda: ca(2), 2 * rows * C * 2),
              ("cross_attention (warp-level kernel)", lambda: ca(1), 2 * rows * C * 2),
              ("torch SDPA (vendor flash kernel, for comparison)", sdpa, 2 * rows * C * 2)]
    out = {"workload": f"HBM-bound kernels, {batch} x {Wd}x{Hh} tokens, hidden {C}", "peak_gbs": peak,
           "peak_source": peaks["source"], "rows": []}
    for name, fn, nbytes in cases:
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["rows"].append({"name": name, "ms": ms, "ms_per_sample": ms / batch, "bytes": nbytes, "gbs": gbs, "frac": gbs / peak})
    print(json.dumps(out))


def gpu_eager_block_tokens_per_s(dev, grid=GRID, iters: int = 5) -> dict:
    """The practical bar: upstream's block as plain torch ops (the restatement in oracle/, which is
    op for op upstream's eager forward) on the GPU in bf16 - cuBLAS GEMMs, cuDNN depthwise conv and
    attention, separate elementwise kernels - on one block of grid[0] x grid[1] tokens at 1.6B width.
    A baseline leg like the CPU one: run after, and outside, every timed region of the product."""
    from oracle import sana_oracle as O
    from sana_b200 import synthetic

    dt = torch.bfloat16
    tokens = grid[0] * grid[1]
    params = synthetic.make_block_params_on_device(C, HID, 0, 0.02, dt, dev)
    g = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn(1, tokens, C, generator=g, device=dev).to(dt)
    y = torch.randn(1, TEXT, C, generator=g, device=dev).to(dt)
    t = (torch.randn(1, 6 * C, generator=g, device=dev) * 0.1).to(dt)
    with torch.no_grad():
        for _ in range(3):
            O.sana_ms_block_forward(x, y, t, params, HEADS, grid)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            O.sana_ms_block_forward(x, y, t, params, HEADS, grid)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {"value": tokens / (ms * 1e-3), "unit": UNIT, "ms_per_block": ms, "dtype": "bf16",
            "what": f"eager torch ops (cuBLAS / cuDNN) of upstream's SanaMSBlock, 1 block x {tokens} tokens at 1.6B width, "
                    f"mean of {iters} runs, CUDA events"}


class KernelTimer:
    """Per-kernel-group device time of eager steps: while active, every operator wrapper of
    sana_b200.ops (and the two NCCL exchanges of the sequence shard, and torch's attention call)
    is bracketed by CUDA events on the current stream."""

    GROUPS = {"gemm": "gemm", "gemm_nvfp4": "gemm", "ln_modulate": "ln_modulate", "la_state": "la_state (+exchange)",
              "la_state_sp": "la_state (+exchange)", "la_apply": "la_apply", "dwconv_glu": "dwconv_glu",
              "cross_attention": "cross_attention_core", "nvfp4_quantize": "nvfp4_quantize", "rmsnorm_": "rmsnorm",
              "ln_modulate_fp4": "ln_modulate", "la_apply_fp4": "la_apply", "nvfp4_quantize_scaled": "nvfp4_quantize",
              "nvfp4_scale_roll": "nvfp4_scale_roll",
              "halo_exchange": "conv_halo"}

    def __init__(self):
        self.events = []
        self._saved = []

    def _wrap(self, owner, name, label):
        fn = getattr(owner, name)
        events = self.events

        def timed(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            events.append((label, e0, e1))
            return r

        self._saved.append((owner, name, fn))
        setattr(owner, name, timed)

    def __enter__(self):
        import torch.nn.functional as F

        from sana_b200 import ops, sharding

        for name, label in self.GROUPS.items():
            self._wrap(ops, name, label)
        self._wrap(F, "scaled_dot_product_attention", "cross_attention_core")
        self._wrap(sharding.SequenceShard, "allreduce_state", "nccl_allreduce")
        return self

    def __exit__(self, *a):
        for owner, name, fn in reversed(self._saved):
            setattr(owner, name, fn)
        self._saved = []

    def summary(self, steps: int) -> dict:
        torch.cuda.synchronize()
        out = {}
        for label, e0, e1 in self.events:
            ent = out.setdefault(label, {"launch_groups": 0, "ms_per_step": 0.0})
            ent["launch_groups"] += 1
            ent["ms_per_step"] += e0.elapsed_time(e1)
        for ent in out.values():
            ent["launch_groups"] //= max(steps, 1)
            ent["ms_per_step"] /= max(steps, 1)
        return out


def seqpar_record(world: int, rank: int, dev, steps: int = 20, warmup: int = 3) -> dict:
    """cfg 4 on this job's GPUs: one SanaMSBlock at 1.6B width on the 21x45x80 = 75 600-token grid,
    the 945 image rows sharded over the ranks; the linear-attention state all-reduce and the conv halo
    rows go through the fused peer-memory kernels.  Timed as CUDA-graph replay and as eager launches
    (max over ranks), then with NCCL doing both exchanges, then once more with events around every
    operator.  This rank's output rows are compared with the unsharded block run on the same GPU."""
    import torch.distributed as dist

    import sana_b200
    from sana_b200 import ops, sharding, synthetic
    from sana_b200.graphs import GraphedForward

    dt = torch.bfloat16
    total = SEQPAR_GRID[0] * SEQPAR_GRID[1] * SEQPAR_GRID[2]
    blk = sana_b200.SanaMSBlock(C, HEADS, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval().to(dev, dt)
    blk.load_state_dict(synthetic.make_block_params_on_device(C, HID, 0, 0.02, dt, dev), strict=True)
    g = torch.Generator(device=dev).manual_seed(4321)  # the same full sequence on every rank
    x_full = torch.randn(1, total, C, generator=g, device=dev).to(dt)
    y = torch.randn(1, TEXT, C, generator=g, device=dev).to(dt)
    t = (torch.randn(1, 6 * C, generator=g, device=dev) * 0.1).to(dt)
    full = blk(x_full, y, t, None, SEQPAR_GRID)  # unsharded, on this GPU, outside any timed region
    shard = sharding.SequenceShard(*SEQPAR_GRID, rank, world, device_steps=True)
    blk.set_sequence_shard(shard)
    a, b = shard.token_range
    xs = shard.scatter_tokens(x_full)
    fused = world > 1
    fused_note = None
    if fused:
        # peer-mapped buffers for the two exchange kernels; if the set-up fails on any rank (no peer access on
        # this box) every rank falls back to the NCCL exchanges and the record says so
        try:
            shard.enable_fused_state_exchange(1, C // 32, dev)
            shard.enable_fused_halo_exchange(SEQPAR_GRID[2] * 2 * HID, dt, dev)
            mine_ok = 1.0
        except Exception as e:  # noqa: BLE001
            mine_ok, fused_note = 0.0, f"{type(e).__name__}: {e}"[:200]
        flag = torch.tensor([mine_ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() < 1.0:
            fused = False
            shard._sp_ptrs = shard._halo_ptrs = None
            fused_note = fused_note or "peer-memory set-up failed on another rank"
        else:
            ops.set_exchange_wait_limit(10.0)  # ranks of a fresh job may reach their first step seconds apart

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        for _ in range(warmup):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        sync_all()
        return ms.item()

    eager = lambda: blk(xs, y, t, None, SEQPAR_GRID)  # noqa: E731
    out = eager()
    err = ((out.float() - full[:, a:b].float()).abs().max() / full.float().abs().max()).item()
    eager_ms = timed(eager, steps)
    sync_all()
    graphed = GraphedForward(lambda v: blk(v, y, t, None, SEQPAR_GRID), xs)
    sync_all()
    gx = graphed.static_args[0]  # replay on the graph's own input buffer: no copy inside the timed region
    graph_ms = timed(lambda: graphed(gx), steps)
    gerr = ((graphed(gx).float() - full[:, a:b].float()).abs().max() / full.float().abs().max()).item()
    nccl_ms = None
    if fused:  # the same block with NCCL all-reduce + send/recv instead of the peer-memory kernels
        saved = shard._sp_ptrs, shard._halo_ptrs
        shard._sp_ptrs = shard._halo_ptrs = None
        nccl_ms = timed(eager, max(steps // 2, 5))
        shard._sp_ptrs, shard._halo_ptrs = saved
    sync_all()
    bsteps = 5
    with KernelTimer() as kt:
        for _ in range(bsteps):
            eager()
        breakdown = kt.summary(bsteps)
    state_status = shard.fused_exchange_status() if fused else 0
    halo_status = shard.fused_halo_status() if fused else 0
    gemm_status = ops.take_gemm_device_status()
    sync_all()
    stats = torch.tensor([err, gerr, float(state_status), float(halo_status)], device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    stats = stats.tolist()
    top = max(breakdown.items(), key=lambda kv: kv[1]["ms_per_step"])
    comm = {k: v["ms_per_step"] for k, v in breakdown.items() if k in ("la_state (+exchange)", "conv_halo")}
    peaks = load_peaks()
    roof_s = block_roofline_seconds(shard.tokens, 1, peaks, C)
    del graphed, full, x_full
    torch.cuda.empty_cache()
    return {
        "workload": f"cfg4: one SanaMSBlock, hidden {C}, 21x45x80 = {total} tokens, 945 image rows sharded over {world} GPU(s)",
        "tokens_per_s": total / (min(graph_ms, eager_ms) * 1e-3), "ms_per_step": min(graph_ms, eager_ms),
        "mode": ("CUDA-graph replay of the sharded block" if graph_ms <= eager_ms else "eager launches") +
                " (the faster of the two ways to run the block, both timed below)",
        "graph_tokens_per_s": total / (graph_ms * 1e-3), "graph_ms_per_step": graph_ms,
        "eager_tokens_per_s": total / (eager_ms * 1e-3), "eager_ms_per_step": eager_ms,
        "nccl_exchange_tokens_per_s": (total / (nccl_ms * 1e-3)) if nccl_ms else None, "nccl_exchange_ms_per_step": nccl_ms,
        "exchange": ("state all-reduce fused into the reduction kernel + conv halo rows pushed by one kernel, both over "
                     "peer memory (plain loads / stores, no multicast)") if fused else
                    ("none (one GPU)" if world == 1 else f"NCCL all-reduce and send / receive (peer-memory set-up failed: {fused_note})"),
        "steps": steps, "warmup": warmup, "rows_per_rank": [r1 - r0 for r0, r1 in shard.ranges],
        "parity_nmax_err": stats[0], "parity_nmax_err_graph": stats[1],
        "parity_against": "the unsharded block on the same GPU, this rank's rows, max over ranks",
        "state_exchange_status": int(stats[2]), "halo_exchange_status": int(stats[3]), "gemm_device_status": gemm_status,
        "kernel_breakdown_rank0_eager": breakdown,
        "largest_kernel_group": {"name": top[0], "ms_per_step": top[1]["ms_per_step"]},
        "exchange_kernels_ms_per_step": comm,
        "block_roofline": {"t_roof_ms": roof_s * 1e3, "frac": roof_s * 1e3 / min(graph_ms, eager_ms)},
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel-rates", type=int, default=0, metavar="SIDE",
                    help="only time the HBM-bound kernels of a block on --batch samples of SIDE x SIDE tokens")
    ap.add_argument("--gemm-rates", type=int, default=0, metavar="TOKENS",
                    help="only time the four projection shapes of a block at this many tokens")
    ap.add_argument("--sustained", action="store_true",
                    help="with --gemm-rates: run our bf16 projections and the vendor library's back to back for two "
                         "seconds each (both under the power cap)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="stack", choices=["stack", "seqpar", "nvfp4", "dit", "small"])
    ap.add_argument("--tokens-side", type=int, default=None,
                    help="stack / dit workloads: side of the square token grid (default 128 = 16 384 tokens)")
    ap.add_argument("--graph", action="store_true",
                    help="replay the forward as one CUDA graph (sana_b200.graphs.GraphedForward)")
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch of the stack workload")
    ap.add_argument("--depth", type=int, default=None, help="blocks in the stack (default 20; 1 for nvfp4)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="seqpar: all-reduce the attention state with NCCL instead of the fused peer-memory kernel")
    ap.add_argument("--measured-scaling", action="store_true",
                    help="nvfp4: quantise every activation with its own measured maximum (two more passes per tensor) "
                         "instead of in the kernel that produces it with the previous step's maximum")
    ap.add_argument("--sdpa-cross-attn", action="store_true",
                    help="use torch SDPA (the vendor flash kernel) for the cross-attention softmax core, for comparison")
    ap.add_argument("--no-seqpar", action="store_true",
                    help="stack workload: leave out the sequence-parallel sub-record (cfg 4 on the same GPUs)")
    ap.add_argument("--no-gpu-eager-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.gemm_rates and args.sustained:
        run_gemm_sustained(args.gemm_rates)
        return
    if args.gemm_rates:
        run_gemm_rates(args.gemm_rates)
        return
    if args.kernel_rates:
        run_kernel_rates(args.kernel_rates, args.batch)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist

    import sana_b200
    from sana_b200 import ops, sharding, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    dt = torch.bfloat16
    peaks = load_peaks()

    nvfp4 = args.workload == "nvfp4"
    whole = args.workload == "dit"
    small = args.workload == "small"
    # widths: Sana-1.6B everywhere except "small" (Sana-0.6B: hidden 1152, 16 heads, FFN 2880, 28 blocks)
    C, HEADS, HID = (1152, 16, 2880) if small else (globals()["C"], globals()["HEADS"], globals()["HID"])
    if args.workload in ("stack", "nvfp4", "dit", "small"):
        depth = args.depth or (1 if nvfp4 else (28 if small else DEPTH))
        if small and args.batch == GLOBAL_BATCH:
            args.batch = 4 * world
        b0, b1 = sharding.batch_partition(args.batch, world)[rank]
        Bl = b1 - b0
        grid = (64, 64) if nvfp4 else ((32, 32) if small else GRID)
        if args.tokens_side and not (nvfp4 or small):
            grid = (args.tokens_side, args.tokens_side)
        tokens = grid[0] * grid[1]
        shard = None
        total_units = args.batch * tokens * depth
        if nvfp4:
            workload = (f"cfg5: {depth} SanaMSBlock(s) at Sana-1.6B width with NVFP4 qkv/out/FFN projections (E2M1, E4M3 "
                        f"scale per 16, fp32 scale per tensor, weights and activations), 64x64 grid = {tokens} tokens, "
                        f"global batch {args.batch}")
        elif small:
            workload = (f"cfg2 width: Sana-0.6B stack, {depth} SanaMSBlocks, hidden {C}, FFN {HID}, 32x32 grid = {tokens} "
                        f"tokens (512 px), global batch {args.batch}" + (", one CUDA graph per step" if args.graph else
                                                                         ", eager launches"))
        elif whole:
            workload = (f"whole Sana-1.6B DiT forward (patch embed + position table, timestep / caption embedders, "
                        f"{depth} SanaMSBlocks, final layer, unpatchify), {grid[0]}x{grid[1]} latent x 32 channels = "
                        f"{tokens} tokens, {TEXT} caption tokens x 2304, global batch {args.batch}")
        else:
            workload = (f"cfg3: Sana-1.6B stack, {depth} SanaMSBlocks, hidden {C}, {C // 32} LA heads x 32, FFN {HID}, "
                        f"{grid[0]}x{grid[1]} grid = {tokens} tokens, global batch {args.batch}")
        parallelism = f"dp{world}"
        scaling = "strong"
    else:
        depth = 1
        Bl = 1
        shard = sharding.SequenceShard(*SEQPAR_GRID, rank, world)
        grid, tokens = SEQPAR_GRID, shard.tokens
        total_units = SEQPAR_GRID[0] * SEQPAR_GRID[1] * SEQPAR_GRID[2]
        workload = (f"cfg4: one SanaMSBlock, hidden {C}, 21x45x80 = 75600 tokens, rows sharded over {world} GPUs "
                    f"(state all-reduce + one-row conv halo)")
        parallelism = f"sp{world}"
        scaling = "strong"

    model = None
    if whole:
        model = sana_b200.SanaMS(input_size=grid[0], patch_size=1, in_channels=32, hidden_size=C, depth=depth,
                                 num_heads=HEADS, mlp_ratio=2.5, class_dropout_prob=0.0, pred_sigma=False,
                                 caption_channels=2304, model_max_length=TEXT, y_norm=True, y_norm_scale_factor=0.01,
                                 attn_type="linear", ffn_type="glumbconv", linear_head_dim=32).eval()
        model = model.to(device=dev, dtype=dt)
        gen = torch.Generator(device=dev).manual_seed(99)
        for name, prm in model.named_parameters():
            if not name.startswith("blocks.") and "norm" not in name:
                prm.data.copy_((torch.randn(prm.shape, generator=gen, device=dev) * 0.02).to(dt))
        stack = sana_b200.BlockStack(C, HEADS, 0)
        stack.blocks = model.blocks
    else:
        stack = sana_b200.BlockStack(C, HEADS, depth).eval()
        stack = stack.to(device=dev, dtype=dt)
    for i, blk in enumerate(stack.blocks):
        blk.load_state_dict(synthetic.make_block_params_on_device(C, HID, i, 0.02, dt, dev), strict=True)
    stack.set_sequence_shard(shard)
    fused_exchange = shard is not None and world > 1 and not args.nccl_exchange
    if fused_exchange:
        shard.device_steps = bool(args.graph)  # the exchange kernels number their own steps under graph replay
        shard.enable_fused_state_exchange(1, C // 32, dev)
        shard.enable_fused_halo_exchange(SEQPAR_GRID[2] * 2 * HID, dt, dev)
    stack.set_nvfp4(nvfp4, delayed_scaling=nvfp4 and not args.measured_scaling, margin=1.0)
    if args.sdpa_cross_attn:
        for blk in stack.blocks:
            blk.cross_attn.softmax_core = "sdpa"

    # host-resident inputs (pinned) for the end-to-end leg; device copies for the kernel leg
    g = torch.Generator().manual_seed(1234 + rank)
    x_h = torch.randn(Bl, tokens, C, generator=g).to(dt).pin_memory()
    y_h = torch.randn(Bl, TEXT, C, generator=g).to(dt).pin_memory()
    t_h = (torch.randn(Bl, 6 * C, generator=g) * 0.1).to(dt).pin_memory()
    out_h = torch.empty(Bl, tokens, C, dtype=dt).pin_memory()
    if whole:  # latents, caption features and timesteps instead of token-major block inputs
        x_h = torch.randn(Bl, 32, grid[0], grid[1], generator=g).to(dt).pin_memory()
        y_h = torch.randn(Bl, 1, TEXT, 2304, generator=g).to(dt).pin_memory()
        t_h = torch.randint(0, 1000, (Bl,), generator=g).to(torch.float32).pin_memory()
        out_h = torch.empty(Bl, 32, grid[0], grid[1], dtype=dt).pin_memory()
    x_d, y_d, t_d = x_h.to(dev), y_h.to(dev), t_h.to(dev)

    def forward(xd, yd, td):
        if whole:
            return model(xd, td, yd, mask=None)
        return stack(xd, yd, td, None, grid)

    if args.graph:
        from sana_b200.graphs import GraphedForward

        if shard is not None and world > 1 and args.nccl_exchange:
            raise SystemExit("--graph needs the peer-memory exchanges (drop --nccl-exchange)")
        eager = forward
        graphed = GraphedForward(lambda a, b, c: eager(a, b, c), x_d, y_d, t_d)
        forward = lambda xd, yd, td: graphed(xd, yd, td)  # noqa: E731
    else:
        eager = forward

    def step():
        return forward(x_d, y_d, t_d)

    # End-to-end leg: every step's inputs come from pinned host memory and its result goes back
    # to pinned host memory, all inside the timed region.  The copies run on a second stream,
    # double-buffered, so that step i+1's upload and step i-1's download overlap step i's kernels
    # (the graph path uploads into the graph's own static inputs instead, on the compute stream).
    copy_stream = torch.cuda.Stream(device=dev)
    e2e_bufs = [tuple(torch.empty_like(v) for v in (x_d, y_d, t_d)) for _ in range(2)]
    e2e_state = {"i": 0, "up": [None, None], "done": [None, None]}

    def _upload(slot):
        with torch.cuda.stream(copy_stream):
            if e2e_state["done"][slot] is not None:  # the step that last read this slot has finished
                copy_stream.wait_event(e2e_state["done"][slot])
            for dst, src in zip(e2e_bufs[slot], (x_h, y_h, t_h)):
                dst.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
            e2e_state["up"][slot] = ev

    def step_e2e():
        if args.graph:
            out_h.copy_(forward(x_h.to(dev, non_blocking=True), y_h.to(dev, non_blocking=True),
                                t_h.to(dev, non_blocking=True)), non_blocking=True)
            return
        cur = torch.cuda.current_stream()
        i = e2e_state["i"]
        slot = i & 1
        if e2e_state["up"][slot] is None:
            _upload(slot)  # first step of a timed run: nothing to overlap with yet
        cur.wait_event(e2e_state["up"][slot])
        e2e_state["up"][slot] = None
        out = forward(*e2e_bufs[slot])
        done = torch.cuda.Event()
        done.record(cur)
        e2e_state["done"][slot] = done
        _upload(slot ^ 1)  # next step's inputs, while this step computes
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done)
            out_h.copy_(out, non_blocking=True)
            out.record_stream(copy_stream)
        e2e_state["i"] = i + 1

    def finish_e2e():
        # the timed region ends only when the last download has landed
        torch.cuda.current_stream().wait_stream(copy_stream)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, finish=None):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        sync_all()
        return ms.item()

    for _ in range(args.warmup):
        step()
    ops.counters.reset()
    ops.counters.gemm_timing = True
    with ClockSampler(local) as clk:
        total_ms = timed(step, args.steps)
    ops.counters.gemm_timing = False
    launches = ops.counters.launches
    eager_ms = None
    if args.graph:
        # a replayed graph runs no Python: per-GEMM events and the launch count come from an
        # eager pass of the same steps (also the "before" figure of the graph)
        ops.counters.reset()
        ops.counters.gemm_timing = True
        eager_ms = timed(lambda: eager(x_d, y_d, t_d), args.steps)
        ops.counters.gemm_timing = False
        launches = ops.counters.launches
    gemm_ms = sum(e0.elapsed_time(e1) for e0, e1, _, _ in ops.counters.gemm_events)
    gemm_flops = sum(f for _, _, f, _ in ops.counters.gemm_events)
    n_gemm = len(ops.counters.gemm_events)
    gemm_bytes = sum(ops.counters.gemm_bytes)  # A + W + out (+ residual) of every timed launch, each once
    by_shape = {}
    for e0, e1, f, label in ops.counters.gemm_events:
        ent = by_shape.setdefault(label, [0, 0.0, 0.0])
        ent[0] += 1
        ent[1] += e0.elapsed_time(e1)
        ent[2] += f
    gemm_breakdown = {k: {"launches": v[0], "avg_ms": v[1] / v[0], "tflops": v[2] / (v[1] * 1e-3) / 1e12}
                      for k, v in by_shape.items()}
    status = ops.take_gemm_device_status() | ops.take_gemm_nvfp4_device_status() | ops.take_cross_attention_device_status()
    fp4_ms = sum(e0.elapsed_time(e1) for e0, e1, _, lab in ops.counters.gemm_events if lab.startswith("nvfp4"))
    fp4_flops = sum(f for _, _, f, lab in ops.counters.gemm_events if lab.startswith("nvfp4"))
    n_fp4 = sum(1 for ev in ops.counters.gemm_events if ev[3].startswith("nvfp4"))

    for _ in range(2):
        step_e2e()
    finish_e2e()
    torch.cuda.synchronize()
    e2e_state["up"] = [None, None]  # the timed run starts cold: its first upload is not pre-issued
    e2e_ms = timed(step_e2e, args.steps, finish_e2e)

    # one more eager step with events around every operator: the per-kernel shares of a step
    with KernelTimer() as kt:
        eager(x_d, y_d, t_d)
        kernel_breakdown = kt.summary(1)
    dw_status = ops.take_dwconv_glu_device_status()
    sp_status = (shard.fused_exchange_status(), shard.fused_halo_status()) if fused_exchange else (0, 0)
    seqpar = None
    if args.workload == "stack" and not args.no_seqpar:
        sync_all()
        seqpar = seqpar_record(world, rank, dev)

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = total_units / (ms_per_step * 1e-3)
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        T_local = Bl * tokens
        roof_s = block_roofline_seconds(T_local, Bl, peaks, C) * depth
        fp4_roofline = None
        if nvfp4 and fp4_ms > 0:
            lib = fp4_library_rate(T_local, 2 * HID, C)  # the vendor FP4 GEMM on the largest projection of the block
            fp4_ach = fp4_flops / (fp4_ms * 1e-3) / 1e12
            fp4_roofline = {"bound": "tensor", "kernel": "gemm_nvfp4_pair_kernel (tcgen05 cta_group::2, kind::mxf4nvf4, block 16)",
                            "achieved": fp4_ach, "unit": "TFLOP/s", "launches": n_fp4, "avg_launch_ms": fp4_ms / n_fp4,
                            "peak": lib.get("fp4_library_tflops"),
                            "peak_source": ("measured in this run: torch._scaled_mm on float4_e2m1fn_x2 operands with E4M3 scales per "
                                            f"16 (the vendor library's block-scaled FP4 GEMM), {T_local}x{2 * HID}x{C}")
                            if "fp4_library_tflops" in lib else lib.get("fp4_library"),
                            "frac": (fp4_ach / lib["fp4_library_tflops"]) if "fp4_library_tflops" in lib else None,
                            "share_of_step": fp4_ms / (eager_ms or total_ms)}
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload, "parallelism": parallelism, "per_gpu_batch": Bl,
                       "l2": "inputs larger than L2 (>3 GB of weights and activations per step)",
                       "cross_attention_core": ("torch SDPA (vendor flash kernel), for comparison" if args.sdpa_cross_attn else
                                                "own tcgen05 kernel (sana_cross_attention); --sdpa-cross-attn times the vendor kernel"),
                       "activation_scaling": (("per-tensor maximum measured on every call (two more passes per activation)"
                                               if args.measured_scaling else
                                               "delayed: FP4 written by the producing kernels with the previous step's maxima")
                                              if nvfp4 else None),
                       "state_exchange": ("state all-reduce fused into the reduction kernel, conv halo rows pushed by one kernel, both "
                                          "over peer memory" if fused_exchange else
                                          ("NCCL all-reduce" if shard is not None and world > 1 else "none"))},
            "roofline": {"bound": "tensor",
                         "kernel": ("gemm_nvfp4_tc_kernel + gemm_bf16_tc_kernel (tcgen05; FP4 and bf16 launches pooled, "
                                    "against the bf16 peak)") if nvfp4 else
                         "gemm_bf16_tc_kernel (tcgen05, all 8 projections of a block)",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"], "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)",
                         "launches": n_gemm, "avg_launch_ms": gemm_ms / max(n_gemm, 1),
                         "share_of_step": gemm_ms / (eager_ms or total_ms),
                         "traffic": (NCU_TRAFFIC_BYTES_PER_LAUNCH_BATCH1 * Bl) if args.workload == "stack" else None,
                         "traffic_source": "one ncu capture at batch 1 (1.958 GB over the 7 launches of a block), scaled by the per-GPU batch",
                         "traffic_algorithmic": gemm_bytes / max(n_gemm, 1)},
            "cuda_graph": bool(args.graph), "eager_ms_per_step": (eager_ms / args.steps) if eager_ms else None,
            "block_roofline": {"t_roof_ms_per_step": roof_s * 1e3, "frac": roof_s * 1e3 / ms_per_step,
                               "formula": "F_gemm/P_tensor + 11.5*T*C*e/BW_hbm, per block"},
            "e2e": {"value": total_units / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": x_h.nbytes + y_h.nbytes + t_h.nbytes, "d2h_bytes_per_step": out_h.nbytes,
                    "ms_per_step": e2e_ms / args.steps},
            "fp4_roofline": fp4_roofline,
            "gemm_breakdown": gemm_breakdown, "kernel_breakdown_ms_per_step": kernel_breakdown, "gpu_launches": launches,
            "gemm_device_status": status, "dwconv_device_status": dw_status,
            "state_exchange_status": sp_status[0], "halo_exchange_status": sp_status[1], "clocks": clk.summary(),
        }
        if seqpar is not None:
            out["seqpar"] = seqpar
        if world == 1 and not args.no_gpu_eager_baseline:
            out["gpu_eager_baseline"] = gpu_eager_block_tokens_per_s(dev)
        if world == 1 and not args.no_cpu_baseline:
            v, cores, sample = cpu_block_tokens_per_s()
            out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        bad = {k: out[k] for k in ("gemm_device_status", "dwconv_device_status", "state_exchange_status",
                                   "halo_exchange_status") if out[k]}
        if seqpar is not None:
            bad.update({"seqpar." + k: seqpar[k] for k in ("state_exchange_status", "halo_exchange_status",
                                                           "gemm_device_status") if seqpar[k]})
        if bad:
            out["failed"] = f"a bounded device wait ran out, the results above are not valid: {bad}"
        print(json.dumps(out))
        if bad:
            if world > 1:
                dist.destroy_process_group()
            sys.exit(1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
