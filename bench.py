#!/usr/bin/env python
"""Benchmark of the W4A16 quantised-linear path on B200.

Workload (default): the decode sweep -- M in {1,4,8,16} over the eight Qwen3.5-4B-like
projection shapes = 32 W4A16 GEMMs per step, synthetic seeded inputs with the distributions
the configuration names (bf16 N(0,1) activations, uniform int4 nibbles, fp16 scales
0.01*|N(0,1)|+1e-3, group 128).  `value` is algorithmic GB/s (weights + scales + activations
+ outputs, each counted once) over the whole step with everything resident in HBM; weights
rotate through 8 distinct copies per shape so that every launch streams from HBM, not L2.

  python bench.py [--gpus N] [--steps K] [--warmup W]          one JSON line (rank 0)
  python bench.py --impl reference ...                          the CPU dequantise+matmul path, same line
  python bench.py --only decode:gate_up:1 --steps 6             one shape, plain launches (for ncu -k)
  python bench.py --only prefill:down:2048 --steps 3
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = {  # name: (k, n)
    "q": (2560, 4096), "k": (2560, 512), "v": (2560, 512), "o": (4096, 2560),
    "gate_up": (2560, 18432), "down": (9216, 2560), "gdn_in": (2560, 8192), "gdn_out": (4096, 2560),
}
DECODE_MS = (1, 4, 8, 16)
PREFILL = [(m, s) for s in ("gate_up", "down") for m in (512, 2048, 8192)]
ROT = 8  # distinct weight copies per shape
SEED = 1234
NCU_TRAFFIC_RATIO = 24.375040 / 24.372224  # dram__bytes_read+write of the captured launch / its algorithmic bytes
L2_BYTES = 126e6


def alg_bytes(m, k, n):
    return k * n / 2 + (k // 128) * n * 2 + m * k * 2 + m * n * 2


def alg_flops(m, k, n):
    return 2.0 * m * n * k


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU dequantise(bf16)-then-matmul path, all host threads
# ----------------------------------------------------------------------------------------------
def cpu_sweep_inputs():
    import numpy as np

    import oracle

    cases = []
    for mi, m in enumerate(DECODE_MS):
        for name, (k, n) in SHAPES.items():
            a, q, s = oracle.synth_inputs(m, k, n, seed=SEED + 17 * mi + len(name))
            cases.append((a, q, s, np.empty((k, n), np.uint16)))
    return cases


def cpu_sweep_once(cases):
    from oracle import C

    t0 = time.perf_counter()
    for a, q, s, scratch in cases:
        C.gemm_cpu_reference(a, q, s, 128, scratch)
    return time.perf_counter() - t0


def sweep_bytes():
    return sum(alg_bytes(m, *SHAPES[s]) for m in DECODE_MS for s in SHAPES)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; this arm is the CPU path on ALL host threads
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import oracle
    from oracle import C

    oracle.build()
    C.set_num_threads(os.cpu_count() or 1)
    cases = cpu_sweep_inputs()
    for _ in range(max(args.warmup, 1) if args.warmup else 0):
        cpu_sweep_once(cases)
    times = [cpu_sweep_once(cases) for _ in range(args.steps)]
    total = sum(times)
    value = sweep_bytes() * args.steps / total / 1e9
    cores = C.num_threads()
    sample = "every step = the full 32-GEMM decode sweep (M in 1,4,8,16 x 8 shapes), dequantise to bf16 then f32 matmul"
    line = {
        "impl": "reference", "metric": "w4a16_decode_sweep_algorithmic_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "kiln's packer/wrapper are Rust (no toolchain here): this arm is the C restatement of its CPU "
                "dequantise-then-matmul convention (oracle/w4a16_oracle.c) on all host threads",
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {
        "workload": "decode sweep: M in {1,4,8,16} x {q 2560->4096, k 2560->512, v 2560->512, o 4096->2560, "
                    "gate+up 2560->18432, down 9216->2560, GDN-in 2560->8192, GDN-out 4096->2560}; int4 group-128, "
                    "fp16 scales, bf16 activations; 32 GEMMs per step",
        "l2": f"weights rotate through {ROT} distinct copies per shape (504 MB between reuses, L2 is 126 MB)",
        "seed": SEED,
    }


# ----------------------------------------------------------------------------------------------
# device side
# ----------------------------------------------------------------------------------------------
class Device:
    def __init__(self, local_rank: int):
        import torch

        import kiln_b200
        from kiln_b200 import _lib

        self.torch, self.k, self.lib = torch, kiln_b200, _lib.lib()
        self.dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(self.dev)
        self.gen = torch.Generator(device=self.dev)
        self.gen.manual_seed(SEED + local_rank)

    def weights(self, k, n, copies):
        t = self.torch
        out = []
        for _ in range(copies):
            b = t.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=t.int32, device=self.dev, generator=self.gen)
            s = (0.01 * t.randn((k // 128, n), device=self.dev, generator=self.gen).abs() + 1e-3).to(t.float16)
            out.append((b, s))
        return out

    def acts(self, m, k):
        t = self.torch
        return t.randn((m, k), device=self.dev, generator=self.gen).to(t.bfloat16)

    def gemm(self, a, w, out):
        return self.k.marlin_w4a16_gemm(a, w[0], w[1], 128, out=out)

    def time_graph(self, fn, launches, reps=10, warm=3):
        """Median microseconds per launch of `fn` captured once in a CUDA graph."""
        t = self.torch
        fn()
        t.cuda.synchronize()
        g = t.cuda.CUDAGraph()
        with t.cuda.graph(g):
            fn()
        for _ in range(warm):
            g.replay()
        t.cuda.synchronize()
        ts = []
        for _ in range(reps):
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            t.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / launches)
        ts.sort()
        return ts[len(ts) // 2]


def decode_detail(d: Device, peaks):
    """Per-shape microseconds, GB/s and fraction of the measured HBM peak (M = 1 and 16)."""
    out = {}
    for name, (k, n) in SHAPES.items():
        copies = max(2, min(64, int(2.2 * L2_BYTES / (k * n / 2)) + 1))
        ws = d.weights(k, n, copies)
        for m in (1, 16):
            a = d.acts(m, k)
            o = d.torch.empty((m, n), dtype=d.torch.bfloat16, device=d.dev)
            nl = max(copies, 32)

            def fn():
                for i in range(nl):
                    d.gemm(a, ws[i % copies], o)

            us = d.time_graph(fn, nl, reps=7)
            gbs = alg_bytes(m, k, n) / us / 1e3
            out[f"{name}:m{m}"] = {"us": round(us, 2), "GBps": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4)}
        del ws
    out.update(fused_rows_detail(d, peaks))
    return out


def small_batch_detail(d: Device, peaks):
    """Continuous-batching row counts (24, 64 and 128 rows) on the four large projections: the tcgen05 kernel that keeps the
    dequantised weights in tensor memory.  Microseconds per launch in a CUDA graph over rotating weight copies, algorithmic
    GB/s and fraction of the measured HBM peak (these sizes are still bound by the weight stream's dequantisation)."""
    out = {}
    for name in ("q", "gate_up", "down", "gdn_in"):
        k, n = SHAPES[name]
        copies = max(2, min(64, int(2.2 * L2_BYTES / (k * n / 2)) + 1))
        ws = d.weights(k, n, copies)
        for m in (24, 64, 128):
            a = d.acts(m, k)
            o = d.torch.empty((m, n), dtype=d.torch.bfloat16, device=d.dev)
            nl = max(copies, 24)

            def fn():
                for i in range(nl):
                    d.gemm(a, ws[i % copies], o)

            us = d.time_graph(fn, nl, reps=5)
            gbs = alg_bytes(m, k, n) / us / 1e3
            out[f"{name}:m{m}"] = {"us": round(us, 2), "GBps": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4)}
        del ws
    return out


def fused_rows_detail(d: Device, peaks):
    """Sibling projections as the library recommends issuing them: q, k, v of an attention layer in ONE grouped launch,
    and gate+up with SwiGLU fused into the epilogue (interleaved columns, [m, 9216] output).  Algorithmic bytes are
    those of the separate GEMMs (the SwiGLU row writes half the output columns)."""
    import kiln_b200
    from kiln_b200 import MarlinPackedProj

    t = d.torch
    out = {}
    k = 2560
    copies = 24
    qkv = [[MarlinPackedProj(b, s, 128, k, n) for (b, s) in d.weights(k, n, copies)] for n in (4096, 512, 512)]
    gu_copies = 14
    gu = [MarlinPackedProj(b, s, 128, k, 18432) for (b, s) in d.weights(k, 18432, gu_copies)]
    for m in (1, 16):
        a = d.acts(m, k)
        outs = [t.empty((m, n), dtype=t.bfloat16, device=d.dev) for n in (4096, 512, 512)]
        nl = 48

        def fn():
            for i in range(nl):
                kiln_b200.grouped_matmul_bf16([a, a, a], [qkv[0][i % copies], qkv[1][i % copies], qkv[2][i % copies]], outs)

        us = d.time_graph(fn, nl, reps=7)
        by = sum(alg_bytes(m, k, n) for n in (4096, 512, 512)) - 2 * m * k * 2  # the activations are read once
        out[f"qkv_grouped:m{m}"] = {"us": round(us, 2), "GBps": round(by / us / 1e3, 1), "frac_hbm": round(by / us / 1e3 / peaks["hbm_gbs"], 4),
                                    "launches": 1}
        o2 = t.empty((m, 9216), dtype=t.bfloat16, device=d.dev)

        def fn2():
            for i in range(nl):
                kiln_b200.swiglu_gate_up(a, gu[i % gu_copies], out=o2)

        us = d.time_graph(fn2, nl, reps=7)
        by = alg_bytes(m, k, 18432) - m * 9216 * 2
        out[f"gate_up_swiglu:m{m}"] = {"us": round(us, 2), "GBps": round(by / us / 1e3, 1), "frac_hbm": round(by / us / 1e3 / peaks["hbm_gbs"], 4)}
    for m in (24, 64):  # continuous-batching row counts: SwiGLU fused into the small-batch tcgen05 kernel's epilogue
        a = d.acts(m, k)
        o2 = t.empty((m, 9216), dtype=t.bfloat16, device=d.dev)
        nl = 28

        def fn3():
            for i in range(nl):
                kiln_b200.swiglu_gate_up(a, gu[i % gu_copies], out=o2)

        us = d.time_graph(fn3, nl, reps=5)
        by = alg_bytes(m, k, 18432) - m * 9216 * 2
        out[f"gate_up_swiglu:m{m}"] = {"us": round(us, 2), "GBps": round(by / us / 1e3, 1), "frac_hbm": round(by / us / 1e3 / peaks["hbm_gbs"], 4)}
    return out


def config0_detail(d: Device, peaks):
    """BASELINE configs[0]: one W4A16 GEMM, M=1, K=2560, N=9216, on the GPU (CUDA-graph replay over rotating weights)
    and through the CPU dequantise-then-matmul path on all host threads, same shape, same run."""
    import numpy as np

    import oracle
    from oracle import C

    m, k, n = 1, 2560, 9216
    copies = int(2.2 * L2_BYTES / (k * n / 2)) + 1
    ws = d.weights(k, n, copies)
    a = d.acts(m, k)
    o = d.torch.empty((m, n), dtype=d.torch.bfloat16, device=d.dev)
    nl = max(copies, 32)

    def fn():
        for i in range(nl):
            d.gemm(a, ws[i % copies], o)

    us = d.time_graph(fn, nl, reps=7)
    del ws
    ah, q, s = oracle.synth_inputs(m, k, n, seed=SEED)
    scratch = np.empty((k, n), np.uint16)
    C.gemm_cpu_reference(ah, q, s, 128, scratch)
    ts = []
    for _ in range(5):
        t0 = time.perf_counter()
        C.gemm_cpu_reference(ah, q, s, 128, scratch)
        ts.append(time.perf_counter() - t0)
    cpu_us = sorted(ts)[len(ts) // 2] * 1e6
    gbs = alg_bytes(m, k, n) / us / 1e3
    return {"m": m, "k": k, "n": n, "gpu_us": round(us, 2), "gpu_GBps": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
            "cpu_us": round(cpu_us, 1), "cpu_threads": C.num_threads(), "cpu_kind": "port (dequantise to bf16, f32 matmul)"}


def prefill_detail(d: Device, peaks):
    """Chunked-prefill GEMMs: microseconds, TFLOP/s, fraction of the measured bf16 tensor peak."""
    out = {}
    t = d.torch
    for m, name in PREFILL:
        k, n = SHAPES[name]
        ws = d.weights(k, n, 2)
        a = d.acts(m, k)
        o = t.empty((m, n), dtype=t.bfloat16, device=d.dev)
        flush = t.empty(int(160e6), dtype=t.uint8, device=d.dev)
        for i in range(3):
            d.gemm(a, ws[i % 2], o)
        t.cuda.synchronize()
        ts = []
        for i in range(7):
            flush.zero_()  # write a buffer larger than L2 between timed launches
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            d.gemm(a, ws[i % 2], o)
            e1.record()
            t.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        us = ts[len(ts) // 2]
        tf = alg_flops(m, k, n) / us / 1e6
        out[f"{name}:m{m}"] = {"us": round(us, 1), "TFLOPs": round(tf, 1), "frac_bf16_burst": round(tf / peaks["bf16_tflops"], 4),
                               "frac_bf16_nominal_2250": round(tf / 2250.0, 4)}
        del ws, a, o, flush
    # gate+up with SwiGLU fused into the tcgen05 epilogue ([m, 9216] output, columns interleaved in runs of 32), same timing
    import kiln_b200
    from kiln_b200 import MarlinPackedProj

    k, n = SHAPES["gate_up"]
    for m in (2048,):
        ws = [MarlinPackedProj(b, s_, 128, k, n) for (b, s_) in d.weights(k, n, 2)]
        a = d.acts(m, k)
        o = t.empty((m, n // 2), dtype=t.bfloat16, device=d.dev)
        flush = t.empty(int(160e6), dtype=t.uint8, device=d.dev)
        for i in range(3):
            kiln_b200.swiglu_gate_up(a, ws[i % 2], out=o)
        t.cuda.synchronize()
        ts = []
        for i in range(7):
            flush.zero_()
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            kiln_b200.swiglu_gate_up(a, ws[i % 2], out=o)
            e1.record()
            t.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        us = ts[len(ts) // 2]
        tf = alg_flops(m, k, n) / us / 1e6
        out[f"gate_up_swiglu:m{m}"] = {"us": round(us, 1), "TFLOPs": round(tf, 1), "frac_bf16_burst": round(tf / peaks["bf16_tflops"], 4),
                                       "frac_bf16_nominal_2250": round(tf / 2250.0, 4)}
        del ws, a, o, flush
    return out


def pack_detail(d: Device):
    """Load-time quantise + pack of one layer's MLP projections (gate, up: 2560 -> 9216; down: 9216 -> 2560) from bf16
    weights already in HBM (device packer), and of one gate projection from host f32 (threaded host packer).  The
    reference packs on the CPU after a device -> host copy (its own figure: 16.9 s for the 96 MLP projections of the model)."""
    import numpy as np

    t = d.torch
    from kiln_b200 import pack as hpack
    from kiln_b200 import pack_from_bf16

    out = {}
    total_ms = 0.0
    for name, (k, n) in (("gate", (2560, 9216)), ("up", (2560, 9216)), ("down", (9216, 2560))):
        w = (t.randn((k, n), device=d.dev, generator=d.gen) * 0.02).to(t.bfloat16)
        pack_from_bf16(w)
        t.cuda.synchronize()
        e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            pack_from_bf16(w)
        e1.record()
        t.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 5
        total_ms += ms
        out[name] = {"device_ms": round(ms, 3), "GBps_read_plus_written": round((k * n * 2 + k * n / 2) / ms / 1e6, 1)}
        del w
    out["mlp_layer_device_ms"] = round(total_ms, 3)
    out["model_96_projections_device_ms"] = round(total_ms * 32, 1)
    wh = (np.random.default_rng(SEED).standard_normal((2560, 9216)) * 0.02).astype(np.float32)
    hpack.quantize_and_pack(wh, 2560, 9216, 128)
    t0 = time.perf_counter()
    hpack.quantize_and_pack(wh, 2560, 9216, 128)
    out["gate_host_all_threads_ms"] = round((time.perf_counter() - t0) * 1e3, 1)
    out["reference_published"] = "16.9 s for the 96 MLP projections, CPU pack after a device->host copy (other hardware)"
    return out


def stack_detail(d: Device, m: int = 64):
    """Config 3: a 32-layer Qwen3.5-4B-like projection stack (24 GDN layers: GDN-in, GDN-out, gate+up, down; 8
    attention layers: q, k, v, o, gate+up, down = 144 GEMMs, distinct random int4 weights per layer, 1.6 GB, so
    every GEMM streams from HBM) at continuous-batch M, activations carried layer to layer.  Between GEMMs
    there are cheap torch elementwise adapters standing in for attention / GDN mixing (slice, SwiGLU,
    residual add, RMS normalisation); they are part of `stack_us`, and `gemm_only_us` is the same 144 GEMMs
    captured without them."""
    t = d.torch
    layers = []
    for li in range(32):
        attn = li % 4 == 3
        names = ["q", "k", "v", "o", "gate_up", "down"] if attn else ["gdn_in", "gdn_out", "gate_up", "down"]
        layers.append((attn, {nm: d.weights(*SHAPES[nm], 1)[0] for nm in names}))
    h0 = d.acts(m, 2560)

    def norm(x):
        xf = x.float()
        return (xf * t.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(t.bfloat16)

    def gemm(x, w):
        o = t.empty((x.shape[0], w[1].shape[1]), dtype=t.bfloat16, device=d.dev)
        return d.gemm(x, w, o)

    def forward(with_adapters=True):
        h = h0
        for attn, w in layers:
            x = norm(h) if with_adapters else h
            if attn:
                q = gemm(x, w["q"])
                k_ = gemm(x, w["k"])
                v_ = gemm(x, w["v"])
                mix = q + t.cat([k_, v_] * 4, dim=1) if with_adapters else q  # stand-in for attention
                o = gemm(mix, w["o"])
            else:
                z = gemm(x, w["gdn_in"])
                mix = (z[:, :4096] * t.sigmoid(z[:, 4096:].float()).to(t.bfloat16)) if with_adapters else z[:, :4096].contiguous()
                o = gemm(mix, w["gdn_out"])
            h = (h + o) if with_adapters else o
            x = norm(h) if with_adapters else h
            gu = gemm(x, w["gate_up"])
            act = (t.nn.functional.silu(gu[:, :9216].float()).to(t.bfloat16) * gu[:, 9216:]) if with_adapters else gu[:, :9216].contiguous()
            dn = gemm(act, w["down"])
            h = (h + dn) if with_adapters else dn
        return h

    out = {"m": m, "gemms": 144, "weight_GB": round(sum(alg_bytes(0, *SHAPES[nm]) for a_, w in layers for nm in w) / 1e9, 3)}
    for key, flag in (("stack_us", True), ("gemm_only_us", False)):
        out[key] = round(d.time_graph(lambda: forward(flag), 1, reps=7), 1)
    bytes_total = sum(alg_bytes(m, *SHAPES[nm]) for a_, w in layers for nm in w)
    flops_total = sum(alg_flops(m, *SHAPES[nm]) for a_, w in layers for nm in w)
    out["gemm_only_GBps"] = round(bytes_total / out["gemm_only_us"] / 1e3, 1)
    out["gemm_only_TFLOPs"] = round(flops_total / out["gemm_only_us"] / 1e6, 1)
    out["ideal_us_at_measured_hbm"] = round(bytes_total / load_peaks()["hbm_gbs"] / 1e3, 1)
    del layers
    return out


def sharded_detail(d: Device, world: int, rank: int):
    """The path's N-sharded configuration: M=16384, K=9216, N=73728 split by columns over the ranks, local
    GEMM + NCCL all-gather of the bf16 slices (blocked [g, M, N/g] result).  Times are max over ranks."""
    import torch.distributed as dist

    t = d.torch
    m, k, n = 16384, 9216, 73728
    nl = n // world
    w = d.weights(k, nl, 1)[0]
    a = d.acts(m, k)
    local = t.empty((m, nl), dtype=t.bfloat16, device=d.dev)
    gathered = t.empty((world, m, nl), dtype=t.bfloat16, device=d.dev) if world > 1 else None
    from kiln_b200.shard import all_gather_columns

    def once():
        e = [t.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        d.gemm(a, w, local)
        e[1].record()
        if world > 1:
            all_gather_columns(local, None, gathered)
        e[2].record()
        t.cuda.synchronize()
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), e[0].elapsed_time(e[2])

    fused_ms = fused_mc_ms = None
    fused_rows = mc_rows = None
    rows = [0, 1, 127, 128, 8191, 12345, m - 2, m - 1]  # sampled rows of the parity check below
    rows_t = t.tensor(rows, device=d.dev)
    if world > 1:
        import kiln_b200
        from kiln_b200 import MarlinPackedProj

        lin = kiln_b200.ColumnParallelLinear(MarlinPackedProj(w[0], w[1], 128, k, nl), rank, world, None)
        sym = kiln_b200.FusedGatherOutput(m, n, d.dev)

        def fused_once(multicast):
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            kiln_b200.fused_column_parallel_gemm(a, lin, sym, multicast=multicast)  # GEMM with store epilogue + barrier
            e1.record()
            t.cuda.synchronize()
            return e0.elapsed_time(e1)

        def fused_time(multicast):
            fused_once(multicast)
            fused_once(multicast)
            dist.barrier()
            fl = sorted(fused_once(multicast) for _ in range(3))[1]
            tt = t.tensor([fl], device=d.dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        fused_ms = fused_time(False)
        t.cuda.synchronize()
        dist.barrier()
        fused_rows = sym.tensor[rows_t].clone()
        # every rank must take the same branch: ask the group whether all of them got a multicast address
        has_mc = t.tensor([1 if sym.multicast_ptr else 0], device=d.dev)
        dist.all_reduce(has_mc, op=dist.ReduceOp.MIN)
        fused_mc_ms = fused_time(True) if int(has_mc.item()) else None
        t.cuda.synchronize()
        dist.barrier()
        mc_rows = sym.tensor[rows_t].clone() if fused_mc_ms else None
        del sym
    once()
    once()
    if world > 1:
        dist.barrier()
    reps = [once() for _ in range(3)]
    med = [sorted(x[i] for x in reps)[1] for i in range(3)]
    if world > 1:
        tt = t.tensor(med, device=d.dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        med = [float(v) for v in tt.tolist()]
    parity = sharded_parity(d, world, rank, a, w, local, gathered, fused_rows, mc_rows, rows, rows_t, k, nl)
    # strong-scaling reference: the unsharded GEMM (all 73728 columns) on one GPU, timed on rank 0 in this same run
    t1_ms = None
    if world > 1:
        if rank == 0:
            wf = d.weights(k, n, 1)[0]
            of = t.empty((m, n), dtype=t.bfloat16, device=d.dev)
            d.gemm(a, wf, of)
            t.cuda.synchronize()
            ts = []
            for _ in range(3):
                e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                e0.record()
                d.gemm(a, wf, of)
                e1.record()
                t.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            t1_ms = sorted(ts)[1]
            del wf, of
        dist.barrier()
    else:
        t1_ms = med[0]
    flops = alg_flops(m, k, n)
    best_ms = min(x for x in (med[2], fused_ms, fused_mc_ms) if x)
    out = {
        "parity": parity,
        "unsharded_gemm_ms_same_run": round(t1_ms, 3) if t1_ms else None,
        "best_ms": round(best_ms, 3),
        "efficiency": round(t1_ms / (world * best_ms), 3) if t1_ms else None,
        "link_frac": round(((world - 1) / world * m * n * 2 / 770e9 * 1e3) / best_ms, 3) if world > 1 else None,
        "m": m, "k": k, "n": n, "n_per_gpu": nl, "gemm_ms": round(med[0], 3), "allgather_ms": round(med[1], 3),
        "total_ms": round(med[2], 3), "TFLOPs_per_gpu_gemm": round(flops / world / med[0] / 1e9, 1),
        "TFLOPs_total_end_to_end": round(flops / med[2] / 1e9, 1),
        "allgather_GBps_per_gpu_recv": round((world - 1) * m * nl * 2 / med[1] / 1e6, 1) if world > 1 else None,
        "layout": "blocked [g, M, N/g]", "scaling": "strong",
        "fused_gemm_allgather_ms": round(fused_ms, 3) if fused_ms else None,
        "fused_TFLOPs_total": round(flops / fused_ms / 1e9, 1) if fused_ms else None,
        "fused_layout": "row-major [M, N] on every GPU (peer stores from the GEMM epilogue + one barrier)",
        "fused_multicast_ms": round(fused_mc_ms, 3) if fused_mc_ms else None,
        "fused_multicast_TFLOPs_total": round(flops / fused_mc_ms / 1e9, 1) if fused_mc_ms else None,
        "fused_multicast_layout": "the same through one multimem.st per piece to the NVSwitch multicast address",
        "fused_roofline": fused_roofline(m, k, n, world, min(x for x in (fused_ms, fused_mc_ms) if x)) if fused_ms else None,
    }
    del w, a, local, gathered
    return out


def sharded_parity(d, world, rank, a, w, local, gathered, fused_rows, mc_rows, rows, rows_t, k, nl):
    """Parity of the sharded outputs on eight sampled rows, every rank taking part:
      * this rank's local GEMM against the fp64 oracle on a 1024-column window of its shard (the packed words of the
        window are unpacked on the host with the oracle's consumer-side unpacker; a column slice of the packed
        tensors is the packed column slice), bound 1e-2;
      * the NCCL-gathered blocks against every rank's own local GEMM, bit for bit;
      * the fused (peer-store) and multicast results against the same, to 2^-7 (the fused launch never splits K,
        the plain one may) and against each other bit for bit."""
    import numpy as np
    import torch.distributed as dist

    import oracle
    from oracle import C

    t = d.torch
    res = {"rows": rows}
    # (1) local GEMM vs oracle on a window of columns
    c0, cw = (nl // 2) // 64 * 64, 1024
    bp = w[0][:, 2 * c0:2 * (c0 + cw)].contiguous().cpu().numpy()
    sp = w[1][:, c0:c0 + cw].contiguous().cpu().numpy()
    q = C.unpack_fragment(np.ascontiguousarray(bp), k, cw)
    perm = C.scale_perm()
    s_nat = np.empty_like(sp)
    s_nat.reshape(sp.shape[0], cw // 64, 64)[:, :, perm] = sp.reshape(sp.shape[0], cw // 64, 64)
    a_rows = a[rows_t].contiguous().cpu().view(t.int16).numpy().view(np.uint16)
    ref = C.gemm_fp64(a_rows, q, s_nat, 128)
    got = oracle.bf16_bits_to_f32(local[rows_t][:, c0:c0 + cw].contiguous().cpu().view(t.int16).numpy().view(np.uint16))
    rel = float(np.abs(got - ref).max() / np.abs(ref).max())
    res["local_vs_oracle_max_rel"] = rel
    ok = rel <= 1e-2
    if world > 1:
        mine = local[rows_t].contiguous()
        every = t.empty((world,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(every.view(world * mine.shape[0], nl), mine)
        res["gathered_bit_equal"] = bool(t.equal(gathered[:, rows_t], every))
        ok = ok and res["gathered_bit_equal"]
        dense = every.permute(1, 0, 2).reshape(len(rows), world * nl).float()
        for key, fr in (("fused", fused_rows), ("multicast", mc_rows)):
            if fr is not None:
                dmax = float((fr.float() - dense).abs().max() / dense.abs().max())
                res[key + "_vs_local_gemms_max_rel"] = dmax
                ok = ok and dmax <= 2.0 ** -7
        if fused_rows is not None and mc_rows is not None:
            res["multicast_equals_peer_stores"] = bool(t.equal(fused_rows, mc_rows))
            ok = ok and res["multicast_equals_peer_stores"]
        flag = t.tensor([1 if ok else 0], device=d.dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        worst = t.tensor([rel], device=d.dev)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        ok = bool(flag.item())
        res["local_vs_oracle_max_rel"] = float(worst.item())
    res["ok"] = ok
    return res


def fused_roofline(m, k, n, world, ms):
    """Target time of the fused GEMM + all-gather = the slower of this GPU's flops at the measured bf16 peak and the
    bytes it must receive from its peers at the measured NVLink peer-copy rate (770 GB/s per direction per GPU)."""
    peaks = load_peaks()
    t_flops = alg_flops(m, k, n) / world / (peaks["bf16_tflops"] * 1e9)  # ms
    t_link = (world - 1) / world * m * n * 2 / 770e9 * 1e3
    target = max(t_flops, t_link)
    return {"bound": "tensor" if t_flops >= t_link else "nvlink", "target_ms": round(target, 3), "achieved_ms": round(ms, 3),
            "frac": round(target / ms, 3), "flops_ms": round(t_flops, 3), "link_ms": round(t_link, 3),
            "peaks": peaks["source"] + " bf16 burst; 770 GB/s measured peer copy"}


def run_only(args):
    """One shape with plain (non-graph) launches over rotating weights: the command ncu profiles."""
    kind, name, m = args.only.split(":")
    m = int(m)
    k, n = SHAPES[name]
    d = Device(0)
    t = d.torch
    copies = max(2, min(64, int(2.2 * L2_BYTES / (k * n / 2)) + 1))
    ws = d.weights(k, n, copies)
    a = d.acts(m, k)
    o = t.empty((m, n), dtype=t.bfloat16, device=d.dev)
    for i in range(args.warmup):
        d.gemm(a, ws[i % copies], o)
    t.cuda.synchronize()
    e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        d.gemm(a, ws[(i + args.warmup) % copies], o)
    e1.record()
    t.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"only": args.only, "us_per_launch_plain": us, "GBps": alg_bytes(m, k, n) / us / 1e3,
                      "TFLOPs": alg_flops(m, k, n) / us / 1e6, "steps": args.steps, "warmup": args.warmup}), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    d = Device(local_rank)
    t = torch

    # ---- resident tensors of the sweep
    ws = {name: d.weights(k, n, ROT) for name, (k, n) in SHAPES.items()}
    # every GEMM of the step has its own activations and its own output; all of them live in two device arenas so that
    # the end-to-end step below can move a whole step's inputs (outputs) with one host->device (device->host) copy
    order = [(m, name) for m in DECODE_MS for name in SHAPES]
    in_elems = [m * SHAPES[name][0] for m, name in order]
    out_elems = [m * SHAPES[name][1] for m, name in order]
    # (two sets of arenas: even steps use set 0, odd steps set 1, so that the end-to-end loop can copy the next step's inputs
    # in and the previous step's outputs out while a step computes)
    arenas_in = [t.randn(sum(in_elems), device=d.dev, generator=d.gen).to(t.bfloat16) for _ in range(2)]
    arenas_out = [t.empty(sum(out_elems), dtype=t.bfloat16, device=d.dev) for _ in range(2)]
    acts, outs = [{}, {}], [{}, {}]
    for b in range(2):
        oi, oo = 0, 0
        for (m, name), ni, no in zip(order, in_elems, out_elems):  # offsets stay 16-byte aligned: every size is a multiple of 256
            acts[b][(m, name)] = arenas_in[b][oi:oi + ni].view(m, SHAPES[name][0])
            outs[b][(m, name)] = arenas_out[b][oo:oo + no].view(m, SHAPES[name][1])
            oi, oo = oi + ni, oo + no

    def step(parity):
        for mi, m in enumerate(DECODE_MS):
            for name, (k, n) in SHAPES.items():
                d.gemm(acts[parity][(m, name)], ws[name][(parity * 4 + mi) % ROT], outs[parity][(m, name)])

    step(0)
    step(1)
    t.cuda.synchronize()
    graphs = []
    launches_per_step = None
    for parity in (0, 1):
        g = t.cuda.CUDAGraph()
        c0 = d.lib.kiln_w4a16_launch_count()
        with t.cuda.graph(g):
            step(parity)
        launches_per_step = int(d.lib.kiln_w4a16_launch_count() - c0)
        graphs.append(g)

    def barrier():
        if world > 1:
            dist.barrier()
        t.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        graphs[i % 2].replay()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # The timed region is `reps` passes of the K-step loop, enough of them to last 0.2 s or more whatever K is (one
    # step is a fraction of a millisecond), so that clocks are sampled under the load that is timed.
    e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        graphs[i % 2].replay()
    e1.record()
    t.cuda.synchronize()
    probe_ms = max(e0.elapsed_time(e1), 1e-3)
    reps = max(1, int(200.0 / probe_ms) + 1)
    if world > 1:
        tt = t.tensor([reps], device=d.dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        reps = int(tt.item())
    barrier()
    e0.record()
    for _ in range(reps):
        for i in range(args.steps):
            graphs[i % 2].replay()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1) / reps
    # a longer untimed run under the same sampler so that clocks are sampled under this load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        for i in range(50):
            graphs[i % 2].replay()
        t.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        tt = t.tensor([elapsed_ms], device=d.dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tt.item())
    ms_per_step = elapsed_ms / args.steps
    step_bytes = sweep_bytes()
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers
    # One step = one pinned-host -> device copy of the 32 activation matrices, the 32 GEMMs (the CUDA graph captured
    # above from kiln_b200.marlin_w4a16_gemm calls, which is how a serving loop issues a decode step) and one
    # device -> pinned-host copy of the 32 outputs.  The three run on three streams chained by events and the host
    # reads step i's outputs while step i+1 computes, as a serving loop overlaps its transfers: every step's copies
    # are inside the timed region, and the region ends when the last step's outputs are in host memory.
    h_in = [a.cpu().pin_memory() for a in arenas_in]
    h_out = [t.empty(a.shape, dtype=a.dtype).pin_memory() for a in arenas_out]
    s_in, s_gemm, s_out = t.cuda.Stream(d.dev), t.cuda.Stream(d.dev), t.cuda.Stream(d.dev)
    ev_in = [t.cuda.Event() for _ in range(2)]     # inputs of the step using buffer set b are on the device
    ev_gemm = [t.cuda.Event() for _ in range(2)]   # its GEMMs are done (inputs may be overwritten, outputs may be copied)
    ev_out = [t.cuda.Event() for _ in range(2)]    # its outputs are in host memory (device outputs may be overwritten)
    checks = []

    def e2e_run(steps):
        for e in ev_in + ev_gemm + ev_out:
            e.record(t.cuda.current_stream(d.dev))
        t.cuda.synchronize()
        for i in range(steps):
            b = i % 2
            with t.cuda.stream(s_in):
                s_in.wait_event(ev_gemm[b])  # the step two back, which read this buffer set
                arenas_in[b].copy_(h_in[b], non_blocking=True)
                ev_in[b].record(s_in)
            with t.cuda.stream(s_gemm):
                s_gemm.wait_event(ev_in[b])
                s_gemm.wait_event(ev_out[b])  # the step two back has left the output arena
                graphs[b].replay()
                ev_gemm[b].record(s_gemm)
            with t.cuda.stream(s_out):
                s_out.wait_event(ev_gemm[b])
                h_out[b].copy_(arenas_out[b], non_blocking=True)
                ev_out[b].record(s_out)
            if i >= 1:  # the host reads the previous step's result while this step runs
                ev_out[1 - b].synchronize()
                checks.append(float(h_out[1 - b][0]))
        ev_out[(steps - 1) % 2].synchronize()
        checks.append(float(h_out[(steps - 1) % 2][0]))

    e2e_run(4)
    barrier()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    e2e_s = time.perf_counter() - t0
    barrier()
    if world > 1:
        tt = t.tensor([e2e_s], device=d.dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    h2d = sum(m * SHAPES[s][0] * 2 for m in DECODE_MS for s in SHAPES)
    d2h = sum(m * SHAPES[s][1] * 2 for m in DECODE_MS for s in SHAPES)
    e2e_value = world * step_bytes * args.steps / e2e_s / 1e9

    line = {
        "metric": "w4a16_decode_sweep_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s / args.steps * 1e3,
                "how": "per step: one pinned-host -> device copy of all 32 activation matrices, one replay of the CUDA graph "
                       "captured from 32 kiln_b200.marlin_w4a16_gemm calls (graph replay, not 32 fresh calls), one device -> "
                       "pinned-host copy of all 32 outputs; copy-in, GEMMs and copy-out on three streams chained by events over two "
                       "buffer sets, the host reads step i's outputs while step i+1 computes; wall clock from the first copy-in to "
                       "the last step's outputs in host memory"},
        "gpu_launches": launches_per_step * args.steps * reps,
        "timed": {"passes_of_the_k_step_loop": reps, "steps_timed": args.steps * reps, "seconds": elapsed_ms * reps / 1e3},
        "clocks": clocks,
        "roofline": {
            "bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": value / world / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (MEASURED_PEAKS.json hbm_gbs, copy)",
            "kernel": "w4a16_decode_kernel",
            # DRAM bytes per (average) launch: the ncu capture of one launch (gate+up, M=1: profiles/decode_kernel_gate_up_m1.txt)
            # read 24.375 MB and wrote 0 against 24.372 MB algorithmic, i.e. every weight byte crosses DRAM exactly once;
            # the figure here scales that ratio to the sweep's average launch
            "traffic": NCU_TRAFFIC_RATIO * step_bytes / launches_per_step,
            "traffic_source": "ncu capture of gate_up M=1 (dram read+write / algorithmic = %.4f), scaled by bytes" % NCU_TRAFFIC_RATIO,
            "per_launch": {"algorithmic_bytes": step_bytes / launches_per_step,
                           "avg_us": ms_per_step * 1e3 / launches_per_step},
            "frac_of_nominal_8TBps": value / world / 8000.0,
        },
        "us_per_gemm_avg": ms_per_step * 1e3 / 32,
    }
    if world > 1:
        line["note"] = "replicas: every rank runs the sweep on its own tokens (data-parallel serving); no collective in the path"

    if rank == 0 and not args.quick:
        del h_in, h_out
        line["decode"] = decode_detail(d, peaks)
        if world == 1:
            line["config0"] = config0_detail(d, peaks)
        line["prefill"] = prefill_detail(d, peaks)
        if world == 1:
            line["small_batch"] = small_batch_detail(d, peaks)
        line["stack_m64"] = stack_detail(d, 64)
        if world == 1:
            line["pack"] = pack_detail(d)
        if world == 1:
            cases = cpu_sweep_inputs()
            cpu_sweep_once(cases)
            reps = 3
            ct = sum(cpu_sweep_once(cases) for _ in range(reps)) / reps
            from oracle import C

            line["cpu_baseline"] = {
                "value": step_bytes / ct / 1e9, "unit": "GB/s", "cores": C.num_threads(), "kind": "port",
                "ms_per_step": ct * 1e3,
                "sample": f"{reps} passes of the full 32-GEMM sweep on the host (dequantise to bf16, f32 matmul)",
            }
    if not args.quick:
        sh = sharded_detail(d, world, rank)  # every rank takes part (collective inside)
        if rank == 0:
            line["sharded"] = sh
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, help="decode:<shape>:<m> or prefill:<shape>:<m>")
    ap.add_argument("--quick", action="store_true", help="skip the per-shape tables and the CPU baseline")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
