#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

Headline workload (one "step"): the fused-dequant GEMVs of one Qwen2.5-7B-shaped decode token
(hidden 3584, intermediate 18944, 28 Q / 4 KV heads x 128, vocab 152064; 28 layers + lm_head),
batch 1, f32 activations, once with Q4_K weights and once with Q4_0 weights, every matrix a
distinct device-resident instance (8 GB of weights, far larger than L2).  Metric: achieved HBM
GB/s on the ALGORITHMIC bytes (weights once + vectors), whole job over all ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N>1 is launched with torch.distributed.run, one rank per GPU; each rank streams its own replica of
the weights (weak scaling, no data-path collective), timing is CUDA events + max over ranks.
`--impl reference` times the CPU oracle (the reference's own implementation is Rust + Metal and
cannot be built or run here) on the host cores for the same metric.
Prints ONE JSON line on rank 0.
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

HIDDEN, INTER, VOCAB, LAYERS = 3584, 18944, 152064, 28
Q_DIM, KV_DIM = 28 * 128, 4 * 128
FMT_Q8_0, FMT_Q4_0, FMT_Q4K, FMT_Q5_0, FMT_Q5K, FMT_Q6K = 0, 1, 2, 3, 4, 5
BLOCK = {FMT_Q8_0: (32, 34), FMT_Q4_0: (32, 18), FMT_Q4K: (256, 144), FMT_Q5_0: (32, 22), FMT_Q5K: (256, 176), FMT_Q6K: (256, 210)}
METRIC = "fused_dequant_gemv_hbm_gbs"


def row_bytes(fmt, k):
    return k // BLOCK[fmt][0] * BLOCK[fmt][1]


def gemv_bytes(fmt, m, k, residual=False, batch=1):
    """Algorithmic bytes of one GEMV: weights once + input + output (+ residual read)."""
    return m * row_bytes(fmt, k) + batch * 4 * k + batch * 4 * m + (batch * 4 * m if residual else 0)


# (name, rows, k, residual): the weight matrices of one layer
LAYER_MATS = [("q", Q_DIM, HIDDEN, False), ("k", KV_DIM, HIDDEN, False), ("v", KV_DIM, HIDDEN, False),
              ("o", HIDDEN, Q_DIM, True), ("gate", INTER, HIDDEN, False), ("up", INTER, HIDDEN, False),
              ("down", HIDDEN, INTER, True)]
LAUNCHES_PER_LAYER = 4   # fused Q|K|V, o-proj (+residual), fused gate/up+SiLU, down (+residual)


def pass_bytes(fmt, layers=LAYERS):
    """Algorithmic bytes of one pass: every weight matrix once, every launch's input and output vectors once."""
    rb_h, rb_i = row_bytes(fmt, HIDDEN), row_bytes(fmt, INTER)
    qkv = (Q_DIM + 2 * KV_DIM) * rb_h + 4 * HIDDEN + 4 * (Q_DIM + 2 * KV_DIM)
    o = HIDDEN * row_bytes(fmt, Q_DIM) + 4 * Q_DIM + 2 * 4 * HIDDEN
    ffn = 2 * INTER * rb_h + 4 * HIDDEN + 4 * INTER
    down = HIDDEN * rb_i + 4 * INTER + 2 * 4 * HIDDEN
    return (qkv + o + ffn + down) * layers + gemv_bytes(fmt, VOCAB, HIDDEN)


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, from the ncu capture of one Q4_K launch.
NCU_TRAFFIC_RATIO = (306.80e6 + 4.71e6) / 307.18e6


EXTRAS_LIMIT_S = 420


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


class GemvSet:
    """Device-resident weights and scratch vectors for one weight format of the workload."""

    def __init__(self, R, ctx, fmt, seed, layers=LAYERS):
        self.R, self.ctx, self.fmt, self.layers = R, ctx, fmt, layers
        sigma = 0.01 if fmt == FMT_Q4K else 0.02
        self.w = []
        for l in range(layers):
            d = {}
            for i, (name, m, k, _) in enumerate(LAYER_MATS):
                buf = ctx.new_buffer(m * row_bytes(fmt, k))
                R.fill_weights(ctx, fmt, buf, m * (k // BLOCK[fmt][0]), seed * 100003 + l * 16 + i, sigma)
                d[name] = buf
            self.w.append(d)
        self.lm_head = ctx.new_buffer(VOCAB * row_bytes(fmt, HIDDEN))
        R.fill_weights(ctx, fmt, self.lm_head, VOCAB * (HIDDEN // BLOCK[fmt][0]), seed * 100003 + 99991, sigma)
        f4 = lambda n: ctx.new_buffer(4 * n)
        self.x, self.xn, self.q, self.kk, self.v = f4(HIDDEN), f4(HIDDEN), f4(Q_DIM), f4(KV_DIM), f4(KV_DIM)
        self.gate, self.up, self.act, self.logits = f4(INTER), f4(INTER), f4(INTER), f4(VOCAB)
        R.fill_normal_f32(ctx, self.xn, HIDDEN, seed + 7, 1.0)
        R.fill_normal_f32(ctx, self.q, Q_DIM, seed + 8, 1.0)
        R.fill_normal_f32(ctx, self.act, INTER, seed + 9, 1.0)
        ctx.call("memset", self.x, 0, 4 * HIDDEN)
        ctx.flush()

    def run(self):
        """All GEMVs of one decode token through the C-ABI operator calls: fused Q|K|V, o-proj + residual, fused
        gate/up + SiLU, down + residual per layer, then lm_head.  The activations that RMSNorm / attention would
        produce are fixed synthetic vectors: only the GEMV family is on this benchmark's path."""
        R, ctx, f = self.R, self.ctx, self.fmt
        n = {FMT_Q4_0: "q4_0", FMT_Q4K: "q4k", FMT_Q8_0: "q8_0"}[f]
        gemv = getattr(R, "gemv_%s_f32in_f32out" % n)
        gemv_add = getattr(R, "gemv_%s_add_f32_f32in" % n)
        qkv = getattr(R, "fused_qkv_%s_f32" % n)
        ffn = getattr(R, "fused_ffn_%s_f32" % n)
        for w in self.w:
            qkv(ctx, w["q"], w["k"], w["v"], self.xn, self.q, self.kk, self.v, Q_DIM, KV_DIM, HIDDEN)
            gemv_add(ctx, w["o"], self.q, self.x, self.x, HIDDEN, Q_DIM)
            ffn(ctx, w["gate"], w["up"], self.xn, self.act, INTER, HIDDEN)
            gemv_add(ctx, w["down"], self.act, self.x, self.x, HIDDEN, INTER)
        gemv(ctx, self.lm_head, self.xn, self.logits, VOCAB, HIDDEN)


def measure_batch8(R, ctx, torch, stream, gset, reps=5):
    """The same GEMV set at batch 8 (the second batch size of the configuration): every matrix is streamed once for 8
    activation rows (integer tensor-core path of gemv_imma.cu); q | k | v and gate | up are one launch each, their
    activations are prepared once.
    Returns (GB/s on the algorithmic bytes, launches per token)."""
    B = 8
    fmt = gset.fmt
    f4 = lambda n: ctx.new_buffer(4 * n * B)
    xn, x, q, kk, v, gate, up, act, logits = (f4(HIDDEN), f4(HIDDEN), f4(Q_DIM), f4(KV_DIM), f4(KV_DIM), f4(INTER), f4(INTER), f4(INTER),
                                              f4(VOCAB))
    for b_, n, sd in ((xn, HIDDEN, 11), (q, Q_DIM, 12), (act, INTER, 13)):
        R.fill_normal_f32(ctx, b_, n * B, sd, 1.0)
    ctx.call("memset", x, 0, 4 * HIDDEN * B)
    l0 = ctx.launches

    def run():
        for w in gset.w:
            R.gemv_batched_multi_f32(ctx, fmt, (w["q"], w["k"], w["v"]), xn, (q, kk, v), (Q_DIM, KV_DIM, KV_DIM), HIDDEN, B)
            R.gemv_batched_f32(ctx, fmt, w["o"], q, x, x, HIDDEN, Q_DIM, B)
            R.gemv_batched_multi_f32(ctx, fmt, (w["gate"], w["up"]), xn, (gate, up), (INTER, INTER), HIDDEN, B)
            R.gemv_batched_f32(ctx, fmt, w["down"], act, x, x, HIDDEN, INTER, B)
        R.gemv_batched_f32(ctx, fmt, gset.lm_head, xn, logits, None, VOCAB, HIDDEN, B)
    run()
    ctx.flush()
    launches = ctx.launches - l0
    ctx.graph_begin(); run(); g = ctx.graph_end()
    for _ in range(2):
        g.launch()
    ctx.flush()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        g.launch()
    e1.record(stream)
    ctx.flush()
    ms = e0.elapsed_time(e1) / reps
    nbytes = sum(gemv_bytes(fmt, m, k, residual=r, batch=B) for _, m, k, r in LAYER_MATS) * gset.layers + gemv_bytes(fmt, VOCAB, HIDDEN, batch=B)
    g.destroy()
    for b_ in (xn, x, q, kk, v, gate, up, act, logits):
        b_.free()
    return nbytes / (ms * 1e-3) / 1e9, int(launches)


def measure_folded(R, ctx, torch, stream, gset, reps=5):
    """The batch-1 set recorded with the opt-in folding of consecutive GEMVs into one persistent launch."""
    ctx.set_tuning("stream_fuse", 1)
    try:
        ctx.graph_begin(); gset.run(); g = ctx.graph_end()
    finally:
        ctx.set_tuning("stream_fuse", 0)
    for _ in range(2):
        g.launch()
    ctx.flush()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        g.launch()
    e1.record(stream)
    ctx.flush()
    ms = e0.elapsed_time(e1) / reps
    out = {"gbs": pass_bytes(gset.fmt, gset.layers) / (ms * 1e-3) / 1e9, "kernel_launches_per_token": g.kernel_launches,
           "gemv_launches_folded": g.fused_launches}
    g.destroy()
    return out


def cpu_sample(fmt_list, threads, min_seconds, layers_sample=2):
    """Oracle GEMV (the engine's CPU dequant formulas + f32 dot, OpenMP over rows) on a bounded sample of
    the workload: `layers_sample` layers + lm_head per format, repeated until `min_seconds` of CPU work.
    Returns (GB/s, seconds, description, threads)."""
    import oracle as O
    O.build_oracle()
    if threads:
        O.set_num_threads(threads)
    rng = np.random.default_rng(1002)
    data = []
    for fmt in fmt_list:
        mats = [(m, k) for _, m, k, _ in LAYER_MATS] * layers_sample + [(VOCAB, HIDDEN)]
        ws = {}
        for m, k in set(mats):
            # random bytes with a small finite f16 scale in each block (content does not affect CPU time)
            rb = row_bytes(fmt, k)
            w = rng.integers(0, 256, (m, rb), dtype=np.uint8)
            bb = BLOCK[fmt][1]
            w.reshape(m, -1, bb)[:, :, 1] = 0x1C
            if fmt == FMT_Q4K:
                w.reshape(m, -1, bb)[:, :, 3] = 0x1C
            ws[(m, k)] = w
        data.append((fmt, mats, ws))
    xs = {k: rng.normal(0, 1, k).astype(np.float32) for k in (HIDDEN, INTER)}
    total_bytes, total_t, passes = 0, 0.0, 0
    while total_t < min_seconds and passes < 1000:
        for fmt, mats, ws in data:
            for m, k in mats:
                t0 = time.perf_counter()
                O.gemv(fmt, ws[(m, k)], xs[k], m, k, O.TIER_DEQUANT)
                total_t += time.perf_counter() - t0
                total_bytes += gemv_bytes(fmt, m, k)
        passes += 1
    desc = "%d layer(s) + lm_head of the workload per format (%s), %d pass(es), %.1f s of CPU work" % (
        layers_sample, "+".join({1: "Q4_0", 2: "Q4_K"}[f] for f in fmt_list), passes, total_t)
    return total_bytes / total_t / 1e9, total_t, desc, O.num_threads()


SHAPES = {
    FMT_Q4K: [(3584, 3584), (512, 3584), (18944, 3584), (3584, 18944), (152064, 3584), (1024, 2048), (2048, 1024), (2048, 2048),
              (50304, 2048)],
    FMT_Q4_0: [(3584, 3584), (512, 3584), (18944, 3584), (3584, 18944), (152064, 3584)],
    FMT_Q8_0: [(1152, 896), (896, 896), (4864, 896), (896, 4864), (151936, 896)],
    FMT_Q6K: [(3584, 18944), (152064, 3584)],
    FMT_Q5K: [(3584, 3584), (152064, 3584)],
    FMT_Q5_0: [(3584, 3584), (18944, 3584)],
}


def run_shapes(R, ctx, torch, stream, reps=20, min_bytes=600e6):
    """Pipelined GB/s per decode shape: each shape is launched over enough distinct weight instances to exceed
    L2 several times (>= 600 MB), recorded as one command list, replayed `reps` times between CUDA events."""
    peak, _ = measured_peak()
    names = {FMT_Q8_0: "q8_0", FMT_Q4_0: "q4_0", FMT_Q4K: "q4k", FMT_Q5_0: "q5_0", FMT_Q5K: "q5k", FMT_Q6K: "q6k"}
    for fmt in (FMT_Q4K, FMT_Q4_0, FMT_Q8_0, FMT_Q6K, FMT_Q5K, FMT_Q5_0):
        for m, k in SHAPES[fmt]:
            for batch in ((1, 8) if fmt <= FMT_Q4K and (m, k) in ((18944, 3584), (4864, 896)) else (1,)):
                wbytes = m * row_bytes(fmt, k)
                n_inst = int(min(64, max(2, np.ceil(min_bytes / wbytes))))
                ws = []
                for i in range(n_inst):
                    b = ctx.new_buffer(wbytes)
                    if fmt <= FMT_Q4K:
                        R.fill_weights(ctx, fmt, b, m * (k // BLOCK[fmt][0]), 17 + i, 0.01)
                    else:   # no generator for these formats: any bytes stream at the same speed; finite scales keep the sums finite
                        ctx.call("memset", b, 0x11, wbytes)
                    ws.append(b)
                x, y = ctx.new_buffer(4 * k * batch), ctx.new_buffer(4 * m * batch)
                R.fill_normal_f32(ctx, x, k * batch, 3, 1.0)

                def run():
                    for w in ws:
                        if batch == 1:
                            getattr(R, "gemv_%s_f32in_f32out" % names[fmt])(ctx, w, x, y, m, k)
                        else:
                            R.gemv_batched_f32(ctx, fmt, w, x, y, None, m, k, batch)
                run()
                ctx.flush()
                ctx.graph_begin(); run(); g = ctx.graph_end()
                for _ in range(3):
                    g.launch()
                ctx.flush()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    g.launch()
                e1.record(stream)
                ctx.flush()
                us = e0.elapsed_time(e1) / reps / n_inst * 1e3
                alg = gemv_bytes(fmt, m, k, batch=batch)
                print(json.dumps({"fmt": names[fmt], "m": m, "k": k, "batch": batch, "instances": n_inst, "us_per_launch": round(us, 2),
                                  "algorithmic_bytes": alg, "gbs": round(alg / us / 1e3, 1), "frac_of_measured_peak": round(alg / us / 1e3 / peak, 3)}),
                      flush=True)
                g.destroy()
                for w in ws:
                    w.free()


def measured_tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def zipf_routing(torch, T, E, k, seed, s=1.1):
    """8 distinct experts per token, expert popularity ~ Zipf(s) over the expert index; uniform routing weights."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    p = 1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float64) ** s
    idx = torch.multinomial((p / p.sum()).float().expand(T, E).contiguous(), k, replacement=False, generator=g).to(torch.int32)
    w = torch.rand(T, k, device="cuda", generator=g)
    return idx, w


def run_block(R, ctx, torch, stream, T=4096, reps=20, E=128, h=2048, ff=768, k=8, zipf_s=1.1, name="qwen3-moe"):
    """Qwen3-MoE-shaped batched MoE block (hidden 2048, 128 experts, top-8, expert intermediate 768, Q4_K experts
    dequantised to bf16 tiles feeding the tcgen05 grouped GEMM), T tokens ~ N(0,1), Zipf(1.1) expert popularity.
    Timed per layer over the expert part (permutation, both grouped GEMMs, combine) with the routing given."""
    rb = lambda kk: kk // 256 * 144
    gate, up, down = ctx.new_buffer(E * ff * rb(h)), ctx.new_buffer(E * ff * rb(h)), ctx.new_buffer(E * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, E * ff, h), (up, E * ff, h), (down, E * h, ff))):
        R.fill_weights(ctx, FMT_Q4K, b, rows * (kk // 256), 5 + i, 0.01)
    x = torch.randn(T, h, device="cuda")
    idx, w = zipf_routing(torch, T, E, k, 1, s=zipf_s)
    out = torch.empty(T, h, device="cuda")
    nbytes = R.moe_grouped_scratch_bytes(ctx, T, h, ff, E, k)
    scratch = ctx.new_buffer(nbytes)
    cnt = torch.bincount(idx.flatten().long(), minlength=E)
    tiles = int(((cnt + 255) // 256).sum().item())                       # 256-slot tiles of the CTA-pair kernel
    full, rest = cnt // 256, cnt % 256
    issued_cols = int((full * 256 + ((rest + 31) // 32) * 32).sum().item())   # MMA N is the tile's slots rounded up to 32

    def step():
        R.moe_experts_grouped_q4k_bf16(ctx, gate, up, down, x, idx, w, None, out, scratch, nbytes, T, h, ff, E, k)
    l0 = ctx.launches
    for _ in range(3):
        step()
    ctx.flush()
    launches_per_layer = (ctx.launches - l0) // 3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        step()
    e1.record(stream)
    ctx.flush()
    ms = e0.elapsed_time(e1) / reps
    flops = 2.0 * T * k * 3 * h * ff                  # useful multiply-adds of the three expert products
    padded = 2.0 * issued_cols * 3 * h * ff            # what the MMAs issue
    peak, kind = measured_tensor_peak()
    wbytes = int((cnt > 0).sum().item()) * 3 * h * ff * 144 // 256       # every expert that has a slot is streamed once
    return {"workload": "%s-shaped MoE block, %d tokens, %d experts top-%d, hidden %d, intermediate %d, Q4_K -> bf16 tiles, "
                        "Zipf(%.1f) routing" % (name, T, E, k, h, ff, zipf_s),
            "weight_gbs": wbytes / (ms * 1e-3) / 1e9,
            "ms_per_layer": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
            "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / peak, "peak_tflops": peak, "peak_kind": kind,
            "issued_over_useful_flops": padded / flops, "token_tiles": tiles, "slots_per_expert_max": int(cnt.max().item()),
            "slots_per_expert_min": int(cnt.min().item()), "launches_per_layer": int(launches_per_layer),
            "finite": bool(torch.isfinite(out).all().item())}


def run_q8_0_pass(R, ctx, torch, stream, layers=24, reps=20):
    """BASELINE configs[0] as a throughput figure: all GEMVs of one Qwen2.5-0.5B-shaped decode token in Q8_0 (hidden 896;
    fused q | k | v 896 -> 1152 with f32 bias; o 896 -> 896 + residual; fused gate / up 896 -> 4864 + SiLU; down 4864 -> 896 +
    residual; 24 layers; lm_head 896 -> 151936), batch 1, f32 activations, every layer a distinct weight instance (0.53 GB per
    token), recorded once and replayed between CUDA events."""
    H, QD, KV, FF, V = 896, 896, 128, 4864, 151936
    rb = lambda k: k // 32 * 34
    f4 = lambda n: ctx.new_buffer(4 * n)
    ws = []
    for l in range(layers):
        d = {}
        for i, (name, m, k) in enumerate((("q", QD, H), ("k", KV, H), ("v", KV, H), ("o", H, QD), ("gate", FF, H), ("up", FF, H), ("down", H, FF))):
            d[name] = ctx.new_buffer(m * rb(k))
            R.fill_weights(ctx, FMT_Q8_0, d[name], m * (k // 32), 9000 + l * 16 + i, 0.02)
        ws.append(d)
    lm = ctx.new_buffer(V * rb(H))
    R.fill_weights(ctx, FMT_Q8_0, lm, V * (H // 32), 9999, 0.02)
    x, xn, q, kk, v, act, logits = f4(H), f4(H), f4(QD), f4(KV), f4(KV), f4(FF), f4(V)
    bq, bk, bv = f4(QD), f4(KV), f4(KV)
    for b_, n, sd in ((xn, H, 1), (q, QD, 2), (act, FF, 3), (bq, QD, 4), (bk, KV, 5), (bv, KV, 6)):
        R.fill_normal_f32(ctx, b_, n, 70 + sd, 1.0)
    ctx.call("memset", x, 0, 4 * H)

    def run():
        for w in ws:
            R.fused_qkv_f32bias_q8_0_f32(ctx, w["q"], w["k"], w["v"], xn, q, kk, v, bq, bk, bv, QD, KV, H)
            R.gemv_q8_0_add_f32_f32in(ctx, w["o"], q, x, x, H, QD)
            R.fused_ffn_q8_0_f32(ctx, w["gate"], w["up"], xn, act, FF, H)
            R.gemv_q8_0_add_f32_f32in(ctx, w["down"], act, x, x, H, FF)
        R.gemv_q8_0_f32in_f32out(ctx, lm, xn, logits, V, H)
    l0 = ctx.launches
    run()
    ctx.flush()
    launches = ctx.launches - l0
    ctx.graph_begin(); run(); g = ctx.graph_end()
    for _ in range(3):
        g.launch()
    ctx.flush()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        g.launch()
    e1.record(stream)
    ctx.flush()
    us = e0.elapsed_time(e1) / reps * 1e3
    g.destroy()
    wbytes = layers * ((QD + 2 * KV) * rb(H) + H * rb(QD) + 2 * FF * rb(H) + H * rb(FF)) + V * rb(H)
    act_bytes = layers * (4 * H + 8 * (QD + 2 * KV) + 4 * QD + 8 * H + 4 * H + 4 * FF + 4 * FF + 8 * H) + 4 * H + 4 * V
    peak, kind = measured_peak()
    gbs = (wbytes + act_bytes) / us / 1e3
    for w in ws:
        for b_ in w.values():
            b_.free()
    lm.free()
    return {"workload": "qwen2.5-0.5b decode GEMV set (24 layers + lm_head), Q8_0, batch 1, f32 activations, f32 q|k|v bias",
            "us_per_token": us, "gbs": gbs, "frac_of_peak": gbs / peak, "peak_kind": kind, "launches_per_token": int(launches),
            "algorithmic_bytes_per_token": int(wbytes + act_bytes),
            "note": "97 launches of 1-10 MB each are bound by launch and pipeline-fill latency; the 145 MB lm_head alone runs at 0.63"}


def run_extras(R, ctx, torch, dist, stream, rank, world, args, decode_only=False, stop=lambda: False):
    """Figures for the other rows of the path: one OLMoE-shaped MoE layer (1/16/256 tokens), the full
    OLMoE-shaped greedy decode (tok/s) and, at N>1, the row-sharded lm_head with its all-gather."""
    out = {}
    E, h, ff, k, L = 64, 2048, 1024, 8, 16

    def timed(fn, reps):
        fn()
        ctx.flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        ctx.flush()
        return e0.elapsed_time(e1) / reps

    # OLMoE-shaped model weights (also the 16 MoE layers timed below), generated on the device
    rb = lambda kk: kk // 256 * 144
    shapes = {"wq": (L * h, h), "wk": (L * h, h), "wv": (L * h, h), "wo": (L * h, h), "gate": (L * E * ff, h),
              "up": (L * E * ff, h), "down": (L * E * h, ff), "lm_head": (50304, h)}
    dev = {}
    for i, (name, (rows, kk)) in enumerate(shapes.items()):
        dev[name] = ctx.new_buffer(rows * rb(kk))
        R.fill_weights(ctx, R.FMT_Q4K, dev[name], rows * (kk // 256), 1004 * 7919 + i + 100 * rank, 0.01)
    for name, n, sig in (("tok_emb", 50304 * h, 0.02), ("router", L * E * h, 0.02)):
        dev[name] = ctx.new_buffer(4 * n)
        R.fill_normal_f32(ctx, dev[name], n, 4242 + len(name), sig)
    ones = np.ones(L * h, np.float32)
    dev["attn_norm"], dev["ffn_norm"], dev["out_norm"] = ctx.buffer_from(ones), ctx.buffer_from(ones), ctx.buffer_from(ones[:h])
    ctx.flush()
    # MoE layer alone: 16 distinct layers per replay (3.6 GB of expert weights: nothing stays in L2)
    moe = {}
    for T in (() if decode_only else (1, 16, 256)):
        x = ctx.new_buffer(T * h * 4)
        R.fill_normal_f32(ctx, x, T * h, 5 + T, 1.0)
        o, idx = ctx.new_buffer(T * h * 4), ctx.new_buffer(T * k * 4)
        nb = R.moe_scratch_bytes(ctx, T, h, ff, E, k)
        scratch = ctx.new_buffer(nb)
        eg, ed = E * ff * rb(h), E * h * rb(ff)

        def run_layers():
            for l in range(L):
                R.moe_layer_q4k(ctx, dev["router"].ptr + l * E * h * 4, dev["gate"].ptr + l * eg, dev["up"].ptr + l * eg,
                                dev["down"].ptr + l * ed, x, None, o, idx, None, scratch, nb, T, h, ff, E, k, 0)
        run_layers()
        ctx.flush()
        ctx.graph_begin(); run_layers(); g = ctx.graph_end()
        ms = timed(g.launch, 5) / L
        U = len(np.unique(idx.download(np.int32, T * k)))
        alg = U * 3 * (h * ff * 144 // 256) + 4 * E * h + T * 8 * h
        moe["T%d" % T] = {"us_per_layer": ms * 1e3, "tokens_per_s": T / (ms * 1e-3), "distinct_experts_last_layer": U,
                          "algorithmic_gbs": alg / (ms * 1e-3) / 1e9}
        g.destroy()
    if not decode_only:
        # the same layer at 256 tokens through the tensor-core block (bf16 operands)
        T = 256
        x = torch.randn(T, h, device="cuda")
        o = torch.empty(T, h, device="cuda")
        nbg = R.moe_grouped_scratch_bytes(ctx, T, h, ff, E, k)
        scratch = ctx.new_buffer(nbg)
        eg, ed = E * ff * rb(h), E * h * rb(ff)
        torch.cuda.synchronize()

        def run_layers_tc():
            for l in range(L):
                R.moe_layer_q4k_bf16(ctx, dev["router"].ptr + l * E * h * 4, dev["gate"].ptr + l * eg, dev["up"].ptr + l * eg,
                                     dev["down"].ptr + l * ed, x, None, o, None, None, scratch, nbg, T, h, ff, E, k, 0)
        run_layers_tc()
        ctx.flush()
        ms = timed(run_layers_tc, 5) / L
        moe["T256_tensor_cores_bf16"] = {"us_per_layer": ms * 1e3, "tokens_per_s": T / (ms * 1e-3)}
        out["moe_layer_olmoe_q4k"] = moe
        scratch.free()
        # Qwen3-MoE-shaped batched block (4096 tokens, 128 experts, Zipf routing) on the tensor cores
        out["moe_block_qwen3_shape_bf16"] = run_block(R, ctx, torch, stream, T=4096, reps=10)
        # dense feed-forward block of a prefill pass at the Qwen2.5-7B shape (hidden 3584, intermediate 18944), 2048 tokens
        Td, hd_, ffd = 2048, HIDDEN, INTER
        wts = [ctx.new_buffer(r * rb(kk)) for r, kk in ((ffd, hd_), (ffd, hd_), (hd_, ffd))]
        for i, (b, (r, kk)) in enumerate(zip(wts, ((ffd, hd_), (ffd, hd_), (hd_, ffd)))):
            R.fill_weights(ctx, R.FMT_Q4K, b, r * (kk // 256), 611 + i, 0.01)
        xd, od = torch.randn(Td, hd_, device="cuda"), torch.empty(Td, hd_, device="cuda")
        nbd = ctx.lib.runit_ffn_q4k_bf16_scratch_bytes(Td, hd_, ffd)
        sd = ctx.new_buffer(nbd)
        msd = timed(lambda: R.ffn_q4k_bf16(ctx, wts[0], wts[1], wts[2], xd, None, 0.0, xd, od, sd, nbd, Td, hd_, ffd), 5)
        fl = 2.0 * 3 * Td * hd_ * ffd
        peak, kind = measured_tensor_peak()
        out["dense_ffn_qwen7b_prefill_bf16"] = {"tokens": Td, "ms": msd, "tflops": fl / (msd * 1e-3) / 1e12,
                                               "frac_of_tensor_peak": fl / (msd * 1e-3) / 1e12 / peak, "peak_tflops": peak, "peak_kind": kind}
        for b in wts + [sd]:
            b.free()
    # full OLMoE-shaped greedy decode: 128-token prompt, 64 greedy steps, f16 KV, no host round trips
    cfg = R.ModelCfg(n_layers=L, hidden=h, n_heads=16, n_kv_heads=16, head_dim=128, vocab=50304, n_experts=E, top_k=k, ff=ff,
                     max_seq=2048, renorm=0, eps=1e-5, theta=10000.0)
    model = R.Model(ctx, cfg, dev)
    prompt = np.random.default_rng(1004).integers(0, 50304, 128).astype(np.int32)
    model.generate_greedy(prompt, 8)
    t0 = time.perf_counter()
    toks = model.generate_greedy(prompt, 64)
    dt_all = time.perf_counter() - t0
    t0 = time.perf_counter()
    model.generate_greedy(prompt, 0)
    dt_prompt = time.perf_counter() - t0
    out["olmoe_decode_q4k"] = {"decode_tok_s": 64 / max(dt_all - dt_prompt, 1e-9), "prompt_tok_s": 128 / dt_prompt,
                               "tokens_total_s": 192 / dt_all, "launches_per_token": int(model.launches_per_token),
                               "note": "wall clock around one call that runs 192 recorded steps and synchronises once"}
    # the same prompts through the batched prefill (tensor-core GEMMs, causal attention over the cache)
    pf = {}
    for n_tok in (128, 1024, 2048):
        pr = np.random.default_rng(n_tok).integers(0, 50304, n_tok).astype(np.int32)
        model.prefill(pr)
        t0 = time.perf_counter()
        for _ in range(3):
            model.prefill(pr)
        dt = (time.perf_counter() - t0) / 3
        pf["T%d" % n_tok] = {"ms": dt * 1e3, "tokens_per_s": n_tok / dt}
    out["olmoe_decode_q4k"]["batched_prefill"] = pf
    # the same request served the way an engine would: the prompt through the batched prefill, then 63 recorded decode steps
    # from the cache it filled (bf16 GEMM operands in the prompt pass: the tokens are compared with the token-by-token run)
    model.prefill(prompt)
    t0 = time.perf_counter()
    nxt = model.prefill(prompt)
    cont = model.generate_greedy(np.array([nxt], np.int32), 63, start_pos=128)
    dt_srv = time.perf_counter() - t0
    out["olmoe_decode_q4k"]["prompt_by_batched_prefill"] = {
        "ms_total": dt_srv * 1e3, "tokens_total_s": 192 / dt_srv,
        "same_tokens_as_token_by_token": bool(np.array_equal(np.asarray(cont, np.int32), np.asarray(toks[128:192], np.int32)))}
    model.close()
    if rank == 0:
        out["gguf_load"] = run_gguf_load(ctx)
        if not decode_only:
            out["q8_0_qwen0_5b_gemv_pass"] = run_q8_0_pass(R, ctx, torch, stream)
    def go_on():
        # the ranks decide together whether the next sharded measurement starts (it holds collectives)
        t = torch.tensor([1 if stop() else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item()) == 0
    if world > 1 and go_on():
        out["lm_head_row_sharded"] = run_sharded_lm_head(R, ctx, torch, dist, stream, rank, world)
    if world > 1 and go_on():
        out["moe_expert_parallel"] = run_expert_parallel(R, ctx, torch, dist, stream, rank, world)
    if world > 1 and go_on():
        try:
            out["olmoe_decode_q4k_expert_parallel"] = run_ep_decode(R, ctx, torch, dist, rank, world)
        except Exception as exc:   # symmetric memory unavailable on this host
            out["olmoe_decode_q4k_expert_parallel"] = {"unavailable": repr(exc)[:200]}
    return out


# ───────────────────────── sharded paths (N > 1) ─────────────────────────

def _time_steps(torch, dist, stream, ctx, fn, steps, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_sharded_lm_head(R, ctx, torch, dist, stream, rank, world, steps=20):
    """Qwen2.5-7B lm_head (152064 x 3584), Q4_K and Q4_0, rows split over the ranks, logits all-gathered."""
    from runit_mac_b200 import parallel as P
    out = {}
    M, K = 152064, 3584
    _, n = P.shard_rows(M, world, rank)
    x = torch.randn(K, dtype=torch.float32, device="cuda")
    for fmt, name in ((2, "q4k"), (1, "q4_0")):
        be = P.CudaBackend(R, ctx, torch)
        rb = R.row_bytes(fmt, K)
        w = ctx.new_buffer(n * rb)
        R.fill_weights(ctx, fmt, w, n * (K // R.BLOCK_ELEMS[fmt]), 1002 + rank, 0.01)
        be.set_lm_head(fmt, w, n, K)
        ms = _time_steps(torch, dist, stream, ctx, lambda: P.sharded_gemv(be, dist, torch, x, M, world, rank), steps, world)
        ms_local = _time_steps(torch, dist, stream, ctx, lambda: be.local_gemv(x), steps, world)
        if world == 1:
            logits, tok = torch.empty(M, dtype=torch.float32, device="cuda"), torch.empty(4, dtype=torch.int32, device="cuda")
            ms_g1 = _time_steps(torch, dist, stream, ctx, lambda: R.gemv_argmax_f32(ctx, fmt, w, x, None, 0.0, logits, tok, M, K), steps, world)
        alg = M * rb + 4 * (K + M)
        out[name] = {"us_per_call": ms * 1e3, "us_local_gemv": ms_local * 1e3, "aggregate_gbs": alg / (ms * 1e-3) / 1e9,
                     "rows_per_rank": n}
        if world == 1:
            out[name]["us_per_call_greedy_epilogue"] = ms_g1 * 1e3
        if world > 1:
            try:
                fused = P.FusedAllGatherGemv(R, ctx, torch, dist, fmt, w, M, K, world, rank)
                ms_f = _time_steps(torch, dist, stream, ctx, lambda: fused(x), steps, world)
                out[name].update({"us_per_call_fused_peer_stores": ms_f * 1e3, "aggregate_gbs_fused": alg / (ms_f * 1e-3) / 1e9})
                # greedy: the argmax runs in the GEMV's epilogue and 8 bytes per rank are exchanged instead of the logits
                greedy = P.FusedGreedyLmHead(R, ctx, torch, dist, fmt, w, M, K, world, rank)
                ms_g = _time_steps(torch, dist, stream, ctx, lambda: greedy(x), steps, world)
                out[name].update({"us_per_call_greedy_pairs": ms_g * 1e3, "aggregate_gbs_greedy": alg / (ms_g * 1e-3) / 1e9})
            except Exception as exc:   # symmetric memory unavailable on this host: keep the NCCL figures
                out[name]["fused_unavailable"] = repr(exc)[:200]
        w.free()
    return out


def run_expert_parallel(R, ctx, torch, dist, stream, rank, world, steps=10):
    """One OLMoE-shaped MoE layer (hidden 2048, 64 experts, top-8, intermediate 1024, Q4_K), experts split 64/G per
    rank, T tokens per rank."""
    from runit_mac_b200 import parallel as P
    E, h, ff, k = 64, 2048, 1024, 8
    n_local = E // world
    rb = lambda kk: kk // 256 * 144
    gate, up = ctx.new_buffer(n_local * ff * rb(h)), ctx.new_buffer(n_local * ff * rb(h))
    down = ctx.new_buffer(n_local * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, n_local * ff, h), (up, n_local * ff, h), (down, n_local * h, ff))):
        R.fill_weights(ctx, 2, b, rows * (kk // 256), 77 + i + 10 * rank, 0.01)
    router = torch.randn(E, h, dtype=torch.float32, device="cuda") * 0.02
    if world > 1:
        dist.broadcast(router, 0)
    be = P.CudaBackend(R, ctx, torch)
    be.set_experts(router, gate, up, down, E, n_local, h, ff, k, False)
    out = {}
    for T in (1, 16):
        x = torch.randn(T, h, dtype=torch.float32, device="cuda")
        ms = _time_steps(torch, dist, stream, ctx, lambda: P.ep_moe_forward(be, dist, torch, x, E, k, False, world, rank), steps, world)
        out["T%d_per_rank" % T] = {"us_per_layer": ms * 1e3, "tokens_per_s_all_ranks": world * T / (ms * 1e-3)}
    if world > 1:
        try:
            fused = P.FusedEpDecodeMoe(R, ctx, torch, dist, router, gate, up, down, E, h, ff, k, False, world, rank, max_tokens=16)
            for T in (1, 16):
                x = torch.randn(T, h, dtype=torch.float32, device="cuda")
                dist.broadcast(x, 0)
                ms = _time_steps(torch, dist, stream, ctx, lambda: fused(x), steps, world)
                out["T%d_replicated_fused_peer_stores" % T] = {"us_per_layer": ms * 1e3, "tokens_per_s": T / (ms * 1e-3)}
        except Exception as exc:   # symmetric memory unavailable on this host: keep the NCCL figures
            out["fused_unavailable"] = repr(exc)[:200]
    for b in (gate, up, down):
        b.free()
    out["qwen3_shape_prefill"] = run_expert_parallel_prefill(R, ctx, torch, dist, stream, rank, world)
    return out


def run_ep_decode(R, ctx, torch, dist, rank, world):
    """Full OLMoE-shaped greedy decode (16 layers, hidden 2048, 64 experts top-8, Q4_K, 128-token prompt + 64 steps) with
    the experts split 64/G per rank and the MoE combine fused over peer memory; attention, router, embeddings and lm_head
    are replicated (same seeds on every rank), every rank decodes the same token stream."""
    from runit_mac_b200 import parallel as P
    import ctypes as C
    import time
    import numpy as np
    import torch.distributed._symmetric_memory as symm
    L, h, E, ff, k, V = 16, 2048, 64, 1024, 8, 50304
    nl = E // world
    rb = lambda kk: kk // 256 * 144
    shapes = {"wq": (L * h, h), "wk": (L * h, h), "wv": (L * h, h), "wo": (L * h, h), "lm_head": (V, h),
              "gate": (L * nl * ff, h), "up": (L * nl * ff, h), "down": (L * nl * h, ff)}
    dev = {}
    for i, (name, (rows, kk)) in enumerate(shapes.items()):
        dev[name] = ctx.new_buffer(rows * rb(kk))
        seed = 90001 + i + (1000 * rank if name in ("gate", "up", "down") else 0)
        R.fill_weights(ctx, R.FMT_Q4K, dev[name], rows * (kk // 256), seed, 0.01)
    for name, n, sig in (("tok_emb", V * h, 0.02), ("router", L * E * h, 0.02)):
        dev[name] = ctx.new_buffer(4 * n)
        R.fill_normal_f32(ctx, dev[name], n, 4242 + len(name), sig)
    ones = np.ones(L * h, np.float32)
    dev["attn_norm"], dev["ffn_norm"], dev["out_norm"] = ctx.buffer_from(ones), ctx.buffer_from(ones), ctx.buffer_from(ones[:h])
    ctx.flush()
    partial = symm.empty(2 * world * h, dtype=torch.float32, device="cuda")
    pad = symm.empty(64, dtype=torch.int32, device="cuda")
    pad.zero_()
    torch.cuda.synchronize()
    hq, hp = symm.rendezvous(partial, dist.group.WORLD), symm.rendezvous(pad, dist.group.WORLD)
    pq = (C.c_void_p * world)(*[int(p) for p in hq.buffer_ptrs])
    pp = (C.c_void_p * world)(*[int(p) for p in hp.buffer_ptrs])
    dist.barrier()
    torch.cuda.synchronize()
    cfg = R.ModelCfg(n_layers=L, hidden=h, n_heads=16, n_kv_heads=16, head_dim=128, vocab=V, n_experts=E, top_k=k, ff=ff,
                     max_seq=2048, renorm=0, eps=1e-5, theta=10000.0)
    model = R.Model(ctx, cfg, dev, ep=(world, rank, pq, pp))
    prompt = np.random.default_rng(1004).integers(0, V, 128).astype(np.int32)
    dist.barrier()
    model.generate_greedy(prompt, 8)
    dist.barrier()
    t0 = time.perf_counter()
    toks = model.generate_greedy(prompt, 64)
    dt_all = time.perf_counter() - t0
    dist.barrier()
    t0 = time.perf_counter()
    model.generate_greedy(prompt, 0)
    dt_prompt = time.perf_counter() - t0
    t = torch.tensor([dt_all, dt_prompt], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    same = torch.tensor(toks[127:].astype(np.int64), device="cuda")
    ref = same.clone()
    dist.broadcast(ref, 0)
    agree = torch.tensor([int(torch.equal(same, ref))], device="cuda")
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    dt_all, dt_prompt = float(t[0].item()), float(t[1].item())
    res = {"decode_tok_s": 64 / max(dt_all - dt_prompt, 1e-9), "prompt_tok_s": 128 / dt_prompt, "tokens_total_s": 192 / dt_all,
           "launches_per_token": int(model.launches_per_token), "experts_per_rank": nl, "ranks_agree_on_tokens": bool(agree.item()),
           "note": "one token stream over the whole group; wall clock (max over ranks) around one call of 192 recorded steps"}
    dist.barrier()
    model.close()
    for b in dev.values():
        b.free()
    return res


def run_expert_parallel_prefill(R, ctx, torch, dist, stream, rank, world, steps=5, T_total=4096):
    """Qwen3-MoE-shaped batched block (hidden 2048, 128 experts, top-8, intermediate 768, Q4_K -> bf16 tensor-core
    GEMMs), 4096 tokens in all (4096/G per rank), experts split 128/G per rank, Zipf(1.1) expert popularity,
    count-exchanged all-to-all dispatch and combine.  Reports the straggler's load beside the mean."""
    from runit_mac_b200 import parallel as P
    E, h, ff, k = 128, 2048, 768, 8
    n_local, T = E // world, T_total // world
    rb = lambda kk: kk // 256 * 144
    gate, up = ctx.new_buffer(n_local * ff * rb(h)), ctx.new_buffer(n_local * ff * rb(h))
    down = ctx.new_buffer(n_local * h * rb(ff))
    for i, (b, rows, kk) in enumerate(((gate, n_local * ff, h), (up, n_local * ff, h), (down, n_local * h, ff))):
        R.fill_weights(ctx, 2, b, rows * (kk // 256), 177 + i + 10 * rank, 0.01)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    p = 1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float64) ** 1.1
    idx = torch.multinomial((p / p.sum()).float().expand(T, E).contiguous(), k, replacement=False, generator=g).to(torch.int32)
    w = torch.rand(T, k, device="cuda", generator=g)
    x = torch.randn(T, h, device="cuda", generator=g)

    class GivenRouting(P.CudaBackend):
        def route(self, _x):
            return idx, w
    be = GivenRouting(R, ctx, torch, grouped_min_slots=256)
    be.set_experts(None, gate, up, down, E, n_local, h, ff, k, False)
    ms = _time_steps(torch, dist, stream, ctx, lambda: P.ep_moe_forward_counted(be, dist, torch, x, E, k, False, world, rank), steps, world)
    recv = torch.bincount((idx // n_local).flatten().long(), minlength=world).to(torch.float64)
    if world > 1:
        dist.all_reduce(recv)
    native = {}
    if world > 1:
        # the same block with the library's own exchange (peer stores, two barrier kernels, no host read), for both
        # expert placements; the routing is the given Zipf routing, so the router weights only have to reproduce it:
        # a one-hot router would need E = h columns; instead the block routes with its own router on x and the given
        # routing is left to the NCCL variant above.  The load figures below are the native block's own.
        try:
            router = torch.randn(E, h, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) * 0.02
            # a popularity that falls with the expert index, as in the Zipf routing above: a bias direction in x
            bias = torch.randn(h, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6))
            router = router + (2.5 / torch.arange(1, E + 1, device="cuda", dtype=torch.float32) ** 0.5)[:, None] * bias[None, :] / h
            xb = x + bias[None, :]
            # one GPU, all experts, all T_total tokens with the same router and token distribution: what the split has to beat
            gate1, up1 = ctx.new_buffer(E * ff * rb(h)), ctx.new_buffer(E * ff * rb(h))
            down1 = ctx.new_buffer(E * h * rb(ff))
            for i, (b, rows, kk) in enumerate(((gate1, E * ff, h), (up1, E * ff, h), (down1, E * h, ff))):
                R.fill_weights(ctx, 2, b, rows * (kk // 256), 377 + i, 0.01)
            x1 = torch.randn(T_total, h, device="cuda", generator=g) + bias[None, :]
            o1 = torch.empty(T_total, h, device="cuda")
            nb1 = R.moe_grouped_scratch_bytes(ctx, T_total, h, ff, E, k)
            s1 = ctx.new_buffer(nb1)
            ms_1 = _time_steps(torch, dist, stream, ctx, lambda: R.moe_layer_q4k_bf16(ctx, router, gate1, up1, down1, x1, None, o1, None, None,
                                                                                      s1, nb1, T_total, h, ff, E, k, 0), steps, world)
            native["one_gpu_all_tokens_same_router_ms"] = ms_1
            for b in (gate1, up1, down1, s1):
                b.free()
            for placement in (0, 1):
                epp = P.FusedEpPrefillMoe(R, ctx, torch, dist, router, gate, up, down, E, h, ff, k, False, world, rank, T, placement=placement)
                ms_n = _time_steps(torch, dist, stream, ctx, lambda: epp(xb), steps, world)
                _o, i_n, _w = epp(xb)
                ctx.flush()
                owner = (i_n % world) if placement else (i_n // n_local)
                rc = torch.bincount(owner.flatten().long(), minlength=world).to(torch.float64)
                dist.all_reduce(rc)
                native["placement_%s" % ("mod" if placement else "block")] = {
                    "ms_per_layer": ms_n, "tokens_per_s_all_ranks": T_total / (ms_n * 1e-3),
                    "slots_per_rank_max": float(rc.max().item()), "slots_per_rank_mean": float(rc.mean().item())}
                del epp
        except Exception as exc:
            native["unavailable"] = repr(exc)[:200]
    return {"native_peer_stores": native, "ms_per_layer": ms, "tokens_per_s_all_ranks": T_total / (ms * 1e-3), "tokens_per_rank": T,
            "slots_per_rank_max": float(recv.max().item()), "slots_per_rank_mean": float(recv.mean().item())}


def run_gguf_load(ctx, layers=2):
    """Model-file load path: a synthetic GGUF file with OLMoE-shaped packed tensors (Q4_K attention matrices and merged
    expert tensors of `layers` layers, ~0.44 GB) is written to a temporary directory, parsed and uploaded tensor by tensor."""
    import struct
    import tempfile
    from runit_mac_b200.gguf import parse_gguf_file
    E, h, ff = 64, 2048, 1024
    rng = np.random.default_rng(5)
    tensors = []
    for l in range(layers):
        for n in ("attn_q", "attn_k", "attn_v", "attn_output"):
            tensors.append(("blk.%d.%s.weight" % (l, n), [h, h], 12, h * (h // 256) * 144))
        for n, (kk, rows) in (("ffn_gate_exps", (h, ff)), ("ffn_up_exps", (h, ff)), ("ffn_down_exps", (ff, h))):
            tensors.append(("blk.%d.%s.weight" % (l, n), [kk, rows, E], 12, E * rows * (kk // 256) * 144))

    def gstr(b):
        return struct.pack("<Q", len(b)) + b
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), 1) + gstr(b"general.architecture") + struct.pack("<I", 8) + gstr(b"olmoe")
    off = 0
    for name, dims, dt, nbytes in tensors:
        head += gstr(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", dt, off)
        off += (nbytes + 31) // 32 * 32
    head += b"\0" * ((len(head) + 31) // 32 * 32 - len(head))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "synthetic.gguf")
        with open(path, "wb") as f:
            f.write(head)
            for _name, _dims, _dt, nbytes in tensors:
                f.write(rng.integers(0, 256, (nbytes + 31) // 32 * 32, dtype=np.uint8).tobytes())
        t0 = time.perf_counter()
        g = parse_gguf_file(path)
        t_parse = time.perf_counter() - t0
        total = sum(t.data_size() for t in g.tensors)
        bufs = [ctx.new_buffer(t.data_size()) for t in g.tensors]
        from runit_mac_b200 import gguf as G
        import ctypes as C
        t0 = time.perf_counter()
        for t, b in zip(g.tensors, bufs):
            G._check(G._api().runit_gguf_upload_tensor(ctx.handle, g._h, t.name.encode(), C.c_void_p(b.ptr), b.nbytes))
        ctx.flush()
        t_up = time.perf_counter() - t0
        g.close()
    for b in bufs:
        b.free()
    return {"file_gb": total / 1e9, "tensors": len(tensors), "parse_ms": t_parse * 1e3, "upload_s": t_up,
            "upload_gbs": total / 1e9 / t_up, "note": "file in the page cache; packed bytes uploaded as stored (wall clock)"}


def run_reference(args):
    """--impl reference: the CPU arm.  The reference's own code for this path is Rust + Apple Metal
    (no toolchain, no Metal here), so the timed implementation is the oracle port of its CPU formulas."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    vals = []
    # calibrate so that K+W steps stay within a few minutes: one step = 1 layer + lm_head per format
    for i in range(args.warmup + args.steps):
        gbs, t, desc, threads = cpu_sample([FMT_Q4K, FMT_Q4_0], cores, 2.0, layers_sample=1)
        if i >= args.warmup:
            vals.append((gbs, t))
    v = float(np.mean([g for g, _ in vals]))
    ms = float(np.mean([t for _, t in vals]) * 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen2.5-7b decode GEMV set, Q4_K + Q4_0, batch 1 (CPU: bounded sample per step)",
                   "l2": "inputs larger than any cache"},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of the workload (default: the full 28)")
    ap.add_argument("--tokens-per-step", type=int, default=25,
                    help="decode tokens (replays of the GEMV set of both formats) that make one step: 25 x 2.1 ms keeps the "
                         "timed region of 20 steps above one second")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--tune", default="", help="key=value[,key=value] kernel tuning knobs (experiments)")
    ap.add_argument("--no-extras", action="store_true", help="skip the MoE-layer / OLMoE-decode / sharded lm_head figures")
    ap.add_argument("--one", default="", help="fmt,m,k[,batch]: launch this one GEMV shape three times and exit (for ncu captures)")
    ap.add_argument("--block", default="", help="T: run the Qwen3-MoE-shaped batched MoE block on T tokens, print its figures and exit")
    ap.add_argument("--block-shape", default="qwen3", choices=("qwen3", "olmoe"), help="shape of the --block run")
    ap.add_argument("--decode", action="store_true", help="only the OLMoE-shaped greedy decode figure (tok/s), then exit")
    ap.add_argument("--prefill", default="", help="T: batched prefill of T tokens on a 2-layer OLMoE-shaped decoder, three times, then exit "
                                                  "(the small case for ncu captures of the prefill kernels)")
    ap.add_argument("--ffn", default="", help="T: the dense feed-forward block (Qwen2.5-7B shape) on T tokens, three times, then exit "
                                              "(the small case for ncu captures of the dense tcgen05 GEMM)")
    ap.add_argument("--shapes", action="store_true", help="per-shape GEMV table (one JSON line per shape) instead of the headline run")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import runit_mac_b200 as R

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        # plain peer loads/stores and plain NCCL rings only: no NVLink multicast objects are bound (see parallel.py)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()   # not the legacy default stream: command lists are recorded on it
    torch.cuda.set_stream(stream)
    ctx = R.Context(local, stream=stream.cuda_stream)   # kernels and torch events share this stream
    for kv in filter(None, args.tune.split(",")):
        k, v = kv.split("=")
        ctx.set_tuning(k, int(v))

    if args.one:
        f, m, k, *rest = args.one.split(",")
        fmt = {"q8_0": FMT_Q8_0, "q4_0": FMT_Q4_0, "q4k": FMT_Q4K, "q5_0": FMT_Q5_0, "q5k": FMT_Q5K, "q6k": FMT_Q6K}[f]
        m, k, batch = int(m), int(k), int(rest[0]) if rest else 1
        w = ctx.new_buffer(m * row_bytes(fmt, k))
        if fmt <= FMT_Q4K:
            R.fill_weights(ctx, fmt, w, m * (k // BLOCK[fmt][0]), 5, 0.01)
        else:       # no generator for these formats: any bytes stream at the same speed
            ctx.call("memset", w, 0x11, m * row_bytes(fmt, k))
        x, y = ctx.new_buffer(4 * k * batch), ctx.new_buffer(4 * m * batch)
        R.fill_normal_f32(ctx, x, k * batch, 3, 1.0)
        for _ in range(3):
            if fmt <= FMT_Q4K:
                R.gemv_batched_f32(ctx, fmt, w, x, y, None, m, k, batch)
            else:
                getattr(R, "gemv_%s_f32in_f32out" % f)(ctx, w, x, y, m, k)
        ctx.flush()
        print(json.dumps({"one": args.one, "launches": ctx.launches}))
        return
    if args.ffn:
        T = int(args.ffn)
        rbq = lambda kk: kk // 256 * 144
        dims = ((INTER, HIDDEN), (INTER, HIDDEN), (HIDDEN, INTER))
        wts = [ctx.new_buffer(r * rbq(kk)) for r, kk in dims]
        for i, (b, (r, kk)) in enumerate(zip(wts, dims)):
            R.fill_weights(ctx, R.FMT_Q4K, b, r * (kk // 256), 611 + i, 0.01)
        xd, od = torch.randn(T, HIDDEN, device="cuda"), torch.empty(T, HIDDEN, device="cuda")
        nbd = ctx.lib.runit_ffn_q4k_bf16_scratch_bytes(T, HIDDEN, INTER)
        sd = ctx.new_buffer(nbd)
        for _ in range(3):
            R.ffn_q4k_bf16(ctx, wts[0], wts[1], wts[2], xd, None, 0.0, xd, od, sd, nbd, T, HIDDEN, INTER)
        ctx.flush()
        print(json.dumps({"ffn_tokens": T, "finite": bool(torch.isfinite(od).all().item()), "launches": ctx.launches}))
        return
    if args.prefill:
        T = int(args.prefill)
        L, h, E, ff = 2, 2048, 64, 1024
        rbq = lambda kk: kk // 256 * 144
        shapes = {"wq": (L * h, h), "wk": (L * h, h), "wv": (L * h, h), "wo": (L * h, h), "gate": (L * E * ff, h),
                  "up": (L * E * ff, h), "down": (L * E * h, ff), "lm_head": (50304, h)}
        dev = {}
        for i, (name, (rows, kk)) in enumerate(shapes.items()):
            dev[name] = ctx.new_buffer(rows * rbq(kk))
            R.fill_weights_q4k_zero_mean(ctx, dev[name], rows * (kk // 256), 31 + i, 6e-5)
        for name, n, sig in (("tok_emb", 50304 * h, 1.0), ("router", L * E * h, 0.02)):
            dev[name] = ctx.new_buffer(4 * n)
            R.fill_normal_f32(ctx, dev[name], n, 77 + len(name), sig)
        ones = np.ones(L * h, np.float32)
        dev["attn_norm"], dev["ffn_norm"], dev["out_norm"] = ctx.buffer_from(ones), ctx.buffer_from(ones), ctx.buffer_from(ones[:h])
        cfg = R.ModelCfg(n_layers=L, hidden=h, n_heads=16, n_kv_heads=16, head_dim=128, vocab=50304, n_experts=E, top_k=8, ff=ff,
                         max_seq=max(2048, T), renorm=0, eps=1e-5, theta=10000.0)
        model = R.Model(ctx, cfg, dev)
        pr = np.random.default_rng(T).integers(0, 50304, T).astype(np.int32)
        toks = [model.prefill(pr) for _ in range(3)]
        print(json.dumps({"prefill_tokens": T, "layers": L, "next_token": toks, "launches": ctx.launches}))
        model.close()
        return
    if args.shapes:
        return run_shapes(R, ctx, torch, stream)
    if args.decode:
        ex = run_extras(R, ctx, torch, dist, stream, rank, world, args, decode_only=True)
        print(json.dumps(ex["olmoe_decode_q4k"]), flush=True)
        return
    if args.block:
        if args.block_shape == "olmoe":     # BASELINE configs[2]: 64 experts, intermediate 1024, routing without skew
            print(json.dumps(run_block(R, ctx, torch, stream, T=int(args.block), reps=max(args.steps // 2, 3), E=64, ff=1024, zipf_s=0.0,
                                       name="olmoe")), flush=True)
        else:
            print(json.dumps(run_block(R, ctx, torch, stream, T=int(args.block), reps=max(args.steps // 2, 3))), flush=True)
        return
    sets = [GemvSet(R, ctx, FMT_Q4K, 1002 + rank, args.layers), GemvSet(R, ctx, FMT_Q4_0, 2002 + rank, args.layers)]
    bytes_fmt = [pass_bytes(s.fmt, args.layers) for s in sets]
    step_bytes = sum(bytes_fmt)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Every op of a pass is recorded once (command list) and replayed: the timed region contains no
    # per-op host work, as in the reference where a token's dispatches sit in one command buffer.
    for s_ in sets:
        s_.run()
    ctx.flush()
    graphs = []
    for s_ in sets:
        ctx.graph_begin()
        s_.run()
        graphs.append(ctx.graph_end())
    launches_per_pass = [args.layers * LAUNCHES_PER_LAYER + 1] * len(sets)

    TPS = max(1, args.tokens_per_step)

    def step():
        for _ in range(TPS):
            for g in graphs:
                g.launch()

    for _ in range(args.warmup):
        step()
    barrier()

    # ── timed region: inputs resident in HBM ──
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    sub = [[torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)] for _ in range(args.steps * TPS * len(sets))]
    barrier()
    ev[0].record(stream)
    for i in range(args.steps):
        for tok in range(TPS):
            for j, g in enumerate(graphs):
                a, b = sub[(i * TPS + tok) * len(sets) + j]
                a.record(stream)
                g.launch()
                b.record(stream)
    ev[1].record(stream)
    barrier()
    launches = args.steps * TPS * sum(launches_per_pass)
    ms = ev[0].elapsed_time(ev[1])
    fmt_ms = [0.0] * len(sets)
    for i in range(args.steps * TPS):
        for j in range(len(sets)):
            a, b = sub[i * len(sets) + j]
            fmt_ms[j] += a.elapsed_time(b)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * step_bytes * TPS * args.steps / (ms_max * 1e-3) / 1e9

    # ── end to end through the public call with HOST buffers: x from pinned memory in, logits out ──
    hx = torch.randn(HIDDEN, dtype=torch.float32).pin_memory()
    hlogits = torch.empty(VOCAB, dtype=torch.float32).pin_memory()
    lib, h = ctx.lib, ctx.handle

    def e2e_step():
        for _ in range(TPS):
            for s_, g in zip(sets, graphs):
                lib.runit_memcpy_h2d(h, s_.xn.ptr, hx.data_ptr(), 4 * HIDDEN)
                g.launch()
                lib.runit_memcpy_d2h(h, hlogits.data_ptr(), s_.logits.ptr, 4 * VOCAB)
                ctx.flush()   # the caller reads the logits before the next token

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        e2e_step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * step_bytes * TPS * args.steps / (float(t.item()) * 1e-3) / 1e9
    if rank == 0 and sampler.proc is not None:
        # a short run can end before nvidia-smi has printed its first line: keep the same load running (untimed) until
        # a few samples exist, so that the clock record is taken under load and never empty
        t_wait = time.perf_counter()
        while len(sampler.rows) < 3 and time.perf_counter() - t_wait < 3.0:
            step()
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None   # sampled over both timed regions
    # side figures on the same resident weights (outside the timed regions): batch 8, and the folded command list
    try:
        b8_gbs, b8_launches = measure_batch8(R, ctx, torch, stream, sets[0])
        b8_q40, _ = measure_batch8(R, ctx, torch, stream, sets[1])
        folded = measure_folded(R, ctx, torch, stream, sets[0])
    except Exception as exc:
        b8_gbs = b8_q40 = b8_launches = None
        folded = {"error": repr(exc)[:200]}

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        # dominant kernel: the Q4_K staged GEMV; its launches = the Q4_K sub-pass (8 per layer incl. one
        # tiny silu-free set: 7 GEMVs per layer + lm_head)
        q4k_launches = launches_per_pass[0]
        q4k_ms = fmt_ms[0] / (args.steps * TPS)
        achieved = bytes_fmt[0] / (q4k_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen2.5-7b decode GEMV set (28 layers: fused q|k|v, o, fused gate/up, down; + lm_head), "
                                   "Q4_K pass + Q4_0 pass, batch 1, f32 activations",
                       "arithmetic": "f32 activations in, f32 accumulation and output; the 4-bit weights meet 16-bit block-fixed-point "
                                     "copies of the activations (per 32-block, power-of-two scale) on the integer tensor cores: "
                                     "within 2e-4 of the output scale of an exact f32 product (bar 1e-3)",
                       "layers": args.layers, "tokens_per_step": TPS, "bytes_per_step": step_bytes * TPS,
                       "l2": "inputs larger than L2: every matrix is a distinct instance, %.1f GB streamed per token" % (step_bytes / 1e9)},
            "roofline": {"bound": "hbm", "kernel": "gemv_staged_kernel<Q4_K,batch 1,integer tensor-core MMAs>", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                         "traffic": NCU_TRAFFIC_RATIO * bytes_fmt[0] / q4k_launches,
                         "traffic_note": "ncu capture of the 152064x3584 Q4_K launch (profiles/gemv_q4k_lm_head_152064x3584_ncu.md): dram read "
                                         "306.80 MB + write 4.71 MB for 307.18 MB algorithmic = x1.0141; scaled to the average launch of "
                                         "the pass (weights are streamed once by every launch, so traffic grows with the bytes); the "
                                         "launches that dominate the pass were captured as well "
                                         "(profiles/gemv_q4k_ffn_shapes_traffic_b200.md): 18944x3584 38.24 MB and 3584x18944 38.30 MB of "
                                         "DRAM traffic for 38.28 MB algorithmic = x1.00",
                         "bytes_per_launch": bytes_fmt[0] / q4k_launches, "launches_per_token": q4k_launches,
                         "avg_launch_us": q4k_ms * 1e3 / q4k_launches},
            "per_format": {"q4k_gbs": achieved, "q4_0_gbs": bytes_fmt[1] / (fmt_ms[1] / (args.steps * TPS) * 1e-3) / 1e9},
            "per_batch": {"1": {"q4k_gbs": achieved, "q4_0_gbs": bytes_fmt[1] / (fmt_ms[1] / (args.steps * TPS) * 1e-3) / 1e9},
                          "8": {"q4k_gbs": b8_gbs, "q4_0_gbs": b8_q40, "frac_of_peak_q4k": (b8_gbs / peak) if b8_gbs else None,
                                "launches_per_token": b8_launches,
                                "note": "same weights, 8 activation rows per GEMV, weights counted once; untimed side run of 5 replays"}},
            "folded_command_list_q4k": folded,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": TPS * 2 * 4 * HIDDEN, "d2h_bytes_per_step": TPS * 2 * 4 * VOCAB},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "extras": {},
        }
        if not args.no_cpu and world == 1:
            gbs, tsec, desc, threads = cpu_sample([FMT_Q4K, FMT_Q4_0], os.cpu_count() or 1, 12.0, layers_sample=2)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc,
                                    "seconds": tsec}
        else:
            line["cpu_baseline"] = None
    # The extras (other rows of the path; at N > 1 they use collectives) must never cost the headline line: if they do
    # not finish in time, rank 0 prints the line without them and the extras stop at their next checkpoint, so that the
    # ranks leave in order (process group destroyed, contexts closed).  Only if a rank is still stuck two minutes later
    # (a collective whose peer is gone) does the process end itself: every wait on peer memory in this library is
    # bounded and symmetric memory is not bound to a multicast object (see runit_mac_b200/parallel.py), so no GPU is
    # left waiting on the rank that leaves.
    state = {"printed": False, "stop": False}
    lock = threading.Lock()

    def emit(extras):
        with lock:
            if rank == 0 and not state["printed"]:
                line["extras"] = extras
                if world > 1 and isinstance(extras, dict):
                    # the paths that are partitioned over the GPUs (the headline value is N replicas, weak scaling)
                    lh = (extras.get("lm_head_row_sharded") or {}).get("q4k") or {}
                    ep = extras.get("olmoe_decode_q4k_expert_parallel") or {}
                    pf = ((extras.get("moe_expert_parallel") or {}).get("qwen3_shape_prefill") or {})
                    line["partitioned"] = {"lm_head_q4k_row_sharded_us": lh.get("us_per_call_fused_peer_stores", lh.get("us_per_call")),
                                           "lm_head_q4k_row_sharded_gbs": lh.get("aggregate_gbs_fused", lh.get("aggregate_gbs")),
                                           "olmoe_decode_expert_parallel_tok_s": ep.get("decode_tok_s"),
                                           "lm_head_q4k_greedy_pairs_us": lh.get("us_per_call_greedy_pairs"),
                                           # the library's own exchange (peer stores), the better of the two expert placements,
                                           # beside one GPU running all tokens and all experts with the same router
                                           "qwen3_prefill_block_expert_parallel_ms": min(
                                               [v["ms_per_layer"] for v in (pf.get("native_peer_stores") or {}).values()
                                                if isinstance(v, dict) and "ms_per_layer" in v] or [pf.get("ms_per_layer")]),
                                           "qwen3_prefill_block_one_gpu_ms": (pf.get("native_peer_stores") or {}).get("one_gpu_all_tokens_same_router_ms"),
                                           "qwen3_prefill_block_nccl_torch_ms": pf.get("ms_per_layer"),
                                           "scaling": "strong (one workload split over the ranks)"}
                print(json.dumps(line), flush=True)
            state["printed"] = True

    def give_up():
        state["stop"] = True
        emit({"error": "extras did not finish within %d s" % EXTRAS_LIMIT_S})
        last = threading.Timer(120, lambda: os._exit(0))
        last.daemon = True
        last.start()
    watchdog = threading.Timer(EXTRAS_LIMIT_S, give_up)
    watchdog.daemon = True
    watchdog.start()
    extras = {}
    if not args.no_extras:
        try:
            extras = run_extras(R, ctx, torch, dist, stream, rank, world, args, stop=lambda: state["stop"])
        except Exception as exc:   # the extras never invalidate the headline line
            extras = {"error": repr(exc)[:300]}
    watchdog.cancel()
    emit(extras)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
