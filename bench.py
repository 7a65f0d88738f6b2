#!/usr/bin/env python
"""Benchmark of the quantized MOSS-Image DiT denoising step on B200.

python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

Default workload `step1024`: the full INT8 'high'-tier denoising step at 1024^2 (42 blocks of d=3072, 24x128 heads, MLP
12288, CFG batch 2 = two 8192-token sequences per image), one image per GPU (no collective: weak scaling). One "step" is
one pass of all blocks over the image's 16384 tokens through the C ABI (b2_dit_step). Other workloads:
  block1024            one block on one 8192-token sequence
  step1024_cfgsplit    the step with the CFG halves on two GPUs (N = 2, strong scaling against step1024 at N = 1)
  step2048             the 2048^2 step (2 x 20480 tokens) on one GPU through b2_dit_step: the base of step2048_ulysses
  step2048_ulysses     the 2048^2 step (two 20480-token sequences) with Ulysses sequence parallelism over N GPUs
  turbo1024            the step with grouped 4-bit weights (W4A8), one image per GPU
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, HEADS = 3072, 24
METRIC = "dit_ms_per_step_1024"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="step1024")
    p.add_argument("--blocks", type=int, default=42)
    p.add_argument("--ffn", type=int, default=12288)
    p.add_argument("--no-profile", action="store_true", help="skip the per-kernel roofline pass and the CPU baseline")
    p.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's own CUDA kernels on this GPU")
    p.add_argument("--no-graph", action="store_true", help="enqueue the step's kernels directly instead of replaying a CUDA graph")
    p.add_argument("--no-ulysses", action="store_true", help="N >= 2: skip the sequence-parallel 2048^2 record added to the line")
    return p.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        time.sleep(0.05)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------------- CPU arm

def cpu_sample(ffn: int, block_tokens: int, attn_tokens: int, threads: int):
    """Times the oracle (a CPU port of the reference's arithmetic) on a bounded sample: one block on `block_tokens`
    tokens (GEMMs and element-wise work, linear in tokens) and the 8-bit attention of one `attn_tokens`-token sequence
    over 24 heads (quadratic in tokens). Returns (seconds_block, seconds_attention)."""
    import numpy as np
    from oracle import oracle_lib as orc
    orc.set_threads(threads)
    rng = np.random.default_rng(0)

    def rb(shape, s=1.0, m=0.0):
        v = (m + rng.standard_normal(shape) * s).astype(np.float32)
        return ((v.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)

    w = {"norm1": rb(D, 0.1, 1.0), "norm2": rb(D, 0.1, 1.0), "q_norm": rb(128, 0.1, 1.0), "k_norm": rb(128, 0.1, 1.0)}
    for name, (n, k) in dict(qkv=(3 * D, D), o=(D, D), up=(2 * ffn, D), down=(D, ffn)).items():
        w[name] = (rng.integers(-127, 128, (n, k), dtype=np.int8), (rng.random(n).astype(np.float32) + 0.5) * 1e-3)
    x, mod = rb((block_tokens, D)), rb(6 * D, 0.1)
    rope = orc.moss_rope_table(1, 1, block_tokens - 1)
    t0 = time.perf_counter()
    orc.block_quant(x, mod, rope, w, np.array([0, block_tokens], np.int32), block_tokens)
    t_block = time.perf_counter() - t0
    qkv = rb((attn_tokens, 3 * HEADS * 128))
    t0 = time.perf_counter()
    orc.attention_q8(qkv, np.array([0, attn_tokens], np.int32), HEADS, attn_tokens, 0.08838834764831845)
    t_attn = time.perf_counter() - t0
    # The block sample contains a (tiny) attention over block_tokens keys; it is left in: < 0.1 % of the sample.
    return t_block, t_attn


def cpu_extrapolate(t_block, t_attn, block_tokens, attn_tokens, seq_len, seqs, blocks):
    """ms per step of `blocks` blocks over `seqs` sequences of `seq_len` tokens, from the sample's two rates."""
    linear = t_block / block_tokens * (seq_len * seqs)
    quad = t_attn * (seq_len / attn_tokens) ** 2 * seqs
    return (linear + quad) * blocks * 1e3


def workload_shape(name: str, world: int):
    """(sequence length, sequences per rank-step, tier name) of a workload."""
    if name == "block1024":
        return 8192, 1
    if name in ("step1024", "turbo1024"):
        return 8192, 2
    if name == "step1024_cfgsplit":
        return 8192, 1
    if name in ("step2048", "step2048_ulysses"):
        return 20480, 2
    raise SystemExit(f"unknown workload {name}")


TIER_NAMES = ["int8", "w4a4_via_int8", "w4a8"]


def workload_config(args, world: int, launch: str):
    """The `config` object of the JSON line: the same for this library's arm and for the reference arm."""
    seq_len, seqs = workload_shape(args.workload, world)
    n_blocks = 1 if args.workload == "block1024" else args.blocks
    strong = args.workload == "step1024_cfgsplit"
    return {"workload": args.workload, "blocks": n_blocks, "d": D, "heads": HEADS, "ffn": args.ffn,
            "tokens_per_gpu_step": seq_len * seqs, "sequences": [seq_len] * seqs,
            "tier": TIER_NAMES[2 if args.workload == "turbo1024" else 0], "attention": "int8_fp8_f32acc",
            "parallelism": "cfg-split2" if strong else f"image-dp{world}",
            "l2": "inputs larger than L2 (block weights stream from HBM every step)", "launch": launch}


CPU_SAMPLE_TOKENS, CPU_SAMPLE_KEYS = 256, 1536  # both CPU legs time the same bounded sample


def run_reference(args, rank, world):
    """The reference arm: the reference engine has no CPU implementation of the quantized block and ships no sm_100
    kernel, so its CPU path for this metric is the oracle port of its arithmetic, run with every host thread on a bounded
    sample per step and extrapolated to the full step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    seq_len, seqs = workload_shape(args.workload, 1)
    blocks = 1 if args.workload == "block1024" else args.blocks
    bt, at = CPU_SAMPLE_TOKENS, CPU_SAMPLE_KEYS
    vals = []
    for i in range(args.warmup + args.steps):
        tb, ta = cpu_sample(args.ffn, bt, at, threads)
        if i >= args.warmup:
            vals.append(cpu_extrapolate(tb, ta, bt, at, seq_len, seqs, blocks))
    v = statistics.mean(vals)
    sample = (f"per step: one block on {bt} tokens + 8-bit attention of one {at}-token sequence x 24 heads, extrapolated "
              f"(linear part by tokens, attention by tokens^2) to {blocks} blocks x {seqs} x {seq_len} tokens; a CPU port of "
              "the reference's arithmetic (the reference has no CPU implementation of the quantized block)")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": v, "higher_is_better": False,
            "scaling": "strong" if args.workload == "step1024_cfgsplit" else "weak", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic", "extrapolated": True,
            "config": workload_config(args, max(1, args.gpus), "cuda graph replay"),
            "cpu_baseline": {"value": v, "unit": "ms", "cores": threads, "kind": "port", "sample": sample, "extrapolated": True},
            "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------- GPU arm

def reference_kernels_on_this_gpu(torch, ops, keep, x, x0, mod, rope, cu, seq_len, L, F):
    """The same step over the reference's own CUDA kernels (its mma.sync INT8 GEMMs and attention, compiled for sm_100a
    into oracle/_ref/libref_cuda.so), sequenced as its run_block_quant does, on this GPU with the same weights and
    inputs: what the reference would do here. Reported beside the CPU baseline; None where that build is absent."""
    from oracle import ref_cuda_lib as refk
    if not refk.available():
        return None
    rb = refk.RefBlock(L, cu, seq_len, D, F, HEADS)

    def ref_step():
        x.copy_(x0)
        for w, _ in keep:
            rb.run(x, mod, rope, w, ops.SM_SCALE)

    ref_step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 2
    e0.record()
    for _ in range(n):
        ref_step()
    e1.record()
    torch.cuda.synchronize()
    return {"value": e0.elapsed_time(e1) / n, "unit": "ms", "kind": "reference CUDA kernels built for sm_100a, device-timed",
            "steps": n, "blocks": len(keep), "per_kernel": profile_kernels(ops, torch, L, F, keep[0][0], iters=4, ref=refk)}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, MB) of the four GEMM launches of one block at 16384 tokens,
# F = 12288, from one ncu capture of exactly those launches. They describe the GEMM kernel as of GEMM_DRAM_COMMIT; a change
# to its tile order or tile shape needs a new capture.
GEMM_DRAM_MB = {"qkv": 83.3 + 255.0, "o": 160.6 + 54.2, "up_gate": 204.0 + 363.1, "down": 606.3 + 86.9}
GEMM_DRAM_COMMIT = "7f7af74"


def gemm_sites(L, F):
    return [("qkv", 3 * D, D, "plain"), ("o", D, D, "gated"), ("up_gate", 2 * F, D, "situ"), ("down", D, F, "gated")]


def profile_kernels(ops, torch, L, F, w, iters=8, ref=None):
    """Per-kernel CUDA-event timings of one block's kernels on L tokens, each launch timed alone after an L2 flush.
    With `ref` (oracle/ref_cuda_lib) the same launches go to the reference's own CUDA kernels instead."""
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    xs = torch.rand(L, device=dev) * 1e-2
    res = torch.randn((L, D), device=dev).to(torch.bfloat16)
    gate = torch.randn(D, device=dev).to(torch.bfloat16)
    out = {}

    def timed(fn):
        ts = []
        for i in range(iters + 2):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            if i >= 2:
                ts.append(e0.elapsed_time(e1))
        return statistics.mean(ts)

    for name, n, k, epi in gemm_sites(L, F):
        xq = torch.randint(-128, 128, (L, k), dtype=torch.int8, device=dev)
        wq, ws = w[name]
        if epi == "plain":
            o = torch.empty((L, n), dtype=torch.bfloat16, device=dev)
            ms = timed((lambda: ref.int8_gemm(xq, xs, wq, ws, o)) if ref else (lambda: ops.int8_gemm(xq, xs, wq, ws, out=o)))
        elif epi == "gated":
            ms = timed((lambda: ref.int8_gemm_gated_residual(xq, xs, wq, ws, gate, res)) if ref
                       else (lambda: ops.int8_gemm_gated_residual(xq, xs, wq, ws, gate, res)))
        else:
            o = torch.empty((L, n // 2), dtype=torch.bfloat16, device=dev)
            ms = timed((lambda: ref.int8_gemm_situ_glu(xq, xs, wq, ws, o)) if ref
                       else (lambda: ops.int8_gemm_situ_glu(xq, xs, wq, ws, out=o)))
        out[name] = {"ms": ms, "tops": 2.0 * L * n * k / ms / 1e9}
        del xq
    x = torch.randn((L, D), device=dev).to(torch.bfloat16)
    q = torch.empty((L, D), dtype=torch.int8, device=dev)
    s = torch.empty(L, dtype=torch.float32, device=dev)
    v = torch.randn(D, device=dev).to(torch.bfloat16)
    ms = timed((lambda: ref.rms_norm_modulate_rotate_quantize(x, v, v, v, q, s)) if ref
               else (lambda: ops.rms_norm_modulate_rotate_quantize(x, v, v, v, q=q, scale=s)))
    out["norm_rotate_quantize"] = {"ms": ms, "gbs": 3.0 * L * D / ms / 1e6}
    ms = timed((lambda: ref.rotate_quantize(x, q, s)) if ref else (lambda: ops.rotate_quantize(x, q=q, scale=s)))
    out["rotate_quantize"] = {"ms": ms, "gbs": 3.0 * L * D / ms / 1e6}
    xf = torch.randn((L, F), device=dev).to(torch.bfloat16)
    qf = torch.empty((L, F), dtype=torch.int8, device=dev)
    ms = timed((lambda: ref.rotate_quantize(xf, qf, s)) if ref else (lambda: ops.rotate_quantize(xf, q=qf, scale=s)))
    out["rotate_quantize_ffn"] = {"ms": ms, "gbs": 3.0 * L * F / ms / 1e6}
    del xf, qf
    # 8-bit attention of the step's sequences (pre-pass with fused QK-norm + RoPE, then the attention kernel).
    qkv = torch.randn((L, 3 * D), device=dev).to(torch.bfloat16)
    views = [qkv.as_strided((L, HEADS, 128), (3 * D, 128, 1), i * D) for i in range(3)]
    o = torch.empty((L, HEADS, 128), dtype=torch.bfloat16, device=dev)
    seqs = max(1, L // 8192)
    sl = L // seqs
    cu = torch.tensor([i * sl for i in range(seqs + 1)], dtype=torch.int32, device=dev)
    rope = ops.moss_rope_table(64, 64, sl - 4096).repeat(seqs, 1).contiguous() if sl >= 4096 else ops.moss_rope_table(1, 1, sl - 1).repeat(seqs, 1).contiguous()
    qn = torch.ones(128, device=dev).to(torch.bfloat16)
    if ref:
        o2 = o.view(L, D)
        wsa = torch.empty(max(256, ref.attention_workspace_bytes(L, seqs, sl, HEADS)), dtype=torch.uint8, device=dev)
        ms = timed(lambda: ref.attention_q8(qkv, HEADS, o2, cu, sl, ops.SM_SCALE, wsa, (qn, qn, rope)))
    else:
        _, wsa = ops.attention_q8(*views, o, cu, cu, sl, ops.SM_SCALE, norm_rope=(qn, qn, rope))
        ms = timed(lambda: ops.attention_q8(*views, o, cu, cu, sl, ops.SM_SCALE, workspace=wsa, norm_rope=(qn, qn, rope)))
    out["attention_q8"] = {"ms": ms, "tops": 4.0 * seqs * sl * sl * D / ms / 1e9}
    if ref:
        return out
    ms = timed(lambda: ops.attention_q8_preprocess(*views, cu, cu, sl, workspace=wsa, norm_rope=(qn, qn, rope)))
    out["attention_prepass"] = {"ms": ms, "gbs": (9.0 * L * D + 256.0 * L) / ms / 1e6}
    return out


def single_gpu_step_ms(torch, ops, synth, seq_lens, blocks, F, steps, warmup, tier=0):
    """ms per step of the whole step on THIS GPU alone through b2_dit_step (CUDA-graph replay): the base the
    sequence-parallel record is compared with, and the grouped 4-bit tier's figure beside the INT8 headline."""
    L, seq_len = sum(seq_lens), max(seq_lens)
    keep, bws = [], []
    for b in range(blocks):
        w = synth.block_weights(D, F, 3000 + 100 * b, tier=tier)
        lin = {n: (ops.make_w4(w[n][0], w[n][1], 64, w[n][2]) if tier == ops.TIER_W4A8 else w[n]) for n in ("qkv", "o", "up_gate", "down")}
        keep.append((w, lin))
        bws.append(ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], lin["qkv"], lin["o"], lin["up_gate"], lin["down"]))
    x0 = synth.activations(L, D, 1003)
    mod = synth.modulation(D, 2001)
    grid = 128 if seq_len > 16384 else 64
    rope = torch.cat([ops.moss_rope_table(grid, grid, s - grid * grid) for s in seq_lens]).contiguous()
    cu = synth.cu_seqlens(seq_lens)
    run = ops.block_run(L, cu, seq_len, D=D, F=F, heads=HEADS, tier=tier)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    x = x0.clone()
    bufs = ops.block_buffers(x, mod, rope, ws)
    ops.dit_step(bws, bufs, run)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.dit_step(bws, bufs, run)
    for _ in range(max(warmup, 3)):
        x.copy_(x0)
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        x.copy_(x0)
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def forward_shell_ms(torch, ops, synth, grid, text_len, rows, blocks, F, steps):
    """ms per call of the whole forward (b2_dit_forward: modulation vectors from the time vector, video embedding, RoPE
    tables, the block loop, head) on `rows` sequences of grid x grid video tokens + text_len text tokens, launched
    eagerly (no graph), and the same call with zero blocks: the shell's own cost."""
    import numpy as np
    bws, keep = [], []
    for b in range(blocks):
        w = synth.block_weights(D, F, 3000 + 100 * b)
        keep.append(w)
        bws.append(ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], w["qkv"], w["o"], w["up_gate"], w["down"]))
    g = torch.Generator(device="cuda").manual_seed(77)
    t = lambda *shape, s=0.02: (torch.randn(*shape, device="cuda", generator=g) * s).to(torch.bfloat16)
    f = lambda *shape, s=0.3: torch.randn(*shape, device="cuda", generator=g) * s
    parts = (t(6 * D, D), f(6 * D), t(2 * D, D), f(2 * D), t(D, 128, s=0.09), t(D, s=0.1), t(D, s=0.1) + 1, t(128, D), t(128, s=0.1))
    latents = torch.randn(1, 128, grid, grid, device="cuda", generator=g)
    texts = [torch.randn(text_len, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(rows)]
    tv = np.random.default_rng(5).normal(0, 1, D).astype(np.float32)
    out = {}
    for name, use in (("forward", bws), ("shell_only", [])):
        model = ops.DitModel(use, F, *parts)
        ws = None
        for _ in range(2):
            _, ws = ops.dit_forward(model, latents, tv, [(x, 0, 0) for x in texts], workspace=ws)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            ops.dit_forward(model, latents, tv, [(x, 0, 0) for x in texts], workspace=ws)
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / steps
        if name == "forward":
            # A launch-bound shape (a 256 x 256 image: 256 video + 64 text tokens per row) eagerly and through the step-graph
            # cache (b2_dit_forward_graphed), both on a stream of their own.
            small = torch.randn(1, 128, 16, 16, device="cuda", generator=g)
            rows_small = [(x[:64], 0, 0) for x in texts]
            side = torch.cuda.Stream()
            graphs = ops.DitGraphs(capacity=2)
            with torch.cuda.stream(side):
                for key, cache in (("forward256_eager_ms", None), ("forward256_graph_ms", graphs)):
                    outs_s = ws_s = None
                    for _ in range(3):
                        outs_s, ws_s = ops.dit_forward(model, small, tv, rows_small, workspace=ws_s, outs=outs_s, graphs=cache)
                    side.synchronize()
                    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s0.record(side)
                    for _ in range(10):
                        ops.dit_forward(model, small, tv, rows_small, workspace=ws_s, outs=outs_s, graphs=cache)
                    s1.record(side)
                    side.synchronize()
                    out[key] = s0.elapsed_time(s1) / 10
            out["forward256_graph_stats"] = graphs.stats()
            graphs.close()
    return out


def load_file_record(torch, ops, synth, F, blocks=2):
    """Weight ingestion: a synthetic INT8 file of `blocks` blocks (official names and configs) written to the temporary
    directory, then opened, checked and copied to the device by b2_dit_file_open; the second open reads from the page cache."""
    import tempfile
    import time
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "dit_int8.safetensors")
        size = synth.write_int8_dit_file(path, blocks, F)
        ms = []
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            f = ops.DitFile(path)
            torch.cuda.synchronize()
            ms.append((time.perf_counter() - t0) * 1e3)
            assert f.num_blocks == blocks and f.tier == ops.TIER_INT8
            f.close()
    return {"file_bytes": size, "blocks": blocks, "open_ms": ms[1], "gb_per_s": size / ms[1] / 1e6, "first_open_ms": ms[0]}


def ulysses_record(torch, dist, ops, synth, args, rank, world):
    """N >= 2: the 2048^2 step (two 20480-token sequences) over all N ranks (groups x sequence parallel), the same step on
    rank 0's GPU alone, the speed-up and the exchange time the step does not hide. Every rank takes part; rank 0 returns
    the record."""
    from owoinfer_b200 import parallel
    steps, warmup = min(args.steps, 5), 3
    ms, rec = parallel.measure_ulysses(rank, world, args.blocks, args.ffn, steps, warmup)
    base = None
    if rank == 0:
        base = single_gpu_step_ms(torch, ops, synth, rec["sequences"], args.blocks, args.ffn, min(args.steps, 3), 3)
        torch.cuda.empty_cache()
    dist.barrier()
    if rank != 0:
        return None
    rec.update({"workload": "step2048_ulysses", "metric": "dit_ms_per_step_2048", "n_gpus": world, "ms_per_step": ms,
                "steps": steps, "warmup": warmup, "single_gpu_ms_per_step": base, "speedup_vs_single_gpu": base / ms,
                "exposed_exchange_frac": None if rec["exposed_exchange_ms"] is None else rec["exposed_exchange_ms"] / ms})
    return rec


def roofline_record(prof, L, F, seq_len, seqs):
    """The `roofline` object: every kernel family of one block with its bound, its achieved rate from the launch times
    measured in this run (CUDA events, each launch alone after an L2 flush) and its share of the block; the top-level
    figures are the tensor-bound kernels (the four GEMM sites and the attention kernel, 85-90 % of a block) taken
    together, i.e. weighted by their time."""
    pk = peaks()
    tensor_peak, hbm_peak = 2.0 * pk["bf16"], pk["hbm_gbs"]
    src = f"{pk['source']} peaks: 2 x bf16 burst for the 8-bit tensor work (no INT8/FP8 figure is measured; nominal dense 4500), copy bandwidth for HBM"
    gemm_ops = sum(2.0 * L * n * k for _, n, k, _ in gemm_sites(L, F))
    gemm_ms = sum(prof[name]["ms"] for name, *_ in gemm_sites(L, F))
    attn_ops = 4.0 * seqs * seq_len * seq_len * D
    pre_ms = prof["attention_prepass"]["ms"]
    attn_ms = max(prof["attention_q8"]["ms"] - pre_ms, 1e-6)
    pre_bytes = 9.0 * L * D + 256.0 * L
    rows = [
        ("int8_gemm_kernel (qkv, o, up_gate, down)", "tensor", gemm_ops / gemm_ms / 1e9, gemm_ms),
        ("attention_kernel", "tensor", attn_ops / attn_ms / 1e9, attn_ms),
        ("attention pre-pass (norm_rope_quant_q, stats, finalize, quant_kv)", "hbm", pre_bytes / pre_ms / 1e6, pre_ms),
        ("rotate_quantize_kernel with the norm prologue (two per block)", "hbm", prof["norm_rotate_quantize"]["gbs"],
         2.0 * prof["norm_rotate_quantize"]["ms"]),
        ("rotate_quantize_kernel (attention output, FFN hidden)", "hbm",
         3.0 * L * (D + F) / (prof["rotate_quantize"]["ms"] + prof["rotate_quantize_ffn"]["ms"]) / 1e6,
         prof["rotate_quantize"]["ms"] + prof["rotate_quantize_ffn"]["ms"]),
    ]
    block_ms = sum(r[3] for r in rows)
    kernels = [{"name": n, "bound": b, "achieved": a, "peak": tensor_peak if b == "tensor" else hbm_peak,
                "unit": "TOP/s" if b == "tensor" else "GB/s", "frac": a / (tensor_peak if b == "tensor" else hbm_peak),
                "ms_per_block": ms, "share_of_block": ms / block_ms} for n, b, a, ms in rows]
    achieved = (gemm_ops + attn_ops) / (gemm_ms + attn_ms) / 1e9
    full = (L, F) == (16384, 12288)
    return {"bound": "tensor", "kernel": "int8_gemm_kernel (4 sites) + attention_kernel of one block, weighted by time",
            "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
            "frac_of_nominal": achieved / 4500.0, "peak_source": src,
            "traffic": sum(GEMM_DRAM_MB.values()) * 1e6 if full else None,
            "traffic_note": ("dram read + write bytes of the four GEMM launches at 16384 tokens, F = 12288, from an ncu capture of the "
                             f"kernel as of commit {GEMM_DRAM_COMMIT} (algorithmic operand + output bytes: 1610.6e6); the attention "
                             "kernel moves its operands through L2 (under 0.2e9 DRAM bytes per launch)"),
            "block_ms_sum_of_kernels": block_ms, "kernels": kernels, "per_kernel": prof}


def main():
    args = parse()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as dist
    from owoinfer_b200 import ops, synth
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.workload == "step2048_ulysses":
        from owoinfer_b200 import parallel
        return parallel.bench_ulysses(args, rank, world, local)

    F = args.ffn
    tier = ops.TIER_W4A8 if args.workload == "turbo1024" else ops.TIER_INT8
    seq_len, seqs = workload_shape(args.workload, world)
    if args.workload == "step1024_cfgsplit" and world != 2:
        raise SystemExit("step1024_cfgsplit runs on exactly 2 GPUs (one CFG half each)")
    n_blocks = 1 if args.workload == "block1024" else args.blocks
    L = seq_len * seqs
    scaling = "strong" if args.workload == "step1024_cfgsplit" else "weak"

    # Weights: every block its own random-init ConvRot weights (~151 MB INT8 per block at F = 12288).
    seed0 = 3000 + 100000 * (0 if scaling == "strong" else rank)
    blocks, keep = [], []
    for b in range(n_blocks):
        w = synth.block_weights(D, F, seed0 + 100 * b, tier=tier)
        lin = {}
        for name in ("qkv", "o", "up_gate", "down"):
            lin[name] = ops.make_w4(w[name][0], w[name][1], 64, w[name][2]) if tier == ops.TIER_W4A8 else w[name]
        blocks.append(ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], lin["qkv"], lin["o"],
                                       lin["up_gate"], lin["down"]))
        keep.append((w, lin))
    cfg_row = rank if scaling == "strong" else 0
    x0 = synth.activations(L, D, 1001 + rank + cfg_row)
    mod = synth.modulation(D, 2001)
    grid = 128 if seq_len > 16384 else 64  # 2048^2: a 128 x 128 latent grid + 4096 text tokens
    rope_one = ops.moss_rope_table(grid, grid, seq_len - grid * grid)
    rope = rope_one.repeat(seqs, 1).contiguous()
    cu = synth.cu_seqlens([seq_len] * seqs)
    run = ops.block_run(L, cu, seq_len, D=D, F=F, heads=HEADS, tier=tier)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    x = x0.clone()
    bufs = ops.block_buffers(x, mod, rope, ws)
    launches_per_block = 12  # the grouped 4-bit tier decodes inside its GEMMs (e4m3 group scales): the same twelve launches

    # The step (504 launches) is captured once into a CUDA graph and replayed, as the reference's engine does with its step
    # graphs; the first SiTU-GLU call fills its tables outside any capture, hence the eager call first.
    graph = None
    if not args.no_graph:
        ops.dit_step(blocks, bufs, run)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ops.dit_step(blocks, bufs, run)

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            ops.dit_step(blocks, bufs, run)

    def step():
        # x keeps evolving across steps (as across denoising steps); re-seed it so values stay in range.
        x.copy_(x0)
        run_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_step = float(elapsed.item()) / args.steps

    # End to end through the public call with host buffers: H2D of the step's tokens, modulation and RoPE table from
    # pinned memory, the step, D2H of the result; one stream synchronisation per step.
    hx = x0.cpu().pin_memory()
    hmod, hrope = mod.cpu().pin_memory(), rope.cpu().pin_memory()
    hout = torch.empty_like(hx).pin_memory()
    h2d = hx.numel() * 2 + hmod.numel() * 2 + hrope.numel() * 2
    d2h = hout.numel() * 2

    def e2e_step():
        x.copy_(hx, non_blocking=True)
        mod.copy_(hmod, non_blocking=True)
        rope.copy_(hrope, non_blocking=True)
        run_step()
        hout.copy_(x, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device="cuda")
    if world > 1:
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e.item())
    g_stat = ops.kernel_status()

    # value: ms per image-step aggregated over the job: N images advance per step under weak scaling.
    units = world if scaling == "weak" else 1
    line = {"metric": ("dit_ms_per_step_2048" if seq_len > 16384 else METRIC), "value": ms_step / units, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": scaling,
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(args, world, "direct" if graph is None else "cuda graph replay"),
            "e2e": {"value": e2e_ms / units, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_block * n_blocks * args.steps, "kernel_status": list(g_stat)}
    if rank == 0:
        line["clocks"] = clocks
        if not args.no_profile:
            prof = profile_kernels(ops, torch, L, F, keep[0][0] if tier == ops.TIER_INT8 else synth.block_weights(D, F, 1, tier=0))
            line["roofline"] = roofline_record(prof, L, F, seq_len, seqs)
            threads = os.cpu_count() or 1
            bt, at = CPU_SAMPLE_TOKENS, CPU_SAMPLE_KEYS
            tb, ta = cpu_sample(F, bt, at, threads)
            v = cpu_extrapolate(tb, ta, bt, at, seq_len, seqs, n_blocks)
            line["cpu_baseline"] = {"value": v, "unit": "ms", "cores": threads, "kind": "port", "extrapolated": True,
                                    "sample": f"one block on {bt} tokens ({tb:.2f} s) + attention of one {at}-token sequence x 24 "
                                              f"heads ({ta:.2f} s), extrapolated to {n_blocks} blocks x {seqs} x {seq_len} tokens"}
            if world == 1 and tier == ops.TIER_INT8 and not args.no_ref_gpu:
                line["reference_gpu"] = reference_kernels_on_this_gpu(torch, ops, keep, x, x0, mod, rope, cu, seq_len, L, F)
            if world == 1 and args.workload == "step1024":
                # The same step with grouped 4-bit weights (W4A8, group 64, e4m3 group scales), decoded inside the GEMMs.
                del blocks, keep, bufs, graph
                torch.cuda.empty_cache()
                line["extra"] = {"turbo1024_ms": single_gpu_step_ms(torch, ops, synth, [seq_len] * seqs, n_blocks, F, min(args.steps, 5), 3,
                                                                    tier=ops.TIER_W4A8)}
                torch.cuda.empty_cache()
                # The step as a caller of the forward sees it: latents + time vector in, velocity latents out.
                fw = forward_shell_ms(torch, ops, synth, 64, seq_len - 64 * 64, seqs, n_blocks, F, min(args.steps, 3))
                line["extra"]["forward1024_ms"] = fw["forward"]
                line["extra"]["forward1024_shell_only_ms"] = fw["shell_only"]
                line["extra"].update({k: v for k, v in fw.items() if k.startswith("forward256_")})
                line["extra"]["load_file"] = load_file_record(torch, ops, synth, F)
    if world > 1 and args.workload == "step1024" and not args.no_ulysses and tier == ops.TIER_INT8:
        # The headline above is image data parallel (no collective). The sequence-parallel configuration, the one with an
        # exchange step, rides along as its own record: free the headline's buffers first.
        del blocks, keep, bufs, ws, graph, x, x0, hx, hout
        torch.cuda.empty_cache()
        rec = ulysses_record(torch, dist, ops, synth, args, rank, world)
        if rank == 0:
            line["ulysses"] = rec
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
