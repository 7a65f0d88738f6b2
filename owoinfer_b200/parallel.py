"""Multi-GPU partitioning of the quantized DiT step: one process per GPU, torch.distributed for the plumbing.

The reference engine is single-GPU; everything here is new. Three ways to spread a step over the GPUs of one node:

  image data parallel   each rank owns whole images (both CFG rows): no data-path collective.
  CFG split             rank 0 runs the conditional row, rank 1 the unconditional row: no data-path collective (the
                        guidance combine of the two velocities is outside the block path).
  Ulysses sequence parallel (2048^2 and above)
                        outside attention every op is token-row-local, so each rank owns a contiguous 1/P slice of every
                        sequence's tokens; inside attention each rank owns H/P heads of the full sequences. Two
                        all-to-alls per block: q, k, v (after QK-norm + RoPE) tokens -> heads, attention output heads ->
                        tokens. Per-(sequence, head) statistics of the attention pre-pass (K mean, V absmax) become local
                        after the first exchange and are summed in the same order as on one GPU, so the N-GPU block
                        output equals the 1-GPU output bit for bit.

The exchange helpers are plain torch + torch.distributed and run on any backend (tests use gloo on CPU); the block
itself calls the CUDA library through `ops`.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------------------------------------- partitions

def partition_items(n_items: int, world: int, rank: int) -> range:
    """Contiguous share of `n_items` independent items (images, CFG rows) owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def ulysses_local_lengths(seq_lens, world: int):
    """Tokens of each sequence held by one rank. Every sequence must split evenly (pad the text part otherwise)."""
    for s in seq_lens:
        if s % world != 0:
            raise ValueError(f"sequence length {s} does not split over {world} ranks")
    return [s // world for s in seq_lens]


def shard_tokens(x_full: torch.Tensor, seq_lens, world: int, rank: int) -> torch.Tensor:
    """Rows of a packed [sum(seq_lens), ...] tensor that `rank` owns: its contiguous 1/world slice of every sequence."""
    parts, start = [], 0
    for s in seq_lens:
        c = s // world
        parts.append(x_full[start + rank * c:start + (rank + 1) * c])
        start += s
    return torch.cat(parts, dim=0)


def unshard_tokens(shards, seq_lens, world: int) -> torch.Tensor:
    """Inverse of shard_tokens given every rank's shard (list indexed by rank)."""
    out = []
    for i, s in enumerate(seq_lens):
        c = s // world
        off = sum(l // world for l in seq_lens[:i])
        for r in range(world):
            out.append(shards[r][off:off + c])
    return torch.cat(out, dim=0)


# ----------------------------------------------------------------------------------------------------------- exchanges

def exchange_tokens_to_heads(qkv_local: torch.Tensor, local_lens, heads: int, group=None):
    """All-to-all #1. qkv_local: [sum(local_lens), 3 * heads * 128] (this rank's tokens of every sequence, all heads).
    Returns one tensor per sequence of shape [world * local_len, 3, heads / world, 128]: the FULL sequence, q / k / v of
    this rank's heads (tokens in sequence order: rank 0's slice, rank 1's slice, ...)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    hp = heads // world
    out, start = [], 0
    for c in local_lens:
        rows = qkv_local[start:start + c].view(c, 3, world, hp, 128)
        send = rows.permute(2, 0, 1, 3, 4).contiguous()           # [dest rank, token, qkv, head, 128]
        recv = torch.empty_like(send)                              # [source rank, token, qkv, head, 128]
        if world > 1:
            dist.all_to_all_single(recv, send, group=group)
        else:
            recv = send
        out.append(recv.view(world * c, 3, hp, 128))
        start += c
    return out


def exchange_heads_to_tokens(attn_full, local_lens, heads: int, group=None) -> torch.Tensor:
    """All-to-all #2. attn_full: per sequence [world * local_len, heads / world, 128] (full sequence, this rank's heads).
    Returns [sum(local_lens), heads * 128]: this rank's tokens of every sequence, all heads."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    hp = heads // world
    parts = []
    for o, c in zip(attn_full, local_lens):
        send = o.reshape(world, c, hp, 128)                        # [dest rank (token slice), token, head, 128]
        recv = torch.empty_like(send)                              # [source rank (head group), token, head, 128]
        if world > 1:
            dist.all_to_all_single(recv, send.contiguous(), group=group)
        else:
            recv = send
        parts.append(recv.permute(1, 0, 2, 3).reshape(c, heads * 128))
    return torch.cat(parts, dim=0)


# ----------------------------------------------------------------------------------------------------------- the block

class UlyssesBlockRunner:
    """One all-INT8 block on this rank's token shard, kernels queued on the current stream, all-to-alls on the process
    group. Buffers are allocated once for the run's shape."""

    def __init__(self, seq_lens, D: int, F: int, heads: int, group=None, device="cuda"):
        from . import ops
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.seq_lens = list(seq_lens)
        self.local_lens = ulysses_local_lengths(self.seq_lens, self.world)
        self.D, self.F, self.heads = D, F, heads
        if heads % self.world != 0:
            raise ValueError(f"{heads} heads do not split over {self.world} ranks")
        self.hp = heads // self.world
        L = sum(self.local_lens)
        self.L = L
        self.xq = torch.empty((L, max(D, F)), dtype=torch.int8, device=device)
        self.scale = torch.empty(L, dtype=torch.float32, device=device)
        self.qkv = torch.empty((L, 3 * D), dtype=torch.bfloat16, device=device)
        self.ffn = torch.empty((L, F), dtype=torch.bfloat16, device=device)
        self.attn_full = [torch.empty((s, self.hp, 128), dtype=torch.bfloat16, device=device) for s in self.seq_lens]
        self.cu_one = [torch.tensor([0, s], dtype=torch.int32, device=device) for s in self.seq_lens]
        self.ws = [torch.empty(max(256, ops.attention_q8_workspace_bytes(s, s, 1, s, self.hp)), dtype=torch.uint8, device=device)
                   for s in self.seq_lens]
        self.comm_stream = torch.cuda.Stream(device=device) if self.world > 1 else None

    def run(self, x, mod, rope_local, w):
        """x: bf16 [L_local, D] updated in place; mod: bf16 [6 D]; rope_local: bf16 [L_local, 128] (this rank's rows of the
        table); w: dict with norm1, norm2, q_norm, k_norm and qkv / o / up_gate / down = (int8 weight, f32 scale).
        The exchanges run on a second stream, one sequence at a time, so that the all-to-all of one sequence overlaps the
        attention of another."""
        ops, D, F = self.ops, self.D, self.F
        xq_d = self.xq[:, :D]
        m = [mod[i * D:(i + 1) * D] for i in range(6)]
        ops.rms_norm_modulate_rotate_quantize(x, w["norm1"], m[1], m[0], q=xq_d, scale=self.scale)
        ops.int8_gemm(xq_d, self.scale, w["qkv"][0], w["qkv"][1], out=self.qkv)
        ops.qk_norm_rope_moss(self.qkv, self.heads, w["q_norm"], w["k_norm"], rope_local)
        cur = torch.cuda.current_stream()
        comm = self.comm_stream if self.world > 1 else cur
        comm.wait_stream(cur)
        n_seq = len(self.seq_lens)
        full, arrived, parts, returned = [None] * n_seq, [], [None] * n_seq, []
        start = 0
        with torch.cuda.stream(comm):
            for i, c in enumerate(self.local_lens):
                full[i] = exchange_tokens_to_heads(self.qkv[start:start + c], [c], self.heads, self.group)[0]
                full[i].record_stream(cur)
                arrived.append(comm.record_event())
                start += c
        for i, t in enumerate(full):
            cur.wait_event(arrived[i])
            s = self.seq_lens[i]
            ops.attention_q8(t[:, 0], t[:, 1], t[:, 2], self.attn_full[i], self.cu_one[i], self.cu_one[i], s, ops.SM_SCALE,
                             workspace=self.ws[i])
            done = cur.record_event()
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                parts[i] = exchange_heads_to_tokens([self.attn_full[i]], [self.local_lens[i]], self.heads, self.group)
                parts[i].record_stream(cur)
                returned.append(comm.record_event())
        for e in returned:
            cur.wait_event(e)
        attn = torch.cat(parts, dim=0) if n_seq > 1 else parts[0]
        ops.rotate_quantize(attn, q=xq_d, scale=self.scale)
        ops.int8_gemm_gated_residual(xq_d, self.scale, w["o"][0], w["o"][1], m[2], x)
        ops.rms_norm_modulate_rotate_quantize(x, w["norm2"], m[4], m[3], q=xq_d, scale=self.scale)
        ops.int8_gemm_situ_glu(xq_d, self.scale, w["up_gate"][0], w["up_gate"][1], out=self.ffn)
        xq_f = self.xq[:, :F]
        ops.rotate_quantize(self.ffn, q=xq_f, scale=self.scale)
        ops.int8_gemm_gated_residual(xq_f, self.scale, w["down"][0], w["down"][1], m[5], x)
        return x


# ----------------------------------------------------------------------------------------------------------- the bench

def bench_ulysses(args, rank: int, world: int, local: int):
    """bench.py --workload step2048_ulysses: the 2048^2 INT8 step (CFG batch 2: two sequences of 16384 image + 4096 text
    tokens) with every sequence's tokens sharded over all ranks. Strong scaling: the job is one image."""
    from . import ops, synth
    D, heads, F = 3072, 24, args.ffn
    seq_lens = [20480, 20480]
    n_blocks = args.blocks
    group = None
    runner = UlyssesBlockRunner(seq_lens, D, F, heads, group)
    weights = [synth.block_weights(D, F, 3000 + 100 * b) for b in range(n_blocks)]
    x_full_rows = sum(seq_lens)
    x0 = shard_tokens(synth.activations(x_full_rows, D, 1003), seq_lens, world, rank).contiguous()
    mod = synth.modulation(D, 2001)
    rope_one = ops.moss_rope_table(128, 128, 4096)
    rope_local = shard_tokens(rope_one.repeat(len(seq_lens), 1), seq_lens, world, rank).contiguous()
    x = x0.clone()

    def step():
        x.copy_(x0)
        for w in weights:
            runner.run(x, mod, rope_local, w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_step = float(elapsed.item()) / args.steps

    hx = x0.cpu().pin_memory()
    hout = torch.empty_like(hx).pin_memory()

    def e2e_step():
        x0.copy_(hx, non_blocking=True)
        step()
        hout.copy_(x, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device="cuda")
    if world > 1:
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    if rank == 0:
        launches = (11 + 4 * len(seq_lens)) * n_blocks * args.steps
        line = {"metric": "dit_ms_per_step_2048", "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": "step2048_ulysses", "blocks": n_blocks, "d": D, "heads": heads, "ffn": F,
                           "sequences": seq_lens, "tier": "int8", "attention": "int8_fp8_f32acc",
                           "parallelism": f"ulysses-sp{world}", "collective": "2 NCCL all-to-alls per block and sequence",
                           "l2": "inputs larger than L2 (block weights stream from HBM every step)"},
                "e2e": {"value": float(e2e.item()), "unit": "ms", "h2d_bytes_per_step": hx.numel() * 2,
                        "d2h_bytes_per_step": hout.numel() * 2},
                "gpu_launches": launches, "kernel_status": list(ops.kernel_status())}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
