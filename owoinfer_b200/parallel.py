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

The sequence-parallel block itself is C++ behind the C ABI (b2_run_block_quant_sp: NCCL point-to-point exchanges, no
packing pass, no allocation); this module holds the partition arithmetic, the load-time QKV row order that path needs,
the glue that builds one communicator per group from a torch.distributed job, and torch re-statements of the two
exchanges that run on any backend (the CPU tests check the layout arithmetic with gloo).
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


# ----------------------------------------------------------------------------------------------------------- layouts

def group_layout(world: int, n_sequences: int):
    """How a job of `world` ranks splits `n_sequences` independent sequences (CFG rows): (groups, sp) with groups * sp ==
    world. Independent sequences go to separate groups first (no collective between them); what is left of the ranks
    shares each sequence's tokens. 8 ranks and 2 sequences: 2 groups x sequence-parallel 4."""
    groups = 1
    for g in range(min(world, n_sequences), 0, -1):
        if world % g == 0 and n_sequences % g == 0:
            groups = g
            break
    return groups, world // groups


def sp_qkv_row_order(heads: int, size: int) -> torch.Tensor:
    """Row order of the fused QKV weight [3 * heads * 128, k] (q heads, k heads, v heads) for a sequence-parallel group of
    `size` ranks: [half h][destination rank r][q | k | v][head r * heads/size + h * hh + j][128], where a rank's heads/size
    heads are processed in two halves of hh heads (one "half" when that number is odd). Apply to the weight rows and to
    the scale vector at load time (index_select)."""
    hp = heads // size
    halves = 2 if hp % 2 == 0 else 1
    idx = torch.arange(3 * heads * 128).view(3, size, halves, hp // halves, 128)   # [qkv, rank, half, head, row]
    return idx.permute(2, 1, 0, 3, 4).reshape(-1)


def permute_qkv(weight: torch.Tensor, scale: torch.Tensor, heads: int, size: int):
    order = sp_qkv_row_order(heads, size).to(weight.device)
    return weight.index_select(0, order).contiguous(), scale.index_select(0, order).contiguous()


def make_sp_comm(group_ranks, rank: int, group=None):
    """One b2_sp_comm over `group_ranks` (global ranks, this rank among them). The id is created by the group's first
    rank and handed round with torch.distributed (the job's default group carries it; `group` is the torch group of
    exactly these ranks, or None when the group is the whole job)."""
    from . import ops
    size = len(group_ranks)
    if size == 1:
        return ops.SpComm(1, 0)
    box = [ops.sp_unique_id() if rank == group_ranks[0] else None]
    dist.broadcast_object_list(box, src=group_ranks[0], group=group)
    return ops.SpComm(size, group_ranks.index(rank), box[0])


class SpBlock:
    """The C++ sequence-parallel block on one rank: buffers sized once for the run, weights in the group's QKV row order."""

    def __init__(self, seq_lens, comm, D: int, F: int, heads: int, device="cuda"):
        from . import ops, synth
        self.ops, self.comm = ops, comm
        self.seq_lens = list(seq_lens)
        self.local_lens = ulysses_local_lengths(self.seq_lens, comm.size)
        self.L = sum(self.local_lens)
        self.cu_full = synth.cu_seqlens(self.seq_lens, device)
        self.run = ops.sp_run(self.seq_lens, comm.size, self.cu_full, D=D, F=F, heads=heads)
        self.ws = torch.empty(ops.block_quant_sp_workspace_bytes(self.run, comm.size), dtype=torch.uint8, device=device)
        self.heads = heads

    def weights(self, w):
        """ops.BlockWeights of a synth.block_weights dict, the QKV rows reordered for this group."""
        qkv = permute_qkv(w["qkv"][0], w["qkv"][1], self.heads, self.comm.size)
        return self.ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], qkv, w["o"], w["up_gate"], w["down"])

    def buffers(self, x_local, mod, rope_full):
        return self.ops.block_buffers(x_local, mod, rope_full, self.ws)


# ----------------------------------------------------------------------------------------------------------- the bench

def measure_ulysses(rank: int, world: int, blocks: int, F: int, steps: int, warmup: int, seq_lens=(20480, 20480)):
    """The 2048^2 INT8 step (CFG batch 2: two sequences of 16384 image + 4096 text tokens) over all ranks of the job:
    the two sequences go to two groups (no collective between them), the ranks of a group share their sequence's tokens
    (Ulysses). Strong scaling: the job is one image. Returns (ms per step as the max over ranks, record of the layout)."""
    from . import ops, synth
    D, heads = 3072, 24
    seq_lens = list(seq_lens)
    n_groups, sp = group_layout(world, len(seq_lens))
    gid, grank = rank // sp, rank % sp
    ranks = list(range(gid * sp, (gid + 1) * sp))
    torch_groups = [dist.new_group(list(range(g * sp, (g + 1) * sp))) for g in range(n_groups)] if world > 1 and sp > 1 and n_groups > 1 else None
    comm = make_sp_comm(ranks, rank, None if torch_groups is None else torch_groups[gid])
    per_group = len(seq_lens) // n_groups
    mine = seq_lens[gid * per_group:(gid + 1) * per_group]          # the sequences this group runs
    first_row = sum(seq_lens[:gid * per_group])
    blk = SpBlock(mine, comm, D, F, heads)
    weights, keep = [], []
    for b in range(blocks):
        w = synth.block_weights(D, F, 3000 + 100 * b)
        keep.append(w)
        weights.append(blk.weights(w))
    x_all = synth.activations(sum(seq_lens), D, 1003)
    x0 = shard_tokens(x_all[first_row:first_row + sum(mine)], mine, sp, grank).contiguous()
    del x_all
    mod = synth.modulation(D, 2001)
    grid = 128
    rope_full = torch.cat([ops.moss_rope_table(grid, grid, s - grid * grid) for s in mine]).contiguous()
    x = x0.clone()
    bufs = blk.buffers(x, mod, rope_full)

    def step():
        x.copy_(x0)
        ops.dit_step_sp(weights, bufs, blk.run, comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed():
        for _ in range(max(warmup, 3)):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        elapsed = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item()) / steps

    ms = timed()
    ms_local = None
    if sp > 1:  # the same step with every message replaced by a copy of equal size on the GPU itself
        comm.local_exchange(True)
        ms_local = timed()
        comm.local_exchange(False)
    hp = heads // sp
    c = sum(mine) // sp
    sent = (sp - 1) * c * (3 * hp * 128 + hp * 128) * 2
    rec = {"layout": f"{n_groups} group(s) x sequence-parallel {sp}", "groups": n_groups, "sp": sp, "sequences": seq_lens,
           "blocks": blocks, "ffn": F, "all_to_all_bytes_sent_per_gpu_per_block": sent, "kernel_status": list(ops.kernel_status()),
           "ms_with_local_copies_for_exchanges": ms_local, "exposed_exchange_ms": None if ms_local is None else ms - ms_local,
           "launches_per_block": 16 + (2 * (sp - 1) * per_group * 2 if sp > 1 else 0)}
    comm.close()
    del weights, keep, blk, bufs
    torch.cuda.empty_cache()
    return ms, rec


def bench_ulysses(args, rank: int, world: int, local: int):
    """bench.py --workload step2048_ulysses: prints the line of the 2048^2 sequence-parallel step on N GPUs."""
    from . import ops
    ms_step, rec = measure_ulysses(rank, world, args.blocks, args.ffn, args.steps, args.warmup)
    if rank == 0:
        line = {"metric": "dit_ms_per_step_2048", "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": "step2048_ulysses", "blocks": args.blocks, "d": 3072, "heads": 24, "ffn": args.ffn,
                           "sequences": rec["sequences"], "tier": "int8", "attention": "int8_fp8_f32acc",
                           "parallelism": rec["layout"], "collective": "2 NCCL point-to-point exchanges per block inside a group",
                           "l2": "inputs larger than L2 (block weights stream from HBM every step)"},
                "ulysses": rec, "gpu_launches": rec["launches_per_block"] * args.blocks * args.steps,
                "kernel_status": list(ops.kernel_status())}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
