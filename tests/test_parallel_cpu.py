"""Host-side logic of the multi-GPU partitioning, on CPU: gloo backend, world size 2 (and 4), child processes.
The Ulysses exchanges must turn token-sharded q/k/v into head-sharded full sequences and back, in sequence order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from owoinfer_b200 import parallel


def test_partition_items():
    for n, world in ((8, 8), (2, 2), (5, 2), (3, 4), (0, 2)):
        got = [list(parallel.partition_items(n, world, r)) for r in range(world)]
        assert sum(got, []) == list(range(n))
        assert max(len(g) for g in got) - min(len(g) for g in got) <= 1


def test_shard_roundtrip_and_uneven_rejected():
    seq = [12, 8]
    x = torch.arange(20 * 3).view(20, 3)
    shards = [parallel.shard_tokens(x, seq, 4, r) for r in range(4)]
    assert all(s.shape[0] == 5 for s in shards)
    assert torch.equal(parallel.unshard_tokens(shards, seq, 4), x)
    with pytest.raises(ValueError):
        parallel.ulysses_local_lengths([10], 4)


def test_group_layout_and_qkv_row_order():
    assert parallel.group_layout(8, 2) == (2, 4) and parallel.group_layout(4, 2) == (2, 2)
    assert parallel.group_layout(2, 2) == (2, 1) and parallel.group_layout(1, 2) == (1, 1)
    assert parallel.group_layout(4, 1) == (1, 4) and parallel.group_layout(6, 4) == (2, 3)
    heads, size = 8, 4
    order = parallel.sp_qkv_row_order(heads, size)
    assert sorted(order.tolist()) == list(range(3 * heads * 128))
    # Column block (half h, rank r) of the reordered GEMM output = [q | k | v] of heads r * hp + h * hh .. + hh - 1.
    hp = heads // size
    hh = hp // 2
    cols = torch.arange(3 * heads * 128).view(3, heads, 128)
    for h in range(2):
        for r in range(size):
            at = (h * size + r) * 3 * hh * 128
            block = order[at:at + 3 * hh * 128].view(3, hh, 128)
            assert torch.equal(block, cols[:, r * hp + h * hh:r * hp + (h + 1) * hh])
    odd = parallel.sp_qkv_row_order(6, 2)   # three heads per rank: one "half"
    assert torch.equal(odd[:3 * 3 * 128].view(3, 3, 128), torch.arange(3 * 6 * 128).view(3, 6, 128)[:, 0:3])
    w = torch.arange(3 * heads * 128 * 2).view(3 * heads * 128, 2)
    pw, ps = parallel.permute_qkv(w, torch.arange(3 * heads * 128), heads, size)
    assert torch.equal(pw[:, 0] // 2, ps) and torch.equal(ps, order)
    one = parallel.sp_qkv_row_order(heads, 1)   # a group of one still runs its heads in two halves
    assert torch.equal(one[:3 * 4 * 128].view(3, 4, 128), cols[:, 0:4]) and torch.equal(one[3 * 4 * 128:].view(3, 4, 128), cols[:, 4:8])


def test_sp_run_is_validated_before_any_work():
    """b2_block_quant_sp_workspace_bytes / b2_run_block_quant_sp refuse runs the path cannot serve (no GPU needed)."""
    import ctypes as C
    from owoinfer_b200 import _lib
    lib = _lib.lib()

    def run(seq_lens, size, heads=24, tier=0, tokens=None):
        r = _lib.SpRun()
        r.struct_size = C.sizeof(_lib.SpRun)
        b = r.local
        b.struct_size = C.sizeof(_lib.BlockRun)
        b.tokens = sum(s // size for s in seq_lens) if tokens is None else tokens
        b.D, b.F, b.heads = heads * 128, 1024, heads
        b.cu_seqlens, b.batch, b.max_seqlen, b.tier = 0x1000, len(seq_lens), max(seq_lens), tier
        arr = (C.c_int32 * len(seq_lens))(*seq_lens)
        r.seq_lens_host = C.cast(arr, C.c_void_p)
        r._keep = arr
        return r

    need = lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096, 2048], 4)), 4)
    assert need > 0
    assert lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096, 2048], 8)), 8) > 0        # 3 heads per rank: one half
    assert lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096, 2050], 4)), 4) == 0       # length not divisible
    assert lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096], 4, tier=2)), 4) == 0     # INT8 tier only
    assert lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096], 4, tokens=1000)), 4) == 0
    assert lib.b2_block_quant_sp_workspace_bytes(C.byref(run([4096], 5)), 5) == 0             # heads % size
    # Argument errors come before anything touches a device.
    assert lib.b2_sp_comm_create(None, C.c_size_t(0), 2, 0, C.byref(C.c_void_p())) == -1      # size 2 without an id
    assert lib.b2_sp_comm_create(None, C.c_size_t(0), 2, 2, C.byref(C.c_void_p())) == -1
    w, a = _lib.BlockWeights(), _lib.BlockBuffers()
    w.struct_size, a.struct_size = C.sizeof(_lib.BlockWeights), C.sizeof(_lib.BlockBuffers)
    assert lib.b2_run_block_quant_sp(C.byref(w), C.byref(a), C.byref(run([4096, 2048], 1)), None, None) == -1
    assert b"communicator" in lib.b2_last_error_message()
    # A group of one needs neither an id nor NCCL, only a device for its stream and events (absent here: a CUDA error,
    # not a crash).
    comm = C.c_void_p()
    rc = lib.b2_sp_comm_create(None, C.c_size_t(0), 1, 0, C.byref(comm))
    assert rc in (0, -8)
    if rc == 0:
        a.x = a.mod = a.rope = a.workspace = 0x10000
        a.workspace_bytes = need - 1
        assert lib.b2_run_block_quant_sp(C.byref(w), C.byref(a), C.byref(run([4096, 2048], 1)), comm, None) == -1
        assert b"workspace" in lib.b2_last_error_message()
        assert lib.b2_sp_comm_destroy(comm) == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, seq_lens, heads, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        total = sum(seq_lens)
        qkv_full = torch.randn((total, 3 * heads * 128), generator=g)      # same on every rank
        local_lens = parallel.ulysses_local_lengths(seq_lens, world)
        mine = parallel.shard_tokens(qkv_full, seq_lens, world, rank).contiguous()
        full = parallel.exchange_tokens_to_heads(mine, local_lens, heads)
        hp = heads // world
        ok = True
        start = 0
        for s, t in zip(seq_lens, full):
            want = qkv_full[start:start + s].view(s, 3, heads, 128)[:, :, rank * hp:(rank + 1) * hp]
            ok = ok and t.shape == (s, 3, hp, 128) and torch.equal(t, want)
            start += s
        # "attention" stand-in: any per-(sequence, head) function of the full sequence; here q + mean_k + v.
        outs = [t[:, 0] + t[:, 1].mean(dim=0, keepdim=True) + t[:, 2] for t in full]
        back = parallel.exchange_heads_to_tokens(outs, local_lens, heads)
        ref_parts, start = [], 0
        for s in seq_lens:
            blk = qkv_full[start:start + s].view(s, 3, heads, 128)
            ref_parts.append((blk[:, 0] + blk[:, 1].mean(dim=0, keepdim=True) + blk[:, 2]).reshape(s, heads * 128))
            start += s
        ref = parallel.shard_tokens(torch.cat(ref_parts), seq_lens, world, rank)
        ok = ok and back.shape == ref.shape and torch.allclose(back, ref, atol=1e-6)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ulysses_exchanges_gloo(world):
    port = _free_port()
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, [16, 8], 8, ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}
