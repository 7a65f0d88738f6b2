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
