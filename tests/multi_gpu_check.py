"""Run under torch.distributed.run on N GPUs of one node (tests/test_gpu_multi.py launches it): the sequence-parallel
all-INT8 block (b2_run_block_quant_sp: every sequence's tokens sharded over the ranks, two NCCL exchanges around
attention) must equal the single-GPU block bit for bit. Rank 0 computes the single-GPU result, every rank its shard; the
shards are gathered and compared. A second pass splits the ranks into two groups of N / 2, one sequence each."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from owoinfer_b200 import ops, parallel, synth  # noqa: E402

D, F, HEADS = 1024, 2048, 8


def single_gpu(x_full, mod, w, rope_full, seq_lens, blocks):
    cu = synth.cu_seqlens(seq_lens)
    run = ops.block_run(sum(seq_lens), cu, max(seq_lens), D=D, F=F, heads=HEADS)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    bw = ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], w["qkv"], w["o"], w["up_gate"], w["down"])
    want = x_full.clone()
    bufs = ops.block_buffers(want, mod, rope_full, ws)
    for _ in range(blocks):
        ops.run_block_quant(bw, bufs, run)
    torch.cuda.synchronize()
    return want


def sharded(x_full, mod, w, rope_full, seq_lens, ranks, rank, torch_group, blocks):
    """The ranks in `ranks` share the sequences `seq_lens` (rows of x_full / rope_full); returns this rank's shard."""
    comm = parallel.make_sp_comm(ranks, rank, torch_group)
    blk = parallel.SpBlock(seq_lens, comm, D, F, HEADS)
    x = parallel.shard_tokens(x_full, seq_lens, comm.size, comm.rank).contiguous()
    bw = blk.weights(w)
    bufs = blk.buffers(x, mod, rope_full)
    for _ in range(blocks):  # the second block runs on the first one's output
        ops.run_block_quant_sp(bw, bufs, blk.run, comm)
    torch.cuda.synchronize()
    comm.close()
    return x


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    seq_lens = [2048, 1536 + 512 * world]
    L = sum(seq_lens)
    x_full = synth.activations(L, D, 1234)
    mod = synth.modulation(D, 2234)
    w = synth.block_weights(D, F, 3234)
    rope_full = ops.moss_rope_table(1, 1, L - 1)
    ok = True

    # 1. every rank shares both sequences
    x = sharded(x_full, mod, w, rope_full, seq_lens, list(range(world)), rank, None, 2)
    shards = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(shards, x)
    if rank == 0:
        want = single_gpu(x_full, mod, w, rope_full, seq_lens, 2)
        got = parallel.unshard_tokens(shards, seq_lens, world)
        ok = torch.equal(got.view(torch.int16), want.view(torch.int16)) and ops.kernel_status() == (0, 0)
        print(f"ulysses world {world}: {'bit-exact' if ok else 'MISMATCH'} against the single-GPU block "
              f"({(got.float() - want.float()).abs().max().item():.3e} max abs diff)", flush=True)

    # 2. two groups of world / 2 ranks, one sequence each (the layout of a CFG pair on 4 or 8 GPUs)
    if world >= 4:
        sp = world // 2
        groups = [dist.new_group(list(range(g * sp, (g + 1) * sp))) for g in range(2)]
        gid = rank // sp
        lens2 = [4096, 4096]
        x2_full = synth.activations(sum(lens2), D, 4321)
        rope2 = ops.moss_rope_table(1, 1, lens2[0] - 1)
        mine = x2_full[gid * lens2[0]:(gid + 1) * lens2[0]]
        x2 = sharded(mine, mod, w, rope2, [lens2[gid]], list(range(gid * sp, (gid + 1) * sp)), rank, groups[gid], 2)
        shards2 = [torch.empty_like(x2) for _ in range(world)]
        dist.all_gather(shards2, x2)
        if rank == 0:
            ok2 = True
            for g in range(2):
                want = single_gpu(x2_full[g * lens2[0]:(g + 1) * lens2[0]], mod, w, rope2, [lens2[g]], 2)
                got = parallel.unshard_tokens(shards2[g * sp:(g + 1) * sp], [lens2[g]], sp)
                ok2 = ok2 and torch.equal(got.view(torch.int16), want.view(torch.int16))
            print(f"ulysses world {world} as 2 groups x {sp}: {'bit-exact' if ok2 else 'MISMATCH'}", flush=True)
            ok = ok and ok2 and ops.kernel_status() == (0, 0)

    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
