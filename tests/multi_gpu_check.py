"""Run under torch.distributed.run on N GPUs of one node (tests/test_gpu_multi.py launches it): the all-INT8 block with
every sequence's tokens sharded over the ranks (two all-to-alls around attention) must equal the single-GPU block bit
for bit. Rank 0 computes the single-GPU result, every rank its shard; the shards are gathered and compared."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from owoinfer_b200 import ops, parallel, synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    D, F, heads = 512, 1024, 4
    seq_lens = [2048, 1536 + 512 * world]
    L = sum(seq_lens)
    x_full = synth.activations(L, D, 1234)
    mod = synth.modulation(D, 2234)
    w = synth.block_weights(D, F, 3234)
    rope_full = ops.moss_rope_table(1, 1, L - 1)
    runner = parallel.UlyssesBlockRunner(seq_lens, D, F, heads)
    x = parallel.shard_tokens(x_full, seq_lens, world, rank).contiguous()
    rope = parallel.shard_tokens(rope_full, seq_lens, world, rank).contiguous()
    for _ in range(2):  # two blocks in a row: the second runs on the first one's output
        runner.run(x, mod, rope, w)
    torch.cuda.synchronize()
    shards = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(shards, x)
    ok = True
    if rank == 0:
        cu = synth.cu_seqlens(seq_lens)
        run = ops.block_run(L, cu, max(seq_lens), D=D, F=F, heads=heads)
        ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
        bw = ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], w["qkv"], w["o"], w["up_gate"], w["down"])
        want = x_full.clone()
        bufs = ops.block_buffers(want, mod, rope_full, ws)
        for _ in range(2):
            ops.run_block_quant(bw, bufs, run)
        torch.cuda.synchronize()
        got = parallel.unshard_tokens(shards, seq_lens, world)
        ok = torch.equal(got.view(torch.int16), want.view(torch.int16)) and ops.kernel_status() == (0, 0)
        print(f"ulysses world {world}: {'bit-exact' if ok else 'MISMATCH'} against the single-GPU block "
              f"({(got.float() - want.float()).abs().max().item():.3e} max abs diff)", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
