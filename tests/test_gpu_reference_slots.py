"""Reference keys ("slots") and the reference prefill tap of a block run (BlockRun of
src/models/moss_dit/dit_block_fused.h:132-147; MossDit::forward, moss_dit.cpp:1283-1300, 1441-1452).

Attention whose keys are [slot A | own] or [own | slot B] is, for the sequence's own queries, the same arithmetic as
self-attention over the longer sequence that starts with the slot rows (when the slot is a whole number of 128-row query
tiles, so that the per-32-row query scales fall on the same rows) or ends with them (when the own rows are a whole number
of 32-row blocks, for the same reason): the tests hold the new paths to the
bits of the self-attention path, which is checked against the oracle and the reference's kernels elsewhere."""
import numpy as np
import pytest
import torch

from owoinfer_b200 import synth

pytestmark = pytest.mark.gpu
D, H = 3072, 24


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from owoinfer_b200 import ops as o
    yield o
    torch.cuda.synchronize()
    assert o.kernel_status() == (0, 0)


def _views(buf, rows0, rows1):
    n = rows1 - rows0
    return tuple(buf[rows0:rows1].as_strided((n, H, 128), (3 * D, 128, 1), buf[rows0:rows1].storage_offset() + i * D) for i in range(3))


@pytest.mark.parametrize("slot_a,slot_b,n0,n1", [(128, 77, 300, 224), (256, 256, 129, 640)])
def test_attention_over_slot_keys_equals_self_attention_over_the_longer_sequences(ops, slot_a, slot_b, n0, n1):
    g = torch.Generator(device="cuda").manual_seed(slot_a + n0)
    rows = slot_a + n0 + n1 + slot_b
    region = torch.randn((rows, 3 * D), device="cuda", generator=g).to(torch.bfloat16)   # [slot A | seq 0 | seq 1 | slot B]
    cu_q = synth.cu_seqlens([n0, n1])
    cu_k = synth.cu_seqlens([slot_a + n0, n1 + slot_b])
    q, _, _ = _views(region, slot_a, slot_a + n0 + n1)
    _, k, v = _views(region, 0, rows)
    out = torch.empty((n0 + n1, H, 128), dtype=torch.bfloat16, device="cuda")
    max_k = max(slot_a + n0, n1 + slot_b)
    ops.attention_q8(q, k, v, out, cu_q, cu_k, max_k, ops.SM_SCALE)
    qs, ks, vs = _views(region, 0, rows)
    full = torch.empty((rows, H, 128), dtype=torch.bfloat16, device="cuda")
    ops.attention_q8(qs, ks, vs, full, cu_k, cu_k, max_k, ops.SM_SCALE)
    torch.cuda.synchronize()
    assert torch.equal(out[:n0].view(torch.int16), full[slot_a:slot_a + n0].view(torch.int16))
    assert torch.equal(out[n0:].view(torch.int16), full[slot_a + n0:slot_a + n0 + n1].view(torch.int16))
    # and it is attention: close to exact fp32 softmax attention over those keys
    kk, vv = k[:slot_a + n0, 3].float(), v[:slot_a + n0, 3].float()
    exact = torch.softmax(q[:n0, 3].float() @ kk.t() * ops.SM_SCALE, dim=-1) @ vv
    rel = (out[:n0, 3].float() - exact).norm() / exact.norm()
    assert rel < 0.05


def _block(ops, F, seed):
    w = synth.block_weights(D, F, seed)
    return ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], w["qkv"], w["o"], w["up_gate"], w["down"]), w


def test_tap_then_slots_round_trip(ops):
    """A reference image is prefilled with tap_only runs, then a generation run reads the tapped keys through its slots:
    the block's output equals the block over the sequences [reference | own] and [own | reference] cut to the own rows,
    whenever everything before attention is row-local (it is: norm, GEMM, QK-norm, RoPE act per token)."""
    F, slot = 512, 128
    bw, w = _block(ops, F, 21)
    mod = synth.modulation(D, 4)
    n0, n1 = 200, 352
    x_ref = synth.activations(slot, D, 8)
    rope_ref = ops.moss_rope_table(8, 8, slot - 64)
    cu_ref = synth.cu_seqlens([slot])
    tap = torch.zeros((slot, 2 * D), dtype=torch.bfloat16, device="cuda")
    run = ops.block_run(slot, cu_ref, slot, D=D, F=F, kv_tap=tap, tap_only=True)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    x_keep = x_ref.clone()
    ops.run_block_quant(bw, ops.block_buffers(x_ref, mod, rope_ref, ws), run)
    torch.cuda.synchronize()
    assert torch.equal(x_ref, x_keep) and tap.abs().max() > 0            # tap_only: the residual stream is untouched

    # The tapped rows are the k | v columns after QK-norm + RoPE of the same tokens.
    y = ops.rms_norm_modulate(x_keep, w["norm1"], mod[D:2 * D], mod[:D])
    xq, xs = ops.rotate_quantize(y)
    qkv = ops.int8_gemm(xq, xs, w["qkv"][0], w["qkv"][1])
    ops.qk_norm_rope_moss(qkv, H, w["q_norm"], w["k_norm"], rope_ref)
    assert torch.equal(tap.view(torch.int16), qkv[:, D:].contiguous().view(torch.int16))

    # Generation run: two sequences, the first reads slot A, the second slot B (both hold the reference's keys).
    x = synth.activations(n0 + n1, D, 9)
    rope = torch.cat([ops.moss_rope_table(8, 8, n - 64) for n in (n0, n1)]).contiguous()
    cu = synth.cu_seqlens([n0, n1])
    cu_k = synth.cu_seqlens([slot + n0, n1 + slot])
    run = ops.block_run(n0 + n1, cu, max(slot + n0, n1 + slot), D=D, F=F, slot_rows=slot, slot_kv=(tap, tap), cu_seqlens_k=cu_k,
                        k0=0, k1=n0 + n1 + 2 * slot)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    got = x.clone()
    ops.run_block_quant(bw, ops.block_buffers(got, mod, rope, ws), run)

    # The same through plain runs over the longer sequences. Per-token work before attention depends on the row count of
    # the tensor only through torch's reduce order in the norm (same for every count from 16 up), so the long run's own
    # rows carry the same q, k, v.
    long_x = torch.cat([x_keep, x[:n0], x[n0:], x_keep]).contiguous()
    long_rope = torch.cat([rope_ref, rope[:n0], rope[n0:], rope_ref]).contiguous()
    long_cu = synth.cu_seqlens([slot + n0, n1 + slot])
    long_run = ops.block_run(long_x.shape[0], long_cu, max(slot + n0, n1 + slot), D=D, F=F, fused_norm_rope=0)
    ws2 = torch.empty(ops.block_quant_workspace_bytes(long_run), dtype=torch.uint8, device="cuda")
    ops.run_block_quant(bw, ops.block_buffers(long_x, mod, long_rope, ws2), long_run)
    torch.cuda.synchronize()
    want = torch.cat([long_x[slot:slot + n0], long_x[slot + n0:slot + n0 + n1]])
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.isfinite(got.float()).all()

    # The slot rows read in place from a QKV-shaped buffer (row stride 3 D, k | v columns), as the reference keeps them.
    wide = torch.zeros((slot, 3 * D), dtype=torch.bfloat16, device="cuda")
    wide[:, D:] = tap
    runw = ops.block_run(n0 + n1, cu, max(slot + n0, n1 + slot), D=D, F=F, slot_rows=slot, slot_kv=(wide[:, D:], wide[:, D:]),
                         cu_seqlens_k=cu_k, k0=0, k1=n0 + n1 + 2 * slot, slot_kv_ld=3 * D)
    gotw = x.clone()
    ops.run_block_quant(bw, ops.block_buffers(gotw, mod, rope, ws), runw)
    torch.cuda.synchronize()
    assert torch.equal(gotw.view(torch.int16), got.view(torch.int16))

    # Only one slot read: the second sequence attends to its own keys alone.
    cu_k1 = synth.cu_seqlens([slot + n0, n1])
    run1 = ops.block_run(n0 + n1, cu, max(slot + n0, n1), D=D, F=F, slot_rows=slot, slot_kv=(tap, None), cu_seqlens_k=cu_k1,
                         k0=0, k1=n0 + n1 + slot)
    got1 = x.clone()
    ops.run_block_quant(bw, ops.block_buffers(got1, mod, rope, ws), run1)
    plain = x[n0:].clone()
    prun = ops.block_run(n1, synth.cu_seqlens([n1]), n1, D=D, F=F, fused_norm_rope=0)
    ops.run_block_quant(bw, ops.block_buffers(plain, mod, rope[n0:].contiguous(), ws), prun)
    torch.cuda.synchronize()
    assert torch.equal(got1[:n0].view(torch.int16), got[:n0].view(torch.int16))
    assert torch.equal(got1[n0:].view(torch.int16), plain.view(torch.int16))


def test_slot_arguments_are_checked(ops):
    cu = synth.cu_seqlens([64])
    with pytest.raises(ValueError, match="cu_seqlens_k"):
        ops.block_quant_workspace_bytes(ops.block_run(64, cu, 64, F=512, slot_rows=16))
    tap = torch.zeros((16, 2 * D), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="slot_kv_ld"):
        ops.block_quant_workspace_bytes(ops.block_run(64, cu, 96, F=512, slot_rows=32, slot_kv=(tap, None), cu_seqlens_k=cu, k0=0, k1=96,
                                                      slot_kv_ld=D))
    with pytest.raises(ValueError, match="no slot_kv"):
        ops.block_quant_workspace_bytes(ops.block_run(64, cu, 96, F=512, slot_rows=16, slot_kv=(tap, None), cu_seqlens_k=cu, k0=0, k1=96))
