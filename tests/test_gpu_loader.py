"""Weight ingestion on the device: a file written with the official tensor names and per-module configs loads into
tensors that run the block loop and the forward to the same bits as the same tensors handed over directly."""
import numpy as np
import pytest
import torch

from owoinfer_b200 import synth
from tests import loader_files as lf

pytestmark = pytest.mark.gpu
D = lf.D


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from owoinfer_b200 import ops as o
    return o


def _direct_block(ops, t, b, tier, group=64):
    """BlockWeights from the file's own tensors (q | k | v stacked), the way a caller without the loader builds them."""
    p = f"layers.{b}.proj."
    dev = lambda x: x.cuda()

    def lin(names):
        w = torch.cat([t[n + ".weight"] for n in names]).cuda()
        if tier == ops.TIER_W4A8:
            s_rel = torch.cat([t[n + ".weight_s_rel"].view(torch.uint8) for n in names]).cuda()
            s_ch = torch.cat([t[n + ".weight_s_channel"] for n in names]).cuda()
            cb = t.get(names[0] + ".weight_codebook")
            return ops.make_w4(w.view(torch.uint8), s_rel, group, s_ch, None if cb is None else cb.cuda())
        scales = [t[n + ".weight_scale"] for n in names]
        scales = [s.expand(t[n + ".weight"].shape[0]) if s.dim() == 0 else s.reshape(-1) for s, n in zip(scales, names)]
        return (w.view(torch.uint8) if tier == ops.TIER_W4A4_VIA_INT8 else w, torch.cat(scales).contiguous().cuda())

    qkv = [p + "qkv"] if p + "qkv.weight" in t else [p + "q", p + "k", p + "v"]
    norms = [dev(t[f"layers.{b}.{n}.weight"]) for n in ("norm1", "norm2", "q_norm", "k_norm")]
    return ops.BlockWeights(*norms, lin(qkv), lin([p + "o"]), lin([p + "ffn_up_gate"]), lin([p + "ffn_down"]))


def _step(ops, blocks, F, tier, seed=5):
    lens = [300, 276]
    L = sum(lens)
    x = synth.activations(L, D, seed)
    mod = synth.modulation(D, seed + 1)
    rope = torch.cat([ops.moss_rope_table(16, 16, n - 256) for n in lens]).contiguous()
    cu = synth.cu_seqlens(lens)
    run = ops.block_run(L, cu, max(lens), D=D, F=F, tier=tier)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    ops.dit_step(blocks, ops.block_buffers(x, mod, rope, ws), run)
    torch.cuda.synchronize()
    return x


def test_int8_file_with_shell(ops, tmp_path):
    F = 512
    t = {}
    t.update(lf.block(0, F, lf.int8_linear, 10))
    t.update(lf.block(1, F, lf.int8_linear, 20, fused_qkv=True))
    t.update(lf.shell(30))
    t["text_embedder.proj.weight"] = torch.zeros((8, 8), dtype=torch.bfloat16)   # other parts of the model are ignored
    f = ops.DitFile(lf.save(tmp_path / "int8.safetensors", t, prefix="model.diffusion_model."))
    assert (f.num_blocks, f.F, f.tier, f.has_shell, f.has_time_embedding) == (2, F, ops.TIER_INT8, True, True)
    direct = [_direct_block(ops, t, b, ops.TIER_INT8) for b in range(2)]
    got, want = _step(ops, f.blocks, F, ops.TIER_INT8), _step(ops, direct, F, ops.TIER_INT8)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)) and torch.isfinite(got.float()).all()
    # The forward from the file's model against the same tensors handed over one by one.
    tv = f.time_vector(0.481)
    w = lambda n: t[n].float().numpy()
    assert np.array_equal(tv, ops.time_vector_fp32(w("time_embedding.0.weight"), w("time_embedding.0.bias"), w("time_embedding.2.weight"),
                                                   w("time_embedding.2.bias"), 0.481))
    c = lambda n: t[n].cuda()
    model = ops.DitModel(direct, F, c("shared_block_modulation.weight"), c("shared_block_modulation.bias").float(),
                         c("video_head_modulation.weight"), c("video_head_modulation.bias").float(), c("video_embedder.weight"),
                         c("video_embedder.bias"), c("final_norm_video.weight"), c("final_linear_video.weight"), None)
    g = torch.Generator(device="cuda").manual_seed(3)
    latents = torch.randn(1, 128, 16, 16, device="cuda", generator=g)
    rows = [(torch.randn(n, D, device="cuda", generator=g).to(torch.bfloat16), 0, 0) for n in (44, 12)]
    got, _ = ops.dit_forward(f.model, latents, tv, rows)
    want, _ = ops.dit_forward(model, latents, tv, rows)
    for a, b in zip(got, want):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32)) and torch.isfinite(a).all() and a.abs().max() > 0
    # The bf16 form of the time modulation from the file's tensors: the same as the same tensors handed over directly, and
    # the same function as the fp32 form up to bf16 rounding.
    mod, head = f.time_modulation_bf16(0.481)
    b16 = lambda n: t[n].cuda().to(torch.bfloat16)
    mod2, head2 = ops.time_modulation_bf16(b16("time_embedding.0.weight"), b16("time_embedding.0.bias"), b16("time_embedding.2.weight"),
                                           b16("time_embedding.2.bias"), b16("shared_block_modulation.weight"),
                                           b16("shared_block_modulation.bias"), b16("video_head_modulation.weight"),
                                           b16("video_head_modulation.bias"), 0.481)
    assert torch.equal(mod.view(torch.int16), mod2.view(torch.int16)) and torch.equal(head.view(torch.int16), head2.view(torch.int16))
    dtv = torch.from_numpy(tv).cuda()
    mod32 = ops.linear_fp32_row(c("shared_block_modulation.weight"), dtv, c("shared_block_modulation.bias").float())
    assert (mod.float() - mod32.float()).abs().max() <= 0.03 * mod32.float().abs().max()
    outs16, _ = ops.dit_forward(f.model, latents, None, rows, mod=mod, head=head)
    assert torch.isfinite(outs16[0]).all()
    f.close()


def test_scalar_scale_is_expanded_to_rows(ops, tmp_path):
    F = 256
    t = lf.block(0, F, lambda n, r, k, s: lf.int8_linear(n, r, k, s, scalar_scale=True), 40)
    f = ops.DitFile(lf.save(tmp_path / "scalar.safetensors", t))
    got = _step(ops, f.blocks, F, ops.TIER_INT8)
    want = _step(ops, [_direct_block(ops, t, 0, ops.TIER_INT8)], F, ops.TIER_INT8)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("fused", [False, True])
def test_w4a4_file(ops, tmp_path, fused):
    F = 256
    t = lf.block(0, F, lf.w4a4_linear, 50, fused_qkv=fused)
    f = ops.DitFile(lf.save(tmp_path / "w4a4.safetensors", t, prefix="diffusion_model."))
    assert f.tier == ops.TIER_W4A4_VIA_INT8 and not f.has_shell
    got = _step(ops, f.blocks, F, f.tier)
    want = _step(ops, [_direct_block(ops, t, 0, f.tier)], F, f.tier)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)) and torch.isfinite(got.float()).all()


@pytest.mark.parametrize("codebook", [False, True])
def test_w4a8_file(ops, tmp_path, codebook):
    F = 256
    t = lf.block(0, F, lambda n, r, k, s: lf.w4a8_linear(n, r, k, s, codebook=codebook), 60)
    f = ops.DitFile(lf.save(tmp_path / "w4a8.safetensors", t))
    assert f.tier == ops.TIER_W4A8
    got = _step(ops, f.blocks, F, f.tier)
    want = _step(ops, [_direct_block(ops, t, 0, f.tier)], F, f.tier)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)) and torch.isfinite(got.float()).all()
    assert ops.w4_invalid_scales(clear=True) == 0


@pytest.mark.parametrize("maker,tier", [("w4a4", 1), ("w4a8", 2), ("w4a8_codebook", 2), ("int8", 0)])
def test_expanded_open_runs_the_int8_tier_with_the_same_bits(ops, tmp_path, maker, tier):
    """b2_dit_file_open_expanded: grouped 4-bit weights expanded once at load, the blocks then run the INT8 tier. What the
    W4A8 tier computes is that expansion followed by the INT8 GEMM, so the step's output does not change by a bit. Other
    files (INT8; W4A4, whose tier quantises the activations to 4 bits as well) load unchanged."""
    F = 256
    make = {"w4a4": lf.w4a4_linear, "w4a8": lf.w4a8_linear, "int8": lf.int8_linear,
            "w4a8_codebook": lambda n, r, k, s: lf.w4a8_linear(n, r, k, s, codebook=True)}[maker]
    t = {}
    for b in range(2):
        t.update(lf.block(b, F, make, 70 + 10 * b))
    path = lf.save(tmp_path / "model.safetensors", t)
    packed, wide = ops.DitFile(path), ops.DitFile(path, expanded=True)
    assert packed.tier == tier and packed.stored_tier == tier
    assert wide.tier == (ops.TIER_INT8 if tier == 2 else tier) and wide.stored_tier == tier and wide.num_blocks == 2
    assert (wide.device_bytes > packed.device_bytes) == (tier == 2)
    want = _step(ops, packed.blocks, F, packed.tier)
    got = _step(ops, wide.blocks, F, wide.tier)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)) and torch.isfinite(got.float()).all()
    assert ops.w4_invalid_scales(clear=True) == 0
