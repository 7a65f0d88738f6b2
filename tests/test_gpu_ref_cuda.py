"""Same-GPU parity: this library's kernels against the reference's own CUDA kernels (compiled for sm_100a from the
reference tree into oracle/_ref/libref_cuda.so) on the same device buffers. Bit-exact for the quantisers, the three GEMM
epilogues and QK-norm + RoPE; attention is compared through its output: both kernels against exact fp32 attention (the
e4m3 rounding of P differs between the two, see the test). Skipped where the
reference build is absent."""
import pytest
import torch

from oracle import ref_cuda_lib as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not ref.available():
        pytest.skip("reference CUDA kernels were not built (oracle/_ref/libref_cuda.so)")
    from owoinfer_b200 import ops as o
    yield o
    torch.cuda.synchronize()
    assert o.kernel_status() == (0, 0)


def _bits(t):
    return t.contiguous().view(torch.int16) if t.dtype == torch.bfloat16 else t.contiguous().view(torch.int32) \
        if t.dtype == torch.float32 else t


def same(a, b):
    return torch.equal(_bits(a), _bits(b))


@pytest.mark.parametrize("m,k", [(1000, 3072), (517, 12288), (64, 256)])
def test_rotate_quantize_same_bits(ops, m, k):
    from owoinfer_b200 import synth
    x = synth.activations(m, k, 11 + k)
    q, s = ops.rotate_quantize(x)
    rq, rs = torch.empty_like(q), torch.empty_like(s)
    ref.rotate_quantize(x, rq, rs)
    assert same(q, rq) and same(s, rs)


@pytest.mark.parametrize("m,k", [(1280, 3072), (4106, 3072), (333, 512)])
def test_norm_modulate_rotate_quantize_same_bits(ops, m, k):
    from owoinfer_b200 import synth
    x = synth.activations(m, k, 21 + m)
    w, sc, sh = synth.vector(k, 1, 0.1, 1.0), synth.vector(k, 2, 0.1), synth.vector(k, 3, 0.1)
    q, s = ops.rms_norm_modulate_rotate_quantize(x, w, sc, sh)
    rq, rs = torch.empty_like(q), torch.empty_like(s)
    ref.rms_norm_modulate_rotate_quantize(x, w, sc, sh, rq, rs)
    # rsqrtf is an approximation on both sides and identical hardware: the same bits.
    assert same(q, rq) and same(s, rs)


@pytest.mark.parametrize("m,n,k", [(1000, 1536, 3072), (4106, 3072, 3072), (130, 512, 12288)])
def test_int8_gemm_epilogues_same_bits(ops, m, n, k):
    from owoinfer_b200 import synth
    x = synth.activations(m, k, 31 + m)
    xq, xs = ops.rotate_quantize(x)
    w, ws = synth.convrot_int8_weight(n, k, 41 + n)
    bias, gate = synth.vector(n, 5, 0.05), synth.vector(n, 6, 0.3)
    out = ops.int8_gemm(xq, xs, w, ws, bias=bias)
    rout = torch.empty_like(out)
    ref.int8_gemm(xq, xs, w, ws, rout, bias=bias)
    assert same(out, rout)
    res = synth.activations(m, n, 51)
    a, b = res.clone(), res.clone()
    ops.int8_gemm_gated_residual(xq, xs, w, ws, gate, a, bias=bias)
    ref.int8_gemm_gated_residual(xq, xs, w, ws, gate, b, bias=bias)
    assert same(a, b)
    glu = ops.int8_gemm_situ_glu(xq, xs, w, ws)
    rglu = torch.empty_like(glu)
    ref.int8_gemm_situ_glu(xq, xs, w, ws, rglu)
    assert same(glu, rglu)


def test_qk_norm_rope_same_bits(ops):
    from owoinfer_b200 import synth
    heads, L = 6, 777
    qkv = synth.activations(L, 3 * heads * 128, 61)
    qn, kn = synth.vector(128, 7, 0.1, 1.0), synth.vector(128, 8, 0.1, 1.0)
    table = ops.moss_rope_table(16, 16, L - 256)
    a, b = qkv.clone(), qkv.clone()
    ops.qk_norm_rope_moss(a, heads, qn, kn, table)
    ref.qk_norm_rope(b, heads, qn, kn, table)
    assert same(a, b)


def _exact_attention(src, lens, heads, scale):
    """fp32 softmax attention per sequence and head on bf16 [total, 3, heads, 128] inputs (head by head: a 20480-key score
    matrix of one head is 1.7 GB in fp32)."""
    total = src.shape[0]
    s4 = src.view(total, 3, heads, 128)
    exact = torch.empty((total, heads, 128), dtype=torch.float32, device="cuda")
    start = 0
    for n in lens:
        for h in range(heads):
            q, k, vv = (s4[start:start + n, i, h].float() for i in range(3))
            p = torch.softmax(q @ k.t() * scale, dim=-1)
            exact[start:start + n, h] = p @ vv
            del p
        start += n
    return exact


def _attention_three_way(ops, qkv, lens, heads, fused, variant=3):
    """This library's attention, the reference's kernel and exact fp32 attention on the same inputs. Returns the L2 and
    worst-element errors of both kernels against exact attention and their mutual L2 distance."""
    from owoinfer_b200 import synth
    total = sum(lens)
    cu = synth.cu_seqlens(lens)
    qn, kn = synth.vector(128, 7, 0.1, 1.0), synth.vector(128, 8, 0.1, 1.0)
    table = ops.moss_rope_table(1, 1, total - 1)
    v = qkv.clone().view(total, 3, heads, 128)  # the fused pre-pass writes the normalised, rotated k back in place
    out = torch.zeros((total, heads, 128), dtype=torch.bfloat16, device="cuda")
    nr = (qn, kn, table) if fused else None
    ops.attention_q8(v[:, 0], v[:, 1], v[:, 2], out, cu, cu, max(lens), ops.SM_SCALE, norm_rope=nr,
                     options=ops.attention_options(variant=variant))
    rout = torch.zeros((total, heads * 128), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(max(256, ref.attention_workspace_bytes(total, len(lens), max(lens), heads)), dtype=torch.uint8,
                     device="cuda")
    ref.attention_q8(qkv.clone(), heads, rout, cu, max(lens), ops.SM_SCALE, ws, nr, variant=variant)
    src = qkv.clone()
    if fused:
        ops.qk_norm_rope_moss(src, heads, qn, kn, table)
    e = _exact_attention(src, lens, heads, ops.SM_SCALE).view(total, -1)
    g, w = out.float().view(total, -1), rout.float()
    err = lambda a: ((a - e).norm() / e.norm()).item()
    worst = lambda a: ((a - e).abs().max() / e.abs().max()).item()
    return dict(ours=err(g), ref=err(w), ours_worst=worst(g), ref_worst=worst(w), mutual=((g - w).norm() / w.norm()).item())


# Same quantised operands and statistics on both sides. P is rounded to e4m3 after a shift by a reference maximum; this
# library raises that maximum only when its headroom runs out (fewer rescales of O), so single P values round differently
# from the reference's and the two outputs differ by about the sum of their own e4m3 errors (up to ~3 % of the output
# norm on flat scores). The bar: as close to exact attention as the reference's kernel (10 % slack on the L2 error, a
# factor 2 on the single worst element) and within 5 % (L2) of the reference's output.
def _check_three_way(r):
    assert r["mutual"] <= 0.05, r
    assert r["ours"] <= 1.1 * r["ref"] + 1e-5, r
    assert r["ours_worst"] <= 2.0 * r["ref_worst"] + 1e-5, r


@pytest.mark.parametrize("lens,fused", [([1280], 0), ([700, 333], 0), ([3200], 1)])
def test_attention_close_to_reference_kernel(ops, lens, fused):
    from owoinfer_b200 import synth
    heads, total = 4, sum(lens)
    qkv = synth.activations(total, 3 * heads * 128, 71 + total)
    _check_three_way(_attention_three_way(ops, qkv, lens, heads, fused))


@pytest.mark.parametrize("lens,fused", [([1280], 0), ([700, 333], 1), ([8192], 1)])
def test_attention_int8_fp8_variant_close_to_reference_kernel(ops, lens, fused):
    """Variant int8_fp8 (the High tier's default: P in [0, 112], V in [-4.5, 4.5]; attention_q8.h:79-88). The reference adds
    each 64-key tile in fp16 and flushes it into fp32; this library adds in fp32 throughout with the variant's ranges, and
    has to be as close to exact attention as the reference's kernel."""
    if not ref.has_attention_variants():
        pytest.skip("the reference shim predates the variant entry")
    from owoinfer_b200 import synth
    total = sum(lens)
    heads = 24 if total >= 8192 else 4
    qkv = synth.activations(total, 3 * heads * 128, 171 + total)
    r = _attention_three_way(ops, qkv, lens, heads, fused, variant=ops.ATTENTION_Q8_FP8)
    print("int8_fp8", lens, r)
    _check_three_way(r)
    r3 = _attention_three_way(ops, qkv, lens, heads, fused)
    assert abs(r["ours"] - r3["ours"]) <= 0.5 * r3["ours"] + 1e-4, (r, r3)   # the narrower ranges cost little


@pytest.mark.parametrize("lens", [[8192], [20480]])
def test_attention_at_benchmark_lengths(ops, lens):
    """The benchmarked attention shapes: one 8192-token sequence (1024^2) and one 20480-token sequence (2048^2) with all
    24 heads and the fused QK-norm + RoPE pre-pass; 64 / 160 query tiles per head and 128 / 320 sub-tiles per row."""
    from owoinfer_b200 import synth
    heads, total = 24, sum(lens)
    qkv = synth.activations(total, 3 * heads * 128, 91 + total)
    r = _attention_three_way(ops, qkv, lens, heads, 1)
    print("attention", lens, r)
    _check_three_way(r)


@pytest.mark.parametrize("keys", [4608, 16384])
def test_attention_peaked_scores(ops, keys):
    """One dominant key per query row over a long flat tail (test_attention_q8.cu:211-218 shapes its inputs the same way to
    reach the low end of the e4m3 range): key j is a scaled copy of query j, so row j's score for key j stands 2^12
    (4608 keys) or 2^14 (16384 keys) above the tail, whose summed weight is still comparable to the dominant key's. The
    reference maximum of this library's softmax sits up to three binades above the row maximum, so the tail's P values
    reach the subnormal end of e4m3 earlier than in the reference's kernel; the output must stay as close to exact
    attention as the reference's."""
    heads = 2
    torch.manual_seed(keys)
    q = torch.randn((keys, heads, 128), device="cuda")
    beta = 9.0 if keys == 4608 else 10.5
    k = beta * q / q.norm(dim=-1, keepdim=True) + 0.02 * torch.randn_like(q)
    v = torch.randn_like(q)
    qkv = torch.stack([q, k, v], dim=1).to(torch.bfloat16).view(keys, 3 * heads * 128).contiguous()
    r = _attention_three_way(ops, qkv, [keys], heads, 0)
    print("peaked", keys, r)
    _check_three_way(r)


def _block_metrics(got, want):
    """cos; max|g-w| / max|w| (a norm-type bound, as the reference's own block tests use); the per-element error
    max |g-w| / (|w| + rms(w)), whose denominator is the element's own size floored at the tensor's rms, so that a large
    value in an outlier channel cannot hide an error on an ordinary element (a floor much below the rms would instead
    measure bf16 rounding flips on elements near zero); and the relative L2 error."""
    g, t = got.float().flatten(), want.float().flatten()
    cos = torch.nn.functional.cosine_similarity(g, t, dim=0).item()
    max_rel = ((g - t).abs().max() / t.abs().max()).item()
    rms = t.pow(2).mean().sqrt()
    per_elem = ((g - t).abs() / (t.abs() + rms)).max().item()
    rel_l2 = ((g - t).norm() / t.norm()).item()
    return cos, max_rel, per_elem, rel_l2


def _ours_vs_ref_block(ops, lens, F, grid, seed, tier=0, attention_variant=3):
    from owoinfer_b200 import synth
    D, heads = 3072, 24
    L = sum(lens)
    x = synth.activations(L, D, 1000 + seed)
    mod = synth.modulation(D, 2000 + seed)
    w = synth.block_weights(D, F, 3000 + seed, tier=tier)
    rope = torch.cat([ops.moss_rope_table(grid, grid, n - grid * grid) for n in lens]).contiguous()
    cu = synth.cu_seqlens(lens)
    run = ops.block_run(L, cu, max(lens), D=D, F=F, heads=heads, tier=tier)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    if tier == ops.TIER_W4A8:
        lin = {n: ops.make_w4(w[n][0], w[n][1], 64, w[n][2]) for n in ("qkv", "o", "up_gate", "down")}
        # What the reference does with such a weight: decode to the INT8 grid, then its INT8 kernels.
        w8 = dict(w)
        for n in lin:
            w8[n] = (ops.decode_grouped_int8(w[n][0], w[n][1], 64), w[n][2])
    else:
        lin, w8 = w, w
    bw = ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], lin["qkv"], lin["o"], lin["up_gate"], lin["down"])
    got = x.clone()
    ops.run_block_quant(bw, ops.block_buffers(got, mod, rope, ws), run)
    want = x.clone()
    ref.RefBlock(L, cu, max(lens), D, F, heads).run(want, mod, rope, w8, ops.SM_SCALE)
    torch.cuda.synchronize()
    return _block_metrics(got, want)


def test_block_close_to_reference_kernels(ops):
    cos, max_rel, per_elem, rel_l2 = _ours_vs_ref_block(ops, [1280], 12288, 32, 7)
    assert cos >= 0.9995 and max_rel <= 1e-2, (cos, max_rel, per_elem, rel_l2)


def test_block_with_the_high_tier_default_attention(ops):
    """AttentionMode::kQ8Fp8 (dit_block_quant.h:60-68), the High tier's default: this library's block with variant int8_fp8
    against the reference's kernels with theirs, one 8192-token sequence at full width."""
    if not ref.has_attention_variants():
        pytest.skip("the reference shim predates the variant entry")
    cos, max_rel, per_elem, rel_l2 = _ours_vs_ref_block(ops, [8192], 12288, 64, 19, attention_variant=ops.ATTENTION_Q8_FP8)
    print("block int8_fp8", dict(cos=cos, max_rel=max_rel, per_elem=per_elem, rel_l2=rel_l2))
    assert cos >= 0.9995 and max_rel <= 1e-2, (cos, max_rel, per_elem, rel_l2)


# The benchmarked block shapes (d = 3072, 24 heads, MLP 12288): one 8192-token sequence, the CFG pair of a 1024^2 step,
# one 20480-token sequence of a 2048^2 step; and the grouped 4-bit tier at full width. Gates: cosine >= 0.9995 and
# max|g-w| / max|w| <= 1e-2 (the reading of "max-relative-error 1e-2" that the reference's own block tests use,
# tests/unit/test_dit_int8.cpp:307-341), plus the per-element error of _block_metrics, printed and bounded.
@pytest.mark.parametrize("lens,grid,tier,w4_route", [([8192], 64, 0, -1), ([8192, 8192], 64, 0, -1), ([20480], 128, 0, -1),
                                                     ([8192], 64, 2, -1), ([8192], 64, 2, 1)])
def test_block_at_benchmark_shapes(ops, lens, grid, tier, w4_route):
    ops.debug_w4a8_route(w4_route)   # the grouped 4-bit tier through its automatic route and through the fused kernel
    try:
        cos, max_rel, per_elem, rel_l2 = _ours_vs_ref_block(ops, lens, 12288, grid, 11 + len(lens) + tier, tier)
    finally:
        ops.debug_w4a8_route(-1)
    print("block", lens, "tier", tier, dict(cos=cos, max_rel=max_rel, per_elem=per_elem, rel_l2=rel_l2))
    assert cos >= 0.9995 and max_rel <= 1e-2, (cos, max_rel, per_elem, rel_l2)
    assert per_elem <= 5e-2 and rel_l2 <= 1e-2, (cos, max_rel, per_elem, rel_l2)
