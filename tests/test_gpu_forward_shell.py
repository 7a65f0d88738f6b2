"""The shell of the DiT forward around the block loop: each exactly specified piece against the CPU oracle (and, where
built, against the reference's own kernels on the same device buffers), the library bf16 linear against float64, and
b2_dit_forward as a whole against the same sequence of already checked calls (bit for bit), with rows that share a
latent and rows that skip blocks. Modelled on tests/unit/test_moss_dit.cpp of the reference."""
import numpy as np
import pytest
import torch

from oracle import oracle_lib as orc
from oracle import ref_cuda_lib as ref
from owoinfer_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from owoinfer_b200 import ops as o
    yield o
    torch.cuda.synchronize()
    assert o.kernel_status() == (0, 0)


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bf_to_f64(u):
    return (np.asarray(u, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def to_bf16(v):
    u = np.ascontiguousarray(v, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bfdev(u):
    return torch.from_numpy(np.ascontiguousarray(u).view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("c,h,w", [(128, 64, 64), (128, 5, 7), (3, 33, 1), (160, 16, 16)])
def test_transposes(ops, c, h, w):
    rng = np.random.default_rng(c + h)
    lat = rng.normal(0, 2, (c, h, w)).astype(np.float32)
    lat[0, 0, 0], lat[-1, -1, -1] = np.float32(1.00390625), np.float32(-3.3895314e38)   # a rounding tie, near bf16 max
    d = torch.from_numpy(lat).cuda()
    tok = ops.latent_to_tokens(d)
    assert np.array_equal(bits(tok), orc.latent_to_tokens(lat))
    back = ops.tokens_to_latent(tok)
    assert np.array_equal(back.cpu().numpy().view(np.uint32), orc.tokens_to_latent(bits(tok)).view(np.uint32))
    # into a column range of a wider token matrix (the input-extension layout), the rest untouched
    wide = torch.full((h * w, c + 24), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.latent_to_tokens(d, tokens=wide, col0=8)
    assert torch.equal(wide[:, 8:8 + c], tok) and (wide[:, :8] == 7).all() and (wide[:, 8 + c:] == 7).all()
    if ref.has_shell_kernels():
        rt = torch.empty_like(tok)
        ref.latent_to_tokens(d, rt)
        assert torch.equal(rt.view(torch.int16), tok.view(torch.int16))
        rl = torch.empty((c, h, w), dtype=torch.float32, device="cuda")
        ref.tokens_to_latent(tok, rl)
        assert torch.equal(rl.view(torch.int32).reshape(c, -1), back.view(torch.int32))


@pytest.mark.parametrize("n,k", [(18432, 3072), (6144, 3072), (37, 256), (5, 8)])
def test_linear_fp32_row_same_bits(ops, n, k):
    rng = np.random.default_rng(n)
    w = to_bf16(rng.normal(0, 0.03, (n, k)))
    x = rng.normal(0, 1.5, k).astype(np.float32)
    bias = rng.normal(0, 0.5, n).astype(np.float32)
    dw, dx, db = bfdev(w), torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda()
    got = ops.linear_fp32_row(dw, dx, db)
    assert np.array_equal(bits(got), orc.linear_fp32_row(w, x, bias))
    exact = bf_to_f64(w) @ x.astype(np.float64) + bias
    assert np.abs(bf_to_f64(bits(got)) - exact).max() <= 2.0 ** -8 * np.abs(exact).max() + 1e-3
    if ref.has_shell_kernels() and k % 8 == 0:
        want = torch.empty_like(got)
        ref.linear_fp32_row(dw, dx, db, want)
        assert torch.equal(want.view(torch.int16), got.view(torch.int16))


def test_time_modulation_chain(ops):
    """moss_dit.cpp:949-969: host time vector (cached per timestep there), then the two modulation linears."""
    rng = np.random.default_rng(5)
    dim = 3072
    w0, b0 = rng.normal(0, 0.06, (dim, 256)).astype(np.float32), rng.normal(0, 0.1, dim).astype(np.float32)
    w2, b2 = rng.normal(0, 0.02, (dim, dim)).astype(np.float32), rng.normal(0, 0.1, dim).astype(np.float32)
    emb, want = orc.time_vector_fp32(w0, b0, w2, b2, 0.7316)
    assert np.array_equal(ops.time_sinusoid(0.7316).view(np.uint32), emb.view(np.uint32))
    tv = ops.time_vector_fp32(w0, b0, w2, b2, 0.7316)
    assert np.array_equal(tv.view(np.uint32), want.view(np.uint32))
    # against plain float64 linear algebra (a different summation order): close, not identical
    h = w0.astype(np.float64) @ emb + b0
    h = h / (1 + np.exp(-h))
    assert np.allclose(tv, w2.astype(np.float64) @ h.astype(np.float32) + b2, rtol=2e-5, atol=2e-5)
    mw = to_bf16(rng.normal(0, 0.02, (6 * dim, dim)))
    mb = rng.normal(0, 0.2, 6 * dim).astype(np.float32)
    mod = ops.linear_fp32_row(bfdev(mw), torch.from_numpy(tv).cuda(), torch.from_numpy(mb).cuda())
    assert np.array_equal(bits(mod), orc.linear_fp32_row(mw, want, mb))


@pytest.mark.parametrize("m", [1, 9, 64, 4096])
def test_rms_norm_modulate_is_the_quantiser_prologue(ops, m):
    rng = np.random.default_rng(m)
    k = 3072
    x = to_bf16(rng.normal(0, 1, (m, k)))
    w, sc, sh = to_bf16(rng.normal(1, 0.1, k)), to_bf16(rng.normal(0, 0.1, k)), to_bf16(rng.normal(0, 0.1, k))
    y = ops.rms_norm_modulate(bfdev(x), bfdev(w), bfdev(sc), bfdev(sh))
    y2 = torch.empty_like(y)
    ops.rms_norm_modulate_rotate_quantize(bfdev(x), bfdev(w), bfdev(sc), bfdev(sh), y=y2)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    want = orc.rms_norm_modulate(x, w, sc, sh)
    # rsqrtf (GPU) against 1 / sqrt (CPU): rare single-step differences
    assert (bits(y) == want).mean() >= 0.999


@pytest.mark.parametrize("m,n,k,bias", [(4096, 3072, 128, True), (4096, 128, 3072, True), (77, 3072, 128, False), (1, 128, 3072, True)])
def test_linear_bf16_against_float64(ops, m, n, k, bias):
    rng = np.random.default_rng(m + n)
    x, w = to_bf16(rng.normal(0, 1, (m, k))), to_bf16(rng.normal(0, 0.05, (n, k)))
    b = to_bf16(rng.normal(0, 0.5, n)) if bias else None
    got = ops.linear_bf16(bfdev(x), bfdev(w), None if b is None else bfdev(b))
    exact = bf_to_f64(x) @ bf_to_f64(w).T + (bf_to_f64(b) if bias else 0.0)
    err = np.abs(bf_to_f64(bits(got)) - exact)
    # fp32 accumulation in the library's order, one rounding to bf16: within one bf16 step of the exact value
    assert (err <= 2.0 ** -8 * np.abs(exact) + 1e-6 * np.sqrt(k)).all()
    # strided input and output rows
    xw = torch.zeros((m, k + 16), dtype=torch.bfloat16, device="cuda")
    xw[:, :k] = bfdev(x)
    ow = torch.full((m, n + 8), 3.0, dtype=torch.bfloat16, device="cuda")
    ops.linear_bf16(xw[:, :k], bfdev(w), None if b is None else bfdev(b), out=ow[:, :n])
    assert torch.equal(ow[:, :n], got) and (ow[:, n:] == 3).all()


def _model(ops, blocks, F, seed):
    rng = np.random.default_rng(seed)
    D = 3072
    t = lambda a: bfdev(to_bf16(a))
    f = lambda a: torch.from_numpy(a.astype(np.float32)).cuda()
    ws = [synth.block_weights(D, F, seed + 100 * i) for i in range(blocks)]
    bws = [ops.BlockWeights(w["norm1"], w["norm2"], w["q_norm"], w["k_norm"], w["qkv"], w["o"], w["up_gate"], w["down"]) for w in ws]
    parts = dict(block_mod_w=t(rng.normal(0, 0.02, (6 * D, D))), block_mod_bias=f(rng.normal(0, 0.3, 6 * D)),
                 head_mod_w=t(rng.normal(0, 0.02, (2 * D, D))), head_mod_bias=f(rng.normal(0, 0.3, 2 * D)),
                 video_w=t(rng.normal(0, 0.09, (D, 128))), video_bias=t(rng.normal(0, 0.1, D)),
                 final_norm=t(rng.normal(1, 0.1, D)), final_w=t(rng.normal(0, 0.02, (128, D))), final_bias=t(rng.normal(0, 0.1, 128)))
    return ops.DitModel(bws, F, **parts), bws, parts, ws


@pytest.mark.parametrize("skips", [(0, 0, 0), (0, 0b10, 0), (0b01, 0b01, 0b10)])
def test_dit_forward_equals_the_sequence_of_its_parts(ops, skips):
    D, F, h, w = 3072, 8192, 16, 24
    hw = h * w
    model, bws, p, _ = _model(ops, 2, F, 3)
    rng = np.random.default_rng(11)
    latents = torch.from_numpy(rng.normal(0, 1, (2, 128, h, w)).astype(np.float32)).cuda()
    texts = [bfdev(to_bf16(rng.normal(0, 1, (s, D)))) for s in (19, 40, 7)]
    latent_of = (0, 0, 1)
    tv = rng.normal(0, 1, D).astype(np.float32)
    outs, _ = ops.dit_forward(model, latents, tv, [(texts[r], skips[r], latent_of[r]) for r in range(3)])
    torch.cuda.synchronize()

    # The same forward, call by call.
    dtv = torch.from_numpy(tv).cuda()
    mod = ops.linear_fp32_row(p["block_mod_w"], dtv, p["block_mod_bias"])
    head = ops.linear_fp32_row(p["head_mod_w"], dtv, p["head_mod_bias"])
    off = [0]
    for t in texts:
        off.append(off[-1] + hw + t.shape[0])
    x = torch.empty((off[-1], D), dtype=torch.bfloat16, device="cuda")
    rope = torch.empty((off[-1], 128), dtype=torch.bfloat16, device="cuda")
    emb = [ops.linear_bf16(ops.latent_to_tokens(latents[l]), p["video_w"], p["video_bias"]) for l in range(2)]
    for r in range(3):
        x[off[r]:off[r] + hw] = emb[latent_of[r]]
        x[off[r] + hw:off[r + 1]] = texts[r]
        rope[off[r]:off[r + 1]] = ops.moss_rope_table(h, w, texts[r].shape[0])
    for bi in range(2):
        r0 = 0
        while r0 < 3:
            if (skips[r0] >> bi) & 1:
                r0 += 1
                continue
            r1 = r0
            while r1 < 3 and not (skips[r1] >> bi) & 1:
                r1 += 1
            lens = [off[r + 1] - off[r] for r in range(r0, r1)]
            cu = synth.cu_seqlens(lens)
            run = ops.block_run(off[r1] - off[r0], cu, max(lens), D=D, F=F)
            ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
            ops.run_block_quant(bws[bi], ops.block_buffers(x[off[r0]:off[r1]], mod, rope[off[r0]:off[r1]], ws), run)
            r0 = r1
    for r in range(3):
        y = ops.rms_norm_modulate(x[off[r]:off[r] + hw], p["final_norm"], head[D:], head[:D])
        want = ops.tokens_to_latent(ops.linear_bf16(y, p["final_w"], p["final_bias"])).reshape(128, h, w)
        assert torch.equal(outs[r].view(torch.int32), want.view(torch.int32)), f"row {r}"
    assert torch.isfinite(outs[0]).all() and outs[0].abs().max() > 0
    if skips == (0, 0, 0):
        # rows 0 and 1 read the same latent but different text: different outputs
        assert not torch.equal(outs[0], outs[1])


def test_dit_forward_rejects_bad_arguments(ops):
    model, _, _, _ = _model(ops, 1, 8192, 9)
    lat = torch.zeros((1, 128, 4, 4), dtype=torch.float32, device="cuda")
    text = torch.zeros((3, 3072), dtype=torch.bfloat16, device="cuda")
    tv = np.zeros(3072, np.float32)
    with pytest.raises(ValueError, match="latent that is not there"):
        ops.dit_forward(model, lat, tv, [(text, 0, 1)])
    with pytest.raises(ValueError, match="1..8 rows"):
        ops.dit_forward(model, lat, tv, [(text, 0, 0)] * 9)
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    outs, ws = ops.dit_forward(model, lat, tv, [(text, 0, 0)], workspace=small)   # too small a workspace is replaced
    assert ws.numel() > small.numel() and torch.isfinite(outs[0]).all()


@pytest.mark.parametrize("h,w,index", [(16, 24, 0), (5, 3, 2), (1, 1, 7)])
def test_reference_rope_table(ops, h, w, index):
    got = bits(ops.moss_rope_table_reference(h, w, index))
    want = orc.moss_rope_table_reference(h, w, index)
    # sinf / cosf of the device against libm: equal except for rare last-place differences before the bf16 rounding
    assert (got == want).mean() >= 0.9995
    assert np.abs(bf_to_f64(got) - bf_to_f64(want)).max() <= 2.0 ** -7
    # axis r carries index + 1 at every row; the centred coordinates are the image table's
    img = bits(ops.moss_rope_table(h, w, 0))
    assert np.array_equal(got[:, 32:64], img[:h * w, 32:64]) and np.array_equal(got[:, 96:128], img[:h * w, 96:128])


def test_reference_images_prefill_then_forward(ops):
    """prefill_references, then a forward that reads the cache through its slots (moss_dit.cpp:1479-1580, 1283-1300,
    1441-1452), against the same work spelt out call by call with the block-level slots and tap (which
    tests/test_gpu_reference_slots.py holds to plain runs over the longer sequences)."""
    D, F, h, w = 3072, 8192, 16, 16
    hw = h * w
    model, bws, p, _ = _model(ops, 2, F, 5)
    rng = np.random.default_rng(21)
    refs = [torch.from_numpy(rng.normal(0, 1, (128, 8, 16)).astype(np.float32)).cuda(),
            torch.from_numpy(rng.normal(0, 1, (128, 16, 8)).astype(np.float32)).cuda()]
    R = 256
    tv0, tv = rng.normal(0, 1, D).astype(np.float32), rng.normal(0, 1, D).astype(np.float32)
    kv = ops.dit_prefill_references(model, refs, tv0)
    torch.cuda.synchronize()
    assert kv.shape == (2, R, 2 * D) and torch.isfinite(kv.float()).all()

    # The prefill call by call: one sequence of the references' tokens, every block tapped.
    mod0 = ops.linear_fp32_row(p["block_mod_w"], torch.from_numpy(tv0).cuda(), p["block_mod_bias"])
    x = torch.cat([ops.linear_bf16(ops.latent_to_tokens(r), p["video_w"], p["video_bias"]) for r in refs]).contiguous()
    rope = torch.cat([ops.moss_rope_table_reference(8, 16, 0), ops.moss_rope_table_reference(16, 8, 1)]).contiguous()
    cu = synth.cu_seqlens([R])
    for bi in range(2):
        tap = torch.empty((R, 2 * D), dtype=torch.bfloat16, device="cuda")
        run = ops.block_run(R, cu, R, D=D, F=F, kv_tap=tap)
        ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
        ops.run_block_quant(bws[bi], ops.block_buffers(x, mod0, rope, ws), run)
        assert torch.equal(kv[bi].view(torch.int16), tap.view(torch.int16)), f"block {bi}"

    # The forward with references: two rows of one latent; row 0 reads slot A, row 1 slot B.
    latents = torch.from_numpy(rng.normal(0, 1, (1, 128, h, w)).astype(np.float32)).cuda()
    texts = [bfdev(to_bf16(rng.normal(0, 1, (s, D)))) for s in (32, 64)]
    for skips in ((0, 0), (0, 0b01), (0b10, 0)):
        outs, _ = ops.dit_forward(model, latents, tv, [(texts[r], skips[r], 0) for r in range(2)], ref_kv=kv)
        dtv = torch.from_numpy(tv).cuda()
        mod = ops.linear_fp32_row(p["block_mod_w"], dtv, p["block_mod_bias"])
        head = ops.linear_fp32_row(p["head_mod_w"], dtv, p["head_mod_bias"])
        off = [0, hw + 32, 2 * hw + 96]
        xs = torch.empty((off[-1], D), dtype=torch.bfloat16, device="cuda")
        rp = torch.empty((off[-1], 128), dtype=torch.bfloat16, device="cuda")
        emb = ops.linear_bf16(ops.latent_to_tokens(latents[0]), p["video_w"], p["video_bias"])
        for r in range(2):
            xs[off[r]:off[r] + hw] = emb
            xs[off[r] + hw:off[r + 1]] = texts[r]
            rp[off[r]:off[r + 1]] = ops.moss_rope_table(h, w, texts[r].shape[0])
        for bi in range(2):
            rows = [r for r in range(2) if not (skips[r] >> bi) & 1]
            if rows == [0, 1]:
                lens = [off[1] - off[0], off[2] - off[1]]
                run = ops.block_run(off[2], synth.cu_seqlens(lens), max(lens) + R, D=D, F=F, slot_rows=R, slot_kv=(kv[bi], kv[bi]),
                                    cu_seqlens_k=synth.cu_seqlens([lens[0] + R, lens[1] + R]), k0=0, k1=off[2] + 2 * R)
                view = xs
                rview = rp
            elif rows == [1]:   # row 1 alone: not at row 0, so its keys are [own | slot B]
                n = off[2] - off[1]
                run = ops.block_run(n, synth.cu_seqlens([n]), n + R, D=D, F=F, slot_rows=R, slot_kv=(None, kv[bi]),
                                    cu_seqlens_k=synth.cu_seqlens([n + R]), k0=R, k1=R + n + R)
                view, rview = xs[off[1]:], rp[off[1]:]
            else:               # row 0 alone: its keys are [slot A | own]
                n = off[1]
                run = ops.block_run(n, synth.cu_seqlens([n]), n + R, D=D, F=F, slot_rows=R, slot_kv=(kv[bi], None),
                                    cu_seqlens_k=synth.cu_seqlens([n + R]), k0=0, k1=R + n)
                view, rview = xs[:off[1]], rp[:off[1]]
            ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
            ops.run_block_quant(bws[bi], ops.block_buffers(view, mod, rview, ws), run)
        for r in range(2):
            y = ops.rms_norm_modulate(xs[off[r]:off[r] + hw], p["final_norm"], head[D:], head[:D])
            want = ops.tokens_to_latent(ops.linear_bf16(y, p["final_w"], p["final_bias"])).reshape(128, h, w)
            assert torch.equal(outs[r].view(torch.int32), want.view(torch.int32)), f"skips {skips} row {r}"
    # the references matter: without them the outputs differ
    plain, _ = ops.dit_forward(model, latents, tv, [(texts[r], 0, 0) for r in range(2)])
    with_refs, _ = ops.dit_forward(model, latents, tv, [(texts[r], 0, 0) for r in range(2)], ref_kv=kv)
    assert not torch.equal(plain[0], with_refs[0])
    with pytest.raises(ValueError, match="one latent and at most 2 rows"):
        ops.dit_forward(model, latents, tv, [(texts[0], 0, 0)] * 3, ref_kv=kv)


def test_input_extension(ops):
    """set_input_extension (moss_dit.cpp:1118-1133): the embedder reads [latent | extra] channels."""
    D, F, h, w, c = 3072, 8192, 8, 8, 16
    rng = np.random.default_rng(31)
    _, bws, p, _ = _model(ops, 1, F, 6)
    ext_w, ext_b = bfdev(to_bf16(rng.normal(0, 0.08, (D, 128 + c)))), bfdev(to_bf16(rng.normal(0, 0.1, D)))
    model = ops.DitModel(bws, F, p["block_mod_w"], p["block_mod_bias"], p["head_mod_w"], p["head_mod_bias"], None, None,
                         p["final_norm"], p["final_w"], p["final_bias"], ext_w=ext_w, ext_bias=ext_b)
    latents = torch.from_numpy(rng.normal(0, 1, (1, 128, h, w)).astype(np.float32)).cuda()
    extra = torch.from_numpy(rng.normal(0, 1, (1, c, h, w)).astype(np.float32)).cuda()
    text = bfdev(to_bf16(rng.normal(0, 1, (9, D))))
    tv = rng.normal(0, 1, D).astype(np.float32)
    got, _ = ops.dit_forward(model, latents, tv, [(text, 0, 0)], extra=extra)
    # the same with a plain embedder over the concatenated channels folded by hand
    tok = torch.empty((h * w, 128 + c), dtype=torch.bfloat16, device="cuda")
    ops.latent_to_tokens(latents[0], tokens=tok)
    ops.latent_to_tokens(extra[0], tokens=tok, col0=128)
    emb = ops.linear_bf16(tok, ext_w, ext_b)
    dtv = torch.from_numpy(tv).cuda()
    mod = ops.linear_fp32_row(p["block_mod_w"], dtv, p["block_mod_bias"])
    head = ops.linear_fp32_row(p["head_mod_w"], dtv, p["head_mod_bias"])
    x = torch.cat([emb, text]).contiguous()
    n = x.shape[0]
    run = ops.block_run(n, synth.cu_seqlens([n]), n, D=D, F=F)
    ws = torch.empty(ops.block_quant_workspace_bytes(run), dtype=torch.uint8, device="cuda")
    ops.run_block_quant(bws[0], ops.block_buffers(x, mod, ops.moss_rope_table(h, w, 9), ws), run)
    y = ops.rms_norm_modulate(x[:h * w], p["final_norm"], head[D:], head[:D])
    want = ops.tokens_to_latent(ops.linear_bf16(y, p["final_w"], p["final_bias"])).reshape(128, h, w)
    assert torch.equal(got[0].view(torch.int32), want.view(torch.int32))
    with pytest.raises(ValueError, match="extra latents"):
        ops.dit_forward(model, latents, tv, [(text, 0, 0)])


def test_step_graphs_replay_the_forward(ops):
    """b2_dit_forward_graphed: the first call of a key captures (or, when a capture cannot be made, runs eagerly), later
    calls replay; the time vector is not part of the graph; a new shape is a new graph; the oldest graph leaves a full
    cache. Every output equals the eager forward's bit for bit."""
    D, F, h, w = 3072, 8192, 8, 12
    model, _, _, _ = _model(ops, 2, F, 5)
    rng = np.random.default_rng(17)
    latents = torch.from_numpy(rng.normal(0, 1, (1, 128, h, w)).astype(np.float32)).cuda()
    texts = [bfdev(to_bf16(rng.normal(0, 1, (s, D)))) for s in (19, 40)]
    tvs = [rng.normal(0, 1, D).astype(np.float32) for _ in range(3)]
    rows = [(texts[0], 0, 0), (texts[1], 0b10, 0)]
    want = [[o.clone() for o in ops.dit_forward(model, latents, tv, rows)[0]] for tv in tvs]
    torch.cuda.synchronize()
    assert not torch.equal(want[0][0], want[1][0])

    graphs = ops.DitGraphs(capacity=1)
    assert graphs.stats() == dict(replays=0, captures=0, collisions=0, eager=0, evictions=0, size=0)
    side = torch.cuda.Stream()
    outs = ws = None
    with torch.cuda.stream(side):
        for i, tv in enumerate(tvs + tvs[:1]):
            outs, ws = ops.dit_forward(model, latents, tv, rows, graphs=graphs, outs=outs, workspace=ws)
            side.synchronize()
            for r in range(2):
                assert torch.equal(outs[r].view(torch.int32), want[i % 3][r].view(torch.int32)), (i, r)
        st = graphs.stats()
        # A cold process may run the first forward eagerly (one-time set-up cannot be captured); it captures on the next call.
        assert st["captures"] == 1 and st["size"] == 1 and st["captures"] + st["eager"] + st["replays"] == 4
        assert st["replays"] >= 2 and graphs.last_replayed and st["collisions"] == 0

        # Another text length: another key. Capacity 1: the first graph leaves.
        rows2 = [(texts[1], 0, 0)]
        want2 = ops.dit_forward(model, latents, tvs[0], rows2)[0][0].clone()
        outs2, ws2 = ops.dit_forward(model, latents, tvs[0], rows2, graphs=graphs)
        side.synchronize()
        assert torch.equal(outs2[0].view(torch.int32), want2.view(torch.int32))
        st2 = graphs.stats()
        assert st2["captures"] == 2 and st2["evictions"] == 1 and st2["size"] == 1 and not graphs.last_replayed
        outs2, ws2 = ops.dit_forward(model, latents, tvs[1], rows2, graphs=graphs, outs=outs2, workspace=ws2)
        side.synchronize()
        assert graphs.last_replayed
        graphs.clear()
        assert graphs.stats()["size"] == 0

    # The default stream cannot be captured: refused before anything runs.
    with pytest.raises(ValueError, match="default stream"):
        ops.dit_forward(model, latents, tvs[0], rows, graphs=graphs)
    # Capacity 0: always eager.
    none = ops.DitGraphs(capacity=0)
    with torch.cuda.stream(side):
        o, _ = ops.dit_forward(model, latents, tvs[2], rows, graphs=none)
        side.synchronize()
    assert torch.equal(o[0].view(torch.int32), want[2][0].view(torch.int32)) and none.stats()["eager"] == 1
    graphs.close()
    none.close()
    assert ops.kernel_status() == (0, 0)


def test_step_graphs_with_reference_images(ops):
    """A captured forward with a reference cache (slot copies inside the blocks) equals the eager one; the reference
    cache's address is part of the key."""
    D, F, h, w = 3072, 8192, 16, 16
    model, _, _, _ = _model(ops, 2, F, 8)
    rng = np.random.default_rng(33)
    refs = [torch.from_numpy(rng.normal(0, 1, (128, 8, 16)).astype(np.float32)).cuda()]
    tv0, tv = rng.normal(0, 1, D).astype(np.float32), rng.normal(0, 1, D).astype(np.float32)
    kv = ops.dit_prefill_references(model, refs, tv0)
    latents = torch.from_numpy(rng.normal(0, 1, (1, 128, h, w)).astype(np.float32)).cuda()
    texts = [bfdev(to_bf16(rng.normal(0, 1, (s, D)))) for s in (32, 64)]
    rows = [(texts[0], 0, 0), (texts[1], 0b01, 0)]
    want = [o.clone() for o in ops.dit_forward(model, latents, tv, rows, ref_kv=kv)[0]]
    torch.cuda.synchronize()
    graphs = ops.DitGraphs(capacity=4)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        outs = ws = None
        for _ in range(3):
            outs, ws = ops.dit_forward(model, latents, tv, rows, ref_kv=kv, graphs=graphs, outs=outs, workspace=ws)
            side.synchronize()
            for r in range(2):
                assert torch.equal(outs[r].view(torch.int32), want[r].view(torch.int32)), r
        assert graphs.last_replayed and graphs.stats()["captures"] == 1
        kv2 = kv.clone()
        ops.dit_forward(model, latents, tv, rows, ref_kv=kv2, graphs=graphs, outs=outs, workspace=ws)
        side.synchronize()
        assert not graphs.last_replayed and graphs.stats()["captures"] == 2      # another cache address: another graph
        assert torch.equal(outs[0].view(torch.int32), want[0].view(torch.int32))
    graphs.close()
    assert ops.kernel_status() == (0, 0)


def test_silu_and_the_bf16_time_modulation(ops):
    """kernels::silu within one bf16 step of the float64 value (expf differs from libm by an ulp at most), and
    MossDit::time_modulation's bf16 form (moss_dit.cpp:970-990) against float64 on the same bf16 weights: the linears are
    the library's (cuBLASLt, as in the reference), so the bar is bf16 rounding of a 3072-term sum, not bits."""
    rng = np.random.default_rng(41)
    x = bfdev(to_bf16(rng.normal(0, 3, 4099)))
    got = ops.silu_bf16(x).float().cpu().numpy().astype(np.float64)
    xv = x.float().cpu().numpy().astype(np.float64)
    want = xv / (1.0 + np.exp(-xv))
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-30)

    D = 3072
    t = lambda a: bfdev(to_bf16(a))
    w = dict(in_w=t(rng.normal(0, 0.06, (D, 256))), in_bias=t(rng.normal(0, 0.1, D)), out_w=t(rng.normal(0, 0.02, (D, D))),
             out_bias=t(rng.normal(0, 0.1, D)), block_mod_w=t(rng.normal(0, 0.02, (6 * D, D))), block_mod_bias=t(rng.normal(0, 0.3, 6 * D)),
             head_mod_w=t(rng.normal(0, 0.02, (2 * D, D))), head_mod_bias=t(rng.normal(0, 0.3, 2 * D)))
    f64 = {k: v.float().cpu().numpy().astype(np.float64) for k, v in w.items()}
    rb = lambda a: to_bf16(a).view(np.uint16).astype(np.uint32).__lshift__(16).view(np.float32).astype(np.float64)
    for timestep in (0.0, 0.731, 640.0):
        mod, head = ops.time_modulation_bf16(**w, timestep=timestep)
        phase = np.float64(np.float32(timestep)) * 10000.0 ** (-np.arange(128, dtype=np.float64) / 128)
        emb = rb(np.concatenate([np.cos(phase), np.sin(phase)]).astype(np.float32).astype(np.float64))
        hid = rb(f64["in_w"] @ emb + f64["in_bias"])
        hid = rb(hid / (1.0 + np.exp(-hid)))
        tim = rb(f64["out_w"] @ hid + f64["out_bias"])
        for got_t, wt, bias in ((mod, "block_mod_w", "block_mod_bias"), (head, "head_mod_w", "head_mod_bias")):
            want = f64[wt] @ tim + f64[bias]
            g = got_t.float().cpu().numpy().astype(np.float64)
            assert np.abs(g - want).max() <= 0.02 * np.abs(want).max(), (timestep, wt, np.abs(g - want).max(), np.abs(want).max())
            assert np.corrcoef(g, want)[0, 1] >= 0.9999


def test_dit_forward_with_given_modulation_vectors(ops):
    """b2_forward::mod / head: a forward handed the vectors it would have computed from the time vector gives the same
    bits, eagerly and through the step graphs (where the two buffers are inputs like any other)."""
    D, F, h, w = 3072, 8192, 8, 8
    model, _, p, _ = _model(ops, 2, F, 12)
    rng = np.random.default_rng(43)
    latents = torch.from_numpy(rng.normal(0, 1, (1, 128, h, w)).astype(np.float32)).cuda()
    rows = [(bfdev(to_bf16(rng.normal(0, 1, (24, D)))), 0, 0)]
    tv = rng.normal(0, 1, D).astype(np.float32)
    want = ops.dit_forward(model, latents, tv, rows)[0][0].clone()
    dtv = torch.from_numpy(tv).cuda()
    mod = ops.linear_fp32_row(p["block_mod_w"], dtv, p["block_mod_bias"])
    head = ops.linear_fp32_row(p["head_mod_w"], dtv, p["head_mod_bias"])
    got = ops.dit_forward(model, latents, None, rows, mod=mod, head=head)[0][0]
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    with pytest.raises(ValueError, match="go together"):
        ops.dit_forward(model, latents, tv, rows, mod=mod)
    graphs = ops.DitGraphs(capacity=2)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        outs = ws = None
        for _ in range(2):
            outs, ws = ops.dit_forward(model, latents, None, rows, mod=mod, head=head, graphs=graphs, outs=outs, workspace=ws)
            side.synchronize()
            assert torch.equal(outs[0].view(torch.int32), want.view(torch.int32))
        assert graphs.last_replayed
        mod.mul_(0.5)                                   # other contents, same buffers: the same graph, another result
        outs, ws = ops.dit_forward(model, latents, None, rows, mod=mod, head=head, graphs=graphs, outs=outs, workspace=ws)
        side.synchronize()
        assert graphs.last_replayed and not torch.equal(outs[0].view(torch.int32), want.view(torch.int32))
    graphs.close()
