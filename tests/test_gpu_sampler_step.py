"""Guidance and velocity update of a denoising step: the four separate entry points and the fused single pass against
the CPU oracle (one fp32 rounding per op, the reference's order) and, where built, against the reference's own sampler
kernels on the same device buffers. Bit-exact. Modelled on PipelineKernels.GuidanceAndIntegratorsMatchTorchOpOrder of the
reference (tests/unit/test_pipeline.cpp:212-242): same odd length, same scalars."""
import itertools

import numpy as np
import pytest
import torch

from oracle import oracle_lib as orc
from oracle import ref_cuda_lib as ref

pytestmark = pytest.mark.gpu

G, S, H, KA, KB = 3.7, 0.85, -0.0412, 1.31, 0.31


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from owoinfer_b200 import ops as o
    return o


def _inputs(n, seed=7, offset=0):
    rng = np.random.default_rng(seed)
    host = [rng.normal(0.0, 1.5, n + offset).astype(np.float32) for _ in range(5)]
    devs = [torch.from_numpy(h).cuda()[offset:] for h in host]
    return [h[offset:] for h in host], devs


def _same(t, a):
    return np.array_equal(t.cpu().numpy().view(np.uint32), np.asarray(a, dtype=np.float32).view(np.uint32))


@pytest.mark.parametrize("n,offset", [(100003, 0), (1 << 20, 0), (4096, 1), (3, 0), (0, 0)])
def test_separate_ops_match_oracle(ops, n, offset):
    (a, b, c, x, _), (da, db, dc, dx, _) = _inputs(n, offset=offset)
    assert _same(ops.cfg_combine(da, db, G), orc.cfg_combine(a, b, G))
    assert _same(ops.slg_correct(da, db, dc, S), orc.slg_correct(a, b, c, S))
    assert _same(ops.euler_update(dx.clone(), da, H), orc.euler_update(x, a, H))
    assert _same(ops.ab2_update(dx.clone(), da, db, H, KA, KB), orc.ab2_update(x, a, b, H, KA, KB))


@pytest.mark.parametrize("cfg,slg,update", list(itertools.product([0, 1], [0, 1], [0, 1, 2])))
def test_fused_step_matches_sequence(ops, cfg, slg, update):
    n = 256 * 4096  # the fp32 latent of a 1024^2 image: 64 channels x 128 x 128
    (c, u, k, x, vp), (dc, du, dk, dx, dvp) = _inputs(n, seed=11)
    v = orc.guided_velocity(c, u if cfg else None, k if slg else None, G, S)
    want_x = x if update == 0 else orc.euler_update(x, v, H) if update == 1 else orc.ab2_update(x, v, vp, H, KA, KB)
    v_out = torch.empty_like(dc)
    got_x = dx.clone()
    ops.guided_velocity_step(dc, x=got_x, v_uncond=du if cfg else None, v_skip=dk if slg else None, v_prev=dvp if update == 2 else None,
                             v_out=v_out, cfg_scale=G, slg_scale=S, h=H, a=KA, b=KB, update=update)
    assert _same(v_out, v)
    assert _same(got_x, want_x)
    if update:  # without the velocity store
        again = dx.clone()
        ops.guided_velocity_step(dc, x=again, v_uncond=du if cfg else None, v_skip=dk if slg else None,
                                 v_prev=dvp if update == 2 else None, cfg_scale=G, slg_scale=S, h=H, a=KA, b=KB, update=update)
        assert _same(again, want_x)


def test_fused_step_in_place_velocity(ops):
    """v_out may be v_cond's own buffer (the reference's guide_prediction writes into a separate tensor; in place saves one)."""
    (c, u, _, x, _), (dc, du, _, dx, _) = _inputs(65536, seed=3)
    v = orc.cfg_combine(c, u, G)
    ops.guided_velocity_step(dc, x=dx, v_uncond=du, v_out=dc, cfg_scale=G, h=H, update=1)
    assert _same(dc, v) and _same(dx, orc.euler_update(x, v, H))


def test_rejects_bad_steps(ops):
    _, (dc, du, dk, dx, dvp) = _inputs(64)
    with pytest.raises(ValueError, match="v_uncond with cfg"):
        _raw_step(ops, dc, dx, cfg=1)
    with pytest.raises(ValueError, match="needs v_prev"):
        ops.guided_velocity_step(dc, x=dx, update=2)
    with pytest.raises(ValueError, match="nothing to write"):
        ops.guided_velocity_step(dc, update=0)
    with pytest.raises(ValueError, match="alias"):
        ops.guided_velocity_step(dc, x=dx, v_prev=dvp, v_out=dvp, update=2)


def _raw_step(ops, dc, dx, cfg):
    import ctypes as C
    from owoinfer_b200 import _lib
    g = _lib.GuidedStep()
    g.struct_size = C.sizeof(_lib.GuidedStep)
    g.x, g.v_cond, g.cfg, g.update, g.n = dx.data_ptr(), dc.data_ptr(), cfg, 1, dc.numel()
    ops.check(_lib.lib().b2_guided_velocity_step(C.byref(g), None))


def test_same_bits_as_reference_sampler_kernels(ops):
    if not ref.has_sampler_kernels():
        pytest.skip("reference sampler kernels were not built (oracle/_ref/libref_cuda.so)")
    n = 100003
    _, (da, db, dc, dx, _) = _inputs(n)
    want = torch.empty_like(da)
    ref.cfg_velocity(da, db, G, want)
    assert torch.equal(ops.cfg_combine(da, db, G).view(torch.int32), want.view(torch.int32))
    ref.slg_velocity(da, db, dc, S, want)
    assert torch.equal(ops.slg_correct(da, db, dc, S).view(torch.int32), want.view(torch.int32))
    rx, ox = dx.clone(), dx.clone()
    ref.velocity_euler(rx, da, H)
    assert torch.equal(ops.euler_update(ox, da, H).view(torch.int32), rx.view(torch.int32))
    rx, ox = dx.clone(), dx.clone()
    ref.ab2(rx, da, db, H, KA, KB)
    assert torch.equal(ops.ab2_update(ox, da, db, H, KA, KB).view(torch.int32), rx.view(torch.int32))
    # The whole guided AB2 step in one launch against the reference's four.
    rv, rx, ox = torch.empty_like(da), dx.clone(), dx.clone()
    ref.cfg_velocity(da, db, G, rv)
    ref.slg_velocity(rv, da, dc, S, rv)
    ref.ab2(rx, rv, db, H, KA, KB)
    ov = torch.empty_like(da)
    ops.guided_velocity_step(da, x=ox, v_uncond=db, v_skip=dc, v_prev=db, v_out=ov, cfg_scale=G, slg_scale=S, h=H, a=KA, b=KB,
                             update=2)
    assert torch.equal(ov.view(torch.int32), rv.view(torch.int32)) and torch.equal(ox.view(torch.int32), rx.view(torch.int32))
