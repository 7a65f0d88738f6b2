"""ctypes bindings of the CPU oracle (oracle/oracle.cpp). TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the product path
(owoinfer_b200) never does. bf16 tensors travel as numpy uint16 arrays holding the raw bits.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_DIR, "liboracle.so")
_REF_PATH = os.path.join(_DIR, "_ref", "libref_codec.so")


def reference_root():
    """Where the reference engine's source tree is, or None: the MOSSINFER_REFERENCE environment variable, else a
    directory named `reference` beside this repository."""
    env = os.environ.get("MOSSINFER_REFERENCE")
    if env:
        return env if os.path.isdir(env) else None
    beside = os.path.join(os.path.dirname(os.path.dirname(_DIR)), "reference")
    return beside if os.path.isdir(os.path.join(beside, "src")) else None


def make_args():
    ref = reference_root()
    return ["make", "-C", _DIR] + ([f"REF={ref}"] if ref else [])


def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref/libref_codec.so when the reference tree is present)."""
    src = os.path.join(_DIR, "oracle.cpp")
    stale = not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(make_args() + ["-B", "all"], stdout=subprocess.DEVNULL)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_up_gate_row.restype = C.c_int64
        _lib.orc_up_gate_row.argtypes = [C.c_int64, C.c_int64]
    return _lib


def ref_codec():
    """The reference's own CPU codec behind a C shim, or None where it was not built (no reference tree)."""
    if not os.path.exists(_REF_PATH):
        return None
    r = C.CDLL(_REF_PATH)
    r.ref_e4m3_to_float.restype = C.c_float
    r.ref_e4m3_to_float.argtypes = [C.c_uint8]
    return r


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


i64, f32, i32 = C.c_int64, C.c_float, C.c_int


def set_threads(n: int) -> None:
    lib().orc_set_threads(i32(n))


def rotate_quantize(x):
    x = _c(x, np.uint16)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    lib().orc_rotate_quantize(_p(x), i64(k), _p(q), i64(k), _p(s), i64(m), i32(k))
    return q, s


def rms_norm_modulate(x, w, sc, sh):
    x = _c(x, np.uint16)
    m, k = x.shape
    y = np.empty((m, k), np.uint16)
    rc = lib().orc_rms_norm_modulate(_p(x), i64(k), _p(_c(w, np.uint16)), _p(_c(sc, np.uint16)), _p(_c(sh, np.uint16)),
                                     _p(y), i64(k), i64(m), i32(k))
    if rc != 0:
        raise ValueError("row length needs torch's cross-warp split")
    return y


def rms_norm_modulate_rotate_quantize(x, w, sc, sh, want_y=False):
    x = _c(x, np.uint16)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    y = np.empty((m, k), np.uint16) if want_y else None
    rc = lib().orc_rms_norm_modulate_rotate_quantize(_p(x), i64(k), _p(_c(w, np.uint16)), _p(_c(sc, np.uint16)),
                                                     _p(_c(sh, np.uint16)), _p(q), i64(k), _p(s), i64(m), i32(k),
                                                     _p(y), i64(k))
    if rc != 0:
        raise ValueError("row length needs torch's cross-warp split")
    return (q, s, y) if want_y else (q, s)


def convrot_quantize_int4(x):
    x = _c(x, np.uint16)
    m, k = x.shape
    q = np.empty((m, k // 2), np.uint8)
    s = np.empty(m, np.float32)
    lib().orc_convrot_quantize_int4(_p(x), i64(k), _p(q), i64(k // 2), _p(s), i64(m), i32(k))
    return q, s


def rms_norm_modulate_convrot_quantize_int4(x, w, sc, sh):
    x = _c(x, np.uint16)
    m, k = x.shape
    q = np.empty((m, k // 2), np.uint8)
    s = np.empty(m, np.float32)
    rc = lib().orc_rms_norm_modulate_convrot_quantize_int4(_p(x), i64(k), _p(_c(w, np.uint16)), _p(_c(sc, np.uint16)),
                                                           _p(_c(sh, np.uint16)), _p(q), i64(k // 2), _p(s), i64(m),
                                                           i32(k))
    if rc != 0:
        raise ValueError("row length needs torch's cross-warp split")
    return q, s


def unpack_int4(packed):
    packed = _c(packed, np.uint8)
    rows, kb = packed.shape
    out = np.empty((rows, kb * 2), np.int8)
    lib().orc_unpack_int4(_p(packed), i64(kb), _p(out), i64(kb * 2), i64(rows), i64(kb * 2))
    return out


def decode_grouped_int8(packed, s_rel, group, codebook=None):
    """s_rel: uint8 (e4m3 bits) or uint16 (fp16 bits) [rows, k/group]."""
    packed = _c(packed, np.uint8)
    rows, kb = packed.shape
    k = kb * 2
    kind = 0 if s_rel.dtype == np.uint8 else 1
    s_rel = np.ascontiguousarray(s_rel)
    cb = None if codebook is None else _c(codebook, np.float32)
    out = np.empty((rows, k), np.int8)
    rc = lib().orc_decode_grouped_int8(_p(packed), _p(s_rel), i32(kind), _p(cb), i64(rows), i64(k), i32(group), _p(out))
    if rc != 0:
        raise ValueError("invalid group scale")
    return out


def decode_grouped_int8_device_rule(packed, s_rel, group, codebook=None):
    """The GPU kernel's rule for untrusted scales: (int8 [rows, k], invalid word); bad groups decode to zeros."""
    packed = _c(packed, np.uint8)
    rows, kb = packed.shape
    k = kb * 2
    kind = 0 if s_rel.dtype == np.uint8 else 1
    s_rel = np.ascontiguousarray(s_rel)
    cb = None if codebook is None else _c(codebook, np.float32)
    out = np.empty((rows, k), np.int8)
    invalid = C.c_uint(0)
    lib().orc_decode_grouped_int8_device_rule(_p(packed), _p(s_rel), i32(kind), _p(cb), i64(rows), i64(k), i32(group),
                                              _p(out), C.byref(invalid))
    return out, int(invalid.value)


def quantize_convrot_rows_bf16(w, g=256):
    w = _c(w, np.uint16)
    rows, k = w.shape
    q = np.empty((rows, k), np.int8)
    s = np.empty(rows, np.float32)
    lib().orc_quantize_convrot_rows_bf16(_p(w), i64(rows), i64(k), i32(g), _p(q), _p(s))
    return q, s


def int8_gemm_acc(xq, wq):
    xq, wq = _c(xq, np.int8), _c(wq, np.int8)
    m, k = xq.shape
    n = wq.shape[0]
    acc = np.empty((m, n), np.int32)
    lib().orc_int8_gemm_acc(_p(xq), i64(k), _p(wq), i64(m), i64(n), i64(k), _p(acc), i64(n))
    return acc


def int8_gemm(xq, xs, wq, ws, bias=None):
    xq, wq = _c(xq, np.int8), _c(wq, np.int8)
    m, k = xq.shape
    n = wq.shape[0]
    out = np.empty((m, n), np.uint16)
    b = None if bias is None else _c(bias, np.uint16)
    lib().orc_int8_gemm(_p(xq), i64(k), _p(_c(xs, np.float32)), _p(wq), _p(_c(ws, np.float32)), i64(m), i64(n), i64(k),
                        _p(b), _p(out), i64(n))
    return out


def int8_gemm_gated_residual(xq, xs, wq, ws, gate, residual, bias=None):
    xq, wq = _c(xq, np.int8), _c(wq, np.int8)
    m, k = xq.shape
    n = wq.shape[0]
    res = np.array(residual, dtype=np.uint16, copy=True, order="C")
    b = None if bias is None else _c(bias, np.uint16)
    lib().orc_int8_gemm_gated_residual(_p(xq), i64(k), _p(_c(xs, np.float32)), _p(wq), _p(_c(ws, np.float32)), i64(m),
                                       i64(n), i64(k), _p(b), _p(_c(gate, np.uint16)), _p(res), i64(n))
    return res


def int8_gemm_situ_glu(xq, xs, wq, ws):
    xq, wq = _c(xq, np.int8), _c(wq, np.int8)
    m, k = xq.shape
    n2 = wq.shape[0]
    out = np.empty((m, n2 // 2), np.uint16)
    lib().orc_int8_gemm_situ_glu(_p(xq), i64(k), _p(_c(xs, np.float32)), _p(wq), _p(_c(ws, np.float32)), i64(m), i64(n2),
                                 i64(k), _p(out), i64(n2 // 2))
    return out


def up_gate_row(n, half):
    return int(lib().orc_up_gate_row(n, half))


def situ_glu(up_gate):
    up_gate = _c(up_gate, np.uint16)
    m, f2 = up_gate.shape
    out = np.empty((m, f2 // 2), np.uint16)
    lib().orc_situ_glu(_p(up_gate), i64(f2), _p(out), i64(f2 // 2), i64(m), i64(f2 // 2))
    return out


def situ_tables():
    gate = np.empty(65536, np.uint16)
    hidden = np.empty(65536, np.uint16)
    lib().orc_situ_tables(_p(gate), _p(hidden))
    return gate, hidden


def qk_norm_rope(qkv, heads, q_norm, k_norm, table):
    qkv = np.array(qkv, dtype=np.uint16, copy=True, order="C")
    tokens, ld = qkv.shape
    table = _c(table, np.uint16)
    lib().orc_qk_norm_rope(_p(qkv), i64(ld), i64(tokens), i32(heads), _p(_c(q_norm, np.uint16)),
                           _p(_c(k_norm, np.uint16)), _p(table), i64(table.shape[1]))
    return qkv


MOSS_ROPE_BANDS = (np.float32(1.0) / np.power(np.float32(10000.0), np.arange(16, dtype=np.float32) / np.float32(16))).astype(np.float32)


def moss_rope_table(height, width, text_length, bands=None):
    n = height * width + text_length
    out = np.empty((n, 128), np.uint16)
    b = _c(MOSS_ROPE_BANDS if bands is None else bands, np.float32)
    lib().orc_moss_rope_table(_p(out), i64(128), i32(height), i32(width), i32(text_length), _p(b))
    return out


def moss_rope_table_reference(height, width, index, bands=None):
    out = np.empty((height * width, 128), np.uint16)
    b = _c(MOSS_ROPE_BANDS if bands is None else bands, np.float32)
    lib().orc_moss_rope_table_reference(_p(out), i64(128), i32(height), i32(width), i32(index), _p(b))
    return out


def attention_prepass(qkv, cu, heads, max_seqlen, v_range=448.0):
    """qkv: uint16 [total, 3*heads*128] (q | k | v columns). Returns dict of natural-layout outputs."""
    qkv = _c(qkv, np.uint16)
    total, ld = qkv.shape
    cu = _c(cu, np.int32)
    batch = len(cu) - 1
    qb, kb = (max_seqlen + 127) // 128 * 4, (max_seqlen + 63) // 64
    o = dict(q_i8=np.zeros((total, heads, 128), np.int8), k_i8=np.zeros((total, heads, 128), np.int8),
             v8=np.zeros((total, heads, 128), np.uint8), q_scale=np.zeros((batch, heads, qb), np.float32),
             k_scale=np.zeros((batch, heads, kb), np.float32), k_mean=np.zeros((batch, heads, 128), np.float32),
             v_scale=np.zeros((batch, heads, 128), np.float32))
    base = qkv.ctypes.data
    hd = heads * 128 * 2
    lib().orc_attention_prepass(C.c_void_p(base), C.c_void_p(base + hd), C.c_void_p(base + 2 * hd), i64(ld), _p(cu),
                                i32(batch), i32(heads), i32(max_seqlen), f32(v_range), _p(o["q_i8"]), _p(o["k_i8"]),
                                _p(o["v8"]), _p(o["q_scale"]), _p(o["k_scale"]), _p(o["k_mean"]), _p(o["v_scale"]))
    return o


def qk_scores(q_i8, k_i8, head, q0, qn, k0, kn):
    heads = q_i8.shape[1]
    s = np.empty((qn, kn), np.int32)
    lib().orc_qk_scores(_p(_c(q_i8, np.int8)), _p(_c(k_i8, np.int8)), i32(heads), i32(head), i64(q0), i32(qn), i64(k0),
                        i32(kn), _p(s))
    return s


def attention_q8(qkv, cu, heads, max_seqlen, sm_scale, p_range=448.0, v_range=448.0, norm_rope=None):
    """Returns (out uint16 [total, heads*128], qkv after the optional in-place norm + RoPE)."""
    qkv = np.array(qkv, dtype=np.uint16, copy=True, order="C")
    total, ld = qkv.shape
    cu = _c(cu, np.int32)
    out = np.zeros((total, heads * 128), np.uint16)
    if norm_rope is None:
        qn = kn = tab = None
        tld = 0
    else:
        qn, kn, tab = (_c(a, np.uint16) for a in norm_rope)
        tld = tab.shape[1]
    lib().orc_attention_q8(_p(qkv), i64(ld), _p(cu), i32(len(cu) - 1), i32(heads), i32(max_seqlen), f32(sm_scale),
                           f32(p_range), f32(v_range), i32(0 if norm_rope is None else 1), _p(qn), _p(kn), _p(tab),
                           i64(tld), _p(out), i64(heads * 128))
    return out, qkv


def attention_exact(q, k, v, cu, sm_scale):
    """q, k, v: uint16 [total, heads, 128] contiguous. Returns float32 [total, heads, 128]."""
    q, k, v = (_c(a, np.uint16) for a in (q, k, v))
    total, heads, _ = q.shape
    cu = _c(cu, np.int32)
    out = np.zeros((total, heads, 128), np.float32)
    lib().orc_attention_exact(_p(q), _p(k), _p(v), i64(heads * 128), _p(cu), i32(len(cu) - 1), i32(heads), f32(sm_scale),
                              _p(out))
    return out


def block_quant(x, mod, rope, w, cu, max_seqlen, heads=24, p_range=448.0, v_range=448.0, tier=0):
    """w: dict with norm1, norm2, q_norm, k_norm (uint16) and qkv/o/up/down = (int8 weight, f32 scale)."""
    x = np.array(x, dtype=np.uint16, copy=True, order="C")
    L, D = x.shape
    F = w["down"][0].shape[1]
    cu = _c(cu, np.int32)
    args = [_p(x), i64(L), i32(D), i32(F), i32(heads), _p(_c(mod, np.uint16)), _p(_c(rope, np.uint16)),
            _p(_c(w["norm1"], np.uint16)), _p(_c(w["norm2"], np.uint16)), _p(_c(w["q_norm"], np.uint16)),
            _p(_c(w["k_norm"], np.uint16))]
    keep = []
    for name in ("qkv", "o", "up", "down"):
        wq, ws = _c(w[name][0], np.int8), _c(w[name][1], np.float32)
        keep += [wq, ws]
        args += [_p(wq), _p(ws)]
    args += [_p(cu), i32(len(cu) - 1), i32(max_seqlen), f32(p_range), f32(v_range), i32(tier)]
    rc = lib().orc_block_quant(*args)
    if rc != 0:
        raise ValueError("orc_block_quant failed")
    return x


# ---------------------------------------------------------------------------------------------- guidance + update
# Four fp32 formulas, one rounding per op, in the reference's order (src/pipeline/samplers/sampler_kernels.cu:209-218,
# 304-310; sequencing src/pipeline/samplers/sampler_driver.cpp:565-577). numpy float32 arithmetic rounds every op once
# and never contracts.

def _f32(a):
    return np.asarray(a, dtype=np.float32)


def cfg_combine(cond, uncond, g):
    c, u, g = _f32(cond), _f32(uncond), np.float32(g)
    return u + g * (c - u)


def slg_correct(pred, cond, skipped, scale):
    p, c, k, s = _f32(pred), _f32(cond), _f32(skipped), np.float32(scale)
    return p + s * (c - k)


def euler_update(x, v, h):
    return _f32(x) + np.float32(h) * _f32(v)


def ab2_update(x, v, v_prev, h, a, b):
    d = np.float32(a) * _f32(v) - np.float32(b) * _f32(v_prev)
    return _f32(x) + np.float32(h) * d


def guided_velocity(v_cond, v_uncond=None, v_skip=None, cfg_scale=0.0, slg_scale=0.0):
    """guide_prediction in velocity space: CFG, then SLG on its result (on v_skip itself when CFG is off)."""
    v = _f32(v_cond)
    if v_uncond is not None:
        v = cfg_combine(v_cond, v_uncond, cfg_scale)
    if v_skip is not None:
        v = slg_correct(v if v_uncond is not None else v_skip, v_cond, v_skip, slg_scale)
    return v


# ---------------------------------------------------------------------------------------------- forward shell

def linear_fp32_row(w_bits, x, bias):
    """bf16 bits [n, k], f32 [k], f32 [n] -> bf16 bits [n], in the reference kernel's order (dit_kernels.cu:79-93)."""
    w = _c(w_bits, np.uint16)
    n, k = w.shape
    out = np.empty(n, np.uint16)
    lib().orc_linear_fp32_row(_p(w), _p(_c(x, np.float32)), _p(_c(bias, np.float32)), _p(out), i32(n), i32(k))
    return out


def time_vector_fp32(w0, b0, w2, b2, timestep):
    """distill.cpp:126-150. Returns (sinusoid f32 [256], time vector f32 [dim])."""
    w0, b0, w2, b2 = (_c(a, np.float32) for a in (w0, b0, w2, b2))
    dim = w2.shape[0]
    emb, time = np.empty(256, np.float32), np.empty(dim, np.float32)
    lib().orc_time_vector_fp32(_p(w0), _p(b0), _p(w2), _p(b2), i64(dim), C.c_float(timestep), _p(emb), _p(time))
    return emb, time


def latent_to_tokens(latents):
    """f32 [C, hw] -> bf16 bits [hw, C] (dit_kernels.cu:19-47: transpose, round to nearest even)."""
    v = np.ascontiguousarray(np.asarray(latents, np.float32).reshape(latents.shape[0], -1).T)
    u = v.view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def tokens_to_latent(tokens_bits):
    """bf16 bits [hw, C] -> f32 [C, hw]."""
    return np.ascontiguousarray((np.asarray(tokens_bits, np.uint16).astype(np.uint32) << 16).view(np.float32).T)
