"""ctypes bindings of oracle/_ref/libref_cuda.so: the reference's own CUDA kernels for the quantized block, compiled
for sm_100a from the reference tree (`make -C oracle ref_cuda`). TEST INFRASTRUCTURE ONLY: the same-GPU checker of the
parity tests and the "reference kernels on this GPU" timing leg of bench.py; the product path never loads it.

Arguments are torch CUDA tensors; work is queued on torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import os

_DIR = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_DIR, "_ref", "libref_cuda.so")
_lib = None
vp, i64, i32, f32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t


def available() -> bool:
    return os.path.exists(_PATH)


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(_PATH)
        l.ref_last_error.restype = C.c_char_p
        l.ref_rotate_quantize.argtypes = [vp, i64, vp, i64, vp, i64, i32, vp]
        l.ref_rms_norm_modulate_rotate_quantize.argtypes = [vp, i64, vp, vp, vp, vp, i64, vp, i64, i32, vp]
        l.ref_int8_gemm.argtypes = [vp, i64, vp, vp, vp, i64, i64, i64, vp, vp, i64, vp]
        l.ref_int8_gemm_gated_residual.argtypes = [vp, i64, vp, vp, vp, i64, i64, i64, vp, vp, vp, i64, vp]
        l.ref_int8_gemm_situ_glu.argtypes = [vp, i64, vp, vp, vp, i64, i64, i64, vp, i64, vp]
        l.ref_qk_norm_rope.argtypes = [vp, i64, i64, i32, vp, vp, vp, i64, vp]
        l.ref_attention_q8_workspace_bytes.restype = sz
        l.ref_attention_q8_workspace_bytes.argtypes = [i64, i32, i32, i32]
        l.ref_attention_q8.argtypes = [vp, i64, i64, i32, vp, i64, vp, i32, i32, f32, vp, sz, i32, vp, vp, vp, vp]
        if hasattr(l, "ref_attention_q8_variant"):
            l.ref_attention_q8_variant.argtypes = [i32, f32, f32, vp, i64, i64, i32, vp, i64, vp, i32, i32, f32, vp, sz, i32, vp, vp, vp, vp]
        if hasattr(l, "ref_cfg_velocity"):
            l.ref_cfg_velocity.argtypes = [vp, vp, f32, vp, i64, vp]
            l.ref_slg_velocity.argtypes = [vp, vp, vp, f32, vp, i64, vp]
            l.ref_velocity_euler.argtypes = [vp, vp, f32, i64, vp]
            l.ref_ab2.argtypes = [vp, vp, vp, f32, f32, f32, i64, vp]
        if hasattr(l, "ref_linear_fp32_row"):
            l.ref_latent_to_tokens.argtypes = [vp, i64, i64, i64, vp, vp]
            l.ref_tokens_to_latent.argtypes = [vp, i64, i64, i64, vp, vp]
            l.ref_linear_fp32_row.argtypes = [vp, i64, i64, vp, vp, vp, vp]
        _lib = l
    return _lib


def _stream():
    import torch
    return vp(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else vp(t.data_ptr())


def _ok(rc):
    if rc != 0:
        raise RuntimeError("reference kernel: " + lib().ref_last_error().decode())


def rotate_quantize(x, q, scale):
    m, k = x.shape
    _ok(lib().ref_rotate_quantize(_p(x), x.stride(0), _p(q), q.stride(0), _p(scale), m, k, _stream()))


def rms_norm_modulate_rotate_quantize(x, w, mod_scale, mod_shift, q, scale):
    m, k = x.shape
    _ok(lib().ref_rms_norm_modulate_rotate_quantize(_p(x), x.stride(0), _p(w), _p(mod_scale), _p(mod_shift), _p(q),
                                                    q.stride(0), _p(scale), m, k, _stream()))


def int8_gemm(xq, xs, w, ws, out, bias=None):
    (m, k), n = xq.shape, w.shape[0]
    _ok(lib().ref_int8_gemm(_p(xq), xq.stride(0), _p(xs), _p(w), _p(ws), m, n, k, _p(bias), _p(out), out.stride(0),
                            _stream()))


def int8_gemm_gated_residual(xq, xs, w, ws, gate, residual, bias=None):
    (m, k), n = xq.shape, w.shape[0]
    _ok(lib().ref_int8_gemm_gated_residual(_p(xq), xq.stride(0), _p(xs), _p(w), _p(ws), m, n, k, _p(bias), _p(gate),
                                           _p(residual), residual.stride(0), _stream()))


def int8_gemm_situ_glu(xq, xs, w, ws, out):
    (m, k), n = xq.shape, w.shape[0]
    _ok(lib().ref_int8_gemm_situ_glu(_p(xq), xq.stride(0), _p(xs), _p(w), _p(ws), m, n, k, _p(out), out.stride(0),
                                     _stream()))


def qk_norm_rope(qkv, heads, q_norm, k_norm, table):
    _ok(lib().ref_qk_norm_rope(_p(qkv), qkv.stride(0), qkv.shape[0], heads, _p(q_norm), _p(k_norm), _p(table),
                               table.stride(0), _stream()))


def attention_workspace_bytes(total, batch, max_seqlen, heads) -> int:
    return int(lib().ref_attention_q8_workspace_bytes(total, batch, max_seqlen, heads))


def has_attention_variants() -> bool:
    return hasattr(lib(), "ref_attention_q8_variant")


def attention_q8(qkv, heads, out, cu, max_seqlen, scale, workspace, norm_rope=None, variant=3, p_range=0.0, v_range=0.0):
    """Self-attention over a fused [total, 3 * heads * 128] buffer; norm_rope = (q_norm, k_norm, table) fuses QK-norm +
    RoPE into the pre-pass (the buffer itself is then left as it was). variant 2 = int8_fp8 (fp16 tile accumulation,
    ranges 112 / 4.5 by default), 3 = int8_fp8_f32acc."""
    nr = norm_rope or (None, None, None)
    if variant != 3 or p_range or v_range:
        _ok(lib().ref_attention_q8_variant(variant, p_range, v_range, _p(qkv), qkv.stride(0), qkv.shape[0], heads, _p(out),
                                           out.stride(0), _p(cu), cu.numel() - 1, max_seqlen, scale, _p(workspace),
                                           workspace.numel(), 1 if norm_rope else 0, _p(nr[0]), _p(nr[1]), _p(nr[2]), _stream()))
        return
    _ok(lib().ref_attention_q8(_p(qkv), qkv.stride(0), qkv.shape[0], heads, _p(out), out.stride(0), _p(cu),
                               cu.numel() - 1, max_seqlen, scale, _p(workspace), workspace.numel(),
                               1 if norm_rope else 0, _p(nr[0]), _p(nr[1]), _p(nr[2]), _stream()))


def cfg_velocity(c, u, g, out):
    _ok(lib().ref_cfg_velocity(_p(c), _p(u), g, _p(out), c.numel(), _stream()))


def slg_velocity(p, c, k, s, out):
    _ok(lib().ref_slg_velocity(_p(p), _p(c), _p(k), s, _p(out), c.numel(), _stream()))


def velocity_euler(x, v, h):
    _ok(lib().ref_velocity_euler(_p(x), _p(v), h, x.numel(), _stream()))


def ab2(x, v, v_prev, h, a, b):
    _ok(lib().ref_ab2(_p(x), _p(v), _p(v_prev), h, a, b, x.numel(), _stream()))


def latent_to_tokens(latents, tokens):
    c, h, w = latents.shape
    _ok(lib().ref_latent_to_tokens(_p(latents), c, h, w, _p(tokens), _stream()))


def tokens_to_latent(tokens, latents):
    c, h, w = latents.shape
    _ok(lib().ref_tokens_to_latent(_p(tokens), c, h, w, _p(latents), _stream()))


def linear_fp32_row(w, x, bias, out):
    _ok(lib().ref_linear_fp32_row(_p(w), w.shape[0], w.shape[1], _p(x), _p(bias), _p(out), _stream()))


def has_shell_kernels() -> bool:
    return available() and hasattr(lib(), "ref_linear_fp32_row")


def has_sampler_kernels() -> bool:
    return available() and hasattr(lib(), "ref_cfg_velocity")


class RefBlock:
    """The all-INT8 block sequenced over the reference's kernels the way its run_block_quant does
    (src/models/moss_dit/dit_block_quant.cpp: norm+quantize, qkv GEMM, 8-bit attention with the fused norm+RoPE pre-pass,
    rotate, o-proj GEMM with gated residual, norm+quantize, up_gate GEMM with SiTU-GLU, rotate, down GEMM with residual)."""

    def __init__(self, tokens, cu, max_seqlen, D, F, heads, attention_variant=3):
        import torch
        dev = "cuda"
        self.D, self.F, self.heads, self.cu, self.max_seqlen = D, F, heads, cu, max_seqlen
        self.attention_variant = attention_variant
        self.xq = torch.empty((tokens, max(D, F)), dtype=torch.int8, device=dev)
        self.scale = torch.empty(tokens, dtype=torch.float32, device=dev)
        self.qkv = torch.empty((tokens, 3 * D), dtype=torch.bfloat16, device=dev)
        self.attn = torch.empty((tokens, D), dtype=torch.bfloat16, device=dev)
        self.ffn = torch.empty((tokens, F), dtype=torch.bfloat16, device=dev)
        self.ws = torch.empty(max(256, attention_workspace_bytes(tokens, cu.numel() - 1, max_seqlen, heads)),
                              dtype=torch.uint8, device=dev)

    def run(self, x, mod, rope, w, sm_scale):
        D, F = self.D, self.F
        m = [mod[i * D:(i + 1) * D] for i in range(6)]
        xq_d, xq_f = self.xq[:, :D], self.xq[:, :F]
        rms_norm_modulate_rotate_quantize(x, w["norm1"], m[1], m[0], xq_d, self.scale)
        int8_gemm(xq_d, self.scale, w["qkv"][0], w["qkv"][1], self.qkv)
        attention_q8(self.qkv, self.heads, self.attn, self.cu, self.max_seqlen, sm_scale, self.ws,
                     (w["q_norm"], w["k_norm"], rope), variant=self.attention_variant)
        rotate_quantize(self.attn, xq_d, self.scale)
        int8_gemm_gated_residual(xq_d, self.scale, w["o"][0], w["o"][1], m[2], x)
        rms_norm_modulate_rotate_quantize(x, w["norm2"], m[4], m[3], xq_d, self.scale)
        int8_gemm_situ_glu(xq_d, self.scale, w["up_gate"][0], w["up_gate"][1], self.ffn)
        rotate_quantize(self.ffn, xq_f, self.scale)
        int8_gemm_gated_residual(xq_f, self.scale, w["down"][0], w["down"][1], m[5], x)
        return x
