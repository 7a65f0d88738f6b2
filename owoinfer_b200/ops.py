"""Host-side mirror of the reference's kernel-level interface for the quantized DiT block, over torch CUDA tensors.

Same names, argument meaning and error behaviour as the reference's C++ entry points (kernels::quant::*,
kernels::quant4::*, attention_q8::attention_q8, kernels::fused::qk_norm_rope_moss, moss_dit::run_block_quant); every
function calls straight into the C ABI of libowoinfer_b200.so on the current torch stream. torch is used for device
memory and streams only. Invalid arguments raise ValueError (the reference throws std::invalid_argument).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import check

TILE_AUTO, TILE_128x256, TILE_128x128, TILE_2CTA_256x256 = 0, 1, 2, 3
TIER_INT8, TIER_W4A4_VIA_INT8, TIER_W4A8 = 0, 1, 2
ATTENTION_Q8_FP8 = 2          # e4m3 P.V with the ranges of the fp16-accumulating variant (112 / 4.5); accumulated in fp32 here
ATTENTION_Q8_FP8_F32ACC = 3


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _ld(t) -> int:
    return t.stride(0) if t.dim() == 2 and t.shape[0] > 1 else t.shape[-1]


# ------------------------------------------------------------------------------------------------ quantisers

def rotate_quantize(x, q=None, scale=None):
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device) if q is None else q
    scale = torch.empty(m, dtype=torch.float32, device=x.device) if scale is None else scale
    check(_lib.lib().b2_rotate_quantize(_ptr(x), C.c_int64(_ld(x)), _ptr(q), C.c_int64(_ld(q)), _ptr(scale), C.c_int64(m),
                                        C.c_int(k), _stream()))
    return q, scale


def rms_norm_modulate_rotate_quantize(x, norm_weight, mod_scale, mod_shift, q=None, scale=None, y=None):
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device) if q is None else q
    scale = torch.empty(m, dtype=torch.float32, device=x.device) if scale is None else scale
    check(_lib.lib().b2_rms_norm_modulate_rotate_quantize(
        _ptr(x), C.c_int64(_ld(x)), _ptr(norm_weight), _ptr(mod_scale), _ptr(mod_shift), _ptr(q), C.c_int64(_ld(q)),
        _ptr(scale), C.c_int64(m), C.c_int(k), _stream(), _ptr(y), C.c_int64(0 if y is None else _ld(y))))
    return q, scale


def convrot_quantize_int4(x, q=None, scale=None):
    m, k = x.shape
    q = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device) if q is None else q
    scale = torch.empty(m, dtype=torch.float32, device=x.device) if scale is None else scale
    check(_lib.lib().b2_convrot_quantize_int4(_ptr(x), C.c_int64(_ld(x)), _ptr(q), C.c_int64(_ld(q)), _ptr(scale),
                                              C.c_int64(m), C.c_int(k), _stream()))
    return q, scale


def rms_norm_modulate_convrot_quantize_int4(x, norm_weight, mod_scale, mod_shift, q=None, scale=None):
    m, k = x.shape
    q = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device) if q is None else q
    scale = torch.empty(m, dtype=torch.float32, device=x.device) if scale is None else scale
    check(_lib.lib().b2_rms_norm_modulate_convrot_quantize_int4(
        _ptr(x), C.c_int64(_ld(x)), _ptr(norm_weight), _ptr(mod_scale), _ptr(mod_shift), _ptr(q), C.c_int64(_ld(q)),
        _ptr(scale), C.c_int64(m), C.c_int(k), _stream()))
    return q, scale


def unpack_int4(packed, out=None):
    rows, kb = packed.shape
    out = torch.empty((rows, kb * 2), dtype=torch.int8, device=packed.device) if out is None else out
    check(_lib.lib().b2_unpack_int4(_ptr(packed), C.c_int64(_ld(packed)), _ptr(out), C.c_int64(_ld(out)), C.c_int64(rows),
                                    C.c_int64(kb * 2), _stream()))
    return out


def decode_grouped_int8(packed, s_rel, group, codebook=None, out=None, invalid=None):
    """invalid: optional uint32/int32 device tensor of one element, OR-ed with 1 when a group scale is NaN or negative."""
    rows, kb = packed.shape
    k = kb * 2
    kind = 0 if s_rel.dtype in (torch.uint8, torch.int8) else 1
    out = torch.empty((rows, k), dtype=torch.int8, device=packed.device) if out is None else out
    check(_lib.lib().b2_decode_grouped_int8(_ptr(packed), _ptr(s_rel), C.c_int(kind), _ptr(codebook), C.c_int64(rows),
                                            C.c_int64(k), C.c_int(group), _ptr(out), _ptr(invalid), _stream()))
    return out


def w4_invalid_scales(clear=False):
    v = C.c_uint(0)
    check(_lib.lib().b2_w4_invalid_scales(C.byref(v), C.c_int(1 if clear else 0)))
    return int(v.value)


# ------------------------------------------------------------------------------------------------ GEMMs

def _operands(x_q, x_scale, w, w_scale):
    m, k = x_q.shape
    return _lib.Int8Operands(x_q.data_ptr(), _ld(x_q), x_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(), m, w.shape[0], k)


def int8_gemm(x_q, x_scale, w, w_scale, bias=None, out=None, tile=TILE_AUTO):
    op = _operands(x_q, x_scale, w, w_scale)
    out = torch.empty((op.m, op.n), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    check(_lib.lib().b2_int8_gemm(C.byref(op), _ptr(bias), _ptr(out), C.c_int64(_ld(out)), _stream(), C.c_int(tile)))
    return out


def int8_gemm_chunked(x_q, x_scale, w, w_scale, chunk_cols, bias=None, out=None, tile=TILE_AUTO):
    """The plain GEMM with its output split by columns: out is [n / chunk_cols, m, chunk_cols]."""
    op = _operands(x_q, x_scale, w, w_scale)
    chunks = op.n // chunk_cols
    out = torch.empty((chunks, op.m, chunk_cols), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    check(_lib.lib().b2_int8_gemm_chunked(C.byref(op), _ptr(bias), _ptr(out), C.c_int64(out.stride(1)), C.c_int(chunk_cols),
                                          C.c_int64(out.stride(0)), _stream(), C.c_int(tile)))
    return out


def rotate_quantize_chunked(x_chunks, q=None, scale=None):
    """x_chunks: bf16 [chunks, m, chunk_cols]; quantises the rows of the column-concatenated [m, chunks * chunk_cols]."""
    chunks, m, cw = x_chunks.shape
    k = chunks * cw
    q = torch.empty((m, k), dtype=torch.int8, device=x_chunks.device) if q is None else q
    scale = torch.empty(m, dtype=torch.float32, device=x_chunks.device) if scale is None else scale
    check(_lib.lib().b2_rotate_quantize_chunked(_ptr(x_chunks), C.c_int64(x_chunks.stride(1)), C.c_int(cw),
                                                C.c_int64(x_chunks.stride(0)), _ptr(q), C.c_int64(_ld(q)), _ptr(scale),
                                                C.c_int64(m), C.c_int(k), _stream()))
    return q, scale


def int8_gemm_gated_residual(x_q, x_scale, w, w_scale, gate, residual, bias=None, tile=TILE_AUTO):
    op = _operands(x_q, x_scale, w, w_scale)
    check(_lib.lib().b2_int8_gemm_gated_residual(C.byref(op), _ptr(bias), _ptr(gate), _ptr(residual),
                                                 C.c_int64(_ld(residual)), _stream(), C.c_int(tile)))
    return residual


def int8_gemm_situ_glu(x_q, x_scale, w, w_scale, out=None, tile=TILE_AUTO):
    op = _operands(x_q, x_scale, w, w_scale)
    out = torch.empty((op.m, op.n // 2), dtype=torch.bfloat16, device=x_q.device) if out is None else out
    check(_lib.lib().b2_int8_gemm_situ_glu(C.byref(op), _ptr(out), C.c_int64(_ld(out)), _stream(), C.c_int(tile)))
    return out


def int8_gemm_acc(x_q, w, tile=TILE_AUTO):
    m, k = x_q.shape
    ones = torch.ones(max(m, w.shape[0], 4), dtype=torch.float32, device=x_q.device)
    op = _operands(x_q, ones, w, ones)
    acc = torch.empty((m, w.shape[0]), dtype=torch.int32, device=x_q.device)
    check(_lib.lib().b2_int8_gemm_acc(C.byref(op), _ptr(acc), C.c_int64(w.shape[0]), _stream(), C.c_int(tile)))
    return acc


def make_w4(packed, s_rel, group, s_channel, codebook=None):
    kind = 0 if s_rel.dtype in (torch.uint8, torch.int8) else 1
    w = _lib.W4Weight(packed.data_ptr(), s_rel.data_ptr(), kind, group, 0 if codebook is None else codebook.data_ptr(),
                      s_channel.data_ptr())
    w._keep = (packed, s_rel, s_channel, codebook)
    return w


def debug_w4a8_route(route: int):
    """-1 automatic, 0 always decode to the scratch, 1 decode inside the GEMM whenever the weight's format allows."""
    check(_lib.lib().b2_debug_w4a8_route(C.c_int(route)))


def w4a8_gemm(x_q, x_scale, w4, n, epilogue=0, aux=None, out=None, scratch=None):
    """scratch: int8 [n, k] for the weights that are decoded ahead of the GEMM (allocated when None); False passes no
    scratch at all (only weights the fused kernel takes: e4m3 scales, tile-sized shapes)."""
    m, k = x_q.shape
    if scratch is False:
        scratch = None
    elif scratch is None:
        scratch = torch.empty((n, k), dtype=torch.int8, device=x_q.device)
    if out is None:
        out = torch.empty((m, n // 2 if epilogue == 2 else n), dtype=torch.bfloat16, device=x_q.device)
    check(_lib.lib().b2_w4a8_gemm(_ptr(x_q), C.c_int64(_ld(x_q)), _ptr(x_scale), C.byref(w4), C.c_int64(m), C.c_int64(n),
                                  C.c_int64(k), C.c_int(epilogue), _ptr(aux), _ptr(out), C.c_int64(_ld(out)),
                                  _ptr(scratch), _stream()))
    return out


# ------------------------------------------------------------------------------------------------ attention side

def qk_norm_rope_moss(qkv, heads, q_norm, k_norm, table):
    check(_lib.lib().b2_qk_norm_rope_moss(_ptr(qkv), C.c_int64(_ld(qkv)), C.c_int64(qkv.shape[0]), C.c_int(heads),
                                          _ptr(q_norm), _ptr(k_norm), _ptr(table), C.c_int64(_ld(table)), _stream()))
    return qkv


def moss_rope_table(height, width, text_length, device="cuda"):
    n = height * width + text_length
    out = torch.empty((n, 128), dtype=torch.bfloat16, device=device)
    check(_lib.lib().b2_moss_rope_table(_ptr(out), C.c_int64(128), C.c_int(height), C.c_int(width), C.c_int(text_length),
                                        _stream()))
    return out


def moss_rope_table_reference(height, width, index, device="cuda"):
    out = torch.empty((height * width, 128), dtype=torch.bfloat16, device=device)
    check(_lib.lib().b2_moss_rope_table_reference(_ptr(out), C.c_int64(128), C.c_int(height), C.c_int(width), C.c_int(index),
                                                  _stream()))
    return out


def _view3(t):
    return _lib.View3(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), t.stride(1))


def attention_options(p_range=0.0, v_range=0.0, variant=ATTENTION_Q8_FP8_F32ACC):
    return _lib.AttentionOptions(variant, p_range, v_range)


def attention_q8_workspace_bytes(total_q, total_k, batch, max_seqlen, heads, kv_heads=None, options=None):
    o = options or attention_options()
    return int(_lib.lib().b2_attention_q8_workspace_bytes(C.byref(o), total_q, total_k, batch, max_seqlen, heads,
                                                          heads if kv_heads is None else kv_heads))


def attention_q8_layout(total_q, total_k, batch, max_seqlen, heads, options=None):
    o = options or attention_options()
    l = _lib.AttentionLayout()
    check(_lib.lib().b2_attention_q8_layout(C.byref(o), C.c_int64(total_q), C.c_int64(total_k), C.c_int(batch),
                                            C.c_int(max_seqlen), C.c_int(heads), C.c_int(heads), C.byref(l)))
    return l


def attention_q8(q, k, v, out, cu_seqlens_q, cu_seqlens_k, max_seqlen, scale, workspace=None, options=None,
                 norm_rope=None):
    """q, k, v, out: bf16 [tokens, heads, 128] views (head_dim contiguous). norm_rope: (q_norm, k_norm, table) or None."""
    o = options or attention_options()
    batch = cu_seqlens_q.shape[0] - 1
    if workspace is None:
        nbytes = attention_q8_workspace_bytes(q.shape[0], k.shape[0], batch, max_seqlen, q.shape[1], k.shape[1], o)
        workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
    nr = None
    if norm_rope is not None:
        nr = _lib.QkNormRope(norm_rope[0].data_ptr(), norm_rope[1].data_ptr(), norm_rope[2].data_ptr(), _ld(norm_rope[2]))
    vq, vk, vv, vo = _view3(q), _view3(k), _view3(v), _view3(out)
    check(_lib.lib().b2_attention_q8(C.byref(o), C.byref(vq), C.byref(vk), C.byref(vv), C.byref(vo), _ptr(cu_seqlens_q),
                                     _ptr(cu_seqlens_k), C.c_int(batch), C.c_int(max_seqlen), C.c_float(scale),
                                     _ptr(workspace), C.c_size_t(workspace.numel()), _stream(),
                                     None if nr is None else C.byref(nr)))
    return out, workspace


def attention_q8_preprocess(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen, workspace=None, options=None, norm_rope=None):
    """The pre-pass of attention_q8 alone; returns the workspace it filled."""
    o = options or attention_options()
    batch = cu_seqlens_q.shape[0] - 1
    if workspace is None:
        nbytes = attention_q8_workspace_bytes(q.shape[0], k.shape[0], batch, max_seqlen, q.shape[1], k.shape[1], o)
        workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
    nr = None
    if norm_rope is not None:
        nr = _lib.QkNormRope(norm_rope[0].data_ptr(), norm_rope[1].data_ptr(), norm_rope[2].data_ptr(), _ld(norm_rope[2]))
    vq, vk, vv = _view3(q), _view3(k), _view3(v)
    check(_lib.lib().b2_attention_q8_preprocess(C.byref(o), C.byref(vq), C.byref(vk), C.byref(vv), _ptr(cu_seqlens_q),
                                                _ptr(cu_seqlens_k), C.c_int(batch), C.c_int(max_seqlen), _ptr(workspace),
                                                C.c_size_t(workspace.numel()), _stream(), None if nr is None else C.byref(nr)))
    return workspace


def attention_q8_debug_scores(q, k, v, out, cu_seqlens_q, cu_seqlens_k, max_seqlen, scale, seq, head, tile_q, workspace=None,
                              options=None, norm_rope=None):
    """attention_q8 that also returns the attention kernel's own int32 Q·K^T accumulators of one (sequence, head, 128-row
    query tile): (int32 [128, 64 * ceil(max_seqlen / 64)], workspace)."""
    o = options or attention_options()
    batch = cu_seqlens_q.shape[0] - 1
    if workspace is None:
        nbytes = attention_q8_workspace_bytes(q.shape[0], k.shape[0], batch, max_seqlen, q.shape[1], k.shape[1], o)
        workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
    nr = None
    if norm_rope is not None:
        nr = _lib.QkNormRope(norm_rope[0].data_ptr(), norm_rope[1].data_ptr(), norm_rope[2].data_ptr(), _ld(norm_rope[2]))
    ld = (max_seqlen + 63) // 64 * 64
    scores = torch.zeros((128, ld), dtype=torch.int32, device=q.device)
    vq, vk, vv, vo = _view3(q), _view3(k), _view3(v), _view3(out)
    check(_lib.lib().b2_attention_q8_debug_scores(C.byref(o), C.byref(vq), C.byref(vk), C.byref(vv), C.byref(vo),
                                                  _ptr(cu_seqlens_q), _ptr(cu_seqlens_k), C.c_int(batch), C.c_int(max_seqlen),
                                                  C.c_float(scale), _ptr(workspace), C.c_size_t(workspace.numel()), _stream(),
                                                  None if nr is None else C.byref(nr), C.c_int(seq), C.c_int(head),
                                                  C.c_int(tile_q), _ptr(scores), C.c_int64(ld)))
    return scores, workspace


def kernel_status():
    g, a = C.c_int(0), C.c_int(0)
    check(_lib.lib().b2_kernel_status(C.byref(g), C.byref(a)))
    return g.value, a.value


def kernel_status_clear():
    check(_lib.lib().b2_kernel_status_clear())


def debug_bounded_wait(wait_limit_ns: int, skip_gemm_stage: bool):
    check(_lib.lib().b2_debug_bounded_wait(C.c_uint64(wait_limit_ns), C.c_int(1 if skip_gemm_stage else 0)))


# ------------------------------------------------------------------------------------------------ block / step

class BlockWeights:
    """Device weights of one all-quantized block (BlockTensors of the reference, restricted to this route).

    qkv / o / up_gate / down: (int8 weight [n, k], f32 scale [n]) for TIER_INT8; (packed int4 uint8 [n, k/2], f32 scale)
    for TIER_W4A4_VIA_INT8; a W4Weight from make_w4 for TIER_W4A8.
    """

    def __init__(self, norm1, norm2, q_norm, k_norm, qkv, o, up_gate, down):
        self.tensors = (norm1, norm2, q_norm, k_norm, qkv, o, up_gate, down)
        s = _lib.BlockWeights()
        s.struct_size = C.sizeof(_lib.BlockWeights)
        s.norm1, s.norm2, s.q_norm, s.k_norm = (t.data_ptr() for t in (norm1, norm2, q_norm, k_norm))
        for name, lin in (("qkv", qkv), ("o", o), ("up_gate", up_gate), ("down", down)):
            l = _lib.Linear()
            if isinstance(lin, _lib.W4Weight):
                l.w4 = C.pointer(lin)
            else:
                l.w, l.scale = lin[0].data_ptr(), lin[1].data_ptr()
            setattr(s, name, l)
        self.struct = s


def block_run(tokens, cu_seqlens, max_seqlen, D=3072, F=12288, heads=24, tier=TIER_INT8, p_range=0.0, v_range=0.0,
              fused_norm_rope=-1, slot_rows=0, slot_kv=(None, None), cu_seqlens_k=None, k0=0, k1=0, kv_tap=None, tap_only=False,
              slot_kv_ld=0, attention_variant=ATTENTION_Q8_FP8_F32ACC):
    r = _lib.BlockRun()
    r.struct_size = C.sizeof(_lib.BlockRun)
    r.tokens, r.D, r.F, r.heads = tokens, D, F, heads
    r.cu_seqlens = cu_seqlens.data_ptr()
    r.batch, r.max_seqlen, r.tier = cu_seqlens.shape[0] - 1, max_seqlen, tier
    r.attention = attention_options(p_range, v_range, attention_variant)
    r.fused_norm_rope = fused_norm_rope
    r.slot_rows, r.k0, r.k1, r.tap_only, r.slot_kv_ld = slot_rows, k0, k1, int(tap_only), slot_kv_ld
    r.slot_kv[0], r.slot_kv[1] = (None if t is None else t.data_ptr() for t in slot_kv)
    r.cu_seqlens_k = None if cu_seqlens_k is None else cu_seqlens_k.data_ptr()
    r.kv_tap = None if kv_tap is None else kv_tap.data_ptr()
    r._keep = (cu_seqlens, slot_kv, cu_seqlens_k, kv_tap)
    return r


def block_quant_workspace_bytes(run) -> int:
    n = int(_lib.lib().b2_block_quant_workspace_bytes(C.byref(run)))
    if n == 0:
        raise ValueError(_lib.lib().b2_last_error_message().decode())
    return n


def block_buffers(x, mod, rope, workspace):
    b = _lib.BlockBuffers()
    b.struct_size = C.sizeof(_lib.BlockBuffers)
    b.x, b.mod, b.rope, b.workspace, b.workspace_bytes = x.data_ptr(), mod.data_ptr(), rope.data_ptr(), workspace.data_ptr(), workspace.numel()
    b._keep = (x, mod, rope, workspace)
    return b


def run_block_quant(weights: BlockWeights, buffers, run):
    check(_lib.lib().b2_run_block_quant(C.byref(weights.struct), C.byref(buffers), C.byref(run), _stream()))


def dit_step(blocks, buffers, run):
    arr = (_lib.BlockWeights * len(blocks))(*[b.struct for b in blocks])
    check(_lib.lib().b2_dit_step(arr, C.c_int(len(blocks)), C.byref(buffers), C.byref(run), _stream()))


SM_SCALE = 1.0 / math.sqrt(128.0)


# ------------------------------------------------------------------------------------------------ sequence parallel

class SpComm:
    """Communicator of one sequence-parallel group (b2_sp_comm). `unique_id` is the bytes rank 0 of the group got from
    sp_unique_id(); size 1 needs none."""

    def __init__(self, size: int, rank: int, unique_id: bytes | None = None):
        self.size, self.rank = size, rank
        self.handle = C.c_void_p()
        buf = (C.c_char * 128).from_buffer_copy(unique_id) if unique_id is not None else None
        check(_lib.lib().b2_sp_comm_create(buf, C.c_size_t(128 if buf is not None else 0), C.c_int(size), C.c_int(rank),
                                           C.byref(self.handle)))

    def local_exchange(self, on: bool):
        check(_lib.lib().b2_sp_comm_local_exchange(self.handle, C.c_int(1 if on else 0)))

    def close(self):
        if self.handle:
            _lib.lib().b2_sp_comm_destroy(self.handle)
            self.handle = C.c_void_p()


def sp_unique_id() -> bytes:
    buf = (C.c_char * 128)()
    check(_lib.lib().b2_sp_unique_id(buf, C.c_size_t(128)))
    return bytes(buf)


def sp_run(seq_lens, size, cu_seqlens_full, D=3072, F=12288, heads=24, fused_norm_rope=-1):
    """b2_sp_run of one rank: seq_lens are the FULL sequence lengths (host ints), cu_seqlens_full their device prefix sums."""
    r = _lib.SpRun()
    r.struct_size = C.sizeof(_lib.SpRun)
    r.local = block_run(sum(s // size for s in seq_lens), cu_seqlens_full, max(seq_lens), D=D, F=F, heads=heads,
                        fused_norm_rope=fused_norm_rope)
    arr = (C.c_int32 * len(seq_lens))(*seq_lens)
    r.seq_lens_host = C.cast(arr, C.c_void_p)
    r._keep = (arr, cu_seqlens_full)
    return r


def block_quant_sp_workspace_bytes(run, size) -> int:
    n = int(_lib.lib().b2_block_quant_sp_workspace_bytes(C.byref(run), C.c_int(size)))
    if n == 0:
        raise ValueError(_lib.lib().b2_last_error_message().decode())
    return n


def run_block_quant_sp(weights: BlockWeights, bufs, run, comm: SpComm):
    check(_lib.lib().b2_run_block_quant_sp(C.byref(weights.struct), C.byref(bufs), C.byref(run), comm.handle, _stream()))


def dit_step_sp(blocks, bufs, run, comm: SpComm):
    arr = (_lib.BlockWeights * len(blocks))(*[b.struct for b in blocks])
    check(_lib.lib().b2_dit_step_sp(arr, C.c_int(len(blocks)), C.byref(bufs), C.byref(run), comm.handle, _stream()))


# ------------------------------------------------------------------------------------------------ guidance + update

def cfg_combine(cond, uncond, g, out=None):
    out = torch.empty_like(cond) if out is None else out
    check(_lib.lib().b2_cfg_combine(_ptr(cond), _ptr(uncond), C.c_float(g), _ptr(out), C.c_int64(cond.numel()), _stream()))
    return out


def slg_correct(pred, cond, skipped, scale, out=None):
    out = torch.empty_like(cond) if out is None else out
    check(_lib.lib().b2_slg_correct(_ptr(pred), _ptr(cond), _ptr(skipped), C.c_float(scale), _ptr(out), C.c_int64(cond.numel()),
                                    _stream()))
    return out


def euler_update(x, v, h):
    check(_lib.lib().b2_euler_update(_ptr(x), _ptr(v), C.c_float(h), C.c_int64(x.numel()), _stream()))
    return x


def ab2_update(x, v, v_prev, h, a, b):
    check(_lib.lib().b2_ab2_update(_ptr(x), _ptr(v), _ptr(v_prev), C.c_float(h), C.c_float(a), C.c_float(b), C.c_int64(x.numel()),
                                   _stream()))
    return x


def guided_velocity_step(v_cond, x=None, v_uncond=None, v_skip=None, v_prev=None, v_out=None, cfg_scale=0.0, slg_scale=0.0,
                         h=0.0, a=0.0, b=0.0, update=0):
    """One pass: guidance (cfg when v_uncond is given, slg when v_skip is given), optional store of the guided velocity,
    and the Euler (update 1) or Adams-Bashforth (update 2) step of x."""
    g = _lib.GuidedStep()
    g.struct_size = C.sizeof(_lib.GuidedStep)
    p = lambda t: None if t is None else t.data_ptr()
    g.x, g.v_cond, g.v_uncond, g.v_skip, g.v_prev, g.v_out = p(x), p(v_cond), p(v_uncond), p(v_skip), p(v_prev), p(v_out)
    g.cfg_scale, g.slg_scale, g.h, g.a, g.b = cfg_scale, slg_scale, h, a, b
    g.cfg, g.slg, g.update, g.n = int(v_uncond is not None), int(v_skip is not None), update, v_cond.numel()
    check(_lib.lib().b2_guided_velocity_step(C.byref(g), _stream()))
    return x if update else v_out


# ------------------------------------------------------------------------------------------------ forward shell

def latent_to_tokens(latents, tokens=None, col0=0):
    """f32 [C, h, w] (or [C, hw]) -> bf16 [hw, C]; into columns [col0, col0 + C) of a wider `tokens` when given."""
    c, hw = latents.shape[0], latents.numel() // latents.shape[0]
    tokens = torch.empty((hw, c), dtype=torch.bfloat16, device=latents.device) if tokens is None else tokens
    dst = C.c_void_p(tokens.data_ptr() + 2 * col0)
    check(_lib.lib().b2_latent_to_tokens(_ptr(latents), C.c_int(c), C.c_int64(hw), dst, C.c_int64(tokens.stride(0)), _stream()))
    return tokens


def tokens_to_latent(tokens, latents=None):
    hw, c = tokens.shape
    latents = torch.empty((c, hw), dtype=torch.float32, device=tokens.device) if latents is None else latents
    check(_lib.lib().b2_tokens_to_latent(_ptr(tokens), _ptr(latents), C.c_int(c), C.c_int64(hw), _stream()))
    return latents


def linear_fp32_row(w, x, bias, out=None):
    n, k = w.shape
    out = torch.empty(n, dtype=torch.bfloat16, device=w.device) if out is None else out
    check(_lib.lib().b2_linear_fp32_row(_ptr(w), _ptr(x), _ptr(bias), _ptr(out), C.c_int(n), C.c_int(k), _stream()))
    return out


def rms_norm_modulate(x, norm_weight, mod_scale, mod_shift, y=None):
    m, k = x.shape
    y = torch.empty((m, k), dtype=torch.bfloat16, device=x.device) if y is None else y
    check(_lib.lib().b2_rms_norm_modulate(_ptr(x), C.c_int64(_ld(x)), _ptr(norm_weight), _ptr(mod_scale), _ptr(mod_shift),
                                          _ptr(y), C.c_int64(_ld(y)), C.c_int64(m), C.c_int(k), _stream()))
    return y


def time_sinusoid(timestep):
    import numpy as np
    emb = np.empty(256, np.float32)
    check(_lib.lib().b2_time_sinusoid(C.c_float(timestep), emb.ctypes.data_as(C.c_void_p)))
    return emb


def time_vector_fp32(w0, b0, w2, b2, timestep):
    """Host: numpy f32 weights of the timestep MLP -> the f32 time vector [dim]."""
    import numpy as np
    w0, b0, w2, b2 = (np.ascontiguousarray(a, np.float32) for a in (w0, b0, w2, b2))
    te = _lib.TimeEmbedding()
    te.struct_size, te.dim = C.sizeof(_lib.TimeEmbedding), w2.shape[0]
    te.w0, te.b0, te.w2, te.b2 = (a.ctypes.data for a in (w0, b0, w2, b2))
    out = np.empty(w2.shape[0], np.float32)
    check(_lib.lib().b2_time_vector_fp32(C.byref(te), C.c_float(timestep), out.ctypes.data_as(C.c_void_p)))
    return out


def linear_bf16(x, w, bias=None, out=None, workspace=None):
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device) if out is None else out
    if workspace is None:
        workspace = torch.empty(_lib.lib().b2_linear_bf16_workspace_bytes(), dtype=torch.uint8, device=x.device)
    check(_lib.lib().b2_linear_bf16(_ptr(x), C.c_int64(_ld(x)), _ptr(w), _ptr(bias), _ptr(out), C.c_int64(_ld(out)),
                                    C.c_int64(m), C.c_int(n), C.c_int(k), _ptr(workspace), C.c_size_t(workspace.numel()),
                                    _stream()))
    return out


class DitModel:
    """b2_dit_model over torch tensors: `blocks` a list of BlockWeights, the rest device tensors (kept alive here)."""

    def __init__(self, blocks, F, block_mod_w, block_mod_bias, head_mod_w, head_mod_bias, video_w, video_bias, final_norm,
                 final_w, final_bias, D=3072, heads=24, ext_w=None, ext_bias=None):
        self.keep = (blocks, block_mod_w, block_mod_bias, head_mod_w, head_mod_bias, video_w, video_bias, final_norm, final_w,
                     final_bias, ext_w, ext_bias)
        self.arr = (_lib.BlockWeights * max(1, len(blocks)))(*[b.struct for b in blocks])
        m = _lib.DitModel()
        m.struct_size, m.blocks, m.num_blocks = C.sizeof(_lib.DitModel), self.arr, len(blocks)
        m.D, m.F, m.heads, m.latent_channels = D, F, heads, 128
        p = lambda t: None if t is None else t.data_ptr()
        m.block_mod_w, m.block_mod_bias, m.head_mod_w, m.head_mod_bias = p(block_mod_w), p(block_mod_bias), p(head_mod_w), p(head_mod_bias)
        m.video_w, m.video_bias, m.final_norm, m.final_w, m.final_bias = p(video_w), p(video_bias), p(final_norm), p(final_w), p(final_bias)
        m.ext_w, m.ext_bias, m.ext_channels = p(ext_w), p(ext_bias), 0 if ext_w is None else ext_w.shape[1] - 128
        self.struct = m


def silu_bf16(x, out=None):
    """kernels::silu: bf16(x / (1 + expf(-x)))."""
    out = torch.empty_like(x) if out is None else out
    check(_lib.lib().b2_silu_bf16(_ptr(x), _ptr(out), x.numel(), _stream()))
    return out


def time_modulation_bf16(in_w, in_bias, out_w, out_bias, block_mod_w, block_mod_bias, head_mod_w, head_mod_bias, timestep):
    """MossDit::time_modulation in its bf16 form: (mod bf16 [6 D], head bf16 [2 D]) on the device. All arguments bf16 device tensors
    (a bias may be None)."""
    m = _lib.TimeMlpBf16()
    m.struct_size, m.dim = C.sizeof(_lib.TimeMlpBf16), out_w.shape[0]
    for name, t in (("in_w", in_w), ("in_bias", in_bias), ("out_w", out_w), ("out_bias", out_bias), ("block_mod_w", block_mod_w),
                    ("block_mod_bias", block_mod_bias), ("head_mod_w", head_mod_w), ("head_mod_bias", head_mod_bias)):
        setattr(m, name, None if t is None else t.data_ptr())
    D = out_w.shape[0]
    mod = torch.empty(6 * D, dtype=torch.bfloat16, device=out_w.device)
    head = torch.empty(2 * D, dtype=torch.bfloat16, device=out_w.device)
    ws = torch.empty(_lib.lib().b2_time_modulation_bf16_workspace_bytes(C.byref(m)), dtype=torch.uint8, device=out_w.device)
    check(_lib.lib().b2_time_modulation_bf16(C.byref(m), C.c_float(timestep), _ptr(mod), _ptr(head), _ptr(ws), ws.numel(), _stream()))
    return mod, head


class DitGraphs:
    """b2_dit_graphs: CUDA graphs of whole forwards, least recently used first out. Creating one touches no device."""

    def __init__(self, capacity=8):
        self.handle = C.c_void_p()
        check(_lib.lib().b2_dit_graphs_create(capacity, C.byref(self.handle)))
        self.last_replayed = False

    def stats(self):
        st = _lib.DitGraphStats()
        check(_lib.lib().b2_dit_graphs_stats(self.handle, C.byref(st)))
        return {name: int(getattr(st, name)) for name, _ in st._fields_}

    def clear(self):
        check(_lib.lib().b2_dit_graphs_clear(self.handle))

    def close(self):
        if self.handle:
            _lib.lib().b2_dit_graphs_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dit_forward(model: DitModel, latents, time_vector, rows, tier=TIER_INT8, workspace=None, extra=None, ref_kv=None,
                graphs=None, outs=None, mod=None, head=None):
    """rows: list of (text bf16 [S, D], skip mask int, latent index). latents f32 [n, 128, h, w]; time_vector numpy f32 [D].
    Returns the per-row outputs f32 [128, h, w] (and the workspace, for reuse). With `graphs` (a DitGraphs) the forward
    goes through b2_dit_forward_graphed on the current (non-default) stream; pass the same `outs` and `workspace` again for
    the call to find its graph."""
    import numpy as np
    n, _, h, w = latents.shape
    if outs is None:
        outs = [torch.empty((128, h, w), dtype=torch.float32, device=latents.device) for _ in rows]
    arr = (_lib.ForwardRow * len(rows))()
    for i, (text, skip, latent) in enumerate(rows):
        arr[i].text, arr[i].text_len, arr[i].skip, arr[i].latent, arr[i].out = text.data_ptr(), text.shape[0], skip, latent, outs[i].data_ptr()
    tv = None if time_vector is None else np.ascontiguousarray(time_vector, np.float32)
    f = _lib.Forward()
    f.struct_size, f.latents, f.num_latents, f.height, f.width = C.sizeof(_lib.Forward), latents.data_ptr(), n, h, w
    f.time_vector, f.rows, f.num_rows, f.tier = (None if tv is None else tv.ctypes.data), arr, len(rows), tier
    f.mod, f.head = (None if mod is None else mod.data_ptr()), (None if head is None else head.data_ptr())
    f.attention = _lib.AttentionOptions(ATTENTION_Q8_FP8_F32ACC, 0.0, 0.0)
    f.extra = None if extra is None else extra.data_ptr()
    f.ref_kv, f.ref_tokens = (None, 0) if ref_kv is None else (ref_kv.data_ptr(), ref_kv.shape[1])
    need = _lib.lib().b2_dit_forward_workspace_bytes(C.byref(model.struct), C.byref(f))
    if need == 0:
        check(-1)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=latents.device)
    f.workspace, f.workspace_bytes = workspace.data_ptr(), workspace.numel()
    if graphs is None:
        check(_lib.lib().b2_dit_forward(C.byref(model.struct), C.byref(f), _stream()))
    else:
        replayed = C.c_int(0)
        check(_lib.lib().b2_dit_forward_graphed(graphs.handle, C.byref(model.struct), C.byref(f), _stream(), C.byref(replayed)))
        graphs.last_replayed = bool(replayed.value)
    return outs, workspace


def dit_prefill_references(model, latents, time_vector, tier=TIER_INT8):
    """latents: list of f32 [128, h, w] reference latents. Returns the cache bf16 [num_blocks, sum h w, 2 D]."""
    import numpy as np
    n = len(latents)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in latents])
    hs, ws = (C.c_int * n)(*[t.shape[1] for t in latents]), (C.c_int * n)(*[t.shape[2] for t in latents])
    total = sum(t.shape[1] * t.shape[2] for t in latents)
    m = model.struct
    kv = torch.empty((m.num_blocks, total, 2 * m.D), dtype=torch.bfloat16, device=latents[0].device)
    tv = np.ascontiguousarray(time_vector, np.float32)
    f = _lib.Prefill()
    f.struct_size, f.latents, f.heights, f.widths, f.num_refs = C.sizeof(_lib.Prefill), ptrs, hs, ws, n
    f.time_vector, f.kv_out, f.tier = tv.ctypes.data, kv.data_ptr(), tier
    f.attention = _lib.AttentionOptions(ATTENTION_Q8_FP8_F32ACC, 0.0, 0.0)
    need = _lib.lib().b2_dit_prefill_workspace_bytes(C.byref(m), C.byref(f))
    if need == 0:
        check(-1)
    ws_buf = torch.empty(need, dtype=torch.uint8, device=latents[0].device)
    f.workspace, f.workspace_bytes = ws_buf.data_ptr(), need
    check(_lib.lib().b2_dit_prefill_references(C.byref(m), C.byref(f), _stream()))
    return kv


# ------------------------------------------------------------------------------------------------ weight ingestion

class _Loaded:
    """A struct that lives in a loaded file (b2_block_weights or b2_dit_model): `.struct` for the calls that take one."""

    def __init__(self, struct, owner):
        self.struct, self.owner = struct, owner


class DitFile:
    """b2_dit_file: the quantized DiT of a ComfyUI-layout safetensors file, on the current device."""

    def __init__(self, path: str, expanded: bool = False):
        """expanded: grouped 4-bit (W4A8) weights are expanded to the INT8 grid once at load (b2_dit_file_open_expanded)."""
        self.handle = C.c_void_p()
        opener = _lib.lib().b2_dit_file_open_expanded if expanded else _lib.lib().b2_dit_file_open
        check(opener(str(path).encode(), C.byref(self.handle)))
        info = _lib.DitFileInfo()
        info.struct_size = C.sizeof(_lib.DitFileInfo)
        check(_lib.lib().b2_dit_file_get_info(self.handle, C.byref(info)))
        self.num_blocks, self.F, self.tier, self.stored_tier = info.num_blocks, info.F, info.tier, info.stored_tier
        self.has_shell, self.has_time_embedding, self.device_bytes = bool(info.has_shell), bool(info.has_time_embedding), info.device_bytes
        model = _lib.lib().b2_dit_file_model(self.handle).contents
        self.model = _Loaded(model, self)
        self.blocks = [_Loaded(model.blocks[i], self) for i in range(self.num_blocks)]

    def time_vector(self, timestep: float):
        import numpy as np
        te = _lib.lib().b2_dit_file_time_embedding(self.handle)
        if not te:
            raise ValueError("the file has no time embedding")
        out = np.empty(te.contents.dim, np.float32)
        check(_lib.lib().b2_time_vector_fp32(te, C.c_float(timestep), out.ctypes.data_as(C.c_void_p)))
        return out

    def time_modulation_bf16(self, timestep: float):
        """(mod bf16 [6 D], head bf16 [2 D]) through the bf16 form of the file's timestep MLP and modulation linears."""
        m = _lib.lib().b2_dit_file_time_mlp_bf16(self.handle)
        if not m:
            raise ValueError("the file lacks the shell or the time embedding")
        D = m.contents.dim
        mod = torch.empty(6 * D, dtype=torch.bfloat16, device="cuda")
        head = torch.empty(2 * D, dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(_lib.lib().b2_time_modulation_bf16_workspace_bytes(m), dtype=torch.uint8, device="cuda")
        check(_lib.lib().b2_time_modulation_bf16(m, C.c_float(timestep), _ptr(mod), _ptr(head), _ptr(ws), ws.numel(), _stream()))
        return mod, head

    def close(self):
        if self.handle:
            _lib.lib().b2_dit_file_close(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
