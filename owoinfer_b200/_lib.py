"""Loads libowoinfer_b200.so and declares its C ABI for ctypes. Fails loudly when the library is missing: there is no
CPU or PyTorch fallback on the product path."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libowoinfer_b200.so")

# Every symbol include/owoinfer_b200.h declares (tests check that the library exports each of them).
EXPORTS = [
    "b2_last_error_message", "b2_numerics_version", "b2_rotate_quantize", "b2_rms_norm_modulate_rotate_quantize",
    "b2_convrot_quantize_int4", "b2_rms_norm_modulate_convrot_quantize_int4", "b2_unpack_int4", "b2_decode_grouped_int8",
    "b2_int8_gemm", "b2_int8_gemm_gated_residual", "b2_int8_gemm_situ_glu", "b2_int8_gemm_acc", "b2_w4a8_gemm", "b2_w4a8_gemm_noalloc", "b2_debug_w4a8_route",
    "b2_qk_norm_rope_moss", "b2_moss_rope_table", "b2_attention_q8_workspace_bytes", "b2_attention_q8",
    "b2_attention_q8_layout", "b2_attention_q8_debug_scores", "b2_attention_q8_preprocess", "b2_block_quant_workspace_bytes", "b2_run_block_quant", "b2_dit_step",
    "b2_kernel_status", "b2_kernel_status_clear", "b2_debug_bounded_wait", "b2_w4_invalid_scales", "b2_rotate_quantize_chunked", "b2_int8_gemm_chunked", "b2_sp_unique_id",
    "b2_sp_comm_create", "b2_sp_comm_destroy", "b2_sp_comm_local_exchange", "b2_block_quant_sp_workspace_bytes", "b2_run_block_quant_sp", "b2_dit_step_sp",
    "b2_cfg_combine", "b2_slg_correct", "b2_euler_update", "b2_ab2_update", "b2_guided_velocity_step",
    "b2_latent_to_tokens", "b2_tokens_to_latent", "b2_linear_fp32_row", "b2_rms_norm_modulate", "b2_time_sinusoid",
    "b2_time_vector_fp32", "b2_linear_bf16_workspace_bytes", "b2_linear_bf16", "b2_dit_forward_workspace_bytes", "b2_dit_forward",
    "b2_moss_rope_table_reference", "b2_dit_prefill_workspace_bytes", "b2_dit_prefill_references",
    "b2_dit_file_open_expanded", "b2_silu_bf16", "b2_time_modulation_bf16_workspace_bytes", "b2_time_modulation_bf16",
    "b2_dit_graphs_create", "b2_dit_graphs_clear", "b2_dit_graphs_destroy", "b2_dit_graphs_stats", "b2_dit_forward_graphed",
    "b2_dit_file_open", "b2_dit_file_get_info", "b2_dit_file_model", "b2_dit_file_time_embedding", "b2_dit_file_time_mlp_bf16", "b2_dit_file_close",
]


class Int8Operands(C.Structure):
    _fields_ = [("x_q", C.c_void_p), ("ldx", C.c_int64), ("x_scale", C.c_void_p), ("w", C.c_void_p),
                ("w_scale", C.c_void_p), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


class W4Weight(C.Structure):
    _fields_ = [("packed", C.c_void_p), ("s_rel", C.c_void_p), ("scale_kind", C.c_int), ("group", C.c_int),
                ("codebook", C.c_void_p), ("s_channel", C.c_void_p)]


class AttentionOptions(C.Structure):
    _fields_ = [("variant", C.c_int), ("p_range", C.c_float), ("v_range", C.c_float)]


class View3(C.Structure):
    _fields_ = [("data", C.c_void_p), ("tokens", C.c_int64), ("heads", C.c_int64), ("row_stride", C.c_int64),
                ("head_stride", C.c_int64)]


class QkNormRope(C.Structure):
    _fields_ = [("q_norm", C.c_void_p), ("k_norm", C.c_void_p), ("table", C.c_void_p), ("table_ld", C.c_int64)]


class AttentionLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("q_i8", "k_i8", "v8", "q_scale", "k_scale", "k_mean", "v_scale", "v_recp",
                                          "part_sum", "part_amax", "total")] + \
               [("padded_k", C.c_int64), ("q_blocks", C.c_int), ("k_blocks", C.c_int), ("chunks", C.c_int)]


class Linear(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scale", C.c_void_p), ("w4", C.POINTER(W4Weight))]


class BlockWeights(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("norm1", C.c_void_p), ("norm2", C.c_void_p), ("q_norm", C.c_void_p),
                ("k_norm", C.c_void_p), ("qkv", Linear), ("o", Linear), ("up_gate", Linear), ("down", Linear)]


class BlockBuffers(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("x", C.c_void_p), ("mod", C.c_void_p), ("rope", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class BlockRun(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("tokens", C.c_int64), ("D", C.c_int), ("F", C.c_int), ("heads", C.c_int),
                ("cu_seqlens", C.c_void_p), ("batch", C.c_int), ("max_seqlen", C.c_int), ("tier", C.c_int),
                ("attention", AttentionOptions), ("fused_norm_rope", C.c_int), ("slot_rows", C.c_int64), ("slot_kv", C.c_void_p * 2), ("slot_kv_ld", C.c_int64),
                ("cu_seqlens_k", C.c_void_p), ("k0", C.c_int64), ("k1", C.c_int64), ("kv_tap", C.c_void_p), ("tap_only", C.c_int)]


class TimeEmbedding(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("dim", C.c_int64), ("w0", C.c_void_p), ("b0", C.c_void_p), ("w2", C.c_void_p),
                ("b2", C.c_void_p)]


class DitModel(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("blocks", C.POINTER(BlockWeights)), ("num_blocks", C.c_int), ("D", C.c_int),
                ("F", C.c_int), ("heads", C.c_int), ("latent_channels", C.c_int), ("block_mod_w", C.c_void_p),
                ("block_mod_bias", C.c_void_p), ("head_mod_w", C.c_void_p), ("head_mod_bias", C.c_void_p),
                ("video_w", C.c_void_p), ("video_bias", C.c_void_p), ("final_norm", C.c_void_p), ("final_w", C.c_void_p),
                ("final_bias", C.c_void_p), ("ext_w", C.c_void_p), ("ext_bias", C.c_void_p), ("ext_channels", C.c_int)]


class ForwardRow(C.Structure):
    _fields_ = [("text", C.c_void_p), ("text_len", C.c_int64), ("skip", C.c_uint64), ("latent", C.c_int), ("out", C.c_void_p)]


class Forward(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("latents", C.c_void_p), ("num_latents", C.c_int), ("height", C.c_int),
                ("width", C.c_int), ("time_vector", C.c_void_p), ("rows", C.POINTER(ForwardRow)), ("num_rows", C.c_int),
                ("tier", C.c_int), ("attention", AttentionOptions), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("extra", C.c_void_p), ("ref_kv", C.c_void_p), ("ref_tokens", C.c_int64), ("mod", C.c_void_p), ("head", C.c_void_p)]


class TimeMlpBf16(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("dim", C.c_int64), ("in_w", C.c_void_p), ("in_bias", C.c_void_p), ("out_w", C.c_void_p),
                ("out_bias", C.c_void_p), ("block_mod_w", C.c_void_p), ("block_mod_bias", C.c_void_p), ("head_mod_w", C.c_void_p),
                ("head_mod_bias", C.c_void_p)]


class DitGraphStats(C.Structure):
    _fields_ = [("replays", C.c_uint64), ("captures", C.c_uint64), ("collisions", C.c_uint64), ("eager", C.c_uint64),
                ("evictions", C.c_uint64), ("size", C.c_size_t)]


class Prefill(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("latents", C.POINTER(C.c_void_p)), ("heights", C.POINTER(C.c_int)),
                ("widths", C.POINTER(C.c_int)), ("num_refs", C.c_int), ("time_vector", C.c_void_p), ("kv_out", C.c_void_p),
                ("tier", C.c_int), ("attention", AttentionOptions), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class DitFileInfo(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("num_blocks", C.c_int), ("F", C.c_int), ("tier", C.c_int), ("has_shell", C.c_int),
                ("has_time_embedding", C.c_int), ("device_bytes", C.c_size_t), ("stored_tier", C.c_int)]


class GuidedStep(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("x", C.c_void_p), ("v_cond", C.c_void_p), ("v_uncond", C.c_void_p),
                ("v_skip", C.c_void_p), ("v_prev", C.c_void_p), ("v_out", C.c_void_p), ("cfg_scale", C.c_float),
                ("slg_scale", C.c_float), ("h", C.c_float), ("a", C.c_float), ("b", C.c_float), ("cfg", C.c_int),
                ("slg", C.c_int), ("update", C.c_int), ("n", C.c_int64)]


class SpRun(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("local", BlockRun), ("seq_lens_host", C.c_void_p)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m owoinfer_b200.build` "
                               "(there is no fallback path)")
        l = C.CDLL(LIB_PATH)
        l.b2_last_error_message.restype = C.c_char_p
        l.b2_numerics_version.restype = C.c_uint32
        l.b2_attention_q8_workspace_bytes.restype = C.c_size_t
        l.b2_attention_q8_workspace_bytes.argtypes = [C.POINTER(AttentionOptions), C.c_int64, C.c_int64, C.c_int, C.c_int,
                                                      C.c_int, C.c_int]
        l.b2_block_quant_workspace_bytes.restype = C.c_size_t
        l.b2_block_quant_workspace_bytes.argtypes = [C.POINTER(BlockRun)]
        l.b2_dit_prefill_workspace_bytes.restype = C.c_size_t
        l.b2_dit_prefill_workspace_bytes.argtypes = [C.POINTER(DitModel), C.POINTER(Prefill)]
        l.b2_dit_file_model.restype = C.POINTER(DitModel)
        l.b2_dit_file_model.argtypes = [C.c_void_p]
        l.b2_dit_file_time_embedding.restype = C.POINTER(TimeEmbedding)
        l.b2_dit_file_time_embedding.argtypes = [C.c_void_p]
        l.b2_dit_file_close.restype = None
        l.b2_dit_file_close.argtypes = [C.c_void_p]
        l.b2_linear_bf16_workspace_bytes.restype = C.c_size_t
        l.b2_dit_forward_workspace_bytes.restype = C.c_size_t
        l.b2_dit_file_time_mlp_bf16.restype = C.POINTER(TimeMlpBf16)
        l.b2_dit_file_time_mlp_bf16.argtypes = [C.c_void_p]
        l.b2_time_modulation_bf16_workspace_bytes.restype = C.c_size_t
        l.b2_time_modulation_bf16_workspace_bytes.argtypes = [C.POINTER(TimeMlpBf16)]
        l.b2_time_modulation_bf16.argtypes = [C.POINTER(TimeMlpBf16), C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        l.b2_silu_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        l.b2_dit_graphs_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
        l.b2_dit_graphs_clear.argtypes = [C.c_void_p]
        l.b2_dit_graphs_destroy.argtypes = [C.c_void_p]
        l.b2_dit_graphs_stats.argtypes = [C.c_void_p, C.POINTER(DitGraphStats)]
        l.b2_dit_forward_graphed.argtypes = [C.c_void_p, C.POINTER(DitModel), C.POINTER(Forward), C.c_void_p, C.POINTER(C.c_int)]
        l.b2_dit_forward_workspace_bytes.argtypes = [C.POINTER(DitModel), C.POINTER(Forward)]
        l.b2_block_quant_sp_workspace_bytes.restype = C.c_size_t
        l.b2_block_quant_sp_workspace_bytes.argtypes = [C.POINTER(SpRun), C.c_int]
        _lib = l
    return _lib


class B2Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


def check(status: int) -> None:
    """Maps a b2_status to the exception the reference would throw: -1 -> ValueError (std::invalid_argument)."""
    if status == 0:
        return
    msg = lib().b2_last_error_message().decode()
    if status == -1:
        raise ValueError(msg)
    raise B2Error(status, msg)
