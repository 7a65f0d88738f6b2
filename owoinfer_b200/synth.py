"""Seeded synthetic inputs with the shapes and value distributions of the quantized DiT block's real operands.

Stand-ins for MOSS-Image activations and weights (there are no checkpoints here): activations bf16 N(0, 1) with 1 % of
the channels multiplied by 20; modulation vectors bf16 N(0, 0.1); norm weights 1 + N(0, 0.1); linear weights N(0, 0.02),
rotated per 256-column group (W · H256) and quantised per output row to INT8 (ConvRot), to int4 (W4A4), or to grouped
4-bit codes with per-group scales (W4A8). Everything is a function of (seed, shape) and works on any torch device.
"""
from __future__ import annotations

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def activations(tokens: int, dim: int, seed: int, device="cuda") -> torch.Tensor:
    g = _gen(seed, device)
    x = torch.randn((tokens, dim), generator=g, device=device, dtype=torch.float32)
    n_out = max(1, dim // 100)
    idx = torch.randperm(dim, generator=g, device=device)[:n_out]
    x[:, idx] *= 20.0
    return x.to(torch.bfloat16)


def vector(dim: int, seed: int, std: float = 0.1, mean: float = 0.0, device="cuda") -> torch.Tensor:
    return (mean + std * torch.randn(dim, generator=_gen(seed, device), device=device, dtype=torch.float32)).to(torch.bfloat16)


def modulation(dim: int, seed: int, device="cuda") -> torch.Tensor:
    """[6 * dim] = shift_a, scale_a, gate_a, shift_f, scale_f, gate_f."""
    return vector(6 * dim, seed, 0.1, 0.0, device)


def hadamard256(device="cuda") -> torch.Tensor:
    """kron^4(H4) / 16 with the regular H4 (entry -1 where the base-4 digits of row and column sum to 3)."""
    h4 = torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=torch.float32, device=device)
    h = h4
    for _ in range(3):
        h = torch.kron(h4, h)
    return h / 16.0


def convrot_int8_weight(n: int, k: int, seed: int, device="cuda", std: float = 0.02):
    """(int8 [n, k], f32 scale [n]): N(0, std) rounded to bf16, rotated per 256 group, absmax / 127 per row."""
    g = _gen(seed, device)
    h = hadamard256(device)
    q = torch.empty((n, k), dtype=torch.int8, device=device)
    s = torch.empty(n, dtype=torch.float32, device=device)
    step = 4096
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        w = (std * torch.randn((r1 - r0, k), generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16).float()
        rot = (w.view(r1 - r0, k // 256, 256) @ h).view(r1 - r0, k)
        sc = (rot.abs().amax(dim=1) * (1.0 / 127.0)).clamp_min(1e-30)
        q[r0:r1] = torch.round(rot / sc[:, None]).clamp_(-128, 127).to(torch.int8)
        s[r0:r1] = sc
    return q, s


def pack_int4(vals: torch.Tensor) -> torch.Tensor:
    """int8 values in [-8, 7] -> uint8 [rows, k/2], even column in the low nibble."""
    v = vals.to(torch.int16) & 0xF
    return (v[:, 0::2] | (v[:, 1::2] << 4)).to(torch.uint8)


def convrot_int4_weight(n: int, k: int, seed: int, device="cuda", std: float = 0.02):
    """(packed int4 uint8 [n, k/2], f32 scale [n]) for the W4A4-through-INT8 route: absmax / 7 per row."""
    g = _gen(seed, device)
    h = hadamard256(device)
    w = (std * torch.randn((n, k), generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16).float()
    rot = (w.view(n, k // 256, 256) @ h).view(n, k)
    sc = (rot.abs().amax(dim=1) / 7.0).clamp_min(1e-30)
    q = torch.round(rot / sc[:, None]).clamp_(-7, 7).to(torch.int8)
    return pack_int4(q), sc


def grouped_w4_weight(n: int, k: int, seed: int, group: int = 64, device="cuda", std: float = 0.02, fp16_scales=True):
    """Grouped 4-bit weight: (packed codes uint8 [n, k/2], s_rel [n, k/group] fp16 or e4m3 bytes, s_channel f32 [n]).

    Codes are level + 8 with level in [-7, 7]; a group's scale is its absmax / 7 relative to the row scale s_channel, so
    that level * s_rel lands on the INT8 grid (|.| <= 127)."""
    g = _gen(seed, device)
    h = hadamard256(device)
    w = (std * torch.randn((n, k), generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16).float()
    rot = (w.view(n, k // 256, 256) @ h).view(n, k)
    s_channel = (rot.abs().amax(dim=1) / 127.0).clamp_min(1e-30)
    grid = rot / s_channel[:, None]                      # |.| <= 127
    gr = grid.view(n, k // group, group)
    s_rel = (gr.abs().amax(dim=2) / 7.0).clamp_min(2.0 ** -6)
    if fp16_scales:
        s_rel_q = s_rel.to(torch.float16)
        s_val = s_rel_q.float()
        s_store = s_rel_q.view(torch.int16)
    else:
        s_rel_q = s_rel.to(torch.float8_e4m3fn)
        s_val = s_rel_q.float()
        s_store = s_rel_q.view(torch.uint8)
    level = torch.round(gr / s_val[:, :, None]).clamp_(-7, 7).to(torch.int8).view(n, k)
    return pack_int4(level + 8), s_store.contiguous(), s_channel


def block_weights(D: int, F: int, seed: int, device="cuda", tier: int = 0, fp16_scales: bool = False):
    """Tensors of one block: norms plus the four linears in the tier's storage (see ops.BlockWeights). The grouped 4-bit
    tier stores its group scales as e4m3 bytes (the reference's file format) unless fp16_scales is set."""
    from . import ops
    w = {
        "norm1": vector(D, seed + 1, 0.1, 1.0, device), "norm2": vector(D, seed + 2, 0.1, 1.0, device),
        "q_norm": vector(128, seed + 3, 0.1, 1.0, device), "k_norm": vector(128, seed + 4, 0.1, 1.0, device),
    }
    shapes = {"qkv": (3 * D, D), "o": (D, D), "up_gate": (2 * F, D), "down": (D, F)}
    for i, (name, (n, k)) in enumerate(shapes.items()):
        if tier == ops.TIER_INT8:
            w[name] = convrot_int8_weight(n, k, seed + 10 + i, device)
        elif tier == ops.TIER_W4A4_VIA_INT8:
            w[name] = convrot_int4_weight(n, k, seed + 10 + i, device)
        else:
            w[name] = grouped_w4_weight(n, k, seed + 10 + i, 64, device, fp16_scales=fp16_scales)
    return w


def cu_seqlens(lengths, device="cuda") -> torch.Tensor:
    out = [0]
    for n in lengths:
        out.append(out[-1] + int(n))
    return torch.tensor(out, dtype=torch.int32, device=device)


def write_int8_dit_file(path, blocks: int, F: int, D: int = 3072, seed: int = 7) -> int:
    """A ComfyUI-layout safetensors file of `blocks` INT8 ConvRot blocks under the official tensor names (random bytes,
    per-module comfy_quant configs): what the loader reads. Returns the file's size in bytes."""
    import json
    import os
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    conf = torch.tensor(list(json.dumps({"format": "int8_tensorwise", "convrot": True, "convrot_groupsize": 256}).encode()),
                        dtype=torch.uint8)
    t = {}
    for b in range(blocks):
        p = f"layers.{b}."
        for name, n in (("norm1", D), ("norm2", D), ("q_norm", 128), ("k_norm", 128)):
            t[p + name + ".weight"] = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
        for name, (n, k) in (("qkv", (3 * D, D)), ("o", (D, D)), ("ffn_up_gate", (2 * F, D)), ("ffn_down", (D, F))):
            m = p + "proj." + name
            t[m + ".weight"] = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
            t[m + ".weight_scale"] = torch.rand(n, generator=g) * 0.02 + 0.001
            t[m + ".comfy_quant"] = conf.clone()
    save_file(t, str(path))
    return os.path.getsize(path)
