"""Synthetic ComfyUI-layout safetensors files of the quantized MOSS-Image DiT (tiny FFN, a few blocks) for the loader
tests: official tensor names, per-module `comfy_quant` configs, the three stored formats."""
import json

import numpy as np
import torch

D = 3072


def config(fmt, **extra):
    d = {"format": fmt}
    d.update(extra)
    return torch.tensor(list(json.dumps(d).encode()), dtype=torch.uint8)


INT8 = dict(fmt="int8_tensorwise", convrot=True, convrot_groupsize=256)


def int8_linear(name, n, k, seed, scalar_scale=False):
    g = torch.Generator().manual_seed(seed)
    t = {name + ".weight": torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g),
         name + ".comfy_quant": config(INT8["fmt"], convrot=True, convrot_groupsize=256)}
    t[name + ".weight_scale"] = (torch.tensor(0.0123, dtype=torch.float32) if scalar_scale
                                 else torch.rand(n, generator=g, dtype=torch.float32) * 0.02 + 0.001)
    return t


def w4a4_linear(name, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return {name + ".weight": torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, generator=g),
            name + ".weight_scale": torch.rand(n, generator=g, dtype=torch.float32) * 0.05 + 0.001,
            name + ".comfy_quant": config("convrot_w4a4", convrot=True, convrot_groupsize=256, quant_group_size=64)}


def w4a8_linear(name, n, k, seed, group=64, codebook=False):
    g = torch.Generator().manual_seed(seed)
    t = {name + ".weight": torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, generator=g),
         name + ".weight_s_rel": (torch.rand((n, k // group), generator=g) * 12 + 1).to(torch.float8_e4m3fn),
         name + ".weight_s_channel": torch.rand(n, generator=g, dtype=torch.float32) * 0.01 + 0.001,
         name + ".comfy_quant": config("asym_w4a8_int8", params={"convrot": True, "convrot_groupsize": 256, "group_size": group})}
    if codebook:
        t[name + ".weight_codebook"] = torch.linspace(-7.5, 7.5, 16, dtype=torch.float32)
    return t


def block(b, F, maker, seed, fused_qkv=False):
    p = f"layers.{b}."
    g = torch.Generator().manual_seed(seed)
    t = {p + "norm1.weight": (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16),
         p + "norm2.weight": (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16),
         p + "q_norm.weight": (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16),
         p + "k_norm.weight": (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)}
    if fused_qkv:
        t.update(maker(p + "proj.qkv", 3 * D, D, seed + 1))
    else:
        for i, part in enumerate("qkv"):
            t.update(maker(p + "proj." + part, D, D, seed + 1 + i))
    t.update(maker(p + "proj.o", D, D, seed + 5))
    t.update(maker(p + "proj.ffn_up_gate", 2 * F, D, seed + 6))
    t.update(maker(p + "proj.ffn_down", D, F, seed + 7))
    return t


def shell(seed, with_time=True):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std)
    t = {"shared_block_modulation.weight": r(6 * D, D).to(torch.bfloat16), "shared_block_modulation.bias": r(6 * D, std=0.3).to(torch.bfloat16),
         "video_head_modulation.weight": r(2 * D, D).to(torch.bfloat16), "video_head_modulation.bias": r(2 * D, std=0.3).to(torch.bfloat16),
         "video_embedder.weight": r(D, 128, std=0.09).to(torch.bfloat16), "video_embedder.bias": r(D, std=0.1).to(torch.bfloat16),
         "final_norm_video.weight": (1 + r(D, std=0.1)).to(torch.bfloat16), "final_linear_video.weight": r(128, D).to(torch.bfloat16)}
    if with_time:
        t.update({"time_embedding.0.weight": r(D, 256, std=0.06).to(torch.bfloat16), "time_embedding.0.bias": r(D, std=0.1).to(torch.bfloat16),
                  "time_embedding.2.weight": r(D, D).to(torch.bfloat16), "time_embedding.2.bias": r(D, std=0.1).to(torch.bfloat16)})
    return t


def save(path, tensors, prefix="", metadata=None):
    from safetensors.torch import save_file
    save_file({prefix + k: v.contiguous() for k, v in tensors.items()}, str(path), metadata=metadata)
    return path
