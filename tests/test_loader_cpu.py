"""Weight ingestion, the part that needs no GPU: the file is described and checked in full (container, names, dtypes,
shapes, configs, scales) before any device memory is asked for, so every refusal can be provoked here. A file that
passes the checks gets as far as the device allocation and fails there on a box without a GPU. Modelled on
tests/unit/test_quant_model.cpp of the reference (hostile headers, wrong layouts, unsupported formats)."""
import json
import struct

import pytest
import torch

from tests import loader_files as lf

F = 256


@pytest.fixture(scope="module")
def ops():
    from owoinfer_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def base():
    return lf.block(0, F, lf.int8_linear, 1)


def refused(ops, path, match):
    with pytest.raises(ValueError, match=match):
        ops.DitFile(path)
    with pytest.raises(ValueError, match=match):   # the expanding open checks the same things before it allocates
        ops.DitFile(path, expanded=True)


def test_container_errors(ops, tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    refused(ops, p, "shorter than a safetensors header")
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    refused(ops, p, "header length")
    p.write_bytes(struct.pack("<Q", 9) + b'{"a": [1}')
    refused(ops, p, "JSON")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    refused(ops, p, "data_offsets outside the file")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    refused(ops, p, "8 bytes for F32")
    hdr = json.dumps({"t": {"dtype": "Q7", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    refused(ops, p, "unknown dtype")
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    refused(ops, p, "not a MOSS-Image DiT file")


def test_model_errors(ops, base, tmp_path):
    p = tmp_path / "m.safetensors"

    def variant(**changes):
        t = dict(base)
        for k, v in changes.items():
            if v is None:
                t.pop(k)
            else:
                t[k] = v
        return lf.save(p, t)

    o = "layers.0.proj.o"
    refused(ops, variant(**{o + ".weight_scale": None}), "weight_scale' missing")
    refused(ops, variant(**{o + ".comfy_quant": None}), "no quantization config")
    refused(ops, variant(**{o + ".comfy_quant": lf.config("int8_tensorwise", convrot=False)}), "plain INT8 without rotation")
    refused(ops, variant(**{o + ".comfy_quant": lf.config("int8_tensorwise", convrot=True, convrot_groupsize=64)}), "rotation group 64")
    refused(ops, variant(**{o + ".comfy_quant": lf.config("nvfp4")}), "nvfp4 is not read")
    refused(ops, variant(**{o + ".comfy_quant": lf.config("fp8_e4m3")}), "not supported")
    refused(ops, variant(**{o + ".weight": torch.zeros((lf.D, lf.D), dtype=torch.uint8)}), "must be I8")
    refused(ops, variant(**{o + ".weight": torch.zeros((lf.D, lf.D // 2), dtype=torch.int8)}), "the DiT's is")
    refused(ops, variant(**{o + ".bias": torch.zeros(lf.D, dtype=torch.bfloat16)}), "bias the DiT does not use")
    bad = base[o + ".weight_scale"].clone()
    bad[17] = float("nan")
    refused(ops, variant(**{o + ".weight_scale": bad}), "not finite and > 0")
    bad[17] = 0.0
    refused(ops, variant(**{o + ".weight_scale": bad}), "not finite and > 0")
    refused(ops, variant(**{"layers.0.norm2.weight": torch.zeros(7, dtype=torch.bfloat16)}), r"must be BF16 \[3072\]")
    # one linear of another tier than the rest
    mixed = {k: None for k in base if k.startswith(o + ".")}
    mixed.update(lf.w4a4_linear(o, lf.D, lf.D, 9))
    refused(ops, variant(**mixed), "another tier")
    # q, k, v in different formats
    q = "layers.0.proj.k"
    mixed = {k: None for k in base if k.startswith(q + ".")}
    mixed.update(lf.w4a4_linear(q, lf.D, lf.D, 9))
    refused(ops, variant(**mixed), "different formats")


def test_a_good_file_reaches_the_device_allocation(ops, base, tmp_path):
    p = lf.save(tmp_path / "ok.safetensors", base, prefix="model.diffusion_model.")
    if torch.cuda.is_available():
        f = ops.DitFile(p)
        assert (f.num_blocks, f.F, f.tier, f.has_shell) == (1, F, ops.TIER_INT8, False)
        f.close()
    else:
        with pytest.raises(RuntimeError):   # a CUDA error, not a refusal of the file
            ops.DitFile(p)


def test_legacy_metadata_configs(ops, base, tmp_path):
    t = {k: v for k, v in base.items() if not k.endswith(".comfy_quant")}
    layers = {k[:-len(".comfy_quant")]: {"format": "int8_tensorwise", "params": {"convrot": True, "convrot_groupsize": 256}}
              for k in base if k.endswith(".comfy_quant")}
    layers.pop("layers.0.proj.ffn_down")
    p = lf.save(tmp_path / "legacy.safetensors", t, metadata={"_quantization_metadata": json.dumps({"layers": layers})})
    refused(ops, p, "ffn_down' missing or without a quantization config")
