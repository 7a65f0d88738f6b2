"""Regenerates the hash-defined inputs of the reference's INT4 golden vectors (tests/unit/test_quant4_kernels.cu:76-130
describes them: a splitmix64 finaliser over the element index, per-channel exponents, five edited rows), so that the
stored outputs under tests/golden/ref/quant4 can pin the oracle bit for bit."""
import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def mix(z):
    z = np.asarray(z, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _bf16_trunc(v):
    return (np.asarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def _bf16_float(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def synth_act(seed, rows, cols):
    c = np.arange(cols, dtype=np.uint64)
    with np.errstate(over="ignore"):
        c_exp = (mix(c * np.uint64(7919) + np.uint64(seed)) % np.uint64(6)).astype(np.int64) - 3
        c_exp = c_exp + np.where(np.arange(cols) % 397 == 5, 6, 0)
        idx = (np.arange(rows, dtype=np.uint64)[:, None] * np.uint64(cols) + c[None, :])
        z = mix(idx + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15))
    m = (128 + (z & np.uint64(0x7F))).astype(np.float32)
    e = ((z >> np.uint64(7)) & np.uint64(7)).astype(np.int64)
    sign = np.where(((z >> np.uint64(10)) & np.uint64(1)) == 1, -1.0, 1.0).astype(np.float32)
    return _bf16_trunc(np.ldexp(sign * m, (c_exp[None, :] - 7 - e).astype(np.int32)))


def quant4_rot3072_input():
    x = synth_act(101, 40, 3072)
    x[3, :] = 0
    x[4, :] = _bf16_trunc(np.ldexp(_bf16_float(x[4]), -10))
    x[5, :] = _bf16_trunc(np.ldexp(_bf16_float(x[5]), -60))
    x[7, :] = _bf16_trunc(np.ldexp(_bf16_float(x[7]), -45))
    x[4, 1000] = _bf16_trunc(np.float32(300.0))
    x[6, :256] = _bf16_trunc(np.float32(1.0))
    return x


def quant4_rot8192_input():
    return synth_act(102, 9, 8192)
