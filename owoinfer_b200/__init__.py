"""owoinfer_b200: the quantized MOSS-Image DiT block on B200 (sm_100a) behind a C ABI.

`ops` mirrors the reference's kernel-level and block-level interfaces over torch CUDA tensors; the arithmetic runs in
libowoinfer_b200.so (hand-written CUDA, built by `python -m owoinfer_b200.build`). There is no CPU fallback.
"""
from . import _lib  # noqa: F401
from . import ops  # noqa: F401

__all__ = ["ops"]
