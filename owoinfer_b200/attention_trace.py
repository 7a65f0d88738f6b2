"""Per-sub-tile timeline of the attention kernel: `python -m owoinfer_b200.attention_trace [--build-only]`.

The kernel carries clock stamps that are compiled out of the product (B2_ATTN_TRACE). This module builds a second copy of
the library with the stamps in (libowoinfer_b200_trace.so beside the product; only attention.cu is recompiled), runs one
sequence of 8192 tokens x 24 heads through it and prints, for the first CTA, how long one softmax warp and the MMA warp
spend between the stamps of a 64-key sub-tile (SM clocks, medians over sub-tiles 8..120; every stamp costs about 20
clocks itself, so the traced period is longer than the product's)."""
import ctypes as C
import os
import subprocess
import sys

from . import _lib, build

TRACE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libowoinfer_b200_trace.so")

# (stamp slot, what has just happened) in program order of a softmax warp's iteration u.
SOFTMAX = [(4, "loop top"), (8, "scale of the sub-tile ready"), (0, "S(u) in registers (tcgen05.wait::ld)"), (1, "pass done: P(u) stored"),
           (9, "vote: nothing to rescale"), (2, "denominator added"), (10, "fence.proxy.async"), (11, "tcgen05 fence + __syncwarp"),
           (3, "arrived on p_full(u)"), (12, "S(u+1) computed, P.V(u-1) landed (s_step wait)"), (13, "loads of S(u+1) issued"),
           (14, "headroom check done")]
MMA = [(5, "p_full(u) seen"), (6, "P.V(u) issued"), (7, "Q.K^T(u+2) issued, step committed")]


def build_trace() -> str:
    build.build()
    obj = os.path.join(build.OBJ, "attention_trace.o")
    src = os.path.join(build.CSRC, "attention.cu")
    if build._stale(obj, [src, os.path.join(build.CSRC, "common.cuh")]):
        subprocess.check_call([build.NVCC, *build.FLAGS, "-DB2_ATTN_TRACE", "-c", src, "-o", obj])
    others = [os.path.join(build.OBJ, s.replace(".cu", ".o")) for s in build.SOURCES if s != "attention.cu"]
    if build._stale(TRACE_LIB, [obj, *others]):
        subprocess.check_call([build.NVCC, "-shared", "-o", TRACE_LIB, obj, *others, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"])
    return TRACE_LIB


def main() -> None:
    path = build_trace()
    if "--build-only" in sys.argv:
        print(path)
        return
    _lib.LIB_PATH = path
    import numpy as np
    import torch
    from . import ops
    L, H = 8192, 24
    torch.manual_seed(0)
    qkv = torch.randn((L, 3 * H * 128), device="cuda").to(torch.bfloat16)
    q3, k3, v3 = (qkv.as_strided((L, H, 128), (3 * H * 128, 128, 1), i * H * 128) for i in range(3))
    out = torch.empty((L, H, 128), dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, L], dtype=torch.int32, device="cuda")
    _, ws = ops.attention_q8(q3, k3, v3, out, cu, cu, L, ops.SM_SCALE)
    ops.attention_q8(q3, k3, v3, out, cu, cu, L, ops.SM_SCALE, workspace=ws)
    torch.cuda.synchronize()
    buf = (C.c_longlong * 4096)()
    fn = C.CDLL(path).b2_attention_trace
    if fn(buf, 4096) != 0:
        raise RuntimeError("the trace could not be read")
    full = np.array(buf[:4096], dtype=np.int64).reshape(-1, 16)
    print("start-up issues with idle softmax warps: Q.K^T(0) incl. the wait for K", int(full[200, 1] - full[200, 0]), "clocks, Q.K^T(1)", int(full[200, 2] - full[200, 1]), "clocks")
    a = full[:128]
    u = np.arange(9, 120)
    med = lambda x: float(np.median(x))
    print("| from -> to (softmax warp %d, sub-tile u) | clocks |" % 2)
    print("|---|---|")
    for (s0, n0), (s1, n1) in zip(SOFTMAX, SOFTMAX[1:]):
        print(f"| {n0} -> {n1} | {med(a[u, s1] - a[u, s0]):.0f} |")
    print(f"| headroom check done -> loop top of u + 1 | {med(a[u + 1, 4] - a[u, 14]):.0f} |")
    print(f"| **period** (loop top to loop top) | **{med(a[u + 1, 4] - a[u, 4]):.0f}** (mean {float(np.mean(a[u + 1, 4] - a[u, 4])):.0f}: sub-tiles with a rescale of O take about a pass longer) |")
    print()
    print("| MMA warp, step u | clocks |")
    print("|---|---|")
    print(f"| step u - 1 committed -> p_full(u) seen (idle) | {med(a[u, 5] - a[u - 1, 7]):.0f} |")
    for (s0, n0), (s1, n1) in zip(MMA, MMA[1:]):
        print(f"| {n0} -> {n1} | {med(a[u, s1] - a[u, s0]):.0f} |")
    print(f"| step committed -> its MMAs complete (the MMA warp's own lane polls the barrier) | {med(a[u, 15] - a[u, 7]):.0f} |")
    print(f"| softmax warp 2 arrived on p_full(u) -> p_full(u) seen (the CTA's last warp arrives later) | {med(a[u, 5] - a[u, 3]):.0f} |")
    print(f"| step u - 1 committed -> softmax warp 2 holds S(u + 1) | {med(a[u, 12] - a[u - 1, 7]):.0f} |")


if __name__ == "__main__":
    main()
