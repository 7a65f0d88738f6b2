"""The scratch-free W4A8 GEMM entry point (b2_w4a8_gemm_noalloc), checked against the regular entry point.

Some hosts cannot lend the library a scratch buffer and must not allocate one: a step loop that keeps the CUDA allocator
off its hot path, or an embedding whose device arena was fixed before it knew it would run 4-bit weights. For them the
decoded weight lands in a 16 MiB array that is part of the library itself. This test calls that entry point through the
C ABI twice in a row (the array keeps the previous call's bytes, so the second call must not be disturbed by them) and
expects exactly the bits of b2_w4a8_gemm; it also checks the size limit. The file name makes pytest collect it last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, xq, xs, w4, m, n, k, epilogue, aux, out, scratch=None):
    args = [C.c_void_p(xq.data_ptr()), C.c_int64(k), C.c_void_p(xs.data_ptr()), C.byref(w4), C.c_int64(m), C.c_int64(n),
            C.c_int64(k), C.c_int(epilogue), C.c_void_p(0 if aux is None else aux.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_int64(out.shape[1])]
    if scratch is not None:
        args.append(C.c_void_p(scratch.data_ptr()))
    args.append(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return getattr(lib, fn_name)(*args)


def test_noalloc_w4a8_gemm_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from owoinfer_b200 import _lib, ops, synth
    lib = _lib.lib()
    torch.manual_seed(11)
    # Two different weights and shapes back to back: the second call finds the first call's bytes in the shared array.
    cases = [(150, 520, 1024, 0), (300, 1024, 2048, 2), (97, 264, 512, 1)]
    for m, n, k, epilogue in cases:
        packed, s_rel, s_ch = synth.grouped_w4_weight(n, k, 40 + n)
        w4 = ops.make_w4(packed, s_rel, 64, s_ch)
        xq = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda")
        xs = torch.rand(m, device="cuda") * 1e-2
        n_out = n // 2 if epilogue == 2 else n
        aux = torch.randn(n, device="cuda").to(torch.bfloat16) if epilogue == 1 else None
        base = torch.randn((m, n_out), device="cuda").to(torch.bfloat16)  # the residual for epilogue 1, overwritten otherwise
        want, got = base.clone(), base.clone()
        scratch = torch.empty((n, k), dtype=torch.int8, device="cuda")
        assert _call(lib, "b2_w4a8_gemm", xq, xs, w4, m, n, k, epilogue, aux, want, scratch) == 0
        for _ in range(2):
            got.copy_(base)
            rc = _call(lib, "b2_w4a8_gemm_noalloc", xq, xs, w4, m, n, k, epilogue, aux, got)
            assert rc == 0, lib.b2_last_error_message().decode()
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # A weight larger than the built-in array is refused with a clear message, before any launch.
    n, k = 4096, 8192  # 32 MiB decoded
    rc = lib.b2_w4a8_gemm_noalloc(None, C.c_int64(k), None, C.byref(w4), C.c_int64(8), C.c_int64(n), C.c_int64(k), C.c_int(0),
                                  None, None, C.c_int64(n), None)
    assert rc == -1 and "does not fit" in lib.b2_last_error_message().decode()
    assert ops.kernel_status() == (0, 0)
