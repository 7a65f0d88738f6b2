"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, and rejects invalid
arguments before any launch with the reference's error behaviour (std::invalid_argument -> status -1 -> ValueError).
No compute call runs here (there is no GPU in this environment)."""
import ctypes as C
import os
import re

import pytest

from owoinfer_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "owoinfer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    declared = header_symbols()
    assert len(declared) >= 20
    missing = [s for s in declared if not hasattr(lib, s)]
    assert not missing, missing
    assert sorted(_lib.EXPORTS) == declared


def test_numerics_versions():
    lib = _lib.lib()
    # quant.h:38, quant4.h:36, w4a8_decode.h:27: bit-identical to the reference's version 1; the attention word carries
    # the reference's contract version (attention_q8.h:73) in its low half and this kernel's own revision above it.
    assert [lib.b2_numerics_version(i) for i in (0, 1, 3)] == [1, 1, 1]
    att = lib.b2_numerics_version(2)
    assert att & 0xFFFF == 1 and att >> 16 >= 1
    assert lib.b2_numerics_version(7) == 0 and lib.b2_numerics_version(-1) == 0


def _status(rc):
    return rc, _lib.lib().b2_last_error_message().decode()


A16 = C.c_void_p(0x1000)  # a 16-byte aligned fake device address: validation never dereferences it
A8 = C.c_void_p(0x1008)


def test_rotate_quantize_rejects_bad_shapes():
    lib = _lib.lib()
    f = lib.b2_rotate_quantize
    # tests/unit/test_quant_kernels.cu:573-606 (argument rejection)
    for k in (0, 100, 255, 32768 + 256):
        rc, msg = _status(f(A16, C.c_int64(max(k, 8)), A16, C.c_int64(max(k, 16)), A16, C.c_int64(4), C.c_int(k), None))
        assert rc == -1 and "multiple of 256" in msg
    rc, msg = _status(f(A16, C.c_int64(256), A16, C.c_int64(256), A16, C.c_int64(-1), C.c_int(256), None))
    assert rc == -1 and "negative" in msg
    rc, msg = _status(f(None, C.c_int64(256), A16, C.c_int64(256), A16, C.c_int64(1), C.c_int(256), None))
    assert rc == -1 and "null" in msg
    rc, msg = _status(f(A8, C.c_int64(256), A16, C.c_int64(256), A16, C.c_int64(1), C.c_int(256), None))
    assert rc == -1 and "aligned" in msg
    rc, msg = _status(f(A16, C.c_int64(260), A16, C.c_int64(256), A16, C.c_int64(1), C.c_int(256), None))  # ldx % 8
    assert rc == -1
    rc, msg = _status(f(A16, C.c_int64(256), A16, C.c_int64(264), A16, C.c_int64(1), C.c_int(256), None))  # ldq % 16
    assert rc == -1
    # m == 0 is a no-op, even with null operands.
    assert f(None, C.c_int64(256), None, C.c_int64(256), None, C.c_int64(0), C.c_int(256), None) == 0


def test_norm_variant_rejects_cross_warp_rows():
    lib = _lib.lib()
    f = lib.b2_rms_norm_modulate_rotate_quantize
    # k = 32768 with one row: torch would split the row across warps (quant.h: "k <= 7680 always works").
    rc, msg = _status(f(A16, C.c_int64(32768), A16, A16, A16, A16, C.c_int64(32768), A16, C.c_int64(1 << 20), C.c_int(32768),
                        None, None, C.c_int64(0)))
    assert rc == -1 and "cross-warp" in msg
    rc, msg = _status(f(A16, C.c_int64(3072), A8, A16, A16, A16, C.c_int64(3072), A16, C.c_int64(4), C.c_int(3072), None,
                        None, C.c_int64(0)))
    assert rc == -1 and "norm_weight" in msg
    rc, msg = _status(f(A16, C.c_int64(3072), A16, A16, A16, A16, C.c_int64(3072), A16, C.c_int64(4), C.c_int(3072), None,
                        A16, C.c_int64(100)))
    assert rc == -1 and "ldy" in msg


def _ops(m=4, n=264, k=512, ldx=512, x=A16, w=A16, ws=A16):
    return _lib.Int8Operands(x.value, ldx, A16.value, w.value, ws.value, m, n, k)


def test_gemm_rejects_bad_operands():
    lib = _lib.lib()
    # tests/unit/test_quant_kernels.cu:871-901
    for bad in (_ops(k=0), _ops(k=131072), _ops(k=520, ldx=520), _ops(ldx=500), _ops(n=0), _ops(m=-1), _ops(w=A8),
                _ops(x=A8)):
        rc, msg = _status(lib.b2_int8_gemm(C.byref(bad), None, A16, C.c_int64(264), None, 0))
        assert rc == -1, msg
    ok = _ops()
    rc, msg = _status(lib.b2_int8_gemm(C.byref(ok), None, A16, C.c_int64(260), None, 0))  # ldo < n
    assert rc == -1 and "row stride" in msg
    rc, msg = _status(lib.b2_int8_gemm(C.byref(_ops(n=260)), None, A16, C.c_int64(264), None, 0))  # n % 8
    assert rc == -1
    rc, msg = _status(lib.b2_int8_gemm_gated_residual(C.byref(ok), None, None, A16, C.c_int64(264), None, 0))
    assert rc == -1 and "gate" in msg
    rc, msg = _status(lib.b2_int8_gemm_situ_glu(C.byref(_ops(n=268)), A16, C.c_int64(136), None, 0))  # F % 4
    assert rc == -1 and "F % 4" in msg
    rc, msg = _status(lib.b2_int8_gemm_situ_glu(C.byref(ok), A16, C.c_int64(130), None, 0))  # ldo < F or % 4
    assert rc == -1
    # m == 0: nothing runs.
    assert lib.b2_int8_gemm(C.byref(_ops(m=0)), None, A16, C.c_int64(264), None, 0) == 0


def _w4(packed=A16, s_rel=A16, kind=0, group=64, s_channel=A16):
    return _lib.W4Weight(packed.value, s_rel.value, kind, group, None, s_channel.value)


def test_w4a8_gemm_checks_every_argument_before_the_decode():
    """Nothing may be launched for a rejected call (the operands here are fake addresses: a launch would fault, and this
    process has no device at all): the GEMM's own argument rules are applied up front."""
    lib = _lib.lib()
    f = lib.b2_w4a8_gemm
    i64 = C.c_int64

    def call(x=A16, ldx=512, xs=A16, w=None, m=4, n=264, k=512, epi=0, aux=None, out=A16, ldo=264, scratch=A16):
        w = _w4() if w is None else w
        return _status(f(x, i64(ldx), xs, C.byref(w), i64(m), i64(n), i64(k), C.c_int(epi), aux, out, i64(ldo), scratch, None))

    assert call(x=None)[0] == -1                 # x_q null with m > 0
    assert call(x=A8)[0] == -1                   # x_q misaligned
    assert call(ldx=500)[0] == -1                # ldx % 16
    assert call(k=520, ldx=520)[0] == -1         # k % 16
    assert call(n=260, ldo=264)[0] == -1         # n % 8
    assert call(out=None)[0] == -1
    assert call(ldo=256)[0] == -1                # ldo < n
    assert call(epi=1, aux=None)[0] == -1        # gated residual without a gate
    assert call(epi=1, aux=A8)[0] == -1          # misaligned gate
    assert call(epi=2, n=268)[0] == -1           # F % 4
    assert call(epi=3)[0] == -1
    rc, msg = call(scratch=None, w=_w4(kind=1))   # fp16 group scales are decoded to a scratch first: it must be there
    assert rc == -1 and "scratch" in msg
    assert call(n=1 << 33)[0] == -1 and call(k=1 << 31, ldx=1 << 31)[0] == -1
    assert call(w=_w4(group=24))[0] == -1        # group % 16
    assert call(w=_w4(group=96))[0] == -1        # k % group
    assert call(w=_w4(kind=2))[0] == -1
    assert call(w=_w4(packed=C.c_void_p(0x1004)))[0] == -1
    assert call(m=0)[0] == 0                     # no-op, nothing decoded


def test_w4a8_noalloc_size_check_cannot_wrap():
    """n * k is compared by division: extents whose 64-bit product wraps to a small number are still refused."""
    lib = _lib.lib()
    f = lib.b2_w4a8_gemm_noalloc
    i64 = C.c_int64
    w = _w4()
    for n, k in ((1 << 33, 1 << 31), (1 << 62, 4), (1 << 40, 1 << 24), (4096, 8192), (0, 512), (512, 0), (-8, 512)):
        rc, msg = _status(f(A16, i64(512), A16, C.byref(w), i64(4), i64(n), i64(k), C.c_int(0), None, A16, i64(264), None))
        assert rc == -1 and "does not fit" in msg, (n, k, msg)


def test_decode_grouped_rejects_bad_extents():
    lib = _lib.lib()
    f = lib.b2_decode_grouped_int8
    i64 = C.c_int64
    assert f(A16, A16, 0, None, i64(1 << 33), i64(512), 64, A16, None, None) == -1
    assert f(A16, A16, 0, None, i64(8), i64(1 << 20), 64, A16, None, None) == -1
    assert f(A16, A16, 0, None, i64(8), i64(512), 24, A16, None, None) == -1
    assert f(A16, A16, 3, None, i64(8), i64(512), 64, A16, None, None) == -1
    assert f(None, None, 0, None, i64(0), i64(512), 64, None, None, None) == 0


def test_attention_rejects_bad_arguments():
    lib = _lib.lib()
    o = _lib.AttentionOptions(3, 0, 0)
    v = _lib.View3(A16.value, 128, 24, 9216, 128)
    out = _lib.View3(A16.value, 128, 24, 3072, 128)
    f = lib.b2_attention_q8
    args = lambda **kw: [C.byref(kw.get("o", o)), C.byref(kw.get("q", v)), C.byref(kw.get("k", v)), C.byref(kw.get("v", v)),
                         C.byref(kw.get("out", out)), A16, A16, C.c_int(1), C.c_int(kw.get("max_seqlen", 128)),
                         C.c_float(kw.get("scale", 0.088)), kw.get("ws", C.c_void_p(0x10000)), C.c_size_t(kw.get("nbytes", 1 << 30)),
                         None, None]
    assert _status(f(*args(scale=0.0)))[0] == -1
    assert _status(f(*args(scale=float("nan"))))[0] == -1
    assert _status(f(*args(max_seqlen=0)))[0] == -1
    assert _status(f(*args(o=_lib.AttentionOptions(0, 0, 0))))[0] == -3  # other variants: not built
    assert _status(f(*args(o=_lib.AttentionOptions(3, 500.0, 0))))[0] == -1  # p_range beyond e4m3
    assert _status(f(*args(q=_lib.View3(A16.value, 128, 24, 9217, 128))))[0] == -1  # stride not % 8
    assert _status(f(*args(k=_lib.View3(A16.value, 128, 12, 9216, 128), v=_lib.View3(A16.value, 128, 12, 9216, 128))))[0] == -3
    rc, msg = _status(f(*args(nbytes=1024)))
    assert rc == -1 and "workspace" in msg
    rc, msg = _status(f(*args(ws=C.c_void_p(0x10010))))
    assert rc == -1 and "workspace" in msg
    need = lib.b2_attention_q8_workspace_bytes(C.byref(o), 128, 128, 1, 128, 24, 24)
    lay = _lib.AttentionLayout()
    assert lib.b2_attention_q8_layout(C.byref(o), C.c_int64(128), C.c_int64(128), 1, 128, 24, 24, C.byref(lay)) == 0
    assert need == lay.total and lay.q_blocks == 4 and lay.k_blocks == 2 and lay.chunks == 1
    assert lay.q_i8 % 256 == 0 and lay.k_i8 % 256 == 0 and lay.v8 % 256 == 0


def test_attention_int8_fp8_ranges_follow_the_reference_rule():
    """attention_q8.h:79-88, attention_q8.cu:255-261: int8_fp8 defaults to 112 / 4.5 and refuses ranges whose 64-key
    partial sum could overflow fp16 (117 / 8.74: 64 * 120 * 9 = 69120), before anything is launched."""
    lib = _lib.lib()
    v = _lib.View3(A16.value, 64, 2, 768, 128)
    cu = A16
    call = lambda o: _status(lib.b2_attention_q8(C.byref(o), C.byref(v), C.byref(v), C.byref(v), C.byref(v), cu, cu, 1, 64,
                                                 C.c_float(0.0883883), None, 0, None, None))
    rc, msg = call(_lib.AttentionOptions(2, 117.0, 8.74))
    assert rc == -1 and "65504" in msg
    rc, msg = call(_lib.AttentionOptions(2, 0.0, 0.0))     # defaults pass the rule; the call then stops at the workspace
    assert rc == -1 and "workspace" in msg
    rc, msg = call(_lib.AttentionOptions(2, 112.0, 9.0))   # 64 * 112 * 9 = 64512: allowed
    assert rc == -1 and "workspace" in msg
    rc, msg = call(_lib.AttentionOptions(1, 0.0, 0.0))     # the fp16 P.V variants are not built
    assert rc == -3 and "only the e4m3" in msg


def test_block_rejects_mismatched_buffers():
    lib = _lib.lib()
    run = _lib.BlockRun()
    run.struct_size = C.sizeof(_lib.BlockRun)
    run.tokens, run.D, run.F, run.heads = 1280, 3072, 12288, 24
    run.cu_seqlens, run.batch, run.max_seqlen, run.tier = A16.value, 1, 1280, 0
    run.attention = _lib.AttentionOptions(3, 0, 0)
    need = lib.b2_block_quant_workspace_bytes(C.byref(run))
    assert need > 1280 * (3 * 3072 * 2 + 12288 * 2)
    w = _lib.BlockWeights()
    w.struct_size = C.sizeof(_lib.BlockWeights)
    b = _lib.BlockBuffers()
    b.struct_size = C.sizeof(_lib.BlockBuffers)
    b.x = b.mod = b.rope = b.workspace = 0x10000
    b.workspace_bytes = need - 1
    rc, msg = _status(lib.b2_run_block_quant(C.byref(w), C.byref(b), C.byref(run), None))
    assert rc == -1 and "workspace" in msg  # dit_block_quant.cpp:268-279: refused before any launch
    b.workspace_bytes = need
    b.x = 0x10010
    rc, msg = _status(lib.b2_run_block_quant(C.byref(w), C.byref(b), C.byref(run), None))
    assert rc == -1 and "256-byte" in msg
    run.D = 3000
    assert lib.b2_block_quant_workspace_bytes(C.byref(run)) == 0
    run.D, run.tier = 3072, 9
    assert _status(lib.b2_run_block_quant(C.byref(w), C.byref(b), C.byref(run), None))[0] == -1


def test_step_graph_cache_handle_and_checks():
    """A cache is host state until its first forward; a graphed forward is refused on the default stream and on a bad
    forward before anything is enqueued (dit_graph.h:49-52: the stream of a capture is not the default stream)."""
    lib = _lib.lib()
    g = C.c_void_p()
    assert lib.b2_dit_graphs_create(4, C.byref(g)) == 0 and g.value
    st = _lib.DitGraphStats()
    assert lib.b2_dit_graphs_stats(g, C.byref(st)) == 0
    assert (st.replays, st.captures, st.collisions, st.eager, st.evictions, st.size) == (0, 0, 0, 0, 0, 0)
    m, f, replayed = _lib.DitModel(), _lib.Forward(), C.c_int(7)
    rc, msg = _status(lib.b2_dit_forward_graphed(g, C.byref(m), C.byref(f), None, C.byref(replayed)))
    assert rc == -1 and "default stream" in msg and replayed.value == 0
    rc, msg = _status(lib.b2_dit_forward_graphed(g, C.byref(m), C.byref(f), C.c_void_p(0x1000), C.byref(replayed)))
    assert rc == -1 and "older header" in msg
    assert _status(lib.b2_dit_forward_graphed(None, C.byref(m), C.byref(f), C.c_void_p(0x1000), None))[0] == -1
    assert lib.b2_dit_graphs_clear(g) == 0 and lib.b2_dit_graphs_destroy(g) == 0 and lib.b2_dit_graphs_destroy(None) == 0


def test_cpp_shim_compiles_against_the_reference_headers():
    """include/owoinfer_b200_shim.hpp takes moss_dit::run_block_quant's parameters in its order
    (src/models/moss_dit/dit_block_quant.h:145-146): checked by the compiler against the reference's own headers."""
    import shutil
    import subprocess
    from oracle import oracle_lib
    ref = oracle_lib.reference_root()
    cuda_inc = "/usr/local/cuda/include"
    if ref is None or shutil.which("g++") is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("needs the reference tree, g++ and the CUDA headers")
    caller = """
#include "owoinfer_b200_shim.hpp"
namespace md = mi::moss_dit;
void call(const md::BlockTensors& w, const md::QuantBlockBuffers& a, const md::BlockRun& run, const md::QkvGemm& g,
          const md::FusedRouteSnapshot& r, cudaStream_t s, void* ws, std::size_t n) {
  // the reference's own entry point and the adapter take the same leading arguments
  void (*ref_fn)(const md::BlockTensors&, const md::QuantBlockBuffers&, const md::BlockRun&, const md::QkvGemm&,
                 const md::FusedRouteSnapshot&, md::AttentionMode, cudaStream_t, int) = &md::run_block_quant;
  (void)ref_fn;
  if (md::b200_can_run(w, a, run, md::AttentionMode::kQ8Fp8F32Acc)) {
    md::run_block_quant_b200(w, a, run, g, r, md::AttentionMode::kQ8Fp8F32Acc, s, 0, ws, n);
  }
  (void)md::b200_workspace_bytes(w, run);
}
"""
    r = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-I", os.path.join(ref, "src"), "-I", os.path.join(ROOT, "include"),
                        "-I", cuda_inc, "-x", "c++", "-"], input=caller, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_python_layer_fails_loudly_without_library(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()
