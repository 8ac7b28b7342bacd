"""The C-ABI shared library: it loads, exports every symbol include/pq_b200.h declares, and its
host-side argument checks reject bad calls before anything is launched (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

from pyraquant_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "pq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    lib = _lib.load()
    names = declared_symbols()
    assert "pq_int8_gemm" in names and "pq_quant_rows" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in pq_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes prototype"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.pq_version() >= 100
    assert _lib.status_str(0) == "ok"
    assert "NULL" in _lib.status_str(1)
    assert "unknown" in _lib.status_str(999)


def test_options_roundtrip():
    old = _lib.get_option("gemm_pn")
    _lib.set_option("gemm_pn", 4)
    assert _lib.get_option("gemm_pn") == 4
    _lib.set_option("gemm_pn", old)
    with pytest.raises(RuntimeError):
        _lib.set_option("no_such_knob", 1)


def test_documented_options_exist():
    """Every knob the header documents is accepted by pq_set_option and starts at 0 or its documented default."""
    header = (ROOT / "include" / "pq_b200.h").read_text()
    block = header[header.index("Internal tuning / test knobs"):header.index("int pq_set_option")]
    names = re.findall(r'"([a-z0-9_]+)"', block)
    assert {"quant_tpr", "gemm_stages", "gemm_block_n", "gemm_pm", "gemm_pn", "gemm_max_ctas", "gemm_epi_warps",
            "gemm_pair", "gemm_debug_timing"} <= set(names)
    for n in names:
        v = _lib.get_option(n)
        _lib.set_option(n, v)
        assert _lib.get_option(n) == v


def test_quant_rows_argument_checks():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.pq_quant_rows(None, 0, 0, 64, 64, None, None, None) == 0            # M == 0: no-op
    assert lib.pq_quant_rows(None, 0, 4, 64, 64, p16, p16, None) == 1              # null x
    assert lib.pq_quant_rows(p16, 7, 4, 64, 64, p16, p16, None) == 4               # bad dtype
    assert lib.pq_quant_rows(p16, 0, 4, 60, 64, p16, p16, None) == 3               # K % 8
    assert lib.pq_quant_rows(p16, 0, 4, 64, 32, p16, p16, None) == 2               # ldx < K
    assert lib.pq_quant_rows(p16 + 2, 0, 4, 64, 64, p16, p16, None) == 3           # misaligned x
    assert lib.pq_quant_rows(p16, 0, -1, 64, 64, p16, p16, None) == 2              # negative M
    assert lib.pq_quant_rows_g32(p16, 0, 4, 72, 72, p16, p16, None) == 3           # K % 32


def test_gemm_argument_checks():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p16 = (ctypes.addressof(buf) + 15) & ~15

    def gemm(xq=p16, ldx=64, s_row=p16, w=p16, ldw=64, s_col=p16, bias=None, t=None, ldt=0, lb=None, ldb=0, R=0,
             lr_dtype=0, out=p16, out_dtype=0, ldo=64, M=8, N=64, K=64, ws=None, ws_bytes=0):
        return lib.pq_int8_gemm(xq, ldx, s_row, w, ldw, s_col, bias, t, ldt, lb, ldb, None, R, lr_dtype, out, out_dtype,
                                ldo, M, N, K, ws, ws_bytes, None, None)

    assert gemm(M=0) == 0
    assert gemm(xq=None) == 1
    assert gemm(K=40, ldx=48, ldw=48) == 3          # K % 16
    assert gemm(ldx=72) == 3                         # ldx % 16
    assert gemm(out_dtype=5) == 4
    assert gemm(ldo=32) == 2                         # ldo < N
    assert gemm(t=p16, ldt=32) == 1                  # t without lb
    assert gemm(t=p16, ldt=16, lb=p16, ldb=64, R=16) == 7    # rank other than 32
    assert gemm(ws=p16, ws_bytes=8) == 8             # workspace too small
    assert gemm(N=0) == 2


def test_gemm_ex_argument_checks():
    """The epilogue variants are refused, before anything is launched, for shapes their store path does not cover."""
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p16 = (ctypes.addressof(buf) + 15) & ~15

    def ex(N=64, ldo=64, epi=1, out=p16, M=8, K=64):
        return lib.pq_int8_gemm_ex(p16, 64, p16, p16, 64, p16, None, None, 0, None, 0, None, 0, 0, out, 0, ldo, M, N, K,
                                   epi, None, 0, None)

    assert ex(M=0) == 0
    assert ex(epi=8) == 7                            # unknown flag
    assert ex(N=40, ldo=40) == 7                     # N % 32
    assert ex(ldo=68) == 7                           # ldo % 8
    assert ex(out=p16 + 4) == 7                      # out not 16-byte aligned
    assert ex(K=40) == 3                             # the plain GEMM's checks still come first
    assert ex(epi=4) == 1                            # the gate flag without a gate vector

    def gated(gate=p16, ld_gate=64, rps=0, N=64, ldo=64):
        return lib.pq_int8_gemm_gated(p16, 64, p16, p16, 64, p16, None, None, 0, None, 0, None, 0, 0, gate, ld_gate, rps,
                                      p16, 0, ldo, 8, N, 64, 1, None, 0, None)
    assert gated(gate=None) == 1
    assert gated(ld_gate=60) == 3                    # gate row stride
    assert gated(gate=p16 + 4) == 3                  # gate not 16-byte aligned
    assert gated(rps=-1) == 3
    assert gated(N=40, ldo=40, ld_gate=40) == 7      # shape outside the CTA-pair kernel's vector store path


def test_gemm_bcast_argument_checks():
    """The broadcast-store GEMM refuses bad destination lists before anything is launched."""
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p16 = (ctypes.addressof(buf) + 15) & ~15

    def bc(more, n, N=64, ldo=64, M=8):
        arr = (ctypes.c_void_p * max(1, len(more)))(*more) if more is not None else None
        return lib.pq_int8_gemm_bcast(p16, 64, p16, p16, 64, p16, None, None, 0, None, 0, None, 0, 0, p16, arr, n, 0, ldo,
                                      M, N, 64, 0, None, 0, None)

    assert bc([p16], 1, M=0) == 0                    # nothing to do
    assert bc([p16] * 8, 8) == 2                     # more than PQ_MAX_OUT_MORE destinations
    assert bc([p16], -1) == 2
    assert bc(None, 1) == 1                          # no list
    assert bc([p16, None], 2) == 1                   # a null destination
    assert bc([p16 + 4], 1) == 3                     # destination not 16-byte aligned
    assert bc([p16], 1, N=40, ldo=40) == 7           # shape outside the CTA-pair kernel's vector store path


def test_scatter_and_gather_argument_checks():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p16 = (ctypes.addressof(buf) + 15) & ~15
    assert lib.pq_scatter_rows(p16, 64, 4, p16, p16, p16, p16, 0, p16, 64, 16, 64, 0, None) == 0   # nothing to do
    assert lib.pq_scatter_rows(p16, 64, 4, p16, p16, p16, p16, 2, p16, 64, 16, 60, 0, None) == 3   # C % 8
    assert lib.pq_scatter_rows(p16, 64, 4, None, p16, p16, p16, 2, p16, 64, 16, 64, 0, None) == 1
    assert lib.pq_gather_rows(p16, 0, 16, 64, 64, None, 4, p16, 64, None) == 1
    assert lib.pq_gather_quant_rows(p16, 0, 16, 64, 64, None, 4, p16, p16, None) == 1
    ada = lambda K=64, ldx=64, x=p16, xm=None, ldxm=0, rps=0, eps=1e-6, M=4: lib.pq_adaln_quant_rows(
        x, 0, M, K, ldx, p16, p16, K, rps, eps, xm, ldxm, p16, p16, None)
    assert ada(M=0) == 0
    assert ada(K=60, ldx=64) == 3                     # K % 8
    assert ada(x=None) == 1
    assert ada(xm=p16, ldxm=32) == 2                  # x_mod rows shorter than K
    assert ada(rps=-1) == 2
    assert ada(eps=-1.0) == 2
    qc = lambda K0=64, K1=64, x1=p16, ld1=64: lib.pq_quant_rows_cat(p16, K0, 64, x1, K1, ld1, 0, 4, p16, p16, None)
    assert lib.pq_quant_rows_cat(p16, 64, 64, p16, 64, 64, 0, 0, p16, p16, None) == 0
    assert qc(x1=None) == 1
    assert qc(K1=60) == 3
    assert qc(K1=128, ld1=64) == 2
    assert lib.pq_quant_rows_cat(p16, 16384, 16384, p16, 64, 64, 0, 4, p16, p16, None) == 7
    dc = lambda K0=64, x1=p16, K1=64: lib.pq_lowrank_down_cat(p16, K0, 128, x1, K1, 64, 0, p16, 128, 32, p16, 32, 4, None, 0, None)
    assert dc(x1=None) == 1
    assert dc(K0=32) == 7                             # seam off the 64-element grid
    assert dc(K1=0) == 2
    assert lib.pq_i8_mma_issue_loop(0, 10, p16, None, 0, None) == 2
    assert lib.pq_wait_probe(None, 256, 1000, None) == 1
    assert lib.pq_wait_probe(p16, 8, 1000, None) == 8
    assert lib.pq_wait_probe(p16, 256, 0, None) == 2
    # group-32 GEMM: K must be whole 128-byte stages
    assert lib.pq_int8_gemm_g32(p16, 96, p16, p16, 96, p16, None, p16, 0, 64, 8, 64, 96, None, 0, None) == 7
    assert lib.pq_int8_gemm_g32(p16, 128, None, p16, 128, p16, None, p16, 0, 64, 8, 64, 128, None, 0, None) == 1


def test_operand_extent_checks_run_on_the_host():
    """The C ABI sees bare pointers; the Python operators check every operand's extent before a launch, so a short
    scale, bias or low-rank tensor is an AssertionError instead of an out-of-bounds device read."""
    import torch
    from pyraquant_b200 import ops
    M, N, K = 8, 64, 64
    f = lambda *shape: torch.zeros(*shape)
    ok = dict(s_row=f(M), w_scale=f(N), bias=f(N), t=f(M, 32), lb=f(32, N), lb_t=f(N, 32))
    ops.check_gemm_extents(M, N, K, **ok)
    ops.check_gemm_extents(M, N, K, f(M), f(N), None, None, None)
    for key, bad in (("s_row", f(M - 1)), ("w_scale", f(N + 1)), ("bias", f(N - 8)), ("t", f(M - 1, 32)),
                     ("lb", f(32, N - 8)), ("lb", f(16, N)), ("lb_t", f(32, N))):
        with pytest.raises(AssertionError):
            ops.check_gemm_extents(M, N, K, **{**ok, key: bad})
    with pytest.raises(AssertionError):
        ops.check_gemm_extents(M, N, K, f(M), f(N), None, f(M, 32), None)          # t without lb
    with pytest.raises(AssertionError):
        ops.check_gemm_extents(M, N, K, f(M), f(N), None, None, None, s_lo=f(N - 1), m_hi=4)
    with pytest.raises(AssertionError):
        ops.check_gemm_extents(M, N, K, f(M), f(N), None, None, None, s_lo=f(N), m_hi=M + 1)
    i = lambda n: torch.zeros(n, dtype=torch.int32)
    ops.check_scatter_extents(10, 16, i(3), i(4), i(5), f(5))
    with pytest.raises(AssertionError):
        ops.check_scatter_extents(10, 16, i(3), i(3), i(5), f(5))                   # ptr too short
    with pytest.raises(AssertionError):
        ops.check_scatter_extents(10, 16, i(3), i(4), i(5), f(4))                   # src / beta differ
    with pytest.raises(AssertionError):
        ops.check_scatter_extents(10, 2, i(3), i(4), i(5), f(5))                    # more tokens than canvas rows
