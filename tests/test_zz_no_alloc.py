"""The allocation-free Linear entry point (pq_int8_linear_noalloc) against the regular entry points.

Some users of this library may never call cudaMalloc -- a serving process whose memory pool owns the whole
device, code running inside a stream capture, a plugin with a fixed budget -- so the library offers one forward
call whose intermediates (int8 codes, row scales) live in a fixed array inside the library instead of in buffers
that somebody has to allocate.  The test drives it through the C ABI twice in a row (the array is reused and keeps
the previous call's contents) and expects exactly the bytes that quant_rows + the fused GEMM produce through the
regular entry points; it also checks that shapes beyond the fixed capacity are refused.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

from pyraquant_b200 import _lib, int8_exec

pytestmark = pytest.mark.gpu


def _noalloc_forward(x, w, s_col, bias, N):
    lib = _lib.load()
    M, K = x.shape
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    word = ctypes.c_void_p()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = lib.pq_int8_linear_noalloc(x.data_ptr(), _lib.DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.DTYPE_FP16,
                                    x.stride(0), w.data_ptr(), w.stride(0), s_col.data_ptr(),
                                    None if bias is None else bias.data_ptr(), out.data_ptr(), N, M, N, K,
                                    ctypes.byref(word), stream)
    assert rc == 0, _lib.status_str(rc)
    raw = ctypes.c_int32(-1)
    assert lib.pq_read_status_word(word.value, ctypes.byref(raw), 0, stream) == 0 and raw.value == 0
    return out


def test_noalloc_linear_matches_regular_path_twice(cuda_dev):
    g = torch.Generator().manual_seed(77)
    # second shape is smaller than the first: leftovers of call one must not leak into call two
    for (M, K, N, dtype, use_bias) in [(1000, 1024, 768, torch.bfloat16, True), (300, 512, 640, torch.float16, False)]:
        x = torch.randn(M, K, generator=g).to(dtype).to(cuda_dev)
        w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(cuda_dev)
        s_col = (torch.rand(N, generator=g) * 1e-3 + 1e-4).to(cuda_dev)
        bias = (torch.randn(N, generator=g) * 0.01).to(cuda_dev) if use_bias else None
        got = _noalloc_forward(x, w, s_col, bias, N)
        xq, sx = int8_exec.quant_rows(x)
        want = int8_exec.int8_gemm_fused(xq, sx, w, s_col, bias, dtype)
        torch.cuda.synchronize()
        assert torch.equal(got, want)                  # same kernels, same inputs: identical bytes
        again = _noalloc_forward(x, w, s_col, bias, N)   # back to back on the same array
        assert torch.equal(again, want)


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch(cuda_dev):
    lib = _lib.load()
    assert lib.pq_noalloc_scratch_bytes() >= 16 * 1024 * 1024
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=cuda_dev)
    w = torch.zeros(64, 64, dtype=torch.int8, device=cuda_dev)
    s = torch.ones(64, device=cuda_dev)
    out = torch.empty(8, 64, dtype=torch.bfloat16, device=cuda_dev)
    args = lambda M, K: (x.data_ptr(), 0, K, w.data_ptr(), K, s.data_ptr(), None, out.data_ptr(), 64, M, 64, K, None, None)
    assert lib.pq_int8_linear_noalloc(*args(16385, 64)) == 8            # too many rows
    assert lib.pq_int8_linear_noalloc(*args(8192, 4096)) == 8           # M * K > 16 MiB
    assert "workspace" in _lib.status_str(8)
    assert lib.pq_int8_linear_noalloc(*args(0, 64)) == 0                # nothing to do
