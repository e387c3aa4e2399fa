"""-m gpu: the allocation-free gate + RMSNorm backward (orbit_gate_norm_bwd_noalloc) against orbit_gate_norm_bwd.

The variant exists for hosts that may not allocate device memory (a plugin that only receives input/output pointers
from the runtime that owns the GPU arena, or a server whose arena is closed after start-up); its scratch is a device
array built into the library.  Called here through the C-ABI directly, twice in a row with different sizes, so that
the second call runs on whatever the first left in the shared scratch.  Same tolerance as the other kernel tests
(identical arithmetic: results must be bitwise equal to the workspace entry point).
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from orbitssm_b200 import _lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _noalloc(y, z, w, rstd, dout):
    M, D = y.shape
    dy = torch.empty_like(y)
    dz = torch.empty((M, D), device=y.device, dtype=y.dtype)
    dw = torch.empty((D,), device=y.device, dtype=torch.float32)
    lib = _lib.load()
    st = lib.orbit_gate_norm_bwd_noalloc(_p(y), _p(z), z.stride(0), _p(w), _p(rstd), _p(dout), _p(dy), _p(dz), D, _p(dw),
                                         M, D, _lib.BF16 if y.dtype == torch.bfloat16 else _lib.F32,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "orbit_gate_norm_bwd_noalloc")
    return dy, dz, dw


def _case(M, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randn(M, D, generator=g).to(dtype).to(DEV)
    zwide = torch.randn(M, D + 64, generator=g).to(dtype).to(DEV)
    z = zwide[:, 32:32 + D]
    w = (1.0 + 0.1 * torch.randn(D, generator=g)).to(DEV)
    dout = torch.randn(M, D, generator=g).to(dtype).to(DEV)
    _, rstd = ops.gate_norm_fwd(y, z, w, 1e-5)
    return y, z, w, rstd, dout


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    for (M, D, dtype, seed) in ((1500, 2048, torch.bfloat16, 0), (77, 512, torch.float32, 1)):
        y, z, w, rstd, dout = _case(M, D, dtype, seed)
        want_dy, want_dz, want_dw = ops.gate_norm_bwd(y, z, w, rstd, dout)
        dy, dz, dw = _noalloc(y, z, w, rstd, dout)
        torch.cuda.synchronize()
        assert torch.equal(dy, want_dy) and torch.equal(dz, want_dz)
        assert torch.equal(dw, want_dw), float((dw - want_dw).abs().max())


def test_sizes_beyond_the_built_in_scratch_are_refused():
    y, z, w, rstd, dout = _case(600, 8192, torch.bfloat16, 2)
    with pytest.raises(NotImplementedError, match="exceed the built-in"):
        _noalloc(y, z, w, rstd, dout)


def test_gate_only_call_needs_no_scratch_and_is_served_at_any_size():
    # w == NULL: there is no weight gradient, hence no partial sums; a size that a norm would be refused at passes
    M, D = 600, 8192
    g = torch.Generator().manual_seed(3)
    y = torch.randn(M, D, generator=g).to(torch.bfloat16).to(DEV)
    z = torch.randn(M, D, generator=g).to(torch.bfloat16).to(DEV)
    dout = torch.randn(M, D, generator=g).to(torch.bfloat16).to(DEV)
    want_dy, want_dz, _ = ops.gate_norm_bwd(y, z, None, None, dout)
    dy, dz = torch.empty_like(y), torch.empty_like(y)
    lib = _lib.load()
    st = lib.orbit_gate_norm_bwd_noalloc(_p(y), _p(z), z.stride(0), None, None, _p(dout), _p(dy), _p(dz), D, None, M, D,
                                         _lib.BF16, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "orbit_gate_norm_bwd_noalloc")
    torch.cuda.synchronize()
    assert torch.equal(dy, want_dy) and torch.equal(dz, want_dz)
