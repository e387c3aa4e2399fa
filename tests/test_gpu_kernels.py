"""-m gpu: every C-ABI kernel against its torch restatement (oracle/abi_reference.py, fp64) on the same seeded inputs.

Tolerances (normwise relative error ||a - r|| / ||r||):
  fp32 IO: 2e-5 forward, 2e-4 gradients (fp32 arithmetic against an fp64 restatement; sums of O(chunk * N) terms);
  bf16 IO: 6e-3 (outputs are rounded once to bfloat16, eps = 2^-8 = 3.9e-3; inputs are identical rounded values).
"""
import ctypes as C

import pytest
import torch

from orbitssm_b200 import _lib, ops
from oracle import abi_reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def tol(dtype, grad=False):
    if dtype == torch.bfloat16:
        return 6e-3
    return 2e-4 if grad else 2e-5


# ---------------------------------------------------------------------------------------------------- conv
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,C,W,pad,use_win", [(2, 77, 64, 4, 24, True), (1, 5, 16, 3, 0, True), (3, 130, 24, 2, 8, False),
                                                 (2, 33, 20, 4, 3, True), (1, 1, 8, 4, 0, True), (2, 256, 256, 4, 128, False)])
def test_conv(dtype, B, L, C, W, pad, use_win):
    g = torch.Generator().manual_seed(0)
    wide = torch.randn(B, L, C + pad, generator=g).to(dtype).to(DEV)
    x = wide[..., pad // 2: pad // 2 + C] if pad else wide            # column slice of a wider buffer (any row stride)
    weight = (torch.randn(C, W, generator=g) * 0.5).to(DEV)
    bias = torch.randn(C, generator=g).to(DEV)
    win = torch.randn(B, C, W, generator=g).to(DEV) if use_win else None
    dy = torch.randn(B, L, C, generator=g).to(dtype).to(DEV)
    y = ops.conv1d_fwd(x, weight, bias, win)
    y_ref = R.conv1d_fwd(x, weight, bias, win)
    assert rel(y, y_ref) < tol(dtype)
    dx, dwin, dw, db = ops.conv1d_bwd(x, weight, bias, win, dy, want_dwindow=use_win)
    rx, rwin, rw, rb = R.conv1d_bwd(x, weight, bias, win, dy, want_dwindow=use_win)
    assert rel(dx, rx) < tol(dtype, True)
    assert rel(dw, rw) < tol(dtype, True) and rel(db, rb) < tol(dtype, True)
    if use_win:
        assert rel(dwin, rwin) < tol(dtype, True)
    # bitwise reproducible (fixed-order reductions)
    dx2, _, dw2, db2 = ops.conv1d_bwd(x, weight, bias, win, dy, want_dwindow=use_win)
    assert torch.equal(dw, dw2) and torch.equal(db, db2) and torch.equal(dx, dx2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,C,W,pad,fwd_win", [(2, 333, 256, 4, 64, True), (1, 70, 1024, 4, 0, False), (3, 37, 128, 3, 8, True),
                                                 (2, 129, 512, 2, 16, False), (1, 2, 256, 4, 0, True), (2, 1100, 128, 4, 0, True)])
def test_conv_streaming_path(dtype, B, L, C, W, pad, fwd_win):
    """Channel counts the streaming kernels serve (whole warps of 8- or 16-byte channel vectors): several token runs per
    row, ragged run ends, a carried window read by the first run, no window gradient."""
    g = torch.Generator().manual_seed(1)
    wide = torch.randn(B, L, C + pad, generator=g).to(dtype).to(DEV)
    x = wide[..., pad // 2: pad // 2 + C] if pad else wide
    weight = (torch.randn(C, W, generator=g) * 0.5).to(DEV)
    bias = torch.randn(C, generator=g).to(DEV)
    win = torch.randn(B, C, W, generator=g).to(DEV) if fwd_win else None
    dy = torch.randn(B, L, C, generator=g).to(dtype).to(DEV)
    y = ops.conv1d_fwd(x, weight, bias, win)
    assert rel(y, R.conv1d_fwd(x, weight, bias, win)) < tol(dtype)
    dxw = torch.full((B, L, C + 16), float("nan"), device=DEV, dtype=dtype)
    dx_out = dxw[..., 8:8 + C]                                          # dx written in place into a strided column range
    dx, _, dw, db = ops.conv1d_bwd(x, weight, bias, win, dy, dx_out=dx_out)
    rx, _, rw, rb = R.conv1d_bwd(x, weight, bias, win, dy)
    assert dx.data_ptr() == dx_out.data_ptr() and torch.isnan(dxw[..., :8]).all() and torch.isnan(dxw[..., 8 + C:]).all()
    assert rel(dx, rx) < tol(dtype, True) and rel(dw, rw) < tol(dtype, True) and rel(db, rb) < tol(dtype, True)
    dx2, _, dw2, db2 = ops.conv1d_bwd(x, weight, bias, win, dy)
    assert torch.equal(dw, dw2) and torch.equal(db, db2) and torch.equal(dx, dx2)
    if fwd_win:                                                         # the same kernels also return the window's gradient
        dx3, dwin, dw3, _ = ops.conv1d_bwd(x, weight, bias, win, dy, want_dwindow=True)
        _, rwin, _, _ = R.conv1d_bwd(x, weight, bias, win, dy, want_dwindow=True)
        assert rel(dwin, rwin) < tol(dtype, True) and torch.equal(dx3, dx) and torch.equal(dw3, dw)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,H,K,Krot,trap", [(2, 77, 32, 32, 16, True), (1, 5, 3, 4, 1, True), (3, 130, 8, 8, 8, False),
                                               (2, 300, 40, 16, 0, True), (1, 1, 2, 1, 1, False)])
def test_hm_tail(dtype, B, L, H, K, Krot, trap):
    """HybridMamba clock tail (step size, trapezoid weight, angle feature scattered to its row pairs) and its backward
    against the torch restatement; raw inputs are column slices of a wider buffer; parameter gradients reproducible."""
    g = torch.Generator().manual_seed(11)
    wide = (torch.randn(B, L, 2 * H + Krot + 6, generator=g) * 2.0).to(dtype).to(DEV)
    dt_raw = wide[..., 2:2 + H]
    trap_raw = wide[..., 2 + H:2 + 2 * H] if trap else None
    th_raw = wide[..., 4 + 2 * H:4 + 2 * H + Krot] if Krot else None
    dt_bias = torch.randn(H, generator=g).to(DEV)
    trap_bias = torch.randn(H, generator=g).to(DEV) if trap else None
    omega = (torch.randn(Krot, generator=g) * 2.0).to(DEV) if Krot else None
    rot_idx = torch.randperm(K, generator=g)[:Krot].sort().values.to(torch.int32).to(DEV) if Krot else None
    delta, lam, feat = ops.hm_tail_fwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K)
    rd, rl, rf = R.hm_tail_fwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K)
    assert rel(delta, rd) < 2e-6 and (lam is None or rel(lam, rl) < 2e-6) and (feat is None or rel(feat, rf) < 2e-6)
    ddelta = torch.randn(B, L, H, generator=g).to(DEV)
    dlam = torch.randn(B, L, H, generator=g).to(DEV) if trap else None
    dfeat = torch.randn(B, L, K, generator=g).to(DEV) if Krot else None
    got = ops.hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, lam, ddelta, dlam, dfeat)
    want = R.hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, lam, ddelta, dlam, dfeat)
    for i, (a_, b_) in enumerate(zip(got, want)):
        assert (a_ is None) == (b_ is None), i
        if a_ is not None:
            assert rel(a_, b_) < (tol(dtype, True) if i < 3 else 2e-5), (i, rel(a_, b_))
    again = ops.hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, lam, ddelta, dlam, dfeat)
    assert all(a_ is None or torch.equal(a_, b_) for a_, b_ in zip(got, again))


def test_cp_state_pack_and_combine():
    """The exchange-step kernels of context parallelism against their torch restatements: the segment's summed log-decay
    (two-stage, fixed order: bitwise reproducible) and the combination of W gathered records, both directions."""
    g = torch.Generator().manual_seed(3)
    B, L, H, Rk, N, G, W = 2, 1000, 6, 2, 8, 4, 5
    n_state, BHR = B * H * Rk * N * G, B * H * Rk
    dA = (-torch.rand(B, L, H, Rk, generator=g) * 0.01).to(DEV)
    rec = torch.zeros(n_state + BHR, device=DEV)
    ops.cp_pack(dA, rec, n_state)
    want = torch.zeros(n_state + BHR)
    R.cp_pack(dA.cpu(), want, n_state)
    assert rel(rec[n_state:], want[n_state:]) < 1e-6
    rec2 = torch.zeros_like(rec)
    ops.cp_pack(dA, rec2, n_state)
    assert torch.equal(rec, rec2)
    for backward in (False, True):
        stride = n_state + BHR + (n_state if backward else 0)
        recs = torch.randn(W, stride, generator=g)
        recs[:, n_state:n_state + BHR] = -torch.rand(W, BHR, generator=g) * 3.0
        for rank in (0, 2, W - 1):
            got = ops.cp_combine(recs.to(DEV), W, rank, n_state, N * G, BHR, backward)
            assert rel(got, R.cp_combine(recs, W, rank, n_state, N * G, BHR, backward)) < 1e-6, (backward, rank)


def test_conv_empty_and_refusals():
    x = torch.zeros(2, 0, 16, device=DEV)
    w = torch.zeros(16, 4, device=DEV)
    assert ops.conv1d_fwd(x, w, None, None).shape == (2, 0, 16)
    with pytest.raises(NotImplementedError):
        ops.conv1d_fwd(torch.zeros(1, 4, 16, device=DEV), torch.zeros(16, 7, device=DEV), None, None)
    with pytest.raises(ValueError, match="CPU tensor"):
        ops.conv1d_fwd(torch.zeros(1, 4, 16), torch.zeros(16, 4), None, None)


# ---------------------------------------------------------------------------------------------------- gate + norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,D,gate,norm", [(37, 256, True, True), (5, 2048, True, True), (64, 4096, True, True),
                                           (19, 64, False, True), (19, 64, True, False), (300, 1024, True, True), (7, 12, True, True),
                                           (9, 9000, True, True), (1001, 2048, False, True), (3, 4096, False, True),
                                           (2501, 512, False, True), (2501, 512, True, True)])
def test_gate_norm(dtype, M, D, gate, norm):
    g = torch.Generator().manual_seed(1)
    y = torch.randn(M, D, generator=g).to(dtype).to(DEV)
    zwide = torch.randn(M, D + 64, generator=g).to(dtype).to(DEV)
    z = zwide[:, 32:32 + D] if gate else None
    w = (1.0 + 0.1 * torch.randn(D, generator=g)).to(DEV) if norm else None
    dout = torch.randn(M, D, generator=g).to(dtype).to(DEV)
    out, rstd = ops.gate_norm_fwd(y, z, w, 1e-5)
    ro, rr = R.gate_norm_fwd(y, z, w, 1e-5)
    assert rel(out, ro) < tol(dtype)
    if norm:
        assert rel(rstd, rr) < 1e-5
    dy, dz, dw = ops.gate_norm_bwd(y, z, w, rstd, dout)
    ry, rz, rw = R.gate_norm_bwd(y, z, w, rstd, dout)
    assert rel(dy, ry) < tol(dtype, True)
    if gate:
        assert rel(dz, rz) < tol(dtype, True)
    if norm:
        assert rel(dw, rw) < tol(dtype, True)
        dy2, _, dw2 = ops.gate_norm_bwd(y, z, w, rstd, dout)
        assert torch.equal(dw, dw2) and torch.equal(dy, dy2)


# ---------------------------------------------------------------------------------------------------- scan
def scan_case(B, L, H, R, O, G, N, dtype, gates, biases, chi, skip, trap, s0, seed=0):
    g = torch.Generator().manual_seed(seed)

    def rn(*s, scale=1.0):
        return torch.randn(*s, generator=g) * scale

    geo = ops.ScanGeometry(H=H, R=R, O=O, G=G, N=N)
    c = dict(geo=geo)
    c["u"] = rn(B, L, H * G * R).to(dtype).to(DEV)
    bc = rn(B, L, (R + O) * N + 16, scale=N ** -0.5 * 2).to(dtype).to(DEV)      # maps live as column slices of a slab
    c["Bhat"] = bc[..., :R * N].unflatten(-1, (R, N))
    c["Chat"] = bc[..., R * N:(R + O) * N].unflatten(-1, (O, N))
    c["gBp"] = (1 + rn(B, L, R, N, scale=0.3)).to(dtype).to(DEV) if gates else None
    c["gCp"] = (1 + rn(B, L, O, N, scale=0.3)).to(dtype).to(DEV) if gates else None
    c["beta"] = rn(H, R, R, N, scale=0.2).to(DEV) if biases else None
    c["gamma"] = rn(H, R, O, N, scale=0.2).to(DEV) if biases else None
    c["chi"] = (0.5 + rn(B, L, H, R, scale=0.2)).to(DEV) if chi else None
    dt = torch.nn.functional.softplus(rn(B, L, H, R) - 2.0)
    rate = torch.exp(torch.rand(H, R, generator=g) * 2.77)                       # 1 .. 16
    c["dA"] = (-(dt * rate)).to(DEV)
    if trap:
        lam = torch.sigmoid(rn(B, L, H, 1))
        lag = dt * (1 - lam)
        wd = lam * dt
        c["w"] = (wd + torch.cat([lag[:, 1:], torch.zeros(B, 1, H, R)], 1)).contiguous().to(DEV)
        c["wd"] = wd.expand(B, L, H, R).contiguous().to(DEV)
    else:
        c["w"] = dt.to(DEV)
        c["wd"] = None
    c["Dg"] = (1 + rn(H, G, R, O, scale=0.3)).to(DEV) if skip else None
    c["S0"] = rn(B, H, R, N, G).to(DEV) if s0 else None
    c["dy"] = rn(B, L, H * G * O).to(dtype).to(DEV)
    c["dS_fin"] = rn(B, H, R, N, G).to(DEV)
    c["euler"] = not trap
    return c


SCAN_CASES = [
    # B, L, H, R, O, G, N, gates, biases, chi, skip, trap, s0
    (2, 70, 3, 1, 1, 16, 16, False, False, False, True, False, False),
    (1, 128, 2, 1, 1, 64, 128, False, False, False, True, False, True),
    (2, 45, 2, 1, 1, 16, 16, False, True, False, True, True, True),
    (1, 37, 2, 4, 4, 16, 128, True, True, True, True, True, True),
    (2, 19, 3, 2, 1, 3, 8, False, False, False, True, False, True),
    (1, 23, 2, 2, 3, 4, 8, True, True, True, False, True, False),
    (1, 1, 1, 1, 1, 8, 8, False, False, False, False, False, True),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", SCAN_CASES)
def test_scan_ieee(dtype, case):
    B, L, H, Rr, O, G, N, gates, biases, chi, skip, trap, s0 = case
    c = scan_case(B, L, H, Rr, O, G, N, dtype, gates, biases, chi, skip, trap, s0)
    geo = c["geo"]
    T = ops.pick_chunk(geo, _lib.PRECISION_IEEE, True, 16)
    args = (c["u"], c["Bhat"], c["gBp"], c["Chat"], c["gCp"], c["beta"], c["gamma"], c["chi"], c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, T, _lib.PRECISION_IEEE, *args, c["S0"])
    ry, rS, _, _ = R.scan_fwd(geo, T, 0, *args, c["S0"])
    assert rel(y, ry) < tol(dtype), "y"
    assert rel(S_fin, rS) < 2e-5, "S_fin"
    g = ops.scan_bwd(geo, T, _lib.PRECISION_IEEE, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    rg = R.scan_bwd(geo, T, 0, *args, None, None, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None, S0=c["S0"])
    for k, v in rg.items():
        if v is None:
            assert g[k] is None, k
            continue
        t = tol(dtype, True) if k == "du" else 2e-4
        assert rel(g[k], v) < t, (k, rel(g[k], v))
    g2 = ops.scan_bwd(geo, T, _lib.PRECISION_IEEE, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    for k, v in g.items():
        if v is not None:
            assert torch.equal(v, g2[k]), ("not reproducible", k)


STEP_CASES = [
    # B, H, R, O, G, N, gates, biases, chi, skip, trap, s0
    (2, 3, 1, 1, 64, 128, False, False, False, True, False, True),      # SISO preset head
    (3, 64, 1, 1, 64, 128, False, False, False, True, False, True),
    (2, 4, 4, 4, 16, 128, True, True, True, True, True, True),          # rank-4 head
    (2, 3, 2, 1, 3, 8, False, False, False, True, False, False),
    (1, 2, 2, 3, 4, 8, True, True, True, False, True, True),
    (5, 2, 1, 1, 300, 16, False, False, False, True, False, True),      # more (g, o) pairs than threads
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", STEP_CASES)
def test_scan_step(case, dtype):
    """The one-launch decode step against the fp64 restatement of the scan on the one token (output and state after
    it), and against the chunked scan kernels at L = 1, which it must reproduce to fp32 rounding."""
    B, H, Rk, O, G, N, gates, biases, chi, skip, trap, s0 = case
    c = scan_case(B, 1, H, Rk, O, G, N, dtype, gates, biases, chi, skip, trap, s0, seed=13)
    geo = c["geo"]
    args = (c["u"], c["Bhat"], c["gBp"], c["Chat"], c["gCp"], c["beta"], c["gamma"], c["chi"], c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S = ops.scan_step(geo, *args, c["S0"])
    ry, rS, _, _ = R.scan_fwd(geo, 1, 0, *args, c["S0"])
    assert rel(S, rS) < 2e-6, ("S", rel(S, rS))
    assert rel(y, ry) < (6e-3 if dtype == torch.bfloat16 else 2e-5), ("y", rel(y, ry))
    T = ops.pick_chunk(geo, _lib.PRECISION_IEEE, False, 64)
    if T > 0:
        y2, S2, _, _ = ops.scan_fwd(geo, T, _lib.PRECISION_IEEE, *args, c["S0"])
        assert rel(S, S2) < 2e-6 and rel(y, y2) < (6e-3 if dtype == torch.bfloat16 else 2e-6)
    y3, S3 = ops.scan_step(geo, *args, c["S0"])
    assert torch.equal(y, y3) and torch.equal(S, S3)


@pytest.mark.parametrize("T", [8, 16, 32, 64])
def test_scan_chunk_length_is_scheduling_only(T):
    c = scan_case(2, 100, 2, 1, 1, 16, 32, torch.float32, False, False, False, True, True, True, seed=3)
    args = (c["u"], c["Bhat"], c["gBp"], c["Chat"], c["gCp"], c["beta"], c["gamma"], c["chi"], c["dA"], c["w"], c["wd"], c["Dg"])
    y, S, _, _ = ops.scan_fwd(c["geo"], T, _lib.PRECISION_IEEE, *args, c["S0"])
    ry, rS, _, _ = R.scan_fwd(c["geo"], 100, 0, *args, c["S0"])
    assert rel(y, ry) < 2e-5 and rel(S, rS) < 2e-5


# ---------------------------------------------------------------------------------------------------- tcgen05 tile
@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 6, 8, 10])
@pytest.mark.parametrize("K,N", [(64, 64), (128, 64), (128, 128), (64, 128)])
def test_umma_tile(mode, K, N):
    g = torch.Generator().manual_seed(mode * 100 + K + N)
    A = torch.randn(128, K, generator=g).to(torch.bfloat16)
    Bm = torch.randn(N, K, generator=g).to(torch.bfloat16)
    want = A.float() @ Bm.float().T
    Ad = (A.T.contiguous() if mode & 1 else A).to(DEV)
    Bd = (Bm.T.contiguous() if mode & 2 else Bm).to(DEV)
    D = torch.full((128, N), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = _lib.load()
    import ctypes as C
    _lib.check(lib.orbit_selftest_umma(C.c_void_p(Ad.data_ptr()), C.c_void_p(Bd.data_ptr()), C.c_void_p(D.data_ptr()), mode, K,
                                       N, C.c_void_p(status.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
               "orbit_selftest_umma")
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded device wait gave up"
    assert rel(D, want) < 1e-5, (mode, K, N, rel(D, want))


# ---------------------------------------------------------------------------------------------------- scan, tcgen05
TC_CASES = [
    # B, L, H, skip, trap, s0
    (1, 128, 1, False, False, False),
    (2, 256, 3, True, False, True),
    (1, 200, 2, True, True, True),
    (2, 37, 2, True, False, True),
    (1, 640, 4, True, True, False),
]


@pytest.mark.parametrize("case", TC_CASES)
def test_scan_tc_forward(case):
    """Forward on the tensor-core tiles (bf16 operands, fp32 accumulate) against the fp64 restatement on the same
    bf16-rounded inputs: y within 1e-2 (operands of the second contraction are rounded to bf16: masked scores and
    entering states), final state within 2e-3."""
    B, L, H, skip, trap, s0 = case
    c = scan_case(B, L, H, 1, 1, 64, 128, torch.bfloat16, False, False, False, skip, trap, s0, seed=5)
    geo = c["geo"]
    args = (c["u"], c["Bhat"], None, c["Chat"], None, None, None, None, c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, 128, _lib.PRECISION_IO, *args, c["S0"])
    ops.check_device_status()
    ry, rS, _, _ = R.scan_fwd(geo, 128, 0, *args, c["S0"])
    assert rel(S_fin, rS) < 2e-3, ("S_fin", rel(S_fin, rS))
    assert rel(y, ry) < 1e-2, ("y", rel(y, ry))


@pytest.mark.parametrize("case", TC_CASES)
def test_scan_tc_backward(case):
    """Backward on the tensor-core tiles against the fp64 restatement on the same bf16-rounded inputs.  Every MMA
    operand (scores, masks, scaled drives, states, summed score gradient) is rounded to bfloat16 (eps 3.9e-3) and
    accumulated in fp32, so gradients are held to 2e-2 normwise; results must be bitwise reproducible."""
    B, L, H, skip, trap, s0 = case
    c = scan_case(B, L, H, 1, 1, 64, 128, torch.bfloat16, False, False, False, skip, trap, s0, seed=7)
    geo = c["geo"]
    args = (c["u"], c["Bhat"], None, c["Chat"], None, None, None, None, c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, 128, _lib.PRECISION_IO, *args, c["S0"])
    g = ops.scan_bwd(geo, 128, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    ops.check_device_status()
    rg = R.scan_bwd(geo, 128, 0, *args, None, None, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None, S0=c["S0"])
    errs = {k: rel(g[k], v) for k, v in rg.items() if v is not None}
    bad = {k: e for k, e in errs.items() if not e < 2e-2}
    assert not bad, (bad, errs)
    g2 = ops.scan_bwd(geo, 128, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    for k, v in g.items():
        if v is not None:
            assert torch.equal(v, g2[k]), ("not reproducible", k)
    if H % 2 == 0:
        # head ranges on separate CTAs (partial buffers of the head-shared map gradients summed by the host)
        g3 = ops.scan_bwd(geo, 128, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None,
                          hsplit=2)
        errs3 = {k: rel(g3[k], v) for k, v in rg.items() if v is not None}
        bad3 = {k: e for k, e in errs3.items() if not e < 2e-2}      # each range rounds its own summed score gradient
        assert not bad3, ("head split", bad3)


@pytest.mark.parametrize("scale,H", [(1.0, 8), (30.0, 2), (300.0, 3)])
def test_scan_tc_strong_decay_many_heads(scale, H):
    """Rank-1 tensor-core tiles with steps scaled up (per-chunk decay sums of several hundred: the split decay factors
    exp(cs_t - cs_end) * exp(cs_end - cs_s) underflow to zero where the exact product does, never to inf/nan) and with
    more heads than the staging rings are deep; forward and backward against the fp64 restatement, head ranges split
    over 1, 2 and H CTAs."""
    B, L = 2, 300
    c = scan_case(B, L, H, 1, 1, 64, 128, torch.bfloat16, False, False, False, True, True, True, seed=21)
    c["dA"] = c["dA"] * scale
    geo = c["geo"]
    args = (c["u"], c["Bhat"], None, c["Chat"], None, None, None, None, c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, 128, _lib.PRECISION_IO, *args, c["S0"])
    ops.check_device_status()
    ry, rS, _, _ = R.scan_fwd(geo, 128, 0, *args, c["S0"])
    assert torch.isfinite(y.float()).all() and torch.isfinite(S_fin).all()
    assert rel(S_fin, rS) < 2e-3 and rel(y, ry) < 1e-2, (rel(S_fin, rS), rel(y, ry))
    rg = R.scan_bwd(geo, 128, 0, *args, None, None, c["dy"], c["dS_fin"], c["euler"], True, S0=c["S0"])
    for k in sorted({1, 2 if H % 2 == 0 else 1, H}):
        g = ops.scan_bwd(geo, 128, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], True, hsplit=k)
        ops.check_device_status()
        for name, v in rg.items():
            if v is not None:
                assert torch.isfinite(g[name].float()).all(), (k, name)
                assert rel(g[name], v) < 2e-2, ("hsplit", k, name, rel(g[name], v))


# ---------------------------------------------------------------------------------------------------- scan, tcgen05 rank 4
MIMO_CASES = [
    # B, L, H, gates, biases, chi, skip, trap, s0
    (1, 32, 1, False, False, False, False, False, False),
    (1, 64, 2, False, True, False, True, False, True),
    (2, 96, 2, True, False, True, True, True, False),
    (1, 77, 3, True, True, True, True, True, True),
    (2, 37, 2, True, True, True, True, False, True),
]


@pytest.mark.parametrize("case", MIMO_CASES)
def test_scan_tc_mimo_forward(case):
    """Forward on the rank-4 tensor-core tiles (R = O = 4, G = 16, N = 128, chunk 32) against the fp64 restatement on
    the same bf16-rounded inputs.  Operand tiles (gate x map + bias, masked scores, entering states) are rounded to
    bfloat16 and accumulated in fp32: y within 1e-2, final state within 4e-3."""
    B, L, H, gates, biases, chi, skip, trap, s0 = case
    c = scan_case(B, L, H, 4, 4, 16, 128, torch.bfloat16, gates, biases, chi, skip, trap, s0, seed=11)
    geo = c["geo"]
    assert ops.pick_chunk(geo, _lib.PRECISION_IO, False, 64) == 32
    args = (c["u"], c["Bhat"], c["gBp"], c["Chat"], c["gCp"], c["beta"], c["gamma"], c["chi"], c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, 32, _lib.PRECISION_IO, *args, c["S0"])
    ops.check_device_status()
    ry, rS, _, _ = R.scan_fwd(geo, 32, 0, *args, c["S0"])
    assert rel(S_fin, rS) < 4e-3, ("S_fin", rel(S_fin, rS))
    assert rel(y, ry) < 1e-2, ("y", rel(y, ry))
    y2, S2, _, _ = ops.scan_fwd(geo, 32, _lib.PRECISION_IO, *args, c["S0"])
    assert torch.equal(y, y2) and torch.equal(S_fin, S2)


@pytest.mark.parametrize("case", MIMO_CASES)
def test_scan_tc_mimo_backward(case):
    """Backward on the rank-4 tensor-core tiles against the fp64 restatement on the same bf16-rounded inputs: every MMA
    operand is rounded to bfloat16 and accumulated in fp32, gradients are held to 2e-2 normwise and must be bitwise
    reproducible."""
    B, L, H, gates, biases, chi, skip, trap, s0 = case
    c = scan_case(B, L, H, 4, 4, 16, 128, torch.bfloat16, gates, biases, chi, skip, trap, s0, seed=13)
    geo = c["geo"]
    assert ops.pick_chunk(geo, _lib.PRECISION_IO, True, 64) == 32
    args = (c["u"], c["Bhat"], c["gBp"], c["Chat"], c["gCp"], c["beta"], c["gamma"], c["chi"], c["dA"], c["w"],
            c["w"] if c["euler"] else c["wd"], c["Dg"])
    y, S_fin, Sin, atot = ops.scan_fwd(geo, 32, _lib.PRECISION_IO, *args, c["S0"])
    g = ops.scan_bwd(geo, 32, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    ops.check_device_status()
    rg = R.scan_bwd(geo, 32, 0, *args, None, None, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None, S0=c["S0"])
    errs = {k: rel(g[k], v) for k, v in rg.items() if v is not None}
    bad = {k: e for k, e in errs.items() if not e < 2e-2}
    assert not bad, (bad, errs)
    g2 = ops.scan_bwd(geo, 32, _lib.PRECISION_IO, *args, Sin, atot, c["dy"], c["dS_fin"], c["euler"], c["S0"] is not None)
    for k, v in g.items():
        if v is not None:
            assert torch.equal(v, g2[k]), ("not reproducible", k)


# ---------------------------------------------------------------------------------------------------- HybridMamba scan
def hm_case(B, L, H, P, N, nrot, trap, carries, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)

    def rn(*s, scale=1.0):
        return torch.randn(*s, generator=g) * scale

    K = N // 2
    c = {}
    c["x"] = rn(B, L, H, P).to(dtype).to(DEV)
    c["delta"] = torch.nn.functional.softplus(rn(B, L, H) - 2.0).to(DEV)
    c["A_log"] = torch.log(1 + 15 * torch.rand(H, P, N, generator=g)).to(DEV)
    if nrot:                                              # rotating pairs share one modulus
        A = c["A_log"].clone()
        A[..., N - 2 * nrot + 1::2] = A[..., N - 2 * nrot::2]
        c["A_log"] = A
    c["Bh"], c["Ch"] = rn(B, L, N).to(DEV), rn(B, L, N).to(DEV)
    c["beta_b"], c["beta_c"] = rn(H, N, scale=0.3).to(DEV), rn(H, N, scale=0.3).to(DEV)
    rot = torch.zeros(K, dtype=torch.uint8)
    rot[K - nrot:] = 1
    c["rot"] = rot.to(DEV) if nrot else None
    c["feat"] = (rn(B, L, K, scale=2.0) * rot).to(DEV) if nrot else None
    c["theta_h"] = (rn(H, K, scale=0.5) * rot).to(DEV) if nrot else None
    c["lam"] = torch.sigmoid(rn(B, L, H)).to(DEV) if trap else None
    c["D"] = (1 + rn(H, scale=0.3)).to(DEV)
    c["h_init"] = rn(B, H, P, N).to(DEV) if carries else None
    c["write_prev"] = rn(B, H, P, N).to(DEV) if (carries and trap) else None
    c["theta_init"] = (rn(B, H, K) * rot).to(DEV) if (carries and nrot) else None
    c["dy"] = rn(B, L, H, P).to(dtype).to(DEV)
    c["dh_final"] = rn(B, H, P, N).to(DEV)
    c["dtheta_final"] = (rn(B, H, K) * rot).to(DEV) if nrot else None
    c["dwrite_last"] = rn(B, H, P, N).to(DEV)
    return c


HM_CASES = [
    # B, L, H, P, N, rotating pairs, trapezoid, carries
    (2, 40, 3, 16, 16, 4, True, True),
    (1, 77, 2, 64, 64, 16, True, True),
    (2, 19, 2, 8, 8, 0, False, False),
    (1, 100, 2, 32, 128, 64, True, False),
    (1, 33, 1, 64, 64, 0, True, True),
]
HM_ARGS = ("x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "rot", "theta_h", "lam", "D", "h_init", "write_prev",
           "theta_init")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", HM_CASES)
def test_hm_scan(dtype, case):
    """Coordinate-decay scan kernels against the fp64 token loop on the same (dtype-rounded) inputs: outputs and carries
    within 2e-4 (fp32) / the bf16 output rounding, every gradient within 5e-3 (fp32 arithmetic, fast exp), results
    bitwise reproducible."""
    c = hm_case(*case, dtype)
    args = [c[k] for k in HM_ARGS]
    y, hN, thN, wl, saved = ops.hm_scan_fwd(*args)
    ry, rh, rth, rwl = R.hm_scan_fwd(*args)
    assert rel(y, ry) < (6e-3 if dtype == torch.bfloat16 else 2e-4), ("y", rel(y, ry))
    assert rel(hN, rh) < 2e-4 and rel(wl, rwl) < 1e-5, (rel(hN, rh), rel(wl, rwl))
    if thN is not None:
        assert rel(thN, rth) < 1e-5
    seeds = (c["dy"], c["dh_final"], c["dtheta_final"], c["dwrite_last"])
    g = ops.hm_scan_bwd(*args, saved, *seeds)
    rg = R.hm_scan_bwd(*args, *seeds)
    errs = {k: rel(g[k], v) for k, v in rg.items() if v is not None and g.get(k) is not None}
    bad = {k: e for k, e in errs.items() if not e < (8e-3 if (k == "x" and dtype == torch.bfloat16) else 5e-3)}
    assert not bad, (bad, errs)
    g2 = ops.hm_scan_bwd(*args, saved, *seeds)
    for k, v in g.items():
        if v is not None:
            assert torch.equal(v, g2[k]), ("not reproducible", k)


# ---------------------------------------------------------------------------------------------------- token tails
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,X,N,norm,bias,add", [(2, 37, 4, 128, True, False, 0.0), (1, 5, 1, 16, True, True, 0.0),
                                                   (3, 19, 2, 8, False, False, 1.0), (2, 64, 4, 128, False, False, 1.0),
                                                   (1, 9, 3, 200, True, True, 0.0)])
def test_token_map(dtype, B, L, X, N, norm, bias, add):
    g = torch.Generator().manual_seed(B * 100 + L)
    slab = torch.randn(B, L, N * X + 24, generator=g).to(dtype).to(DEV)       # the map reads a column range of a wider slab
    src = slab[..., 8:8 + N * X]
    w = (1 + 0.3 * torch.randn(N, generator=g)).to(DEV) if norm else None
    b = (0.2 * torch.randn(N, generator=g)).to(DEV) if bias else None
    out, rstd = ops.token_map_fwd(src, w, b, add, 1e-5, X, N)
    rout, rr = R.token_map_fwd(src, w, b, add, 1e-5, X, N)
    assert rel(out, rout) < tol(dtype)
    if norm:
        assert rel(rstd, rr) < 1e-5
    dout = torch.randn(B, L, X, N, generator=g).to(dtype).to(DEV)
    dslab = torch.full_like(slab, float("nan"))
    dsrc, dw, db = ops.token_map_bwd(src, w, rstd, dout, X, N, bias, dsrc_out=dslab[..., 8:8 + N * X])
    rd, rw, rb = R.token_map_bwd(src, w, rstd, dout, X, N, bias)
    assert dsrc.data_ptr() == dslab[..., 8:8 + N * X].data_ptr()
    assert rel(dsrc, rd) < tol(dtype, True)
    assert torch.isnan(dslab[..., :8]).all() and torch.isnan(dslab[..., 8 + N * X:]).all()      # nothing written outside the range
    if norm:
        assert rel(dw, rw) < 2e-4 if dtype == torch.float32 else rel(dw, rw) < 6e-3
    if bias:
        assert rel(db, rb) < 2e-5
    d2, w2, b2 = ops.token_map_bwd(src, w, rstd, dout, X, N, bias)
    assert torch.equal(d2, dsrc) and (dw is None or torch.equal(dw, w2)) and (db is None or torch.equal(db, b2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("a_act,per_sib,trap,rmix", [(0, False, False, False), (0, False, True, True), (1, False, True, True),
                                                     (1, True, False, True), (2, True, True, False)])
@pytest.mark.parametrize("B,L,H,Rr", [(2, 23, 3, 2), (3, 700, 64, 1), (2, 257, 24, 4)])
def test_token_clock(dtype, a_act, per_sib, trap, rmix, B, L, H, Rr):
    import ctypes as C
    g = torch.Generator().manual_seed(a_act * 10 + trap)
    HR = H * Rr
    slab = torch.randn(B, L, 4 * HR + 16, generator=g).to(dtype).to(DEV)
    dt_raw = slab[..., 0:HR]
    a_raw = (slab[..., HR + 2:HR + 2 + (HR if per_sib else H)] * 2.0) if a_act else None
    if a_raw is not None:
        a_raw = a_raw.contiguous()
    trap_raw = slab[..., 2 * HR + 4:2 * HR + 4 + H] if trap else None
    rmix_raw = slab[..., 3 * HR + 8:3 * HR + 8 + HR] if rmix else None
    A_log = torch.randn(H, Rr, generator=g).to(DEV) if a_act == 0 else None
    r_mix = torch.randn(H, Rr, generator=g).to(DEV) if rmix else None
    o = ops.token_clock_fwd(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, per_sib, H, Rr)
    t = dict(dt_raw=dt_raw, a_raw=a_raw, trap_raw=trap_raw, rmix_raw=rmix_raw, A_log=A_log, r_mix=r_mix, a_act=a_act,
             a_per_sibling=per_sib, H=H, R=Rr)
    ro, _ = R._clock(t, torch.float64)
    for k in ("dA", "w", "wd", "chi", "lag0"):
        if ro[k] is None:
            assert o[k] is None, k
        else:
            assert rel(o[k], ro[k]) < 2e-6, (k, rel(o[k], ro[k]))
    gr = {k: torch.randn(B, L, H, Rr, generator=g).to(DEV) for k in ("ddA", "dw", "dwd", "dchi")}
    gr["dlag0"] = torch.randn(B, H, Rr, generator=g).to(DEV)
    got = ops.token_clock_bwd(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, per_sib, H, Rr, gr, bias_sums=True)
    with torch.enable_grad():
        ro, leaves = R._clock(t, torch.float64, leaves=True)
        loss = sum((ro[k] * gr["d" + k].double()).sum() for k in ("dA", "w", "wd", "chi", "lag0") if ro[k] is not None)
        live = [k for k, v in leaves.items() if v is not None]
        want = dict(zip(live, torch.autograd.grad(loss, [leaves[k] for k in live], allow_unused=True)))
    for k, v in want.items():
        if v is None:
            continue
        lim = 2e-5 if (dtype == torch.float32 or k in ("A_log", "r_mix")) else 6e-3
        assert rel(got[k].reshape(v.shape), v) < lim, (k, rel(got[k].reshape(v.shape), v))
    # gradients of the slab biases: column sums of the raw gradients taken BEFORE the rounding to the IO dtype, so fp32-exact
    # for bf16 activations too; fixed-order two-stage reduction: bitwise reproducible
    for key, raw in (("dt_bias", "dt_raw"), ("a_bias", "a_raw"), ("trap_bias", "trap_raw")):
        if want.get(raw) is None:
            assert got.get(key) is None, key
            continue
        ref = want[raw].reshape(-1, want[raw].shape[-1]).sum(0)
        assert rel(got[key], ref) < 2e-5, (key, rel(got[key], ref))
    again = ops.token_clock_bwd(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, per_sib, H, Rr, gr, bias_sums=True)
    assert torch.equal(again["dt_bias"], got["dt_bias"])


def test_bounded_wait_winds_down_and_reports():
    """A device-side wait that runs out: the kernel sets the status word, frees its tensor memory and returns; the host
    maps the word to ORBIT_ERR_DEVICE_TIMEOUT, and the next tensor-core launch works (nothing faulted, nothing leaked)."""
    lib = _lib.load()
    status = ops._status_word(torch.device(DEV, torch.cuda.current_device()))
    status.zero_()
    _lib.check(lib.orbit_selftest_wait_timeout(C.c_void_p(status.data_ptr()), 200, C.c_void_p(torch.cuda.current_stream().cuda_stream)),
               "orbit_selftest_wait_timeout")
    with pytest.raises(RuntimeError, match="ORBIT_ERR_DEVICE_TIMEOUT"):
        ops.check_device_status()
    assert int(status.item()) == 0                                   # the check clears the word
    ops.check_device_status()
    test_umma_tile(0, 128, 128)
    # the layer's opt-in check: with `check_waits` a forward whose launches left the word set raises instead of returning
    from orbitssm_b200 import SSDMimoSSM, mamba2_config
    layer = SSDMimoSSM(mamba2_config(128, d_state=128, d_head=64), execution={"precision": "io"}).to(DEV)
    layer.check_waits = True
    x = torch.randn(1, 130, 128, device=DEV, dtype=torch.bfloat16)
    layer(x)                                                         # clean run: nothing to report
    _lib.check(lib.orbit_selftest_wait_timeout(C.c_void_p(status.data_ptr()), 200, C.c_void_p(torch.cuda.current_stream().cuda_stream)),
               "orbit_selftest_wait_timeout")
    with pytest.raises(RuntimeError, match="ORBIT_ERR_DEVICE_TIMEOUT"):
        layer(x)
    layer(x)                                      # tensor memory was freed: a tile runs right after
