"""CPU restatement of the reference's HybridMamba layer (TEST INFRASTRUCTURE, not product code).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this module; the
package never does.  It restates, in plain torch ops (fp64 in -> fp64 throughout, anything else -> fp32 law
arithmetic), what the reference's ``backend="torch"`` route computes for one `HybridMambaSSM` call on the
coordinate-decay rows (``coord_static`` real rows and ``coord_static`` rotating pairs), from a parameter dict keyed
by the reference's ``state_dict`` names.  Token-major tensors throughout ([B, L, ...]).

Pinned: ``tests/test_oracle_golden.py`` checks it against vectors produced by running the reference itself
(``tests/golden/make_golden_hm.py``): outputs, carried state (hidden_state, theta, write_prev, conv_state) and all
gradients, including a continuation segment.

Reference lines followed (paths inside the reference project):
  * input GEMM, drive conv, epilogue:   src/orbit_ssm/ssm/hybrid_mamba.py:2729-2794, 2844-2852
  * token slab order and split:         src/orbit_ssm/ssm/hybrid_mamba.py:1609-1660
  * maps (clock, B/C norms, angle):     src/orbit_ssm/ssm/hybrid_mamba.py:1695-1740, 1950-2013, 971-1011
  * row layout (pair-tied stores):      src/orbit_ssm/ssm/hybrid_mamba.py:696-735, 1196-1199
  * the recurrence:                     src/orbit_ssm/kernels/hybrid_mamba_mh/torch_scan.py:44-76, 180-279
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from .ssd_oracle import causal_conv_silu, law_dtype, _rms


def hm_plan(cfg: dict) -> SimpleNamespace:
    """Row plan of a coordinate-decay config: which of the N state rows rotate, the pair-tied row gather."""
    d_model = cfg["d_model"]
    d_inner = cfg.get("d_inner") or int(round(cfg.get("expand", 2) * d_model))
    N = cfg.get("d_state", 64)
    P = cfg.get("d_head") or (d_inner // cfg["n_heads"] if cfg.get("n_heads") else 64)
    H = d_inner // P
    rot, used = [], 0
    blocks = cfg["row_blocks"]
    for i, blk in enumerate(blocks):
        rows = N - used if i == len(blocks) - 1 else int(round(blk["frac"] * N))
        rot += [bool(blk.get("complex", False))] * rows
        used += rows
    rep = [n - 1 if (rot[n] and n % 2) else n for n in range(N)]
    store = [n for n in range(N) if rep[n] == n]
    col = {n: i for i, n in enumerate(store)}
    a_idx = [col[rep[n]] for n in range(N)]
    pairs = [k for k in range(N // 2) if rot[2 * k]] if any(rot) else []
    rule = cfg.get("write_rule")
    return SimpleNamespace(d_model=d_model, d_inner=d_inner, N=N, P=P, H=H, rot=rot, a_idx=a_idx, rot_pairs=pairs,
                           K=N // 2, trap=(rule is None or rule == "trapezoid"), d_conv=cfg.get("d_conv", 4),
                           out_norm=bool(cfg.get("out_norm", False)), eps=cfg.get("norm_eps", 1e-5))


def _rotate(v, ang):
    """Rotate interleaved pairs (2k, 2k+1) of the last axis of v [..., N] by ang [..., N/2]
    (reference: torch_scan.py:44-48)."""
    a, b = v[..., 0::2], v[..., 1::2]
    c, s = ang.cos(), ang.sin()
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


def hm_scan(x, delta, A_log, Bh, Ch, *, beta_b=None, beta_c=None, feat=None, rot_rows=None, theta_h=None, lam=None,
            D=None, h_init=None, write_prev=None, theta_init=None):
    """The coordinate-decay recurrence, one token at a time (reference: torch_scan.py:51-76, 180-279).

    x [B,L,H,P], delta [B,L,H] (after softplus), A_log [H,P,N] (kernel rows), Bh/Ch [B,L,N] (normed maps),
    beta_b/beta_c [H,N], feat [B,L,K] angle features on the K = N/2 pair axis (zero on real pairs), rot_rows [N] bool,
    theta_h [H,K] read offset in the scan's frame, lam [B,L,H] trapezoid weights or None (Euler), D [H].
    Returns y [B,L,H,P], h_final [B,H,P,N], theta_final [B,H,K] (None without rotation), write_last [B,H,P,N]."""
    f = law_dtype(x)
    Bsz, L, H, P = x.shape
    N = A_log.shape[-1]
    xf, dt = x.to(f), delta.to(f)
    rate = -(A_log.to(f)).exp()                                             # c1 [H,P,N]
    h = xf.new_zeros(Bsz, H, P, N) if h_init is None else h_init.to(f)
    prev = xf.new_zeros(Bsz, H, P, N) if write_prev is None else write_prev.to(f)
    th = None
    if feat is not None:
        th = xf.new_zeros(Bsz, H, N // 2) if theta_init is None else theta_init.to(f)
        mask = torch.as_tensor(rot_rows, device=x.device)
    ys = []
    for t in range(L):
        w = Bh[:, t].to(f)[:, None].expand(Bsz, H, N)
        r = Ch[:, t].to(f)[:, None].expand(Bsz, H, N)
        if beta_b is not None:
            w = w + beta_b.to(f)[None]
        if beta_c is not None:
            r = r + beta_c.to(f)[None]
        if feat is not None:
            th = th + dt[:, t][:, :, None] * feat[:, t].to(f)[:, None]     # [B,H,K]
            w = torch.where(mask, _rotate(w, th), w)
            r = torch.where(mask, _rotate(r, th if theta_h is None else th + theta_h.to(f)[None]), r)
        a = (rate[None] * dt[:, t][:, :, None, None]).exp()                 # [B,H,P,N]
        raw = xf[:, t][..., None] * w[:, :, None]
        d = dt[:, t][:, :, None, None]
        if lam is None:
            drive = d * raw
        else:
            lm = lam[:, t].to(f)[:, :, None, None]
            drive = d * (lm * raw + (1 - lm) * a * prev)
        h = a * h + drive
        prev = raw
        ys.append((h * r[:, :, None]).sum(-1))
    y = torch.stack(ys, 1)                                                  # [B,L,H,P]
    if D is not None:
        y = y + D.to(f)[None, None, :, None] * xf
    return y, h, th, prev


def hm_layer(cfg: dict, prm: dict, x, state=None, return_state=False):
    """One `HybridMambaSSM` call (reference: hybrid_mamba.py:2729-2852).  ``prm``: the reference's state_dict."""
    pl = hm_plan(cfg)
    f = law_dtype(x)
    Bsz, L, _ = x.shape
    H, P, N, K = pl.H, pl.P, pl.N, pl.K
    g = lambda k: prm[k].to(x.dtype) if k in prm else None
    xz = F.linear(x, g("in_proj.weight"))
    xd, z = xz[..., :pl.d_inner], xz[..., pl.d_inner:]
    new_state = {}
    if pl.d_conv > 0:
        win = None if state is None else state["conv_state"]
        xd, win = causal_conv_silu(xd, g("conv1d.weight"), g("conv1d.bias"), win)
        new_state["conv_state"] = win
    # token maps, all read from the layer input
    dt_lin = F.linear(x, g("dt_low.weight")) if "dt_low.weight" in prm else x
    dt_lin = F.linear(dt_lin, g("dt_proj.weight"))
    delta = F.softplus(dt_lin.to(f) + prm["dt_bias"].to(f))                 # [B,L,H]
    bc = F.linear(x, g("bc_proj.weight")).to(f)
    Bh, Ch = bc[..., :N], bc[..., N:]
    if "b_norm.weight" in prm:
        Bh = _rms(Bh, prm["b_norm.weight"].to(f), pl.eps)
    if "c_norm.weight" in prm:
        Ch = _rms(Ch, prm["c_norm.weight"].to(f), pl.eps)
    feat = th_h = th0 = None
    if pl.rot_pairs:
        idx = torch.tensor(pl.rot_pairs, device=x.device)
        q = F.linear(x, g("theta_proj.weight")).to(f)                       # [B,L,n_rot]
        om = (math.pi * torch.tanh(prm["theta_freq"].to(f)) if "theta_freq" in prm
              else torch.full((len(pl.rot_pairs),), math.pi, dtype=f, device=x.device))
        feat = q.new_zeros(Bsz, L, K).index_copy(-1, idx, om * torch.tanh(q))
        if "theta_h" in prm:
            th_h = q.new_zeros(H, K).index_copy(-1, idx, -prm["theta_h"].to(f))
        if state is not None:
            th0 = q.new_zeros(Bsz, H, K).index_copy(-1, idx, state["theta"].to(f))
    lam = None
    if pl.trap:
        lam = torch.sigmoid(F.linear(x, g("trap_proj.weight"), g("trap_proj.bias")).to(f))
    A_log = prm["A_log"].to(f)[..., torch.tensor(pl.a_idx, device=x.device)]
    y, hN, thN, wl = hm_scan(
        xd.reshape(Bsz, L, H, P), delta, A_log, Bh, Ch, beta_b=prm.get("beta_b"), beta_c=prm.get("beta_c"), feat=feat,
        rot_rows=pl.rot, theta_h=th_h, lam=lam, D=prm.get("D"),
        h_init=None if state is None else state["hidden_state"],
        write_prev=None if (state is None or not pl.trap) else state["write_prev"], theta_init=th0)
    y = y.reshape(Bsz, L, pl.d_inner)
    yg = y * F.silu(z.to(f))
    if pl.out_norm:
        yg = _rms(yg, prm["norm.weight"].to(f), pl.eps)
    out = F.linear(yg.to(x.dtype), g("out_proj.weight"))
    if not return_state:
        return out
    new_state["hidden_state"] = hN
    if pl.rot_pairs:
        new_state["theta"] = thN[..., torch.tensor(pl.rot_pairs, device=x.device)]
    if pl.trap:
        new_state["write_prev"] = wl
    return out, new_state
