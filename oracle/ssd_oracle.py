"""CPU restatement of the reference's SSD-MIMO layer (TEST INFRASTRUCTURE, not product code).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this
module; the package never does.  It restates, in plain torch ops on whatever device/dtype the inputs have
(fp64 in -> fp64 throughout, anything else -> fp32 law arithmetic), what the reference's ``backend="torch"``
route computes for one `SSDMimoSSM` call, from a parameter dict keyed by the reference's ``state_dict`` names.

Pinned: ``tests/test_oracle_golden.py`` checks every function here against vectors produced by running the
reference itself (``tests/golden/make_golden.py``), outputs, carried state and all gradients.

Reference lines followed (paths inside the reference project):
  * input GEMM, drive conv, gate, output norm, out_proj: src/orbit_ssm/ssm/ssd_mimo.py:4541-4593, 4509-4539
  * B|C conv with its carried window:                    src/orbit_ssm/ssm/ssd_mimo_torch.py:122-145
  * per-token law (maps, clocks, rates, weights):        src/orbit_ssm/ssm/ssd_mimo_torch.py:161-267
  * chunked dual:                                        src/orbit_ssm/ssm/ssd_mimo_torch.py:663-708, 750-795
  * token recurrence:                                    src/orbit_ssm/ssm/ssd_mimo_torch.py:314-385, 845-888
  * skip, gate, carries:                                 src/orbit_ssm/ssm/ssd_mimo_torch.py:600-643
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def law_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.float64 if x.dtype == torch.float64 else torch.float32


# ----------------------------------------------------------------------------------------------------
#  depthwise causal conv + SiLU (drive conv and B|C conv share it)
# ----------------------------------------------------------------------------------------------------
def causal_conv_silu(x, weight, bias, window=None):
    """x [B, L, C] token-major raw inputs, weight [C, 1, W] or [C, W], bias [C], ``window`` [B, C, W] the last W
    raw inputs before this call (None = zeros).  Returns (silu(conv) [B, L, C], new window [B, C, W]).

    y[b,t,c] = silu(bias[c] + sum_j w[c,j] * xin[b, t - (W-1) + j, c])   (reference: layers/conv.py:280-328,
    ssd_mimo.py:4561-4592 for the window convention: index -1 newest, the non-oldest W-1 slots prefix the call).
    """
    Bsz, L, C = x.shape
    w = weight.reshape(C, -1).to(x.dtype)
    W = w.shape[1]
    if window is None:
        window = x.new_zeros(Bsz, C, W)
    full = torch.cat([window.to(x.dtype).transpose(1, 2), x], dim=1)           # [B, W+L, C]
    acc = bias.to(x.dtype).expand(Bsz, L, C)
    for j in range(W):
        acc = acc + full[:, j + 1: j + 1 + L] * w[:, j]
    return F.silu(acc), full[:, -W:].transpose(1, 2)


def _rms(x, weight, eps):
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * weight


def _pass_min(x, lo):      # clamp_min whose gradient passes at the boundary (reference: ssd_mimo.py:292-297)
    return torch.where(x >= lo, x, x.clamp_min(lo).detach())


def _pass_max(x, hi):
    return torch.where(x <= hi, x, x.clamp_max(hi).detach())


def rate_heavy_tail(v, floor=1e-4):
    """|a| = max(ht(v), floor), ht(v) = 1 + v (v >= 0), 1 / (1 - v) (v < 0)  (reference: ssd_mimo.py:300-304)."""
    return _pass_min(_pass_min(v, 0.0) + torch.reciprocal(1.0 - _pass_max(v, 0.0)), floor)


def rate_softplus(v, floor=1e-4):
    return _pass_min(F.softplus(v), floor)


def skip_gains(spec, D):
    """Logical [H, G, R, O] skip gains (reference: ssd_mimo.py:2872-2878)."""
    H, G, R, O = spec.H, spec.G, spec.R, spec.O
    if spec.skip_sharing == "head":
        return D[:, None, None, None].expand(H, G, R, O)
    if spec.skip_sharing == "channel":
        return D[..., None].expand(H, G, R, O)
    return D


# ----------------------------------------------------------------------------------------------------
#  per-token law
# ----------------------------------------------------------------------------------------------------
def token_law(spec, prm, slab, b_src, c_src, f):
    """Everything the scan needs per token, from the fused slab [B, L, tok_width] and the (convolved) raw
    B / C columns (column index n*R + q / n*O + o).

    Returns dict: Bbar [B,L,H|1,R|1,Q,N], Cbar [B,L,H|1,R|1,O,N], dt, dA [B,L,H,R], lam [B,L,H] | None,
    chi [(B,L,)H,R] | None.   (reference: ssd_mimo_torch.py:161-267)
    """
    Bsz, L = slab.shape[:2]
    H, R, O, N = spec.H, spec.R, spec.O, spec.N

    def part(key):
        o, wd = spec.slab_off[key]
        return slab[..., o:o + wd].to(f)

    Bm = b_src.to(f).reshape(Bsz, L, N, R).transpose(-1, -2)                   # [B,L,q,n]
    Cm = c_src.to(f).reshape(Bsz, L, N, O).transpose(-1, -2)                   # [B,L,o,n]
    if spec.b_norm:
        Bm = _rms(Bm, prm["B_norm.weight"].to(f), spec.map_eps)
    if spec.c_norm:
        Cm = _rms(Cm, prm["C_norm.weight"].to(f), spec.map_eps)
    if spec.bc_bias and not spec.head_bias:                                    # shared bias: before the gates
        Bm = Bm + prm["B_bias"].to(f)
        Cm = Cm + prm["C_bias"].to(f)
    if spec.use_g_b:                                                           # sibling r's gate scales all q
        gB = 1.0 + part("gB").reshape(Bsz, L, N, R).transpose(-1, -2)          # [B,L,r,n]
        Bbar = gB[:, :, None, :, None, :] * Bm[:, :, None, None, :, :]         # [B,L,1,r,q,n]
    else:
        Bbar = Bm[:, :, None, None, :, :]
    if spec.use_g_c:
        Cm = Cm * (1.0 + part("gC").reshape(Bsz, L, N, O).transpose(-1, -2))
    Cbar = Cm[:, :, None, None, :, :]
    if spec.head_bias:                                                         # per-(h,r) bias, after the gate
        Bbar = Bbar + prm["B_bias"].to(f).transpose(-1, -2)                    # [H,R,q,N]
        Cbar = Cbar + prm["C_bias"].to(f).transpose(-1, -2)

    dt = F.softplus(part("dt")).reshape(Bsz, L, H, R)
    if spec.a_dyn:
        va = part("a")
        mag = rate_heavy_tail(va) if spec.a_act == "heavy_tail" else rate_softplus(va)
        rate = mag.reshape(Bsz, L, H, R) if spec.a_dyn_per_sibling else mag.reshape(Bsz, L, H, 1)
    else:
        rate = prm["A_log"].to(f).exp()
    dA = -(dt * rate)
    lam = torch.sigmoid(part("trap")) if spec.use_trap else None
    chi = None
    if spec.r_mix_mode != "none":
        chi = prm["r_mix"].to(f)
        if spec.r_mix_dyn:
            chi = chi + part("rmix").reshape(Bsz, L, H, R)
    return dict(Bbar=Bbar, Cbar=Cbar, dt=dt, dA=dA, lam=lam, chi=chi)


# ----------------------------------------------------------------------------------------------------
#  scans
# ----------------------------------------------------------------------------------------------------
def scan_recurrent(Bt, Cq, u, dt, dA, lam, f0, v_prev):
    """The defining token recurrence in folded coordinates (reference: ssd_mimo_torch.py:345-370).

    Bt [B,L,H,R,Q,N], Cq [B,L,H,R,O,N] (chi folded in), u [B,L,H,G,Q], dt/dA [B,L,H,R], lam [B,L,H] | None,
    f0, v_prev [B,H,G,R,N] | None.   Returns y [B,L,H,G,O], f_last, v_last.
    """
    Bsz, L, H, R, Q, N = Bt.shape
    G = u.shape[3]
    f = f0 if f0 is not None else u.new_zeros(Bsz, H, G, R, N)
    vp = v_prev if v_prev is not None else u.new_zeros(Bsz, H, G, R, N)
    ys = []
    v = vp
    for t in range(L):
        v = torch.einsum("bhgq,bhrqn->bhgrn", u[:, t], Bt[:, t])
        a = dA[:, t].exp()[:, :, None, :, None]
        d = dt[:, t][:, :, None, :, None]
        if lam is not None:
            l = lam[:, t][:, :, None, None, None]
            f = a * (f + d * (1.0 - l) * vp) + d * l * v
        else:
            f = a * f + d * v
        vp = v
        ys.append(torch.einsum("bhgrn,bhron->bhgo", f, Cq[:, t]))
    y = torch.stack(ys, dim=1) if ys else u.new_zeros(Bsz, 0, H, G, Cq.shape[4])
    return y, f, v


def scan_chunked(Bt, Cq, u, dA, w, wd, S0, T):
    """Chunked dual with collapsed one-tap weights (reference: ssd_mimo_torch.py:663-708).

    Same operands as `scan_recurrent`; ``w`` / ``wd`` [B,L,H,R] are the off-diagonal / own-token write weights,
    ``S0`` [B,H,R,N,G] | None the collapsed entering state.  Returns y [B,L,H,G,O] and the final state [B,H,R,N,G].
    """
    Bsz, L, H, R, Q, N = Bt.shape
    O, G = Cq.shape[4], u.shape[3]
    nc = -(-L // T)
    pad = nc * T - L

    def ch(t):
        if pad:
            t = torch.cat([t, t.new_zeros(Bsz, pad, *t.shape[2:])], dim=1)
        return t.reshape(Bsz, nc, T, *t.shape[2:])

    Bc, Cc, uc, dAc, wc, wdc = (ch(t) for t in (Bt, Cq, u, dA, w, wd))
    cs = torch.cumsum(dAc, dim=2)                                              # [B,nc,T,H,R]
    tri = torch.ones(T, T, dtype=torch.bool, device=u.device).tril(-1)         # s < t
    # exp of a difference taken first; every admitted exponent is <= 0
    diff = (cs[:, :, :, None] - cs[:, :, None, :]).masked_fill(~tri[None, None, :, :, None, None], float("-inf"))
    Wm = torch.exp(diff) * wc[:, :, None, :]                                   # [B,nc,t,s,H,R]
    eye = torch.eye(T, dtype=torch.bool, device=u.device)[None, None, :, :, None, None]
    Wm = torch.where(eye, wdc[:, :, :, None], Wm)                              # own-token weight ASSIGNED
    score = torch.einsum("bcthron,bcshrqn->bchrotqs", Cc, Bc)
    M = (score * Wm.permute(0, 1, 4, 5, 2, 3)[:, :, :, :, None, :, None, :]).sum(3)   # [B,nc,H,o,t,q,s]
    y = torch.einsum("bchotqs,bcshgq->bcthgo", M, uc)
    dend = torch.exp(cs[:, :, -1:, :, :] - cs) * wc                            # [B,nc,T,H,R]
    Z = torch.einsum("bcshrqn,bcshr,bcshgq->bchrng", Bc, dend, uc)
    S = S0 if S0 is not None else u.new_zeros(Bsz, H, R, N, G)
    enter = []
    tot = cs[:, :, -1].exp()                                                   # [B,nc,H,R]
    for c in range(nc):
        enter.append(S)
        S = tot[:, c][:, :, :, None, None] * S + Z[:, c]
    Sin = torch.stack(enter, dim=1)                                            # [B,nc,H,R,N,G]
    y = y + torch.einsum("bcthron,bchrng,bcthr->bcthgo", Cc, Sin, cs.exp())
    return y.reshape(Bsz, nc * T, H, G, O)[:, :L], S


# ----------------------------------------------------------------------------------------------------
#  the layer
# ----------------------------------------------------------------------------------------------------
def ssd_layer(spec, prm, x, state=None, return_state=False, route="chunked", chunk=None):
    """One `SSDMimoSSM` call: x [B, L, d_model] -> y [B, L, d_model] (and the carried state dict).

    ``prm``: tensors under the reference's state_dict names.  ``state``: dict with the config's carries
    (hidden_state [B,H,P,N] with P index g*R+r, write_prev, bc_conv_state [B,NR+NO,W], conv_state [B,d_inner,W]).
    """
    f = law_dtype(x)
    Bsz, L, _ = x.shape
    H, G, R, O, N, P = spec.H, spec.G, spec.R, spec.O, spec.N, spec.P
    state = state or {}
    xa = x.to(f)
    w_in = prm["in_proj.weight"].to(f)
    drive = xa @ w_in[:spec.d_inner].T
    z = xa @ w_in[spec.d_inner:].T
    ws, bs = [], []
    for key, attr, width, has_bias in spec.slab:
        ws.append(prm[attr + ".weight"].to(f))
        bs.append(prm[attr + ".bias"].to(f) if has_bias else xa.new_zeros(width))
    slab = xa @ torch.cat(ws, 0).T + torch.cat(bs, 0)

    new = {}
    if spec.d_conv > 0:
        drive, new["conv_state"] = causal_conv_silu(drive, prm["conv1d.weight"], prm["conv1d.bias"],
                                                    state.get("conv_state"))
    ob, wb = spec.slab_off["B"]
    oc, wc_ = spec.slab_off["C"]
    b_src, c_src = slab[..., ob:ob + wb], slab[..., oc:oc + wc_]
    if spec.bc_conv:
        bc, new["bc_conv_state"] = causal_conv_silu(torch.cat([b_src, c_src], -1), prm["bc_conv1d.conv.weight"],
                                                    prm["bc_conv1d.conv.bias"], state.get("bc_conv_state"))
        b_src, c_src = bc[..., :wb], bc[..., wb:]
    law = token_law(spec, prm, slab, b_src, c_src, f)
    Bt = law["Bbar"].expand(Bsz, L, H, R, R, N)
    Cq = law["Cbar"] if law["chi"] is None else law["Cbar"] * law["chi"][..., None, None]
    Cq = Cq.expand(Bsz, L, H, R, O, N)
    u = drive.reshape(Bsz, L, H, G, R)
    dt, dA, lam = law["dt"], law["dA"], law["lam"]

    h0 = state.get("hidden_state")
    wp = state.get("write_prev")
    f0 = h0.to(f).reshape(Bsz, H, G, R, N) if h0 is not None else None
    vp = wp.to(f).reshape(Bsz, H, G, R, N) if wp is not None else None
    if wp is not None and lam is None:
        raise ValueError("state carry 'write_prev' with write_rule='euler'")
    if route == "recurrent" or L == 0:
        y, f_last, v_last = scan_recurrent(Bt, Cq, u, dt, dA, lam, f0, vp)
    else:
        if lam is not None:
            lag = dt * (1.0 - lam[..., None])
            wd = lam[..., None] * dt
            w = wd + torch.cat([lag[:, 1:], lag.new_zeros(Bsz, 1, H, R)], dim=1)
        else:
            w = wd = dt
        S0 = f0.permute(0, 1, 3, 4, 2) if f0 is not None else None
        if vp is not None:
            shift = vp.permute(0, 1, 3, 4, 2) * lag[:, 0][..., None, None]
            S0 = shift if S0 is None else S0 + shift
        T = max(1, min(int(chunk or (16 if N <= 64 else 32)), L))
        y, S_fin = scan_chunked(Bt, Cq, u, dA, w, wd, S0, T)
        f_last = S_fin.permute(0, 1, 4, 2, 3)
        v_last = torch.einsum("bhgq,bhrqn->bhgrn", u[:, -1], Bt[:, -1]) if lam is not None else None

    if spec.skip:
        uw = u if law["chi"] is None else u * law["chi"][..., None, :]           # chi [H,R] or [B,L,H,R]
        y = y + torch.einsum("blhgr,hgro->blhgo", uw, skip_gains(spec, prm["D"].to(f)))
    y = y.reshape(Bsz, L, H * G * O)
    y = y * F.silu(z)
    if spec.out_norm:
        y = _rms(y, prm["norm.weight"].to(f), spec.norm_eps)
    out = (y @ prm["out_proj.weight"].to(f).T).to(x.dtype)
    if not return_state:
        return out
    new["hidden_state"] = f_last.reshape(Bsz, H, P, N)
    if lam is not None:
        new["write_prev"] = v_last.reshape(Bsz, H, P, N)
    return out, new
