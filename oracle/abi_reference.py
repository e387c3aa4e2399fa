"""Torch restatements of the C-ABI operators (TEST INFRASTRUCTURE, not product code).

Each function has the signature and return layout of its counterpart in ``orbitssm_b200/ops.py`` and computes the
same quantity with plain torch ops (gradients through torch autograd), on any device.  Uses:
  * ``-m gpu`` tests compare every CUDA kernel with these on the same seeded inputs;
  * CPU tests substitute them for the kernels to check the layer's host logic (token law, state folding, layout
    permutations, autograd wiring) against the golden vectors without a GPU.
The scan follows the reference's chunked dual through ``ssd_oracle.scan_chunked``
(reference: src/orbit_ssm/ssm/ssd_mimo_torch.py:663-708) after building the per-kernel-head maps
(reference: src/orbit_ssm/ssm/ssd_mimo_torch.py:195-210).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ssd_oracle as O


def _f(t, dt=torch.float64):
    return None if t is None else t.detach().to(dt)


# ---- conv --------------------------------------------------------------------------------------------
def _conv(x, weight, bias, window, silu):
    Bsz, L, C = x.shape
    W = weight.shape[-1]
    win = window if window is not None else x.new_zeros(Bsz, C, W)
    full = torch.cat([win.transpose(1, 2), x], dim=1)
    acc = (bias if bias is not None else x.new_zeros(C)).expand(Bsz, L, C)
    for j in range(W):
        acc = acc + full[:, j + 1: j + 1 + L] * weight[:, j]
    return F.silu(acc) if silu else acc


def conv1d_fwd(x, weight, bias, window, silu=True, compute=torch.float64):
    y = _conv(_f(x, compute), _f(weight, compute), _f(bias, compute), _f(window, compute), silu)
    return y.to(x.dtype)


def conv1d_bwd(x, weight, bias, window, dy, silu=True, want_dwindow=False, dx_out=None, compute=torch.float64):
    xs = _f(x, compute).requires_grad_(True)
    ws = _f(weight, compute).requires_grad_(True)
    bs = _f(bias, compute).requires_grad_(True) if bias is not None else None
    wins = _f(window, compute).requires_grad_(True) if window is not None else None
    ins = [t for t in (xs, ws, bs, wins) if t is not None]
    with torch.enable_grad():
        y = _conv(xs, ws, bs, wins, silu)
        gs = torch.autograd.grad(y, ins, _f(dy, compute), allow_unused=True)
    g = dict(zip([id(t) for t in ins], gs))
    dwin = None
    if want_dwindow and wins is not None:
        dwin = g[id(wins)].to(torch.float32).clone()
        dwin[..., 0] = 0.0                       # slot 0 of the window never enters the conv
    dx = g[id(xs)].to(x.dtype)
    if dx_out is not None:
        dx_out.copy_(dx)
        dx = dx_out
    return (dx, dwin, g[id(ws)].to(torch.float32), None if bs is None else g[id(bs)].to(torch.float32))


# ---- gate + norm -------------------------------------------------------------------------------------
def _gate_norm(y, z, w, eps):
    g = y if z is None else y * F.silu(z)
    if w is None:
        return g, None
    rstd = torch.rsqrt(g.square().mean(-1, keepdim=True) + eps)
    return g * rstd * w, rstd.squeeze(-1)


def gate_norm_fwd(y, z, w, eps, compute=torch.float64):
    out, rstd = _gate_norm(_f(y, compute), _f(z, compute), _f(w, compute), eps)
    return out.to(y.dtype), None if rstd is None else rstd.to(torch.float32)


def gate_norm_bwd(y, z, w, rstd, dout, eps=1e-5, dz_out=None, compute=torch.float64):
    ys = _f(y, compute).requires_grad_(True)
    zs = _f(z, compute).requires_grad_(True) if z is not None else None
    ws = _f(w, compute).requires_grad_(True) if w is not None else None
    ins = [t for t in (ys, zs, ws) if t is not None]
    with torch.enable_grad():
        out, _ = _gate_norm(ys, zs, ws, eps)
        gs = dict(zip([id(t) for t in ins], torch.autograd.grad(out, ins, _f(dout, compute))))
    dz = None if zs is None else gs[id(zs)].to(y.dtype)
    if dz is not None and dz_out is not None:
        dz_out.copy_(dz)
        dz = dz_out
    return (gs[id(ys)].to(y.dtype), dz, None if ws is None else gs[id(ws)].to(torch.float32))


# ---- scan --------------------------------------------------------------------------------------------
def _scan(geo, T, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0):
    Bsz, L = u.shape[:2]
    H, R, Oo, G, N = geo.H, geo.R, geo.O, geo.G, geo.N
    Bt = Bhat[:, :, None, None]                                         # [B,L,1,1,q,N]
    if gBp is not None:
        Bt = gBp[:, :, None, :, None, :] * Bt                           # [B,L,1,r,q,N]
    if beta is not None:
        Bt = Bt + beta
    Ct = Chat if gCp is None else Chat * gCp
    Ct = Ct[:, :, None, None]
    if gamma is not None:
        Ct = Ct + gamma
    Bt = Bt.expand(Bsz, L, H, R, R, N)
    Cq = Ct.expand(Bsz, L, H, R, Oo, N)
    if chi is not None:
        Cq = Cq * chi[..., None, None]
    uu = u.reshape(Bsz, L, H, G, R)
    y, S_fin = O.scan_chunked(Bt, Cq, uu, dA, w, wd, S0, T)
    if Dg is not None:
        uw = uu if chi is None else uu * chi[..., None, :]
        y = y + torch.einsum("blhgr,hgro->blhgo", uw, Dg)
    return y.reshape(Bsz, L, H * G * Oo), S_fin


def pick_chunk(geo, precision, backward, limit):
    return min(int(limit), 16)


def scan_fwd(geo, T, precision, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0, compute=torch.float64):
    args = [_f(t, compute) for t in (u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0)]
    y, S_fin = _scan(geo, T, *args)
    # the third slot (the kernels' saved chunk states) carries S0 here: this restatement re-runs the forward in backward
    return y.to(u.dtype), S_fin.to(torch.float32), (None if S0 is None else S0.detach().clone()), None


def scan_bwd(geo, T, precision, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, Sin, atot, dy, dS_fin, euler,
             want_dS0, S0=None, compute=torch.float64):
    if S0 is None and Sin is not None and Sin.dim() == 5:
        S0 = Sin
    names = ("u", "Bhat", "gBp", "Chat", "gCp", "beta", "gamma", "chi", "dA", "w", "wd", "Dg", "S0")
    vals = dict(zip(names, (u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, None if euler else wd, Dg, S0)))
    leaf = {k: (None if v is None else _f(v, compute).requires_grad_(True)) for k, v in vals.items()}
    ins = [(k, v) for k, v in leaf.items() if v is not None]
    with torch.enable_grad():
        y, S_fin = _scan(geo, T, leaf["u"], leaf["Bhat"], leaf["gBp"], leaf["Chat"], leaf["gCp"], leaf["beta"],
                         leaf["gamma"], leaf["chi"], leaf["dA"], leaf["w"], leaf["w"] if euler else leaf["wd"], leaf["Dg"],
                         leaf["S0"])
        loss = (y * _f(dy, compute)).sum()
        if dS_fin is not None:
            loss = loss + (S_fin * _f(dS_fin, compute)).sum()
        gs = dict(zip([k for k, _ in ins], torch.autograd.grad(loss, [v for _, v in ins], allow_unused=True)))

    def g(k, dt=torch.float32):
        t = gs.get(k)
        if t is None:
            return None if vals[k] is None else torch.zeros_like(vals[k], dtype=dt)
        return t.to(dt)

    return dict(du=g("u", u.dtype), dBhat=g("Bhat"), dgBp=g("gBp"), dChat=g("Chat"), dgCp=g("gCp"), dbeta=g("beta"),
                dgamma=g("gamma"), dchi=g("chi"), ddA=g("dA"), dw=g("w"), dwd=g("wd"), dDg=g("Dg"),
                dS0=g("S0") if want_dS0 else None)


# ---- scan, phase by phase (the decomposition the kernels use; drives the context-parallel tests on CPU) -------
def _chunk_local(geo, T, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, Sin):
    """Chunk-local quantities with the entering states `Sin` [B, nc, H, R, N, G] taken as given:
    y [B, L, H*G*O], Z [B, nc, H, R, N, G] (chunk-local state), tot [B, nc, H, R] (chunk decay)."""
    Bsz, L = u.shape[:2]
    H, R, Oo, G, N = geo.H, geo.R, geo.O, geo.G, geo.N
    Bt = Bhat[:, :, None, None]
    if gBp is not None:
        Bt = gBp[:, :, None, :, None, :] * Bt
    if beta is not None:
        Bt = Bt + beta
    Ct = Chat if gCp is None else Chat * gCp
    Ct = Ct[:, :, None, None]
    if gamma is not None:
        Ct = Ct + gamma
    Bt = Bt.expand(Bsz, L, H, R, R, N)
    Cq = Ct.expand(Bsz, L, H, R, Oo, N)
    if chi is not None:
        Cq = Cq * chi[..., None, None]
    uu = u.reshape(Bsz, L, H, G, R)
    nc = -(-L // T)
    pad = nc * T - L

    def ch(t):
        if pad:
            t = torch.cat([t, t.new_zeros(Bsz, pad, *t.shape[2:])], dim=1)
        return t.reshape(Bsz, nc, T, *t.shape[2:])

    Bc, Cc, uc, dAc, wc, wdc = (ch(t) for t in (Bt, Cq, uu, dA, w, wd))
    cs = torch.cumsum(dAc, dim=2)
    tri = torch.ones(T, T, dtype=torch.bool, device=u.device).tril(-1)
    diff = (cs[:, :, :, None] - cs[:, :, None, :]).masked_fill(~tri[None, None, :, :, None, None], float("-inf"))
    Wm = torch.exp(diff) * wc[:, :, None, :]
    eye = torch.eye(T, dtype=torch.bool, device=u.device)[None, None, :, :, None, None]
    Wm = torch.where(eye, wdc[:, :, :, None], Wm)
    score = torch.einsum("bcthron,bcshrqn->bchrotqs", Cc, Bc)
    M = (score * Wm.permute(0, 1, 4, 5, 2, 3)[:, :, :, :, None, :, None, :]).sum(3)
    y = torch.einsum("bchotqs,bcshgq->bcthgo", M, uc)
    dend = torch.exp(cs[:, :, -1:, :, :] - cs) * wc
    Z = torch.einsum("bcshrqn,bcshr,bcshgq->bchrng", Bc, dend, uc)
    tot = cs[:, :, -1].exp()
    y = y + torch.einsum("bcthron,bchrng,bcthr->bcthgo", Cc, Sin, cs.exp())
    y = y.reshape(Bsz, nc * T, H, G, Oo)[:, :L]
    if Dg is not None:
        uw = uu if chi is None else uu * chi[..., None, :]
        y = y + torch.einsum("blhgr,hgro->blhgo", uw, Dg)
    return y.reshape(Bsz, L, H * G * Oo), Z, tot


def run_phase(a, name, phase, state_in, state_out, dtype_code, precision, compute=torch.float64):
    """Torch restatement of `orbit_ssd_scan_phase` on the tensors named in ``a.t`` (same in-place buffer protocol)."""
    t = a.t
    geo, T = t["geo"], a.T
    names = ("u", "Bhat", "gBp", "Chat", "gCp", "beta", "gamma", "chi", "dA", "w", "wd", "Dg")
    Sin, atot = t["Sin"], t["atot"]
    nc = a.nc
    if phase == 0:                                            # chunk_state
        ins = [_f(t[k], compute) for k in names]
        _, Z, tot = _chunk_local(geo, T, *ins, _f(Sin, compute)[:, :nc] * 0)
        Sin[:, :nc].copy_(Z)
        atot[:, :nc].copy_(tot)
    elif phase in (1, 6):                                     # state pass (6: dry)
        S = torch.zeros_like(Sin[:, 0]) if state_in is None else state_in.clone().to(Sin.dtype)
        for c in range(nc):
            z = Sin[:, c].clone()
            if phase == 1:
                Sin[:, c] = S
            S = atot[:, c][..., None, None] * S + z
        state_out.copy_(S)
    elif phase == 2:                                          # chunk_out
        ins = [_f(t[k], compute) for k in names]
        y, _, _ = _chunk_local(geo, T, *ins, _f(Sin, compute)[:, :nc])
        t["y"].copy_(y)
    elif phase == 3:                                          # chunk_dstate
        ins = [_f(t[k], compute) for k in names]
        S = _f(Sin, compute)[:, :nc].requires_grad_(True)
        with torch.enable_grad():
            y, _, _ = _chunk_local(geo, T, *ins, S)
            (g,) = torch.autograd.grad(y, S, _f(t["dy"], compute))
        t["dS"][:, :nc].copy_(g)
    elif phase in (4, 7):                                     # reverse pass (7: dry)
        dS = t["dS"]
        D = torch.zeros_like(dS[:, 0]) if state_in is None else state_in.clone().to(dS.dtype)
        for c in range(nc - 1, -1, -1):
            g = dS[:, c].clone()
            if phase == 4:
                dS[:, c] = D
            D = atot[:, c][..., None, None] * D + g
        if state_out is not None:
            state_out.copy_(D)
    elif phase == 5:                                          # chunk_grads
        leaf = {k: (None if t[k] is None else _f(t[k], compute).requires_grad_(True)) for k in names}
        with torch.enable_grad():
            y, Z, tot = _chunk_local(geo, T, *[leaf[k] for k in names], _f(Sin, compute)[:, :nc])
            Sout = tot[..., None, None] * _f(Sin, compute)[:, :nc] + Z
            loss = (y * _f(t["dy"], compute)).sum() + (Sout * _f(t["dS"], compute)[:, :nc]).sum()
            ins = [(k, v) for k, v in leaf.items() if v is not None]
            gs = dict(zip([k for k, _ in ins], torch.autograd.grad(loss, [v for _, v in ins], allow_unused=True)))
        out = t["out"]

        def put(dst, key):
            if dst is not None:
                g = gs.get(key)
                dst.copy_(torch.zeros_like(dst) if g is None else g.reshape(dst.shape))

        put(out["du"], "u"); put(out["dBhat"], "Bhat"); put(out["dgBp"], "gBp"); put(out["dChat"], "Chat")
        put(out["dgCp"], "gCp"); put(out["ddA"], "dA"); put(out["dw"], "w"); put(out["dchi"], "chi")
        if t["dwd"] is not None:
            put(t["dwd"], "wd")                               # own-token weight: a separate buffer even when w and wd coincide
        for part, key in ((t["dbeta_part"], "beta"), (t["dgamma_part"], "gamma"), (t["dDg_part"], "Dg")):
            if part is not None:
                part.zero_()
                part[0].copy_(gs[key])
    else:
        raise ValueError(f"unknown phase {phase}")


# ---- HybridMamba coordinate-decay scan ------------------------------------------------------------------
_HM_KEYS = ("x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "theta_h", "lam", "D", "h_init", "write_prev",
            "theta_init")


def _hm(ins, rot):
    from . import hm_oracle as HM
    rot_rows = None if rot is None else torch.repeat_interleave(rot.to(torch.bool).cpu(), 2).to(ins["x"].device)
    return HM.hm_scan(ins["x"], ins["delta"], ins["A_log"], ins["Bh"], ins["Ch"], beta_b=ins["beta_b"], beta_c=ins["beta_c"],
                      feat=ins["feat"], rot_rows=rot_rows, theta_h=ins["theta_h"], lam=ins["lam"], D=ins["D"],
                      h_init=ins["h_init"], write_prev=ins["write_prev"], theta_init=ins["theta_init"])


def hm_scan_fwd(x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, rot, theta_h, lam, D, h_init, write_prev, theta_init,
                compute=torch.float64):
    """Same arguments as ``ops.hm_scan_fwd``; returns (y, h_final, theta_final, write_last) in `compute` precision."""
    ins = dict(zip(_HM_KEYS, (x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, theta_h, lam, D, h_init, write_prev, theta_init)))
    ins = {k: _f(v, compute) for k, v in ins.items()}
    return _hm(ins, rot)


def hm_scan_bwd(x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, rot, theta_h, lam, D, h_init, write_prev, theta_init,
                dy, dh_final, dtheta_final, dwrite_last, compute=torch.float64):
    """Gradients of sum(y dy) + sum(h_final dh_final) + ... with respect to every floating argument (dict keyed like the
    arguments), through torch autograd over the token loop."""
    ins = dict(zip(_HM_KEYS, (x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, theta_h, lam, D, h_init, write_prev, theta_init)))
    ins = {k: (None if v is None else _f(v, compute).requires_grad_(True)) for k, v in ins.items()}
    with torch.enable_grad():
        y, hN, thN, wl = _hm(ins, rot)
        loss = (y * _f(dy, compute)).sum()
        if dh_final is not None:
            loss = loss + (hN * _f(dh_final, compute)).sum()
        if dtheta_final is not None and thN is not None:
            loss = loss + (thN * _f(dtheta_final, compute)).sum()
        if dwrite_last is not None:
            loss = loss + (wl * _f(dwrite_last, compute)).sum()
        live = [k for k, v in ins.items() if v is not None]
        grads = torch.autograd.grad(loss, [ins[k] for k in live], allow_unused=True)
    out = {k: None for k in _HM_KEYS}
    for k, gv in zip(live, grads):
        out[k] = torch.zeros_like(ins[k]) if gv is None else gv
    return out


def run_hm(a, name, backward, dtype_code, compute=torch.float64):
    """Torch restatement of `orbit_hm_scan_fwd` / `_bwd` on the tensors named in ``a.t`` (same buffer protocol: the
    forward fills y, carries and the chunk-entering states; the backward fills the partial-sum buffers, whole sums in
    slot 0 of their leading axis)."""
    t = a.t
    args = [t.get(k) for k in ("x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "rot", "theta_h", "lam", "D",
                               "h_init", "write_prev", "theta_init")]
    if not backward:
        y, hN, thN, wl = hm_scan_fwd(*args, compute=compute)
        t["y"].copy_(y.reshape(t["y"].shape))
        t["h_final"].copy_(hN)
        t["write_last"].copy_(wl)
        if t["theta_final"] is not None:
            t["theta_final"].copy_(thN)
        t["hck"].zero_()                                  # this restatement replays from the inputs, not from checkpoints
        if t["thck"] is not None:
            t["thck"].zero_()
        return
    g = hm_scan_bwd(*args, t["dy"], t["dh_final"], t["dtheta_final"], t["dwrite_last"], compute=compute)
    t["dx"].copy_(g["x"].reshape(t["dx"].shape))
    t["ddelta"].copy_(g["delta"])
    for dst, key in (("dlam", "lam"), ("dh_init", "h_init"), ("dwrite_prev", "write_prev"), ("dtheta_init", "theta_init")):
        if t.get(dst) is not None:
            if g[key] is None:
                # gradient of an absent (zero) carry: differentiate again with an explicit zero carry
                zero = dict(h_init=torch.zeros_like(t["dh_init"]), write_prev=torch.zeros_like(t["dh_init"]),
                            theta_init=None if t.get("dtheta_init") is None else torch.zeros_like(t["dtheta_init"]))
                args2 = list(args)
                for i, k in ((12, "h_init"), (13, "write_prev"), (14, "theta_init")):
                    if args2[i] is None and zero[k] is not None and (k != "write_prev" or t.get("lam") is not None):
                        args2[i] = zero[k]
                g2 = hm_scan_bwd(*args2, t["dy"], t["dh_final"], t["dtheta_final"], t["dwrite_last"], compute=compute)
                g = {**g, **{k: g2[k] for k in ("h_init", "write_prev", "theta_init")}}
            t[dst].copy_(g[key])
    for dst, key in (("dA_log_part", "A_log"), ("dBh_part", "Bh"), ("dCh_part", "Ch"), ("dbeta_b_part", "beta_b"),
                     ("dbeta_c_part", "beta_c"), ("dfeat_part", "feat"), ("dtheta_h_part", "theta_h"), ("dD_part", "D")):
        if t.get(dst) is not None:
            t[dst].zero_()
            t[dst][0].copy_(g[key])


# ---- token tails ------------------------------------------------------------------------------------------
def _map(src, weight, bias, add, eps, X, N):
    B, L = src.shape[:2]
    m = src.reshape(B, L, N, X).transpose(-1, -2)
    if weight is not None:
        m = m * torch.rsqrt(m.square().mean(-1, keepdim=True) + eps) * weight
    if bias is not None:
        m = m + bias
    return m + add


def token_map_fwd(src, weight, bias, add, eps, X, N, compute=torch.float64):
    s = _f(src, compute)
    out = _map(s, _f(weight, compute), _f(bias, compute), add, eps, X, N)
    rstd = None
    if weight is not None:
        B, L = src.shape[:2]
        rstd = torch.rsqrt(s.reshape(B, L, N, X).transpose(-1, -2).square().mean(-1) + eps).to(torch.float32)
    return out.to(src.dtype).contiguous(), rstd


def token_map_bwd(src, weight, rstd, dout, X, N, want_dbias, dsrc_out=None, eps=1e-5, compute=torch.float64):
    s = _f(src, compute).requires_grad_(True)
    w = _f(weight, compute).requires_grad_(True) if weight is not None else None
    b = torch.zeros(N, dtype=compute, device=src.device, requires_grad=True) if want_dbias else None
    ins = [t for t in (s, w, b) if t is not None]
    with torch.enable_grad():
        out = _map(s, w, b, 0.0, eps, X, N)
        gs = dict(zip([id(t) for t in ins], torch.autograd.grad(out, ins, _f(dout, compute))))
    dsrc = gs[id(s)].to(src.dtype)
    if dsrc_out is not None:
        dsrc_out.copy_(dsrc)
        dsrc = dsrc_out
    return (dsrc, None if w is None else gs[id(w)].to(torch.float32), None if b is None else gs[id(b)].to(torch.float32))


def _clock(t, compute, leaves=False):
    dev = t["dt_raw"].device
    B, L = t["dt_raw"].shape[:2]
    H, Rr = t["H"], t["R"]

    def leaf(v):
        if v is None:
            return None
        v = _f(v, compute)
        return v.requires_grad_(True) if leaves else v

    dt_raw, a_raw, trap_raw, rmix_raw = leaf(t["dt_raw"]), leaf(t.get("a_raw")), leaf(t.get("trap_raw")), leaf(t.get("rmix_raw"))
    A_log, r_mix = leaf(t.get("A_log")), leaf(t.get("r_mix"))
    dt = F.softplus(dt_raw).reshape(B, L, H, Rr)
    if t["a_act"] == 0:
        rate = A_log.exp().reshape(H, Rr)
    else:
        mag = (O._pass_min(O._pass_min(a_raw, 0.0) + torch.reciprocal(1.0 - O._pass_max(a_raw, 0.0)), 1e-4) if t["a_act"] == 1
               else O._pass_min(F.softplus(a_raw), 1e-4))
        rate = mag.reshape(B, L, H, Rr) if t["a_per_sibling"] else mag.reshape(B, L, H, 1)
    dA = -(dt * rate)
    wd = lag0 = chi = None
    if trap_raw is not None:
        lam = torch.sigmoid(trap_raw)[..., None]
        lag = dt * (1.0 - lam)
        wd = lam * dt
        w = wd + torch.cat([lag[:, 1:], lag.new_zeros(B, 1, H, Rr)], dim=1)
        lag0 = lag[:, 0]
    else:
        w = dt
    if r_mix is not None:
        chi = r_mix.reshape(H, Rr) + (rmix_raw.reshape(B, L, H, Rr) if rmix_raw is not None else 0.0)
        chi = chi.expand(B, L, H, Rr)
    return dict(dA=dA, w=w, wd=wd, chi=chi, lag0=lag0), dict(dt_raw=dt_raw, a_raw=a_raw, trap_raw=trap_raw, rmix_raw=rmix_raw,
                                                              A_log=A_log, r_mix=r_mix)


def run_clock(a, name, backward, dtype_code, compute=torch.float64):
    """Torch restatement of `orbit_token_clock_fwd` / `_bwd` on the tensors named in ``a.t``."""
    t = a.t
    if not backward:
        out, _ = _clock(t, compute)
        for k in ("dA", "w", "wd", "chi", "lag0"):
            if t.get(k) is not None:
                t[k].copy_(out[k])
        return
    with torch.enable_grad():
        out, leaves = _clock(t, compute, leaves=True)
        loss = (out["dA"] * _f(t["ddA"], compute)).sum() + (out["w"] * _f(t["dw"], compute)).sum()
        for k, gk in (("wd", "dwd"), ("chi", "dchi"), ("lag0", "dlag0")):
            if out[k] is not None and t.get(gk) is not None:
                loss = loss + (out[k] * _f(t[gk], compute)).sum()
        live = [k for k, v in leaves.items() if v is not None]
        gs = dict(zip(live, torch.autograd.grad(loss, [leaves[k] for k in live], allow_unused=True)))
    for key in ("dt_raw", "a_raw", "trap_raw", "rmix_raw"):
        dst = t.get("d_" + key)
        if dst is not None:
            gv = gs.get(key)
            dst.copy_(torch.zeros_like(leaves[key]) if gv is None else gv)
    if t.get("g_alog") is not None:
        # per-row term of dA_log: d dA / d A_log = dA itself (rate = exp(A_log))
        t["g_alog"].copy_(_f(t["ddA"], compute) * out["dA"].detach())
    if t.get("bias_sums") is not None:
        # gradients of the slab biases: column sums of the unrounded raw gradients, [ dt | a | trap ]
        cols = [gs[k].reshape(-1, gs[k].shape[-1]).sum(0) for k in ("dt_raw", "a_raw", "trap_raw") if leaves.get(k) is not None and gs.get(k) is not None]
        t["bias_sums"].copy_(torch.cat(cols).to(t["bias_sums"].dtype))


def run_step(a, S0, S_fin, dtype_code, compute=torch.float64):
    """Restatement of orbit_ssd_scan_step: the forward scan on the one token."""
    t = a.t
    geo = t["geo"]
    y, S, _, _ = scan_fwd(geo, 1, 0, t["u"], t["Bhat"], t["gBp"], t["Chat"], t["gCp"], t["beta"], t["gamma"], t["chi"], t["dA"],
                          t["w"], t["wd"], t["Dg"], S0, compute=compute)
    t["y"].copy_(y.to(t["y"].dtype))
    S_fin.copy_(S.to(S_fin.dtype))


# ---- HybridMamba clock tail (torch restatement of orbit_hm_tail_fwd / orbit_hm_tail_bwd) ---------------------------------
def _hm_tail(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, compute):
    delta = torch.nn.functional.softplus(dt_raw.to(compute) + dt_bias.to(compute))
    lam = None
    if trap_raw is not None:
        lam = torch.sigmoid(trap_raw.to(compute) + (trap_bias.to(compute) if trap_bias is not None else 0.0))
    feat = None
    if th_raw is not None:
        q = th_raw.to(compute)
        feat = q.new_zeros(*q.shape[:-1], K).index_copy(-1, rot_idx.long(), omega.to(compute) * torch.tanh(q))
    return delta, lam, feat


def hm_tail_fwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, compute=torch.float64):
    with torch.no_grad():
        delta, lam, feat = _hm_tail(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, compute)
    f = torch.float32
    return delta.to(f), None if lam is None else lam.to(f), None if feat is None else feat.to(f)


def hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, lam, ddelta, dlam, dfeat, compute=torch.float64):
    ins = [None if v is None else v.detach().to(compute).requires_grad_(True) for v in (dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega)]
    with torch.enable_grad():
        outs = _hm_tail(*ins, rot_idx, K, compute)
        loss = 0.0
        for o, g in zip(outs, (ddelta, dlam, dfeat)):
            if o is not None and g is not None:
                loss = loss + (o * g.to(compute)).sum()
    have = [v for v in ins if v is not None]
    grads = iter(torch.autograd.grad(loss, have, allow_unused=True)) if torch.is_tensor(loss) else iter([None] * len(have))
    full = [None if v is None else next(grads) for v in ins]
    full = [torch.zeros_like(v) if (g is None and v is not None) else g for g, v in zip(full, ins)]
    io = dt_raw.dtype
    f = torch.float32
    return (full[0].to(io), None if full[1] is None else full[1].to(io), None if full[2] is None else full[2].to(io),
            full[3].to(f), None if (full[4] is None or trap_raw is None) else full[4].to(f), None if full[5] is None else full[5].to(f))


# ---- context-parallel exchange records (torch restatements of orbit_cp_state_pack / orbit_cp_state_combine) ----------
def cp_pack(dA, record, n_state):
    record[n_state:n_state + dA.shape[0] * dA.shape[2] * dA.shape[3]] = dA.sum(1).reshape(-1).to(record.dtype)


def cp_combine(records, world, rank, n_state, per_head, BHR, backward):
    st = records[:, :n_state].double()
    dec = records[:, n_state:n_state + BHR].double().exp().repeat_interleave(per_head, dim=1)
    if not backward:
        S = torch.zeros(n_state, dtype=torch.float64)
        for j in range(rank):
            S = dec[j] * S + st[j]
        return S.to(records.dtype)
    ext = records[:, n_state + BHR:n_state + BHR + n_state].double()
    d = ext[world - 1]
    for j in range(world - 1, rank, -1):
        d = ext[j - 1] + st[j] + dec[j] * d
    return d.to(records.dtype)
