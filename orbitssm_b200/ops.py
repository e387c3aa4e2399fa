"""Tensor-level operators over the C-ABI kernels, with their autograd wiring.

Each ``*_fwd`` / ``*_bwd`` function takes CUDA tensors, hands raw pointers to ``liborbit_b200.so`` on the current
stream and returns tensors; the `torch.autograd.Function` classes below compose them.  They mirror the reference's
operator seams: `causal_conv1d_cl_fwd/_bwd` (reference: src/orbit_ssm/layers/conv.py:219-277), `gated_rms_norm`
(src/orbit_ssm/layers/norms.py:133-168) and `ssd_mimo_scan` (src/orbit_ssm/kernels/ssd_mimo/autograd.py:2247).
A CPU tensor at any of these entries is refused by name (reference: src/orbit_ssm/kernels/input_checks.py).
"""
from __future__ import annotations

import ctypes as C
import functools
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


#: number of this library's kernel launches since import (each C-ABI call adds the launches it makes)
LAUNCHES = 0
#: when a list, every timed region appends (name, start_event, end_event) recorded on the current stream
_TIMING = None


def set_timing(collector):
    """Give a list to collect (name, start, end) CUDA-event triples around every kernel group; None switches it off."""
    global _TIMING
    _TIMING = collector


class _timed:
    def __init__(self, name, launches):
        self.name, self.launches = name, launches

    def __enter__(self):
        global LAUNCHES
        LAUNCHES += self.launches
        if _TIMING is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _TIMING is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _TIMING.append((self.name, self.e0, e1))
        return False


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def on_device(t) -> bool:
    """Is `t` where the kernels can reach it (a CUDA tensor)?"""
    return t.is_cuda


def _require_cuda(who, *tensors):
    for t in tensors:
        if t is not None and not on_device(t):
            raise ValueError(f"{who}: got a CPU tensor; backend='cuda' runs on a CUDA device only and has no CPU route "
                             f"(the reference's backend='torch' is the CPU implementation)")


def _dtype_code(who, t):
    if t.dtype not in _DT:
        raise NotImplementedError(f"{who}: activations must be float32 or bfloat16, got {t.dtype}")
    return _DT[t.dtype]


def _f32(t):
    if t is None:
        return None
    return t.detach().to(torch.float32).contiguous()


# ----------------------------------------------------------------------------------------------------
#  first-order only: the kernels' backward passes record no autograd graph
# ----------------------------------------------------------------------------------------------------
class _SecondOrderTrap(torch.autograd.Function):
    """Identity on a gradient a kernel produced; differentiating through it raises."""

    @staticmethod
    def forward(ctx, who, g, anchor):
        ctx.who = who
        return g.view_as(g)

    @staticmethod
    def backward(ctx, *_):
        raise RuntimeError(
            f"{ctx.who}: second-order gradients (create_graph=True, then differentiating the result) are not served: the "
            "backward of this operator is a CUDA kernel that records no autograd graph, so a second derivative would "
            "silently lack the kernel's part.  The reference's backend='torch' route is differentiable to any order.")


def first_order_only(who):
    """Decorator for an `autograd.Function.backward` that runs kernels.  With ``create_graph=True`` autograd calls the
    backward in grad mode; the kernels then run under ``no_grad`` and each gradient they return is tied to a node whose
    own backward raises, so a later attempt to differentiate it fails by name instead of returning a wrong number
    (reference behaviour: src/orbit_ssm/kernels/autograd_guard.py).  In an ordinary backward this costs one test."""
    def deco(bwd):
        @functools.wraps(bwd)
        def guarded(ctx, *grads):
            if not torch.is_grad_enabled():
                return bwd(ctx, *grads)
            with torch.no_grad():
                out = bwd(ctx, *grads)
            ref = next((g for g in grads if torch.is_tensor(g)), None)
            anchor = torch.zeros((), device=None if ref is None else ref.device, requires_grad=True)

            def tie(o):
                return _SecondOrderTrap.apply(who, o, anchor) if (torch.is_tensor(o) and o.is_floating_point()) else o
            return tuple(tie(o) for o in out) if isinstance(out, tuple) else tie(out)
        return guarded
    return deco


# ----------------------------------------------------------------------------------------------------
#  fused projection output -> column views
# ----------------------------------------------------------------------------------------------------
class GradArena:
    """The gradient buffer of one fused projection output, shared by the consumers of its column views: the conv and
    gate backward kernels write their input gradients straight into their column range (strided rows), so that
    `SplitColumnsFn.backward` has nothing left to copy for those ranges.  One arena per forward call."""

    def __init__(self):
        self.buf = None
        self.shape = self.offsets = None

    def bind(self, shape, sizes):
        self.shape, self.offsets, o = tuple(shape), [], 0
        for w in sizes:
            self.offsets.append((o, w))
            o += w

    def view(self, index, like):
        """Column range `index` of the (lazily allocated) buffer, or None when the arena cannot serve `like` (a tensor
        of the range's shape: [..., width])."""
        if self.shape is None or like.dim() != len(self.shape) or tuple(like.shape[:-1]) != self.shape[:-1]:
            return None
        o, w = self.offsets[index]
        if like.shape[-1] != w:
            return None
        if self.buf is None:
            self.buf = torch.empty(self.shape, device=like.device, dtype=like.dtype)
        if self.buf.dtype != like.dtype:
            return None
        return self.buf[..., o:o + w]


class SplitColumnsFn(torch.autograd.Function):
    """Column views of the fused projection output; the backward assembles the views' gradients into ONE buffer in a
    single pass (autograd's own slice backward would zero-fill and add one full-width buffer per view).  With a
    `GradArena` the ranges whose gradient was already written in place by its producer are not copied at all."""

    @staticmethod
    def forward(ctx, proj, arena, *sizes):
        ctx.sizes, ctx.shape, ctx.arena = sizes, proj.shape, arena
        if arena is not None:
            arena.bind(proj.shape, sizes)
        outs, o = [], 0
        for w in sizes:
            outs.append(proj[..., o:o + w])
            o += w
        return tuple(outs)

    @staticmethod
    @first_order_only("SplitColumnsFn")
    def backward(ctx, *grads):
        ref = next(g for g in grads if g is not None)
        arena = ctx.arena
        if arena is not None and arena.buf is not None and arena.buf.dtype == ref.dtype:
            out = arena.buf
        else:
            out = torch.empty(ctx.shape, device=ref.device, dtype=ref.dtype)
        o = 0
        for w, g in zip(ctx.sizes, grads):
            dst = out[..., o:o + w]
            if g is None:
                dst.zero_()
            elif not (g.data_ptr() == dst.data_ptr() and g.stride() == dst.stride() and g.shape == dst.shape):
                dst.copy_(g)
            o += w
        if o < ctx.shape[-1]:
            out[..., o:].zero_()
        return (out, None) + (None,) * len(ctx.sizes)


def _mm_f32(a, b):
    """a @ b accumulated and returned in float32 (16-bit operands on a CUDA device: one GEMM with an fp32 result, no
    16-bit rounding of the product and no cast pass after it)."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16):
        return torch.mm(a, b, out_dtype=torch.float32)
    return (a @ b).to(torch.float32)


class ProjectFn(torch.autograd.Function):
    """``x @ cat(weights)^T`` (+ `bias` on the columns from `bias_off`, + `pad` zero columns, or + `residual`) as ONE node over the
    parameters themselves: the projections of a layer that share an input (drive | gate | token slab; reference:
    src/orbit_ssm/ssm/ssd_mimo.py:4545-4558, src/orbit_ssm/ssm/hybrid_mamba.py:2729-2759) or a single projection.

    The fp32 master weights are cast into one buffer of the IO dtype in a single pass (no concatenated fp32 copy);
    backward forms the weight gradient as one GEMM with an fp32 result and hands each parameter its row range of it
    (no cast or split pass), and reduces the bias gradient over the biased columns only (a linear layer's own backward
    would sum every column of the gradient)."""

    @staticmethod
    def forward(ctx, x, residual, pad, bias, bias_off, *weights):
        io, K = x.dtype, x.shape[-1]
        sizes = [int(w.shape[0]) for w in weights]
        n_tot = sum(sizes) + int(pad)
        wcat = torch.empty((n_tot, K), device=x.device, dtype=io)
        o = 0
        for w, n in zip(weights, sizes):
            wcat[o:o + n].copy_(w)
            o += n
        if pad:
            wcat[o:].zero_()
        x2 = x.reshape(-1, K)
        bfull = None
        if bias is not None:
            bfull = torch.zeros((n_tot,), device=x.device, dtype=io)
            bfull[bias_off:bias_off + bias.shape[0]].copy_(bias)
        if residual is not None:
            # residual + x W^T in the GEMM's own epilogue (beta = 1): the block's residual add costs no pass of its own
            if bias is not None or pad or residual.dtype != io:
                raise ValueError("ProjectFn: a residual goes with one unpadded, unbiased projection in the IO dtype")
            out = torch.addmm(residual.reshape(-1, n_tot), x2, wcat.t())
        else:
            out = F.linear(x2, wcat, bfull)
        ctx.save_for_backward(x2, wcat)
        ctx.meta = (sizes, [w.dtype for w in weights], None if bias is None else (int(bias_off), int(bias.shape[0]), bias.dtype),
                    x.shape)
        return out.view(*x.shape[:-1], n_tot)

    @staticmethod
    @first_order_only("fused projection")
    def backward(ctx, dproj):
        x2, wcat = ctx.saved_tensors
        sizes, wdts, bmeta, xshape = ctx.meta
        d2 = dproj.reshape(-1, dproj.shape[-1])
        dx = (d2 @ wcat).view(xshape) if ctx.needs_input_grad[0] else None
        dres = dproj if ctx.needs_input_grad[1] else None
        dws = [None] * len(sizes)
        if any(ctx.needs_input_grad[5:]):
            dW = _mm_f32(d2.t(), x2)
            o = 0
            for i, (n, dt) in enumerate(zip(sizes, wdts)):
                if ctx.needs_input_grad[5 + i]:
                    dws[i] = dW[o:o + n] if dt == torch.float32 else dW[o:o + n].to(dt)
                o += n
        db = None
        if bmeta is not None and ctx.needs_input_grad[3]:
            off, nb, bdt = bmeta
            db = d2[:, off:off + nb].sum(0).to(bdt)      # fp32 accumulation, result in the IO dtype (as a linear layer's own backward)
        return (dx, dres, None, db, None, *dws)


# ----------------------------------------------------------------------------------------------------
#  conv
# ----------------------------------------------------------------------------------------------------
def _rows(who, x):
    """(batch_stride, row_stride) of a [B, L, C] tensor whose channel run is contiguous."""
    if x.dim() != 3 or (x.shape[-1] > 1 and x.stride(-1) != 1):
        raise ValueError(f"{who}: expected [B, L, C] with a contiguous channel run, got shape {tuple(x.shape)} "
                         f"strides {x.stride()}")
    return x.stride(0), x.stride(1)


def conv1d_fwd(x, weight, bias, window, silu=True):
    """x [B, L, C] (any batch/row strides), weight [C, W] fp32, bias [C] fp32 | None, window [B, C, W] fp32 | None."""
    _require_cuda("conv1d_fwd", x, weight, bias, window)
    B, L, Cc = x.shape
    W = weight.shape[-1]
    bs, rs = _rows("conv1d_fwd", x)
    y = torch.empty((B, L, Cc), device=x.device, dtype=x.dtype)
    if B * L == 0:
        return y
    if W < 2 or W > 4:
        raise NotImplementedError(f"conv1d_fwd: conv width W={W}: the kernel serves 2..4")
    lib = _lib.load()
    with _timed("conv1d_fwd", 1):
        _lib.check(lib.orbit_conv1d_fwd(_ptr(x), bs, rs, _ptr(weight), _ptr(bias), _ptr(window), _ptr(y), B, L, Cc, W,
                                        _dtype_code("conv1d_fwd", x), int(silu), _stream()), "orbit_conv1d_fwd")
    return y


def conv1d_bwd(x, weight, bias, window, dy, silu=True, want_dwindow=False, dx_out=None):
    """Returns (dx [B, L, C], dwindow | None, dweight [C, W], dbias [C] | None); `dx_out` (same shape, contiguous
    channel run, any row strides) receives dx in place."""
    _require_cuda("conv1d_bwd", x, weight, bias, window, dy)
    B, L, Cc = x.shape
    W = weight.shape[-1]
    bs, rs = _rows("conv1d_bwd", x)
    dy = dy.contiguous()
    dx = dx_out if dx_out is not None else torch.empty((B, L, Cc), device=x.device, dtype=x.dtype)
    dwin = torch.empty((B, Cc, W), device=x.device, dtype=torch.float32) if want_dwindow else None
    dweight = torch.empty((Cc, W), device=x.device, dtype=torch.float32)
    dbias = torch.empty((Cc,), device=x.device, dtype=torch.float32) if bias is not None else None
    lib = _lib.load()
    nbytes = lib.orbit_conv1d_bwd_workspace_bytes(B, L, Cc, W)
    ws = torch.empty((max(int(nbytes), 4),), device=x.device, dtype=torch.uint8)
    with _timed("conv1d_bwd", 2 if B * L else 0):
        _lib.check(lib.orbit_conv1d_bwd(_ptr(x), bs, rs, _ptr(weight), _ptr(bias), _ptr(window), _ptr(dy), _ptr(dx),
                                        dx.stride(0), dx.stride(1), _ptr(dwin), _ptr(dweight), _ptr(dbias), _ptr(ws),
                                        int(nbytes), B, L, Cc, W, _dtype_code("conv1d_bwd", x), int(silu), _stream()),
                   "orbit_conv1d_bwd")
    return dx, dwin, dweight, dbias


class CausalConvFn(torch.autograd.Function):
    """y = silu(causal depthwise conv(x) + bias) on token-major x, with the carried window as a differentiable input."""

    @staticmethod
    def forward(ctx, x, weight, bias, window, slot=None):
        w32, b32, win32 = _f32(weight.reshape(weight.shape[0], -1)), _f32(bias), _f32(window)
        y = conv1d_fwd(x, w32, b32, win32)
        ctx.save_for_backward(x, w32, b32, win32)
        ctx.meta = (weight.shape, weight.dtype, None if bias is None else bias.dtype,
                    None if window is None else window.dtype)
        ctx.slot = slot            # (GradArena, column-range index) of x, or None
        return y

    @staticmethod
    @first_order_only("causal conv1d")
    def backward(ctx, dy):
        x, w32, b32, win32 = ctx.saved_tensors
        wshape, wdt, bdt, windt = ctx.meta
        want_win = win32 is not None and ctx.needs_input_grad[3]
        dx_out = ctx.slot[0].view(ctx.slot[1], x) if (ctx.slot is not None and ctx.needs_input_grad[0]) else None
        if dx_out is not None:
            dx, dwin, dw, db = conv1d_bwd(x, w32, b32, win32, dy, want_dwindow=want_win, dx_out=dx_out)
        else:
            dx, dwin, dw, db = conv1d_bwd(x, w32, b32, win32, dy, want_dwindow=want_win)
        return (dx if ctx.needs_input_grad[0] else None,
                dw.reshape(wshape).to(wdt) if ctx.needs_input_grad[1] else None,
                db.to(bdt) if (db is not None and ctx.needs_input_grad[2]) else None,
                dwin.to(windt) if want_win else None, None)


# ----------------------------------------------------------------------------------------------------
#  gate + RMSNorm
# ----------------------------------------------------------------------------------------------------
def _rows2(who, t, D):
    if t.dim() != 2 or t.shape[1] != D or (D > 1 and t.stride(1) != 1):
        raise ValueError(f"{who}: expected [M, {D}] with a contiguous row, got {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def gate_norm_fwd(y, z, w, eps):
    """y [M, D] contiguous, z [M, D] (row stride free) | None, w [D] fp32 | None -> (out [M, D], rstd [M] | None)."""
    _require_cuda("gate_norm_fwd", y, z, w)
    M, D = y.shape
    y = y.contiguous()
    zs = _rows2("gate_norm_fwd", z, D) if z is not None else 0
    out = torch.empty_like(y)
    rstd = torch.empty((M,), device=y.device, dtype=torch.float32) if w is not None else None
    lib = _lib.load()
    with _timed("gate_norm_fwd", 1 if M else 0):
        _lib.check(lib.orbit_gate_norm_fwd(_ptr(y), _ptr(z), zs, _ptr(w), _ptr(out), _ptr(rstd), M, D, float(eps),
                                           _dtype_code("gate_norm_fwd", y), _stream()), "orbit_gate_norm_fwd")
    return out, rstd


def gate_norm_bwd(y, z, w, rstd, dout, dz_out=None):
    """Returns (dy [M, D], dz [M, D] | None, dw [D] | None); `dz_out` ([M, D], contiguous rows, any row stride)
    receives dz in place."""
    _require_cuda("gate_norm_bwd", y, z, w, rstd, dout)
    M, D = y.shape
    dout = dout.contiguous()
    zs = _rows2("gate_norm_bwd", z, D) if z is not None else 0
    dy = torch.empty_like(y)
    dz = (dz_out if dz_out is not None else torch.empty((M, D), device=y.device, dtype=y.dtype)) if z is not None else None
    dzs = D if dz is None else dz.stride(0)
    dw = torch.empty((D,), device=y.device, dtype=torch.float32) if w is not None else None
    lib = _lib.load()
    nbytes = lib.orbit_gate_norm_bwd_workspace_bytes(M, D)
    ws = torch.empty((max(int(nbytes), 4),), device=y.device, dtype=torch.uint8)
    with _timed("gate_norm_bwd", (2 if w is not None else 1) if M else 0):
        _lib.check(lib.orbit_gate_norm_bwd(_ptr(y), _ptr(z), zs, _ptr(w), _ptr(rstd), _ptr(dout), _ptr(dy), _ptr(dz),
                                           dzs, _ptr(dw), _ptr(ws), int(nbytes), M, D, _dtype_code("gate_norm_bwd", y),
                                           _stream()), "orbit_gate_norm_bwd")
    return dy, dz, dw


class GateNormFn(torch.autograd.Function):
    """out = rms_norm(y * silu(z)) * w over the last axis; z and/or w may be None."""

    @staticmethod
    def forward(ctx, y, z, w, eps, slot=None):
        ctx.slot = slot            # (GradArena, column-range index) of z, or None
        shp = y.shape
        D = shp[-1]
        y2 = y.reshape(-1, D)
        z2 = None
        if z is not None:
            z2 = z.reshape(-1, D) if z.is_contiguous() else _as_rows(z, D)
        w32 = _f32(w)
        out, rstd = gate_norm_fwd(y2, z2, w32, eps)
        ctx.save_for_backward(y2, z2, w32, rstd)
        ctx.meta = (shp, None if w is None else w.dtype)
        return out.reshape(shp)

    @staticmethod
    @first_order_only("gate + RMSNorm")
    def backward(ctx, dout):
        y2, z2, w32, rstd = ctx.saved_tensors
        shp, wdt = ctx.meta
        dz_view = None
        if ctx.slot is not None and z2 is not None and ctx.needs_input_grad[1]:
            dz_view = ctx.slot[0].view(ctx.slot[1], dout)
        if dz_view is not None:
            dy, dz, dw = gate_norm_bwd(y2, z2, w32, rstd, dout.reshape(-1, shp[-1]), dz_out=dz_view.view(-1, shp[-1]))
            dz = dz_view
        else:
            dy, dz, dw = gate_norm_bwd(y2, z2, w32, rstd, dout.reshape(-1, shp[-1]))
            dz = None if dz is None else dz.reshape(shp)
        return (dy.reshape(shp), dz, None if dw is None else dw.to(wdt), None, None)


def _as_rows(t, D):
    """View [..., D] with uniform row stride as [M, D] without copying when the leading axes collapse; else copy."""
    try:
        return t.view(-1, D)
    except RuntimeError:
        # leading axes (B, L) of a column slice collapse whenever stride(0) == L * stride(1)
        if t.dim() == 3 and t.stride(0) == t.shape[1] * t.stride(1) and t.stride(2) == 1:
            return t.as_strided((t.shape[0] * t.shape[1], D), (t.stride(1), 1))
        return t.reshape(-1, D)


# ----------------------------------------------------------------------------------------------------
#  SSD-MIMO scan
# ----------------------------------------------------------------------------------------------------
@dataclass
class ScanGeometry:
    H: int
    R: int
    O: int
    G: int
    N: int


def head_split(B, nc, H, R, precision, device) -> int:
    """How many head ranges a (batch, chunk) of the tensor-core scan is split into: the smallest k in {1, 2, 4, 8}
    dividing H whose grid B * nc * k fills whole waves of one CTA per SM best (one CTA per (batch, chunk) leaves the
    last wave partly empty: 256 CTAs on 148 SMs run as long as 296)."""
    if precision != _lib.PRECISION_IO or device.type != "cuda":
        return 1
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    best, best_eff = 1, 0.0
    for k in (1, 2, 4, 8):
        if H % k:
            continue
        units = B * nc * k
        eff = units / (-(-units // sms) * sms)
        if eff > best_eff + 0.02:
            best, best_eff = k, eff
    return best


def pick_chunk(geo: ScanGeometry, precision: int, backward: bool, limit: int) -> int:
    return int(_lib.load().orbit_ssd_scan_pick_chunk(geo.R, geo.O, geo.G, geo.N, precision, int(backward), int(limit)))


def _tok_stride(who, t, inner):
    """Token stride (elements) of a [B, L, X, N] map whose [X, N] block is contiguous and whose batch stride is L * token stride."""
    if t.dim() == 4 and t.shape[1] == 1 and (t.shape[3] == 1 or t.stride(3) == 1) and (t.shape[2] == 1 or t.stride(2) == t.shape[3]):
        return t.stride(0)                    # one token per batch row: the kernels' (b * L + t) * stride is b * batch stride
    ok = (t.dim() == 4 and (t.shape[3] == 1 or t.stride(3) == 1) and (t.shape[2] == 1 or t.stride(2) == t.shape[3])
          and (t.shape[0] == 1 or t.stride(0) == t.shape[1] * t.stride(1)))
    if not ok:
        raise ValueError(f"{who}: expected [B, L, {inner}, N] with contiguous [{inner}, N] blocks and collapsible (B, L), "
                         f"got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(1)


def run_phase(a, name, phase, state_in, state_out, dtype_code, precision):
    """One phase of the scan through the C-ABI (`a` is the filled argument block; `a.t` names its tensors)."""
    with _timed(name, 2 if (precision == _lib.PRECISION_IO and phase == _lib.PHASE_CHUNK_GRADS and a.R == 1) else 1):
        _lib.check(_lib.load().orbit_ssd_scan_phase(C.byref(a), phase, _ptr(state_in), _ptr(state_out), dtype_code, precision,
                                                    _stream()), "orbit_ssd_scan_phase(" + name + ")")


def cp_pack(dA, record, n_state):
    """Sum the segment's log-decays dA [B, L, H, R] over L into the record behind its state part (`orbit_cp_state_pack`)."""
    B, L, H, R = dA.shape
    lib = _lib.load()
    nbytes = int(lib.orbit_cp_state_pack_workspace_bytes(B, L, H * R))
    ws = torch.empty((max(nbytes, 4),), device=dA.device, dtype=torch.uint8)
    with _timed("cp_state_pack", 2):
        _lib.check(lib.orbit_cp_state_pack(_ptr(dA), _ptr(record), B, L, H * R, int(n_state), _ptr(ws), nbytes, _stream()),
                   "orbit_cp_state_pack")


def cp_combine(records, world, rank, n_state, per_head, BHR, backward):
    """Entering state (forward) or leaving-state gradient (backward) of rank `rank` from the gathered records
    [world, stride] (`orbit_cp_state_combine`).  Returns a flat fp32 tensor of n_state elements."""
    out = torch.empty((n_state,), device=records.device, dtype=torch.float32)
    with _timed("cp_state_combine", 1):
        _lib.check(_lib.load().orbit_cp_state_combine(_ptr(records), records.stride(0), int(world), int(rank), int(n_state),
                                                      int(per_head), int(BHR), int(bool(backward)), _ptr(out), _stream()),
                   "orbit_cp_state_combine")
    return out


class ContextParallel:
    """The ranks of one context-parallel group: consecutive ranks hold consecutive segments of the sequence.

    The recurrence is linear in the state, so a rank needs from its predecessors only what their segments contribute:
    F_j (final state of segment j started from zero) and A_j (its total log-decay per kernel head).  ONE all-gather of
    the packed records (F, A) per direction replaces a serial hand-off, and one small kernel forms
    S_r = sum_{j<r} exp(A_{j+1} + .. + A_{r-1}) F_j  (and the mirror image for the state gradient in backward).  The same
    terms as the reference's in-GPU chunk-parallel pass (src/orbit_ssm/kernels/ssd_mimo/chunkpar.py:19-25) and its state
    continuation contract (src/orbit_ssm/ssm/ssd_mimo_torch.py:677-679).
    """

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def gather_records(self, record):
        """record [stride] fp32 of this rank -> [world, stride], one collective."""
        record = record.contiguous()
        out = torch.empty((self.world * record.numel(),), device=record.device, dtype=record.dtype)
        self.dist.all_gather_into_tensor(out, record, group=self.group)
        return out.view(self.world, record.numel())


class HaloFn(torch.autograd.Function):
    """Conv window of a context-parallel segment: the last W-1 raw rows of the previous rank's segment (zeros on
    rank 0), as a [B, C, W] window whose slot 0 is unused.  Backward returns the window's gradient to its owner."""

    @staticmethod
    def forward(ctx, tail, cp, W):
        # tail [B, W-1, C]: this rank's own last rows, sent to the next rank
        ctx.cp, ctx.W = cp, W
        dist = cp.dist
        tail = tail.contiguous()
        recv = torch.zeros_like(tail)
        reqs = []
        if cp.rank + 1 < cp.world:
            reqs.append(dist.P2POp(dist.isend, tail, dist.get_global_rank(cp.group, cp.rank + 1) if cp.group else cp.rank + 1,
                                   group=cp.group))
        if cp.rank > 0:
            reqs.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(cp.group, cp.rank - 1) if cp.group else cp.rank - 1,
                                   group=cp.group))
        if reqs:
            for r in dist.batch_isend_irecv(reqs):
                r.wait()
        win = tail.new_zeros(tail.shape[0], tail.shape[2], W)
        win[..., 1:] = recv.transpose(1, 2)
        return win

    @staticmethod
    @first_order_only("context-parallel conv halo")
    def backward(ctx, dwin):
        cp, W = ctx.cp, ctx.W
        dist = cp.dist
        send = dwin[..., 1:].transpose(1, 2).contiguous()          # gradient of the previous rank's last rows
        recv = torch.zeros_like(send)
        reqs = []
        if cp.rank > 0:
            reqs.append(dist.P2POp(dist.isend, send, dist.get_global_rank(cp.group, cp.rank - 1) if cp.group else cp.rank - 1,
                                   group=cp.group))
        if cp.rank + 1 < cp.world:
            reqs.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(cp.group, cp.rank + 1) if cp.group else cp.rank + 1,
                                   group=cp.group))
        if reqs:
            for r in dist.batch_isend_irecv(reqs):
                r.wait()
        return recv, None, None


class LagHaloFn(torch.autograd.Function):
    """Trapezoid write across a context-parallel cut.  The scan works on one-tap weights w_t = wd_t + lag_{t+1}: the lagged
    half of token t + 1's write, lag_{t+1} = dt_{t+1} (1 - lam_{t+1}), multiplies the write of token t (reference:
    src/orbit_ssm/ssm/ssd_mimo_torch.py:769-788).  For the last token of a segment, t + 1 is the first token of the NEXT
    rank: every rank sends the lag of its first token [B, H, R] to its predecessor and gets its successor's (zeros on the
    last rank).  Backward returns the gradient to its owner the other way."""

    @staticmethod
    def forward(ctx, lag0, cp):
        ctx.cp = cp
        dist = cp.dist
        lag0 = lag0.contiguous()
        recv = torch.zeros_like(lag0)
        peer = (lambda r: dist.get_global_rank(cp.group, r) if cp.group else r)
        reqs = []
        if cp.rank > 0:
            reqs.append(dist.P2POp(dist.isend, lag0, peer(cp.rank - 1), group=cp.group))
        if cp.rank + 1 < cp.world:
            reqs.append(dist.P2POp(dist.irecv, recv, peer(cp.rank + 1), group=cp.group))
        if reqs:
            for r in dist.batch_isend_irecv(reqs):
                r.wait()
        return recv

    @staticmethod
    @first_order_only("context-parallel trapezoid lag")
    def backward(ctx, dnext):
        cp = ctx.cp
        dist = cp.dist
        send = dnext.contiguous()                      # gradient of the successor's lag, computed here
        recv = torch.zeros_like(send)                  # gradient of this rank's own lag, computed by the predecessor
        peer = (lambda r: dist.get_global_rank(cp.group, r) if cp.group else r)
        reqs = []
        if cp.rank + 1 < cp.world:
            reqs.append(dist.P2POp(dist.isend, send, peer(cp.rank + 1), group=cp.group))
        if cp.rank > 0:
            reqs.append(dist.P2POp(dist.irecv, recv, peer(cp.rank - 1), group=cp.group))
        if reqs:
            for r in dist.batch_isend_irecv(reqs):
                r.wait()
        return recv, None


def scan_fwd(geo, T, precision, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0, cp=None):
    """Forward scan.  Returns (y [B, L, H*G*O], S_fin [B, H, R, N, G] fp32, Sin, atot); with the tensor-core precision
    `Sin` is the pair (None, Sin16): the backward of the rank-1 tiles reads the bfloat16 state tiles only (the fp32 buffer holds
    chunk-local values after the state pass and is dropped); the rank-4 tiles keep the fp32 states.  With `cp` (a `ContextParallel`) the
    segment is continued from its predecessors' segments and S_fin is the state at this segment's end."""
    _require_cuda("ssd_scan_fwd", u, Bhat, Chat, dA)
    B, L = u.shape[:2]
    H, R, O, G, N = geo.H, geo.R, geo.O, geo.G, geo.N
    if T <= 0:
        raise NotImplementedError(f"ssd_scan: no chunk length fits this geometry (R={R} O={O} G={G} N={N}) in shared memory")
    nc = max(1, -(-L // T))
    dev = u.device
    a = _lib.ScanArgs()
    a.B, a.L, a.H, a.R, a.O, a.G, a.N, a.T, a.nc = B, L, H, R, O, G, N, T, (-(-L // T))
    u = u.contiguous()
    y = torch.empty((B, L, H * G * O), device=dev, dtype=u.dtype)
    Sin = torch.empty((B, nc, H, R, N, G), device=dev, dtype=torch.float32)
    atot = torch.empty((B, nc, H, R), device=dev, dtype=torch.float32)
    S_fin = torch.empty((B, H, R, N, G), device=dev, dtype=torch.float32)
    keep = _fill_common(a, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg)
    if u.is_cuda:
        a.Sin, a.atot, a.y = Sin.data_ptr(), atot.data_ptr(), y.data_ptr()
    Sin16 = None
    if precision == _lib.PRECISION_IO and geo.R == 1:    # bf16 state tiles are read by the rank-1 tensor-core kernels only
        Sin16 = torch.empty((B, nc, H, R, N, G), device=dev, dtype=torch.bfloat16)
        a.Sin16 = Sin16.data_ptr()
    a.hsplit = head_split(B, nc, H, R, precision, dev)
    a.t = dict(geo=geo, u=u, Bhat=Bhat, gBp=gBp, Chat=Chat, gCp=gCp, beta=beta, gamma=gamma, chi=chi, dA=dA, w=w, wd=wd,
               Dg=Dg, Sin=Sin, atot=atot, y=y)
    dt = _dtype_code("ssd_scan_fwd", u)
    run_phase(a, "scan_chunk_state", _lib.PHASE_CHUNK_STATE, None, None, dt, precision)
    if cp is not None:
        # this rank's record [F | A]: the dry pass writes F (started from the sequence's initial state on rank 0, from zero
        # elsewhere: an initial state is a property of the whole sequence, so only rank 0's is read) straight into it
        n_state, BHR = S_fin.numel(), B * H * R
        rec = torch.empty((n_state + BHR,), device=dev, dtype=torch.float32)
        first = S0 if cp.rank == 0 else None
        run_phase(a, "scan_state_pass_dry", _lib.PHASE_STATE_PASS_DRY, first, rec[:n_state].view_as(S_fin), dt, precision)
        cp_pack(dA, rec, n_state)
        recs = cp.gather_records(rec)
        S0 = first if cp.rank == 0 else cp_combine(recs, cp.world, cp.rank, n_state, N * G, BHR, False).view_as(S_fin)
    run_phase(a, "scan_state_pass", _lib.PHASE_STATE_PASS, S0, S_fin, dt, precision)
    run_phase(a, "scan_chunk_out", _lib.PHASE_CHUNK_OUT, None, None, dt, precision)
    del keep
    return y, S_fin, (Sin if Sin16 is None else (None, Sin16)), atot


_STATUS = {}


def _status_word(device):
    """Per-device int32 the tensor-core kernels set when one of their bounded waits gives up."""
    key = (device.type, device.index)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_device_status(device=None):
    """Raise if a kernel reported a wait that ran out (synchronises the device; for tests and end-of-run checks)."""
    for key, t in _STATUS.items():
        if int(t.item()) != 0:
            t.zero_()
            raise RuntimeError(f"orbit_b200: a bounded device-side wait gave up on {key}: the outputs of the affected launches "
                               f"are incomplete (ORBIT_ERR_DEVICE_TIMEOUT, status {_lib.ERR_DEVICE_TIMEOUT})")


def _fill_common(a, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg):
    a.u = u.data_ptr()
    if u.is_cuda:
        a.status = _status_word(u.device).data_ptr()
    a.Bhat, a.b_ts = Bhat.data_ptr(), _tok_stride("ssd_scan", Bhat, "R")
    a.Chat, a.c_ts = Chat.data_ptr(), _tok_stride("ssd_scan", Chat, "O")
    if gBp is not None:
        a.gBp, a.gb_ts = gBp.data_ptr(), _tok_stride("ssd_scan", gBp, "R")
    if gCp is not None:
        a.gCp, a.gc_ts = gCp.data_ptr(), _tok_stride("ssd_scan", gCp, "O")
    for name, t in (("beta", beta), ("gamma", gamma), ("chi", chi), ("dA", dA), ("w", w), ("wd", wd), ("Dg", Dg)):
        if t is not None:
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise ValueError(f"ssd_scan: {name} must be contiguous float32")
            setattr(a, name, t.data_ptr())
    return (u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg)


def scan_bwd(geo, T, precision, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, Sin, atot, dy, dS_fin,
             euler, want_dS0, cp=None, hsplit=1):
    """Backward scan.  Returns a dict of gradients (fp32 unless noted): du (IO dtype), dBhat, dgBp, dChat, dgCp, dbeta,
    dgamma, dchi, ddA, dw, dwd, dDg, dS0."""
    B, L = u.shape[:2]
    H, R, O, G, N = geo.H, geo.R, geo.O, geo.G, geo.N
    Sin, Sin16 = Sin if isinstance(Sin, tuple) else (Sin, None)
    nc = (Sin if Sin is not None else Sin16).shape[1]
    dev = u.device
    f32 = dict(device=dev, dtype=torch.float32)
    a = _lib.ScanArgs()
    a.B, a.L, a.H, a.R, a.O, a.G, a.N, a.T, a.nc = B, L, H, R, O, G, N, T, (-(-L // T))
    u = u.contiguous()
    dy = dy.contiguous()
    keep = _fill_common(a, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg)
    out = dict(du=torch.empty_like(u), dBhat=torch.empty((B, L, R, N), **f32), dChat=torch.empty((B, L, O, N), **f32),
               ddA=torch.empty((B, L, H, R), **f32), dw=torch.empty((B, L, H, R), **f32))
    out["dgBp"] = torch.empty((B, L, R, N), **f32) if gBp is not None else None
    out["dgCp"] = torch.empty((B, L, O, N), **f32) if gCp is not None else None
    out["dwd"] = None if euler else torch.empty((B, L, H, R), **f32)
    out["dchi"] = torch.empty((B, L, H, R), **f32) if chi is not None else None
    slots = B * nc
    pb = torch.empty((slots, H, R, R, N), **f32) if beta is not None else None
    pg = torch.empty((slots, H, R, O, N), **f32) if gamma is not None else None
    pd = torch.empty((slots, H, G, R, O), **f32) if Dg is not None else None
    dS = torch.empty((B, nc, H, R, N, G), **f32)
    dS0 = torch.empty((B, H, R, N, G), **f32) if want_dS0 else None
    dS16 = du32 = None
    if precision == _lib.PRECISION_IO and R == 1:        # rank-1 tensor-core tiles read bf16 state tiles by TMA
        dS16 = torch.empty((B, nc, H, R, N, G), device=dev, dtype=torch.bfloat16)
        a.Sin16, a.dS16 = Sin16.data_ptr(), dS16.data_ptr()
    elif precision == _lib.PRECISION_IO:                 # rank-4 tiles sum du over the siblings of a head in fp32
        du32 = torch.empty(u.shape, **f32)
        a.du32 = du32.data_ptr()
    a.Sin = Sin.data_ptr() if Sin is not None else None
    a.atot, a.dS, a.dy, a.du = atot.data_ptr(), dS.data_ptr(), dy.data_ptr(), out["du"].data_ptr()
    a.dBhat, a.dChat, a.ddA, a.dw = (out[k].data_ptr() for k in ("dBhat", "dChat", "ddA", "dw"))
    # The rank-1 gradient kernels keep one CTA per (batch, chunk) by default: their per-CTA epilogue (128 KB of map
    # gradients written, then read and written again) outweighs the wave-quantisation gain of a head split (measured at
    # configs 2 and 5).  The rank-4 kernels walk 4 H kernel heads per CTA, so their epilogue is negligible: they split.
    if precision != _lib.PRECISION_IO:
        a.hsplit = 1
    elif R == 1:
        a.hsplit = int(hsplit) if H % max(int(hsplit), 1) == 0 else 1
    else:
        a.hsplit = head_split(B, nc, H, R, precision, dev) if hsplit == 1 else int(hsplit)
    parts = None
    if a.hsplit > 1:          # every head range writes its own partial of the head-shared map gradients
        k = a.hsplit
        parts = dict(dBhat=torch.empty((k, B, L, R, N), **f32), dChat=torch.empty((k, B, L, O, N), **f32))
        if R > 1:
            if out["dgBp"] is not None:
                parts["dgBp"] = torch.empty((k, B, L, R, N), **f32)
            if out["dgCp"] is not None:
                parts["dgCp"] = torch.empty((k, B, L, O, N), **f32)
        for key, v in parts.items():
            setattr(a, key, v.data_ptr())
    for k in ("dgBp", "dgCp", "dwd", "dchi"):
        if out[k] is not None and not (parts is not None and k in parts):
            setattr(a, k, out[k].data_ptr())
    if pb is not None:
        a.dbeta_part = pb.data_ptr()
    if pg is not None:
        a.dgamma_part = pg.data_ptr()
    if pd is not None:
        a.dDg_part = pd.data_ptr()
    # Euler: one buffer serves both write weights, so the own-token gradient must land in dw as well: the kernel is
    # given separate buffers and the two are summed here.
    dwd_tmp = None
    if euler:
        dwd_tmp = torch.empty((B, L, H, R), **f32)
        a.dwd = dwd_tmp.data_ptr()
    a.t = dict(geo=geo, u=u, Bhat=Bhat, gBp=gBp, Chat=Chat, gCp=gCp, beta=beta, gamma=gamma, chi=chi, dA=dA, w=w, wd=wd,
               Dg=Dg, Sin=Sin, atot=atot, dy=dy, dS=dS, out=out, dbeta_part=pb, dgamma_part=pg, dDg_part=pd,
               dwd=(dwd_tmp if euler else out["dwd"]), du32=du32, dS16=dS16)
    dt = _dtype_code("ssd_scan_bwd", u)
    run_phase(a, "scan_chunk_dstate", _lib.PHASE_CHUNK_DSTATE, None, None, dt, precision)
    if cp is not None:
        # this rank's record [E | A | X]; one all-gather, then the gradient of the state leaving this segment
        n_state, BHR = B * H * R * N * G, B * H * R
        rec = torch.empty((2 * n_state + BHR,), **f32)
        run_phase(a, "scan_state_pass_bwd_dry", _lib.PHASE_STATE_PASS_BWD_DRY, None, rec[:n_state].view(B, H, R, N, G), dt, precision)
        cp_pack(dA, rec, n_state)
        if dS_fin is not None:
            rec[n_state + BHR:].copy_(dS_fin.reshape(-1))
        else:
            rec[n_state + BHR:].zero_()
        recs = cp.gather_records(rec)
        dS_fin = cp_combine(recs, cp.world, cp.rank, n_state, N * G, BHR, True).view(B, H, R, N, G)
    run_phase(a, "scan_state_pass_bwd", _lib.PHASE_STATE_PASS_BWD, dS_fin, dS0, dt, precision)
    run_phase(a, "scan_chunk_grads", _lib.PHASE_CHUNK_GRADS, None, None, dt, precision)
    del keep
    if parts is not None:
        for key, v in parts.items():
            out[key] = v.sum(0)
    if euler:
        out["dw"] = out["dw"] + dwd_tmp
    out["dbeta"] = pb.sum(0) if pb is not None else None
    out["dgamma"] = pg.sum(0) if pg is not None else None
    out["dDg"] = pd.sum(0) if pd is not None else None
    out["dS0"] = dS0
    return out


def scan_step(geo, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0):
    """One token of the scan in one launch (`orbit_ssd_scan_step`; inference only): operands as `scan_fwd` with L = 1.
    Returns (y [B, 1, H*G*O], S_fin [B, H, R, N, G] fp32)."""
    _require_cuda("ssd_scan_step", u, Bhat, Chat, dA)
    B, L = u.shape[:2]
    if L != 1:
        raise ValueError(f"ssd_scan_step: one token per call, got L={L}")
    H, R, O, G, N = geo.H, geo.R, geo.O, geo.G, geo.N
    a = _lib.ScanArgs()
    a.B, a.L, a.H, a.R, a.O, a.G, a.N, a.T, a.nc = B, 1, H, R, O, G, N, 1, 1
    u = u.contiguous()
    y = torch.empty((B, 1, H * G * O), device=u.device, dtype=u.dtype)
    S_fin = torch.empty((B, H, R, N, G), device=u.device, dtype=torch.float32)
    keep = _fill_common(a, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg)
    a.y = y.data_ptr() if y.is_cuda else None
    a.t = dict(geo=geo, u=u, Bhat=Bhat, gBp=gBp, Chat=Chat, gCp=gCp, beta=beta, gamma=gamma, chi=chi, dA=dA, w=w, wd=wd, Dg=Dg, y=y)
    run_step(a, S0, S_fin, _dtype_code("ssd_scan_step", u))
    del keep
    return y, S_fin


def run_step(a, S0, S_fin, dtype_code):
    """The one-token scan launch through the C-ABI (`a.t`: the tensors behind the pointers, for the CPU host-logic tests)."""
    with _timed("scan_step", 1):
        _lib.check(_lib.load().orbit_ssd_scan_step(C.byref(a), _ptr(S0), _ptr(S_fin), dtype_code, _stream()), "orbit_ssd_scan_step")


class SSDScanFn(torch.autograd.Function):
    """The chunked SSD-MIMO scan as one autograd node (state in, state out, exact gradients through both)."""

    @staticmethod
    def forward(ctx, geo, T, precision, euler, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0, cp=None):
        tens = [None if t is None else t.detach() for t in (u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, S0)]
        u_, Bhat_, gBp_, Chat_, gCp_, beta_, gamma_, chi_, dA_, w_, wd_, Dg_, S0_ = tens
        y, S_fin, Sin, atot = scan_fwd(geo, T, precision, u_, Bhat_, gBp_, Chat_, gCp_, beta_, gamma_, chi_, dA_, w_,
                                       w_ if euler else wd_, Dg_, S0_, cp=cp)
        Sin, Sin16 = Sin if isinstance(Sin, tuple) else (Sin, None)
        ctx.save_for_backward(u_, Bhat_, gBp_, Chat_, gCp_, beta_, gamma_, chi_, dA_, w_, wd_, Dg_, Sin, atot, Sin16)
        ctx.cfg = (geo, T, precision, euler, cp)
        ctx.in_dtypes = [None if t is None else t.dtype for t in (u, Bhat, gBp, Chat, gCp)]
        ctx.set_materialize_grads(False)
        return y, S_fin

    @staticmethod
    @first_order_only("SSD-MIMO scan")
    def backward(ctx, dy, dS_fin):
        u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, wd, Dg, Sin, atot, Sin16 = ctx.saved_tensors
        if Sin16 is not None:
            Sin = (Sin, Sin16)
        geo, T, precision, euler, cp = ctx.cfg
        if dy is None:
            dy = torch.zeros((*u.shape[:2], geo.H * geo.G * geo.O), device=u.device, dtype=u.dtype)
        if dS_fin is not None:
            dS_fin = dS_fin.to(torch.float32).contiguous()
        g = scan_bwd(geo, T, precision, u, Bhat, gBp, Chat, gCp, beta, gamma, chi, dA, w, w if euler else wd, Dg, Sin,
                     atot, dy, dS_fin, euler, ctx.needs_input_grad[16], cp=cp)
        dts = ctx.in_dtypes

        def cast(t, dt):
            return None if t is None else t.to(dt)

        return (None, None, None, None, g["du"], cast(g["dBhat"], dts[1]), cast(g["dgBp"], dts[2]),
                cast(g["dChat"], dts[3]), cast(g["dgCp"], dts[4]), g["dbeta"], g["dgamma"], g["dchi"], g["ddA"], g["dw"],
                g["dwd"], g["dDg"], g["dS0"], None)


# ----------------------------------------------------------------------------------------------------
#  token tails (maps and clocks between the input GEMM and the scan)
# ----------------------------------------------------------------------------------------------------
def _row_view(who, t):
    """[B, L, W] tensor with a contiguous last axis whose batch stride equals L * row stride -> (rows M, row stride)."""
    if t.dim() != 3 or (t.shape[-1] > 1 and t.stride(-1) != 1) or (t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1)):
        raise ValueError(f"{who}: expected [B, L, W] rows with uniform row stride, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.shape[0] * t.shape[1], t.stride(1)


def token_map_fwd(src, weight, bias, add, eps, X, N):
    """src [B, L, N*X] (slab columns, (n, x) interleaved) -> (out [B, L, X, N] IO dtype, rstd [B, L, X] | None)."""
    _require_cuda("token_map_fwd", src, weight, bias)
    M, rs = _row_view("token_map_fwd", src)
    B, L = src.shape[:2]
    out = torch.empty((B, L, X, N), device=src.device, dtype=src.dtype)
    rstd = torch.empty((B, L, X), device=src.device, dtype=torch.float32) if weight is not None else None
    with _timed("token_map_fwd", 1 if M else 0):
        _lib.check(_lib.load().orbit_token_map_fwd(_ptr(src), rs, _ptr(weight), _ptr(bias), float(add), float(eps), _ptr(out),
                                                   _ptr(rstd), M, X, N, _dtype_code("token_map_fwd", src), _stream()),
                   "orbit_token_map_fwd")
    return out, rstd


def token_map_bwd(src, weight, rstd, dout, X, N, want_dbias, dsrc_out=None):
    """Returns (dsrc [B, L, N*X], dweight [N] | None, dbias [N] | None); `dsrc_out` receives dsrc in place."""
    _require_cuda("token_map_bwd", src, weight, rstd, dout)
    M, rs = _row_view("token_map_bwd", src)
    dout = dout.contiguous()
    dsrc = dsrc_out if dsrc_out is not None else torch.empty(src.shape, device=src.device, dtype=src.dtype)
    _, drs = _row_view("token_map_bwd", dsrc)
    f32 = dict(device=src.device, dtype=torch.float32)
    dweight = torch.empty((N,), **f32) if weight is not None else None
    dbias = torch.empty((N,), **f32) if want_dbias else None
    lib = _lib.load()
    nbytes = lib.orbit_token_map_bwd_workspace_bytes(N)
    ws = torch.empty((int(nbytes),), device=src.device, dtype=torch.uint8) if (dweight is not None or dbias is not None) else None
    with _timed("token_map_bwd", (2 if ws is not None else 1) if M else 0):
        _lib.check(lib.orbit_token_map_bwd(_ptr(src), rs, _ptr(weight), _ptr(rstd), _ptr(dout), _ptr(dsrc), drs, _ptr(dweight),
                                           _ptr(dbias), _ptr(ws), int(nbytes) if ws is not None else 0, M, X, N,
                                           _dtype_code("token_map_bwd", src), _stream()), "orbit_token_map_bwd")
    return dsrc, dweight, dbias


class TokenMapFn(torch.autograd.Function):
    """out[b, l, x, :] = rmsnorm_N(src[b, l, n*X + x]) * weight + bias + add  (weight / bias optional)."""

    @staticmethod
    def forward(ctx, src, weight, bias, add, eps, X, N, slot=None):
        w32, b32 = _f32(weight), _f32(bias)
        out, rstd = token_map_fwd(src, w32, b32, add, eps, X, N)
        ctx.save_for_backward(src, w32, rstd)
        ctx.meta = (X, N, None if weight is None else weight.dtype, None if bias is None else bias.dtype, slot)
        return out

    @staticmethod
    @first_order_only("token map tail")
    def backward(ctx, dout):
        src, w32, rstd = ctx.saved_tensors
        X, N, wdt, bdt, slot = ctx.meta
        dsrc_out = slot[0].view(slot[1], src) if slot is not None else None
        dsrc, dw, db = token_map_bwd(src, w32, rstd, dout.to(src.dtype), X, N, bdt is not None, dsrc_out=dsrc_out)
        return (dsrc, None if dw is None else dw.to(wdt), None if db is None else db.to(bdt), None, None, None, None, None)


def _fill_clock(a, t):
    dt_raw = t["dt_raw"]
    B, L = dt_raw.shape[:2]
    a.M, a.L, a.H, a.R = B * L, L, t["H"], t["R"]
    a.a_act, a.a_per_sibling = t["a_act"], int(t["a_per_sibling"])
    for key, rs in (("dt_raw", "dt_rs"), ("a_raw", "a_rs"), ("trap_raw", "trap_rs"), ("rmix_raw", "rmix_rs"),
                    ("d_dt_raw", "ddt_rs"), ("d_a_raw", "da_rs"), ("d_trap_raw", "dtrap_rs"), ("d_rmix_raw", "drmix_rs")):
        v = t.get(key)
        if v is not None:
            _, stride = _row_view("token_clock", v)
            setattr(a, rs, stride)
            if v.is_cuda:
                setattr(a, key, v.data_ptr())
    for key in ("A_log", "r_mix", "dA", "w", "wd", "chi", "lag0", "ddA", "dw", "dwd", "dchi", "dlag0", "g_alog", "sum_part",
                "bias_sums"):
        v = t.get(key)
        if v is not None and v.is_cuda:
            setattr(a, key, v.data_ptr())
    if t.get("sum_part") is not None:
        a.sum_part_bytes = t["sum_part"].numel() * t["sum_part"].element_size()
    a.t = t


def run_clock(a, name, backward, dtype_code):
    """One clock-tail launch through the C-ABI (`a.t`: the tensors behind the pointers, for the CPU host-logic tests)."""
    fn = _lib.load().orbit_token_clock_bwd if backward else _lib.load().orbit_token_clock_fwd
    with _timed(name, 1 if a.M else 0):
        _lib.check(fn(C.byref(a), dtype_code, _stream()), name)


def token_clock_fwd(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, a_per_sibling, H, R):
    """Raw slab columns [B, L, .] -> dict(dA, w, wd | None, chi | None, lag0 | None), fp32 [B, L, H, R] ([B, H, R] for lag0)."""
    _require_cuda("token_clock_fwd", dt_raw, a_raw, trap_raw, rmix_raw)
    B, L = dt_raw.shape[:2]
    f32 = dict(device=dt_raw.device, dtype=torch.float32)
    t = dict(dt_raw=dt_raw, a_raw=a_raw, trap_raw=trap_raw, rmix_raw=rmix_raw, A_log=_f32(A_log), r_mix=_f32(r_mix), a_act=a_act,
             a_per_sibling=a_per_sibling, H=H, R=R)
    t["dA"] = torch.empty((B, L, H, R), **f32)
    t["w"] = torch.empty((B, L, H, R), **f32)
    t["wd"] = torch.empty((B, L, H, R), **f32) if trap_raw is not None else None
    t["lag0"] = torch.empty((B, H, R), **f32) if trap_raw is not None else None
    t["chi"] = torch.empty((B, L, H, R), **f32) if r_mix is not None else None
    a = _lib.ClockArgs()
    _fill_clock(a, t)
    run_clock(a, "token_clock_fwd", False, _dtype_code("token_clock_fwd", dt_raw))
    return {k: t[k] for k in ("dA", "w", "wd", "chi", "lag0")}


def token_clock_bwd(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, a_per_sibling, H, R, g, outs=None, bias_sums=False):
    """`g`: dict of gradients ddA, dw, dwd, dchi, dlag0 (None = zero).  Returns dict(dt_raw, a_raw, trap_raw, rmix_raw,
    A_log, r_mix); `outs` may carry in-place destinations for the four raw gradients.  With `bias_sums` the dict also has
    dt_bias [H*R], a_bias ([H*R] or [H], dynamic rate only) and trap_bias ([H], trapezoid only): the sums over rows of the raw
    gradients BEFORE they are rounded to the IO dtype, i.e. the gradients of the slab biases in fp32."""
    B, L = dt_raw.shape[:2]
    dev = dt_raw.device
    f32 = dict(device=dev, dtype=torch.float32)
    outs = outs or {}

    def dest(key, like):
        if like is None:
            return None
        v = outs.get(key)
        return v if v is not None else torch.empty(like.shape, device=dev, dtype=like.dtype)

    def zeros_like_out(v, shape):
        return torch.zeros(shape, **f32) if v is None else v.to(torch.float32).contiguous()

    t = dict(dt_raw=dt_raw, a_raw=a_raw, trap_raw=trap_raw, rmix_raw=rmix_raw, A_log=_f32(A_log), r_mix=_f32(r_mix), a_act=a_act,
             a_per_sibling=a_per_sibling, H=H, R=R)
    t["ddA"] = zeros_like_out(g.get("ddA"), (B, L, H, R))
    t["dw"] = zeros_like_out(g.get("dw"), (B, L, H, R))
    t["dwd"] = None if (trap_raw is None or g.get("dwd") is None) else g["dwd"].to(torch.float32).contiguous()
    t["dchi"] = None if (r_mix is None or g.get("dchi") is None) else g["dchi"].to(torch.float32).contiguous()
    t["dlag0"] = None if (trap_raw is None or g.get("dlag0") is None) else g["dlag0"].to(torch.float32).contiguous()
    t["d_dt_raw"] = dest("dt_raw", dt_raw)
    t["d_a_raw"] = dest("a_raw", a_raw)
    t["d_trap_raw"] = dest("trap_raw", trap_raw)
    t["d_rmix_raw"] = dest("rmix_raw", rmix_raw)
    t["g_alog"] = torch.empty((B, L, H, R), **f32) if a_act == 0 else None
    n_a = 0 if a_act == 0 else (H * R if a_per_sibling else H)
    n_t = H if trap_raw is not None else 0
    if bias_sums:
        nbytes = int(_lib.load().orbit_token_clock_bwd_workspace_bytes(B * L, H, R, int(a_act), int(bool(a_per_sibling)), int(n_t > 0)))
        t["sum_part"] = torch.empty((max(nbytes // 4, 1),), **f32)
        t["bias_sums"] = torch.empty((H * R + n_a + n_t,), **f32)
    a = _lib.ClockArgs()
    _fill_clock(a, t)
    run_clock(a, "token_clock_bwd", True, _dtype_code("token_clock_bwd", dt_raw))
    out = dict(dt_raw=t["d_dt_raw"], a_raw=t["d_a_raw"], trap_raw=t["d_trap_raw"], rmix_raw=t["d_rmix_raw"],
               A_log=None if t["g_alog"] is None else t["g_alog"].sum((0, 1)),
               r_mix=None if t["dchi"] is None else t["dchi"].sum((0, 1)))
    if bias_sums:
        bs = t["bias_sums"]
        out["dt_bias"] = bs[:H * R]
        out["a_bias"] = bs[H * R:H * R + n_a] if n_a else None
        out["trap_bias"] = bs[H * R + n_a:] if n_t else None
    return out


class TokenClockFn(torch.autograd.Function):
    """Clocks of the scan from the raw slab columns; absent outputs (wd, chi, lag0) come back as empty tensors."""

    @staticmethod
    def forward(ctx, dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix, a_act, a_per_sibling, H, R, slots=None,
                dt_bias=None, a_bias=None, trap_bias=None):
        # The three biases are already inside the raw columns (added in the projection's epilogue); they are inputs here only
        # so that their gradients come from this node: the sums of the unrounded raw gradients, not of the rounded slab.
        ctx.bias_meta = [None if b is None else (b.shape, b.dtype) for b in (dt_bias, a_bias, trap_bias)]
        o = token_clock_fwd(dt_raw, a_raw, trap_raw, rmix_raw, None if A_log is None else A_log.detach(),
                            None if r_mix is None else r_mix.detach(), a_act, a_per_sibling, H, R)
        ctx.save_for_backward(dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix)
        ctx.meta = (a_act, a_per_sibling, H, R, slots or {})
        ctx.set_materialize_grads(False)
        empty = o["dA"].new_zeros(0)
        return o["dA"], o["w"], (o["wd"] if o["wd"] is not None else empty), (o["chi"] if o["chi"] is not None else empty), \
            (o["lag0"] if o["lag0"] is not None else empty)

    @staticmethod
    @first_order_only("token clock tail")
    def backward(ctx, ddA, dw, dwd, dchi, dlag0):
        dt_raw, a_raw, trap_raw, rmix_raw, A_log, r_mix = ctx.saved_tensors
        a_act, a_per_sibling, H, R, slots = ctx.meta
        outs = {}
        for key, like in (("dt_raw", dt_raw), ("a_raw", a_raw), ("trap_raw", trap_raw), ("rmix_raw", rmix_raw)):
            if like is not None and key in slots:
                outs[key] = slots[key][0].view(slots[key][1], like)
        want_bias = any(ctx.needs_input_grad[11:14])
        g = token_clock_bwd(dt_raw, a_raw, trap_raw, rmix_raw, None if A_log is None else A_log.detach(),
                            None if r_mix is None else r_mix.detach(), a_act, a_per_sibling, H, R,
                            dict(ddA=ddA, dw=dw, dwd=dwd, dchi=dchi, dlag0=dlag0), outs, bias_sums=want_bias)

        def bias_grad(i, key):
            meta = ctx.bias_meta[i]
            if meta is None or not ctx.needs_input_grad[11 + i] or g.get(key) is None:
                return None
            return g[key].reshape(meta[0]).to(meta[1])
        return (g["dt_raw"], g["a_raw"], g["trap_raw"], g["rmix_raw"],
                None if (A_log is None or g["A_log"] is None) else g["A_log"].reshape(A_log.shape).to(A_log.dtype),
                None if (r_mix is None or g["r_mix"] is None) else g["r_mix"].reshape(r_mix.shape).to(r_mix.dtype),
                None, None, None, None, None, bias_grad(0, "dt_bias"), bias_grad(1, "a_bias"), bias_grad(2, "trap_bias"))


# ----------------------------------------------------------------------------------------------------
#  HybridMamba clock tail (step size, trapezoid weight, angle feature)
# ----------------------------------------------------------------------------------------------------
def hm_tail_fwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K):
    """Slab columns [B, L, .] (IO dtype, any uniform row stride) -> (delta [B, L, H], lam [B, L, H] | None,
    feat [B, L, K] | None), fp32 (`orbit_hm_tail_fwd`)."""
    _require_cuda("hm_tail_fwd", dt_raw, trap_raw, th_raw)
    B, L, H = dt_raw.shape
    f32 = dict(device=dt_raw.device, dtype=torch.float32)
    delta = torch.empty((B, L, H), **f32)
    lam = torch.empty((B, L, H), **f32) if trap_raw is not None else None
    feat = torch.empty((B, L, K), **f32) if th_raw is not None else None
    a = _lib.HmTailArgs()
    a.M, a.H, a.K, a.Krot = B * L, H, K, (0 if th_raw is None else th_raw.shape[-1])
    for key, rs, v in (("dt_raw", "dt_rs", dt_raw), ("trap_raw", "trap_rs", trap_raw), ("th_raw", "th_rs", th_raw)):
        if v is not None:
            setattr(a, rs, _row_view("hm_tail", v)[1])
            setattr(a, key, v.data_ptr())
    keep = [_f32(dt_bias), _f32(trap_bias), _f32(omega), rot_idx]
    a.dt_bias, a.trap_bias, a.omega = _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2])
    a.rot_idx = _ptr(rot_idx) if th_raw is not None else None
    a.delta, a.lam, a.feat = _ptr(delta), _ptr(lam), _ptr(feat)
    with _timed("hm_tail_fwd", 1 if B * L else 0):
        _lib.check(_lib.load().orbit_hm_tail_fwd(C.byref(a), _dtype_code("hm_tail_fwd", dt_raw), _stream()), "orbit_hm_tail_fwd")
    del keep
    return delta, lam, feat


def hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K, lam, ddelta, dlam, dfeat):
    """Returns (d dt_raw, d trap_raw | None, d th_raw | None) in the IO dtype and (d dt_bias, d trap_bias | None,
    d omega | None) fp32 (`orbit_hm_tail_bwd`); a missing upstream gradient counts as zero."""
    _require_cuda("hm_tail_bwd", dt_raw, trap_raw, th_raw)
    B, L, H = dt_raw.shape
    dev, io = dt_raw.device, dt_raw.dtype
    f32 = dict(device=dev, dtype=torch.float32)
    Krot = 0 if th_raw is None else th_raw.shape[-1]
    d_dt = torch.empty((B, L, H), device=dev, dtype=io)
    d_trap = torch.empty((B, L, H), device=dev, dtype=io) if trap_raw is not None else None
    d_th = torch.empty((B, L, Krot), device=dev, dtype=io) if th_raw is not None else None
    g_dtb = torch.empty((H,), **f32)
    g_trb = torch.empty((H,), **f32) if trap_raw is not None else None
    g_om = torch.empty((Krot,), **f32) if th_raw is not None else None
    lib = _lib.load()
    nbytes = int(lib.orbit_hm_tail_bwd_workspace_bytes(B * L, H, Krot))
    ws = torch.empty((max(nbytes, 4),), device=dev, dtype=torch.uint8)
    a = _lib.HmTailArgs()
    a.M, a.H, a.K, a.Krot = B * L, H, K, Krot
    for key, rs, v in (("dt_raw", "dt_rs", dt_raw), ("trap_raw", "trap_rs", trap_raw), ("th_raw", "th_rs", th_raw),
                       ("d_dt_raw", "d_dt_rs", d_dt), ("d_trap_raw", "d_trap_rs", d_trap), ("d_th_raw", "d_th_rs", d_th)):
        if v is not None:
            setattr(a, rs, _row_view("hm_tail", v)[1])
            setattr(a, key, v.data_ptr())
    keep = [_f32(dt_bias), _f32(trap_bias), _f32(omega), rot_idx] + [None if g is None else _f32(g).contiguous() for g in (ddelta, dlam, dfeat)]
    a.dt_bias, a.trap_bias, a.omega = _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2])
    a.rot_idx = _ptr(rot_idx) if th_raw is not None else None
    a.lam = _ptr(lam)
    a.ddelta, a.dlam, a.dfeat = _ptr(keep[4]), _ptr(keep[5]), _ptr(keep[6])
    a.d_dt_bias, a.d_trap_bias, a.d_omega = _ptr(g_dtb), _ptr(g_trb), _ptr(g_om)
    a.part, a.part_bytes = _ptr(ws), nbytes
    with _timed("hm_tail_bwd", 2 if B * L else 0):
        _lib.check(lib.orbit_hm_tail_bwd(C.byref(a), _dtype_code("hm_tail_bwd", dt_raw), _stream()), "orbit_hm_tail_bwd")
    del keep
    return d_dt, d_trap, d_th, g_dtb, g_trb, g_om


class HMTailFn(torch.autograd.Function):
    """Clocks and angle feature of the HybridMamba scan as one node: (dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega)
    -> (delta, lam, feat); reference: src/orbit_ssm/ssm/hybrid_mamba.py:1890-1931, 971-1000."""

    @staticmethod
    def forward(ctx, dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K):
        delta, lam, feat = hm_tail_fwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, K)
        ctx.save_for_backward(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, lam)
        ctx.K = K
        ctx.set_materialize_grads(False)
        return delta, lam, feat

    @staticmethod
    @first_order_only("HybridMamba clock tail")
    def backward(ctx, ddelta, dlam, dfeat):
        dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, lam = ctx.saved_tensors
        d_dt, d_trap, d_th, g_dtb, g_trb, g_om = hm_tail_bwd(dt_raw, trap_raw, th_raw, dt_bias, trap_bias, omega, rot_idx, ctx.K,
                                                             lam, ddelta, dlam, dfeat)

        def like(g, p):
            return None if (g is None or p is None) else g.to(p.dtype)
        return (d_dt, d_trap, d_th, like(g_dtb, dt_bias), like(g_trb, trap_bias), like(g_om, omega), None, None)


# ----------------------------------------------------------------------------------------------------
#  HybridMamba coordinate-decay scan
# ----------------------------------------------------------------------------------------------------
def run_hm(a, name, backward, dtype_code):
    """One HybridMamba scan launch through the C-ABI.  `a.t` carries the tensors behind the pointers (the CPU host-logic
    tests replace this function with a torch restatement that reads and fills them)."""
    fn = _lib.load().orbit_hm_scan_bwd if backward else _lib.load().orbit_hm_scan_fwd
    with _timed(name, 1):
        _lib.check(fn(C.byref(a), dtype_code, _stream()), name)


_HM_IN = ("x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "rot", "theta_h", "lam", "D", "h_init",
          "write_prev", "theta_init")


def _hm_fill(a, t):
    x = t["x"]
    B, L, H, P = x.shape
    N = t["A_log"].shape[-1]
    a.B, a.L, a.H, a.P, a.N = B, L, H, P, N
    a.Tc = _lib.HM_CHUNK
    a.nck = -(-L // a.Tc)
    if x.is_cuda:
        for k in _HM_IN:
            if t.get(k) is not None:
                setattr(a, k, t[k].data_ptr())
    a.t = t


def hm_scan_fwd(x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, rot, theta_h, lam, D, h_init, write_prev, theta_init):
    """Forward of the coordinate-decay scan.  x [B, L, H, P] (IO dtype); delta, lam [B, L, H]; A_log [H, P, N];
    Bh, Ch [B, L, N]; feat [B, L, N/2]; rot uint8 [N/2]; theta_h [H, N/2]; D [H]; carries h_init / write_prev
    [B, H, P, N], theta_init [B, H, N/2] (fp32; None = zero).  Returns (y [B, L, H, P], h_final, theta_final or None,
    write_last, saved) with `saved` = (hck, thck), the chunk-entering states the backward replays from."""
    _require_cuda("hm_scan", x, delta, A_log, Bh, Ch)
    B, L, H, P = x.shape
    N = A_log.shape[-1]
    K = N // 2
    dev = x.device
    f32 = dict(device=dev, dtype=torch.float32)
    t = dict(x=x.contiguous(), delta=_f32(delta), A_log=_f32(A_log), Bh=_f32(Bh), Ch=_f32(Ch), beta_b=_f32(beta_b),
             beta_c=_f32(beta_c), feat=_f32(feat), rot=rot, theta_h=_f32(theta_h), lam=_f32(lam), D=_f32(D),
             h_init=_f32(h_init), write_prev=_f32(write_prev), theta_init=_f32(theta_init))
    a = _lib.HmArgs()
    _hm_fill(a, t)
    t["y"] = torch.empty_like(t["x"])
    t["h_final"] = torch.empty((B, H, P, N), **f32)
    t["theta_final"] = torch.empty((B, H, K), **f32) if feat is not None else None
    t["write_last"] = torch.empty((B, H, P, N), **f32)
    t["hck"] = torch.empty((B, H, a.nck, P, N), **f32)
    t["thck"] = torch.empty((B, H, a.nck, K), **f32) if feat is not None else None
    if x.is_cuda:
        for k in ("y", "h_final", "theta_final", "write_last", "hck", "thck"):
            if t[k] is not None:
                setattr(a, k, t[k].data_ptr())
    run_hm(a, "hm_scan_fwd", False, _dtype_code("hm_scan", x))
    return t["y"], t["h_final"], t["theta_final"], t["write_last"], (t["hck"], t["thck"])


def hm_scan_bwd(x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, rot, theta_h, lam, D, h_init, write_prev, theta_init,
                saved, dy, dh_final, dtheta_final, dwrite_last):
    """Backward of the coordinate-decay scan: a dict of gradients keyed like the forward's arguments (fp32; dx in the IO
    dtype).  Sums over batch (parameters) and heads (shared maps) of the kernel's partial buffers are taken here."""
    B, L, H, P = x.shape
    N = A_log.shape[-1]
    K = N // 2
    dev = x.device
    f32 = dict(device=dev, dtype=torch.float32)
    hck, thck = saved
    t = dict(x=x.contiguous(), delta=_f32(delta), A_log=_f32(A_log), Bh=_f32(Bh), Ch=_f32(Ch), beta_b=_f32(beta_b),
             beta_c=_f32(beta_c), feat=_f32(feat), rot=rot, theta_h=_f32(theta_h), lam=_f32(lam), D=_f32(D),
             h_init=_f32(h_init), write_prev=_f32(write_prev), theta_init=_f32(theta_init))
    a = _lib.HmArgs()
    _hm_fill(a, t)
    t.update(hck=hck, thck=thck, dy=dy.contiguous(), dh_final=_f32(dh_final), dtheta_final=_f32(dtheta_final),
             dwrite_last=_f32(dwrite_last))
    t["dx"] = torch.empty_like(t["x"])
    t["ddelta"] = torch.empty((B, L, H), **f32)
    t["dlam"] = torch.empty((B, L, H), **f32) if lam is not None else None
    t["dA_log_part"] = torch.empty((B, H, P, N), **f32)
    t["dBh_part"] = torch.empty((H, B, L, N), **f32)
    t["dCh_part"] = torch.empty((H, B, L, N), **f32)
    t["dbeta_b_part"] = torch.empty((B, H, N), **f32) if beta_b is not None else None
    t["dbeta_c_part"] = torch.empty((B, H, N), **f32) if beta_c is not None else None
    t["dfeat_part"] = torch.empty((H, B, L, K), **f32) if feat is not None else None
    t["dtheta_h_part"] = torch.empty((B, H, K), **f32) if theta_h is not None else None
    t["dD_part"] = torch.empty((B, H), **f32) if D is not None else None
    t["dh_init"] = torch.empty((B, H, P, N), **f32)
    t["dwrite_prev"] = torch.empty((B, H, P, N), **f32) if lam is not None else None
    t["dtheta_init"] = torch.empty((B, H, K), **f32) if feat is not None else None
    if x.is_cuda:
        for k in ("hck", "thck", "dy", "dh_final", "dtheta_final", "dwrite_last", "dx", "ddelta", "dlam", "dA_log_part",
                  "dBh_part", "dCh_part", "dbeta_b_part", "dbeta_c_part", "dfeat_part", "dtheta_h_part", "dD_part",
                  "dh_init", "dwrite_prev", "dtheta_init"):
            if t[k] is not None:
                setattr(a, k, t[k].data_ptr())
    run_hm(a, "hm_scan_bwd", True, _dtype_code("hm_scan", x))

    def s0(v):
        return None if v is None else v.sum(0)

    return dict(x=t["dx"], delta=t["ddelta"], A_log=t["dA_log_part"].sum(0), Bh=t["dBh_part"].sum(0), Ch=t["dCh_part"].sum(0),
                beta_b=s0(t["dbeta_b_part"]), beta_c=s0(t["dbeta_c_part"]), feat=s0(t["dfeat_part"]),
                theta_h=s0(t["dtheta_h_part"]), lam=t["dlam"], D=s0(t["dD_part"]), h_init=t["dh_init"],
                write_prev=t["dwrite_prev"], theta_init=t["dtheta_init"])


class HMScanFn(torch.autograd.Function):
    """The coordinate-decay scan as one autograd node: carries in (h_init, write_prev, theta_init), carries out
    (h_final, theta_final, write_last), exact gradients through all of them."""

    @staticmethod
    def forward(ctx, rot, x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, theta_h, lam, D, h_init, write_prev, theta_init):
        ins = [None if v is None else v.detach() for v in
               (x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, theta_h, lam, D, h_init, write_prev, theta_init)]
        x_, delta_, A_, Bh_, Ch_, bb_, bc_, feat_, thh_, lam_, D_, h0_, wp_, th0_ = ins
        y, hN, thN, wl, saved = hm_scan_fwd(x_, delta_, A_, Bh_, Ch_, bb_, bc_, feat_, rot, thh_, lam_, D_, h0_, wp_, th0_)
        ctx.save_for_backward(*ins, saved[0], saved[1])
        ctx.rot = rot
        ctx.in_dtypes = [None if v is None else v.dtype for v in
                         (x, delta, A_log, Bh, Ch, beta_b, beta_c, feat, theta_h, lam, D, h_init, write_prev, theta_init)]
        ctx.set_materialize_grads(False)
        if thN is None:
            thN = x.new_zeros((), dtype=torch.float32)
        return y, hN, thN, wl

    @staticmethod
    @first_order_only("HybridMamba scan")
    def backward(ctx, dy, dhN, dthN, dwl):
        *ins, hck, thck = ctx.saved_tensors
        x, delta, A_log, Bh, Ch, bb, bc, feat, thh, lam, D, h0, wp, th0 = ins
        if dy is None:
            dy = torch.zeros_like(x)
        if feat is None:
            dthN = None
        g = hm_scan_bwd(x, delta, A_log, Bh, Ch, bb, bc, feat, ctx.rot, thh, lam, D, h0, wp, th0, (hck, thck), dy.to(x.dtype),
                        dhN, dthN, dwl)
        keys = ("x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "theta_h", "lam", "D", "h_init", "write_prev",
                "theta_init")
        out = []
        for k, v, dt in zip(keys, ins, ctx.in_dtypes):
            gv = g[k] if v is not None else None
            out.append(None if gv is None else gv.to(dt))
        return (None, *out)
