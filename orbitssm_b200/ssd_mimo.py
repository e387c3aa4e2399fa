"""`SSDMimoSSM`: the SSD-MIMO layer behind ``backend="cuda"`` on B200.

Same construction, call signature, parameter names/shapes (``state_dict`` interchanges with the reference layer) and
recurrent-`State` contract as the reference's `SSDMimoSSM` (reference: src/orbit_ssm/ssm/ssd_mimo.py:4145-4658), with
the hot path on hand-written sm_100a kernels reached through the C-ABI library:

    x -> [one GEMM: drive | gate z | token slab] -> causal conv + SiLU (drive; B|C when ``bc_conv``)
      -> token law (maps, clocks, decay, write weights) -> chunked SSD-MIMO scan (+ D skip)
      -> gate y*silu(z) (+ RMSNorm when ``out_norm``) -> out_proj

The two projections are library GEMMs (cuBLAS through torch); everything between them is this package's CUDA.
There is no CPU route and no other backend here: a CPU tensor is refused by name.
"""
from __future__ import annotations

import contextlib
import math
import warnings

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, ops
from .config import BACKENDS, PRECISIONS, Execution, SSDMimoConfig, as_execution, resolve_ssd_spec
from .state import State, StateLifecycle


def _init_dt_bias(n, dt_min, dt_max, floor):
    """softplus(bias) log-uniform in [dt_min, dt_max] (reference: src/orbit_ssm/layers/init.py:58-71)."""
    lo, hi = math.log(dt_min), math.log(dt_max)
    dt = torch.exp(torch.rand(n) * (hi - lo) + lo).clamp(min=floor)
    return dt + torch.log(-torch.expm1(-dt))


def _bc_bias_init(shape, mode, R, N):
    """"ones", or sibling r offset along the r-th DCT-II row (reference: ssd_mimo.py:501-516)."""
    base = torch.ones(shape)
    if mode == "ones" or len(shape) < 4 or R < 2:
        return base
    r_off = torch.linspace(0.0, math.log(2.0), R)
    k = torch.arange(R).float()[:, None]
    n = torch.arange(N).float()[None, :]
    dct = torch.cos(math.pi * k * (n + 0.5) / N)
    return base + (r_off[:, None] * dct)[None, :, :, None]


class NonTensorCoreRouteWarning(UserWarning):
    """A bf16 ``precision="io"`` layer ran its scan on the fp32 kernels because its geometry is outside the tcgen05
    tile envelopes (the reason is in the message and in ``last_route()``)."""


_WARNED_ROUTES = set()


def _warn_fp32_route(reason):
    """No silent demotion (reference rule: src/orbit_ssm/layers/routes.py:33-48): say once per reason that a layer asked
    for the tensor-core precision and got the fp32 kernels, which are one to two orders of magnitude slower."""
    if reason in _WARNED_ROUTES:
        return
    _WARNED_ROUTES.add(reason)
    warnings.warn(f"SSDMimoSSM: precision='io' with bf16 activations asks for the tcgen05 scan kernels, but {reason}; the scan "
                  "runs on the fp32 kernels instead (much slower).  Adapt the config to a tensor-core envelope "
                  "(R = O = 1, N = 128, G = 64 with head-shared maps; or R = O = 4, N = 128, G = 16), or set "
                  "precision='ieee' to ask for the fp32 kernels.", NonTensorCoreRouteWarning, stacklevel=4)


class _BCConv(nn.Module):
    """Holder that gives the B|C conv its reference parameter names ``bc_conv1d.conv.{weight,bias}``."""

    def __init__(self, channels, d_conv):
        super().__init__()
        self.conv = nn.Conv1d(channels, channels, kernel_size=d_conv, groups=channels, padding=d_conv - 1, bias=True)


def _pass_min(x, lo):
    return torch.where(x >= lo, x, x.clamp_min(lo).detach())


def _pass_max(x, hi):
    return torch.where(x <= hi, x, x.clamp_max(hi).detach())


class SSDMimoSSM(StateLifecycle, nn.Module):
    """SSD-MIMO layer; see the module docstring.  ``SSDMimoSSM(config, execution=None)``."""

    config_family = "ssd_mimo"

    def __init__(self, config, execution=None):
        nn.Module.__init__(self)
        if isinstance(config, dict):
            config = SSDMimoConfig.from_dict(config)
        if not isinstance(config, SSDMimoConfig):
            raise TypeError(f"config must be an SSDMimoConfig or its dict, got {type(config).__name__}")
        self.config = config
        s = self.spec = resolve_ssd_spec(config)
        H, G, R, O, N = s.H, s.G, s.R, s.O, s.N
        self.d_model, self.d_inner, self.d_conv, self.d_out, self.d_gate = s.d_model, s.d_inner, s.d_conv, s.d_out, s.d_out
        self.H, self.P, self.G, self.R, self.O, self.N = H, s.P, G, R, O, N
        d_sel = s.d_model

        # Parameter creation follows the reference's order (ssd_mimo.py:4278-4306, 646-856) so that the same
        # torch seed draws the same weights.
        self.in_proj = nn.Linear(s.d_model, 2 * s.d_inner, bias=False)
        self.conv1d = (nn.Conv1d(s.d_inner, s.d_inner, kernel_size=s.d_conv, groups=s.d_inner, padding=s.d_conv - 1,
                                 bias=True) if s.d_conv > 0 else None)
        if s.skip:
            shape = {"input_output": (H, G, R, O), "channel": (H, G, R), "head": (H,)}[s.skip_sharing]
            self.D = nn.Parameter(torch.ones(shape))
            self.D._no_weight_decay = True
        if s.r_mix_mode != "none":
            self.r_mix = nn.Parameter(torch.full((H, R), 1.0 / R))
            if s.r_mix_dyn:
                self.r_mix_proj = nn.Linear(d_sel, H * R, bias=False)
                nn.init.zeros_(self.r_mix_proj.weight)
        self.B_proj = nn.Linear(d_sel, N * R, bias=False)
        self.C_proj = nn.Linear(d_sel, N * O, bias=False)
        self.bc_conv1d = _BCConv(N * R + N * O, s.d_conv) if s.bc_conv else None
        if s.use_g_b:
            self.gB_proj = nn.Linear(d_sel, N * R, bias=False)
            nn.init.zeros_(self.gB_proj.weight)
        if s.use_g_c:
            self.gC_proj = nn.Linear(d_sel, N * O, bias=False)
            nn.init.zeros_(self.gC_proj.weight)
        self.dt_proj = nn.Linear(d_sel, H * R, bias=True)
        with torch.no_grad():
            self.dt_proj.bias.copy_(_init_dt_bias(H * R, s.dt_min, s.dt_max, s.dt_init_floor))
        self.dt_proj.bias._no_reinit = True
        if s.a_dyn:
            self.a_dyn_proj = nn.Linear(d_sel, H * R if s.a_dyn_per_sibling else H, bias=s.a_proj_bias)
            if self.a_dyn_proj.bias is not None:
                nn.init.zeros_(self.a_dyn_proj.bias)
                self.a_dyn_proj.bias._no_weight_decay = True
        else:
            r_off = torch.linspace(0.0, math.log(2.0), R)
            hbase = torch.exp(torch.linspace(math.log(0.05), math.log(2.0), H))
            self.A_log = nn.Parameter((hbase[:, None] * torch.exp(r_off)[None, :]).log())
            self.A_log._no_weight_decay = True
        if s.b_norm:
            self.B_norm = nn.RMSNorm(N, eps=s.map_eps)
        if s.c_norm:
            self.C_norm = nn.RMSNorm(N, eps=s.map_eps)
        if s.bc_bias:
            bshape = {"shared": (N,), "head": (H, R, N, R)}[s.bias_gran]
            cshape = {"shared": (N,), "head": (H, R, N, O)}[s.bias_gran]
            self.B_bias = nn.Parameter(_bc_bias_init(bshape, s.bc_bias_init, R, N))
            self.C_bias = nn.Parameter(_bc_bias_init(cshape, s.bc_bias_init, R, N))
        self.register_buffer("pair_layout_code", torch.tensor(0, dtype=torch.int64), persistent=True)
        if s.use_trap:
            self.trap_proj = nn.Linear(d_sel, H, bias=s.trap_proj_bias)
            if self.trap_proj.bias is not None:
                nn.init.zeros_(self.trap_proj.bias)
        if self.d_gate != s.d_inner:
            self.in_proj = nn.Linear(s.d_model, s.d_inner + self.d_gate, bias=False)
        self.norm = _OutNorm(self.d_out, s.norm_eps) if s.out_norm else nn.Identity()
        self.out_proj = nn.Linear(self.d_out, s.d_model, bias=False)

        self.tok_width = s.tok_width
        # column ranges of the slab as the forward splits them (B | C kept together when they share a conv)
        pk = [(k, w) for k, _, w, _ in s.slab]
        if s.bc_conv:
            pk = [("BC", pk[0][1] + pk[1][1])] + pk[2:]
        self._part_keys, self._part_widths = tuple(k for k, _ in pk), tuple(w for _, w in pk)
        self._proj_keys = tuple(k for k, _, _, _ in s.slab)
        self._proj_attrs = tuple(a for _, a, _, _ in s.slab)
        self._proj_widths = tuple(w for _, _, w, _ in s.slab)
        # fused projection width padded so every column slice stays 16-byte aligned in bf16 and fp32
        self._proj_total = s.d_inner + self.d_gate + s.tok_width
        self._proj_pad = (-self._proj_total) % 8

        self.backend, self.precision, self.chunk_size, self.kernel_options = "cuda", "io", "auto", {}
        self._route_note = None
        #: opt-in: read the device status word at the end of every forward (one host synchronisation per call) and raise if
        #: a bounded device-side wait of the tensor-core kernels gave up (ORBIT_ERR_DEVICE_TIMEOUT); `check_device_status()`
        #: does the same on demand, e.g. once per training step
        self.check_waits = False
        self._final_state = None
        self._cp = None
        self.set_execution(as_execution(execution))

    def set_context_parallel(self, group="world"):
        """Split the SEQUENCE across the ranks of `group` (a torch.distributed process group; "world" = the default
        group; None switches it off): rank r's `forward` then takes the r-th contiguous segment of the sequence and
        returns that segment's outputs.  The chunk state and the conv windows cross ranks inside the layer, forward
        and backward.  A `state` passed to `forward` is the state BEFORE the whole sequence: rank 0 reads it, the other
        ranks' is ignored; the State a rank returns is the one at the end of its own segment (the last rank's is the
        sequence's).  No counterpart in the reference, which is single-process; the exchanged quantities are those
        of its State continuation contract (reference: src/orbit_ssm/ssm/ssd_mimo.py:4377-4400, 4565)."""
        if group is None:
            self._cp = None
        else:
            self._cp = ops.ContextParallel(None if group == "world" else group)
        return self

    # -- execution (reference: ssd_mimo.py:4196-4244, execution.py:111-167) --------------------------------
    def _check_execution(self, ex: Execution) -> dict:
        f, out = ex.fields(), {}
        if "backend" in f:
            if f["backend"] not in BACKENDS:
                raise ValueError(f"SSDMimoSSM: backend must be one of {BACKENDS} (this package is the CUDA backend; the "
                                 f"reference's 'torch' / 'sequential' routes are its own), got {f['backend']!r}")
            out["backend"] = f["backend"]
        if "precision" in f:
            if f["precision"] not in PRECISIONS:
                raise ValueError(f"SSDMimoSSM: precision must be one of {PRECISIONS}, got {f['precision']!r}")
            out["precision"] = f["precision"]
        if "chunk_size" in f:
            c = f["chunk_size"]
            if c != "auto" and (isinstance(c, bool) or not isinstance(c, int) or c < 16 or c & (c - 1)):
                raise ValueError(f"SSDMimoSSM: chunk_size must be 'auto' or a power of two >= 16, got {c!r}")
            out["chunk_size"] = c
        if f.get("checkpoint"):
            raise ValueError("SSDMimoSSM: checkpoint=True is refused (the layer has no activation checkpointing)")
        if "kernel_options" in f:
            if not isinstance(f["kernel_options"], dict):
                raise TypeError("SSDMimoSSM: kernel_options must be a dict")
            if f["kernel_options"]:
                raise ValueError(f"SSDMimoSSM: unknown kernel option(s) {sorted(f['kernel_options'])}; this backend has none")
            out["kernel_options"] = {}
        return out

    def set_execution(self, execution):
        out = self._check_execution(as_execution(execution))      # validate everything before changing anything
        for k, v in out.items():
            setattr(self, k, v)
        return self

    @contextlib.contextmanager
    def execution(self, execution):
        old = Execution(backend=self.backend, precision=self.precision, chunk_size=self.chunk_size,
                        kernel_options=dict(self.kernel_options))
        self.set_execution(execution)
        try:
            yield self
        finally:
            self.set_execution(old)

    @staticmethod
    def check_device_status():
        """Raise `RuntimeError` (ORBIT_ERR_DEVICE_TIMEOUT) if a tensor-core kernel launched since the last check reported a
        bounded wait that ran out: its outputs are incomplete.  Synchronises the device."""
        ops.check_device_status()

    def last_route(self):
        """Which scan kernels the last forward used ("tcgen05" or "fp32"), and why when it was not the first."""
        return self._route_note

    # -- state ---------------------------------------------------------------------------------------------
    def _init_state(self, batch_size, device=None, dtype=None):
        dev = device if device is not None else next(self.parameters()).device
        if dtype is None:
            dtype = self._default_state_dtype()
        st = State(hidden_state=torch.zeros(batch_size, self.H, self.P, self.N, device=dev, dtype=dtype))
        if self.spec.use_trap:
            st["write_prev"] = torch.zeros_like(st["hidden_state"])
        if self.bc_conv1d is not None:
            st["bc_conv_state"] = torch.zeros(batch_size, self.N * self.R + self.N * self.O, self.d_conv, device=dev,
                                              dtype=dtype)
        if self.conv1d is not None:
            st["conv_state"] = torch.zeros(batch_size, self.d_inner, self.d_conv, device=dev, dtype=dtype)
        return st

    def hidden_state_shape(self):
        return (self.H, self.P, self.N)

    # -- fused projection weights --------------------------------------------------------------------------
    def tok_proj_weight(self):
        """Packed token-projection weight [tok_width, d_model] and bias (reference: ssd_mimo.py:1050-1085)."""
        ws = [getattr(self, a).weight for a in self._proj_attrs]
        bs = []
        for a, wd_ in zip(self._proj_attrs, self._proj_widths):
            b = getattr(self, a).bias
            bs.append(b if b is not None else ws[0].new_zeros(wd_))
        return torch.cat(ws, 0), torch.cat(bs, 0)

    def _tok_bias(self):
        """Bias of the token slab columns (zeros where a map has none), or None when no map has one."""
        if all(getattr(self, a).bias is None for a in self._proj_attrs):
            return None
        ref = getattr(self, self._proj_attrs[0]).weight
        return torch.cat([getattr(self, a).bias if getattr(self, a).bias is not None else ref.new_zeros(wd_)
                          for a, wd_ in zip(self._proj_attrs, self._proj_widths)], 0)

    def _fused_weight(self, dtype):
        wt, bt = self.tok_proj_weight()
        parts_w = [self.in_proj.weight, wt]
        parts_b = [bt.new_zeros(self.d_inner + self.d_gate), bt]
        if self._proj_pad:
            parts_w.append(wt.new_zeros(self._proj_pad, self.d_model))
            parts_b.append(bt.new_zeros(self._proj_pad))
        return torch.cat(parts_w, 0).to(dtype), torch.cat(parts_b, 0).to(dtype)

    # -- token law (reference: ssd_mimo_torch.py:161-267, 769-788) ----------------------------------------------
    def _token_law(self, parts, b_src, c_src, io, arena=None, slot_of=None):
        """Per-token operands of the scan from the slab columns (`parts`: key -> column view).  Maps and clocks run in the
        token-tail kernels (fp32 arithmetic; maps handed to the scan in the IO dtype; clocks, decays, weights fp32)."""
        s = self.spec
        H, R, O, N = s.H, s.R, s.O, s.N
        f = torch.float32
        slot_of = slot_of or {}

        def slot(key):
            return (arena, slot_of[key]) if (arena is not None and key in slot_of) else None

        def base_map(src, key, X, norm, bias):
            plain = not (norm is not None or bias is not None)
            if X == 1 and plain:
                return src.unsqueeze(2)                                       # [B, L, 1, N] view of the source columns
            return ops.TokenMapFn.apply(src, None if norm is None else norm.weight, bias, 0.0, s.map_eps, X, N,
                                        slot(key) if src is parts.get(key) else None)

        shared = s.bc_bias and not s.head_bias
        Bhat = base_map(b_src, "B", R, self.B_norm if s.b_norm else None, self.B_bias if shared else None)
        Chat = base_map(c_src, "C", O, self.C_norm if s.c_norm else None, self.C_bias if shared else None)
        gBp = ops.TokenMapFn.apply(parts["gB"], None, None, 1.0, s.map_eps, R, N, slot("gB")) if s.use_g_b else None
        gCp = ops.TokenMapFn.apply(parts["gC"], None, None, 1.0, s.map_eps, O, N, slot("gC")) if s.use_g_c else None
        beta = self.B_bias.to(f).transpose(-1, -2).contiguous() if s.head_bias else None       # [H, R, q, N]
        gamma = self.C_bias.to(f).transpose(-1, -2).contiguous() if s.head_bias else None      # [H, R, o, N]

        a_act = 0 if not s.a_dyn else (1 if s.a_act == "heavy_tail" else 2)
        rmix_raw = parts.get("rmix") if (s.r_mix_mode != "none" and s.r_mix_dyn) else None
        slots = {k2: slot(k) for k, k2 in (("dt", "dt_raw"), ("a", "a_raw"), ("trap", "trap_raw"), ("rmix", "rmix_raw"))
                 if slot(k) is not None}
        # the clock node also owns the gradients of the slab biases (the projection got them detached): it sums the raw
        # gradients before they are rounded into the slab gradient
        dA, w, wd_, chi, lag0 = ops.TokenClockFn.apply(
            parts["dt"], parts.get("a") if s.a_dyn else None, parts.get("trap") if s.use_trap else None, rmix_raw,
            None if s.a_dyn else self.A_log, self.r_mix if s.r_mix_mode != "none" else None, a_act,
            bool(s.a_dyn and s.a_dyn_per_sibling), H, R, slots, self.dt_proj.bias,
            self.a_dyn_proj.bias if s.a_dyn else None, self.trap_proj.bias if s.use_trap else None)
        if not s.use_trap:
            wd_, lag0 = None, None
        if s.r_mix_mode == "none":
            chi = None
        Dg = None
        if s.skip:
            D = self.D.to(f)
            if s.skip_sharing == "head":
                Dg = D[:, None, None, None].expand(H, s.G, R, O)
            elif s.skip_sharing == "channel":
                Dg = D[..., None].expand(H, s.G, R, O)
            else:
                Dg = D
            Dg = Dg.contiguous()
        return dict(Bhat=Bhat, Chat=Chat, gBp=gBp, gCp=gCp, beta=beta, gamma=gamma, dA=dA, w=w, wd=wd_, chi=chi, Dg=Dg, lag0=lag0)

    # -- forward -------------------------------------------------------------------------------------------
    #: `forward` takes the block's residual stream and returns ``residual + mixer(x)`` (added in the output GEMM's epilogue)
    fused_residual = True

    def forward(self, x, *, state=None, return_state=False, _residual=None):
        """x [B, L, d_model] -> y [B, L, d_model], or (y, State) with ``return_state=True``; ``state`` continues a
        previous call (reference: ssd_mimo.py:4367-4400)."""
        if x.dim() != 3 or x.shape[-1] != self.d_model:
            raise ValueError(f"SSDMimoSSM: expected x of shape [B, L, {self.d_model}], got {tuple(x.shape)}")
        if not ops.on_device(x):
            raise ValueError("SSDMimoSSM(backend='cuda'): got a CPU tensor; this backend runs on a CUDA device only "
                             "(use the reference's backend='torch' on CPU)")
        s = self.spec
        Bsz, L, _ = x.shape
        H, G, R, O, N, P = s.H, s.G, s.R, s.O, s.N, s.P
        cp = self._cp if (self._cp is not None and self._cp.world > 1) else None
        if cp is not None:
            if L < max(s.d_conv, 1):
                raise ValueError(f"SSDMimoSSM: a context-parallel segment needs at least d_conv={s.d_conv} tokens")
        if state is not None:
            state = self.resolve_state(state, batch_size=Bsz, device=x.device)
            if "write_prev" in state and not s.use_trap:
                raise ValueError("state carry 'write_prev' with write_rule='euler'")
        io = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        if io not in (torch.float32, torch.bfloat16):
            raise NotImplementedError(f"SSDMimoSSM(backend='cuda'): IO dtype must be float32 or bfloat16, got {io}")
        want_state = return_state
        with torch.autocast("cuda", enabled=False):
            xa = x.to(io)
            # [B, L, drive | z | slab | pad]: one GEMM over the parameters themselves (cast once into the IO dtype)
            tok_bias = self._tok_bias()                  # dt / a / trap biases: their gradients come from the clock node
            proj = ops.ProjectFn.apply(xa, None, self._proj_pad, None if tok_bias is None else tok_bias.detach(),
                                       s.d_inner + self.d_gate, self.in_proj.weight,
                                       *[getattr(self, a).weight for a in self._proj_attrs])
            # every consumer of a column range writes that range of d(proj) in place (conv, gate, token tails)
            arena = ops.GradArena()
            keys, widths = self._part_keys, self._part_widths
            drive_raw, z, *cols = ops.SplitColumnsFn.apply(proj, arena, s.d_inner, self.d_gate, *widths)
            parts = dict(zip(keys, cols))
            slot_of = {k: 2 + i for i, k in enumerate(keys)}
            new = State()
            if self.conv1d is not None:
                win = state["conv_state"] if state is not None else None
                if cp is not None:
                    win = _cp_window(win, ops.HaloFn.apply(drive_raw[:, L - (s.d_conv - 1):], cp, s.d_conv), cp)
                u = (ops.CausalConvFn.apply(drive_raw, self.conv1d.weight, self.conv1d.bias, win, (arena, 0)) if L > 0
                     else drive_raw.contiguous())
                if want_state:
                    new["conv_state"] = _next_window(win, drive_raw, s.d_conv)
            else:
                u = drive_raw.contiguous()
            wb, wc = s.slab_off["B"][1], s.slab_off["C"][1]
            if self.bc_conv1d is not None:
                bc_raw = parts["BC"]                                           # B | C adjacent at the slab head
                win = state["bc_conv_state"] if state is not None else None
                if cp is not None:
                    win = _cp_window(win, ops.HaloFn.apply(bc_raw[:, L - (s.d_conv - 1):], cp, s.d_conv), cp)
                bc = (ops.CausalConvFn.apply(bc_raw, self.bc_conv1d.conv.weight, self.bc_conv1d.conv.bias, win,
                                             (arena, slot_of["BC"])) if L > 0
                      else bc_raw.contiguous())
                if want_state:
                    new["bc_conv_state"] = _next_window(win, bc_raw, s.d_conv)
                b_src, c_src = ops.SplitColumnsFn.apply(bc, None, wb, wc)
            else:
                b_src, c_src = parts["B"], parts["C"]

            h0 = state["hidden_state"] if state is not None else None
            wp = state.get("write_prev") if state is not None else None
            if cp is not None and cp.rank > 0:
                h0 = wp = None            # an initial State belongs to the whole sequence: only rank 0 reads it
            if L == 0:
                y = u.new_zeros(Bsz, 0, self.d_out)
                hidden = h0.to(torch.float32) if h0 is not None else u.new_zeros(Bsz, H, P, N, dtype=torch.float32)
                v_last = wp.to(torch.float32) if wp is not None else torch.zeros_like(hidden)
            else:
                law = self._token_law(parts, b_src, c_src, io, arena, slot_of)
                if cp is not None and s.use_trap:
                    # two-endpoint write across the cut: the lagged half of the next segment's first write rides on this
                    # segment's last token (its own lag0 goes to the previous rank the same way)
                    nxt = ops.LagHaloFn.apply(law["lag0"], cp)
                    last = torch.tensor([L - 1], device=nxt.device)
                    law["w"] = law["w"].index_add(1, last, nxt.unsqueeze(1))
                S0 = None
                if h0 is not None:
                    S0 = h0.to(torch.float32).reshape(Bsz, H, G, R, N).permute(0, 1, 3, 4, 2)
                    if wp is not None:
                        S0 = S0 + wp.to(torch.float32).reshape(Bsz, H, G, R, N).permute(0, 1, 3, 4, 2) \
                            * law["lag0"][..., None, None]
                    S0 = S0.contiguous()
                geo = ops.ScanGeometry(H=H, R=R, O=O, G=G, N=N)
                if L == 1 and cp is None and not torch.is_grad_enabled():
                    # decode: the one-token law in one launch (no chunk tiles, no state pass)
                    self._route_note = "step"
                    y, S_fin = ops.scan_step(geo, u, law["Bhat"], law["gBp"], law["Chat"], law["gCp"], law["beta"], law["gamma"],
                                             law["chi"], law["dA"], law["w"], law["w"] if not s.use_trap else law["wd"],
                                             law["Dg"], S0)
                else:
                    precision, T = self._route(io, geo, torch.is_grad_enabled())
                    y, S_fin = ops.SSDScanFn.apply(geo, T, precision, not s.use_trap, u, law["Bhat"], law["gBp"], law["Chat"],
                                                   law["gCp"], law["beta"], law["gamma"], law["chi"], law["dA"], law["w"],
                                                   law["wd"], law["Dg"], S0, cp)
                hidden = S_fin.permute(0, 1, 4, 2, 3).reshape(Bsz, H, P, N)
                v_last = None
                if want_state and s.use_trap:
                    v_last = self._last_write(u, law, Bsz)
            y = ops.GateNormFn.apply(y, z, self.norm.weight if s.out_norm else None, s.norm_eps, (arena, 1)) if L > 0 else y
            fuse = _residual is not None and _residual.dtype == io and _residual.shape == x.shape
            out = ops.ProjectFn.apply(y, _residual if fuse else None, 0, None, 0, self.out_proj.weight)
            if _residual is not None and not fuse:
                out = _residual + out
        if self.check_waits:
            ops.check_device_status()
        if not want_state:
            return out
        new["hidden_state"] = hidden
        if s.use_trap:
            new["write_prev"] = v_last
        ordered = State({k: new[k] for k in self._state_schema() if k in new})
        ordered = self._conform_carries(ordered, state)
        self._final_state = ordered
        return out, ordered

    def _route(self, io, geo, needs_grad):
        lib = _lib.load()
        limit = 64 if self.chunk_size == "auto" else int(self.chunk_size)
        s = self.spec
        shared_maps = not (s.use_g_b or s.use_g_c or s.head_bias or s.r_mix_mode != "none")
        if self.precision == "io" and io == torch.bfloat16:
            # rank-1 tiles serve head-shared maps only; rank-4 tiles take gates, per-head biases and the sibling mix
            rank1 = geo.R == 1 and geo.O == 1
            T = ops.pick_chunk(geo, _lib.PRECISION_IO, needs_grad, 128 if self.chunk_size == "auto" else limit) \
                if (shared_maps or not rank1) else 0
            if T > 0:
                self._route_note = "tcgen05"
                return _lib.PRECISION_IO, T
            why = (f"geometry R={geo.R} O={geo.O} G={geo.G} N={geo.N} is outside the tensor-core tiles" if (shared_maps or not rank1)
                   else "the rank-1 tiles serve head-shared maps only (no gates, per-head biases or sibling mix)")
            self._route_note = f"fp32 ({why})"
            _warn_fp32_route(why)
        else:
            self._route_note = "fp32"
        T = ops.pick_chunk(geo, _lib.PRECISION_IEEE, needs_grad, limit)
        if T <= 0:
            raise NotImplementedError(
                f"SSDMimoSSM: the fp32 scan kernels cannot hold one token of this geometry in shared memory "
                f"(R={geo.R} O={geo.O} G={geo.G} N={geo.N}); reduce d_state or the head width")
        return _lib.PRECISION_IEEE, T

    def _last_write(self, u, law, Bsz):
        """write_prev carry: vtil at the last token, [B, H, P, N] (reference: ssd_mimo_torch.py:789-792)."""
        s = self.spec
        f = torch.float32
        Bl = law["Bhat"][:, -1].to(f)                                          # [B, q, N]
        Bt = Bl[:, None, None]                                                 # [B, 1, 1, q, N]
        if law["gBp"] is not None:
            Bt = law["gBp"][:, -1].to(f)[:, None, :, None, :] * Bt             # [B, 1, r, q, N]
        if law["beta"] is not None:
            Bt = Bt + law["beta"]
        Bt = Bt.expand(Bsz, s.H, s.R, s.R, s.N)
        ul = u[:, -1].to(f).reshape(Bsz, s.H, s.G, s.R)
        return torch.einsum("bhgq,bhrqn->bhgrn", ul, Bt).reshape(Bsz, s.H, s.P, s.N)

    def step(self, x_t, state=None):
        """One token: ``x_t [B, d_model]``, ``state`` from `init_state` or a previous call -> ``(y_t [B, d_model], State)``
        (reference: ssd_mimo.py:4629, ssd_mimo_torch.py:388-490).  Runs the layer on a length-1 sequence with the same carry
        contract as `forward`, so a sequence stepped token by token equals the sequence run at once.  Under
        ``torch.no_grad()`` (decoding) the scan of the token is the one-launch step kernel; with gradients enabled it is the
        chunked scan on a one-token chunk."""
        if x_t.dim() != 2 or x_t.shape[-1] != self.d_model:
            raise ValueError(f"SSDMimoSSM.step: expected x_t of shape [B, {self.d_model}], got {tuple(x_t.shape)}")
        if state is None:
            raise ValueError("SSDMimoSSM.step: `state` is required (start from layer.init_state(batch_size))")
        y, new = self.forward(x_t.unsqueeze(1), state=state, return_state=True)
        return y.squeeze(1), new


class _OutNorm(nn.Module):
    """Parameter holder for the output RMSNorm (``norm.weight``); the arithmetic runs in the fused gate+norm kernel."""

    def __init__(self, d, eps):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d))


def _cp_window(carried, halo, cp):
    """Conv window of a context-parallel segment: the previous rank's last rows (`halo`); on rank 0, where the halo is zero,
    the window carried in by the caller's State (an initial state belongs to the whole sequence: only rank 0's is read).
    The sum keeps rank 0's halo in the autograd graph, so that its backward still receives what rank 1 sends."""
    if carried is None or cp.rank != 0:
        return halo
    return carried.to(halo.dtype) + halo


def _next_window(prev, raw, W):
    """The carried window after this call: the last W raw inputs [B, C, W], index -1 newest, left-filled from the
    previous window (zeros at sequence start).  Differentiable (reference: ssd_mimo.py:4585-4591)."""
    Bsz, L, Cc = raw.shape
    cur = raw.transpose(1, 2)
    if L >= W:
        return cur[..., L - W:]
    if prev is None:
        prev = raw.new_zeros(Bsz, Cc, W)
    return torch.cat([prev.to(raw.dtype), cur], dim=-1)[..., -W:]
