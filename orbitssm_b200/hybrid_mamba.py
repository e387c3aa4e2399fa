"""`HybridMambaSSM`: the HybridMamba layer on the sm_100a kernels of this package (`backend="cuda"`).

Interface, parameter names and shapes, State keys and refusals follow the reference's layer
(src/orbit_ssm/ssm/hybrid_mamba.py:2613-2870 layer, 440-935 scan core), so a reference ``state_dict`` loads here and
the two produce the same numbers.  One call:

    x [B, L, d_model] -- one GEMM --> drive | gate z | token slab (clock | B,C | angle | trapezoid)
    drive -- depthwise causal conv + SiLU (CUDA) --> x_t [B, L, H, P]
    slab  -- clock softplus, B/C RMSNorm, angle feature, trapezoid sigmoid (fp32) --> delta, Bh, Ch, feat, lam
    coordinate-decay scan (CUDA, `ops.HMScanFn`) --> y [B, L, H, P], carries (hidden_state, theta, write_prev)
    y * silu(z) (-> RMSNorm) (CUDA) --> out_proj

Everything is token-major (the reference keeps the drive channel-major; layouts inside the layer are this package's
choice).  Served: ``coord_static`` row blocks, real or rotating pairs; see `config.resolve_hm_spec` for the refusals.
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .config import BACKENDS, Execution, HybridMambaConfig, as_execution, resolve_hm_spec
from .ssd_mimo import _OutNorm, _init_dt_bias, _next_window
from .state import State, StateLifecycle

FREQ_INIT = 3.8          # raw pair frequency: omega = pi tanh(3.8) = 0.999 pi (reference: layers/init.py:49)


class HybridMambaSSM(StateLifecycle, nn.Module):
    """HybridMamba layer; see the module docstring.  ``HybridMambaSSM(config, execution=None)``."""

    config_family = "hybrid_mamba"

    def __init__(self, config, execution=None):
        nn.Module.__init__(self)
        if isinstance(config, dict):
            config = HybridMambaConfig.from_dict(config)
        if not isinstance(config, HybridMambaConfig):
            raise TypeError(f"config must be a HybridMambaConfig or its dict, got {type(config).__name__}")
        self.config = config
        s = self.spec = resolve_hm_spec(config)
        H, P, N = s.H, s.P, s.N
        self.d_model, self.d_inner, self.d_conv, self.H, self.P, self.N = s.d_model, s.d_inner, s.d_conv, H, P, N
        self.d_state, self.out_width = N, s.d_inner
        d_sel = s.d_model
        # Parameter creation follows the reference's order (hybrid_mamba.py:2647-2675, 660-930) so that the same torch
        # seed draws the same weights.
        self.in_proj = nn.Linear(s.d_model, 2 * s.d_inner, bias=False)
        self.conv1d = (nn.Conv1d(s.d_inner, s.d_inner, kernel_size=s.d_conv, groups=s.d_inner, padding=s.d_conv - 1,
                                 bias=True) if s.d_conv > 0 else None)
        if s.dt_rank is not None:
            self.dt_low = nn.Linear(d_sel, s.dt_rank, bias=False)
            self.dt_proj = nn.Linear(s.dt_rank, H, bias=False)
        else:
            self.dt_low = None
            self.dt_proj = nn.Linear(d_sel, H, bias=False)
        if s.dt_init is not None:
            std = self.dt_proj.in_features ** -0.5 * s.dt_scale
            if s.dt_init == "constant":
                nn.init.constant_(self.dt_proj.weight, std)
            else:
                nn.init.uniform_(self.dt_proj.weight, -std, std)
        self.dt_bias = nn.Parameter(_init_dt_bias(H, s.dt_min, s.dt_max, s.dt_init_floor))
        self.dt_bias._no_weight_decay = True
        self.bc_proj = nn.Linear(d_sel, 2 * N, bias=False)
        self.b_norm = nn.RMSNorm(N, eps=s.norm_eps) if s.b_norm else None
        self.c_norm = nn.RMSNorm(N, eps=s.norm_eps) if s.c_norm else None
        self.beta_b = nn.Parameter(torch.zeros(H, N)) if s.bc_bias else None
        self.beta_c = nn.Parameter(torch.zeros(H, N)) if s.bc_bias else None
        # one stored decay per real row and per rotating pair (reference: hybrid_mamba.py:700-735)
        A = torch.tensor(s.ladder, dtype=torch.float32).repeat(H, P, 1)
        self.A_log = nn.Parameter(torch.log(A))
        self.A_log._no_weight_decay = True
        if s.has_rot:
            self.theta_proj = nn.Linear(d_sel, len(s.rot_pairs), bias=False)
            if s.learn_theta_freq:
                self.theta_freq = nn.Parameter(torch.full((len(s.rot_pairs),), FREQ_INIT))
                self.theta_freq._no_weight_decay = True
            if s.use_theta_h:
                self.theta_h = nn.Parameter(torch.zeros(H, len(s.rot_pairs)))
                self.theta_h._no_weight_decay = True
                self.register_buffer("theta_h_convention", torch.tensor(1, dtype=torch.int64), persistent=True)
        else:
            self.theta_proj = None
        if s.use_trap:
            self.trap_proj = nn.Linear(d_sel, H, bias=True)
            nn.init.zeros_(self.trap_proj.bias)
        else:
            self.trap_proj = None
        self.register_buffer("proj_source_code", torch.tensor(1, dtype=torch.int64), persistent=True)   # 1 = "layer_input"
        if s.skip:
            self.D = nn.Parameter(torch.ones(H))
            self.D._no_weight_decay = True
        else:
            self.D = None
        self.norm = _OutNorm(s.d_inner, s.norm_eps) if s.out_norm else nn.Identity()
        self.out_proj = nn.Linear(s.d_inner, s.d_model, bias=False)

        self.register_buffer("a_log_idx", torch.tensor(s.a_idx, dtype=torch.long), persistent=False)
        self.register_buffer("rot_pair_idx", torch.tensor(s.rot_pairs, dtype=torch.long), persistent=False)
        rot = torch.zeros(max(s.K, 1), dtype=torch.uint8)
        if s.rot_pairs:
            rot[torch.tensor(s.rot_pairs)] = 1
        self.register_buffer("rot_mask", rot, persistent=False)
        # token slab: clock | B,C | angle | trapezoid (reference order: hybrid_mamba.py:1609-1610)
        self._slab = [("dt", self.dt_low if self.dt_low is not None else self.dt_proj), ("bc", self.bc_proj)]
        if s.has_rot:
            self._slab.append(("theta", self.theta_proj))
        if s.use_trap:
            self._slab.append(("trap", self.trap_proj))
        self.tok_width = sum(m.weight.shape[0] for _, m in self._slab)
        self._proj_pad = (-(2 * s.d_inner + self.tok_width)) % 8
        self.backend, self.kernel_options = "cuda", {}
        self._route_note = None
        self._final_state = None
        self.set_execution(as_execution(execution))

    # -- execution (reference: hybrid_mamba.py:2574-2580) ------------------------------------------------------
    def _check_execution(self, ex: Execution) -> dict:
        f, out = ex.fields(), {}
        if "backend" in f:
            if f["backend"] not in BACKENDS:
                raise ValueError(f"HybridMambaSSM: backend must be one of {BACKENDS} (this package is the CUDA backend), "
                                 f"got {f['backend']!r}")
            out["backend"] = f["backend"]
        if f.get("precision") is not None:
            raise ValueError("HybridMambaSSM: precision is not an option of this layer (the scan runs in fp32)")
        if f.get("chunk_size") not in (None, "auto"):
            raise ValueError("HybridMambaSSM: chunk_size must be 'auto'")
        if "kernel_options" in f:
            if not isinstance(f["kernel_options"], dict):
                raise TypeError("HybridMambaSSM: kernel_options must be a dict")
            if f["kernel_options"]:
                raise ValueError(f"HybridMambaSSM: unknown kernel option(s) {sorted(f['kernel_options'])}; this backend has none")
            out["kernel_options"] = {}
        return out

    def set_execution(self, execution):
        out = self._check_execution(as_execution(execution))
        for k, v in out.items():
            setattr(self, k, v)
        return self

    @contextlib.contextmanager
    def execution(self, execution):
        old = Execution(backend=self.backend, kernel_options=dict(self.kernel_options))
        self.set_execution(execution)
        try:
            yield self
        finally:
            self.set_execution(old)

    def last_route(self):
        return self._route_note

    # -- state (reference: hybrid_mamba.py:2866-2880; keys hidden_state, theta, write_prev, conv_state) ---------
    def _init_state(self, batch_size, device=None, dtype=None):
        dev = device if device is not None else next(self.parameters()).device
        if dtype is None:
            dtype = self._default_state_dtype()
        s = self.spec
        st = State(hidden_state=torch.zeros(batch_size, s.H, s.P, s.N, device=dev, dtype=dtype))
        if s.has_rot:
            # the running phase is held in fp32 at least, whatever dtype the other carries take
            st["theta"] = torch.zeros(batch_size, s.H, len(s.rot_pairs), device=dev,
                                      dtype=torch.promote_types(dtype, torch.float32))
        if s.use_trap:
            st["write_prev"] = torch.zeros_like(st["hidden_state"])
        if self.conv1d is not None:
            st["conv_state"] = torch.zeros(batch_size, s.d_inner, s.d_conv, device=dev, dtype=dtype)
        return st

    def hidden_state_shape(self):
        return (self.H, self.P, self.N)

    # -- fused projection ----------------------------------------------------------------------------------------
    def tok_proj_weight(self):
        """Packed token-projection weight [tok_width, d_model] (reference: hybrid_mamba.py:1633-1641)."""
        return torch.cat([m.weight for _, m in self._slab], 0)

    def _fused_weight(self, dtype):
        parts = [self.in_proj.weight, self.tok_proj_weight()]
        if self._proj_pad:
            parts.append(parts[0].new_zeros(self._proj_pad, self.d_model))
        return torch.cat(parts, 0).to(dtype)

    def _rot_idx32(self, device):
        """Row-pair index of each rotating pair as int32 on `device` (what the clock-tail kernel scatters by)."""
        t = getattr(self, "_rot_idx32_cache", None)
        if t is None or t.device != device:
            t = self.rot_pair_idx.to(device=device, dtype=torch.int32).contiguous()
            self._rot_idx32_cache = t
        return t

    def _maps(self, slab, io):
        """Scan operands from the slab columns (reference: hybrid_mamba.py:1695-1740, 1950-2013, 971-1011); fp32."""
        s = self.spec
        f = torch.float32
        keys = [key for key, _ in self._slab]
        cols = ops.SplitColumnsFn.apply(slab, None, *[m.weight.shape[0] for _, m in self._slab])
        out = dict(zip(keys, cols))
        dt_lin = out["dt"]
        if self.dt_low is not None:
            dt_lin = F.linear(dt_lin, self.dt_proj.weight.to(io))
        # clocks and angle feature in the clock-tail kernel (fp32 out); the rotation rate omega is a [Krot] parameter map
        om = None
        if s.has_rot:
            om = (math.pi * torch.tanh(self.theta_freq.to(f)) if s.learn_theta_freq
                  else torch.full((len(s.rot_pairs),), math.pi, dtype=f, device=slab.device))
        delta, lam, feat = ops.HMTailFn.apply(dt_lin, out["trap"] if s.use_trap else None, out["theta"] if s.has_rot else None,
                                              self.dt_bias, self.trap_proj.bias if s.use_trap else None, om,
                                              self._rot_idx32(slab.device) if s.has_rot else None, s.K)
        # B / C maps: RMSNorm over the N state rows in the token-tail kernel (IO dtype out, like the drive)
        Braw, Craw = out["bc"][..., :s.N], out["bc"][..., s.N:]
        Bh = (ops.TokenMapFn.apply(Braw, self.b_norm.weight, None, 0.0, s.norm_eps, 1, s.N, None).squeeze(2)
              if self.b_norm is not None else Braw.to(f))
        Ch = (ops.TokenMapFn.apply(Craw, self.c_norm.weight, None, 0.0, s.norm_eps, 1, s.N, None).squeeze(2)
              if self.c_norm is not None else Craw.to(f))
        th_h = None
        if s.has_rot and s.use_theta_h:
            # the scan rotates the read map by Theta + offset with the offset in its own frame: -theta_h
            th_h = delta.new_zeros(s.H, s.K).index_copy(-1, self.rot_pair_idx, -self.theta_h.to(f))
        return delta, Bh, Ch, feat, th_h, lam

    # -- forward --------------------------------------------------------------------------------------------------
    #: `forward` takes the block's residual stream and returns ``residual + mixer(x)`` (added in the output GEMM's epilogue)
    fused_residual = True

    def forward(self, x, *, state=None, return_state=False, _residual=None):
        """x [B, L, d_model] -> y [B, L, d_model], or (y, State) with ``return_state=True``; ``state`` continues a
        previous call (reference: hybrid_mamba.py:2706-2830)."""
        if x.dim() != 3 or x.shape[-1] != self.d_model:
            raise ValueError(f"HybridMambaSSM: expected x of shape [B, L, {self.d_model}], got {tuple(x.shape)}")
        if not ops.on_device(x):
            raise ValueError("HybridMambaSSM(backend='cuda'): got a CPU tensor; this backend runs on a CUDA device only "
                             "(use the reference's backend='torch' on CPU)")
        s = self.spec
        Bsz, L, _ = x.shape
        if L == 0:
            raise ValueError("HybridMambaSSM: empty sequence")
        if state is not None:
            state = self.resolve_state(state, batch_size=Bsz, device=x.device)
        io = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        if io not in (torch.float32, torch.bfloat16):
            raise NotImplementedError(f"HybridMambaSSM(backend='cuda'): IO dtype must be float32 or bfloat16, got {io}")
        f = torch.float32
        with torch.autocast("cuda", enabled=False):
            xa = x.to(io)
            proj = ops.ProjectFn.apply(xa, None, self._proj_pad, None, 0, self.in_proj.weight, *[m.weight for _, m in self._slab])
            arena = ops.GradArena()        # conv and gate backward write d(drive), dz straight into d(proj)
            drive_raw, z, slab = ops.SplitColumnsFn.apply(proj, arena, s.d_inner, s.d_inner, self.tok_width)
            new = State()
            if self.conv1d is not None:
                win = state["conv_state"] if state is not None else None
                u = ops.CausalConvFn.apply(drive_raw, self.conv1d.weight, self.conv1d.bias, win, (arena, 0))
                if return_state:
                    new["conv_state"] = _next_window(win, drive_raw, s.d_conv)
            else:
                u = drive_raw.contiguous()
            delta, Bh, Ch, feat, th_h, lam = self._maps(slab, io)
            h0 = state["hidden_state"].to(f) if state is not None else None
            wp = state["write_prev"].to(f) if (state is not None and s.use_trap) else None
            th0 = None
            if state is not None and s.has_rot:
                th0 = h0.new_zeros(Bsz, s.H, s.K).index_copy(-1, self.rot_pair_idx, state["theta"].to(f))
            A_log = self.A_log.to(f)[..., self.a_log_idx]
            y, hN, thN, wl = ops.HMScanFn.apply(
                self.rot_mask if s.has_rot else None, u.reshape(Bsz, L, s.H, s.P), delta, A_log, Bh, Ch,
                None if self.beta_b is None else self.beta_b.to(f), None if self.beta_c is None else self.beta_c.to(f),
                feat, th_h, lam, None if self.D is None else self.D.to(f), h0, wp, th0)
            self._route_note = "fp32 coordinate scan"
            y = ops.GateNormFn.apply(y.reshape(Bsz, L, s.d_inner), z, self.norm.weight if s.out_norm else None, s.norm_eps,
                                     (arena, 1))
            fuse = _residual is not None and _residual.dtype == io and _residual.shape == x.shape
            out = ops.ProjectFn.apply(y, _residual if fuse else None, 0, None, 0, self.out_proj.weight)
            if _residual is not None and not fuse:
                out = _residual + out
        if not return_state:
            return out
        new["hidden_state"] = hN
        if s.has_rot:
            new["theta"] = thN.index_select(-1, self.rot_pair_idx)
        if s.use_trap:
            new["write_prev"] = wl
        ordered = State({k: new[k] for k in self._state_schema() if k in new})
        ordered = self._conform_carries(ordered, state)
        self._final_state = ordered
        return out, ordered

    def step(self, x_t, state=None):
        """One token: ``x_t [B, d_model]``, ``state`` from `init_state` or a previous call -> ``(y_t [B, d_model], State)``
        (reference: hybrid_mamba.py:2876).  Runs the layer on a length-1 sequence: the same kernels and the same carry contract as
        `forward`, so a sequence stepped token by token equals the sequence run at once; there is no separate decode
        kernel (a step costs the layer's launch count)."""
        if x_t.dim() != 2 or x_t.shape[-1] != self.d_model:
            raise ValueError(f"HybridMambaSSM.step: expected x_t of shape [B, {self.d_model}], got {tuple(x_t.shape)}")
        if state is None:
            state = self.init_state(x_t.shape[0], device=x_t.device)
        y, new = self.forward(x_t.unsqueeze(1), state=state, return_state=True)
        return y.squeeze(1), new
