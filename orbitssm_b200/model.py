"""Residual containers around a mixer: `ResidualBlock` (``x + mixer(norm(x))``) and `BlockStack` (blocks, then a final
RMSNorm), with per-layer State lists (reference: src/orbit_ssm/model.py:51-118 and 150-255).  The pre-norms run on
this package's gate + RMSNorm kernels with no gate (one kernel forward, one backward plus the weight-gradient column
sum).  Only mixer-only blocks (``d_mlp = 0``) are built.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import ops
from .config import as_execution


class RMSNorm(nn.Module):
    """``weight * x * rsqrt(mean(x^2) + eps)`` in the input dtype, fp32 accumulation and fp32 weight (reference:
    src/orbit_ssm/layers/norms.py:10-58, the ``fused=True`` form the backbone norms use)."""

    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d))

    def forward(self, x):
        return ops.GateNormFn.apply(x, None, self.weight, self.eps)


class ResidualBlock(nn.Module):
    def __init__(self, mixer, d_model, d_mlp=0):
        super().__init__()
        if d_mlp:
            raise NotImplementedError("ResidualBlock: the SwiGLU sublayer (d_mlp > 0) is outside this package")
        self.norm = RMSNorm(d_model)
        self.mixer = mixer
        self.d_mlp = 0
        out_proj = getattr(mixer, "out_proj", None)
        if isinstance(out_proj, nn.Linear):
            out_proj.weight._normalize_w_num_layers = True       # residual-out tag (reference: layers/init.py:118-160)

    n_residuals = 1

    def forward(self, x, state=None, return_state=False):
        fused = getattr(self.mixer, "fused_residual", False)      # this package's mixers add the residual in their output GEMM
        if state is None and not return_state:
            return self.mixer(self.norm(x), _residual=x) if fused else x + self.mixer(self.norm(x))
        if fused:
            y, state = self.mixer(self.norm(x), state=state, return_state=True, _residual=x)
        else:
            y, state = self.mixer(self.norm(x), state=state, return_state=True)
            y = x + y
        return (y, state) if return_state else y

    def step(self, x_t, state=None):
        """One token through the block: ``x_t [B, d_model]`` -> ``(x_t + mixer.step(norm(x_t)), State)`` (reference:
        src/orbit_ssm/model.py:110-115).  A missing `state` starts from zero carries."""
        if state is None:
            state = self.init_state(x_t.shape[0], device=x_t.device)
        y_t, state = self.mixer.step(self.norm(x_t), state)
        return x_t + y_t, state

    def init_state(self, batch_size, **kw):
        return self.mixer.init_state(batch_size, **kw)

    def validate_state(self, state, **kw):
        return self.mixer.validate_state(state, **kw)


class BlockStack(nn.Module):
    def __init__(self, blocks, d_model, *, residual_rescale=True):
        super().__init__()
        self.layers = nn.ModuleList(blocks)
        self.norm_f = RMSNorm(d_model)
        self.residual_rescale = bool(residual_rescale)
        if self.residual_rescale and len(self.layers):
            n = sum(getattr(b, "n_residuals", 1) for b in self.layers)
            for p in self.parameters():                           # GPT-2 style depth rescale of tagged weights
                if getattr(p, "_normalize_w_num_layers", False):
                    nn.init.kaiming_uniform_(p, a=math.sqrt(5))
                    with torch.no_grad():
                        p.div_(math.sqrt(n))

    @classmethod
    def from_mixers(cls, mixers, d_model, d_mlp=0, *, residual_rescale=True):
        return cls([ResidualBlock(m, d_model, d_mlp) for m in mixers], d_model, residual_rescale=residual_rescale)

    @property
    def ssm_layers(self):
        return tuple(b.mixer for b in self.layers)

    def set_execution(self, execution):
        for m in self.ssm_layers:           # validate every target before changing any
            m._check_execution(as_execution(execution))
        for m in self.ssm_layers:
            m.set_execution(execution)
        return self

    def init_state(self, batch_size, **kw):
        return [b.init_state(batch_size, **kw) for b in self.layers]

    def step(self, x_t, state=None):
        """One token through every block and the final norm: ``x_t [B, d_model]`` -> ``(y_t, [State per layer])``."""
        states = list(state) if state is not None else [None] * len(self.layers)
        if len(states) != len(self.layers):
            raise ValueError(f"state must contain exactly {len(self.layers)} layer states")
        out = []
        for b, s in zip(self.layers, states):
            x_t, s = b.step(x_t, s)
            out.append(s)
        return self.norm_f(x_t), out

    def forward(self, x, state=None, return_state=False):
        if state is None and not return_state:
            for b in self.layers:
                x = b(x)
            return self.norm_f(x)
        if state is not None:
            if not isinstance(state, (list, tuple)) or len(state) != len(self.layers):
                raise ValueError(f"state must contain exactly {len(self.layers)} layer states")
            for b, s in zip(self.layers, state):
                if s is not None:
                    b.validate_state(s, batch_size=x.shape[0], device=x.device)
        states = state if state is not None else [None] * len(self.layers)
        out = []
        for b, s in zip(self.layers, states):
            x, s = b(x, state=s, return_state=True)
            out.append(s)
        y = self.norm_f(x)
        return (y, out) if return_state else y
