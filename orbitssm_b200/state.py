"""The recurrent carry (`State`) and its lifecycle, as the reference defines them
(reference: src/orbit_ssm/layers/state.py:31-366).

A `State` is a plain dict of tensors: ``hidden_state`` [B, H, P, N] (P index = g*R + r), and, depending on the
config, ``write_prev`` (trapezoid lag, same shape), ``bc_conv_state`` [B, N*R+N*O, d_conv] and ``conv_state``
[B, d_inner, d_conv] (raw-input windows, index -1 newest).  Default carry dtype: promote(parameter dtype, fp32);
a returned carry keeps the dtype of the carry it was given.
"""
from __future__ import annotations

import torch


def _map(value, fn):
    if torch.is_tensor(value):
        return fn(value)
    if isinstance(value, State):
        return State({k: _map(v, fn) for k, v in value.items()})
    if isinstance(value, dict):
        return {k: _map(v, fn) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_map(v, fn) for v in value)
    return value


class State(dict):
    """dict subclass moved/cast/detached as one object (reference: layers/state.py:31-115)."""

    @property
    def hidden_state(self):
        return self["hidden_state"]

    def to(self, device=None, dtype=None):
        def cast(t):
            target = dtype if dtype is not None and t.is_floating_point() else t.dtype
            return t.to(device=device if device is not None else t.device, dtype=target)
        return State(_map(dict(self), cast))

    def detach(self):
        return State(_map(dict(self), lambda t: t.detach()))

    def clone(self):
        return State(_map(dict(self), lambda t: t.clone()))

    def index_select(self, indices):
        if not torch.is_tensor(indices) or indices.ndim != 1 or indices.dtype != torch.long:
            raise ValueError("indices must be a one-dimensional int64 tensor")
        return State(_map(dict(self), lambda t: t.index_select(0, indices.to(t.device)) if t.ndim else t))

    def to_dict(self):
        return dict(self)

    @classmethod
    def from_dict(cls, d):
        return cls(d)


class StateLifecycle:
    """allocate / validate / reset / load / read; a layer implements `_init_state` only
    (reference: layers/state.py:210-343)."""

    def _state_schema(self):
        schema = getattr(self, "_cached_state_schema", None)
        if schema is None:
            with torch.no_grad():
                schema = self._init_state(1, device="meta", dtype=torch.float32)
            self._cached_state_schema = schema
        return schema

    def _default_state_dtype(self):
        p = next(self.parameters(), None)
        return torch.float32 if p is None else torch.promote_types(p.dtype, torch.float32)

    def validate_state(self, state, *, batch_size=None, device=None):
        if not isinstance(state, dict) or not torch.is_tensor(state.get("hidden_state")):
            raise ValueError("state must contain a batch-resolved tensor")
        ref = state["hidden_state"]
        batch_size = ref.shape[0] if batch_size is None else batch_size
        device = ref.device if device is None else torch.device(device)
        schema = self._state_schema()
        missing, extra = schema.keys() - state.keys(), state.keys() - schema.keys()
        if missing or extra:
            raise ValueError(f"state: missing keys {sorted(missing)}, unknown keys {sorted(extra)}")
        for k, exp in schema.items():
            v = state[k]
            if not torch.is_tensor(v):
                raise TypeError(f"state.{k} must be a tensor")
            shape = (batch_size, *exp.shape[1:])
            if tuple(v.shape) != shape:
                raise ValueError(f"state.{k}: expected shape {shape}, got {tuple(v.shape)}")
            if not v.is_floating_point():
                raise TypeError(f"state.{k}: incompatible dtype {v.dtype}")
            if v.device != device:
                raise ValueError(f"state.{k}: expected device {device}, got {v.device}")
        return state

    def _conform_carries(self, out, ref=None):
        """Returned carries take the dtype of the carry supplied, else the default carry dtype
        (reference: layers/state.py:242-269).  `.to` keeps the autograd graph."""
        default = self._default_state_dtype()
        res = State()
        for k, v in out.items():
            want = ref.get(k) if isinstance(ref, dict) else None
            target = want.dtype if torch.is_tensor(want) and want.is_floating_point() else default
            res[k] = v if (not torch.is_tensor(v) or not v.is_floating_point() or v.dtype == target) else v.to(target)
        return res

    def init_state(self, batch_size, device=None, dtype=None, *, h_init=None, overrides=None):
        if isinstance(batch_size, bool) or not isinstance(batch_size, int) or batch_size < 0:
            raise ValueError("batch_size must be a nonnegative integer")
        if dtype is None:
            dtype = self._default_state_dtype()
        state = self._init_state(batch_size, device=device, dtype=dtype)
        updates = dict(overrides or {})
        if h_init is not None:
            if "hidden_state" in updates:
                raise ValueError("pass h_init or overrides['hidden_state'], not both")
            exp = state["hidden_state"]
            if torch.is_tensor(h_init) and tuple(h_init.shape) == tuple(exp.shape[1:]):
                h_init = h_init.unsqueeze(0).expand(batch_size, *h_init.shape)
            updates["hidden_state"] = h_init
        unknown = updates.keys() - state.keys()
        if unknown:
            raise ValueError(f"unknown state overrides: {sorted(unknown)}")
        for k, v in updates.items():
            tgt = state[k]
            if not torch.is_tensor(v) or tuple(v.shape) != tuple(tgt.shape):
                raise ValueError(f"state.{k}: expected shape {tuple(tgt.shape)}")
            state[k] = v.to(device=tgt.device, dtype=tgt.dtype)      # keeps autograd (learned initial states)
        return State(state)

    def resolve_state(self, state, *, batch_size, device, dtype=None, h_init=None):
        if state is not None:
            if h_init is not None:
                raise ValueError("pass h_init OR state, not both")
            return self.validate_state(state, batch_size=batch_size, device=device)
        return self.init_state(batch_size, device=device, h_init=h_init)

    def reset_state(self, state, mask=None, keys=None):
        self.validate_state(state)
        ref = state["hidden_state"]
        sel = tuple(state) if keys is None else ((keys,) if isinstance(keys, str) else tuple(keys))
        unknown = set(sel) - state.keys()
        if unknown:
            raise ValueError(f"unknown state keys: {sorted(unknown)}")
        fresh = self.init_state(ref.shape[0], device=ref.device, dtype=ref.dtype)
        if mask is not None:
            if not torch.is_tensor(mask) or mask.ndim != 1 or mask.dtype not in (torch.bool, torch.long):
                raise ValueError("mask must be a one-dimensional bool mask or int64 batch indices")
            if mask.dtype == torch.bool and mask.numel() != ref.shape[0]:
                raise ValueError("boolean mask length must equal batch size")
            mask = mask.to(ref.device)
        for k in sel:
            if mask is None:
                state[k] = fresh[k].to(state[k].dtype)
            else:
                v = state[k].clone()
                v[mask] = fresh[k][mask].to(v.dtype)
                state[k] = v
        return state

    def set_state(self, state, other):
        self.validate_state(other)
        repl = {k: v.clone() for k, v in other.items()}
        state.clear()
        state.update(repl)
        return state

    def get_state(self):
        final = getattr(self, "_final_state", None)
        if final is None:
            raise RuntimeError(f"{type(self).__name__}: no state recorded; call forward(return_state=True)")
        return final
