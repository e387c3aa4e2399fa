"""The recurrent carry (`State`) and the bookkeeping a layer inherits for it (`StateLifecycle`).

The public surface is the reference's (src/orbit_ssm/layers/state.py:31-366): a `State` is a dict of batched tensors
that a layer returns from ``forward(..., return_state=True)`` and accepts back as ``state=``; a layer offers
``init_state / validate_state / resolve_state / reset_state / set_state / get_state``.  The implementation here is built
around one table per layer, its *carry layout*: for every carry its name, its per-sample shape and whether it is a
phase.  Every check and every conversion below is a walk over that table.

Carries of this package's layers (all flat tensors, batch on axis 0):
  ``hidden_state`` [B, H, P, N]   scan state, channel index P = g * R + r
  ``write_prev``   [B, H, P, N]   last write of a trapezoid layer
  ``conv_state``   [B, d_inner, d_conv], ``bc_conv_state`` [B, N*R + N*O, d_conv]   raw-input windows, newest last
  ``theta``        [B, H, K]      running rotation phase of the HybridMamba layer
Dtype law: a fresh carry is promote(parameter dtype, fp32); a returned carry takes the dtype of the carry supplied for it;
a phase accumulates angles over the whole sequence and is therefore never held below fp32.
"""
from __future__ import annotations

from typing import NamedTuple

import torch

#: carries that accumulate an angle; half precision would lose the phase after a few hundred tokens
PHASE_CARRIES = frozenset({"theta", "rot_ang", "c3_phase"})
_HALF = (torch.float16, torch.bfloat16)


class CarrySlot(NamedTuple):
    """One row of a layer's carry layout."""
    name: str
    sample_shape: tuple     # shape without the batch axis
    phase: bool


def _floor_dtype(name, dtype):
    """The dtype a carry called `name` may be held in when `dtype` is asked for."""
    return torch.float32 if (name in PHASE_CARRIES and dtype in _HALF) else dtype


class State(dict):
    """A dict of carry tensors handled as one object (moved, cast, detached, sliced along the batch)."""

    @property
    def hidden_state(self):
        return self["hidden_state"]

    def _each(self, fn):
        """A new State with `fn(name, tensor)` in place of every tensor; other values are kept as they are."""
        return State({k: (fn(k, v) if torch.is_tensor(v) else v) for k, v in self.items()})

    def to(self, device=None, dtype=None):
        """Move and/or cast.  `dtype` touches floating carries only; a phase carry stops at fp32 on the way down."""
        def move(name, t):
            kw = {}
            if device is not None:
                kw["device"] = device
            if dtype is not None and t.is_floating_point():
                kw["dtype"] = _floor_dtype(name, dtype)
            return t.to(**kw) if kw else t
        return self._each(move)

    def detach(self):
        return self._each(lambda _, t: t.detach())

    def clone(self):
        return self._each(lambda _, t: t.clone())

    def index_select(self, indices):
        """The carries of the batch rows `indices` (1-D int64), in that order."""
        if not (torch.is_tensor(indices) and indices.dim() == 1 and indices.dtype == torch.int64):
            raise ValueError(f"State.index_select takes a 1-D int64 tensor of batch rows, got "
                             f"{type(indices).__name__ if not torch.is_tensor(indices) else (indices.dtype, tuple(indices.shape))}")
        return self._each(lambda _, t: t.index_select(0, indices.to(t.device)) if t.dim() else t)

    def to_dict(self):
        return dict(self)

    @classmethod
    def from_dict(cls, d):
        return cls(d)


class StateLifecycle:
    """Carry bookkeeping for a layer that implements ``_init_state(batch_size, device=, dtype=) -> State``."""

    # -- the layout table ---------------------------------------------------------------------------------
    def _carry_layout(self):
        """Tuple of `CarrySlot`, in the order `_init_state` creates the carries (found once, on the meta device)."""
        layout = getattr(self, "_carry_layout_cache", None)
        if layout is None:
            with torch.no_grad():
                probe = self._init_state(1, device="meta", dtype=torch.float32)
            layout = tuple(CarrySlot(k, tuple(v.shape[1:]), k in PHASE_CARRIES) for k, v in probe.items())
            self._carry_layout_cache = layout
        return layout

    def _state_schema(self):
        """Carry names in layout order, as a dict name -> per-sample shape."""
        return {s.name: s.sample_shape for s in self._carry_layout()}

    def _default_state_dtype(self):
        p = next(self.parameters(), None)
        return torch.float32 if p is None else torch.promote_types(p.dtype, torch.float32)

    def _check_against_layout(self, tensors, batch_size, device, what):
        """`tensors`: name -> value for some or all slots.  Raises on a value that does not fit its slot."""
        for slot in self._carry_layout():
            if slot.name not in tensors:
                continue
            v = tensors[slot.name]
            if not torch.is_tensor(v):
                raise TypeError(f"{what}[{slot.name!r}] is a {type(v).__name__}; a tensor is needed")
            want = (batch_size, *slot.sample_shape)
            if tuple(v.shape) != want:
                raise ValueError(f"{what}[{slot.name!r}] has shape {tuple(v.shape)}; this layer carries {want}")
            if not v.is_floating_point():
                raise TypeError(f"{what}[{slot.name!r}] has dtype {v.dtype}; carries are floating point")
            if slot.phase and v.dtype in _HALF:
                raise TypeError(f"{what}[{slot.name!r}] is a phase held in {v.dtype}; phases need float32 or wider")
            if device is not None and v.device != torch.device(device):
                raise ValueError(f"{what}[{slot.name!r}] lives on {v.device}; the call runs on {torch.device(device)}")

    # -- public lifecycle ---------------------------------------------------------------------------------
    def validate_state(self, state, *, batch_size=None, device=None):
        """Check `state` against this layer's carry layout; returns it unchanged."""
        if not isinstance(state, dict) or not torch.is_tensor(state.get("hidden_state")):
            raise ValueError("a state is a dict of batched tensors with at least 'hidden_state'")
        names = [s.name for s in self._carry_layout()]
        absent = [n for n in names if n not in state]
        foreign = [k for k in state if k not in names]
        if absent or foreign:
            raise ValueError(f"state does not match this layer's carries {names}: absent {absent}, not a carry {sorted(foreign)}")
        h = state["hidden_state"]
        self._check_against_layout(state, h.shape[0] if batch_size is None else batch_size,
                                   h.device if device is None else device, "state")
        return state

    def _conform_carries(self, out, ref=None):
        """Cast the carries a call produced to the dtype of the carry it was given (else the default carry dtype,
        phases never below fp32).  Casting keeps the autograd graph."""
        default = self._default_state_dtype()
        res = State()
        for k, v in out.items():
            if torch.is_tensor(v) and v.is_floating_point():
                given = ref.get(k) if isinstance(ref, dict) else None
                target = given.dtype if (torch.is_tensor(given) and given.is_floating_point()) else default
                target = _floor_dtype(k, target)
                v = v if v.dtype == target else v.to(target)
            res[k] = v
        return res

    def init_state(self, batch_size, device=None, dtype=None, *, h_init=None, overrides=None):
        """Zero carries for `batch_size` sequences.  `h_init` ([*hidden shape] or [B, *hidden shape]) seeds the scan
        state, `overrides` any carry by name; both keep their autograd graph (learned initial states)."""
        if type(batch_size) is not int or batch_size < 0:
            raise ValueError(f"init_state: batch_size is a count of sequences (int >= 0), got {batch_size!r}")
        state = self._init_state(batch_size, device=device, dtype=self._default_state_dtype() if dtype is None else dtype)
        seeds = dict(overrides or {})
        if h_init is not None:
            if "hidden_state" in seeds:
                raise ValueError("init_state: the scan state is seeded twice (h_init and overrides['hidden_state'])")
            layout = {s.name: s for s in self._carry_layout()}
            if torch.is_tensor(h_init) and tuple(h_init.shape) == layout["hidden_state"].sample_shape:
                h_init = h_init.unsqueeze(0).expand(batch_size, *h_init.shape)
            seeds["hidden_state"] = h_init
        strangers = sorted(k for k in seeds if k not in state)
        if strangers:
            raise ValueError(f"init_state: {strangers} are not carries of this layer (it has {list(state)})")
        self._check_against_layout({k: v for k, v in seeds.items()}, batch_size, None, "init_state seed")
        for k, v in seeds.items():
            state[k] = v.to(device=state[k].device, dtype=_floor_dtype(k, state[k].dtype))
        return State(state)

    def resolve_state(self, state, *, batch_size, device, dtype=None, h_init=None):
        """The state a call starts from: the one supplied (validated) or a fresh one."""
        if state is None:
            return self.init_state(batch_size, device=device, dtype=dtype, h_init=h_init)
        if h_init is not None:
            raise ValueError("a call takes a full `state` or an `h_init` seed, not both")
        return self.validate_state(state, batch_size=batch_size, device=device)

    def reset_state(self, state, mask=None, keys=None):
        """Zero the carries `keys` (default: all) of the batch rows `mask` (bool mask or int64 rows; default: all rows).
        Entries of `state` are replaced, tensors are never written in place."""
        self.validate_state(state)
        h = state["hidden_state"]
        chosen = list(state) if keys is None else ([keys] if isinstance(keys, str) else list(keys))
        strangers = sorted(k for k in chosen if k not in state)
        if strangers:
            raise ValueError(f"reset_state: {strangers} are not carries of this state")
        rows = None
        if mask is not None:
            ok = torch.is_tensor(mask) and mask.dim() == 1 and mask.dtype in (torch.bool, torch.int64)
            if not ok or (mask.dtype == torch.bool and mask.numel() != h.shape[0]):
                raise ValueError("reset_state: `mask` is a bool mask over the batch or a 1-D int64 tensor of batch rows")
            rows = mask.to(h.device)
        zero = self.init_state(h.shape[0], device=h.device, dtype=h.dtype)
        for k in chosen:
            fresh = zero[k].to(state[k].dtype)
            if rows is None:
                state[k] = fresh
            else:
                kept = state[k].clone()
                kept[rows] = fresh[rows]
                state[k] = kept
        return state

    def set_state(self, state, other):
        """Make `state` a copy of `other` (validated) in place of its entries."""
        self.validate_state(other)
        copies = {k: v.clone() for k, v in other.items()}
        state.clear()
        state.update(copies)
        return state

    def get_state(self):
        """The State the last ``forward(..., return_state=True)`` returned."""
        last = getattr(self, "_final_state", None)
        if last is None:
            raise RuntimeError(f"{type(self).__name__} has recorded no state yet: call forward(..., return_state=True) first")
        return last
