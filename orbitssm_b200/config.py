"""Architecture (`SSDMimoConfig`) and run-time (`Execution`) descriptions of the SSD-MIMO layer.

Field names, defaults and refusals follow the reference's keyword-only dataclasses
(reference: src/orbit_ssm/config.py:36-141 shared fields, src/orbit_ssm/ssm/ssd_mimo.py:3782-3941
`SSDMimoConfig`, src/orbit_ssm/execution.py:24-85 `Execution`), so a config dict written for the
reference builds the same layer here.  Only the part of the config surface that the CUDA backend
serves is resolved; everything else is refused by name (`NotImplementedError`), never ignored.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field, fields
from types import SimpleNamespace
from typing import Any

BACKENDS = ("cuda", "auto")
PRECISIONS = ("io", "ieee")
WRITE_RULES = ("trapezoid", "euler")
HEAD_DYNAMIC, HEAD_STATIC = "head_dynamic", "head_static"


def _positive_int(v, name):
    if isinstance(v, bool) or not isinstance(v, int) or v < 1:
        raise ValueError(f"{name} must be a positive int, got {v!r}")
    return v


def _strict_from_dict(cls, d):
    """Strict dict constructor: only field names, bools must be bools (reference:
    src/orbit_ssm/validation.py:161-178)."""
    if not isinstance(d, dict):
        raise TypeError(f"{cls.__name__}.from_dict needs a dict, got {type(d).__name__}")
    names = {f.name: f for f in fields(cls)}
    unknown = sorted(set(d) - set(names))
    if unknown:
        raise TypeError(f"{cls.__name__}: unknown key(s) {unknown}; valid keys: {', '.join(sorted(names))}")
    return cls(**d)


def _check_bool_fields(obj):
    for f in fields(obj):
        if f.type in ("bool", "bool | None") and getattr(obj, f.name) is not None \
                and not isinstance(getattr(obj, f.name), bool):
            raise TypeError(f"{type(obj).__name__}.{f.name} must be a bool, got {getattr(obj, f.name)!r}")


@dataclass
class Execution:
    """How a layer runs (reference: src/orbit_ssm/execution.py:24-85).  None = leave unchanged.

    backend     "cuda" (the sm_100a kernels of this package) or "auto" (= "cuda"; a CPU tensor is refused
                by name, there is no CPU route here).
    precision   "io": scan operands in the IO dtype (bf16 tensor-core tiles, fp32 accumulate and state);
                "ieee": fp32 operands on the FP32 pipe.
    chunk_size  "auto" or a power of two in {16, 32, 64, 128}.
    checkpoint  False is what the layer does; True is refused (reference: ssd_mimo.py:4196-4199).
    """
    backend: str | None = None
    precision: str | None = None
    chunk_size: int | str | None = None
    checkpoint: bool | None = None
    kernel_options: dict | None = None

    def __post_init__(self):
        _check_bool_fields(self)
        if isinstance(self.kernel_options, dict):
            bad = [k for k in self.kernel_options if not isinstance(k, str)]
            if bad:
                raise TypeError(f"Execution: kernel_options must be a dict with str keys, got key(s) {bad!r}")

    @classmethod
    def from_dict(cls, d):
        return _strict_from_dict(cls, d)

    def fields(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self) if getattr(self, f.name) is not None}


def as_execution(x) -> Execution:
    if x is None:
        return Execution()
    if isinstance(x, Execution):
        return x
    if isinstance(x, dict):
        return Execution.from_dict(x)
    raise TypeError(f"execution must be an Execution or a dict, got {type(x).__name__}")


@dataclass(kw_only=True)
class SSDMimoConfig:
    """Architecture of an `SSDMimoSSM` layer (reference: src/orbit_ssm/ssm/ssd_mimo.py:3782-3941).

    Every field has the reference's name, meaning and default.  Rotating ("complex") row blocks and
    ``proj_source="main_branch"`` are outside the CUDA backend and are refused when the layer is built.
    """
    d_model: int | None = None
    d_state: int = 64
    expand: float | None = None
    d_conv: int = 4
    d_inner: int | None = None
    d_ssm_in: int = 1
    d_ssm_out: int | None = None
    n_groups: int | None = None
    n_heads: int | None = None
    d_head: int | None = None
    write_rule: str | None = None
    proj_source: str = "layer_input"
    bc_conv: bool | None = None
    dt_min: float = 1e-3
    dt_max: float = 1e-1
    dt_init_floor: float = 1e-4
    skip: bool = True
    skip_sharing: str = "head"
    out_norm: bool = False
    row_blocks: list | tuple | None = None
    theta_per_head: bool | None = None
    learn_theta_freq: bool | None = None
    use_theta_h: bool | None = None
    omega_layout: str | None = None
    theta_init: str | None = None
    b_norm: bool | None = None
    c_norm: bool | None = None
    bc_bias: str | None = None
    b_gate: bool | None = None
    c_gate: bool | None = None
    pair_layout: str = "interleaved"
    a_dyn_per_sibling: bool = False
    a_act: str = "heavy_tail"
    r_mix: str = "auto"
    r_mix_dyn: bool | None = None
    bc_bias_init: str | None = None
    a_proj_bias: bool = True
    trap_proj_bias: bool = True

    def __post_init__(self):
        _check_bool_fields(self)
        if isinstance(self.d_conv, bool) or not isinstance(self.d_conv, int) or self.d_conv < 0:
            raise ValueError(f"d_conv must be a nonnegative int, got {self.d_conv!r}")
        for name in ("d_model", "d_state", "d_inner", "d_ssm_in", "d_ssm_out", "n_groups", "n_heads", "d_head"):
            if getattr(self, name) is not None:
                _positive_int(getattr(self, name), name)
        if self.expand is not None and not self.expand > 0:
            raise ValueError(f"expand must be positive, got {self.expand!r}")
        if not (0 < self.dt_min <= self.dt_max) or self.dt_init_floor <= 0:
            raise ValueError("need 0 < dt_min <= dt_max and dt_init_floor > 0")
        if self.width() is not None:
            resolve_ssd_spec(self)          # validate now; the layer resolves it again, identically

    # -- width rule (reference: src/orbit_ssm/configuration.py:48-65) -------------------------------
    def width(self, d_model=None):
        d_model = self.d_model if d_model is None else d_model
        if d_model is None:
            return self.d_inner
        if self.expand is None:
            return self.d_inner if self.d_inner is not None else int(d_model * 2.0)
        derived = _positive_int(int(d_model * self.expand), "expanded d_inner")
        if self.d_inner is not None and self.d_inner != derived:
            raise ValueError(f"d_inner={self.d_inner} conflicts with int(d_model*expand)={derived}; give only one of them")
        return derived

    def layer_width(self) -> int:
        if self.d_model is not None:
            return self.d_model
        if self.d_inner is not None and self.expand is None:
            return self.d_inner
        raise TypeError("SSDMimoConfig: the layer width d_model is not set; give d_model or build with config.build(d_model)")

    def replace(self, **kw):
        return dataclasses.replace(self, **kw)

    @classmethod
    def from_dict(cls, d):
        return _strict_from_dict(cls, d)

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    def build(self, d_model=None, execution=None):
        from .ssd_mimo import SSDMimoSSM
        cfg = self if d_model is None else self.replace(d_model=d_model)
        return SSDMimoSSM(cfg, execution=execution)


def mamba2_config(d_model: int, *, expand: int = 2, d_state: int = 128, d_head: int = 64, n_groups: int = 1,
                  d_conv: int = 4, **overrides) -> SSDMimoConfig:
    """The Mamba-2 preset of the reference (src/orbit_ssm/presets.py:93-154): SISO, static per-head decay,
    Euler write, joint B|C conv, no B/C norms, biases or gates, D skip per head, output RMSNorm."""
    if n_groups != 1:
        raise ValueError(f"mamba2_config: n_groups must be 1 (one B/C shared by every head), got {n_groups}")
    d_inner = int(expand) * d_model
    if d_inner % d_head:
        raise ValueError(f"mamba2_config: d_inner={d_inner} (expand*d_model) is not a multiple of d_head={d_head}")
    core = dict(d_ssm_in=1, d_ssm_out=1, n_groups=d_head, n_heads=d_inner // d_head, proj_source="layer_input",
                bc_conv=True, row_blocks=[{"frac": 1.0, "decay": HEAD_STATIC, "complex": False}], skip=True,
                skip_sharing="head", write_rule="euler", out_norm=True, b_norm=False, c_norm=False, bc_bias="none",
                b_gate=False, c_gate=False, r_mix_dyn=False, dt_min=1e-3, dt_max=1e-1)
    core.update(overrides)
    return SSDMimoConfig(d_model=d_model, d_state=d_state, expand=float(expand), d_conv=d_conv, **core)


def _resolve_geometry(d_inner, R, n_groups, n_heads, d_head):
    """``n_heads * d_head == d_inner`` and ``d_head == n_groups * R`` (reference: ssd_mimo.py:112-126,
    configuration.py:68-108); default head width ``max(1, 64 // R) * R``."""
    if n_groups is not None:
        gw = n_groups * R
        if d_head is not None and d_head != gw:
            raise ValueError(f"conflicting d_head: {{'d_head': {d_head}, 'n_groups_times_d_ssm_in': {gw}}}")
        d_head = gw
    if n_heads is None and d_head is None:
        d_head = max(1, 64 // R) * R
    if d_head is None:
        if d_inner % n_heads:
            raise ValueError(f"d_inner={d_inner} is not divisible by n_heads={n_heads}")
        d_head = d_inner // n_heads
    if n_heads is None:
        if d_inner % d_head:
            raise ValueError(f"d_inner={d_inner} is not divisible by d_head={d_head}")
        n_heads = d_inner // d_head
    if n_heads * d_head != d_inner:
        raise ValueError(f"n_heads*d_head={n_heads * d_head} != d_inner={d_inner}")
    if d_head % R:
        raise ValueError(f"d_head={d_head} must be divisible by d_ssm_in={R}")
    return n_heads, d_head, d_head // R


def resolve_ssd_spec(cfg: SSDMimoConfig, d_model: int | None = None) -> SimpleNamespace:
    """Resolve a config into the flat facts the layer, the kernels and the CPU checker read.

    Mirrors what `_SSDMimoScan.__init__` derives (reference: ssd_mimo.py:575-884): geometry, the decay law,
    map options, sibling mix, and the column order of the fused token slab.
    """
    d_model = cfg.layer_width() if d_model is None else d_model
    d_inner = cfg.width(d_model)
    R = cfg.d_ssm_in
    O = R if cfg.d_ssm_out is None else cfg.d_ssm_out
    N = cfg.d_state
    H, P, G = _resolve_geometry(d_inner, R, cfg.n_groups, cfg.n_heads, cfg.d_head)
    write_rule = "trapezoid" if cfg.write_rule is None else cfg.write_rule
    if write_rule == "zoh":
        raise NotImplementedError("write_rule='zoh' is not implemented")
    if write_rule not in WRITE_RULES:
        raise ValueError(f"write_rule must be one of {WRITE_RULES}, got {write_rule!r}")
    if cfg.proj_source not in ("layer_input", "main_branch"):
        raise ValueError(f"proj_source must be 'layer_input' or 'main_branch', got {cfg.proj_source!r}")
    if cfg.proj_source != "layer_input":
        raise NotImplementedError("proj_source='main_branch' is outside the CUDA backend (token maps read the layer input)")
    bc_conv = bool(cfg.bc_conv)
    if bc_conv and cfg.d_conv <= 0:
        raise ValueError("bc_conv=True requires d_conv > 0")
    if cfg.d_conv not in (0, 2, 3, 4):
        raise NotImplementedError(f"d_conv={cfg.d_conv}: the CUDA conv kernel serves widths 2..4 (and 0 = no conv)")

    # row blocks: one decay law for the whole state; a complex block is the rotating part (not served)
    blocks = cfg.row_blocks
    if blocks is None:
        blocks = [{"frac": 1.0, "decay": HEAD_DYNAMIC}]
    if len(blocks) < 1 or len(blocks) > 2:
        raise ValueError("row_blocks: SSD-MIMO takes one or two blocks")
    decays = set()
    for b in blocks:
        b = dict(b) if isinstance(b, dict) else dataclasses.asdict(b)
        unknown = set(b) - {"rows", "frac", "decay", "complex", "gate"}
        if unknown:
            raise TypeError(f"row_blocks: unknown block key(s) {sorted(unknown)}")
        if b.get("complex"):
            raise NotImplementedError("complex (rotating) row blocks are outside the CUDA backend")
        if b.get("gate") is False:
            raise NotImplementedError("row blocks with gate=False are outside the CUDA backend")
        d = b.get("decay") or HEAD_DYNAMIC
        if d not in (HEAD_DYNAMIC, HEAD_STATIC):
            raise ValueError(f"row_blocks: decay must be 'head_dynamic' or 'head_static' for SSD-MIMO, got {d!r}")
        decays.add(d)
    if len(decays) != 1:
        raise ValueError("row_blocks: both blocks are rows of one scan with one decay per head; their decays must agree")
    a_dyn = decays.pop() == HEAD_DYNAMIC
    if not a_dyn and (cfg.a_dyn_per_sibling or cfg.a_act != "heavy_tail" or not cfg.a_proj_bias):
        raise ValueError("a_dyn_per_sibling / a_act / a_proj_bias belong to the 'head_dynamic' rate; no block uses it")
    if cfg.a_act not in ("heavy_tail", "softplus"):
        raise ValueError(f"a_act must be 'heavy_tail' or 'softplus', got {cfg.a_act!r}")
    for name in ("theta_per_head", "learn_theta_freq", "use_theta_h", "omega_layout", "theta_init"):
        if getattr(cfg, name) is not None:
            raise ValueError(f"{name} needs a complex row block")
    if cfg.pair_layout != "interleaved":
        raise NotImplementedError("pair_layout='half' needs a complex row block")

    b_norm = True if cfg.b_norm is None else cfg.b_norm
    c_norm = True if cfg.c_norm is None else cfg.c_norm
    bias_gran = "head" if cfg.bc_bias is None else cfg.bc_bias
    if bias_gran not in ("head", "shared", "none"):
        raise ValueError(f"bc_bias must be 'head', 'shared' or 'none', got {bias_gran!r}")
    use_g_b = (R > 1) if cfg.b_gate is None else cfg.b_gate
    use_g_c = (O > 1) if cfg.c_gate is None else cfg.c_gate
    init = cfg.bc_bias_init or "auto"
    if init not in ("auto", "ones", "spread"):
        raise ValueError(f"bc_bias_init must be 'auto', 'ones' or 'spread', got {init!r}")
    if init == "auto":
        init = "ones" if (R == 1 or bias_gran != "head") else "spread"

    if cfg.r_mix not in ("auto", "learned", "none"):
        raise ValueError(f"r_mix must be 'auto', 'learned' or 'none', got {cfg.r_mix!r}")
    r_mix_mode = ("none" if R == 1 else "learned") if cfg.r_mix == "auto" else cfg.r_mix
    r_mix_dyn = cfg.r_mix_dyn
    if r_mix_dyn is None:
        r_mix_dyn = R > 1 and r_mix_mode != "none"
    if r_mix_mode == "none" and r_mix_dyn:
        raise ValueError("r_mix_dyn=True needs an active sibling mix, but r_mix resolved to 'none'")
    if cfg.skip_sharing not in ("input_output", "channel", "head"):
        raise ValueError("skip_sharing must be input_output, channel, or head")
    use_trap = write_rule == "trapezoid"
    if not use_trap and not cfg.trap_proj_bias:
        raise ValueError(f"trap_proj_bias=False, but write_rule={write_rule!r} builds no trapezoid weight projection")

    # token slab: packed column order of the fused token-map projection (reference: ssd_mimo.py:858-876)
    slab = [("B", "B_proj", N * R, False), ("C", "C_proj", N * O, False)]
    if use_g_b:
        slab.append(("gB", "gB_proj", N * R, False))
    if use_g_c:
        slab.append(("gC", "gC_proj", N * O, False))
    slab.append(("dt", "dt_proj", H * R, True))
    if a_dyn:
        slab.append(("a", "a_dyn_proj", H * R if cfg.a_dyn_per_sibling else H, bool(cfg.a_proj_bias)))
    if use_trap:
        slab.append(("trap", "trap_proj", H, bool(cfg.trap_proj_bias)))
    if r_mix_dyn:
        slab.append(("rmix", "r_mix_proj", H * R, False))
    offs, o = {}, 0
    for key, _, width, _ in slab:
        offs[key] = (o, width)
        o += width

    return SimpleNamespace(
        d_model=d_model, d_inner=d_inner, d_conv=cfg.d_conv, H=H, P=P, G=G, R=R, O=O, N=N, d_out=H * G * O,
        a_dyn=a_dyn, a_dyn_per_sibling=bool(cfg.a_dyn_per_sibling), a_act=cfg.a_act, a_proj_bias=bool(cfg.a_proj_bias),
        write_rule=write_rule, use_trap=use_trap, trap_proj_bias=bool(cfg.trap_proj_bias),
        b_norm=b_norm, c_norm=c_norm, bias_gran=bias_gran, bc_bias=bias_gran != "none", head_bias=bias_gran == "head",
        bc_bias_init=init, use_g_b=bool(use_g_b), use_g_c=bool(use_g_c), r_mix_mode=r_mix_mode, r_mix_dyn=bool(r_mix_dyn),
        skip=bool(cfg.skip), skip_sharing=cfg.skip_sharing, bc_conv=bc_conv, out_norm=bool(cfg.out_norm),
        dt_min=cfg.dt_min, dt_max=cfg.dt_max, dt_init_floor=cfg.dt_init_floor,
        slab=tuple(slab), slab_off=offs, tok_width=o, norm_eps=1e-5, map_eps=1e-5)


# ----------------------------------------------------------------------------------------------------
#  HybridMamba
# ----------------------------------------------------------------------------------------------------
COORD_STATIC = "coord_static"


@dataclass(kw_only=True)
class HybridMambaConfig:
    """Architecture of a `HybridMambaSSM` layer (reference: src/orbit_ssm/ssm/hybrid_mamba.py:2904-3100).

    Every field has the reference's name, meaning and default.  The CUDA backend serves the per-coordinate static
    decay law (``coord_static`` row blocks, real or rotating pairs), Euler or trapezoid write, B/C RMSNorm, per-head
    additive map biases, learned pair frequencies and read offsets; gates, the dynamic / potential laws, flat
    (per-head) laws, ``proj_source="main_branch"`` and the joint B|C conv are refused by name when the layer is built.
    """
    d_model: int | None = None
    d_state: int = 64
    expand: float | None = None
    d_conv: int = 4
    d_inner: int | None = None
    d_ssm_in: int = 1
    d_ssm_out: int | None = None
    n_groups: int | None = None
    n_heads: int | None = None
    d_head: int | None = None
    write_rule: str | None = None
    proj_source: str | None = None
    bc_conv: bool | None = None
    dt_min: float = 1e-3
    dt_max: float = 1e-1
    dt_init_floor: float = 1e-4
    skip: bool = True
    skip_sharing: str = "head"
    out_norm: bool = False
    row_blocks: list | tuple | None = field(default_factory=lambda: [{"frac": 1.0, "decay": COORD_STATIC}])
    theta_per_head: bool | None = None
    learn_theta_freq: bool | None = None
    use_theta_h: bool | None = None
    omega_layout: str | None = None
    theta_init: str | None = None
    b_norm: bool | None = None
    c_norm: bool | None = None
    bc_bias: str | None = None
    b_gate: bool | None = None
    c_gate: bool | None = None
    bc_gate_act: str | None = None
    bc_gate_bias: bool | None = None
    bc_gate_pos: str | None = None
    dt_rank: int | str | None = "adaptive"
    force_dt_dense: bool = False
    dt_init: str | None = "random"
    dt_scale: float = 1.0
    dyn_res: str = "n"
    dyn_act: str | int = "heavy_tail"
    mu_res: str = "n"
    mu_cap: float = 4.0
    a_floor: float = 1e-4
    a_act: str = "heavy_tail"
    norm_eps: float = 1e-5
    learnable_h_init: bool = False
    gate_init: str = "kaiming_uniform"

    def __post_init__(self):
        _check_bool_fields(self)
        if isinstance(self.d_conv, bool) or not isinstance(self.d_conv, int) or self.d_conv < 0:
            raise ValueError(f"d_conv must be a nonnegative int, got {self.d_conv!r}")
        for name in ("d_model", "d_state", "d_inner", "n_heads", "d_head"):
            if getattr(self, name) is not None:
                _positive_int(getattr(self, name), name)
        # fields this family cannot honour (reference: hybrid_mamba.py:3077-3081)
        if self.d_ssm_in != 1 or self.d_ssm_out not in (None, 1) or self.n_groups is not None:
            raise ValueError("HybridMambaConfig: d_ssm_in != 1, d_ssm_out other than 1 and n_groups are not part of this family")
        if self.expand is not None and not self.expand > 0:
            raise ValueError(f"expand must be positive, got {self.expand!r}")
        if not (0 < self.dt_min <= self.dt_max) or self.dt_init_floor <= 0:
            raise ValueError("need 0 < dt_min <= dt_max and dt_init_floor > 0")
        if self.write_rule is not None and self.write_rule not in WRITE_RULES:
            raise ValueError(f"write_rule must be one of {WRITE_RULES} or None, got {self.write_rule!r}")
        if self.width() is not None:
            resolve_hm_spec(self)

    width = SSDMimoConfig.width

    def layer_width(self) -> int:
        if self.d_model is not None:
            return self.d_model
        if self.d_inner is not None and self.expand is None:
            return self.d_inner
        raise TypeError("HybridMambaConfig: the layer width d_model is not set; give d_model or build with config.build(d_model)")

    def replace(self, **kw):
        return dataclasses.replace(self, **kw)

    @classmethod
    def from_dict(cls, d):
        return _strict_from_dict(cls, d)

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    def build(self, d_model=None, execution=None):
        from .hybrid_mamba import HybridMambaSSM
        cfg = self if d_model is None else self.replace(d_model=d_model)
        return HybridMambaSSM(cfg, execution=execution)


def resolve_dt_rank(dt_rank, *, d_sel, heads, d_model, force_dt_dense=False):
    """Rank of the clock projection: None = dense; "auto" = ceil(width / 16); "adaptive" = that rank only when it saves
    multiplies (reference: src/orbit_ssm/configuration.py:21-42)."""
    if force_dt_dense:
        if dt_rank is not None and dt_rank != "adaptive":
            raise ValueError("force_dt_dense conflicts with an explicit bottleneck dt_rank")
        return None
    if dt_rank is None:
        return None
    if dt_rank not in ("adaptive", "auto"):
        return _positive_int(dt_rank, "dt_rank")
    rank = (d_model + 15) // 16
    if dt_rank == "auto" or rank * (d_sel + heads) < d_sel * heads:
        return rank
    return None


def resolve_hm_spec(cfg: HybridMambaConfig, d_model: int | None = None) -> SimpleNamespace:
    """Resolved geometry and row plan of a HybridMamba layer; refuses, by name, what the CUDA backend does not serve
    (reference: hybrid_mamba.py:540-735 row plan and pair-tied stores, 2620-2675 layer geometry)."""
    who = "HybridMambaSSM(backend='cuda')"
    d_model = cfg.d_model if d_model is None else d_model
    if d_model is None:
        d_model = cfg.layer_width()
    d_inner = cfg.width(d_model)
    N = cfg.d_state
    if cfg.n_heads is not None and cfg.d_head is not None and cfg.n_heads * cfg.d_head != d_inner:
        raise ValueError(f"conflicting n_heads={cfg.n_heads}, d_head={cfg.d_head} for d_inner={d_inner}")
    P = cfg.d_head if cfg.d_head is not None else (d_inner // cfg.n_heads if cfg.n_heads is not None else 64)
    if d_inner % P:
        raise ValueError(f"d_inner={d_inner} is not a multiple of d_head={P}")
    H = d_inner // P
    blocks = list(cfg.row_blocks or [{"frac": 1.0, "decay": COORD_STATIC}])
    rot, used = [], 0
    for i, blk in enumerate(blocks):
        if not isinstance(blk, dict) or "decay" not in blk:
            raise TypeError("row_blocks entries are dicts with 'frac' and 'decay'")
        unknown = set(blk) - {"frac", "decay", "complex", "gate"}
        if unknown:
            raise TypeError(f"row_blocks: unknown key(s) {sorted(unknown)}")
        if blk["decay"] != COORD_STATIC:
            raise NotImplementedError(f"{who}: row block decay {blk['decay']!r} is not served (only 'coord_static')")
        if blk.get("gate"):
            raise NotImplementedError(f"{who}: gated row blocks are not served")
        rows = N - used if i == len(blocks) - 1 else int(round(float(blk.get("frac", 1.0)) * N))
        if rows <= 0:
            raise ValueError("row_blocks: every block needs at least one row and the fractions must sum to 1")
        cx = bool(blk.get("complex", False))
        if cx and rows % 2:
            raise ValueError(f"a rotating block needs an even row count, got {rows}")
        if cx and used % 2:
            raise ValueError("a rotating block must start on an even row")
        rot += [cx] * rows
        used += rows
    if used != N:
        raise ValueError(f"row_blocks sizes sum to {used}, d_state is {N}")
    has_rot = any(rot)
    for name, served in (("b_gate", (None, False)), ("c_gate", (None, False)), ("bc_gate_act", (None,)),
                         ("bc_gate_bias", (None, False)), ("bc_gate_pos", (None,)), ("proj_source", (None, "layer_input")),
                         ("bc_conv", (None, False)), ("theta_per_head", (None, False)), ("omega_layout", (None, "pair")),
                         ("theta_init", (None, "kaiming")), ("learnable_h_init", (False,)), ("skip_sharing", ("head",)),
                         ("bc_bias", (None, "head", "none"))):
        if getattr(cfg, name) not in served:
            raise NotImplementedError(f"{who}: {name}={getattr(cfg, name)!r} is not served")
    rep = [n - 1 if (rot[n] and n % 2) else n for n in range(N)]
    store = [n for n in range(N) if rep[n] == n]
    col = {n: i for i, n in enumerate(store)}
    a_idx = [col[rep[n]] for n in range(N)]
    # S4D-real ladder restarting in each block; a rotating block's ladder runs over its pairs
    ladder, pos = [], 0
    for i, blk in enumerate(blocks):
        rows = (N - pos) if i == len(blocks) - 1 else int(round(float(blk.get("frac", 1.0)) * N))
        ladder += list(range(1, (rows // 2 if blk.get("complex", False) else rows) + 1))
        pos += rows
    rot_pairs = [k for k in range(N // 2) if rot[2 * k]] if has_rot else []
    use_trap = cfg.write_rule is None or cfg.write_rule == "trapezoid"
    bias = "head" if cfg.bc_bias is None else cfg.bc_bias
    dt_rank = resolve_dt_rank(cfg.dt_rank, d_sel=d_model, heads=H, d_model=d_model, force_dt_dense=cfg.force_dt_dense)
    if cfg.dt_init not in (None, "random", "constant"):
        raise ValueError("dt_init must be None, 'random', or 'constant'")
    return SimpleNamespace(
        d_model=d_model, d_inner=d_inner, d_conv=cfg.d_conv, H=H, P=P, N=N, K=N // 2, rot=rot, has_rot=has_rot,
        rot_pairs=rot_pairs, a_idx=a_idx, n_store=len(store), ladder=ladder, use_trap=use_trap,
        b_norm=cfg.b_norm is None or cfg.b_norm, c_norm=cfg.c_norm is None or cfg.c_norm, bc_bias=bias == "head",
        learn_theta_freq=has_rot and (cfg.learn_theta_freq is None or cfg.learn_theta_freq),
        use_theta_h=has_rot and (cfg.use_theta_h is None or cfg.use_theta_h), skip=cfg.skip, out_norm=cfg.out_norm,
        dt_rank=dt_rank, dt_init=cfg.dt_init, dt_scale=float(cfg.dt_scale), dt_min=cfg.dt_min, dt_max=cfg.dt_max,
        dt_init_floor=cfg.dt_init_floor, norm_eps=cfg.norm_eps)
