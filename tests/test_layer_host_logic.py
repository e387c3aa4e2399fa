"""Host logic of `SSDMimoSSM` on CPU: the C-ABI kernels are replaced by their torch restatements
(oracle/abi_reference.py), everything else (fused projection, token law, state folding, layouts, autograd wiring,
State contract) is the product code, checked against vectors produced by the reference."""
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from orbitssm_b200 import ops
from orbitssm_b200.config import SSDMimoConfig
from orbitssm_b200.ssd_mimo import SSDMimoSSM
from oracle import abi_reference as R


@pytest.fixture
def cpu_kernels(monkeypatch):
    # the scan goes through the product's own phase sequencing (ops.scan_fwd / scan_bwd); only the C-ABI call is replaced
    for name in ("conv1d_fwd", "conv1d_bwd", "gate_norm_fwd", "gate_norm_bwd", "run_phase", "pick_chunk", "token_map_fwd",
                 "token_map_bwd", "run_clock", "run_step"):
        monkeypatch.setattr(ops, name, getattr(R, name))
    monkeypatch.setattr(ops, "on_device", lambda t: True)
    monkeypatch.setattr(ops, "_require_cuda", lambda who, *t: None)
    monkeypatch.setattr(ops, "_dtype_code", lambda who, t: 0)


def _rel(a, b):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def _layer(rec, dtype=torch.float32):
    layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]))
    missing, unexpected = layer.load_state_dict(rec["state_dict"], strict=True), None
    return layer.to(dtype)


def _run(layer, rec, x, dy, state, exact):
    x = x.clone().requires_grad_(True)
    if state is not None:
        state = {k: v.clone().to(torch.float32).requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    if exact:
        y = layer(x)
        (y ** 2).mean().backward()
        st = None
    else:
        y, st = layer(x, state=state, return_state=True)
        loss = (y * dy).sum() + (st["hidden_state"] * rec["gh"]).sum()
        if "write_prev" in st:
            loss = loss + (st["write_prev"] * rec["gw"]).sum()
        loss.backward()
    grads = {n: p.grad for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad
    return y.detach(), st, grads


def _check(got, want, tol, what):
    y, st, grads = got
    assert _rel(y, want["y"]) < tol, (what, "y", _rel(y, want["y"]))
    if want.get("state") is not None:
        assert list(st) == list(want["state"]), (what, list(st), list(want["state"]))
        for k, v in want["state"].items():
            assert st[k].dtype == torch.float32
            assert _rel(st[k].detach(), v) < tol, (what, "state", k, _rel(st[k].detach(), v))
    for k, v in want["grads"].items():
        assert k in grads, (what, "missing grad", k)
        assert _rel(grads[k], v) < tol, (what, "grad", k, _rel(grads[k], v))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_layer_matches_reference(name, cpu_kernels):
    rec = load_golden(name)
    layer = _layer(rec)
    got = _run(layer, rec, rec["x"], rec["dy"], None, rec["exact"])
    _check(got, rec["f64"], 2e-4, name)
    if "f64_cont" in rec:
        c = rec["f64_cont"]
        s = c["split"]
        got = _run(layer, rec, rec["x"][:, s:], rec["dy"][:, s:], c["state_in"], False)
        _check(got, c, 2e-4, name + " continuation")


def test_same_seed_draws_reference_weights():
    """Construction order mirrors the reference, so torch.manual_seed(0) gives the reference's default init."""
    rec = load_golden("cfg1_exact")
    torch.manual_seed(0)
    layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]))
    sd = layer.state_dict()
    assert list(sd) == list(rec["state_dict"])
    for k, v in rec["state_dict"].items():
        assert torch.equal(sd[k].float(), v.float()), k


def test_split_equals_whole(cpu_kernels):
    rec = load_golden("dyn_trap_conv")
    layer = _layer(rec)
    x = rec["x"]
    y_all, s_all = layer(x, return_state=True)
    st, ys = None, []
    for a, b in ((0, 5), (5, 6), (6, 6), (6, 37)):
        y, st = layer(x[:, a:b], state=st, return_state=True)
        ys.append(y)
    assert _rel(torch.cat(ys, 1), y_all) < 1e-5
    for k in s_all:
        assert _rel(st[k], s_all[k]) < 1e-5, k


def test_cpu_tensor_is_refused_by_name():
    rec = load_golden("euler_r2o1")
    layer = _layer(rec)
    with pytest.raises(ValueError, match="CPU tensor"):
        layer(rec["x"])


def test_execution_and_config_refusals():
    rec = load_golden("euler_r2o1")
    layer = _layer(rec)
    with pytest.raises(ValueError):
        layer.set_execution({"backend": "torch"})
    with pytest.raises(ValueError):
        layer.set_execution({"checkpoint": True})
    with pytest.raises(TypeError):
        layer.set_execution({"nope": 1})
    with pytest.raises(ValueError):
        layer.set_execution({"chunk_size": 24})
    before = (layer.backend, layer.precision, layer.chunk_size)
    with pytest.raises(ValueError):
        layer.set_execution({"precision": "ieee", "backend": "sequential"})     # nothing changes on a refusal
    assert (layer.backend, layer.precision, layer.chunk_size) == before
    with layer.execution({"precision": "ieee"}):
        assert layer.precision == "ieee"
    assert layer.precision == "io"
    with pytest.raises(TypeError):
        SSDMimoConfig.from_dict({"d_model": 8, "bogus": 1})
    with pytest.raises(NotImplementedError):
        SSDMimoSSM(SSDMimoConfig(d_model=16, d_state=8, n_groups=8,
                                 row_blocks=[{"frac": 0.5, "complex": True}, {"frac": 0.5}]))
    with pytest.raises(ValueError, match="conflicting d_head"):
        SSDMimoConfig(d_model=2048, expand=2.0, d_state=128, d_ssm_in=4, d_ssm_out=4, n_groups=8, d_head=64)


def test_state_lifecycle(cpu_kernels):
    rec = load_golden("dyn_trap_conv")
    layer = _layer(rec)
    st = layer.init_state(2)
    assert list(st) == ["hidden_state", "write_prev", "bc_conv_state", "conv_state"]
    assert all(v.dtype == torch.float32 for v in st.values())
    with pytest.raises(ValueError):
        layer.validate_state({"hidden_state": st["hidden_state"]})
    _, s1 = layer(rec["x"], state=st, return_state=True)
    assert layer.get_state() is s1
    bf = layer.init_state(2, dtype=torch.bfloat16)
    _, s2 = layer(rec["x"], state=bf, return_state=True)
    assert all(v.dtype == torch.bfloat16 for v in s2.values())          # a returned carry keeps the supplied dtype
    layer.reset_state(s1, mask=torch.tensor([True, False]))
    assert float(s1["hidden_state"][0].abs().sum()) == 0.0 and float(s1["hidden_state"][1].abs().sum()) > 0.0


# ---------------------------------------------------------------------------------------------------- HybridMamba
from conftest import HM_GOLDEN_CASES                                    # noqa: E402
from orbitssm_b200.config import HybridMambaConfig                      # noqa: E402
from orbitssm_b200.hybrid_mamba import HybridMambaSSM                   # noqa: E402


@pytest.fixture
def cpu_hm_kernels(monkeypatch):
    for name in ("conv1d_fwd", "conv1d_bwd", "gate_norm_fwd", "gate_norm_bwd", "run_hm", "token_map_fwd", "token_map_bwd",
                 "hm_tail_fwd", "hm_tail_bwd"):
        monkeypatch.setattr(ops, name, getattr(R, name))
    monkeypatch.setattr(ops, "on_device", lambda t: True)
    monkeypatch.setattr(ops, "_require_cuda", lambda who, *t: None)
    monkeypatch.setattr(ops, "_dtype_code", lambda who, t: 0)


def _run_hm(layer, rec, x, dy, state):
    x = x.clone().requires_grad_(True)
    if state is not None:
        state = {k: v.clone().to(torch.float32).requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    y, st = layer(x, state=state, return_state=True)
    loss = (y * dy).sum()
    for k, g in rec["gs"].items():
        if k in st:
            loss = loss + (st[k] * g).sum()
    loss.backward()
    grads = {n: p.grad for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad
    return y.detach(), st, grads


@pytest.mark.parametrize("name", HM_GOLDEN_CASES)
def test_hm_layer_matches_reference(name, cpu_hm_kernels):
    """`HybridMambaSSM` host logic (fused projection, maps, pair-tied stores, carries, autograd wiring) against the
    reference's fp64 results, with the C-ABI kernels replaced by their torch restatements."""
    rec = load_golden(name)
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    layer.load_state_dict(rec["state_dict"], strict=True)
    got = _run_hm(layer, rec, rec["x"], rec["dy"], None)
    _check(got, rec["f64"], 2e-4, name)
    c = rec["f64_cont"]
    s = c["split"]
    got = _run_hm(layer, rec, rec["x"][:, s:], rec["dy"][:, s:], c["state_in"])
    _check(got, c, 2e-4, name + " continuation")


@pytest.mark.parametrize("name", HM_GOLDEN_CASES)
def test_hm_same_seed_same_weights(name):
    """Parameter creation order and initialisers match the reference: the same torch seed draws the same weights."""
    rec = load_golden(name)
    torch.manual_seed(0)
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    sd = layer.state_dict()
    assert list(sd) == list(rec["fresh_state_dict"]), (list(sd), list(rec["fresh_state_dict"]))
    for k, v in rec["fresh_state_dict"].items():
        assert sd[k].shape == v.shape and torch.equal(sd[k].float(), v), k


def test_hm_refusals():
    with pytest.raises(NotImplementedError):
        HybridMambaSSM(HybridMambaConfig(d_model=32, d_state=8, d_head=8, row_blocks=[{"frac": 1.0, "decay": "coord_dynamic"}]))
    with pytest.raises(NotImplementedError):
        HybridMambaSSM(HybridMambaConfig(d_model=32, d_state=8, d_head=8, b_gate=True))
    with pytest.raises(ValueError):
        HybridMambaConfig(d_model=32, d_ssm_in=2)
    layer = HybridMambaSSM(HybridMambaConfig(d_model=32, d_state=8, d_head=8))
    with pytest.raises(ValueError):
        layer(torch.zeros(1, 4, 32))                    # CPU tensor: refused by name, no CPU route
    with pytest.raises(ValueError):
        layer.set_execution({"precision": "ieee"})


# ---------------------------------------------------------------------------------------------------- decode step
def test_step_equals_forward(cpu_kernels):
    """`step` token by token from a carried State equals `forward` on the same tokens (outputs and every carry)."""
    rec = load_golden("dyn_trap_conv")
    layer = _layer(rec)
    x = rec["x"][:, :9]
    with torch.no_grad():
        y_all, s_all = layer(x, return_state=True)
        y_head, st = layer(x[:, :5], return_state=True)
        ys = [y_head]
        for t in range(5, 9):
            y_t, st = layer.step(x[:, t], st)
            assert y_t.shape == (x.shape[0], layer.d_model)
            ys.append(y_t.unsqueeze(1))
    assert _rel(torch.cat(ys, 1), y_all) < 1e-5
    for k in s_all:
        assert _rel(st[k], s_all[k]) < 1e-5, k
    with pytest.raises(ValueError):
        layer.step(x[:, 0], None)


def test_hm_step_equals_forward(cpu_hm_kernels):
    rec = load_golden("hm_small")
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    layer.load_state_dict(rec["state_dict"], strict=True)
    x = rec["x"][:, :8]
    with torch.no_grad():
        y_all, s_all = layer(x, return_state=True)
        st, ys = None, []
        for t in range(8):
            y_t, st = layer.step(x[:, t], st)
            ys.append(y_t.unsqueeze(1))
    assert _rel(torch.cat(ys, 1), y_all) < 1e-5
    for k in s_all:
        assert _rel(st[k], s_all[k]) < 1e-5, k


def test_block_stack_wiring(cpu_kernels):
    """BlockStack = pre-norm residual blocks, then the final norm (reference: src/orbit_ssm/model.py:51-118, 150-255)."""
    import torch.nn.functional as F
    from orbitssm_b200 import BlockStack, mamba2_config

    torch.manual_seed(5)
    cfg = mamba2_config(32, d_state=16, d_head=8)
    mixers = [SSDMimoSSM(cfg) for _ in range(2)]
    stack = BlockStack.from_mixers(mixers, 32)
    with torch.no_grad():
        for b in stack.layers:
            b.norm.weight.uniform_(0.5, 1.5)
        stack.norm_f.weight.uniform_(0.5, 1.5)
    x = torch.randn(2, 24, 32, requires_grad=True)
    y, states = stack(x, return_state=True)
    assert len(states) == 2 and y.shape == x.shape
    y.square().mean().backward()
    ref = x.detach().clone().requires_grad_(True)
    h = ref
    for b in stack.layers:
        h = h + b.mixer(F.rms_norm(h, (32,), b.norm.weight, b.norm.eps))
    yr = F.rms_norm(h, (32,), stack.norm_f.weight, stack.norm_f.eps)
    assert _rel(y, yr) < 1e-5
    g_norm = stack.norm_f.weight.grad.clone()
    stack.zero_grad()
    yr.square().mean().backward()
    assert _rel(x.grad, ref.grad) < 1e-4 and _rel(g_norm, stack.norm_f.weight.grad) < 1e-4
