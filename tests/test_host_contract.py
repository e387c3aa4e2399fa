"""Host-side contracts that need no GPU: the carry dtype law, first-order-only backward passes, the no-silent-demotion
rule, token stepping through the containers, and this package's layer dropped into the reference's own `CausalLM`
(where the reference checkout is present).  Kernels are replaced by their torch restatements, as in
test_layer_host_logic.py."""
import os
import sys
import warnings

import pytest
import torch

from conftest import load_golden
from test_layer_host_logic import _layer, _rel, cpu_hm_kernels, cpu_kernels  # noqa: F401  (fixtures)
from orbitssm_b200 import BlockStack, HybridMambaConfig, HybridMambaSSM, SSDMimoConfig, SSDMimoSSM, State, mamba2_config

# the reference checkout: $ORBIT_REFERENCE, else a directory "reference" beside this repository
REFERENCE = os.environ.get("ORBIT_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


# ---------------------------------------------------------------------------------------------------- carries
def test_phase_carries_never_drop_below_fp32(cpu_hm_kernels):
    """reference: src/orbit_ssm/layers/state.py:28, 87, 149"""
    rec = load_golden("hm_small")
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    layer.load_state_dict(rec["state_dict"], strict=True)
    st = layer.init_state(2, dtype=torch.bfloat16)
    assert st["hidden_state"].dtype == torch.bfloat16 and st["theta"].dtype == torch.float32
    moved = State(st).to(dtype=torch.bfloat16)
    assert moved["theta"].dtype == torch.float32 and moved["conv_state"].dtype == torch.bfloat16
    assert State(st).to(dtype=torch.float64)["theta"].dtype == torch.float64
    bad = State(st)
    bad["theta"] = st["theta"].to(torch.bfloat16)
    with pytest.raises(TypeError, match="phase"):
        layer.validate_state(bad)
    _, out = layer(rec["x"], state=st, return_state=True)
    assert out["theta"].dtype == torch.float32 and out["hidden_state"].dtype == torch.bfloat16


def test_state_checks_name_the_offending_carry(cpu_kernels):
    layer = _layer(load_golden("dyn_trap_conv"))
    st = layer.init_state(2)
    with pytest.raises(ValueError, match="absent"):
        layer.validate_state({"hidden_state": st["hidden_state"]})
    wrong = State(st)
    wrong["conv_state"] = st["conv_state"][:, :-1]
    with pytest.raises(ValueError, match="conv_state"):
        layer.validate_state(wrong)
    with pytest.raises(ValueError, match="not carries"):
        layer.init_state(2, overrides={"nope": torch.zeros(1)})
    with pytest.raises(ValueError, match="seeded twice"):
        layer.init_state(2, h_init=st["hidden_state"], overrides={"hidden_state": st["hidden_state"]})
    with pytest.raises(ValueError, match="not both"):
        layer.resolve_state(st, batch_size=2, device="cpu", h_init=st["hidden_state"])
    with pytest.raises(ValueError, match="int64"):
        st.index_select(torch.tensor([0.0]))
    one = st.index_select(torch.tensor([1]))
    assert one["hidden_state"].shape[0] == 1
    seeded = layer.init_state(2, h_init=torch.ones(layer.H, layer.P, layer.N))
    assert float(seeded["hidden_state"].min()) == 1.0 and seeded["hidden_state"].shape[0] == 2


# ---------------------------------------------------------------------------------------------------- autograd
def test_double_backward_raises_by_name(cpu_kernels):
    """reference: src/orbit_ssm/kernels/autograd_guard.py (second derivatives through a kernel backward must not be
    silently wrong)."""
    layer = _layer(load_golden("euler_r2o1"))
    x = load_golden("euler_r2o1")["x"].clone().requires_grad_(True)
    y = layer(x)
    (g,) = torch.autograd.grad(y.square().sum(), x, create_graph=True)
    assert g.requires_grad
    with pytest.raises(RuntimeError, match="second-order"):
        g.square().sum().backward()
    # an ordinary backward is untouched
    x2 = x.detach().clone().requires_grad_(True)
    layer(x2).square().sum().backward()
    assert _rel(x2.grad, g) < 1e-6


# ---------------------------------------------------------------------------------------------------- routes
def test_fp32_route_of_a_tensor_core_request_warns_once(monkeypatch):
    """reference: src/orbit_ssm/layers/routes.py:33-48 (no silent demotion)."""
    from orbitssm_b200 import ops, ssd_mimo
    monkeypatch.setattr(ops, "pick_chunk", lambda geo, precision, backward, limit: 0 if precision == 1 else 16)
    monkeypatch.setattr(ssd_mimo, "_WARNED_ROUTES", set())
    layer = SSDMimoSSM(SSDMimoConfig(d_model=32, d_state=16, n_groups=8))          # G = 8, N = 16: outside both envelopes
    geo = ops.ScanGeometry(H=layer.H, R=1, O=1, G=8, N=16)
    with pytest.warns(ssd_mimo.NonTensorCoreRouteWarning, match="runs on the fp32 kernels"):
        layer._route(torch.bfloat16, geo, True)
    assert "fp32" in layer.last_route()
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        layer._route(torch.bfloat16, geo, True)                                     # second time: silent
        layer.set_execution({"precision": "ieee"})
        layer._route(torch.bfloat16, geo, True)                                     # asked for fp32: nothing to say
    monkeypatch.setattr(ops, "pick_chunk", lambda *a: 0)
    with pytest.raises(NotImplementedError, match="shared memory"):
        layer._route(torch.float32, geo, True)


# ---------------------------------------------------------------------------------------------------- containers
def test_stack_step_equals_forward(cpu_kernels):
    """Stepping token by token through `ResidualBlock.step` / `BlockStack.step` equals the sequence at once
    (reference: src/orbit_ssm/model.py:110-115)."""
    torch.manual_seed(7)
    cfg = mamba2_config(32, d_state=16, d_head=8)
    stack = BlockStack.from_mixers([SSDMimoSSM(cfg) for _ in range(2)], 32)
    x = torch.randn(2, 7, 32)
    with torch.no_grad():
        y_all, s_all = stack(x, return_state=True)
        st, ys = None, []
        for t in range(x.shape[1]):
            y_t, st = stack.step(x[:, t], st)
            ys.append(y_t.unsqueeze(1))
    assert _rel(torch.cat(ys, 1), y_all) < 1e-5
    for a, b in zip(st, s_all):
        for k in b:
            assert _rel(a[k], b[k]) < 1e-5, k
    with pytest.raises(ValueError):
        stack.step(x[:, 0], [None])


# ---------------------------------------------------------------------------------------------------- drop-in
@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "src", "orbit_ssm")), reason="reference checkout not present")
def test_layer_drops_into_the_reference_causal_lm(cpu_kernels):
    """`CausalLM.register_mixer` (reference: src/orbit_ssm/model.py:568-586) builds this package's `SSDMimoSSM` inside the
    reference's own CausalLM / BlockStack / ResidualBlock; with the reference model's weights loaded (strict) the logits,
    the carried states and the parameter gradients match the reference's `backend="torch"` model."""
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(REFERENCE, "src"))
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from orbit_ssm import SSDMimoConfig as RefConfig
            from orbit_ssm.model import CausalLM
    finally:
        sys.path.remove(os.path.join(REFERENCE, "src"))
    opts = dict(d_state=16, expand=2.0, d_conv=4, n_groups=8, bc_conv=True, out_norm=True)
    if "orbit_b200_ssd" not in CausalLM.registered_mixers():
        CausalLM.register_mixer("orbit_b200_ssd", lambda d_model, **kw: SSDMimoSSM(SSDMimoConfig(d_model=d_model, **kw)))
    torch.manual_seed(0)
    ours = CausalLM(vocab_size=50, d_model=32, n_layers=2, layers={"type": "orbit_b200_ssd", **opts})
    torch.manual_seed(0)
    ref = CausalLM(vocab_size=50, d_model=32, n_layers=2, layers=RefConfig(d_model=32, **opts), execution={"backend": "torch"})
    assert isinstance(ours.backbone.layers[0].mixer, SSDMimoSSM)
    assert list(ours.state_dict()) == list(ref.state_dict())
    ours.load_state_dict(ref.state_dict(), strict=True)
    ids = torch.randint(0, 50, (2, 19), generator=torch.Generator().manual_seed(3))
    lo, so = ours(ids, return_state=True)
    lr, sr = ref(ids, return_state=True)
    assert _rel(lo, lr) < 1e-4
    for a, b in zip(so, sr):
        assert list(a) == list(b)
        for k in b:
            assert _rel(a[k], b[k]) < 1e-4, k
    lo.square().mean().backward()
    lr.square().mean().backward()
    go, gr = dict(ours.named_parameters()), dict(ref.named_parameters())
    for k, p in gr.items():
        if p.grad is not None:
            assert go[k].grad is not None and _rel(go[k].grad, p.grad) < 2e-3, k
    # a continued call from the carried states
    l2o = ours(ids, state=[State(s).detach() for s in so])
    l2r = ref(ids, state=[s.detach() for s in sr])
    assert _rel(l2o, l2r) < 1e-4


def test_graph_capture_refuses_by_name_without_cuda():
    """No silent eager fallback: where a step cannot be captured the helpers raise `CaptureError` with a reason tag
    (reference: src/orbit_ssm/graphs.py:449, `graphed_step` refuses instead of running eagerly)."""
    import torch
    from orbitssm_b200 import CaptureError, GraphedDecode, GraphedStep
    if torch.cuda.is_available():
        pytest.skip("needs a host without CUDA")
    lin = torch.nn.Linear(4, 4)
    with pytest.raises(CaptureError) as e:
        GraphedStep(lin, torch.zeros(2, 4))
    assert e.value.reason == "no-cuda"
    with pytest.raises(CaptureError) as e:
        GraphedDecode(lin, 2)
    assert e.value.reason == "no-cuda"
