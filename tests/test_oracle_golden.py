"""Pins the CPU checker (oracle/ssd_oracle.py) to vectors produced by running the reference itself."""
import pytest
import torch

from conftest import GOLDEN_CASES, HM_GOLDEN_CASES, load_golden
from orbitssm_b200.config import SSDMimoConfig, resolve_ssd_spec
from oracle import hm_oracle as HM
from oracle import ssd_oracle as O


def _rel(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def _run(spec, prm, x, dy, gh, gw, state, exact, route, chunk=None):
    prm = {k: v.double().requires_grad_(v.is_floating_point()) for k, v in prm.items()}
    x = x.double().requires_grad_(True)
    if state is not None:
        state = {k: v.double().requires_grad_(True) for k, v in state.items()}
    if exact:
        y = O.ssd_layer(spec, prm, x, route=route, chunk=chunk)
        (y ** 2).mean().backward()
        st = None
    else:
        y, st = O.ssd_layer(spec, prm, x, state=state, return_state=True, route=route, chunk=chunk)
        loss = (y * dy.double()).sum() + (st["hidden_state"] * gh.double()).sum()
        if "write_prev" in st:
            loss = loss + (st["write_prev"] * gw.double()).sum()
        loss.backward()
    grads = {k: v.grad for k, v in prm.items() if v.is_floating_point() and v.grad is not None}
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
        assert set(st) == set(want["state"]), (what, set(st), set(want["state"]))
        for k, v in want["state"].items():
            assert st[k].shape == v.shape
            assert _rel(st[k].detach(), v) < tol, (what, "state", k, _rel(st[k].detach(), v))
    for k, v in want["grads"].items():
        assert k in grads, (what, "missing grad", k)
        assert _rel(grads[k], v) < tol, (what, "grad", k, _rel(grads[k], v))


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("route", ["chunked", "recurrent"])
def test_oracle_matches_reference_fp64(name, route):
    rec = load_golden(name)
    if route == "recurrent" and rec["x"].shape[1] > 100:
        pytest.skip("token loop kept to short cases")
    spec = resolve_ssd_spec(SSDMimoConfig(**rec["config"]))
    got = _run(spec, rec["state_dict"], rec["x"], rec["dy"], rec["gh"], rec["gw"], None, rec["exact"], route)
    _check(got, rec["f64"], 1e-9, name)
    if "f64_cont" in rec:
        c = rec["f64_cont"]
        s = c["split"]
        got = _run(spec, rec["state_dict"], rec["x"][:, s:], rec["dy"][:, s:], rec["gh"], rec["gw"], c["state_in"],
                   False, route)
        _check(got, c, 1e-9, name + " continuation")


def test_config1_known_answer():
    """Benchmark configuration 1: seed 0 default init, x = randn(2,256,64): mean(y^2) recorded from the reference."""
    rec = load_golden("cfg1_exact")
    spec = resolve_ssd_spec(SSDMimoConfig(**rec["config"]))
    y = O.ssd_layer(spec, rec["state_dict"], rec["x"])
    assert abs(float((y ** 2).mean()) - rec["mean_y2_f32"]) < 1e-6 * rec["mean_y2_f32"] + 1e-9


@pytest.mark.parametrize("chunk", [1, 7, 16, 64])
def test_chunk_length_is_scheduling_only(chunk):
    rec = load_golden("dyn_trap_conv")
    spec = resolve_ssd_spec(SSDMimoConfig(**rec["config"]))
    prm = {k: v.double() for k, v in rec["state_dict"].items()}
    y0, s0 = O.ssd_layer(spec, prm, rec["x"].double(), return_state=True, route="recurrent")
    y1, s1 = O.ssd_layer(spec, prm, rec["x"].double(), return_state=True, chunk=chunk)
    assert _rel(y1, y0) < 1e-10
    for k in s0:
        assert _rel(s1[k], s0[k]) < 1e-10


def test_empty_and_single_token():
    rec = load_golden("euler_r2o1")
    spec = resolve_ssd_spec(SSDMimoConfig(**rec["config"]))
    prm = {k: v.double() for k, v in rec["state_dict"].items()}
    x = rec["x"].double()
    y_all, s_all = O.ssd_layer(spec, prm, x, return_state=True)
    st, ys = None, []
    for t in range(x.shape[1]):
        y, st = O.ssd_layer(spec, prm, x[:, t:t + 1], state=st, return_state=True)
        ys.append(y)
    assert _rel(torch.cat(ys, 1), y_all) < 1e-10
    assert _rel(st["hidden_state"], s_all["hidden_state"]) < 1e-10
    y0, s0 = O.ssd_layer(spec, prm, x[:, :0], state=s_all, return_state=True)
    assert y0.shape[1] == 0 and torch.equal(s0["hidden_state"], s_all["hidden_state"].reshape(s0["hidden_state"].shape))


# ---------------------------------------------------------------------------------------------------- HybridMamba
def _run_hm(cfg, prm, x, dy, gs, state):
    prm = {k: v.double().requires_grad_(v.is_floating_point() and v.dim() > 0) for k, v in prm.items()}
    x = x.double().requires_grad_(True)
    if state is not None:
        state = {k: v.double().requires_grad_(True) for k, v in state.items()}
    y, st = HM.hm_layer(cfg, prm, x, state, True)
    loss = (y * dy.double()).sum()
    for k, g in gs.items():
        if k in st:
            loss = loss + (st[k] * g.double()).sum()
    loss.backward()
    grads = {k: v.grad for k, v in prm.items() if v.grad is not None}
    grads["x"] = x.grad
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad
    return y.detach(), st, grads


@pytest.mark.parametrize("name", HM_GOLDEN_CASES)
def test_hm_oracle_matches_reference_fp64(name):
    """oracle/hm_oracle.py against the reference's own fp64 results: output, every carry, every gradient, and a
    continuation segment started from the first segment's State."""
    rec = load_golden(name)
    got = _run_hm(rec["config"], rec["state_dict"], rec["x"], rec["dy"], rec["gs"], None)
    _check(got, rec["f64"], 1e-9, name)
    c = rec["f64_cont"]
    s = c["split"]
    got = _run_hm(rec["config"], rec["state_dict"], rec["x"][:, s:], rec["dy"][:, s:], rec["gs"], c["state_in"])
    _check(got, c, 1e-9, name + " continuation")
