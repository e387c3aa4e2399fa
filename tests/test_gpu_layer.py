"""-m gpu: the whole `SSDMimoSSM` layer on the CUDA kernels against vectors produced by the reference
(tests/golden/*.pt: fp64 oracle results for output, carried State and every gradient).

Bounds (normwise relative error), after the reference's own CUDA-vs-oracle bounds
(reference: tests/test_ssd_endpoint.py:252-274, 303, 326, 432-436):
  fp32 IO, precision "ieee":  y, state 2e-4;  gradients 5e-3
  bf16 IO (fp32 parameters, the training convention):  y, state 2.5e-2;  gradients 6e-2
"""
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from orbitssm_b200.config import SSDMimoConfig
from orbitssm_b200.ssd_mimo import SSDMimoSSM

pytestmark = pytest.mark.gpu
DEV = "cuda"
BOUNDS = {torch.float32: (2e-4, 5e-3), torch.bfloat16: (2.5e-2, 6e-2)}


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def build(rec, precision):
    layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]), execution={"precision": precision})
    layer.load_state_dict(rec["state_dict"], strict=True)
    return layer.to(DEV)


def run(layer, rec, x, dy, state, exact, io):
    x = x.to(DEV).to(io).requires_grad_(True)
    if state is not None:
        state = {k: v.to(DEV).float().requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    if exact:
        y = layer(x)
        (y.float() ** 2).mean().backward()
        st = None
    else:
        y, st = layer(x, state=state, return_state=True)
        loss = (y.float() * dy.to(DEV)).sum() + (st["hidden_state"] * rec["gh"].to(DEV)).sum()
        if "write_prev" in st:
            loss = loss + (st["write_prev"] * rec["gw"].to(DEV)).sum()
        loss.backward()
    grads = {n: p.grad for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad
    return y.detach(), st, grads


def check(got, want, bounds, what):
    y, st, grads = got
    ty, tg = bounds
    worst = {}
    assert rel(y, want["y"]) < ty, (what, "y", rel(y, want["y"]))
    if want.get("state") is not None:
        assert list(st) == list(want["state"])
        for k, v in want["state"].items():
            assert rel(st[k], v) < ty, (what, "state", k, rel(st[k], v))
    for k, v in want["grads"].items():
        assert k in grads, (what, "missing grad", k)
        worst[k] = rel(grads[k], v)
    bad = {k: e for k, e in worst.items() if not e < tg}
    assert not bad, (what, "gradients out of bound", bad)


@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_layer_matches_reference(name, io):
    rec = load_golden(name)
    layer = build(rec, "ieee" if io == torch.float32 else "io")
    got = run(layer, rec, rec["x"], rec["dy"], None, rec["exact"], io)
    check(got, rec["f64"], BOUNDS[io], name)
    if "f64_cont" in rec:
        c = rec["f64_cont"]
        s = c["split"]
        got = run(layer, rec, rec["x"][:, s:], rec["dy"][:, s:], c["state_in"], False, io)
        check(got, c, BOUNDS[io], name + " continuation")


def test_config1_known_answer():
    rec = load_golden("cfg1_exact")
    layer = build(rec, "ieee")
    y = layer(rec["x"].to(DEV))
    got = float((y.double() ** 2).mean())
    assert abs(got - rec["mean_y2_f32"]) < 1e-4 * rec["mean_y2_f32"]


def test_autocast_convention():
    """fp32 input and parameters under bf16 autocast: the training convention of the reference's benchmarks."""
    rec = load_golden("cfg2_small")
    layer = build(rec, "io")
    x = rec["x"].to(DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = layer(x)
    assert y.dtype == torch.bfloat16
    assert rel(y, rec["f64"]["y"]) < 2.5e-2


def test_split_equals_whole_and_is_reproducible():
    rec = load_golden("dyn_trap_conv")
    layer = build(rec, "ieee")
    x = rec["x"].to(DEV)
    y_all, s_all = layer(x, return_state=True)
    y_again, _ = layer(x, return_state=True)
    assert torch.equal(y_all, y_again)
    st, ys = None, []
    for a, b in ((0, 5), (5, 6), (6, 6), (6, 37)):
        y, st = layer(x[:, a:b], state=st, return_state=True)
        ys.append(y)
    assert rel(torch.cat(ys, 1), y_all) < 1e-5
    for k in s_all:
        assert rel(st[k], s_all[k]) < 1e-5, k


# ---------------------------------------------------------------------------------------------------- HybridMamba
from conftest import HM_GOLDEN_CASES                                    # noqa: E402
from orbitssm_b200.config import HybridMambaConfig                      # noqa: E402
from orbitssm_b200.hybrid_mamba import HybridMambaSSM                   # noqa: E402


def run_hm(layer, rec, x, dy, state, io):
    x = x.to(DEV).to(io).requires_grad_(True)
    if state is not None:
        state = {k: v.to(DEV).float().requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    y, st = layer(x, state=state, return_state=True)
    loss = (y.float() * dy.to(DEV)).sum()
    for k, g in rec["gs"].items():
        if k in st:
            loss = loss + (st[k] * g.to(DEV)).sum()
    loss.backward()
    grads = {n: p.grad for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad
    return y.detach(), st, grads


@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", HM_GOLDEN_CASES)
def test_hm_layer_matches_reference(name, io):
    """The whole `HybridMambaSSM` layer on the CUDA kernels against the reference's fp64 results (same bounds as the
    SSD layer), first segment and continuation from the reference's own carried State."""
    rec = load_golden(name)
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    layer.load_state_dict(rec["state_dict"], strict=True)
    layer = layer.to(DEV)
    got = run_hm(layer, rec, rec["x"], rec["dy"], None, io)
    check(got, rec["f64"], BOUNDS[io], name)
    c = rec["f64_cont"]
    s = c["split"]
    got = run_hm(layer, rec, rec["x"][:, s:], rec["dy"][:, s:], c["state_in"], io)
    check(got, c, BOUNDS[io], name + " continuation")


def test_hm_split_equals_whole_and_is_reproducible():
    rec = load_golden("hm_small")
    layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    layer.load_state_dict(rec["state_dict"], strict=True)
    layer = layer.to(DEV)
    x = rec["x"].to(DEV)
    y_all, s_all = layer(x, return_state=True)
    y_again, _ = layer(x, return_state=True)
    assert torch.equal(y_all, y_again)
    st, ys = None, []
    for a, b in ((0, 5), (5, 6), (6, 33), (33, 40)):
        y, st = layer(x[:, a:b], state=st, return_state=True)
        ys.append(y)
    assert rel(torch.cat(ys, 1), y_all) < 1e-5
    for k in s_all:
        assert rel(st[k], s_all[k]) < 1e-5, k


@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_block_stack_norms_match_aten(io, monkeypatch):
    """BlockStack (pre-norm residual blocks + final norm) with its norms on this package's kernels against the same
    stack with ATen's rms_norm (reference: src/orbit_ssm/model.py:51-118, 150-255; layers/norms.py:10-58)."""
    import torch.nn.functional as F
    from orbitssm_b200 import BlockStack, mamba2_config, model

    torch.manual_seed(3)
    cfg = mamba2_config(128, d_state=128, d_head=64)
    precision = "ieee" if io == torch.float32 else "io"
    mixers = [SSDMimoSSM(cfg, execution={"precision": precision}) for _ in range(2)]
    stack = BlockStack.from_mixers(mixers, 128).to(DEV)
    with torch.no_grad():
        for b in stack.layers:
            b.norm.weight.uniform_(0.5, 1.5)
        stack.norm_f.weight.uniform_(0.5, 1.5)
    x = torch.randn(2, 200, 128, device=DEV).to(io)
    dy = torch.randn(2, 200, 128, device=DEV).to(io)

    def run_once():
        xx = x.clone().requires_grad_(True)
        stack.zero_grad()
        y = stack(xx)
        y.backward(dy)
        return y, xx.grad, stack.norm_f.weight.grad.clone(), stack.layers[0].norm.weight.grad.clone()

    got = run_once()
    monkeypatch.setattr(model.RMSNorm, "forward",
                        lambda self, t: F.rms_norm(t.float(), self.weight.shape, self.weight, self.eps).to(t.dtype))
    want = run_once()
    tol = 1e-4 if io == torch.float32 else 3e-2
    for g, w, what in zip(got, want, ("y", "dx", "d norm_f.weight", "d layers[0].norm.weight")):
        assert rel(g, w) < tol, (what, rel(g, w))


@pytest.mark.parametrize("name,io", [("dyn_trap_conv", torch.float32), ("cfg2_small", torch.float32), ("cfg2_small", torch.bfloat16),
                                     ("cfg3_small", torch.bfloat16)])
def test_step_equals_forward_on_device(name, io):
    """Decoding: `step` under no_grad (the one-launch step kernel for the scan of the token) token by token from a carried
    State equals `forward` on the same tokens, for the output and every carry (reference contract:
    src/orbit_ssm/ssm/ssd_mimo_torch.py:388-490)."""
    rec = load_golden(name)
    layer = build(rec, "ieee" if io == torch.float32 else "io")
    x = rec["x"][:, :12].to(DEV).to(io)
    with torch.no_grad():
        y_all, s_all = layer(x, return_state=True)
        y_head, st = layer(x[:, :7], return_state=True)
        ys = [y_head]
        for t in range(7, 12):
            y_t, st = layer.step(x[:, t], st)
            assert layer.last_route() == "step"
            ys.append(y_t.unsqueeze(1))
    ty = 1e-5 if io == torch.float32 else 2.5e-2
    assert rel(torch.cat(ys, 1), y_all) < ty, rel(torch.cat(ys, 1), y_all)
    for k in s_all:
        assert rel(st[k], s_all[k]) < ty, (k, rel(st[k], s_all[k]))


def test_graphed_training_step_equals_eager():
    """One captured forward + backward (CUDA graph, static buffers) replayed on two different inputs against the same
    steps run eagerly: output, input gradient and every parameter gradient (reference: src/orbit_ssm/graphs.py:449)."""
    from orbitssm_b200 import BlockStack, GraphedStep, mamba2_config
    torch.manual_seed(3)
    cfg = mamba2_config(128, d_state=128, d_head=64)
    stack = BlockStack.from_mixers([SSDMimoSSM(cfg, execution={"precision": "io"}) for _ in range(2)], 128).to(DEV)
    xs = [torch.randn(2, 300, 128, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    dys = [torch.randn(2, 300, 128, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    g = GraphedStep(stack, xs[0], dys[0], amp_dtype=torch.bfloat16)
    # the eager comparison below runs on another stream than the one the capture made the gradient accumulators on
    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
    for x, dy in zip(xs, dys):
        y = g.step(x, dy).clone()
        got = {n: p.grad.clone() for n, p in stack.named_parameters()}      # step() re-attaches its static gradient buffers
        gx = g.x_grad.clone()
        for p in stack.parameters():
            p.grad = None
        xe = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            ye = stack(xe)
        ye.backward(dy)
        assert rel(y, ye) < 1e-3 and rel(gx, xe.grad) < 1e-3
        for n, p in stack.named_parameters():
            assert rel(got[n], p.grad) < 1e-3, n
        for p in stack.parameters():
            p.grad = None


def test_graphed_decode_equals_eager_steps():
    """Decode steps replayed from one CUDA graph with the State at fixed addresses against eager `step` calls."""
    from orbitssm_b200 import BlockStack, GraphedDecode, mamba2_config
    torch.manual_seed(4)
    cfg = mamba2_config(128, d_state=128, d_head=64)
    stack = BlockStack.from_mixers([SSDMimoSSM(cfg, execution={"precision": "io"}) for _ in range(2)], 128).to(DEV)
    x = torch.randn(3, 6, 128, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        st, ys = None, []
        for t in range(x.shape[1]):
            y_t, st = stack.step(x[:, t], st)
            ys.append(y_t)
    dec = GraphedDecode(stack, 3, device=DEV, dtype=torch.bfloat16)
    for t in range(x.shape[1]):
        y_t = dec.step(x[:, t])
        assert rel(y_t, ys[t]) < 1e-3, t
    for a_, b_ in zip(dec.state, st):
        for k in b_:
            assert rel(a_[k], b_[k]) < 1e-3, k


@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_input_forms(io):
    """What a caller may hand the layer besides a contiguous, grad-requiring input: strided views (every other token, a
    column window of a wider tensor), an input without gradient, `no_grad` / `inference_mode`, and an output gradient that
    is an expanded scalar (`y.sum().backward()`: every stride 0).  Each must give what the contiguous call gives: outputs
    bit for bit, gradients to rounding (the library GEMMs may pick another split for another operand layout)."""
    rec = load_golden("cfg2_long")
    layer = build(rec, "ieee" if io == torch.float32 else "io")
    x0 = rec["x"].to(DEV).to(io)
    B, L, D = x0.shape
    tol = 1e-5 if io == torch.float32 else 1e-2

    def grads_of(x, loss_of):
        layer.zero_grad()
        y = layer(x)
        loss_of(y).backward()
        return y.detach(), {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}

    def same(got, want, what):
        for n in want:
            assert rel(got[n], want[n]) < tol, (what, n, rel(got[n], want[n]))

    xc = x0.clone().requires_grad_(True)
    y_ref, g_ref = grads_of(xc, lambda y: (y * torch.ones_like(y)).sum())
    dx_ref = xc.grad.clone()
    # the same gradient as an expanded scalar
    xc2 = x0.clone().requires_grad_(True)
    y2, g2 = grads_of(xc2, lambda y: y.sum())
    assert torch.equal(y2, y_ref) and rel(xc2.grad, dx_ref) < tol
    same(g2, g_ref, "expanded output gradient")
    # strided views of the same values
    wide = torch.zeros(B, 2 * L, D + 16, device=DEV, dtype=io)
    wide[:, ::2, 8:8 + D] = x0
    xs = wide[:, ::2, 8:8 + D].detach().requires_grad_(True)
    assert not xs.is_contiguous()
    y3, g3 = grads_of(xs, lambda y: (y * torch.ones_like(y)).sum())
    assert torch.equal(y3, y_ref) and rel(xs.grad, dx_ref) < tol
    same(g3, g_ref, "strided input")
    # no input gradient wanted
    y4, g4 = grads_of(x0.clone(), lambda y: (y * torch.ones_like(y)).sum())
    assert torch.equal(y4, y_ref)
    same(g4, g_ref, "input without gradient")
    with torch.no_grad():
        assert torch.equal(layer(x0), y_ref)
    with torch.inference_mode():
        assert torch.equal(layer(x0), y_ref)
