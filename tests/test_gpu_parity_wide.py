"""-m gpu: value parity at the benchmark configurations' full WIDTH, and the 16-bit test policy over several input draws.

1. Every single-GPU benchmark configuration (2, 3, 4 and the config-5 layer) at its full width and head count on a
   [1, 512, d_model] slice of its input, bf16 activations over fp32 parameters on the tensor-core / coordinate-scan
   kernels, against the CPU oracle in fp64 on the same seeded inputs and weights: output, carried state, input
   gradient and every parameter gradient.
2. The reference's 16-bit policy (reference: tests/_tolerance.py:949-977, 1000-1075): at least five input draws per
   case; each draw within the bound, and the signed bias of each tensor pooled over the draws (additive:
   mean(a - e) / rms(e); gain: <a - e, e> / <e, e>) not systematically away from zero: a failure needs |mean| >= bound / 4,
   |t| > 3 and |trimmed mean| >= bound / 4 together.

Bounds (normwise relative error): about twice what these kernels measure (y 5e-3 .. 6e-3, carried state up to 8e-3, input
gradient up to 7e-3, parameter gradients up to 1.5e-2), inside the reference's own CUDA-vs-oracle bounds for bf16 (y 2.5e-2,
gradients 6e-2; reference: tests/test_ssd_endpoint.py:252-274, 303, 326).  Gradients of parameters with a handful of
elements (per-head scalars, 16 pair frequencies) are sums over every token with heavy cancellation, so their relative
error has a heavy tail from draw to draw; they follow the reference's typical-scale rule (reference:
tests/_tolerance.py:1035-1049): median over the draws within the bound (6e-2), no single draw beyond twice that.
"""
import math

import pytest
import torch

import bench
from conftest import load_golden
from oracle import hm_oracle, ssd_oracle
from orbitssm_b200 import HybridMambaConfig, HybridMambaSSM, SSDMimoConfig, SSDMimoSSM
from orbitssm_b200.config import resolve_ssd_spec

pytestmark = pytest.mark.gpu
DEV = "cuda"
BOUND_Y, BOUND_H, BOUND_DX, BOUND_G = 1.2e-2, 1.6e-2, 1.4e-2, 3e-2
SMALL, BOUND_SMALL = 256, 6e-2            # parameters with fewer elements than SMALL: typical-scale rule


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def signed_bias(a, e):
    a, e = a.detach().double().cpu().flatten(), e.detach().double().cpu().flatten()
    d = a - e
    ee = (e * e).sum().clamp_min(1e-300)
    return float(d.mean() / (ee / e.numel()).sqrt()), float((d * e).sum() / ee)


def oracle_run(layer, x, dy, gh):
    """fp64 CPU oracle of `layer` (same weights) on (x, dy): y, hidden state, dx and parameter gradients of
    sum(y * dy) + sum(hidden * gh)."""
    prm = {}
    for k, v in layer.state_dict().items():
        v = v.detach().cpu()
        prm[k] = v.double().requires_grad_(True) if (v.is_floating_point() and v.dim() > 0) else v
    xr = x.detach().double().cpu().requires_grad_(True)
    if isinstance(layer, HybridMambaSSM):
        yr, sr = hm_oracle.hm_layer(layer.config.to_dict(), prm, xr, None, True)
    else:
        yr, sr = ssd_oracle.ssd_layer(resolve_ssd_spec(layer.config), prm, xr, return_state=True)
    ((yr * dy.double().cpu()).sum() + (sr["hidden_state"] * gh.double().cpu()).sum()).backward()
    grads = {k: v.grad for k, v in prm.items() if torch.is_tensor(v) and v.requires_grad and v.grad is not None}
    return yr.detach(), sr["hidden_state"].detach(), xr.grad, grads


def gpu_run(layer, x, dy, gh):
    xx = x.to(DEV).to(torch.bfloat16).requires_grad_(True)
    layer.zero_grad()
    y, st = layer(xx, return_state=True)
    ((y.float() * dy.to(DEV)).sum() + (st["hidden_state"].float() * gh.to(DEV)).sum()).backward()
    grads = {n: p.grad for n, p in layer.named_parameters() if p.grad is not None}
    return y.detach(), st["hidden_state"].detach(), xx.grad, grads


def compare(got, want, what):
    """Returns {tensor name: (error, bound)}; asserts every bound."""
    y, h, dx, g = got
    yr, hr, dxr, gr = want
    out = {"y": (rel(y, yr), BOUND_Y), "hidden_state": (rel(h, hr), BOUND_H), "dx": (rel(dx, dxr), BOUND_DX)}
    for k, v in gr.items():
        assert k in g, (what, "missing gradient", k)
        # a single draw of a small parameter may sit in the tail: twice the typical-scale bound
        out["d " + k] = (rel(g[k], v), BOUND_G if v.numel() >= SMALL else 2 * BOUND_SMALL)
    print(what, {k: f"{e:.2e}" for k, (e, _) in out.items()})
    bad = {k: e for k, (e, b) in out.items() if not e < b}
    assert not bad, (what, "out of bound", bad)
    return out


@pytest.mark.parametrize("name", ["cfg2", "cfg5", "cfg3", "cfg4"])
def test_full_width_slice_matches_oracle(name):
    wl = bench.WORKLOADS[name]
    torch.manual_seed(0)
    layer = bench.make_mixer(bench.make_config(wl), execution={"precision": "io"})
    bench.init_params(layer)
    layer = layer.to(DEV)
    g = torch.Generator().manual_seed(11)
    # bf16-representable inputs, so that both sides see the same numbers
    x = torch.randn(1, 512, wl["d_model"], generator=g).to(torch.bfloat16).float()
    dy = torch.randn(1, 512, wl["d_model"], generator=g).to(torch.bfloat16).float()
    gh = torch.randn(1, layer.H, layer.P, layer.N, generator=g)
    got = gpu_run(layer, x, dy, gh)
    if not isinstance(layer, HybridMambaSSM):
        assert layer.last_route() == "tcgen05", layer.last_route()
    compare(got, oracle_run(layer, x, dy, gh), name + " [1,512,%d]" % wl["d_model"])


def _pooled_verdict(vals, bound):
    n = len(vals)
    mean = sum(vals) / n
    sd = math.sqrt(sum((v - mean) ** 2 for v in vals) / (n - 1))
    t = 0.0 if mean == 0.0 else (math.inf if sd == 0.0 else mean / (sd / math.sqrt(n)))
    k = int(0.10 * n)
    core = sorted(vals)[k:n - k]
    trimmed = sum(core) / len(core)
    lim = bound / 4
    return (abs(mean) >= lim and abs(t) > 3.0 and abs(trimmed) >= lim), mean, t


@pytest.mark.parametrize("case", ["cfg5_long", "cfg3_long", "hm_cfg4_long"])
def test_bf16_draws_within_bound_and_unbiased(case):
    rec = load_golden(case)
    if case.startswith("hm"):
        layer = HybridMambaSSM(HybridMambaConfig(**rec["config"]))
    else:
        layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]), execution={"precision": "io"})
    layer.load_state_dict(rec["state_dict"], strict=True)
    layer = layer.to(DEV)
    B, L, dm = rec["x"].shape
    pools, small = {}, {}
    for draw in range(5):
        g = torch.Generator().manual_seed(1000 + 7919 * draw)
        x = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).float()
        dy = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).float()
        gh = torch.randn(B, layer.H, layer.P, layer.N, generator=g)
        got = gpu_run(layer, x, dy, gh)
        want = oracle_run(layer, x, dy, gh)
        errs = compare(got, want, f"{case} draw {draw}")
        for k, v in want[3].items():
            if v.numel() < SMALL:
                small.setdefault(k, []).append(errs["d " + k][0])
        named = {"y": (got[0], want[0], BOUND_Y), "hidden_state": (got[1], want[1], BOUND_H), "dx": (got[2], want[2], BOUND_DX)}
        for k, v in want[3].items():
            if v.numel() >= SMALL:                    # a bias over a handful of elements is noise
                named["d " + k] = (got[3][k], v, BOUND_G)
        for k, (a, e, b) in named.items():
            add, gain = signed_bias(a, e)
            pools.setdefault(k, (b, [], []))
            pools[k][1].append(add)
            pools[k][2].append(gain)
    biased = {}
    for k, (b, adds, gains) in pools.items():
        for kind, vals in (("additive", adds), ("gain", gains)):
            fails, mean, t = _pooled_verdict(vals, b)
            if fails:
                biased[(k, kind)] = (mean, t, b / 4)
    assert not biased, ("systematic 16-bit bias (mean, t, limit)", biased)
    off = {k: sorted(v)[len(v) // 2] for k, v in small.items() if not sorted(v)[len(v) // 2] < BOUND_SMALL}
    assert not off, ("median error of a small parameter's gradient over the draws", off)
