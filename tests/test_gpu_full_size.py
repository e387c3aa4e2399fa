"""-m gpu: the layers at the benchmark configurations' full sizes, checked through size-independent properties (no CPU
checker finishes these sizes in seconds): a sequence run in two segments with the carried State equals the whole
sequence; repeated runs are bitwise identical; outputs and every gradient are finite; the scan is linear in the drive
path (the output gradient of 2*dy is twice the gradient of dy)."""
import pytest
import torch

import bench

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def build(name):
    wl = bench.WORKLOADS[name]
    torch.manual_seed(0)
    layer = bench.make_mixer(bench.make_config(wl), execution={"precision": "io"})
    bench.init_params(layer)
    return wl, layer.to(DEV)


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4"])
def test_full_size_properties(name):
    wl, layer = build(name)
    B, L, dm = wl["B"], wl["L"], wl["d_model"]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).to(DEV)
    dy = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).to(DEV)

    def run(xx, dd):
        xx = xx.clone().requires_grad_(True)
        for p in layer.parameters():
            p.grad = None
        y = layer(xx)
        y.backward(dd)
        return y.detach(), xx.grad.detach(), {n: p.grad.detach().clone() for n, p in layer.named_parameters() if p.grad is not None}

    y1, dx1, gw1 = run(x, dy)
    y2, dx2, gw2 = run(x, dy)
    assert torch.isfinite(y1.float()).all() and torch.isfinite(dx1.float()).all()
    assert torch.equal(y1, y2) and torch.equal(dx1, dx2), "not reproducible"
    for n in gw1:
        assert torch.isfinite(gw1[n]).all(), n
        assert torch.equal(gw1[n], gw2[n]), ("not reproducible", n)
    # the backward is linear in dy
    _, dx3, gw3 = run(x, dy * 2)
    assert rel(dx3.float(), 2 * dx1.float()) < 1e-2
    for n in ("in_proj.weight", "out_proj.weight"):
        assert rel(gw3[n], 2 * gw1[n]) < 1e-2, n
    # two segments with the carried State == the whole sequence (bf16 outputs: segment boundaries move chunk boundaries)
    with torch.no_grad():
        cut = L // 2 + 37
        ya, st = layer(x[:, :cut], return_state=True)
        yb, st2 = layer(x[:, cut:], state=st, return_state=True)
        y_all, st_all = layer(x, return_state=True)
    assert rel(torch.cat([ya, yb], 1).float(), y_all.float()) < 2e-2
    assert rel(st2["hidden_state"], st_all["hidden_state"]) < 2e-2
