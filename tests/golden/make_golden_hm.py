"""Generate the HybridMamba golden vectors under tests/golden/ by RUNNING THE REFERENCE ITSELF on CPU.

    python tests/golden/make_golden_hm.py /path/to/reference [case ...]      (no case names = all of them)

Same recipe as make_golden.py, for `HybridMambaSSM` (`backend="torch"`): config, the reference layer's ``state_dict``
(every parameter moved off its init value), seeded inputs, and the reference's fp64 / fp32 results: output, carried
State (hidden_state, theta, write_prev, conv_state), gradients of ``sum(y*dy) + sum(hidden*gh) + sum(write_prev*gw) +
sum(theta*gt)`` with respect to the input, every parameter and every supplied carry, plus a continuation segment started
from the first segment's State.  Nothing here is imported by the tests; they only read the ``.pt`` files.
"""
import os
import sys
import warnings

import torch

if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/the/reference/checkout")
REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, REF + "/src")
warnings.filterwarnings("ignore")

from orbit_ssm import HybridMambaSSM, HybridMambaConfig          # noqa: E402  (the reference package)

OUT = os.path.dirname(os.path.abspath(__file__))
HALF = [{"frac": .5, "decay": "coord_static"}, {"frac": .5, "decay": "coord_static", "complex": True}]
CASES = {
    # benchmark configuration 4's structure (half real rows, half rotating pairs, trapezoid, gated RMSNorm) at toy width
    "hm_small": dict(cfg=dict(d_model=64, d_state=16, expand=2, d_conv=4, out_norm=True, d_head=16, row_blocks=HALF),
                     B=2, L=40, split=17),
    # config 4's head geometry (P = 64, N = 64: 32 real rows + 16 pairs) at 2 heads
    "hm_cfg4_small": dict(cfg=dict(d_model=64, d_state=64, expand=2, d_conv=4, out_norm=True, row_blocks=HALF),
                          B=1, L=48, split=20),
    # the same geometry over ten 32-token checkpoint intervals of the backward kernel, cut at 143 = 4 * 32 + 15
    "hm_cfg4_long": dict(cfg=dict(d_model=64, d_state=64, expand=2, d_conv=4, out_norm=True, row_blocks=HALF),
                         B=1, L=320, split=143),
    # Euler write, real rows only, no output norm (gate, then out_proj)
    "hm_euler": dict(cfg=dict(d_model=32, d_state=8, expand=1, d_conv=3, out_norm=False, d_head=8, write_rule="euler",
                              row_blocks=[{"frac": 1.0, "decay": "coord_static"}]), B=2, L=19, split=7),
}


def build(case, dtype):
    torch.manual_seed(0)
    cfg = HybridMambaConfig(**case["cfg"])
    layer = HybridMambaSSM(cfg, execution={"backend": "torch"})
    fresh = {k: v.clone() for k, v in layer.state_dict().items()}
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in layer.parameters():
            p.add_(0.05 * torch.randn(p.shape, generator=g) * (1.0 + p.abs()))
        # keep rotating pairs tied (one modulus per pair is a property of the stored layout: nothing to re-tie)
    return cfg, layer.to(dtype), fresh


def run(layer, x, dy, state, gs):
    x = x.clone().requires_grad_(True)
    if state is not None:
        state = {k: v.clone().requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    y, st = layer(x, state=state, return_state=True)
    loss = (y * dy).sum()
    for k, g in gs.items():
        if k in st:
            loss = loss + (st[k] * g.to(st[k].dtype)).sum()
    loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad.detach().clone()
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad.detach().clone()
    return y.detach(), {k: v.detach().clone() for k, v in st.items()}, grads


def main():
    only = set(sys.argv[2:])
    for name, case in CASES.items():
        if only and name not in only:
            continue
        rec = {}
        for tag, dtype in (("f64", torch.float64), ("f32", torch.float32)):
            cfg, layer, fresh = build(case, dtype)
            g = torch.Generator().manual_seed(2)
            x = torch.randn(case["B"], case["L"], cfg.d_model, generator=g)
            dy = torch.randn(case["B"], case["L"], cfg.d_model, generator=g)
            probe = layer.init_state(case["B"])
            gs = {k: torch.randn(v.shape, generator=g) for k, v in probe.items() if k != "conv_state"}
            if tag == "f64":
                rec["config"] = dict(case["cfg"])
                rec["state_dict"] = {k: v.float() for k, v in layer.state_dict().items()}
                rec["fresh_state_dict"] = {k: v.float() for k, v in fresh.items()}     # default init under seed 0
                rec["x"], rec["dy"], rec["gs"] = x, dy, gs
                rec["state_keys"] = {k: tuple(v.shape) for k, v in probe.items()}
            gsd = {k: v.to(dtype) for k, v in gs.items()}
            y, st, grads = run(layer, x.to(dtype), dy.to(dtype), None, gsd)
            rec[tag] = dict(y=y, state=st, grads=grads) if tag == "f64" else dict(y=y, state=st)
            s = case["split"]
            _, st1, _ = run(layer, x[:, :s].to(dtype), dy[:, :s].to(dtype), None, gsd)
            y2, st2, grads2 = run(layer, x[:, s:].to(dtype), dy[:, s:].to(dtype), st1, gsd)
            if tag == "f64":
                rec["f64_cont"] = dict(split=s, state_in=st1, y=y2, state=st2, grads=grads2)
        torch.save(rec, os.path.join(OUT, name + ".pt"))
        print(name, rec["state_keys"], {k: tuple(v.shape) for k, v in rec["state_dict"].items()},
              os.path.getsize(os.path.join(OUT, name + ".pt")) // 1024, "KiB")


if __name__ == "__main__":
    main()
