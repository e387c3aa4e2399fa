"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE ITSELF on CPU.

Usage (only where the reference checkout is available; the fixtures it writes are committed):

    python tests/golden/make_golden.py /path/to/reference [case ...]      (no case names = all of them)

Every fixture is one ``torch.save`` dict: the config (field names shared by the reference's `SSDMimoConfig` and
this package's), the reference layer's ``state_dict`` (every parameter moved off its init value so that
zero-initialised projections take part), the seeded inputs, and what the reference's ``backend="torch"`` route
returned for them in fp64 (the oracle precision) and fp32: output, carried State, gradients of
``sum(y*dy) + sum(hidden*gh) (+ sum(write_prev*gw))`` with respect to the input, every parameter and every
supplied carry.  Nothing here is imported by the tests; they only read the ``.pt`` files.
"""
import sys
import warnings

import torch

if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/the/reference/checkout")
REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, REF + "/src")
warnings.filterwarnings("ignore")

from orbit_ssm import SSDMimoSSM, SSDMimoConfig          # noqa: E402  (the reference package)
from orbit_ssm.presets import mamba2_config              # noqa: E402

import os                                                 # noqa: E402
OUT = os.path.dirname(os.path.abspath(__file__))

HS = [{"frac": 1.0, "decay": "head_static"}]
CASES = {
    # Benchmark configuration 1 exactly: default init under seed 0, x = randn(2, 256, 64), loss mean(y^2)
    "cfg1_exact": dict(cfg=dict(d_model=64, d_state=16, expand=1.0, d_conv=0, d_ssm_in=1, d_ssm_out=1, n_groups=16),
                       B=2, L=256, exact=True),
    # config-2 geometry (Mamba-2 preset: P=64, N=128, Euler, joint B|C conv, output norm) at 2 heads
    "cfg2_small": dict(preset=dict(d_model=64, d_state=128, d_head=64), B=1, L=96, split=40),
    # config-3 geometry (R=O=4, G=16, N=128, trapezoid, gates, per-(h,r) biases, dynamic sibling mix) at 2 heads
    "cfg3_small": dict(cfg=dict(d_model=64, expand=2.0, d_state=128, d_ssm_in=4, d_ssm_out=4, n_heads=2, d_head=64,
                                d_conv=4, write_rule="trapezoid", row_blocks=HS), B=1, L=80, split=33),
    # option coverage at toy sizes
    "dyn_trap_conv": dict(cfg=dict(d_model=32, d_state=16, expand=2.0, d_conv=4, n_groups=8, bc_conv=True,
                                   out_norm=True), B=2, L=37, split=19),
    "softplus_sib": dict(cfg=dict(d_model=32, d_state=8, expand=1.0, d_conv=3, d_ssm_in=2, d_ssm_out=2, n_groups=4,
                                  a_act="softplus", a_dyn_per_sibling=True, bc_bias="shared",
                                  skip_sharing="input_output"), B=1, L=21, split=8),
    # The tensor-core tiles of this package work on 128-token (rank 1) and 32-token (rank 4) chunks: these cases are long
    # enough to cross several chunk boundaries, and their continuation cut falls inside a chunk.
    # config-2 geometry, 2 heads, 4 chunks of 128 (the last one partial), cut at 200 = 128 + 72
    "cfg2_long": dict(preset=dict(d_model=64, d_state=128, d_head=64), B=2, L=416, split=200),
    # config-5 head geometry (P = 64, N = 128) at 4 heads, cut at 150 = 128 + 22
    "cfg5_long": dict(preset=dict(d_model=128, d_state=128, d_head=64), B=1, L=400, split=150),
    # config-3 geometry at 2 heads, 7 chunks of 32, cut at 100 = 3 * 32 + 4
    "cfg3_long": dict(cfg=dict(d_model=64, expand=2.0, d_state=128, d_ssm_in=4, d_ssm_out=4, n_heads=2, d_head=64,
                               d_conv=4, write_rule="trapezoid", row_blocks=HS), B=1, L=224, split=100),
    "euler_r2o1": dict(cfg=dict(d_model=24, d_state=8, expand=1.0, d_conv=2, d_ssm_in=2, d_ssm_out=1, n_groups=3,
                                write_rule="euler", row_blocks=HS, skip_sharing="channel", b_norm=False,
                                r_mix="none", bc_bias="none"), B=2, L=18, split=5),
}


def build(case, dtype):
    torch.manual_seed(0)
    cfg = mamba2_config(**case["preset"]) if "preset" in case else SSDMimoConfig(**case["cfg"])
    layer = SSDMimoSSM(cfg, execution={"backend": "torch"})
    if not case.get("exact"):
        g = torch.Generator().manual_seed(1)
        with torch.no_grad():
            for p in layer.parameters():
                p.add_(0.05 * torch.randn(p.shape, generator=g) * (1.0 + p.abs()))
    return cfg, layer.to(dtype)


def run(layer, x, dy, state=None, gh=None, gw=None, exact=False):
    x = x.clone().requires_grad_(True)
    if state is not None:
        state = {k: v.clone().requires_grad_(True) for k, v in state.items()}
    layer.zero_grad()
    if exact:
        y = layer(x)
        (y ** 2).mean().backward()
        st = None
    else:
        y, st = layer(x, state=state, return_state=True)
        loss = (y * dy).sum() + (st["hidden_state"] * gh).sum()
        if "write_prev" in st:
            loss = loss + (st["write_prev"] * gw).sum()
        loss.backward()
    grads = {n: p.grad.detach().clone() for n, p in layer.named_parameters() if p.grad is not None}
    grads["x"] = x.grad.detach().clone()
    if state is not None:
        for k, v in state.items():
            if v.grad is not None:
                grads["state." + k] = v.grad.detach().clone()
    return y.detach(), (None if st is None else {k: v.detach().clone() for k, v in st.items()}), grads


def main():
    only = set(sys.argv[2:])
    for name, case in CASES.items():
        if only and name not in only:
            continue
        rec = {}
        for tag, dtype in (("f64", torch.float64), ("f32", torch.float32)):
            cfg, layer = build(case, dtype)
            g = torch.Generator().manual_seed(2)
            if case.get("exact"):
                torch.manual_seed(0)
                _, fresh = build(case, torch.float32)           # same RNG stream as README usage: init then randn
                x = torch.randn(case["B"], case["L"], cfg.d_model)
            else:
                x = torch.randn(case["B"], case["L"], cfg.d_model, generator=g)
            dy = torch.randn(case["B"], case["L"], cfg.d_model, generator=g)
            gh = torch.randn(case["B"], layer.H, layer.P, layer.N, generator=g)
            gw = torch.randn(case["B"], layer.H, layer.P, layer.N, generator=g)
            if tag == "f64":
                rec["config"] = {k: v for k, v in cfg.layer_kwargs().items()}
                rec["state_dict"] = {k: v.float() for k, v in layer.state_dict().items()}
                rec["x"], rec["dy"], rec["gh"], rec["gw"] = x, dy, gh, gw
                rec["exact"] = bool(case.get("exact"))
            y, st, grads = run(layer, x.to(dtype), dy.to(dtype), None, gh.to(dtype), gw.to(dtype),
                               exact=case.get("exact", False))
            # fp64 = the oracle precision (everything kept); fp32 = "the reference fp32 result" (output and carries)
            rec[tag] = dict(y=y, state=st, grads=grads) if tag == "f64" else dict(y=y, state=st)
            if "split" in case:
                # continuation: the second segment started from the first segment's State
                s = case["split"]
                _, st1, _ = run(layer, x[:, :s].to(dtype), dy[:, :s].to(dtype), None, gh.to(dtype), gw.to(dtype))
                y2, st2, grads2 = run(layer, x[:, s:].to(dtype), dy[:, s:].to(dtype), st1, gh.to(dtype), gw.to(dtype))
                if tag == "f64":
                    rec["f64_cont"] = dict(split=s, state_in=st1, y=y2, state=st2, grads=grads2)
        if rec["exact"]:
            rec["mean_y2_f32"] = float((rec["f32"]["y"] ** 2).mean())
        # keep the fixtures small: fp64 results stored as fp64, inputs as fp32
        torch.save(rec, os.path.join(OUT, name + ".pt"))
        print(name, {k: (tuple(v.shape)) for k, v in rec["state_dict"].items() if v.dim() > 1 and v.numel() > 4096},
              os.path.getsize(os.path.join(OUT, name + ".pt")) // 1024, "KiB")


if __name__ == "__main__":
    main()
