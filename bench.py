"""Benchmark of the SSD-MIMO layer hot path: layer forward + backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5a|cfg5b|cfg5|cfg4|cfg3|cfg2] [--impl reference]

One "step" = y = layer(x); y.backward(dy) on one batch of synthetic input (x ~ N(0,1), fixed random dy; bf16
activations over fp32 parameters).  Workloads (BASELINE.json `configs`):
  cfg5a (default) BASELINE config 5a: 4-block BlockStack of the d_model-2048 SISO layer, batch-sharded, x [8, 4096, 2048]
        per GPU: the d2048 bf16 configuration the metric is quoted on "at 1/2/4/8 B200" (weak scaling, no collective)
  cfg5b BASELINE config 5b: one d_model-2048 layer, B = 1, L = 262144 split over the GPUs (context parallel, strong scaling)
  cfg3  SSD-MIMO rank-4 layer, d_model 2048, x [4, 4096, 2048] (rank-4 tcgen05 tiles); at N = 1 the default run also
        measures it briefly and reports it under "other_workloads"
  cfg4  HybridMamba layer (coordinate-decay rows, half of them rotating pairs), d_model 1024, x [8, 2048, 1024]; also
        reported under "other_workloads" by the default run
  cfg2  Mamba-2 preset SISO layer, d_model 1024, x [8, 2048, 1024]
  cfg5  one layer of cfg5a at x [4, 4096, 2048]
With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same per-GPU batch on its own shard of the
batch: no collective on the data path, weak scaling.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "layer fwd+bwd tokens/s (SSD-MIMO d2048 bf16)"
WORKLOADS = {
    "cfg3": dict(B=4, L=4096, d_model=2048, kind="mimo4", chunk_acct=32,
                 desc="SSD-MIMO rank-4 (R=O=4, G=16, H=64, N=128) trapezoid layer, d_model 2048, x [4,4096,2048]"),
    "cfg2": dict(B=8, L=2048, d_model=1024, kind="m2", chunk_acct=64,
                 desc="SSD-MIMO SISO Mamba-2 preset (H=32, P=64, N=128) layer, d_model 1024, x [8,2048,1024]"),
    "cfg5": dict(B=4, L=4096, d_model=2048, kind="m2", chunk_acct=64,
                 desc="SSD-MIMO SISO Mamba-2 preset (H=64, P=64, N=128) layer, d_model 2048, x [4,4096,2048]"),
    "cfg4": dict(B=8, L=2048, d_model=1024, kind="hm", chunk_acct=32,
                 desc="HybridMamba layer (H=32, P=64, N=64: 32 real rows + 16 rotating pairs, coord_static, trapezoid, gated "
                      "RMSNorm), d_model 1024, x [8,2048,1024]"),
    # BASELINE config 5: (a) a 4-block BlockStack of the d2048 SISO layer, batch-sharded, 8 rows per GPU (B = 64 at
    # 8 GPUs); (b) one layer, B = 1, L = 262144, context-parallel over the GPUs (strong scaling)
    "cfg5a": dict(B=8, L=4096, d_model=2048, kind="m2", chunk_acct=64, blocks=4,
                  desc="4-block BlockStack of the SSD-MIMO SISO Mamba-2 preset layer (H=64, P=64, N=128), d_model 2048, "
                       "x [8,4096,2048] per GPU"),
    "cfg5b": dict(B=1, L=262144, d_model=2048, kind="m2", chunk_acct=64, cp=True,
                  desc="one SSD-MIMO SISO Mamba-2 preset layer, d_model 2048, B=1, L=262144 split over the GPUs "
                       "(context parallel: chunk state all-gathered over NVLink)"),
    # reduced batches of the same layers, for profiler captures that must stay small
    # (sized so that the scan kernels launch exactly one CTA per SM: 4 x 37 chunks = 148)
    "cfg5s": dict(B=4, L=4736, d_model=2048, kind="m2", chunk_acct=64,
                  desc="profiling case: the cfg5 layer at x [4,4736,2048]"),
    "cfg4s": dict(B=4, L=1024, d_model=1024, kind="hm", chunk_acct=32,
                  desc="profiling case: the cfg4 layer at x [4,1024,1024]"),
    "cfg3s": dict(B=4, L=1184, d_model=2048, kind="mimo4", chunk_acct=32,
                  desc="profiling case: the cfg3 layer at x [4,1184,2048]"),
}


# DRAM bytes per token (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the profiling cases cfg5s /
# cfg3s / cfg4s, divided by their token counts; profiles/scan_dram_traffic.md).  Traffic grows in proportion to the tokens
# a launch processes, so `roofline.traffic` of a full-size launch is this figure times its tokens.
DRAM_BYTES_PER_TOKEN = {
    "m2": {"scan_chunk_grads": 68451.0, "scan_chunk_out": 23852.0, "scan_chunk_state": 22452.0},
    "mimo4": {"scan_chunk_grads": 416550.0},
    "hm": {"hm_scan_bwd": 41920.0, "hm_scan_fwd": 13610.0},
}


def make_config(wl):
    from orbitssm_b200 import HybridMambaConfig, SSDMimoConfig, mamba2_config
    if wl["kind"] == "m2":
        return mamba2_config(wl["d_model"])
    if wl["kind"] == "hm":
        return HybridMambaConfig(d_model=wl["d_model"], d_state=64, expand=2, d_conv=4, out_norm=True,
                                 row_blocks=[{"frac": .5, "decay": "coord_static"},
                                             {"frac": .5, "decay": "coord_static", "complex": True}])
    return SSDMimoConfig(d_model=wl["d_model"], expand=2.0, d_state=128, d_ssm_in=4, d_ssm_out=4, n_heads=64, d_head=64,
                         d_conv=4, write_rule="trapezoid", row_blocks=[{"frac": 1.0, "decay": "head_static"}])


def make_mixer(cfg, execution=None):
    from orbitssm_b200 import HybridMambaConfig, HybridMambaSSM, SSDMimoSSM
    if isinstance(cfg, HybridMambaConfig):
        return HybridMambaSSM(cfg)
    return SSDMimoSSM(cfg, execution=execution)


def init_params(layer, seed=0):
    """A_log <- log U(log 1, log 16) per (head, sibling) as BASELINE.json states; everything else default init
    (HybridMamba keeps its default per-coordinate ladder)."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        if hasattr(layer, "A_log") and layer.config_family == "ssd_mimo":
            hi = float(torch.log(torch.tensor(16.0)))
            layer.A_log.copy_(torch.rand(layer.A_log.shape, generator=g) * hi)      # A = exp(A_log) in [1, 16], log-uniform


def scan_flops(spec, B, L, T):
    """Algorithmic flops of the scan per forward and per phase kernel (dense contractions only):
    per (batch, kernel head, chunk): s1 = (O T)(R T) N score, s2 = (O T)(R T) G intra output, s3 = N (R T) G chunk state,
    s4 = (O T) N G state read; forward = 2 (s1+s2+s3+s4); backward = 2 x forward."""
    R, O, G, N, Hk = spec.R, spec.O, spec.G, spec.N, spec.H * spec.R
    nc = -(-L // T)
    s1, s2, s3, s4 = (O * T) * (R * T) * N, (O * T) * (R * T) * G, N * (R * T) * G, (O * T) * N * G
    unit = B * Hk * nc
    return dict(fwd=2 * unit * (s1 + s2 + s3 + s4), scan_chunk_state=2 * unit * s3, scan_chunk_out=2 * unit * (s1 + s2 + s4),
                scan_chunk_dstate=2 * unit * s4, scan_chunk_grads=2 * unit * (2 * s1 + 2 * s2 + 2 * s3 + s4))


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        busy = [s for s in sm if s > 0.5 * max(sm)] if sm else []
        return dict(sm_mhz=statistics.median(busy) if busy else None, sm_max_mhz=max(mx) if mx else None, reasons=reasons,
                    samples=len(sm))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


# ----------------------------------------------------------------------------------------------------
#  CPU arm: the reference's CPU route restated in oracle/ (the only place the bench runs it), bounded sample
# ----------------------------------------------------------------------------------------------------
def cpu_step_time_hm(wl, sample_B, sample_L, steps, warmup):
    from oracle import hm_oracle
    torch.manual_seed(0)
    cfg = make_config(wl)
    layer = make_mixer(cfg)
    prm = {k: v.detach().clone().requires_grad_(v.is_floating_point() and v.dim() > 0) for k, v in layer.state_dict().items()}
    x = torch.randn(sample_B, sample_L, wl["d_model"], requires_grad=True)
    dy = torch.randn(sample_B, sample_L, wl["d_model"])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        hm_oracle.hm_layer(cfg.to_dict(), prm, x).backward(dy)
        dt = time.perf_counter() - t0
        for v in prm.values():
            v.grad = None
        x.grad = None
        if i >= warmup:
            times.append(dt)
    return statistics.median(times)


def cpu_step_time(wl, sample_B, sample_L, steps, warmup):
    if wl["kind"] == "hm":
        return cpu_step_time_hm(wl, sample_B, sample_L, steps, warmup)
    from orbitssm_b200.config import resolve_ssd_spec
    from orbitssm_b200 import SSDMimoSSM
    from oracle import ssd_oracle
    torch.manual_seed(0)
    cfg = make_config(wl)
    spec = resolve_ssd_spec(cfg)
    layer = SSDMimoSSM(cfg)
    init_params(layer)
    prm = {k: v.detach().clone().requires_grad_(v.is_floating_point()) for k, v in layer.state_dict().items()}
    x = torch.randn(sample_B, sample_L, wl["d_model"], requires_grad=True)
    dy = torch.randn(sample_B, sample_L, wl["d_model"])
    times = []
    blocks = wl.get("blocks", 1)

    def rms(h):
        return h * torch.rsqrt(h.square().mean(-1, keepdim=True) + 1e-5)

    for i in range(warmup + steps):
        t0 = time.perf_counter()
        y = x
        for _ in range(blocks):                       # a BlockStack: x + layer(norm(x)) per block, then the final norm
            y = y + ssd_oracle.ssd_layer(spec, prm, rms(y)) if blocks > 1 else ssd_oracle.ssd_layer(spec, prm, y)
        if blocks > 1:
            y = rms(y)
        y.backward(dy)
        dt = time.perf_counter() - t0
        for v in prm.values():
            v.grad = None
        x.grad = None
        if i >= warmup:
            times.append(dt)
    return statistics.median(times)


def run_reference(args, wl, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_B, sample_L = 1, 256 if wl["kind"] == "m2" else 128
    t = cpu_step_time(wl, sample_B, sample_L, max(1, min(args.steps, 5)), max(1, min(args.warmup, 1)))
    tok = sample_B * sample_L / t
    cores = torch.get_num_threads()
    sample = f"x [{sample_B},{sample_L},{wl['d_model']}] fp32 of the same layer (tokens/s is linear in tokens), median step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tok, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": name + ": " + wl["desc"]},
        "cpu_baseline": {"value": tok, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": tok, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def side_measure(wl, dev, steps=2, warmup=1):
    """A short device-timed measurement of another workload (same step definition), reported beside the headline."""
    torch.manual_seed(0)
    layer = make_mixer(make_config(wl), execution={"precision": "io"})
    init_params(layer)
    layer = layer.to(dev)
    x = torch.randn(wl["B"], wl["L"], wl["d_model"], device=dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(wl["B"], wl["L"], wl["d_model"], device=dev).to(torch.bfloat16)
    ms = []
    for i in range(warmup + steps):
        x.grad = None
        for p in layer.parameters():
            p.grad = None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        layer(x).backward(dy)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ms.append(e0.elapsed_time(e1))
    t = statistics.mean(ms)
    return {"workload": wl["desc"], "value": wl["B"] * wl["L"] / (t * 1e-3), "unit": "tokens/s", "ms_per_step": t,
            "route": layer.last_route(), "steps": steps, "warmup": warmup}


# ----------------------------------------------------------------------------------------------------
#  GPU arm
# ----------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5a", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args, wl, args.workload)

    from orbitssm_b200 import ops
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ["NCCL_DEBUG"] = "WARN"          # keep NCCL's banner off stdout: the driver reads one JSON line
        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)

    torch.manual_seed(0)
    cfg = make_config(wl)
    nblocks = wl.get("blocks", 1)
    mixers = [make_mixer(cfg, execution={"precision": "io"}) for _ in range(nblocks)]
    for m in mixers:
        init_params(m)
    mixer0 = mixers[0]
    if nblocks > 1:
        from orbitssm_b200 import BlockStack
        layer = BlockStack.from_mixers(mixers, wl["d_model"]).to(dev)
    else:
        layer = mixer0.to(dev)
    use_cp = bool(wl.get("cp")) and world > 1
    if use_cp:
        mixer0.set_context_parallel("world")
    B, L, dm = wl["B"], wl["L"], wl["d_model"]
    if wl.get("cp"):
        L = L // world                                                # this rank's segment of the sequence
    g = torch.Generator().manual_seed(100 + rank)                     # each rank: its own shard of the global batch
    x_host = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).pin_memory()
    dy_host = torch.randn(B, L, dm, generator=g).to(torch.bfloat16).pin_memory()
    y_host = torch.empty(B, L, dm, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(B, L, dm, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(dev).requires_grad_(True)
    dy = dy_host.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB L2

    bf16_cast = nblocks > 1       # the stack's own norms follow the activations: run it under bf16 autocast

    def step():
        x.grad = None
        for p in layer.parameters():
            p.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf16_cast):
            y = layer(x)
        y.backward(dy)
        return y

    def run_e2e(n):
        """n end-to-end steps: every step's inputs come from pinned host memory and its outputs go back to pinned host
        memory inside the timed window.  Uploads of step i+1 and downloads of step i run on their own streams under the
        compute of the neighbouring step (double-buffered device inputs), as a training loop with a prefetching loader
        does.  Returns the elapsed milliseconds (CUDA events on the compute stream, which joins the copy streams)."""
        main = torch.cuda.current_stream()
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        xin = [torch.empty(x_host.shape, dtype=x_host.dtype, device=dev) for _ in range(2)]
        dyin = [torch.empty(dy_host.shape, dtype=dy_host.dtype, device=dev) for _ in range(2)]
        ev_up = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]

        def upload(i):
            b = i & 1
            with torch.cuda.stream(up):
                if i >= 2:
                    up.wait_event(ev_done[b])            # the step that read this buffer pair has finished
                xin[b].copy_(x_host, non_blocking=True)
                dyin[b].copy_(dy_host, non_blocking=True)
                ev_up[b].record(up)

        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        up.wait_stream(main)
        down.wait_stream(main)
        upload(0)
        for i in range(n):
            b = i & 1
            flush.zero_()
            if i + 1 < n:
                upload(i + 1)
            main.wait_event(ev_up[b])
            xd = xin[b].detach().requires_grad_(True)
            for p in layer.parameters():
                p.grad = None
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf16_cast):
                y = layer(xd)
            y.backward(dyin[b])
            ev_done[b].record(main)
            down.wait_event(ev_done[b])
            with torch.cuda.stream(down):
                y_host.copy_(y, non_blocking=True)
                dx_host.copy_(xd.grad, non_blocking=True)
            y.record_stream(down)
            xd.grad.record_stream(down)
        main.wait_stream(down)
        e1.record(main)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    timing = []
    ops.set_timing(timing)
    launches0 = ops.LAUNCHES
    ev = []
    sync_all()
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        ev.append((e0, e1))
    sync_all()
    launches = ops.LAUNCHES - launches0
    ops.set_timing(None)
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    per_kernel = {}
    for name, a, b in timing:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    # end to end: host buffers in, host buffers out
    run_e2e(2)
    sync_all()
    e2e_ms = run_e2e(args.steps)
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([total_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tokens = B * L * world * args.steps                              # cfg5b: L is the per-rank segment
    value = tokens / (total_ms * 1e-3)
    pk = peaks()
    spec = mixer0.spec
    kern_ms = {k: statistics.mean(v) for k, v in per_kernel.items()}
    roofline = None
    fl, dom = {}, None
    if wl["kind"] == "hm":
        # the coordinate scan has no contraction: it is bound by exp (MUFU) and FP32 issue; HBM is the nearest roofline
        # the contract names.  Algorithmic bytes = compulsory IO of the launch: drive in, output (or its gradient) in/out,
        # maps and clocks (and their gradients) once; checkpoints and partial-sum buffers are not counted.
        es, D_in, Nn, Hh = 2, spec.d_inner, spec.N, spec.H
        maps = B * L * (2 * Nn + spec.K + 2 * Hh) * 4
        byts = {"hm_scan_fwd": B * L * D_in * es * 2 + maps, "hm_scan_bwd": B * L * D_in * es * 3 + 2 * maps}
        dom = max(byts, key=lambda k: kern_ms.get(k, 0.0))
        ach = byts[dom] / (kern_ms[dom] * 1e-3) / 1e9
        upd = B * L * Hh * spec.P * Nn / (kern_ms[dom] * 1e-3)
        roofline = dict(bound="hbm", kernel=dom, achieved=ach, peak=pk["hbm_gbs"], unit="GB/s", frac=ach / pk["hbm_gbs"],
                        traffic=None, peak_source=pk["source"] + " (copy)", ms_per_launch=kern_ms[dom],
                        note="issue-bound (one exp + ~10 FP32 ops per state element per token), not HBM-bound",
                        state_updates_per_s=upd, route=mixer0.last_route())
    else:
        fl = scan_flops(spec, B, L, wl["chunk_acct"])
        scan_names = [k for k in kern_ms if k in fl]
        dom = max(scan_names, key=lambda k: kern_ms[k]) if scan_names else None
    if dom and wl["kind"] != "hm":
        ach = fl[dom] / (kern_ms[dom] * 1e-3) / 1e12
        roofline = dict(bound="tensor", kernel=dom, achieved=ach, peak=pk["tflops"], unit="TFLOP/s", frac=ach / pk["tflops"],
                        traffic=None, peak_source=pk["source"] + " (sustained bf16 GEMM)", ms_per_launch=kern_ms[dom],
                        route=mixer0.last_route())
    if roofline is not None:
        per_tok = DRAM_BYTES_PER_TOKEN.get(wl["kind"], {}).get(roofline["kernel"])
        if per_tok is not None:
            roofline["traffic"] = per_tok * B * L
            roofline["traffic_source"] = "ncu capture of the profiling case, scaled by tokens per launch"
    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong" if wl.get("cp") else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload + ": " + wl["desc"], "per_gpu_batch": B, "seq_len": L, "blocks": nblocks,
                   "l2": "256 MB buffer written between timed steps",
                   "parallelism": (f"context-parallel x{world}: all-gather of segment states + conv halos" if use_cp
                                   else f"batch-sharded x{world}, no collective")},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * x_host.numel() * 2,
                "copies": "pinned host buffers; upload of step i+1 and download of step i overlap the compute of their neighbours",
                "d2h_bytes_per_step": 2 * y_host.numel() * 2},
        "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
        "kernel_ms": {k: round(v, 4) for k, v in sorted(kern_ms.items())},
        "kernel_ms_sum": round(sum(kern_ms[k] * len(per_kernel[k]) for k in kern_ms) / args.steps, 4),
    }
    if world == 1 and not args.no_cpu_baseline:
        sB, sL = 1, 256 if wl["kind"] == "m2" else 128
        tcpu = cpu_step_time(wl, sB, sL, 3, 1)
        out["cpu_baseline"] = {"value": sB * sL / tcpu, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"x [{sB},{sL},{dm}] fp32 of the same layer, median of 3 steps after 1 warm-up",
                               "host_cpus": os.cpu_count()}
    if world == 1 and args.workload == "cfg5a" and not args.no_cpu_baseline:
        out["other_workloads"] = {"cfg3": side_measure(WORKLOADS["cfg3"], dev), "cfg4": side_measure(WORKLOADS["cfg4"], dev)}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
