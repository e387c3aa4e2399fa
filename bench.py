"""Benchmark of the SSD-MIMO layer hot path: layer forward + backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5a|cfg5b|cfg5|cfg4|cfg3|cfg2] [--impl reference]

One "step" = y = layer(x); y.backward(dy) on one batch of synthetic input (x ~ N(0,1), fixed random dy; bf16
activations over fp32 parameters).  Workloads (the benchmark configurations this metric is defined on):
  cfg5a (default) configuration 5a: 4-block BlockStack of the d_model-2048 SISO layer, global batch 64 x 4096 tokens split
        over the GPUs by batch rows (64 / N rows per GPU: strong scaling, no collective on the data path): the d2048 bf16
        configuration the metric is quoted on "at 1/2/4/8 B200"
  cfg5b configuration 5b: one d_model-2048 layer, B = 1, L = 262144 split over the GPUs (context parallel, strong
        scaling); with N > 1 the default run also measures it for a few steps under "other_workloads"
  cfg3  SSD-MIMO rank-4 layer, d_model 2048, x [4, 4096, 2048] (rank-4 tcgen05 tiles); at N = 1 the default run also
        measures it (same steps and warm-up) and reports it, with its own roofline block, under "other_workloads"
  cfg4  HybridMamba layer (coordinate-decay rows, half of them rotating pairs), d_model 1024, x [8, 2048, 1024]; also
        reported under "other_workloads" by the default run
  cfg2  Mamba-2 preset SISO layer, d_model 1024, x [8, 2048, 1024]
  cfg5  one layer of cfg5a at x [4, 4096, 2048]
With N > 1 (launched by torchrun, one rank per GPU) every rank runs its own rows of the global batch; the ranks meet
only at the barriers around the timed region.  Prints ONE JSON line on rank 0.
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
    # configuration 5: (a) a 4-block BlockStack of the d2048 SISO layer, global batch 64 split over the GPUs by rows;
    # (b) one layer, B = 1, L = 262144, context-parallel over the GPUs.  Both strong scaling.
    "cfg5a": dict(B=64, L=4096, d_model=2048, kind="m2", chunk_acct=64, blocks=4, split_batch=True,
                  desc="4-block BlockStack of the SSD-MIMO SISO Mamba-2 preset layer (H=64, P=64, N=128), d_model 2048, "
                       "global x [64,4096,2048] split over the GPUs by batch rows"),
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
# cfg3s / cfg4s, divided by their token counts).  Traffic grows in proportion to the tokens a launch processes, so
# `roofline.traffic` of a full-size launch is this figure times its tokens.
DRAM_BYTES_PER_TOKEN = {
    "m2": {"scan_chunk_grads": 69695.0, "scan_chunk_out": 24008.0, "scan_chunk_state": 22630.0},
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
    """A_log <- log U(log 1, log 16) per (head, sibling) as the benchmark configurations state; everything else default init
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


def run_reference(args, wl, name, out_stream=sys.stdout):
    """The reference arm: the CPU route of the layer (the oracle port) on all host threads, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the other ranks of this arm exit at once, so rank 0 takes the host
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_B, sample_L = 1, 256 if wl["kind"] == "m2" else 128
    t = cpu_step_time(wl, sample_B, sample_L, max(1, min(args.steps, 5)), max(1, min(args.warmup, 1)))
    tok = sample_B * sample_L / t
    sample = f"x [{sample_B},{sample_L},{wl['d_model']}] fp32 of the same layer (tokens/s is linear in tokens), median step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tok, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong" if (wl.get("cp") or wl.get("split_batch")) else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": name + ": " + wl["desc"]},
        "cpu_baseline": {"value": tok, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": tok, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), file=out_stream, flush=True)


# ----------------------------------------------------------------------------------------------------
#  GPU arm
# ----------------------------------------------------------------------------------------------------
class Env:
    """Rank, world and device of this process (one process per GPU)."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            # NCCL's own log (communicator sizes, transports) goes to stderr unless the caller chose otherwise: stdout
            # carries the one JSON line
            if "NCCL_DEBUG" not in os.environ:
                os.environ["NCCL_DEBUG"] = "INFO"
                os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
                os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
            dist.init_process_group("nccl", device_id=self.dev)

    def sync(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def roofline_block(wl, spec, route, B, L, kern_ms, pk):
    """`roofline` of the dominant kernel of one step over x [B, L, .] from the CUDA-event times per kernel group."""
    if wl["kind"] == "hm":
        # the coordinate scan has no contraction: it is bound by exp (MUFU) and FP32 issue; HBM is the nearest roofline
        # the contract names.  Algorithmic bytes = compulsory IO of the launch: drive in, output (or its gradient) in/out,
        # maps and clocks (and their gradients) once; checkpoints and partial-sum buffers are not counted.
        es, D_in, Nn, Hh = 2, spec.d_inner, spec.N, spec.H
        maps = B * L * (2 * Nn + spec.K + 2 * Hh) * 4
        byts = {"hm_scan_fwd": B * L * D_in * es * 2 + maps, "hm_scan_bwd": B * L * D_in * es * 3 + 2 * maps}
        dom = max(byts, key=lambda k: kern_ms.get(k, 0.0))
        ach = byts[dom] / (kern_ms[dom] * 1e-3) / 1e9
        roofline = dict(bound="hbm", kernel=dom, achieved=ach, peak=pk["hbm_gbs"], unit="GB/s", frac=ach / pk["hbm_gbs"],
                        traffic=None, peak_source=pk["source"] + " (copy)", ms_per_launch=kern_ms[dom],
                        note="issue-bound (one exp + ~10 FP32 ops per state element per token), not HBM-bound",
                        state_updates_per_s=B * L * Hh * spec.P * Nn / (kern_ms[dom] * 1e-3), route=route)
    else:
        fl = scan_flops(spec, B, L, wl["chunk_acct"])
        names = [k for k in kern_ms if k in fl]
        if not names:
            return None
        dom = max(names, key=lambda k: kern_ms[k])
        ach = fl[dom] / (kern_ms[dom] * 1e-3) / 1e12
        roofline = dict(bound="tensor", kernel=dom, achieved=ach, peak=pk["tflops"], unit="TFLOP/s", frac=ach / pk["tflops"],
                        traffic=None, peak_source=pk["source"] + " (sustained bf16 GEMM)", ms_per_launch=kern_ms[dom], route=route)
        # the whole scan (all phases of both directions) against the same peak: 3 x forward flops
        scan_ms = sum(v for k, v in kern_ms.items() if k.startswith("scan_"))
        if scan_ms > 0:
            roofline["whole_scan"] = dict(ms=scan_ms, achieved=3 * fl["fwd"] / (scan_ms * 1e-3) / 1e12,
                                          frac=3 * fl["fwd"] / (scan_ms * 1e-3) / 1e12 / pk["tflops"])
    per_tok = DRAM_BYTES_PER_TOKEN.get(wl["kind"], {}).get(roofline["kernel"])
    if per_tok is not None:
        roofline["traffic"] = per_tok * B * L
        roofline["traffic_source"] = "ncu capture of the profiling case, scaled by tokens per launch"
    return roofline


def measure(env, wl, name, steps, warmup, e2e_regions=3, cp_world=None):
    """Time `steps` fwd+bwd steps of workload `wl` on this rank's share after `warmup` untimed ones (CUDA events around
    every step on the compute stream, L2 flushed between steps), then `e2e_regions` end-to-end regions of the same
    steps with host buffers.  `cp_world`: ranks the sequence is split over (context parallel), None = env.world for a
    context-parallel workload.  Returns a dict on every rank (times are max over ranks)."""
    from orbitssm_b200 import ops
    dev, world, rank = env.dev, env.world, env.rank
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
    B, L, dm = wl["B"], wl["L"], wl["d_model"]
    if cp_world is None:
        cp_world = world if wl.get("cp") else 1
    use_cp = bool(wl.get("cp")) and cp_world > 1
    if use_cp:
        mixer0.set_context_parallel("world")
    if wl.get("cp"):
        L = L // cp_world                                             # this rank's segment of the sequence
    shards = 1
    if wl.get("split_batch"):
        if B % world:
            raise SystemExit(f"{name}: the global batch {B} does not split over {world} GPUs")
        B, shards = B // world, world                                 # this rank's rows of the global batch
    elif not wl.get("cp"):
        shards = world                                                # every rank runs its own copy of the batch (weak)
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
                # detached: copying a graph-carrying tensor into y_host would chain every step's graph behind y_host
                y_host.copy_(y.detach(), non_blocking=True)
                dx_host.copy_(xd.grad, non_blocking=True)
            y.record_stream(down)
            xd.grad.record_stream(down)
            del y, xd            # drop this step's autograd graph before the next forward allocates its own
        main.wait_stream(down)
        e1.record(main)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    torch.cuda.reset_peak_memory_stats(dev)
    for _ in range(warmup):
        step()
    env.sync()
    timing = []
    ops.set_timing(timing)
    launches0 = ops.LAUNCHES
    ev = []
    env.sync()
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        ev.append((e0, e1))
    env.sync()
    launches = ops.LAUNCHES - launches0
    ops.set_timing(None)
    ops.check_device_status()                 # a bounded device-side wait that gave up voids the numbers: raise, exit non-zero
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    mem_gb = {"timed": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)}
    per_kernel = {}
    for kname, a, b in timing:
        per_kernel.setdefault(kname, []).append(a.elapsed_time(b))
    # end to end: host buffers in, host buffers out; several regions, the median is reported
    e2e = []
    if e2e_regions:
        run_e2e(2)
        env.sync()
        for _ in range(e2e_regions):
            e2e.append(run_e2e(steps))
            env.sync()
        ops.check_device_status()
        mem_gb["e2e"] = round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)
    red = env.max_over_ranks([total_ms] + e2e)
    total_ms, e2e = red[0], red[1:]
    tokens = B * L * steps * (cp_world if wl.get("cp") else shards)
    kern_ms = {k: statistics.mean(v) for k, v in per_kernel.items()}
    out = dict(
        value=tokens / (total_ms * 1e-3), ms_per_step=total_ms / steps, tokens_per_step=tokens // steps, B=B, L=L,
        blocks=nblocks, use_cp=use_cp, launches=launches, kern_ms=kern_ms, route=mixer0.last_route(), spec=mixer0.spec,
        kernel_ms_sum=sum(kern_ms[k] * len(per_kernel[k]) for k in kern_ms) / steps,
        h2d=2 * x_host.numel() * 2, d2h=2 * y_host.numel() * 2, mem_gb=mem_gb)
    if e2e:
        med = statistics.median(e2e)
        out["e2e"] = {"value": tokens / (med * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": out["h2d"],
                      "d2h_bytes_per_step": out["d2h"], "regions": len(e2e), "region_steps": steps,
                      "ms_per_step_median": med / steps, "ms_per_step_min": min(e2e) / steps, "ms_per_step_max": max(e2e) / steps,
                      "copies": "pinned host buffers; upload of step i+1 and download of step i overlap the compute of their "
                                "neighbours; the median of the regions is reported"}
    if use_cp:
        mixer0.set_context_parallel(None)
    del layer, mixers, x, dy, flush
    torch.cuda.empty_cache()
    return out


def other_workload(env, key, steps, warmup, pk, **kw):
    """Another workload measured with the same step definition, steps and warm-up, reported beside the headline."""
    wl = WORKLOADS[key]
    m = measure(env, wl, key, steps, warmup, e2e_regions=0, **kw)
    return {"workload": key + ": " + wl["desc"], "value": m["value"], "unit": "tokens/s", "ms_per_step": m["ms_per_step"],
            "route": m["route"], "steps": steps, "warmup": warmup, "gpu_launches": m["launches"],
            "roofline": roofline_block(wl, m["spec"], m["route"], m["B"], m["L"], m["kern_ms"], pk),
            "kernel_ms": {k: round(v, 4) for k, v in sorted(m["kern_ms"].items())}}


def _json_only_stdout():
    """Keep the process's real stdout for the one JSON line: everything else that writes to file descriptor 1 (NCCL's
    version banner with NCCL_DEBUG=INFO, library chatter) goes to stderr from here on.  Returns the stream to print to."""
    real = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    return real


def graphed_workload(env, key, steps, warmup):
    """A launch-bound workload (small layer) stepped eagerly and as one captured CUDA graph (`orbitssm_b200.GraphedStep`):
    the same forward + backward, CUDA events around every step, L2 flushed between steps."""
    from orbitssm_b200 import GraphedStep
    wl = WORKLOADS[key]
    torch.manual_seed(0)
    layer = make_mixer(make_config(wl), execution={"precision": "io"}).to(env.dev)
    init_params(layer)
    x = torch.randn(wl["B"], wl["L"], wl["d_model"], device=env.dev, dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=env.dev)
    xe = x.clone().requires_grad_(True)

    def eager():
        xe.grad = None
        for p in layer.parameters():
            p.grad = None
        layer(xe).backward(dy)

    # the eager steps run on another stream than the one the capture made the gradient accumulators on: expected here
    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
    g = GraphedStep(layer, x, dy, warmup=max(3, warmup))

    def timed(fn):
        for _ in range(warmup):
            fn()
        ev = []
        for _ in range(steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            ev.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in ev) / steps

    t_eager = timed(eager)
    t_graph = timed(lambda: g.step(x, dy))
    tokens = wl["B"] * wl["L"]
    del g, layer, flush
    torch.cuda.empty_cache()
    return {"workload": key + ": " + wl["desc"] + ", one step captured as a CUDA graph", "value": tokens / (t_graph * 1e-3),
            "unit": "tokens/s", "ms_per_step": t_graph, "eager_ms_per_step": t_eager, "steps": steps, "warmup": warmup}


def main():
    out_stream = _json_only_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5a", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the workload's (global) batch rows")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        wl["B"] = args.batch
        wl["desc"] += f" (batch rows overridden to {args.batch})"
    if args.impl == "reference":
        return run_reference(args, wl, args.workload, out_stream)

    env = Env()
    world, rank = env.world, env.rank
    args.warmup = max(args.warmup, 3)
    pk = peaks()
    sampler = ClockSampler(env.local)
    if rank == 0:
        sampler.start()
    m = measure(env, wl, args.workload, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None

    others = {}
    if args.workload == "cfg5a" and not args.no_other_workloads:
        if world == 1:
            # the other single-GPU configurations, same steps and warm-up, each with its own roofline block
            for key in ("cfg3", "cfg4"):
                others[key] = other_workload(env, key, args.steps, args.warmup, pk)
            # a launch-bound size: the d_model-1024 layer eagerly and as one captured graph
            others["cfg2_graphed"] = graphed_workload(env, "cfg2", args.steps, args.warmup)
        else:
            # configuration 5b: the one mode with communication on the data path.  Rank 0 first runs the whole sequence
            # alone (the N = 1 time the strong-scaling figure divides by), then all ranks run it context-parallel.
            k5 = max(3, min(args.steps, 5))
            solo = None
            if rank == 0:
                solo_env = _Solo(env)
                solo = other_workload(solo_env, "cfg5b", k5, args.warmup, pk, cp_world=1)
            env.sync()
            cpm = other_workload(env, "cfg5b", k5, args.warmup, pk)
            if rank == 0:
                cpm["n1_ms_per_step"] = solo["ms_per_step"]
                cpm["scaling"] = "strong"
                cpm["n_gpus"] = world
                cpm["speedup_over_n1"] = solo["ms_per_step"] / cpm["ms_per_step"]
                cpm["parallelism"] = f"context-parallel x{world}: all-gather of segment states + conv halos (NCCL)"
                others["cfg5b"] = cpm
    if rank != 0:
        env.close()
        return

    B, L, nblocks = m["B"], m["L"], m["blocks"]
    strong = bool(wl.get("cp") or wl.get("split_batch"))
    out = {
        "metric": METRIC, "value": m["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload + ": " + wl["desc"], "global_batch": wl["B"] if strong else wl["B"] * world,
                   "per_gpu_batch": B, "seq_len": L, "blocks": nblocks, "tokens_per_step": m["tokens_per_step"],
                   "l2": "256 MB buffer written between timed steps",
                   "parallelism": (f"context-parallel x{world}: all-gather of segment states + conv halos" if m["use_cp"]
                                   else f"batch rows split x{world}, no collective on the data path")},
        "e2e": m.get("e2e"), "gpu_launches": m["launches"], "clocks": clocks,
        "roofline": roofline_block(wl, m["spec"], m["route"], B, L, m["kern_ms"], pk),
        "kernel_ms": {k: round(v, 4) for k, v in sorted(m["kern_ms"].items())},
        "kernel_ms_sum": round(m["kernel_ms_sum"], 4), "peak_device_memory_gib": m["mem_gb"],
    }
    if world == 1 and not args.no_cpu_baseline:
        sB, sL = 1, 256 if wl["kind"] == "m2" else 128
        tcpu = cpu_step_time(wl, sB, sL, 3, 1)
        out["cpu_baseline"] = {"value": sB * sL / tcpu, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"x [{sB},{sL},{wl['d_model']}] fp32 of the same layer, median of 3 steps after 1 warm-up",
                               "host_cpus": os.cpu_count()}
    if others:
        out["other_workloads"] = others
    print(json.dumps(out), file=out_stream, flush=True)
    env.close()


class _Solo:
    """An `Env` view for work that one rank does alone while the others wait at the next barrier."""

    def __init__(self, env):
        self.dev, self.local, self.rank, self.world, self.dist = env.dev, env.local, 0, 1, env.dist

    def sync(self):
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        return [float(v) for v in values]


if __name__ == "__main__":
    main()
