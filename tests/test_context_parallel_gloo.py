"""Context parallelism on CPU: two gloo ranks each take half of the sequence through the product's own protocol
(halo exchange of the conv windows, all-gather of the segment states, the mirror image in backward); the kernels are
replaced by their torch restatements.  Outputs and gradients must equal the single-rank golden vectors of the
reference."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out, cont=False, fixture="cfg2_small"):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from conftest import load_golden
        from orbitssm_b200 import ops
        from orbitssm_b200.config import SSDMimoConfig
        from orbitssm_b200.ssd_mimo import SSDMimoSSM
        from oracle import abi_reference as R
        for name in ("conv1d_fwd", "conv1d_bwd", "gate_norm_fwd", "gate_norm_bwd", "pick_chunk", "run_phase", "token_map_fwd",
                     "token_map_bwd", "run_clock", "cp_pack", "cp_combine"):
            setattr(ops, name, getattr(R, name))
        ops.on_device = lambda t: True
        ops._require_cuda = lambda who, *t: None
        ops._dtype_code = lambda who, t: 0
        torch.set_num_threads(2)
        rec = load_golden(fixture)
        layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]))
        layer.load_state_dict(rec["state_dict"])
        layer.set_context_parallel("world")
        L = rec["x"].shape[1]
        cuts = [0, 41 * L // 96, L] if world == 2 else [0, 30 * L // 96, 61 * L // 96, L]
        state, want, xs, dys = None, rec["f64"], rec["x"], rec["dy"]
        if cont:
            # the continuation fixture: the sequence after the cut, started from the reference's carried State.  The State
            # belongs to the whole sequence: rank 0 reads it, the other ranks' copy is ignored.
            c = rec["f64_cont"]
            s0 = c["split"]
            xs, dys, want = rec["x"][:, s0:], rec["dy"][:, s0:], c
            state = {k: v.clone().float().requires_grad_(rank == 0) for k, v in c["state_in"].items()}
            L = xs.shape[1]
            cuts = [0, (2 * L) // 5, L] if world == 2 else [0, L // 3, (2 * L) // 3, L]
        a, b = cuts[rank], cuts[rank + 1]
        x = xs[:, a:b].clone().requires_grad_(True)
        y, st = layer(x, state=state, return_state=True)
        loss = (y * dys[:, a:b]).sum()
        if rank == world - 1:
            loss = loss + (st["hidden_state"] * rec["gh"]).sum()
            if "write_prev" in st:
                loss = loss + (st["write_prev"] * rec["gw"]).sum()
        loss.backward()

        def rel(p, q):
            p, q = p.detach().double(), q.double()
            return float((p - q).norm() / q.norm().clamp_min(1e-300))

        errs = {"y": rel(y, want["y"][:, a:b]), "dx": rel(x.grad, want["grads"]["x"][:, a:b])}
        if rank == world - 1:
            for k, v in want["state"].items():
                if k in ("hidden_state", "write_prev"):
                    errs[k] = rel(st[k], v)
        if cont and rank == 0:
            for k, v in state.items():
                if v.grad is not None or ("state." + k) in want["grads"]:
                    errs["dstate." + k] = rel(v.grad, want["grads"]["state." + k])
        for n, p in layer.named_parameters():
            g = p.grad.clone()
            dist.all_reduce(g)                                   # parameter gradients add over the segments
            errs["d" + n] = rel(g, want["grads"][n])
        out[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,cont,fixture", [(2, False, "cfg2_small"), (3, False, "cfg2_small"), (2, True, "cfg2_small"),
                                                (3, True, "cfg2_small"), (2, False, "dyn_trap_conv"), (3, True, "dyn_trap_conv")])
def test_two_segments_equal_the_whole_sequence(world, cont, fixture):
    """Euler write (config-2 geometry) and the two-endpoint trapezoid write (whose lag term crosses the cut), from a zero
    state and continued from a carried State."""
    port = 29500 + (os.getpid() % 2000) + world + 10 * int(cont) + 20 * int(fixture != "cfg2_small")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out, cont, fixture), nprocs=world, join=True)
    for rank in range(world):
        bad = {k: e for k, e in out[rank].items() if not e < 2e-4}
        assert not bad, (rank, bad)
