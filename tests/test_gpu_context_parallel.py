"""-m gpu, needs >= 2 GPUs (skipped otherwise): the layer context-parallel over two B200s (NCCL all-gather of the
segment states, P2P halo exchange) against the reference's single-sequence golden vectors.  Bounds as in
test_gpu_layer.py."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, io_name, out, fixture="cfg2_small"):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from conftest import load_golden
        from orbitssm_b200.config import SSDMimoConfig
        from orbitssm_b200.ssd_mimo import SSDMimoSSM
        io = getattr(torch, io_name)
        rec = load_golden(fixture)
        layer = SSDMimoSSM(SSDMimoConfig(**rec["config"]), execution={"precision": "ieee" if io == torch.float32 else "io"})
        layer.load_state_dict(rec["state_dict"])
        layer = layer.to("cuda")
        layer.set_context_parallel("world")
        L = rec["x"].shape[1]
        cut = (41 * L) // 96
        a, b = (0, cut) if rank == 0 else (cut, L)
        x = rec["x"][:, a:b].to("cuda").to(io).requires_grad_(True)
        y, st = layer(x, return_state=True)
        loss = (y.float() * rec["dy"][:, a:b].to("cuda")).sum()
        if rank == world - 1:
            loss = loss + (st["hidden_state"] * rec["gh"].to("cuda")).sum()
            if "write_prev" in st:
                loss = loss + (st["write_prev"] * rec["gw"].to("cuda")).sum()
        loss.backward()
        want = rec["f64"]

        def rel(p, q):
            p, q = p.detach().double().cpu(), q.double()
            return float((p - q).norm() / q.norm().clamp_min(1e-300))

        errs = {"y": rel(y, want["y"][:, a:b]), "dx": rel(x.grad, want["grads"]["x"][:, a:b])}
        if rank == world - 1:
            errs["hidden"] = rel(st["hidden_state"], want["state"]["hidden_state"])
            if "write_prev" in st:
                errs["hidden.write_prev"] = rel(st["write_prev"], want["state"]["write_prev"])
        for n, p in layer.named_parameters():
            g = p.grad.clone()
            dist.all_reduce(g)
            errs["d" + n] = rel(g, want["grads"][n])
        out[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("io_name,fixture", [("float32", "cfg2_small"), ("bfloat16", "cfg2_small"), ("float32", "dyn_trap_conv"),
                                             ("bfloat16", "cfg3_small")])
def test_two_gpus_equal_the_whole_sequence(io_name, fixture):
    """Euler write at config-2 geometry, and the two-endpoint trapezoid write (its lag term crosses the cut): the fp32
    kernels on a small dynamic-decay layer and the rank-4 tensor-core tiles at config-3 geometry."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, 29650 + (os.getpid() % 300), io_name, out, fixture), nprocs=2, join=True)
    ty, tg = (2e-4, 5e-3) if io_name == "float32" else (2.5e-2, 6e-2)
    for rank in range(2):
        bad = {k: e for k, e in out[rank].items() if not e < (ty if k in ("y", "hidden", "hidden.write_prev") else tg)}
        assert not bad, (rank, bad, dict(out[rank]))
