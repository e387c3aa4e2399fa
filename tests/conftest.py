import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    import torch
    return torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)


GOLDEN_CASES = ("cfg1_exact", "cfg2_small", "cfg3_small", "dyn_trap_conv", "softplus_sib", "euler_r2o1",
                # several chunks of the tensor-core tiles, continuation cut inside a chunk
                "cfg2_long", "cfg5_long", "cfg3_long")
HM_GOLDEN_CASES = ("hm_small", "hm_cfg4_small", "hm_euler", "hm_cfg4_long")
