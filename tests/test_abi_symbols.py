"""The C-ABI library loads without a GPU and exports exactly what include/orbit_b200.h declares (no compute calls)."""
import ctypes
import os
import re

from orbitssm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "orbit_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(orbit_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared()
    assert len(names) >= 12
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header declarations differ"


import pytest


@pytest.mark.parametrize("struct,mirror", [("orbit_scan_args", "ScanArgs"), ("orbit_hm_args", "HmArgs"), ("orbit_clock_args", "ClockArgs"),
                                           ("orbit_hm_tail_args", "HmTailArgs")])
def test_args_mirror_matches_header_field_order(struct, mirror):
    text = open(os.path.join(ROOT, "include", "orbit_b200.h")).read()
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = decl.split(",")
        first = names[0].split()[-1]
        fields += [first.lstrip("*")] + [n.strip().lstrip("*") for n in names[1:]]
    assert fields == [f[0] for f in getattr(_lib, mirror)._fields_]


def test_pure_queries_run_on_cpu():
    lib = _lib.load()
    assert lib.orbit_built_for_sm() == 100
    ws = lib.orbit_conv1d_bwd_workspace_bytes(2, 64, 8, 4)
    assert ws > 0 and ws % (2 * 8 * 5 * 4) == 0          # [batch * token runs, C, W + 1] floats
    assert lib.orbit_ssd_scan_pick_chunk(1, 1, 64, 128, _lib.PRECISION_IEEE, 1, 64) in (16, 32, 64)
