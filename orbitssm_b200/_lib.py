"""ctypes binding of the C-ABI library ``liborbit_b200.so`` (declared in ``include/orbit_b200.h``).

The library is built in-tree by ``orbitssm_b200.build`` (nvcc, sm_100a).  There is no other implementation of these
entry points in the package: if the library is missing or a call fails, the error is raised, never papered over.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liborbit_b200.so")

F32, BF16 = 0, 1
PRECISION_IEEE, PRECISION_IO = 0, 1
PHASE_CHUNK_STATE, PHASE_STATE_PASS, PHASE_CHUNK_OUT, PHASE_CHUNK_DSTATE, PHASE_STATE_PASS_BWD, PHASE_CHUNK_GRADS = range(6)
PHASE_STATE_PASS_DRY, PHASE_STATE_PASS_BWD_DRY = 6, 7

ERR_DEVICE_TIMEOUT = 5     # ORBIT_ERR_DEVICE_TIMEOUT: a bounded device-side wait gave up (read from the status word)

_STATUS_EXC = {1: ValueError, 2: NotImplementedError, 3: RuntimeError, 4: ValueError, 5: RuntimeError}


class OrbitLibraryError(RuntimeError):
    pass


class ScanArgs(C.Structure):
    """Mirror of ``orbit_scan_args`` (include/orbit_b200.h); field order and types must match the header."""
    _fields_ = (
        [(n, C.c_int) for n in ("B", "L", "H", "R", "O", "G", "N", "T", "nc", "hsplit")]
        + [(n, C.c_void_p) for n in ("u", "Bhat", "gBp", "Chat", "gCp")]
        + [(n, C.c_int64) for n in ("b_ts", "gb_ts", "c_ts", "gc_ts")]
        + [(n, C.c_void_p) for n in ("beta", "gamma", "chi", "dA", "w", "wd", "Dg", "Sin", "atot", "dS", "y", "dy", "du",
                                     "dBhat", "dgBp", "dChat", "dgCp", "ddA", "dw", "dwd", "dchi", "dbeta_part",
                                     "dgamma_part", "dDg_part", "status", "Sin16", "dS16", "du32")]
    )


class HmArgs(C.Structure):
    """Mirror of ``orbit_hm_args`` (include/orbit_b200.h); field order and types must match the header."""
    _fields_ = (
        [(n, C.c_int) for n in ("B", "L", "H", "P", "N", "Tc", "nck")]
        + [(n, C.c_void_p) for n in (
            "x", "delta", "A_log", "Bh", "Ch", "beta_b", "beta_c", "feat", "rot", "theta_h", "lam", "D", "h_init",
            "write_prev", "theta_init", "y", "h_final", "theta_final", "write_last", "hck", "thck",
            "dy", "dh_final", "dtheta_final", "dwrite_last", "dx", "ddelta", "dlam", "dA_log_part", "dBh_part",
            "dCh_part", "dbeta_b_part", "dbeta_c_part", "dfeat_part", "dtheta_h_part", "dD_part", "dh_init",
            "dwrite_prev", "dtheta_init")]
    )


class ClockArgs(C.Structure):
    """Mirror of ``orbit_clock_args`` (include/orbit_b200.h); field order and types must match the header."""
    _fields_ = [
        ("M", C.c_int64), ("L", C.c_int), ("H", C.c_int), ("R", C.c_int), ("a_act", C.c_int), ("a_per_sibling", C.c_int),
        ("dt_raw", C.c_void_p), ("dt_rs", C.c_int64), ("a_raw", C.c_void_p), ("a_rs", C.c_int64),
        ("trap_raw", C.c_void_p), ("trap_rs", C.c_int64), ("rmix_raw", C.c_void_p), ("rmix_rs", C.c_int64),
        ("A_log", C.c_void_p), ("r_mix", C.c_void_p),
        ("dA", C.c_void_p), ("w", C.c_void_p), ("wd", C.c_void_p), ("chi", C.c_void_p), ("lag0", C.c_void_p),
        ("ddA", C.c_void_p), ("dw", C.c_void_p), ("dwd", C.c_void_p), ("dchi", C.c_void_p), ("dlag0", C.c_void_p),
        ("d_dt_raw", C.c_void_p), ("ddt_rs", C.c_int64), ("d_a_raw", C.c_void_p), ("da_rs", C.c_int64),
        ("d_trap_raw", C.c_void_p), ("dtrap_rs", C.c_int64), ("d_rmix_raw", C.c_void_p), ("drmix_rs", C.c_int64),
        ("g_alog", C.c_void_p),
        ("sum_part", C.c_void_p), ("sum_part_bytes", C.c_int64), ("bias_sums", C.c_void_p),
    ]


class HmTailArgs(C.Structure):
    """Mirror of ``orbit_hm_tail_args`` (include/orbit_b200.h); field order and types must match the header."""
    _fields_ = [
        ("M", C.c_int64), ("H", C.c_int), ("K", C.c_int), ("Krot", C.c_int),
        ("dt_raw", C.c_void_p), ("dt_rs", C.c_int64), ("trap_raw", C.c_void_p), ("trap_rs", C.c_int64),
        ("th_raw", C.c_void_p), ("th_rs", C.c_int64),
        ("dt_bias", C.c_void_p), ("trap_bias", C.c_void_p), ("omega", C.c_void_p), ("rot_idx", C.c_void_p),
        ("delta", C.c_void_p), ("lam", C.c_void_p), ("feat", C.c_void_p),
        ("ddelta", C.c_void_p), ("dlam", C.c_void_p), ("dfeat", C.c_void_p),
        ("d_dt_raw", C.c_void_p), ("d_dt_rs", C.c_int64), ("d_trap_raw", C.c_void_p), ("d_trap_rs", C.c_int64),
        ("d_th_raw", C.c_void_p), ("d_th_rs", C.c_int64),
        ("d_dt_bias", C.c_void_p), ("d_trap_bias", C.c_void_p), ("d_omega", C.c_void_p),
        ("part", C.c_void_p), ("part_bytes", C.c_int64),
    ]


HM_CHUNK = 32     # checkpoint interval (tokens) the HybridMamba backward kernel is written for

_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol include/orbit_b200.h declares
SIGNATURES = {
    "orbit_last_error": (C.c_char_p, []),
    "orbit_version": (C.c_char_p, []),
    "orbit_built_for_sm": (_I, []),
    "orbit_conv1d_fwd": (_I, [_P, _L, _L, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "orbit_conv1d_bwd_workspace_bytes": (_L, [_I, _I, _I, _I]),
    "orbit_conv1d_bwd": (_I, [_P, _L, _L, _P, _P, _P, _P, _P, _L, _L, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _P]),
    "orbit_gate_norm_fwd": (_I, [_P, _P, _L, _P, _P, _P, _L, _I, _F, _I, _P]),
    "orbit_gate_norm_bwd_workspace_bytes": (_L, [_L, _I]),
    "orbit_gate_norm_bwd": (_I, [_P, _P, _L, _P, _P, _P, _P, _P, _L, _P, _P, _L, _L, _I, _I, _P]),
    "orbit_gate_norm_bwd_noalloc": (_I, [_P, _P, _L, _P, _P, _P, _P, _P, _L, _P, _L, _I, _I, _P]),
    "orbit_ssd_scan_pick_chunk": (_I, [_I, _I, _I, _I, _I, _I, _I]),
    "orbit_ssd_scan_phase": (_I, [C.POINTER(ScanArgs), _I, _P, _P, _I, _I, _P]),
    "orbit_ssd_scan_fwd": (_I, [C.POINTER(ScanArgs), _P, _P, _I, _I, _P]),
    "orbit_ssd_scan_bwd": (_I, [C.POINTER(ScanArgs), _P, _P, _I, _I, _P]),
    "orbit_ssd_scan_step": (_I, [C.POINTER(ScanArgs), _P, _P, _I, _P]),
    "orbit_token_map_fwd": (_I, [_P, _L, _P, _P, _F, _F, _P, _P, _L, _I, _I, _I, _P]),
    "orbit_token_map_bwd_workspace_bytes": (_L, [_I]),
    "orbit_token_map_bwd": (_I, [_P, _L, _P, _P, _P, _P, _L, _P, _P, _P, _L, _L, _I, _I, _I, _P]),
    "orbit_token_clock_fwd": (_I, [C.POINTER(ClockArgs), _I, _P]),
    "orbit_token_clock_bwd_workspace_bytes": (_L, [_L, _I, _I, _I, _I, _I]),
    "orbit_token_clock_bwd": (_I, [C.POINTER(ClockArgs), _I, _P]),
    "orbit_hm_scan_fwd": (_I, [C.POINTER(HmArgs), _I, _P]),
    "orbit_hm_scan_bwd": (_I, [C.POINTER(HmArgs), _I, _P]),
    "orbit_hm_tail_fwd": (_I, [C.POINTER(HmTailArgs), _I, _P]),
    "orbit_hm_tail_bwd_workspace_bytes": (_L, [_L, _I, _I]),
    "orbit_hm_tail_bwd": (_I, [C.POINTER(HmTailArgs), _I, _P]),
    "orbit_cp_record_floats": (_L, [_L, _I, _I]),
    "orbit_cp_state_pack_workspace_bytes": (_L, [_I, _I, _I]),
    "orbit_cp_state_pack": (_I, [_P, _P, _I, _I, _I, _L, _P, _L, _P]),
    "orbit_cp_state_combine": (_I, [_P, _L, _I, _I, _L, _I, _I, _I, _P, _P]),
    "orbit_selftest_umma": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "orbit_selftest_wait_timeout": (_I, [_P, _I, _P]),
}

_lib = None


def load():
    """Load the shared library once; raises `OrbitLibraryError` (with the build command) when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise OrbitLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m orbitssm_b200.build` (nvcc, sm_100a). "
            "backend='cuda' has no other implementation.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise OrbitLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(status: int, who: str):
    """Raise the Python exception that matches a nonzero status (the message is the library's own text)."""
    if status == 0:
        return
    msg = load().orbit_last_error().decode("utf-8", "replace")
    raise _STATUS_EXC.get(status, RuntimeError)(f"{who}: {msg} (status {status})")
