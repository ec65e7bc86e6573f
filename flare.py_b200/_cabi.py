"""ctypes binding of libflare_b200.so (the C ABI declared in include/flare_b200.h).

The library is the only implementation: if it is missing or was not built
there is no fallback and importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libflare_b200.so"

F32, F16, BF16 = 0, 1, 2
TERM_GATHER, TERM_SCATTER, TERM_BOTH = 1, 2, 3
PATH_AUTO, PATH_SIMT, PATH_TC_EXACT = 0, 1, 2

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class FlareProblem(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("M", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("scale", C.c_float), ("n_splits", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("y_stride", C.c_int64 * 3), ("dy_stride", C.c_int64 * 3), ("dk_stride", C.c_int64 * 3),
        ("dv_stride", C.c_int64 * 3),
        ("dropout_p", C.c_float), ("dropout_seed", C.c_uint64),
    ]


class FlarePeers(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("bufs", C.c_void_p), ("mine", C.c_void_p),
                ("flags", C.c_void_p), ("epoch", C.c_int32)]


_P = C.POINTER(FlareProblem)
_G = C.POINTER(FlarePeers)
_vp, _i, _sz, _i64 = C.c_void_p, C.c_int, C.c_size_t, C.c_int64

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "flare_version": (_i, []),
    "flare_last_error": (C.c_char_p, []),
    "flare_set_path": (_i, [_i]),
    "flare_pick_splits": (_i, [_P]),
    "flare_fwd_workspace_bytes": (_sz, [_P]),
    "flare_bwd_workspace_bytes": (_sz, [_P]),
    "flare_mixer_fwd": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "flare_mixer_bwd": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "flare_gather_partial": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_combine": (_i, [_P, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "flare_combine_peers": (_i, [_P, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "flare_reduce_sum_peers": (_i, [_vp, _i, _i64, _i, _vp, _vp]),
    "flare_peer_barrier": (_i, [_G, _vp]),
    "flare_cp_mixer_fwd": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _G, _vp]),
    "flare_cp_mixer_bwd": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _G, _G, _vp]),
    "flare_scatter": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_bwd_dz_partial": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_reduce_sum": (_i, [_vp, _i, _i64, _i, _vp, _vp]),
    "flare_bwd_tokens": (_i, [_P, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_bwd_main": (_i, [_P, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_gather_noalloc": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_causal_workspace_bytes": (_sz, [_P]),
    "flare_causal_prefill": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_causal_decode": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_causal_bwd_workspace_bytes": (_sz, [_P]),
    "flare_causal_bwd": (_i, [_P, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_causal_linear_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "flare_causal_linear": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "flare_triple_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "flare_triple_outer": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, C.c_float, _vp, _vp, _vp]),
    "flare_triple_contract": (_i, [_i, _i, _i, _i, _i, _i, _vp, _i64, _i64, _i64, _vp, _vp, C.c_float, _vp, _vp]),
    "flare_device_status": (_i, [C.POINTER(C.c_int), _i]),
    "flare_probe_ex2": (_i, [_i, _i, _vp, _vp]),
    "flare_pass_counts": (_i, [C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "flare_bwd_dq_partial": (_i, [_P, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {PKG / 'build.py'}` "
            "(nvcc, sm_100a). flare_b200 has no other implementation to fall back to.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class FlareError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise FlareError(f"{what} failed (code {rc}): {lib.flare_last_error().decode()}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream
