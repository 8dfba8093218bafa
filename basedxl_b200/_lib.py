"""ctypes binding of libbasedxl_b200.so (C ABI declared in include/basedxl_b200.h).

There is no fallback: if the shared library is missing or a call fails, the
error is raised to the caller.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libbasedxl_b200.so")

_vp, _ll, _i, _f = C.c_void_p, C.c_longlong, C.c_int, C.c_float



class GemmFusedArgs(C.Structure):
    """``bxl_gemm_fused_args`` of include/basedxl_b200.h."""

    _fields_ = [
        ("A", _vp), ("lda", _ll), ("B", _vp), ("ldb", _ll), ("bias", _vp), ("bias_f32", _vp), ("residual", _vp), ("ldr", _ll),
        ("C", _vp), ("ldc", _ll), ("C2", _vp), ("ldc2", _ll), ("n_split", _i), ("geglu", _i),
        ("ln_partials", _vp), ("ln_parts", _i), ("ln_colsum", _vp), ("ln_eps", _f),
        ("row_stats", _vp), ("row_stats_capacity", _ll), ("M", _i), ("N", _i), ("K", _i),
    ]


# name -> (restype, argtypes); mirrors include/basedxl_b200.h one to one
SIGNATURES = {
    "bxl_init": (_i, []),
    "bxl_last_error": (C.c_char_p, []),
    "bxl_device_status": (_i, [C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "bxl_sm_count": (_i, []),
    "bxl_set_pdl": (_i, [_i]),
    "bxl_set_static_weights": (_i, [_i]),
    "bxl_debug_force_tiles": (_i, [_i, _i, _i]),
    "bxl_debug_force_tile_order": (_i, [_i]),
    "bxl_debug_force_attn_split": (_i, [_i]),
    "bxl_gemm_f16": (_i, [_vp, _ll, _vp, _ll, _i, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _vp]),
    "bxl_gemm_dual_f16": (_i, [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _i, _vp, _ll, _i, _i, _i, _vp]),
    "bxl_gemm_geglu_f16": (_i, [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _i, _i, _i, _vp]),
    "bxl_gemm_fused_f16": (_i, [C.POINTER(GemmFusedArgs), C.POINTER(_i), _vp]),
    "bxl_gemm_split_workspace_bytes": (_ll, [_i, _i, _i]),
    "bxl_gemm_split_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _ll, _vp]),
    "bxl_conv_weight_pack_f16": (_i, [_vp, _vp, _i, _i, _vp]),
    "bxl_conv3x3_halo_f16": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "bxl_conv3x3_direct_f16": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "bxl_halo_pack_f16": (_i, [_vp, _ll, _vp, _i, _i, _i, _i, _i, _vp]),
    "bxl_groupnorm_scratch_bytes": (_ll, [_i, _i]),
    "bxl_groupnorm_stats_f16": (_i, [_vp, _ll, _i, _i, _i, _i, _vp, _vp, _ll, _vp]),
    "bxl_groupnorm_stats_noalloc_max_bg": (_ll, []),
    "bxl_groupnorm_stats_noalloc_f16": (_i, [_vp, _ll, _i, _i, _i, _i, _vp, _vp]),
    "bxl_groupnorm_apply_f16": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _vp, C.POINTER(_vp), _i, _i, _i, _f, _vp, _vp, _i, _vp]),
    "bxl_groupnorm_fused_f16": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _i, _vp, C.POINTER(_vp), _i, _i, _i, _f, _vp, _vp, _i, _vp, _vp]),
    "bxl_attn_fwd_f16": (_i, [_vp, _ll, _ll, C.POINTER(_vp), _i, _ll, _ll, _i, _vp, _ll, _ll, _i, _i, _i, _i, _f, _vp]),
    "bxl_comm_ctl_bytes": (_ll, []),
    "bxl_comm_ipc_export": (_i, [_vp, C.c_char_p, C.POINTER(_ll)]),
    "bxl_comm_ipc_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "bxl_comm_ipc_close": (_i, [_vp]),
    "bxl_comm_exchange": (_i, [_vp, C.POINTER(_vp), _ll, _vp, C.POINTER(_vp), _i, _i, _i, C.c_double, _vp]),
    "bxl_upsample2x_f16": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "bxl_layernorm_f16": (_i, [_vp, _vp, _vp, _vp, _ll, _i, _f, _vp]),
    "bxl_geglu_f16": (_i, [_vp, _vp, _ll, _i, _vp]),
    "bxl_cfg_euler_step": (_i, [_vp, _vp, _vp, _ll, _f, _f, _f, _vp]),
}


class BxlError(RuntimeError):
    pass


_lib = None


def load() -> C.CDLL:
    """Load the shared library and declare every entry point.  Needs no GPU."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BxlError(
            f"{LIB_PATH} not found: build it with `python -m basedxl_b200.build` (there is no fallback path)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


_inited_devices: set[int] = set()


def lib() -> C.CDLL:
    """The loaded library, initialised for the current CUDA device."""
    import torch

    l = load()
    if not torch.cuda.is_available():
        raise BxlError("basedxl_b200 needs a CUDA device (sm_100a); none is available and there is no CPU path")
    dev = torch.cuda.current_device()
    if dev not in _inited_devices:
        torch.cuda.init()
        check(l.bxl_init(), l, kernels=0)
        _inited_devices.add(dev)
    return l


# kernels of this library enqueued so far by this process (each successful
# compute call adds the number of kernels it launches)
launches = 0


def check(rc: int, l: C.CDLL | None = None, kernels: int = 1) -> None:
    global launches
    if rc != 0:
        l = l or load()
        raise BxlError(f"libbasedxl_b200 error {rc}: {l.bxl_last_error().decode()}")
    launches += kernels


def device_status() -> None:
    """Synchronise and raise if any kernel recorded a failed bounded wait."""
    l = lib()
    code, site, block = _i(0), _i(0), _i(0)
    check(l.bxl_device_status(C.byref(code), C.byref(site), C.byref(block)), l, kernels=0)
