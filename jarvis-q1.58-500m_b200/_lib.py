"""ctypes binding of libjarvis_b200.so.

There is no CPU fallback and no alternative backend: if the shared object is missing or a
call fails, a RuntimeError carrying the library's own message is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import re

from . import build as _build

_LIB = None
_HEADER = os.path.join(os.path.dirname(_build.PKG_DIR), "include", "jarvis_b200.h")

OK, ERR_ARG, ERR_CUDA = 0, -1, 1
EPI_BF16, EPI_GELU_BF16, EPI_RESID_F32, EPI_F32 = 0, 1, 2, 3
ATTN_QK_PREPARED = 1   # JB200_ATTN_QK_PREPARED

_P = C.c_void_p
_I = C.c_int
_Z = C.c_size_t
_F = C.c_float

# name -> (restype, argtypes); must list every function declared in include/jarvis_b200.h
PROTOTYPES = {
    "jb200_last_error": (C.c_char_p, []),
    "jb200_abi_version": (_I, []),
    "jb200_kernel_launches": (C.c_longlong, [_I]),
    "jb200_set_dependent_launch": (_I, [_I]),
    "jb200_device_status": (_I, [C.POINTER(C.c_uint), _I]),
    "jb200_selftest_bounded_wait": (_I, [_I, _P]),
    "jb200_pack_ternary_scratch_bytes": (_Z, [_I, _I]),
    "jb200_pack_ternary": (_I, [_P, _I, _I, _P, _P, _P, _P, _P]),
    "jb200_pack_codes": (_I, [_P, _Z, _P, _P]),
    "jb200_unpack_ternary": (_I, [_P, _Z, _I, _P, _P]),
    "jb200_ternary_linear": (_I, [_P, _I, _I, _P, _P, _I, _I, _I, _P, _I, _I, _P]),
    "jb200_prepare_weights": (_I, [_P, _Z, _P, _P]),
    "jb200_dense_linear": (_I, [_P, _I, _I, _P, _I, _I, _P, _I, _P]),
    "jb200_host_decode16_prepared": (None, [C.c_uint32, C.POINTER(C.c_uint32)]),
    "jb200_rmsnorm": (_I, [_P, _I, _P, _F, _P, _I, _I, _I, _P]),
    "jb200_embedding": (_I, [_P, _P, _I, _P, _I, _I, _P]),
    "jb200_attn_scan": (_I, [_P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P]),
    "jb200_qkv_linear_rope": (_I, [_P, _I, _I, _P, _P, _I, _I, _I, _P, _P, _I, _P, _I, _I, _P, _I, _I, _P]),
    "jb200_attn_scan_scratch_bytes": (_Z, [_I, _I, _I]),
    "jb200_router_top2": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "jb200_rmsnorm_router": (_I, [_P, _P, _F, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P]),
    "jb200_moe_metadata_scratch_bytes": (_Z, [_I, _I, _I]),
    "jb200_moe_metadata": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "jb200_moe_metadata_static_max_assignments": (_I, []),
    "jb200_moe_metadata_static": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "jb200_moe_dispatch_gather": (_I, [_P, _P, _I, _I, _I, _P, _P]),
    "jb200_moe_scatter_combine": (_I, [_P, _P, _P, _I, _I, _I, _P, _I, _P, _P]),
    "jb200_moe_finalize": (_I, [_P, _P, _P, _I, C.c_longlong, C.c_longlong, _F, _P, _P]),
    "jb200_lsf_scan": (_I, [_P, _I, _P, _P, _P, _P, _F, _F, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P]),
    "jb200_lsf_scan_scratch_bytes": (_Z, [_I, _I, _I]),
    "jb200_lsf_step_norm": (_I, [_P, _P, _P, _P, _I, C.c_longlong, C.c_longlong, _F, _P, _P, _F, _F, _P, _P, _P, _P, _F, _P,
                                 _I, _I, _P]),
    "jb200_peer_buffer_alloc": (_I, [_Z, _P, _P]),
    "jb200_peer_buffer_open": (_I, [_P, _P]),
    "jb200_peer_buffer_close": (_I, [_P]),
    "jb200_peer_buffer_free": (_I, [_P]),
    "jb200_peer_barrier": (_I, [_P, _I, _I, _P]),
    "jb200_ep_pull_gather": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "jb200_ep_pull_combine": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "jb200_sample": (_I, [_P, _I, _I, _I, _I, _F, _I, _F, _P, _P, _P, _P]),
    "jb200_host_decode16": (None, [C.c_uint32, C.POINTER(C.c_uint32)]),
    "jb200_ternary_linear_grouped": (_I, [_P, _I, _I, _P, _P, _I, _I, _P, _I, _P, _I, _I, _P]),
}


def declared_symbols() -> list[str]:
    """Function names declared in include/jarvis_b200.h."""
    with open(_HEADER) as fh:
        text = re.sub(r"/\*.*?\*/", "", fh.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(jb200_[a-z0-9_]+)\s*\(", text)))


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Load (building first if the sources changed and nvcc is present) the shared library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_build.LIB_PATH) or not _build.is_current():
        try:
            _build.build()
        except Exception as exc:  # no nvcc on this machine, or a compile error
            if not os.path.exists(_build.LIB_PATH):
                raise RuntimeError(
                    f"libjarvis_b200.so is not built and cannot be built here ({exc}); "
                    "there is no fallback path"
                ) from exc
    lib = C.CDLL(_build.LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def last_error() -> str:
    return load().jb200_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != OK:
        kind = "argument error" if rc == ERR_ARG else "CUDA error"
        raise RuntimeError(f"{what}: {kind}: {last_error()}")


def device_status(clear: bool = True) -> int:
    st = C.c_uint(0)
    check(load().jb200_device_status(C.byref(st), 1 if clear else 0), "jb200_device_status")
    return int(st.value)


def set_dependent_launch(enable: bool) -> bool:
    """Programmatic dependent launch of the library's kernels on/off; returns the previous setting."""
    return bool(load().jb200_set_dependent_launch(1 if enable else 0))


def kernel_launches(reset: bool = False) -> int:
    return int(load().jb200_kernel_launches(1 if reset else 0))
