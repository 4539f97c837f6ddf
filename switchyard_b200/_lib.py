"""ctypes binding of the C ABI in include/switchyard_b200.h.

The shared library is built in-tree (`python -m switchyard_b200.build`) and loaded from this
directory. There is no fallback: if the library is missing, or a call fails, a RuntimeError is
raised. ctypes releases the GIL for the duration of every call, so one host thread per GPU can
drive the kernels concurrently (the reference's extension releases it too,
switchyard/csrc/moe_kernels.cu:491-500)."""

import ctypes
import os
from ctypes import c_char_p, c_int, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libswitchyard_b200.so")

SY_DTYPE_F16, SY_DTYPE_BF16 = 0, 1
SY_ERR_DEVICE = -3

# name -> (restype, argtypes); must list every symbol the header declares
SYMBOLS = {
    "sy_last_error": (c_char_p, []),
    "sy_version": (c_char_p, []),
    "sy_device_status": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "sy_set_wait_limit_ns": (c_int, [ctypes.c_uint64]),
    "sy_wait_limit_ns": (ctypes.c_uint64, []),
    "sy_route": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "sy_sort_scratch_bytes": (c_size_t, [c_int, c_int]),
    "sy_sort_by_expert": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "sy_route_sort_max_choices": (c_int, []),
    "sy_route_sort": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "sy_route_fused_max_tokens": (c_int, []),
    "sy_route_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "sy_sort_by_expert_static": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p]),
    "sy_grouped_gemv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_void_p]),
    "sy_grouped_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_void_p]),
    "sy_force_compute_tile": (c_int, [c_int]),
    "sy_expert_ffn_scratch_bytes": (c_size_t, [c_int]),
    "sy_expert_ffn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "sy_expert_ffn_combine_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "sy_expert_ffn_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                      c_void_p]),
    "sy_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "sy_combine_add": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "sy_gather_rows": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "sy_copy_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "sy_enable_peer_access": (c_int, [c_int, c_int, ctypes.POINTER(c_int)]),
    "sy_grouped_segments": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "sy_ep_dispatch_scratch_bytes": (c_size_t, [c_int]),
    "sy_ep_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "sy_ep_expert_ffn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                 c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p]),
    "sy_ep_wait": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "sy_ep_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                              c_int, c_void_p]),
    "sy_ep_combine_add": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                  c_void_p, c_int, c_void_p]),
    "sy_ipc_export": (c_int, [c_void_p, c_void_p, ctypes.POINTER(ctypes.c_uint64)]),
    "sy_ipc_open": (c_int, [c_void_p, ctypes.c_uint64, ctypes.POINTER(c_void_p)]),
    "sy_ipc_close": (c_int, [c_void_p, ctypes.c_uint64]),
}

_LIB = None


def load():
    """The loaded library, with argument types set. Raises if it has not been built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m switchyard_b200.build` "
                "(nvcc, sm_100a). switchyard_b200 has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _LIB = lib
    return _LIB


def check(rc, what, lib=None):
    """Raises RuntimeError with the library's message unless rc is SY_OK. `lib`: the object the
    call was made on when it is not the loaded library (tests substitute one)."""
    if rc != 0:
        msg = (lib or load()).sy_last_error().decode(errors="replace")
        raise RuntimeError(f"switchyard_b200.{what} failed ({rc}): {msg}")
