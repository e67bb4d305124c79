"""ctypes binding of the kernel library.  There is no fallback: if the library
cannot be built or loaded, or the device is not a CUDA device, every op raises.
"""

from __future__ import annotations

import ctypes
import threading

_lock = threading.Lock()
_lib = None
launches = {"own": 0, "library": 0}     # kernels launched since import: this package's, and library products


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import library_path
                try:
                    path = library_path()
                    _lib = _declare(ctypes.CDLL(path))
                except Exception as e:          # noqa: BLE001
                    raise KernelError(
                        "the sm_100a kernel library is not available and there is no other path: "
                        f"{e}") from e
    return _lib


def _declare(L):
    c_int, c_float, c_void_p, c_size_t = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
    L.sllm_last_error.restype = ctypes.c_char_p
    L.sllm_last_error.argtypes = []
    sigs = {
        "sllm_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "sllm_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_size_t, c_void_p, c_float, c_void_p, c_int,
                             c_int, c_int, c_void_p],
        "sllm_silu_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "sllm_gather_rows": [c_void_p, c_int, c_int, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "sllm_rope_kv_write": [c_void_p, c_int, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "sllm_gemm_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "sllm_attention_simt": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
        "sllm_sample_rows": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "sllm_repetition_penalty": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "sllm_mark_seen": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "sllm_penalty_seen": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "sllm_attention_mma_supports": [c_int],
        "sllm_attention_tma_supports": [c_int, c_int],
        "sllm_attention_tma_decode": [c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_float, c_int, c_void_p, c_void_p],
        "sllm_wait_probe": [c_void_p, ctypes.c_ulonglong, c_void_p, c_void_p],
        "sllm_attention_tc_supports": [c_int, c_int],
        "sllm_attention_tc": [c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p],
        "sllm_gemm_tcgen05_supports": [c_int, c_int, c_int],
        "sllm_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "sllm_linear_tc_supports": [c_int, c_int, c_int],
        "sllm_linear_tc_splits": [c_int, c_int],
        "sllm_linear_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "sllm_linear_ws_supports": [c_int, c_int, c_int],
        "sllm_linear_ws": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
        "sllm_linear_ws_rope_supports": [c_int, c_int, c_int, c_int, c_int, c_int, c_int],
        "sllm_linear_ws_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "sllm_linear_stream_supports": [c_int, c_int, c_int],
        "sllm_linear_stream_splits": [c_int, c_int],
        "sllm_linear_stream": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_void_p],
        "sllm_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_float, c_int, c_void_p],
    }
    for name, argtypes in sigs.items():
        fn = getattr(L, name)
        fn.restype = c_int
        fn.argtypes = argtypes
    return L


def declare_optional(name: str, argtypes) -> bool:
    """Declare an entry point that newer libraries have; False if absent."""
    L = lib()
    try:
        fn = getattr(L, name)
    except AttributeError:
        return False
    fn.restype = ctypes.c_int
    fn.argtypes = argtypes
    return True


def call(name: str, *args) -> None:
    L = lib()
    rc = getattr(L, name)(*args)
    launches["own"] += 1
    if rc != 0:
        msg = L.sllm_last_error().decode(errors="replace")
        raise KernelError(f"{name} failed (code {rc}): {msg}")
