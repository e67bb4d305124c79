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
    L.sllm_num_sms.restype = c_int
    L.sllm_num_sms.argtypes = []
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
        "sllm_attention_tma_ctas_per_sm": [c_int],
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
        "sllm_gemm_pair_supports": [c_int, c_int, c_int],
        "sllm_gemm_pair": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        "sllm_gemm_pair_parts": [c_int],
        "sllm_gemm_pair_parts_of": [c_int, c_int],
        "sllm_gemm_pair_splits": [c_int, c_int],
        "sllm_linear_tc_supports": [c_int, c_int, c_int],
        "sllm_linear_tc_splits": [c_int, c_int],
        "sllm_linear_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "sllm_linear_ws_supports": [c_int, c_int, c_int],
        "sllm_linear_ws": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                           c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "sllm_linear_ws_parts": [c_int, c_int],
        "sllm_linear_stream_silu_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int,
                                           c_void_p],
        "sllm_linear_ws_rope_supports": [c_int, c_int, c_int, c_int, c_int, c_int, c_int],
        "sllm_linear_ws_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_float, c_int, c_void_p],
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


class KernelTimes:
    """Device time per entry point, for measurement: inside ``with KernelTimes() as kt:`` every launch
    is bracketed by two CUDA events on the current stream; ``kt.table()`` gives, per entry point, the
    number of launches and the summed milliseconds (the reference's counterpart is a host stopwatch
    around its steps, serving/diag.py:132-149).  Events between kernels keep one launch from starting
    under the tail of the one before, so the sum is an upper bound on what the same kernels take back
    to back.  Not for use while a CUDA graph is captured."""

    active = None

    def __init__(self):
        self.pairs: dict[str, list] = {}

    def __enter__(self):
        KernelTimes.active = self
        return self

    def __exit__(self, *exc):
        KernelTimes.active = None

    def table(self) -> dict:
        import torch
        torch.cuda.synchronize()
        return {name: (len(p), sum(a.elapsed_time(b) for a, b in p)) for name, p in self.pairs.items()}


_fns: dict = {}


def call(name: str, *args) -> None:
    fn = _fns.get(name)
    if fn is None:
        fn = _fns[name] = getattr(lib(), name)
    kt = KernelTimes.active
    if kt is None:
        rc = fn(*args)
    else:
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = fn(*args)
        b.record()
        kt.pairs.setdefault(name, []).append((a, b))
    launches["own"] += 1
    if rc != 0:
        msg = lib().sllm_last_error().decode(errors="replace")
        raise KernelError(f"{name} failed (code {rc}): {msg}")
