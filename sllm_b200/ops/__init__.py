"""The operations a step is made of, each a hand-written sm_100a kernel.

Tensors must lie on a CUDA device and be contiguous; there is no CPU path and no
library model code behind these functions.  Matrix products of the bfloat16
path with many rows go to cuBLAS (as the reference's engine does,
kernels/cuda/kernels.cu:752-767); everything else, and every product of the
float32 path, runs in this package's own kernels.
"""

from __future__ import annotations

import functools
import os

import torch

from ._lib import KernelError, KernelTimes, call, launches, lib  # noqa: F401

F32, BF16 = 0, 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16")


def _dtc(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16")


def _chk(*tensors) -> None:
    for t in tensors:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            if not t.is_cuda:
                raise KernelError("the kernels run on a CUDA device only; got a tensor on " + str(t.device))
            raise KernelError("the kernels take contiguous tensors")


def _p(t):
    return None if t is None else t.data_ptr()


# the raw handle of the current stream: torch's quick accessor where this torch has it (the public
# `current_stream()` builds a Stream object, several microseconds a launch)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_current_device = getattr(torch._C, "_cuda_getDevice", None)      # (torch.cuda.current_device() checks initialisation each time)


def _stream():
    if _raw_stream is not None:
        return _raw_stream(_current_device() if _current_device is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def embed_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """float32 ``[T, H]`` rows of ``table`` (``[V, H]``) at int32 ``ids``."""
    _chk(table, ids)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    call("sllm_embed_gather", _p(table), _dt(table), _p(ids), _p(out), T, H, V, _stream())
    return out


def add_rmsnorm(residual: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype) -> torch.Tensor:
    """``residual += delta`` (in place, if delta is given; a 3-d delta is a stack of
    partial sums) and return ``rmsnorm(residual) * weight`` in ``out_dtype``."""
    _chk(residual, delta, weight)
    rows, H = residual.shape
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream and the gain are float32")
    parts, stride = 1, 0
    if delta is not None:
        if delta.dim() == 3:
            parts, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        if tuple(delta.shape[-2:]) != (rows, H):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not fit residual {(rows, H)}")
    out = torch.empty((rows, H), dtype=out_dtype, device=residual.device)
    call("sllm_add_rmsnorm", _p(residual), _p(delta), _dt(delta) if delta is not None else F32, parts, stride,
         _p(weight), float(eps), _p(out), _dtc(out_dtype), rows, H, _stream())
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias) -> torch.Tensor:
    """True float32 ``x @ w.T + bias``: CUDA-core FMA, fixed summation order."""
    _chk(x, w, bias)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    call("sllm_gemm_f32", _p(x), _p(w), _p(bias), _p(out), M, N, K, _stream())
    return out


TCGEN05_MIN_ROWS = 128    # below this a 128-row tile is mostly padding
PAIR_SILU_FROM_ROWS = 64  # from here on gate|up with its activation goes to the CTA-pair kernel (see `linear_silu_mul`)
STREAM_MAX_ROWS = 32      # beyond this the kernel's shared-memory reads of the activations bound it


@functools.lru_cache(maxsize=4096)
def stream_supports(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming kernel is the one for this product (it is not where the tensor-core form
    of the same job is the faster one: see `linear_tc_supports`)."""
    if not (M <= STREAM_MAX_ROWS and bool(lib().sllm_linear_stream_supports(int(M), int(N), int(K)))):
        return False
    return not linear_tc_supports(M, N, K)


def linear_stream(x, w, bias, out_dtype, *, splits: int = 1, silu: bool = False):
    """The weight-streaming kernel for at most 64 tokens.  With ``splits`` > 1 the result is
    a float32 stack ``[splits', M, N]`` of partial sums (bias in the first) that the consumer
    adds; with ``silu`` the matrix is gate|up interleaved in blocks of 8 and the result is
    ``silu(gate) * up`` of width N/2."""
    _chk(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    L = lib()
    real = L.sllm_linear_stream_splits(K, int(splits)) if splits > 1 else 1
    partial = None
    if real > 1:
        partial = torch.empty((real, M, N), dtype=torch.float32, device=x.device)
        out = None
    else:
        out = torch.empty((M, N // 2 if silu else N), dtype=out_dtype, device=x.device)
    call("sllm_linear_stream", _p(x), _p(w), _p(bias), _p(out), _dtc(out_dtype), _p(partial), M, N, K,
         real if real > 1 else 1, 1 if silu else 0, _stream())
    return partial if real > 1 else out


_tc_status: dict = {}      # device -> int32[1]: non-zero once a wait inside a tcgen05 kernel ran out
_tc_used = {"since_check": 0}


def _status_word(device) -> torch.Tensor:
    t = _tc_status.get(device)
    if t is None:
        t = _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def status_word_launches() -> int:
    """Launches since the last check of kernels that report through the status word."""
    return _tc_used["since_check"]


def note_status_word_launches(n: int) -> None:
    """A replayed CUDA graph launched ``n`` such kernels (the capture counted them once)."""
    _tc_used["since_check"] += int(n)


def check_tcgen05_status() -> None:
    """Raise if a bounded wait inside a TMA-fed kernel (the tcgen05 product, the TMA attention) gave
    up since the last check (reads one int from each device that ran such a kernel; synchronises)."""
    if not _tc_used["since_check"]:
        return
    _tc_used["since_check"] = 0
    for dev, t in _tc_status.items():
        code = int(t.item())
        if code:
            t.zero_()
            who = {1: "gemm_tcgen05: the TMA producer", 2: "gemm_tcgen05: the MMA issuer", 3: "gemm_tcgen05: the epilogue",
                   11: "attention_tma: the producer", 12: "attention_tma: a compute warp",
                   41: "gemm_pair: the TMA producer", 42: "gemm_pair: the MMA issuer", 43: "gemm_pair: the epilogue",
                   31: "linear_tc: the TMA producer", 32: "linear_tc: the MMA issuer", 33: "linear_tc: the epilogue",
                   }.get(code, f"code {code}")
            raise KernelError(f"{who} on {dev}: a bounded wait ran out; the result is not valid")


@functools.lru_cache(maxsize=4096)
def tcgen05_supports(M: int, N: int, K: int) -> bool:
    return bool(lib().sllm_gemm_tcgen05_supports(int(M), int(N), int(K)))


def gemm_tcgen05(x, w, bias, out_dtype, *, silu: bool = False):
    """``x @ w.T (+ bias)`` on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory);
    with ``silu`` the matrix is gate|up interleaved in blocks of 8 and the bfloat16 result is
    ``silu(gate) * up`` of width N/2."""
    _chk(x, w, bias)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05: bfloat16 operands only")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    if silu:
        epi, out = 2, torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    elif out_dtype == torch.float32:
        epi, out = 0, torch.empty((M, N), dtype=torch.float32, device=x.device)
    else:
        epi, out = 1, torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    call("sllm_gemm_tcgen05", _p(x), _p(w), _p(bias), _p(out), M, N, K, epi, _p(_status_word(x.device)), _stream())
    _tc_used["since_check"] += 1
    return out


# which products of prompt portions (more than 128 rows) run on this package's CTA-pair kernel: "all", "fused" (only
# gate|up with its SiLU epilogue; the plain products go to the library) or "off" (the one-CTA kernel for gate|up)
_PAIR_GEMM = os.environ.get("SLLM_PAIR_GEMM", "all")


@functools.lru_cache(maxsize=4096)
def pair_supports(M: int, N: int, K: int) -> bool:
    return bool(lib().sllm_gemm_pair_supports(int(M), int(N), int(K)))


@functools.lru_cache(maxsize=4096)
def pair_tiles_wide(M: int, N: int) -> bool:
    """Whether tiles of 256 x 512 serve an [M, N] result better than tiles of 256 x 256.  The pairs of SMs run
    the tiles in waves; a wide tile takes twice a narrow one's time and a quarter less traffic from L2, but its
    epilogue is not hidden behind the next tile's products.  So: wide where it needs no more time in waves and a
    pair has few tiles anyway (the attention and down projections of a prompt portion: one wave in place of one
    and a half), narrow where a pair walks many tiles (gate|up: sixteen each at 2,048 rows)."""
    pairs = max(num_sms() // 2, 1)
    mt = -(-M // 256)
    waves_narrow = -(-(mt * -(-N // 256)) // pairs)
    waves_wide = -(-(mt * -(-N // 512)) // pairs)
    return 2 * waves_wide <= waves_narrow and waves_narrow < 4


@functools.lru_cache(maxsize=4096)
def pair_wide_cols(M: int, N: int):
    """`pair_tiles_wide` for the epilogues that also have wide tiles of 448, 384 and 320 columns (float32 result,
    residual).  Measured, a wave of wide tiles takes time in proportion to 256 + its columns (the operands a pair
    pulls per k block) and a wave of 256-wide tiles as much as 384 such units (2,048 rows, K = 5,120, us a wave:
    48 / 50 / 55 / 63 at 320 / 384 / 448 / 512 columns, 30.5 at 256).  A narrower wide tile is taken where it
    beats both the 512-wide and the 256-wide tiles by that count: 2,048 x 3,584 (the attention and down
    projections of a 7B model) has 56 tiles of 512 for 74 pairs of SMs and 64 of 448 (58 -> 53 us and 232 -> 214
    with the residual epilogue); 1,024 x 5,120 goes from 77 us to 60 at 320 columns.
    False: 256 x 256; True: 256 x 512; else the width."""
    pairs = max(num_sms() // 2, 1)
    mt = -(-M // 256)
    waves_narrow = -(-(mt * -(-N // 256)) // pairs)
    if waves_narrow >= 4:
        return False
    best, best_cost = False, waves_narrow * 384
    if pair_tiles_wide(M, N):
        best, best_cost = True, min(best_cost, -(-(mt * -(-N // 512)) // pairs) * 768)
    for cols in (448, 384, 320):
        cost = -(-(mt * -(-N // cols)) // pairs) * (256 + cols)
        if cost < best_cost:
            best, best_cost = cols, cost
    return best


@functools.lru_cache(maxsize=4096)
def pair_tiles_slim(M: int, N: int) -> bool:
    """Whether tiles of 256 x 128 serve an [M, N] result better than tiles of 256 x 256: where the wider ones
    would leave at least half of the pairs of SMs without a tile (a prompt portion of 512 tokens times the
    q|k|v matrix: 36 tiles for 74 pairs; 30.6 -> 25.5 us).  The gain is small, since a pair is bound by the rate
    at which it pulls its operands and half the width moves three quarters of the bytes; where K is long enough
    the product is cut along K instead (`pair_splits`)."""
    pairs = max(num_sms() // 2, 1)
    return 2 * (-(-M // 256) * -(-N // 256)) <= pairs


PAIR_SPLIT_MAX = 8            # slices of K at most (each leaves a float32 copy of the result for the consumer to add)
PAIR_SPLIT_MIN_BLOCKS = 8     # 64-wide k blocks a slice has at least
PAIR_US_PER_K_BLOCK = 0.4     # a pair of SMs on one 256 x 256 tile, per 64-wide k block (measured: 116 us for K = 18,944)
PAIR_US_PER_ELEMENT = 2.4e-6  # one more float32 copy of the result for the next kernel to add, per element (whole portions
                              # of 192 to 1,024 tokens were timed with 0.5, 1.0 and 2.4: the last gave the best choices)
PAIR_SPLIT_GAIN = 0.85        # slices only where the whole path (slices, then a kernel that adds them) takes this share
PAIR_SPLIT_GAIN_WAVES = 0.8    # the same where the unsliced tiles are more than one wave


@functools.lru_cache(maxsize=4096)
def pair_splits(M: int, N: int, K: int) -> int:
    """Slices of K for the CTA-pair product of an [M, N] result with few 256 x 256 tiles: a pair of SMs pulls its
    operands through shared memory at a rate of its own, so a product whose tiles leave most pairs idle takes as
    long as its tiles' K, whatever the GPU could do (512 tokens times the down projection: 28 tiles for 74 pairs,
    116 us; the library's product 56).  With S slices a unit is (tile, slice), the units run in waves over the pairs
    and the time goes as waves / S; the slices' partial sums are a stack for the consumer to add (512 tokens, down:
    66 us in two slices).  The choice weighs that against the fused epilogues the unsliced product keeps: waves x K
    blocks for the products, a copy of the result per slice written and read, three copies for the residual
    epilogue's traffic (in a graph, measured: within 10 % of this at 192 to 1,024 tokens)."""
    pairs = max(num_sms() // 2, 1)
    tiles = -(-M // 256) * -(-N // 256)
    k_blocks = -(-K // 64)
    t_tile, t_copy = k_blocks * PAIR_US_PER_K_BLOCK, M * N * PAIR_US_PER_ELEMENT
    whole = -(-tiles // pairs) * t_tile + 3 * t_copy
    best, best_cost = 1, whole
    for s in range(2, PAIR_SPLIT_MAX + 1):
        if k_blocks // s < PAIR_SPLIT_MIN_BLOCKS:
            break
        cost = -(-tiles * s // pairs) / s * t_tile + (s + 2) * t_copy
        if cost < best_cost:
            best, best_cost = s, cost
    # (more than one wave of tiles: whole portions gained where the model promised a quarter (hidden 5,120, 1,024
    # tokens: 7.7 -> 7.3 ms for 8 layers) and not where it promised a fifth (hidden 3,584, 1,792 tokens))
    gain = PAIR_SPLIT_GAIN if tiles <= pairs else PAIR_SPLIT_GAIN_WAVES
    return best if best_cost <= gain * whole else 1


def gemm_pair(x, w, bias, out_dtype, *, silu: bool = False, wide: "bool | str | None" = None, scale: "RowScale | None" = None,
              residual=None, next_gain=None, splits: int = 1):
    """The same product and epilogues as `gemm_tcgen05`, by pairs of CTAs on 256 x 256 tiles, on
    256 x 512 tiles (``wide=True``; by default where those fill the GPU at least as well; ``wide=448``, ``384`` or
    ``320``: tiles of that many columns, float32 result or residual epilogue, chosen by `pair_wide_cols` where
    they fill the pairs of SMs better) or on 256 x 128 tiles (``wide="slim"``; by default where the result has few tiles)
    (``tcgen05.mma`` with ``cta_group::2``: each CTA loads half of each operand).
    ``scale``: a norm still owed on ``x`` (`RowScale`).  ``residual`` (float32 ``[M, N]``): the product is added
    into it in place and None is returned; with ``next_gain`` the kernel also writes the next norm's input in the
    owed form and ``(xg, RowScale)`` comes back (the scale's eps left at 0 for the caller to set).
    ``splits`` > 1 (float32 result, no other epilogue): K in that many slices, the result a stack ``[splits', M, N]``
    of partial sums (bias in the first) for the consumer to add."""
    _chk(x, w, bias, residual, next_gain)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_pair: bfloat16 operands only")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    out = xg = ssq = None
    stride = 0
    plain_or_residual = not silu and (residual is not None or out_dtype == torch.float32)
    if wide is None:
        wide = False if splits > 1 else "slim" if pair_tiles_slim(M, N) else \
            pair_wide_cols(M, N) if plain_or_residual else pair_tiles_wide(M, N)
    code = 2 if wide == "slim" else 0 if wide is False else 1 if wide is True or wide == 512 else int(wide)
    if code > 2 and (code not in (448, 384, 320) or not plain_or_residual):
        raise KernelError(f"gemm_pair: tiles of {wide} columns (448, 384 or 320, and only with a float32 result or a residual)")
    if residual is not None:
        if silu or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError(f"gemm_pair: residual {tuple(residual.shape)} {residual.dtype} does not fit [{M}, {N}] float32")
        epi = 3
        if next_gain is not None:
            if next_gain.dtype != torch.float32 or next_gain.numel() != N:
                raise KernelError("gemm_pair: the next norm's gain is float32 of N values")
            parts = pair_parts(N, code)
            stride = (parts + 3) & ~3
            xg = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            ssq = torch.empty((M, stride), dtype=torch.float32, device=x.device)
    elif silu:
        epi, out = 2, torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    elif out_dtype == torch.float32:
        real = int(lib().sllm_gemm_pair_splits(K, int(splits))) if splits > 1 else 1
        epi, out = 0, torch.empty((real, M, N) if real > 1 else (M, N), dtype=torch.float32, device=x.device)
    else:
        epi, out = 1, torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if splits > 1 and (epi != 0 or scale is not None):
        raise KernelError("gemm_pair: slices of K leave float32 partial sums: no other epilogue, no owed norm")
    call("sllm_gemm_pair", _p(x), _p(w), _p(bias), _p(out), M, N, K, epi, code, int(splits),
         *(scale.args_with_stride() if scale is not None else (None, 0, 0, 0.0, 0)),
         _p(residual), _p(next_gain), _p(xg), _p(ssq), stride, _p(_status_word(x.device)), _stream())
    _tc_used["since_check"] += 1
    if residual is not None:
        return (xg, RowScale(ssq, pair_parts(N, code), 0.0, N)) if next_gain is not None else None
    return out


@functools.lru_cache(maxsize=256)
def pair_parts(N: int, form: int = 0) -> int:
    """Partial sums of squares per row that `gemm_pair`'s residual epilogue writes for N columns with tiles of the
    form ``form`` (the kernel's code: 0, 1, 2, or 448, 384, 320)."""
    return int(lib().sllm_gemm_pair_parts_of(int(N), int(form)))


LINEAR_TC_MAX_ROWS = 128  # the tokens are the tensor core's N side: one tile of at most 128
# Plain products go to it only where it beats the library: a reduction of at least this length with at
# most this many tokens (at 7B sizes, 64 tokens: down 29.3 against 30.7 us; qkv 11.6 against 9.2 us).
LINEAR_TC_SPLIT_MIN_K = 8192
LINEAR_TC_SPLIT_MAX_ROWS = 64


_LINEAR_TC = os.environ.get("SLLM_LINEAR_TCGEN05", "1") != "0"     # 0: 33..128 tokens on the library product


# From how many tokens on it takes a product over from the streaming kernel, by the matrix's size (in-graph
# times at 7B sizes, us, streaming kernel / this one).  A small matrix (q|k|v, o_proj: under 2^25 elements)
# stays with the streaming kernel as far as that goes (24 tokens: 9.1 / 10.1, 7.2 / 9.3).  A large one moves
# from 17 tokens on (24 tokens: gate|up 52.0 / 48.3, down 28.9 / 26.9; 16 tokens: 45.2 / 52.3, 24.3 / 26.3).
# A very wide one (the output head: at least four 128-row tiles an SM) moves from 9 on (16 tokens: 190.5 /
# 179.6; 32 tokens: 222.7 / 180.4; 8 tokens: 184.3 / 179.7, left where it is).
LINEAR_TC_LARGE = 1 << 25
LINEAR_TC_LARGE_FROM_ROWS = 17
LINEAR_TC_WIDE_TILES_PER_SM = 4
LINEAR_TC_WIDE_FROM_ROWS = 9


def _tc_from_rows(N: int, K: int) -> int:
    if N * K < LINEAR_TC_LARGE:
        return STREAM_MAX_ROWS + 1
    if -(-N // 128) >= LINEAR_TC_WIDE_TILES_PER_SM * num_sms():
        return LINEAR_TC_WIDE_FROM_ROWS
    return LINEAR_TC_LARGE_FROM_ROWS


@functools.lru_cache(maxsize=4096)
def linear_tc_supports(M: int, N: int, K: int) -> bool:
    if not (_LINEAR_TC and M <= LINEAR_TC_MAX_ROWS and bool(lib().sllm_linear_tc_supports(int(M), int(N), int(K)))):
        return False
    return M >= _tc_from_rows(N, K)


@functools.lru_cache(maxsize=4096)
def _tc_splits(N: int, K: int) -> int:
    """Slices of K so that (tiles of 128 rows) x slices comes to about one unit per SM, each slice
    at least eight 64-wide k blocks long."""
    tiles = -(-N // 128)
    return max(1, min(num_sms() // tiles, (K // 64) // 8))


def linear_tc(x, w, bias, out_dtype, *, splits: int = 1, silu: bool = False):
    """The weight-streaming product on the tcgen05 tensor cores for up to 128 tokens.  With
    ``splits`` > 1 the result is a float32 stack ``[splits', M, N]`` of partial sums (bias in the
    first) that the consumer adds; with ``silu`` the matrix is gate|up interleaved in blocks of 8
    and the bfloat16 result is ``silu(gate) * up`` of width N/2."""
    _chk(x, w, bias)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("linear_tc: bfloat16 operands only")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    real = 1
    if silu:
        epi, out = 2, torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    elif out_dtype == torch.float32:
        real = int(lib().sllm_linear_tc_splits(K, int(splits))) if splits > 1 else 1
        epi = 0
        out = torch.empty((real, M, N) if real > 1 else (M, N), dtype=torch.float32, device=x.device)
    else:
        epi, out = 1, torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    call("sllm_linear_tc", _p(x), _p(w), _p(bias), _p(out), M, N, K, real, epi, _p(_status_word(x.device)), _stream())
    _tc_used["since_check"] += 1
    return out


WS_MAX_COLS = 8192        # wider products have CTAs enough for the 128-row streaming kernel
WS_MAX_ROWS = 32          # one, two or four 8-token tiles (with fewer k blocks in flight the more tiles, so that two CTAs still share an SM)
# Four tiles (17..32 tokens, one k block in flight per group) stream slowly, so only where little streams and the
# fused epilogues save kernels: a short reduction, a matrix of at most 2^24 elements, and rows enough for one and a
# half CTAs an SM (q|k|v and o_proj at a hidden size of 3,584: decode at batch 24 and 32 +2.5 %; at hidden sizes of
# 1,536 and 2,048 the k-split kernel with its norm and rotary kernels stayed the faster, 2.05 against 2.21 ms a step).
WS_ROWS32_MAX_ELEMENTS = int(os.environ.get("SLLM_WS_ROWS32_MAX_ELEMENTS", str(1 << 24)))
WS_ROWS32_MAX_K = 4096
MAX_SCALE_PARTS_ROWS32 = 192   # the table of partial sums a four-tile consumer keeps (streams of up to 3,072 columns)


@functools.lru_cache(maxsize=4096)
def ws_supports(M: int, N: int, K: int) -> bool:
    """Whether the warp-split kernel is the one for this product.  With two token tiles (9..16 tokens) only where
    its 16-row CTAs fit the GPU at once: at N = 5120 (320 to 592 CTAs for 296 places) it falls behind the k-split
    kernel by more than the fused epilogues save (16 tokens, K = 27648: 64.3 against 49.2 us)."""
    if not (M <= WS_MAX_ROWS and N <= WS_MAX_COLS and bool(lib().sllm_linear_ws_supports(int(M), int(N), int(K)))):
        return False
    return _ws_tokens_ok(M, N, K)


def _ws_tokens_ok(M: int, N: int, K: int) -> bool:
    if M <= 8:
        return True
    if -(-N // 16) > 2 * num_sms():
        return False
    return M <= 16 or (N * K <= WS_ROWS32_MAX_ELEMENTS and K <= WS_ROWS32_MAX_K and 2 * -(-N // 16) >= 3 * num_sms())


class RowScale:
    """An RMSNorm still owed on an activation: the activation is bfloat16(stream * gain), ``ssq`` is float32
    ``[M, stride]`` (stride = ``parts`` rounded up to 4) with ``parts`` partial sums of squares of each row of
    the stream (``width`` wide), and whoever multiplies the activation by a matrix multiplies each row of the
    result by ``rsqrt(sum(ssq[row, :parts]) / width + eps)``: W (x g / rms) = (W (x g)) / rms."""
    __slots__ = ("ssq", "parts", "eps", "width")

    def __init__(self, ssq, parts: int, eps: float, width: int):
        self.ssq, self.parts, self.eps, self.width = ssq, int(parts), float(eps), int(width)

    def args(self):
        return _p(self.ssq), self.parts, self.eps, self.width

    def args_with_stride(self):
        return _p(self.ssq), self.parts, self.ssq.shape[1], self.eps, self.width


_NO_SCALE = (None, 0, 0.0, 0)
MAX_SCALE_PARTS = 608          # partial sums a consumer keeps in shared memory per row


def linear_ws(x, w, bias, out_dtype, residual=None, scale: RowScale | None = None, next_gain=None):
    """The warp-split streaming kernel (at most 16 tokens): ``x @ w.T (+ bias)`` in ``out_dtype``,
    or, given ``residual`` (float32 ``[M, N]``), added into it in place (returns None).  ``scale``: a norm
    still owed on ``x`` (`RowScale`).  ``next_gain`` (with ``residual``): the gain of the norm that follows; the
    kernel then also writes that norm's input in the owed form and ``(xg, RowScale)`` is returned (the scale's
    eps is left at 0 for the caller to set)."""
    _chk(x, w, bias, residual, next_gain)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit w {tuple(w.shape)}")
    out = None
    if residual is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    elif residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
        raise KernelError(f"linear: residual {tuple(residual.shape)} {residual.dtype} does not fit [{M}, {N}] float32")
    xg = ssq = None
    parts = 0
    if next_gain is not None:
        if residual is None or next_gain.dtype != torch.float32 or next_gain.numel() != N:
            raise KernelError("linear_ws: the next norm's input needs the residual epilogue and a float32 gain of N values")
        parts = int(lib().sllm_linear_ws_parts(N, K))
        xg = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ssq = torch.empty((M, (parts + 3) & ~3), dtype=torch.float32, device=x.device)
    call("sllm_linear_ws", _p(x), _p(w), _p(bias), _p(out), _dtc(out_dtype), _p(residual), M, N, K,
         *(scale.args() if scale is not None else _NO_SCALE), _p(next_gain), _p(xg), _p(ssq), _stream())
    if next_gain is not None:
        return xg, RowScale(ssq, parts, 0.0, N)
    return out


def _pair_rows(M: int) -> bool:
    return _PAIR_GEMM == "all" and M > TCGEN05_MIN_ROWS


def can_accumulate(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `linear_accumulate` has a kernel for these operands: few tokens (the warp-split streaming
    kernel) or a prompt portion (the CTA-pair product)."""
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda):
        return False
    M, K = x.shape
    N = w.shape[0]
    if ws_supports(M, N, K):
        return True
    # (a result of so few tiles that it is better cut along K leaves partial sums, which a norm kernel adds)
    return _pair_rows(M) and N % 4 == 0 and pair_supports(M, N, K) and pair_splits(M, N, K) == 1


def linear_accumulate(x, w, bias, residual) -> None:
    """``residual += x @ w.T (+ bias)`` in one kernel (see `can_accumulate`)."""
    if ws_supports(x.shape[0], w.shape[0], x.shape[1]):
        linear_ws(x, w, bias, torch.float32, residual=residual)
    else:
        gemm_pair(x, w, bias, torch.float32, residual=residual)


_NORM_FUSED = os.environ.get("SLLM_NORM_FUSED", "1") != "0"     # 0: every RMSNorm of a step is a kernel of its own


def can_accumulate_norm(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `linear_accumulate_norm` has a kernel for these operands."""
    if not (_NORM_FUSED and can_accumulate(x, w)):
        return False
    M, N = x.shape[0], w.shape[0]
    if ws_supports(M, N, x.shape[1]):
        return int(lib().sllm_linear_ws_parts(N, x.shape[1])) <= (MAX_SCALE_PARTS if M <= 16 else MAX_SCALE_PARTS_ROWS32)
    return N % 8 == 0


def linear_accumulate_norm(x, w, bias, residual, gain, eps: float):
    """``residual += x @ w.T (+ bias)`` and, from the same kernel, the input of the RMSNorm (``gain``, ``eps``)
    that follows, in the owed form: ``(bfloat16(residual * gain), RowScale)``."""
    if ws_supports(x.shape[0], w.shape[0], x.shape[1]):
        xg, scale = linear_ws(x, w, bias, torch.float32, residual=residual, next_gain=gain)
    else:
        xg, scale = gemm_pair(x, w, bias, torch.float32, residual=residual, next_gain=gain)
    scale.eps = float(eps)
    return xg, scale


def linear_scaled_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `linear` takes ``x`` with a norm still owed (``scale=``): a prompt portion on the CTA-pair product."""
    M, K = x.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _pair_rows(M)
            and pair_supports(M, w.shape[0], K))


def _stream_splits(N: int, K: int) -> int:
    ctas = -(-N // 128)
    return max(1, min(2 * num_sms() // ctas, K // 128, 16))


def linear(x: torch.Tensor, w: torch.Tensor, bias, out_dtype: torch.dtype, allow_partials: bool = False,
           scale: "RowScale | None" = None) -> torch.Tensor:
    """``x @ w.T (+ bias)``; ``w`` is ``[N, K]``.  float32 operands: this package's
    float32 kernel.  bfloat16 operands, float32 accumulation, result in ``out_dtype``: up
    to 64 rows the weight-streaming kernel (which, if ``allow_partials``, may return a
    float32 stack of partial sums ``[parts, M, N]`` for the consumer to add); beyond that
    the library product."""
    if x.dtype != w.dtype:
        raise KernelError(f"linear: x is {x.dtype}, w is {w.dtype}")
    if scale is not None:                       # a norm still owed on x (see `linear_scaled_supports`)
        if not linear_scaled_supports(x, w):
            raise KernelError("linear: no kernel takes this input with its norm still owed")
        return gemm_pair(x, w, bias, out_dtype, scale=scale)
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the float32 path keeps float32 results")
        return gemm_f32(x, w, bias)
    _chk(x, w, bias)
    if not x.is_cuda:
        raise KernelError("linear: CUDA only")
    M, K = x.shape
    N = w.shape[0]
    if ws_supports(M, N, K):
        return linear_ws(x, w, bias, out_dtype)
    if stream_supports(M, N, K):
        splits = _stream_splits(N, K) if (allow_partials and out_dtype == torch.float32) else 1
        return linear_stream(x, w, bias, out_dtype, splits=splits)
    if allow_partials and out_dtype == torch.float32 and M <= LINEAR_TC_SPLIT_MAX_ROWS and K >= LINEAR_TC_SPLIT_MIN_K \
            and linear_tc_supports(M, N, K):
        # a long reduction into few columns (the down projection): slices of K over all the SMs
        return linear_tc(x, w, bias, out_dtype, splits=_tc_splits(N, K))
    if N * K >= LINEAR_TC_LARGE and -(-N // 128) >= num_sms() and linear_tc_supports(M, N, K):
        return linear_tc(x, w, bias, out_dtype)      # a large matrix whose 128-row tiles are enough for every SM
    if _PAIR_GEMM == "all" and M > TCGEN05_MIN_ROWS and pair_supports(M, N, K):
        # prompt portions: pairs of CTAs on the tensor cores (tcgen05.mma with cta_group::2); a result of few tiles in
        # slices of K where the consumer adds partial sums
        if allow_partials and out_dtype == torch.float32 and pair_splits(M, N, K) > 1:
            return gemm_pair(x, w, bias, out_dtype, splits=pair_splits(M, N, K))
        return gemm_pair(x, w, bias, out_dtype)
    launches["library"] += 1
    if out_dtype == torch.float32:
        out = torch.mm(x, w.t(), out_dtype=torch.float32)
    else:
        out = torch.mm(x, w.t())
    if bias is not None:
        out += bias.to(out.dtype)
    return out


def silu_mul(gu: torch.Tensor, interleave: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``silu(gate) * up`` of ``gu [T, 2I]`` whose columns alternate between gate
    and up in blocks of ``interleave``."""
    _chk(gu)
    T, two_i = gu.shape
    I = two_i // 2
    out = torch.empty((T, I), dtype=out_dtype, device=gu.device)
    call("sllm_silu_mul", _p(gu), _dt(gu), _p(out), _dtc(out_dtype), T, I, int(interleave), _stream())
    return out


def silu_scaled_supports(x, w_gate_up, interleave: int, out_dtype) -> bool:
    """Whether `linear_silu_mul` takes an input whose norm is still owed (``scale``)."""
    M, K = x.shape
    N = w_gate_up.shape[0]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and interleave == 8 and N % 16 == 0):
        return False
    return (M <= 32 and stream_supports(M, N, K)) or (M > TCGEN05_MIN_ROWS and _PAIR_GEMM != "off" and pair_supports(M, N, K))


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, interleave: int, out_dtype: torch.dtype,
                    scale: RowScale | None = None) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` with gate and up rows interleaved in one matrix.  ``scale``: a norm still
    owed on ``x`` (`RowScale`; see `silu_scaled_supports`)."""
    if scale is not None:
        if not silu_scaled_supports(x, w_gate_up, interleave, out_dtype):
            raise KernelError("linear_silu_mul: no kernel takes this input with its norm still owed")
        _chk(x, w_gate_up, scale.ssq)
        M, K = x.shape
        N = w_gate_up.shape[0]
        if M > 32:
            return gemm_pair(x, w_gate_up, None, out_dtype, silu=True, scale=scale)
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        call("sllm_linear_stream_silu_scaled", _p(x), _p(w_gate_up), _p(out), M, N, K, *scale.args(), _stream())
        return out
    if x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and interleave == 8 and x.is_cuda:
        M, K = x.shape
        N = w_gate_up.shape[0]
        if stream_supports(M, N, K):
            return linear_stream(x, w_gate_up, None, out_dtype, silu=True)
        if PAIR_SILU_FROM_ROWS <= M <= TCGEN05_MIN_ROWS and N % 16 == 0 and _PAIR_GEMM != "off" and pair_supports(M, N, K):
            # 64..128 tokens: still bound by reading W once, and the pair kernel's narrow tiles (two accumulators, the
            # epilogue under the next tile) stream it faster than `linear_tc`, whose accumulator is 128 columns wide there
            # (in a graph, 7B sizes, us: 64 tokens 51.0 against 53.4, 96 tokens 51.8 / 57.9, 128 tokens 53.1 / 61.9)
            return gemm_pair(x, w_gate_up, None, out_dtype, silu=True, wide=False)
        if N % 16 == 0 and linear_tc_supports(M, N, K):
            return linear_tc(x, w_gate_up, None, out_dtype, silu=True)
        if M > TCGEN05_MIN_ROWS and N % 16 == 0 and _PAIR_GEMM != "off" and pair_supports(M, N, K):
            # many rows: pairs of CTAs on the tensor cores, the activation applied as the tile leaves tensor memory
            return gemm_pair(x, w_gate_up, None, out_dtype, silu=True)
        if M > TCGEN05_MIN_ROWS and N % 16 == 0 and tcgen05_supports(M, N, K):
            return gemm_tcgen05(x, w_gate_up, None, out_dtype, silu=True)
    gu = linear(x, w_gate_up, None, x.dtype)
    return silu_mul(gu, interleave, out_dtype)


_QKV_ROPE = os.environ.get("SLLM_QKV_ROPE_FUSED", "1") != "0"     # 0: the product, then the rotary kernel


def qkv_rope_supports(x, w, table, rotary_dim, nq, nkv, hd, k_cache) -> bool:
    """Whether `linear_rope_kv_write` takes the product: bfloat16, few tokens, the whole head rotated
    (or no rotation at all), a head size that is a multiple of 16."""
    if not (_QKV_ROPE and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16):
        return False
    rot = int(rotary_dim) if table is not None else 0
    M, K = x.shape
    return M <= WS_MAX_ROWS and _ws_tokens_ok(M, w.shape[0], K) and bool(lib().sllm_linear_ws_rope_supports(int(M), int(w.shape[0]), int(K), int(nq), int(nkv),
                                                                          int(hd), rot))


def linear_rope_kv_write(x, w, bias, positions, table, rotary_dim, nq, nkv, hd, slot_mapping, k_cache, v_cache,
                         scale: RowScale | None = None):
    """``x @ w.T`` for the fused q|k|v matrix with what follows it in an attention layer done in the
    product's epilogue: bias, rotary encoding of the query and key heads by the tokens' positions,
    the new keys and values written to ``slot_mapping`` of the paged caches (not written when it is
    None).  Returns the rotated queries ``[T, nq*hd]`` bfloat16.  Few tokens only (`qkv_rope_supports`).
    ``scale``: a norm still owed on ``x`` (`RowScale`)."""
    _chk(x, w, bias, positions, table, slot_mapping, k_cache, v_cache)
    M, K = x.shape
    N = w.shape[0]
    rot = int(rotary_dim) if table is not None else 0
    num_pages, nkv_c, page_size, hd_c = k_cache.shape
    if (nkv_c, hd_c) != (nkv, hd) or tuple(v_cache.shape) != tuple(k_cache.shape):
        raise KernelError("linear_rope_kv_write: the caches are [pages, kv heads, page size, head size]")
    if table is not None and (table.dtype != torch.float32 or tuple(table.shape[1:]) != (2, rot // 2)):
        raise KernelError("linear_rope_kv_write: rotary table must be float32 [positions, 2, rotary_dim/2]")
    q = torch.empty((M, nq * hd), dtype=torch.bfloat16, device=x.device)
    max_pos = table.shape[0] if table is not None else 0
    call("sllm_linear_ws_rope", _p(x), _p(w), _p(bias), M, N, K, _p(positions), _p(table), rot, max_pos, nq, nkv, hd,
         _p(slot_mapping), page_size, num_pages, _p(k_cache), _p(v_cache), _p(q),
         *(scale.args() if scale is not None else _NO_SCALE), _stream())
    return q


def rope_kv_write(qkv, bias, positions, table, rotary_dim, nq, nkv, hd, slot_mapping, k_cache, v_cache,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """Bias, rotary encoding and the cache write for the fused q|k|v rows.
    Returns the rotated queries ``[T, nq*hd]`` in ``out_dtype``; keys and values go
    to ``slot_mapping`` in ``k_cache``/``v_cache`` ``[pages, nkv, page_size, hd]``
    (not written when ``slot_mapping`` is None)."""
    _chk(qkv, bias, positions, table, slot_mapping, k_cache, v_cache)
    parts, part_stride = 1, 0
    if qkv.dim() == 3:                       # a stack of partial sums from a k-split product
        parts, part_stride = qkv.shape[0], qkv.shape[1] * qkv.shape[2]
    T = qkv.shape[-2]
    if qkv.shape[-1] != (nq + 2 * nkv) * hd:
        raise KernelError(f"rope_kv_write: qkv width {qkv.shape[1]} is not (nq+2nkv)*hd")
    if k_cache.dtype != out_dtype or v_cache.dtype != out_dtype:
        raise KernelError("rope_kv_write: the cache and the queries share one dtype")
    num_pages, nkv_c, page_size, hd_c = k_cache.shape
    if (nkv_c, hd_c) != (nkv, hd) or tuple(v_cache.shape) != tuple(k_cache.shape):
        raise KernelError(f"rope_kv_write: cache shape {tuple(k_cache.shape)} does not fit nkv={nkv} hd={hd}")
    max_pos = 0
    if rotary_dim:
        if table is None or table.dtype != torch.float32 or tuple(table.shape[1:]) != (2, rotary_dim // 2):
            raise KernelError("rope_kv_write: rotary table must be float32 [positions, 2, rotary_dim/2]")
        max_pos = table.shape[0]
    q = torch.empty((T, nq * hd), dtype=out_dtype, device=qkv.device)
    call("sllm_rope_kv_write", _p(qkv), _dt(qkv), parts, part_stride, _p(bias), _p(positions), _p(table), int(rotary_dim), max_pos,
         nq, nkv, hd, _p(slot_mapping), page_size, num_pages, _p(k_cache), _p(v_cache), _p(q), _dtc(out_dtype),
         T, _stream())
    return q


def attention_simt(q, k_cache, v_cache, block_tables, positions, seq_of_token, nq, nkv, hd, scale, window):
    """The CUDA-core attention kernel: any head size up to 256, float32 arithmetic."""
    _chk(q, k_cache, v_cache, block_tables, positions, seq_of_token)
    T = q.shape[0]
    if q.dtype != k_cache.dtype:
        raise KernelError("attention: queries and cache share one dtype")
    page_size = k_cache.shape[2]
    out = torch.empty_like(q)
    call("sllm_attention_simt", _p(q), _p(k_cache), _p(v_cache), _dt(q), _p(block_tables),
         block_tables.shape[1], _p(positions), _p(seq_of_token), T, nq, nkv, hd, page_size, float(scale),
         int(window or 0), _p(out), _stream())
    return out


_num_sms: dict = {}


def num_sms() -> int:
    """Streaming multiprocessors of the current device (the library asks the driver, once per device):
    what the dispatch sizes k-splits and context splits for."""
    dev = _current_device() if _current_device is not None else torch.cuda.current_device()
    n = _num_sms.get(dev)
    if n is None:
        n = _num_sms[dev] = max(1, int(lib().sllm_num_sms()))
    return n


def attention_tiles(q_lens, group_size: int, device, ctx_lens=None, large_rows: int = 128):
    """Tiles of (token, head-in-group) rows for the tensor-core attention kernels: requests
    whose rows fit one 16-row tile go to the decode form, the others are cut into tiles of
    `large_rows` rows (128, or 256 for the tcgen05 form with two row tiles a CTA) for the
    prefill form.  Returns ``(small, large)``, each ``None`` or
    ``(tile_seq, tile_row0, count)`` on the device."""
    small_s, large_s, large_r = [], [], []
    ctx_before = [(c - n) for c, n in zip(ctx_lens, q_lens)] if ctx_lens else [0] * len(q_lens)
    for s, n in enumerate(q_lens):
        rows = n * group_size
        if rows <= 16:
            small_s.append(s)
        else:
            for r0 in range(0, rows, large_rows):
                large_s.append(s)
                large_r.append(r0)

    # the tiles with the most keys to walk first: a long tile that starts last would run alone
    order = sorted(range(len(large_s)), key=lambda i: -(large_r[i] // max(group_size, 1) + ctx_before[large_s[i]]))
    large_s, large_r = [large_s[i] for i in order], [large_r[i] for i in order]

    def up(seqs, rows):
        if not seqs:
            return None
        t = torch.tensor([seqs, rows], dtype=torch.int32).to(device, non_blocking=True)
        return t[0], t[1], len(seqs)
    return up(small_s, [0] * len(small_s)), up(large_s, large_r)


SPLIT_OVERHEAD_TILES = 3      # what a CTA of the decode form costs before and after its keys, in 64-key tiles
MAX_SPLITS = 128              # the merge kernel keeps one weight a range in shared memory
SPLIT_MIN_KEYS = 128          # a range has at least two key tiles (one request at 1,024 keys: 11.0 us in 4 ranges, 8.6 in 8)
MMA_MAX_SPLITS = 32           # the mma.sync form's merge walks the ranges one after the other


@functools.lru_cache(maxsize=4096)
def choose_splits(num_small: int, nkv: int, max_ctx: int, ctas_per_sm: int = 2, max_splits: int = 0) -> int:
    """How many ways the decode form cuts the context: the cut whose CTAs finish first, counted in waves of
    ``ctas_per_sm`` CTAs an SM times the 64-key tiles a CTA walks (plus its fixed cost); never less than
    ``SPLIT_MIN_KEYS`` keys a range, at most ``MAX_SPLITS`` ranges (one request at 32,768 keys and 4 KV heads: 74 ranges of 7 tiles
    fill the GPU once, where 32 ranges of 16 tiles left more than half of it idle).  A cut one CTA larger than a wave costs a whole second wave, so the
    number of ranges is not simply "two CTAs an SM"."""
    ctas = max(num_small * nkv, 1)
    slots = max(1, ctas_per_sm * num_sms())
    best, best_cost = 1, None
    for s in range(1, max(1, min(max_ctx // SPLIT_MIN_KEYS, max_splits or MAX_SPLITS)) + 1):
        tiles = -(-(-(-max_ctx // s)) // 64)              # the kernel rounds a range up to whole tiles
        if -(-max_ctx // (tiles * 64)) != s:              # so some counts leave their last ranges empty
            continue
        # (the last term: every range of every tile leaves a partial result that the merge reads again)
        cost = -(-ctas * s // slots) * (tiles + SPLIT_OVERHEAD_TILES) + 0.5 * ctas * s / slots
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attention_mma(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles, decode: bool, num_splits: int,
                  nq, nkv, hd, scale, window, out=None):
    """The tensor-core attention kernel on one tile list (see `attention_tiles`); the merge of a split context
    touches the rows of that list's requests only."""
    _chk(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles[0], tiles[1])
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("attention_mma: bfloat16 only")
    T = q.shape[0]
    if out is None:
        out = torch.empty_like(q)
    part_o = part_lse = None
    if num_splits > 1:
        part_o = torch.empty((num_splits, T, nq, hd), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((num_splits, T, nq), dtype=torch.float32, device=q.device)
    call("sllm_attention_mma", _p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_o), _p(part_lse), _p(block_tables),
         block_tables.shape[1], _p(q_start), _p(ctx_len), _p(tiles[0]), _p(tiles[1]), tiles[2], 1 if decode else 0,
         num_splits, T, nq, nkv, hd, k_cache.shape[2], float(scale), int(window or 0), _stream())
    if num_splits > 1:
        launches["own"] += 1          # the combine kernel
    return out


@functools.lru_cache(maxsize=4096)
def tma_attention_supports(hd: int, page_size: int) -> bool:
    return bool(lib().sllm_attention_tma_supports(int(hd), int(page_size)))


@functools.lru_cache(maxsize=16)
def _tma_ctas_per_sm(hd: int) -> int:
    return int(lib().sllm_attention_tma_ctas_per_sm(int(hd)))


def attention_tma_decode(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles, num_splits: int,
                         nq, nkv, hd, scale, window, out=None):
    """The decode form fed by TMA (16-row tiles only; see `attention_tiles`)."""
    _chk(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles[0], tiles[1])
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("attention_tma: bfloat16 only")
    T = q.shape[0]
    if out is None:
        out = torch.empty_like(q)
    part_o = part_lse = None
    if num_splits > 1:
        part_o = torch.empty((num_splits, T, nq, hd), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((num_splits, T, nq), dtype=torch.float32, device=q.device)
    call("sllm_attention_tma_decode", _p(q), _p(k_cache), _p(v_cache), k_cache.shape[0], _p(out), _p(part_o),
         _p(part_lse), _p(block_tables), block_tables.shape[1], _p(q_start), _p(ctx_len), _p(tiles[0]), _p(tiles[1]),
         tiles[2], num_splits, T, nq, nkv, hd, k_cache.shape[2], float(scale), int(window or 0),
         _p(_status_word(q.device)), _stream())
    _tc_used["since_check"] += 1
    if num_splits > 1:
        launches["own"] += 1
    return out


_TC_ATTENTION = os.environ.get("SLLM_ATTENTION_TCGEN05", "1") != "0"     # 0: prompt portions on the mma.sync form


def wait_probe(limit_ns: int, device="cuda"):
    """Run the kernel that waits on a barrier nothing arrives at (see csrc/wait_probe.cu); returns
    ``(status, waited_ns)``: 99 and about ``limit_ns`` when the bounded wait gave up as it must."""
    status = torch.zeros(1, dtype=torch.int32, device=device)
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    call("sllm_wait_probe", _p(status), int(limit_ns), _p(waited), _stream())
    return int(status.item()), int(waited.item())


@functools.lru_cache(maxsize=4096)
def tc_attention_supports(hd: int, page_size: int) -> bool:
    return bool(lib().sllm_attention_tc_supports(int(hd), int(page_size)))


@functools.lru_cache(maxsize=4096)
def choose_tc_splits(num_tiles: int, nkv: int, max_ctx: int) -> tuple[int, int]:
    """(ranges, 64-key tiles a range) for the prefill form: few row tiles over a long context are cut
    so that about two CTAs an SM run, each range at least 16 key tiles long."""
    key_tiles = max(1, -(-max_ctx // 64))
    ctas = max(num_tiles * nkv, 1)
    want = max(1, min(2 * num_sms() // ctas, key_tiles // 16, 32))
    per = -(-key_tiles // want)
    return -(-key_tiles // per), per


def attention_tc(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles, nq, nkv, hd, scale, out=None,
                 row_tiles: int = 1, splits: tuple[int, int] = (1, 0)):
    """The prefill form on tcgen05 (tiles of 128 * row_tiles rows, row_tiles 1 or 2; no window; see
    `attention_tiles`).  ``splits`` = (ranges, 64-key tiles a range) cuts the context into ranges
    that run as CTAs of their own and are merged afterwards; ranges x tiles must cover the longest
    context among the tiles' requests."""
    _chk(q, k_cache, v_cache, block_tables, q_start, ctx_len, tiles[0], tiles[1])
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: bfloat16 only")
    if out is None:
        out = torch.empty_like(q)
    n_splits, per = int(splits[0]), int(splits[1])
    part_o = part_lse = None
    T = q.shape[0]
    if n_splits > 1:
        part_o = torch.empty((n_splits, T, nq, hd), dtype=torch.float32, device=q.device)
        part_lse = torch.full((n_splits, T, nq), float("-inf"), dtype=torch.float32, device=q.device)
        launches["library"] += 1           # the fill
    call("sllm_attention_tc", _p(q), _p(k_cache), _p(v_cache), k_cache.shape[0], _p(out), _p(block_tables),
         block_tables.shape[1], _p(q_start), _p(ctx_len), _p(tiles[0]), _p(tiles[1]), tiles[2], int(row_tiles), nq, nkv,
         hd, k_cache.shape[2], float(scale), n_splits, max(per, 1), T, _p(part_o), _p(part_lse),
         _p(_status_word(q.device)), _stream())
    if n_splits > 1:
        launches["own"] += 1               # the merge kernel
    _tc_used["since_check"] += 1
    return out


@functools.lru_cache(maxsize=4096)
def mma_supports(hd: int) -> bool:
    return bool(lib().sllm_attention_mma_supports(int(hd)))


def paged_attention(q, k_cache, v_cache, step, group: int, nq, nkv, hd, scale, window):
    """Causal attention of the step's tokens over their requests' pages.  bfloat16 with a head size
    the tensor-core kernels take: requests of at most 16 (token, head-in-group) rows go to the decode
    form (fed by TMA where the head and page sizes allow, split over the context), the others to the
    prefill form in 128-row tiles (on tcgen05 where there is no window and the sizes allow, else on
    mma.sync).  Otherwise the CUDA-core kernel."""
    g = step.groups[group]
    if q.dtype != torch.bfloat16 or not mma_supports(hd):
        return attention_simt(q, k_cache, v_cache, g.block_tables, step.positions, step.seq_of_token,
                              nq, nkv, hd, scale, window)
    G = nq // nkv
    use_tc = not window and _TC_ATTENTION and tc_attention_supports(hd, k_cache.shape[2])
    key = ("mma", G, nkv, use_tc)
    if key not in step.attn_tiles:
        # 128-row CTAs, two per SM.  (The kernel also has a form with two row tiles a CTA, one CTA per SM,
        # that fetches each key/value tile once for 256 rows; measured at 28/4 heads of 128 it is the
        # slower one at every length: 106 against 99 us for 2048 tokens, 787 against 733 us for 8192.)
        rows = 128
        small, large = attention_tiles(step.q_lens, G, q.device, step.ctx_lens, rows)
        tma = tma_attention_supports(hd, k_cache.shape[2])
        per_sm = _tma_ctas_per_sm(hd) if tma else 2
        # the decode form's cut of the context, by the longest context among ITS requests (a step may also hold prompt
        # portions: their rows are the prefill form's, and the decode form's merge touches its own requests' rows only)
        splits = 1
        if small:
            small_ctx = max((c for c, n in zip(step.ctx_lens, step.q_lens) if n * G <= 16), default=step.max_ctx_len) \
                if step.ctx_lens else step.max_ctx_len
            splits = choose_splits(small[2], nkv, small_ctx, per_sm, 0 if tma else MMA_MAX_SPLITS)
        tc_splits = choose_tc_splits(large[2], nkv, step.max_ctx_len) if (large and use_tc) else (1, 0)
        step.attn_tiles[key] = (small, large, splits, rows, tc_splits)
    small, large, splits, rows, tc_splits = step.attn_tiles[key]
    out = torch.empty_like(q)
    if small and tma_attention_supports(hd, k_cache.shape[2]):
        attention_tma_decode(q, k_cache, v_cache, g.block_tables, step.q_start, step.ctx_len, small, splits,
                             nq, nkv, hd, scale, window, out)
    elif small:
        attention_mma(q, k_cache, v_cache, g.block_tables, step.q_start, step.ctx_len, small, True, splits,
                      nq, nkv, hd, scale, window, out)
    if large and use_tc:
        attention_tc(q, k_cache, v_cache, g.block_tables, step.q_start, step.ctx_len, large, nq, nkv, hd, scale, out,
                     row_tiles=rows // 128, splits=tc_splits)
    elif large:
        attention_mma(q, k_cache, v_cache, g.block_tables, step.q_start, step.ctx_len, large, False, 1,
                      nq, nkv, hd, scale, window, out)
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """``x[rows]``; a 3-d ``x`` is a stack of partial sums, added while gathering."""
    _chk(x, rows)
    parts, stride = 1, 0
    if x.dim() == 3:
        parts, stride = x.shape[0], x.shape[1] * x.shape[2]
    R, (n, H) = rows.numel(), x.shape[-2:]
    out = torch.empty((R, H), dtype=x.dtype, device=x.device)
    call("sllm_gather_rows", _p(x), _dt(x), parts, stride, _p(rows), _p(out), R, H, n, _stream())
    return out


def sample_rows(logits: torch.Tensor, temperature=None, uniform=None, top_k=None, top_p=None) -> torch.Tensor:
    """int32 token per row of float32 ``logits [R, V]``: the first maximum where the
    row's temperature is <= 0 (or none is given), else inverse-CDF sampling of
    softmax(logits / temperature) at the row's uniform (float64), over the tokens that
    the row's ``top_k`` (int32, <= 0: no filter) and then ``top_p`` (float32, < 0: no
    filter) keep."""
    _chk(logits, temperature, uniform, top_k, top_p)
    R, V = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("sample_rows: logits are float32")
    if temperature is not None and (temperature.dtype != torch.float32 or uniform is None
                                    or uniform.dtype != torch.float64):
        raise KernelError("sample_rows: temperature float32 and uniform float64, one per row")
    if (top_k is not None or top_p is not None) and temperature is None:
        raise KernelError("sample_rows: top_k/top_p filter sampled rows; give temperatures")
    if (top_k is not None and (top_k.dtype != torch.int32 or top_k.numel() != R)) or \
            (top_p is not None and (top_p.dtype != torch.float32 or top_p.numel() != R)):
        raise KernelError("sample_rows: top_k int32 and top_p float32, one per row")
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    call("sllm_sample_rows", _p(logits), R, V, _p(temperature), _p(uniform), _p(top_k), _p(top_p), _p(out), _stream())
    return out


def repetition_penalty_(logits: torch.Tensor, pair_row, pair_id, pair_penalty) -> torch.Tensor:
    """In place on float32 ``logits [R, V]``: for each (row, id, penalty) triple a positive
    logit is divided by the penalty and a negative one multiplied.  A (row, id) pair must
    appear once; ids outside the vocabulary are ignored."""
    _chk(logits, pair_row, pair_id, pair_penalty)
    R, V = logits.shape
    n = pair_row.numel()
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("repetition_penalty_: logits are contiguous float32")
    if pair_row.dtype != torch.int32 or pair_id.dtype != torch.int32 or pair_penalty.dtype != torch.float32 \
            or pair_id.numel() != n or pair_penalty.numel() != n:
        raise KernelError("repetition_penalty_: rows and ids int32, penalties float32, one per pair")
    call("sllm_repetition_penalty", _p(logits), R, V, _p(pair_row), _p(pair_id), _p(pair_penalty), n, _stream())
    return logits


def mark_seen(seen: torch.Tensor, step) -> None:
    """Record the step's tokens in ``seen [slots, V]`` (uint8): ``seen[slot of the token's request,
    token id] = 1``.  ``step`` is the `StepContext` (token ids, request of each token, state slots,
    all on the device)."""
    _chk(seen, step.token_ids, step.seq_of_token, step.state_slots)
    if seen.dtype != torch.uint8 or seen.dim() != 2:
        raise KernelError("mark_seen: the table is uint8 [slots, V]")
    call("sllm_mark_seen", _p(seen), seen.shape[0], seen.shape[1], _p(step.token_ids), _p(step.seq_of_token),
         _p(step.state_slots), int(step.num_tokens), _stream())


def penalty_from_seen_(logits: torch.Tensor, seen: torch.Tensor, step, penalty: torch.Tensor) -> torch.Tensor:
    """The repetition penalty in place on float32 ``logits [R, V]`` (row r belongs to the request of
    token ``step.logit_rows[r]``): every id that request has seen has a positive logit divided by
    ``penalty[r]`` and a negative one multiplied; rows with penalty 0 or 1 stay as they are."""
    _chk(logits, seen, penalty, step.logit_rows, step.seq_of_token, step.state_slots)
    R, V = logits.shape
    if logits.dtype != torch.float32 or seen.dtype != torch.uint8 or seen.shape[1] != V:
        raise KernelError("penalty_from_seen_: float32 logits [R, V] and a uint8 table [slots, V]")
    if penalty.dtype != torch.float32 or penalty.numel() != R or step.logit_rows.numel() < R:
        raise KernelError("penalty_from_seen_: one float32 penalty and one wanted row per logits row")
    call("sllm_penalty_seen", _p(logits), R, V, _p(seen), seen.shape[0], _p(step.logit_rows), _p(step.seq_of_token),
         _p(step.state_slots), _p(penalty), _stream())
    return logits
