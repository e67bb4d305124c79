"""The entry point that allocates nothing, called through its exported C symbol.

`sllm_linear_stream_noalloc` is for callers that must not allocate device memory when they
need a product (a frozen or measured memory pool, a loop that may not take the driver's
allocation lock, a host that owns all device memory): the k-split partial sums live in an
array inside the library instead of caller-supplied scratch.  Here it is called twice in a
row through ctypes, with different inputs, and compared with the ordinary entry point
(`sllm_linear_stream`, unsplit, writing straight to its output) within the tolerance of the
kernel tests.  The file's name makes pytest collect it last.
"""

import ctypes

import pytest
import torch

from tests.conftest import cuda_or_skip

pytestmark = pytest.mark.gpu


def _lib():
    from sllm_b200.ops._lib import lib
    L = lib()
    c_int, c_void_p = ctypes.c_int, ctypes.c_void_p
    fn = L.sllm_linear_stream_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    return L, fn


def test_no_alloc_entry_point_twice_in_a_row():
    cuda_or_skip()
    L, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(21)
    M, N, K, splits = 8, 4608, 3584, 7
    outs, wants = [], []
    # everything the calls need exists before the first of them
    cases = []
    for _ in range(2):
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
        b = torch.randn(N, device="cuda", generator=g)
        cases.append((x, w, b, torch.full((M, N), float("nan"), device="cuda"), torch.empty(M, N, device="cuda")))
    # a first call ahead of the measurement: it looks the array's address up and lets the driver load the
    # kernels' code, neither of which a later call repeats
    x, w, b, out, _ = cases[0]
    assert fn(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, splits, stream) == 0, L.sllm_last_error().decode()
    out.fill_(float("nan"))
    torch.cuda.synchronize()
    # two counters: torch's own allocator, and the driver's free memory (which a cudaMalloc inside the
    # entry point would lower without torch knowing of it)
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    for x, w, b, out, want in cases:
        rc = fn(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, splits, stream)
        assert rc == 0, L.sllm_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] >= free_before, "the driver's free memory shrank during the calls"
    for x, w, b, out, want in cases:
        # the ordinary entry point, unsplit: float32 result, no scratch
        rc = L.sllm_linear_stream(x.data_ptr(), w.data_ptr(), b.data_ptr(), want.data_ptr(), 0, None, M, N, K, 1, 0, stream)
        assert rc == 0, L.sllm_last_error().decode()
    torch.cuda.synchronize()
    for x, w, b, out, want in cases:
        assert not out.isnan().any()
        torch.testing.assert_close(out, want, rtol=2e-3, atol=2e-3)
        torch.testing.assert_close(out, x.float() @ w.float().t() + b, rtol=2e-3, atol=2e-3)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    cuda_or_skip()
    L, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    M, N, K = 64, 152064, 256            # 2 splits x 64 x 152064 floats: far beyond the built-in scratch
    x = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(M, N, device="cuda")
    assert fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, K, 2, stream) != 0
    assert b"scratch holds" in L.sllm_last_error()
    assert fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, 200, 2, stream) != 0      # K not a multiple of 128
