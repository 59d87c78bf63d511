"""GPU test of b200_fp8_mm_static_scratch, the entry point for callers that cannot allocate.

Some users of this library are handed input and output pointers and nothing else: an engine
plug-in inside its enqueue hook, a serving loop that may not pay for the allocator's implicit
device synchronisation, a process that froze its memory pools after start-up. Split-K plans need
scratch memory, and the ordinary entry point makes the caller supply it; this one uses a fixed
8 MiB array that is part of the library's device image instead.

The file is named so that pytest collects it last: should it fail, a run that stops at the first
failure has already run everything else. It must also pass on its own in a fresh process (then
its first call is the one that looks up the array's device address).

Checked here, through the C ABI (ctypes, raw pointers): on two calls in a row, with different
problems so that the second one meets the first one's leftovers in the shared array, the result
equals what the ordinary entry point produces with a caller-owned workspace - within the
tolerance every parity test in this repository uses (|c - ref| <= 1e-3 + 2e-2 |ref| on the bf16
output), and in fact bit for bit, since both run the same plan. A problem whose plan needs more
than the built-in array is refused with a distinct error code and launches nothing."""
import ctypes

import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from amd_developer_challenge_2025_b200 import _lib
from amd_developer_challenge_2025_b200.fp8_mm import check_device_status
from oracle import fp8_mm_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-3
ERR_SCRATCH_LIMIT = 10


def call_static_scratch(a, b, a_s, b_s, c, n_phase=0):
    """The raw C-ABI call: pointers, sizes, strides, status words, stream. No workspace."""
    lib = _lib.load()
    status = torch.zeros(4, dtype=torch.int32, device=c.device)
    m, k = a.shape
    n = b.shape[0]
    rc = lib.b200_fp8_mm_static_scratch(
        a.data_ptr(), b.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), c.data_ptr(), m, n, k,
        a.stride(0), b.stride(0), a_s.stride(0), a_s.stride(1), b_s.stride(0), b_s.stride(1), c.stride(0), n_phase,
        status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, status.tolist()


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    limit = _lib.load().b200_fp8_mm_static_scratch_limit()
    assert limit == 8 << 20
    # both problems get split-K plans, i.e. they really use scratch, and both fit the built-in array
    problems = [(256, 1536, 7168, 41), (512, 512, 7168, 42)]
    for (m, n, k, seed) in problems:
        plan = pkg.describe(m, n, k)
        assert plan.split_k > 1 and 0 < pkg.workspace_bytes(m, n, k) <= limit
    for (m, n, k, seed) in problems:
        a, b, a_s, b_s, _ = pkg.make_inputs(m, n, k, seed, device="cuda")
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        pkg.fp8_mm(a, b, a_s, b_s, want)           # existing entry point, workspace owned by the caller
        check_device_status()
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc, status = call_static_scratch(a, b, a_s, b_s, got)
        assert rc == 0, _lib.strerror(rc)
        assert status[0] == 0, status
        ok, excess, max_err = oracle.check(got, want.cpu(), RTOL, ATOL)
        assert ok, (excess, max_err)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))   # same plan, same bits
        ok, excess, max_err = oracle.check(got, oracle.dequant_matmul(a, b, a_s, b_s), RTOL, ATOL)
        assert ok, (excess, max_err)


def test_plans_without_a_split_need_no_scratch_and_also_work():
    m, n, k = 300, 640, 512
    assert pkg.describe(m, n, k).split_k == 1
    a, b, a_s, b_s, _ = pkg.make_inputs(m, n, k, 43, device="cuda")
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc, status = call_static_scratch(a, b, a_s, b_s, got)
    assert rc == 0 and status[0] == 0
    ok, excess, max_err = oracle.check(got, oracle.dequant_matmul(a, b, a_s, b_s), RTOL, ATOL)
    assert ok, (excess, max_err)


def test_a_plan_beyond_the_built_in_scratch_is_refused():
    m, n, k = 896, 1216, 32768
    limit = _lib.load().b200_fp8_mm_static_scratch_limit()
    assert pkg.workspace_bytes(m, n, k) > limit
    # refused before any pointer is looked at: small stand-in tensors are enough
    t8 = torch.zeros(16, dtype=torch.uint8, device="cuda")
    f32 = torch.zeros(16, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = _lib.load().b200_fp8_mm_static_scratch(
        t8.data_ptr(), t8.data_ptr(), f32.data_ptr(), f32.data_ptr(), t8.data_ptr(), m, n, k,
        k, k, k // 128, 1, k // 128, 1, n, 0, status.data_ptr(), ctypes.c_void_p(0))
    assert rc == ERR_SCRATCH_LIMIT
    assert "8 MiB" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]


def test_a_refused_call_puts_nothing_on_the_stream():
    """Argument checks come before the clearing of the shared array's counters: a call that is refused
    (here: an n_phase that is not a multiple of 32) must not enqueue anything. A stream capture serves
    as the recorder of what reaches the stream; the refused call must leave the captured graph empty."""
    from cuda.bindings import runtime as rt

    m, n, k = 256, 1536, 7168   # a split-K plan: an accepted call would clear counters first
    a, b, a_s, b_s, _ = pkg.make_inputs(m, n, k, 44, device="cuda")
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    rc, status = call_static_scratch(a, b, a_s, b_s, c)   # set-up call, outside the recording
    assert rc == 0 and status[0] == 0
    lib = _lib.load()
    status_t = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    (err,) = rt.cudaStreamBeginCapture(stream.cuda_stream, rt.cudaStreamCaptureMode.cudaStreamCaptureModeThreadLocal)
    assert err == rt.cudaError_t.cudaSuccess
    try:
        rc = lib.b200_fp8_mm_static_scratch(
            a.data_ptr(), b.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), c.data_ptr(), m, n, k,
            a.stride(0), b.stride(0), a_s.stride(0), a_s.stride(1), b_s.stride(0), b_s.stride(1), c.stride(0), 16,
            status_t.data_ptr(), stream.cuda_stream)
    finally:
        err, graph = rt.cudaStreamEndCapture(stream.cuda_stream)
    assert err == rt.cudaError_t.cudaSuccess
    assert rc == 5   # B200_FP8_MM_ERR_PHASE
    err, _nodes, count = rt.cudaGraphGetNodes(graph, 0)
    assert err == rt.cudaError_t.cudaSuccess and count == 0
    rt.cudaGraphDestroy(graph)
    torch.cuda.synchronize()
    assert status_t.tolist() == [0, 0, 0, 0]
