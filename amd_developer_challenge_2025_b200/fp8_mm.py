"""Host side of the operator: argument checks, workspace cache, the C-ABI call.

Mirrors the reference's pybind launcher `fp8_mm(a, b, as, bs, c, c_tmp)`
(1-amd-fp8-mm/amd-fp8-mm-submission.py:514-579) with the checks it lacks."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

SCALE_BLOCK = 128


@dataclass(frozen=True)
class Plan:
    block_m: int = 0
    block_n: int = 0
    cta_pair: int = 0
    split_k: int = 0
    stages: int = 0
    grid: int = 0
    tiles: int = 0
    smem_bytes: int = 0
    store_bufs: int = 0
    full_tiles: int = 0

    def to_c(self) -> _lib.CPlan:
        return _lib.CPlan(self.block_m, self.block_n, self.cta_pair, self.split_k, self.stages, self.grid,
                          self.tiles, self.smem_bytes, self.store_bufs, self.full_tiles)

    @staticmethod
    def from_c(c: _lib.CPlan) -> "Plan":
        return Plan(c.block_m, c.block_n, c.cta_pair, c.split_k, c.stages, c.grid, c.tiles, c.smem_bytes,
                    c.store_bufs, c.full_tiles)


class Fp8MmError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        super().__init__(f"b200_fp8_mm error {code}: {_lib.strerror(code)}{(' (' + what + ')') if what else ''}")


class Fp8MmDeviceError(RuntimeError):
    """A bounded wait inside the kernel expired; the output is not valid."""


def describe(m: int, n: int, k: int, n_phase: int = 0, sm_count: int = 0) -> Plan:
    """The tile/launch plan the library picks for this problem (host arithmetic only)."""
    out = _lib.CPlan()
    rc = _lib.load().b200_fp8_mm_describe(m, n, k, n_phase, sm_count, ctypes.byref(out))
    if rc != 0:
        raise Fp8MmError(rc)
    return Plan.from_c(out)


def estimate_clocks(m: int, n: int, k: int, sm_count: int = 0) -> float:
    """The selector's cost estimate (SM clocks) for the plan it would pick; host arithmetic only."""
    v = float(_lib.load().b200_fp8_mm_estimate_clocks(m, n, k, sm_count))
    if v < 0:
        raise Fp8MmError(2)
    return v


def workspace_bytes(m: int, n: int, k: int, plan: Plan | None = None) -> int:
    lib = _lib.load()
    if plan is None:
        return int(lib.b200_fp8_mm_workspace_bytes(m, n, k))
    cp = plan.to_c()
    return int(lib.b200_fp8_mm_plan_workspace_bytes(m, n, k, ctypes.byref(cp)))


# Scratch owned by the Python side (the library allocates nothing). The reference allocates its split-K
# scratch on every call (1-amd-fp8-mm/amd-fp8-mm-submission.py:600); here it is cached, one buffer per
# (device, stream): split-K launches count arrivals in the buffer's first 4096 bytes and park fp32 partials
# behind them, so two launches that may overlap on the GPU (different streams) must not share one. Launches
# on one stream run in order and can. A buffer that has to grow is replaced, and the old one is kept alive
# for the life of the process: a launch queued earlier may still be using it, and handing its memory back
# to the caching allocator would let another stream's allocation overwrite it.
_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_retired_workspaces: list[torch.Tensor] = []
_status: dict[int, torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int, stream: int) -> torch.Tensor | None:
    if nbytes == 0:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
        # zeroed on the stream that will use it (the current one): the counters must start at zero
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _status_words(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _status.get(idx)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=device)
        _status[idx] = st
    return st


def _check(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


# Argument signatures that already passed validation -> (workspace bytes, C plan or None). A repeat
# call with the same shapes, strides, dtypes and device skips the checks: the operator is called in
# tight loops and the kernel for a small problem runs for only a few microseconds.
_validated: dict[tuple, tuple] = {}


def _validate(a, b, a_scale, b_scale, c, n_phase, plan):
    _check(a.is_cuda and b.is_cuda and a_scale.is_cuda and b_scale.is_cuda and c.is_cuda,
           "all five tensors must be CUDA tensors (there is no CPU path)")
    _check(a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn, "a and b must be float8_e4m3fn")
    _check(a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32, "scales must be float32")
    _check(c.dtype == torch.bfloat16, "c must be bfloat16")
    _check(a.dim() == 2 and b.dim() == 2 and c.dim() == 2, "a, b, c must be 2-D")
    m, k = a.shape
    n = b.shape[0]
    _check(b.shape[1] == k, "a and b disagree on K")
    _check(tuple(c.shape) == (m, n), "c must be [M, N]")
    _check(k % SCALE_BLOCK == 0, "K must be a multiple of 128")
    kb = k // SCALE_BLOCK
    nb = (n + n_phase + SCALE_BLOCK - 1) // SCALE_BLOCK
    _check(tuple(a_scale.shape) == (m, kb), f"a_scale must be [{m}, {kb}]")
    _check(tuple(b_scale.shape) == (nb, kb), f"b_scale must be [{nb}, {kb}]")
    mn_major = False
    for name, t, rows in (("a", a, m), ("b", b, n)):
        k_major = t.stride(1) == 1 and t.stride(0) >= k
        mn = t.stride(0) == 1 and t.stride(1) >= rows
        _check(k_major or mn, f"{name} must have either K contiguous or its {'M' if name == 'a' else 'N'} "
                              "dimension contiguous")
        pitch = t.stride(0) if k_major else t.stride(1)
        _check(pitch % 16 == 0 and t.data_ptr() % 16 == 0, f"{name}: pitch and base address must be multiples of 16")
        mn_major = mn_major or not k_major
    _check(c.stride(1) == 1, "c must have N contiguous")
    dev = a.device
    _check(all(t.device == dev for t in (b, a_scale, b_scale, c)), "tensors on different devices")
    return workspace_bytes(m, n, k, plan), (plan.to_c() if plan is not None else None)


def fp8_mm(a, b, a_scale, b_scale, c, n_phase: int = 0, plan: Plan | None = None, check: bool = False):
    """c[M,N] (bf16) = block-scaled a[M,K] @ b[N,K]^T on the current CUDA stream; returns c.

    a [M,K], b [N,K]: float8_e4m3fn, each either with K contiguous or with its M / N dimension
    contiguous (the `[K][M]` storage the reference's harness hands over, e.g. `x.t().contiguous().t()`);
    the other stride a multiple of 16. a_scale: fp32 [M, K/128], any strides.
    b_scale: fp32 [ceil((N+n_phase)/128), K/128], any strides. `n_phase`: offset of b's first
    row inside its 128-row scale block (0 unless b is a column shard of a larger matrix).
    `plan`: force tile parameters (sweeps/tests). `check`: synchronise and raise if a wait
    inside the kernel expired. Asynchronous otherwise, like the reference's launcher."""
    lib = _lib.load()
    sa, sb, sas, sbs, sc = a.stride(), b.stride(), a_scale.stride(), b_scale.stride(), c.stride()
    key = (a.shape, b.shape, a_scale.shape, b_scale.shape, c.shape, sa, sb, sas, sbs, sc,
           a.dtype, b.dtype, a_scale.dtype, b_scale.dtype, c.dtype,
           a.device, b.device, a_scale.device, b_scale.device, c.device, n_phase, plan)
    cached = _validated.get(key)
    if cached is None:
        cached = _validate(a, b, a_scale, b_scale, c, n_phase, plan)
        if len(_validated) > 4096:
            _validated.clear()
        _validated[key] = cached
    nbytes, cplan = cached
    m, k = a.shape
    n = b.shape[0]
    dev = a.device
    if dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            return fp8_mm(a, b, a_scale, b_scale, c, n_phase, plan, check)
    stream = torch.cuda.current_stream(dev).cuda_stream
    ws = _workspace(dev, nbytes, stream)
    st = _status_words(dev)
    args = (
        a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(),
        m, n, k,
        sa[0], sa[1], sb[0], sb[1], sas[0], sas[1], sbs[0], sbs[1], sc[0], n_phase,
        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
        st.data_ptr(), stream,
    )
    rc = lib.b200_fp8_mm_strided(*args, ctypes.byref(cplan) if cplan is not None else None)
    if rc != 0:
        raise Fp8MmError(rc, f"M={m} N={n} K={k}")
    if check:
        check_device_status(dev)
    return c


def selftest_wait_expiry(device="cuda", limit_ms: float = 5.0):
    """Diagnostics: makes one wait inside the kernel run out on purpose, in the allowed way. A 128 x 64 x 256
    problem is launched with every wait limited to `limit_ms` and with the copy of its second K block left
    out; the kernel gives up that wait, returns by itself and reports it. Returns the four status words
    [code, role/barrier, block, phase]; code 1 is WAIT_EXPIRED. The status words are cleared again, so the
    next launch starts clean."""
    from .inputs import make_inputs

    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    lib = _lib.load()
    with torch.cuda.device(dev):
        a, b, a_s, b_s, c = make_inputs(128, 64, 256, seed=1, device=dev)
        st = _status_words(dev)
        torch.cuda.synchronize(dev)
        rc = lib.b200_fp8_mm_selftest_wait_expiry(
            a.data_ptr(), b.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), c.data_ptr(), 128, 64, 256,
            a.stride(0), b.stride(0), a_s.stride(0), a_s.stride(1), b_s.stride(0), b_s.stride(1), c.stride(0),
            int(limit_ms * 1e6), 1, st.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise Fp8MmError(rc, "selftest_wait_expiry")
        torch.cuda.synchronize(dev)
        words = st.tolist()
        st.zero_()
        torch.cuda.synchronize(dev)
    return words


def fp8_mm_grouped(a, b, a_scale, b_scale, c, m_valid=None, plan: Plan | None = None, check: bool = False):
    """c[g] (bf16 [G,M,N]) = block-scaled a[g] ([G,M,K]) @ b[g]^T ([G,N,K]) for every group g in one launch.

    The FP8 block-scaled form of the per-expert GEMMs the reference's MoE submission runs as fp16
    `torch.bmm` (2-amd-moe/amd-moe-submission.py:604-611). a_scale: fp32 [G, M, K/128]; b_scale: fp32
    [G, ceil(N/128), K/128]; any strides for the scales, K contiguous for a and b. `m_valid`: optional
    int32 CUDA tensor [G]; rows at or past m_valid[g] of group g are neither computed nor written."""
    lib = _lib.load()
    _check(all(t.is_cuda for t in (a, b, a_scale, b_scale, c)), "all tensors must be CUDA tensors (there is no CPU path)")
    _check(a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn, "a and b must be float8_e4m3fn")
    _check(a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32, "scales must be float32")
    _check(c.dtype == torch.bfloat16, "c must be bfloat16")
    _check(a.dim() == 3 and b.dim() == 3 and c.dim() == 3, "a, b, c must be 3-D: [groups, rows, cols]")
    g, m, k = a.shape
    n = b.shape[1]
    _check(b.shape[0] == g and b.shape[2] == k, "a and b disagree on groups or K")
    _check(tuple(c.shape) == (g, m, n), "c must be [G, M, N]")
    _check(k % SCALE_BLOCK == 0, "K must be a multiple of 128")
    kb, nb = k // SCALE_BLOCK, (n + SCALE_BLOCK - 1) // SCALE_BLOCK
    _check(tuple(a_scale.shape) == (g, m, kb), f"a_scale must be [{g}, {m}, {kb}]")
    _check(tuple(b_scale.shape) == (g, nb, kb), f"b_scale must be [{g}, {nb}, {kb}]")
    _check(a.stride(2) == 1 and b.stride(2) == 1 and c.stride(2) == 1, "a, b need K contiguous, c needs N contiguous")
    for name, t in (("a", a), ("b", b)):
        _check(t.stride(1) % 16 == 0 and t.stride(0) % 16 == 0 and t.data_ptr() % 16 == 0,
               f"{name}: row pitch, group pitch and base address must be multiples of 16")
    dev = a.device
    _check(all(t.device == dev for t in (b, a_scale, b_scale, c)), "tensors on different devices")
    if m_valid is not None:
        _check(m_valid.is_cuda and m_valid.device == dev and m_valid.dtype == torch.int32
               and tuple(m_valid.shape) == (g,) and m_valid.is_contiguous(), "m_valid must be a contiguous int32 CUDA tensor [G]")
    if plan is not None:
        _check(plan.split_k <= 1, "grouped launches use whole tiles (no split-K)")
    if dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            return fp8_mm_grouped(a, b, a_scale, b_scale, c, m_valid, plan, check)
    st = _status_words(dev)
    cplan = plan.to_c() if plan is not None else None
    rc = lib.b200_fp8_mm_grouped(
        a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(), g, m, n, k,
        a.stride(1), a.stride(0), b.stride(1), b.stride(0),
        a_scale.stride(0), a_scale.stride(1), a_scale.stride(2),
        b_scale.stride(0), b_scale.stride(1), b_scale.stride(2),
        c.stride(1), c.stride(0),
        m_valid.data_ptr() if m_valid is not None else None,
        st.data_ptr(), torch.cuda.current_stream(dev).cuda_stream,
        ctypes.byref(cplan) if cplan is not None else None)
    if rc != 0:
        raise Fp8MmError(rc, f"G={g} M={m} N={n} K={k}")
    if check:
        check_device_status(dev)
    return c


def check_device_status(device=None):
    """Synchronises and raises Fp8MmDeviceError if any launch since the last check gave up a wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(dev)
    st = _status_words(dev)
    words = st.tolist()
    if words[0] != 0:
        st.zero_()
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        for (d, _stream), ws in _workspaces.items():
            if d == idx:
                ws[:4096].zero_()  # split-K counters may be mid-count after an aborted launch
        raise Fp8MmDeviceError(
            f"kernel wait expired: code={words[0]} where=0x{words[1]:x} block={words[2]} parity={words[3]}")


class _HostPipeline:
    """Per-device state of `fp8_mm_host`: three streams (copies in, GEMMs, copies out) and the device
    buffers of the last problem shape, kept between calls so that a call allocates nothing."""

    def __init__(self, dev: torch.device):
        self.dev = dev
        self.s_in = torch.cuda.Stream(dev)
        self.s_mm = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.key = None
        self.bufs = None

    def buffers(self, m, n, k, nb):
        key = (m, n, k, nb)
        if self.key != key:
            dev = self.dev
            self.bufs = (
                torch.empty(m, k, dtype=torch.float8_e4m3fn, device=dev),
                torch.empty(n, k, dtype=torch.float8_e4m3fn, device=dev),
                torch.empty(m, k // SCALE_BLOCK, dtype=torch.float32, device=dev),
                torch.empty(nb, k // SCALE_BLOCK, dtype=torch.float32, device=dev),
                torch.empty(m, n, dtype=torch.bfloat16, device=dev),
            )
            self.key = key
        return self.bufs


_host_pipelines: dict[int, _HostPipeline] = {}


def host_row_chunks(m: int, chunk_rows: int = 1024) -> list[tuple[int, int]]:
    """Row ranges [r0, r1) the host entry point cuts a problem into: a short first range, so that the
    first copy of c back to the host can start as early as possible, then `chunk_rows` rows each
    (multiples of 128, the kernel's row block), and a short last range, because the last range's GEMM and
    its copy back to the host are the part of the call that nothing else overlaps."""
    if m <= 512:
        return [(0, m)]
    out = [(0, 256)]
    r = 256
    while r < m:
        out.append((r, min(m, r + chunk_rows)))
        r += chunk_rows
    r0, r1 = out[-1]
    if r1 - r0 > 256:
        out[-1] = (r0, r1 - 256)
        out.append((r1 - 256, r1))
    return out


def fp8_mm_host(a, b, a_scale, b_scale, c, device="cuda", n_phase: int = 0, chunk_rows: int = 1024):
    """The same operator for HOST tensors (pinned memory for full speed): returns c, filled, when done.

    b, b_scale and a_scale are copied to `device` first; a is then streamed in row ranges, each range's
    GEMM runs as soon as its rows have landed, and its rows of c are copied back while later ranges are
    still arriving, so both directions of the host link and the SMs work at the same time (three
    streams, events between them). Every range is an independent GEMM over whole rows with the plan the
    library picks for its size; the result meets the same tolerance as one GEMM over the whole problem
    (and equals it bit for bit unless a range's plan splits K, which only changes the order in which K
    ranges are added). Device buffers are kept per device between calls of the same shape. This is the
    call the end-to-end benchmark times."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    for name, t in (("a", a), ("b", b), ("a_scale", a_scale), ("b_scale", b_scale), ("c", c)):
        _check(not t.is_cuda, f"{name} must be a host tensor")
    _check(a.is_contiguous() and b.is_contiguous() and a_scale.is_contiguous() and b_scale.is_contiguous()
           and c.is_contiguous(), "host tensors must be contiguous")
    m, k = a.shape
    n = b.shape[0]
    pipe = _host_pipelines.get(dev.index)
    if pipe is None:
        pipe = _host_pipelines[dev.index] = _HostPipeline(dev)
    da, db, das, dbs, dc = pipe.buffers(m, n, k, b_scale.shape[0])
    caller = torch.cuda.current_stream(dev)
    pipe.s_in.wait_stream(caller)
    pipe.s_mm.wait_stream(caller)
    pipe.s_out.wait_stream(caller)
    with torch.cuda.device(dev):
        with torch.cuda.stream(pipe.s_in):
            db.copy_(b, non_blocking=True)
            dbs.copy_(b_scale, non_blocking=True)
            das.copy_(a_scale, non_blocking=True)
        for (r0, r1) in host_row_chunks(m, chunk_rows):
            with torch.cuda.stream(pipe.s_in):
                da[r0:r1].copy_(a[r0:r1], non_blocking=True)
            pipe.s_mm.wait_stream(pipe.s_in)
            with torch.cuda.stream(pipe.s_mm):
                fp8_mm(da[r0:r1], db, das[r0:r1], dbs, dc[r0:r1], n_phase=n_phase)
            pipe.s_out.wait_stream(pipe.s_mm)
            with torch.cuda.stream(pipe.s_out):
                c[r0:r1].copy_(dc[r0:r1], non_blocking=True)
    pipe.s_out.synchronize()
    caller.wait_stream(pipe.s_out)
    return c
