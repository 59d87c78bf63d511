"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerance is the contract's: |c - ref| <= 1e-3 + 2e-2 * |ref| on the bf16 output, inputs
e4m3fn on both sides. Small and medium shapes are compared with the CPU oracle directly;
the largest configurations are checked on sampled rows plus size-independent properties
(exact linearity in power-of-two scales, shard/whole agreement, run-to-run determinism)."""
import os

import numpy as np
import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from amd_developer_challenge_2025_b200.fp8_mm import Fp8MmError, Plan, check_device_status
from oracle import fp8_mm_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-3
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run(a, b, a_s, b_s, c, **kw):
    out = pkg.fp8_mm(a, b, a_s, b_s, c, **kw)
    check_device_status(c.device)
    return out


def assert_close(c, ref, what=""):
    ok, excess, max_err = oracle.check(c, ref, RTOL, ATOL)
    assert ok, f"{what}: worst excess over tolerance {excess}, max abs err {max_err}"


def cuda_inputs(m, n, k, seed):
    return pkg.make_inputs(m, n, k, seed, device="cuda")


# ------------------------------------------------------------------ golden fixtures


@pytest.mark.parametrize("name", ["one_block", "ragged_n", "n576_like", "shard_phase64", "odd_m"])
def test_golden_fixture(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    m, n, k, seed, phase = (int(v) for v in z["meta"])
    a = torch.from_numpy(z["a"]).view(torch.float8_e4m3fn).cuda()
    b = torch.from_numpy(z["b"]).view(torch.float8_e4m3fn).cuda()
    a_s = torch.from_numpy(z["a_scale"]).cuda()
    b_s = torch.from_numpy(z["b_scale"]).cuda()
    want = torch.from_numpy(z["c_bf16_bits"]).view(torch.bfloat16)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    run(a, b, a_s, b_s, c, n_phase=phase)
    assert_close(c, want, name)


# ------------------------------------------------------------------ the named configurations


@pytest.mark.parametrize("m,n,k,seed", [
    (256, 1536, 7168, 8135),   # the CPU-runnable configuration
    (2048, 576, 7168, 12346),  # skinny N, long K (5 scale rows for 4.5 blocks)
    (2048, 7168, 512, 17512),  # short K
    (2048, 7168, 256, 5364),   # two scale blocks only
])
def test_named_config_against_cpu_oracle(m, n, k, seed):
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, seed)
    c.fill_(float("nan"))
    out = pkg.custom_kernel((a, b, a_s, b_s, c))
    check_device_status()
    assert out is c
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), f"{m}x{n}x{k}")


def test_headline_config_rows_and_properties():
    """M=8192, N=4608, K=7168: sampled rows against the oracle, exact linearity, determinism."""
    m, n, k = 8192, 4608, 7168
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 65436)
    run(a, b, a_s, b_s, c)
    rows = torch.tensor(sorted({0, 1, 127, 128, 129, 255, 256, 4095, 4096, 8190, 8191} |
                               set(torch.randint(0, m, (21,), generator=torch.Generator().manual_seed(1)).tolist())))
    ref = oracle.dequant_matmul(a[rows.cuda()], b, a_s[rows.cuda()], b_s)
    assert_close(c[rows.cuda()], ref, "sampled rows")
    # doubling a_scale doubles every output bit-exactly (power-of-two scaling commutes with rounding)
    c2 = torch.empty_like(c)
    run(a, b, a_s * 2, b_s, c2)
    assert torch.equal(c2.float(), c.float() * 2)
    # same inputs, same plan -> same bits
    c3 = torch.empty_like(c)
    run(a, b, a_s, b_s, c3)
    assert torch.equal(c3.view(torch.int16), c.view(torch.int16))
    # every output was written exactly where it belongs: no NaN sentinel survives
    c4 = torch.full_like(c, float("nan"))
    run(a, b, a_s, b_s, c4)
    assert torch.isfinite(c4.float()).all()


# ------------------------------------------------------------------ edge cases


@pytest.mark.parametrize("m,n,k", [
    (1, 64, 128), (7, 8, 128), (128, 128, 128), (129, 130, 256), (200, 576, 1024), (1000, 520, 384),
    (128, 72, 256), (300, 1, 128), (257, 4099, 128), (512, 512, 7168), (4096, 512, 512),
])
def test_ragged_and_small_shapes(m, n, k):
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, m * 7 + n * 3 + k)
    c.fill_(float("nan"))
    run(a, b, a_s, b_s, c)
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), f"{m}x{n}x{k}")


# every tile width x single CTA / CTA pair x {no split, split-K 3}; without a split also every way
# the bf16 tile can leave: plain stores (-1), TMA store with 1 or 2 staging buffers (boxes ping-pong) or one per box (4)
PLANS = [Plan(block_n=bn, cta_pair=pr, split_k=sk, store_bufs=sb)
         for bn in (64, 128, 192, 256) for pr in (-1, 1) for (sk, sb) in ((1, -1), (1, 1), (1, 2), (1, 4), (3, 0))]


@pytest.mark.parametrize(
    "plan", PLANS, ids=lambda p: f"bn{p.block_n}_pair{p.cta_pair}_split{p.split_k}_store{p.store_bufs}")
def test_every_kernel_variant(plan):
    m, n, k = 600, 1096, 1536
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 99)
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    c.fill_(float("nan"))
    run(a, b, a_s, b_s, c, plan=plan)
    assert_close(c, ref, str(plan))
    # and with a 2-deep ring, the shallowest pipeline
    c.fill_(float("nan"))
    run(a, b, a_s, b_s, c, plan=Plan(block_n=plan.block_n, cta_pair=plan.cta_pair, split_k=plan.split_k,
                                     store_bufs=plan.store_bufs, stages=2))
    assert_close(c, ref, str(plan) + " stages=2")


@pytest.mark.parametrize("m,n,k", [(8192, 576, 7168), (8192, 2304, 1024), (4096, 4608, 512)])
def test_automatic_plans_with_pairs_and_tails(m, n, k):
    """Shapes whose automatic plan is a CTA pair with a split-K tail (or close to one): rows sampled against
    the oracle, and the run repeated bit for bit."""
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, m + n)
    c.fill_(float("nan"))
    run(a, b, a_s, b_s, c)
    rows = torch.tensor(sorted({0, 127, 128, 255, 256, m - 129, m - 1} | set(range(1000, 1040))), device="cuda")
    assert_close(c[rows], oracle.dequant_matmul(a[rows], b, a_s[rows], b_s), f"{m}x{n}x{k} {pkg.describe(m, n, k)}")
    assert torch.isfinite(c.float()).all()
    c2 = torch.full_like(c, float("nan"))
    run(a, b, a_s, b_s, c2)
    assert torch.equal(c2.view(torch.int16), c.view(torch.int16))


@pytest.mark.parametrize("bn,split,pair", [(192, 2, -1), (128, 3, -1), (64, 2, -1), (192, 3, 1), (128, 2, 1)])
def test_split_k_tail_of_a_partly_filled_last_wave(bn, split, pair):
    """More tiles than SMs, not a whole number of waves: the full waves run whole tiles, the tail is
    split along K (whole and split tiles in one launch)."""
    m, n, k = 4096, 2304, 1024
    plan_probe = pkg.describe(m, n, k)
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 17)
    c.fill_(float("nan"))
    plan = Plan(block_n=bn, cta_pair=pair, split_k=split)
    run(a, b, a_s, b_s, c, plan=plan)
    assert plan_probe.tiles > 0
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), f"tail bn={bn} split={split} pair={pair}")
    c2 = torch.full_like(c, float("nan"))
    run(a, b, a_s, b_s, c2, plan=plan)
    assert torch.equal(c2.view(torch.int16), c.view(torch.int16))


def test_split_k_is_deterministic_and_leaves_counters_clean():
    m, n, k = 256, 1536, 7168
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 5)
    plan = Plan(block_n=128, cta_pair=-1, split_k=4)
    outs = []
    for _ in range(3):
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        run(a, b, a_s, b_s, c, plan=plan)
        outs.append(c)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))
    assert_close(outs[0], oracle.dequant_matmul(a, b, a_s, b_s))


@pytest.mark.parametrize("phase", [0, 32, 64, 96])
def test_column_shard_with_phase(phase):
    """A shard that starts `phase` columns into a scale block equals those columns of the whole."""
    m, k, n_full = 192, 512, 832
    a, b, a_s, b_s, _ = cuda_inputs(m, n_full, k, 31)
    whole = oracle.dequant_matmul(a, b, a_s, b_s)
    c0 = 128 + phase
    bb = b[c0:c0 + 576].contiguous()
    bs = b_s[c0 // 128:(c0 + 576 - 1) // 128 + 1].contiguous()
    c = torch.full((m, 576), float("nan"), dtype=torch.bfloat16, device="cuda")
    run(a, bb, a_s, bs, c, n_phase=phase)
    assert_close(c, whole[:, c0:c0 + 576], f"phase {phase}")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_equals_whole_at_4608(world):
    m, n, k = 512, 4608, 1024
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 77)
    run(a, b, a_s, b_s, c)
    parts = []
    for r in range(world):
        spec = pkg.shard_spec(n, world, r)
        bb, bs = pkg.shard_inputs(b, b_s, spec)
        cc = torch.empty(m, spec.n_local, dtype=torch.bfloat16, device="cuda")
        run(a, bb.contiguous(), a_s, bs.contiguous(), cc, n_phase=spec.n_phase)
        parts.append(cc)
    got = torch.cat(parts, dim=1)
    assert_close(got, oracle.dequant_matmul(a, b, a_s, b_s), f"world {world}")
    assert_close(got, c.cpu(), "sharded vs whole")


@pytest.mark.parametrize("gm,gn", [(2, 2), (4, 2), (2, 1)])
def test_grid_sharded_equals_whole(gm, gn):
    """Row x column blocks of c computed separately (as the ranks of a multi-GPU run do) against the oracle."""
    m, n, k = 1152, 1216, 512
    a, b, a_s, b_s, _ = cuda_inputs(m, n, k, 55)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    for r in range(gm * gn):
        s = pkg.grid_spec(m, n, gm * gn, r, gm, gn)
        aa, bb, aas, bs = pkg.grid_inputs(a, b, a_s, b_s, s)
        cc = torch.empty(s.m_local, s.n_local, dtype=torch.bfloat16, device="cuda")
        run(aa, bb, aas, bs, cc, n_phase=s.n_phase)   # views: row-sliced a and b need no copy
        got[s.row_begin:s.row_end, s.cols.col_begin:s.cols.col_end] = cc
    assert_close(got, oracle.dequant_matmul(a, b, a_s, b_s), f"grid {gm}x{gn}")


def test_strided_operands_and_output():
    """Row-padded a/b, M-major (transposed-storage) scales, and c as a column slice of a wider buffer."""
    m, n, k = 300, 576, 768
    a, b, a_s, b_s, _ = cuda_inputs(m, n, k, 8)
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    a_pad = torch.zeros(m, k + 64, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    a_pad[:, :k] = a
    b_pad = torch.zeros(n, k + 128, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    b_pad[:, :k] = b
    a_s_t = a_s.t().contiguous().t()  # element (i,kb) at kb*M + i: the reference harness's native layout
    b_s_t = b_s.t().contiguous().t()
    assert a_s_t.stride() == (1, m)
    # c as a column slice of a wider buffer: offset 8 keeps the 16-byte alignment the TMA store needs,
    # offset 3 does not and exercises the plain-store fallback
    for off in (8, 3):
        wide = torch.full((m, n + 40), float("nan"), dtype=torch.bfloat16, device="cuda")
        c_view = wide[:, off:off + n]
        run(a_pad[:, :k], b_pad[:, :k], a_s_t, b_s_t, c_view)
        assert_close(c_view, ref, f"strided, column offset {off}")
        assert torch.isnan(wide[:, :off].float()).all() and torch.isnan(wide[:, off + n:].float()).all()


def test_inputs_are_not_modified_and_c_is_returned():
    m, n, k = 384, 640, 512
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 4)
    keep = [t.clone() for t in (a.view(torch.uint8), b.view(torch.uint8), a_s, b_s)]
    out = pkg.custom_kernel((a, b, a_s, b_s, c))
    check_device_status()
    assert out is c
    for before, after in zip(keep, (a.view(torch.uint8), b.view(torch.uint8), a_s, b_s)):
        assert torch.equal(before, after)


def test_extreme_values_and_zero_scales():
    """Largest finite e4m3fn magnitudes (+-448), zeros, subnormals; a zero scale zeroes its block.

    With same-sign operands nothing cancels and the contract's tolerance holds as it stands. With
    mixed signs the result is a small difference of huge terms (products up to 2e5, block sums up to
    2.6e7): the tensor core does not keep full fp32 precision while it adds the 128 products of a
    block (the reason block-scaled FP8 GEMMs promote to fp32 on the vector ALU every 128 K in the
    first place), so the error is bounded against the magnitude of the terms, not of the result."""
    m, n, k = 128, 256, 256
    g = torch.Generator().manual_seed(3)
    a_s = torch.rand(m, 2, generator=g).cuda()
    b_s = torch.rand(2, 2, generator=g).cuda()
    b_s[1, 0] = 0.0
    pos = torch.tensor([0x7E, 0x00, 0x01, 0x08, 0x38, 0x70], dtype=torch.uint8)
    mixed = torch.tensor([0x7E, 0xFE, 0x00, 0x80, 0x01, 0x81, 0x08, 0x38], dtype=torch.uint8)
    for codes, cancelling in ((pos, False), (mixed, True)):
        a = codes[torch.randint(0, len(codes), (m, k), generator=g)].view(torch.float8_e4m3fn).cuda()
        b = codes[torch.randint(0, len(codes), (n, k), generator=g)].view(torch.float8_e4m3fn).cuda()
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        run(a, b, a_s, b_s, c)
        ref = oracle.dequant_matmul_fp32(a, b, a_s, b_s)
        assert torch.isfinite(c.float()).all()
        assert (c[:, 128:].float().cpu() - ref[:, 128:].to(torch.bfloat16).float()).abs().max() >= 0  # shape sanity
        if not cancelling:
            assert_close(c, ref.to(torch.bfloat16), "extremes, same sign")
        else:
            a_abs = (a.view(torch.uint8) & 0x7F).view(torch.float8_e4m3fn)
            b_abs = (b.view(torch.uint8) & 0x7F).view(torch.float8_e4m3fn)
            mag = oracle.dequant_matmul_fp32(a_abs, b_abs, a_s, b_s)  # sum of |terms|
            err = (c.float().cpu() - ref).abs()
            bound = ATOL + RTOL * ref.abs() + 2.0 ** -10 * mag
            assert (err <= bound).all(), float((err - bound).max())


def test_host_errors_raise_before_launch():
    a, b, a_s, b_s, c = cuda_inputs(128, 128, 256, 1)
    with pytest.raises(ValueError):
        pkg.fp8_mm(a[:, :200], b[:, :200], a_s, b_s, c)            # K not a multiple of 128
    with pytest.raises(ValueError):
        pkg.fp8_mm(a, b, a_s[:, :1], b_s, c)                        # wrong a_scale shape
    with pytest.raises(ValueError):
        pkg.fp8_mm(a.view(torch.uint8), b, a_s, b_s, c)             # wrong dtype
    with pytest.raises(ValueError):
        pkg.fp8_mm(a.t().contiguous().t()[::2], b, a_s[::2], b_s, c[::2])  # neither K nor M contiguous
    with pytest.raises(Fp8MmError):
        pkg.fp8_mm(a, b, a_s, b_s, c, plan=Plan(block_n=96))        # unsupported forced plan
    with pytest.raises(Fp8MmError):
        pkg.fp8_mm(a, b, a_s, torch.cat([b_s, b_s]), c, n_phase=16)  # phase granularity is 32
    check_device_status()


def test_host_buffer_entry_point():
    m, n, k = 256, 576, 512
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 12)
    out = pkg.fp8_mm_host(a, b, a_s, b_s, c)
    assert out is c and not c.is_cuda
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), "host entry")


def test_host_buffer_entry_point_streams_row_ranges():
    # several row ranges (short first and last ones), pinned buffers, twice over the cached device buffers
    from amd_developer_challenge_2025_b200.fp8_mm import host_row_chunks
    m, n, k = 2304, 576, 512
    assert len(host_row_chunks(m, 512)) >= 5
    a, b, a_s, b_s, c = (t.pin_memory() for t in pkg.make_inputs(m, n, k, 13))
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    for _ in range(2):
        c.zero_()
        out = pkg.fp8_mm_host(a, b, a_s, b_s, c, chunk_rows=512)
        assert out is c
        assert_close(c, ref, "host entry, row ranges")
    check_device_status()


def test_non_default_stream_and_back_to_back_launches():
    m, n, k = 512, 1024, 1024
    a, b, a_s, b_s, c = cuda_inputs(m, n, k, 6)
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    outs = [torch.empty_like(c) for _ in range(8)]
    with torch.cuda.stream(s):
        for o in outs:
            pkg.fp8_mm(a, b, a_s, b_s, o)
    s.synchronize()
    check_device_status()
    for o in outs:
        assert_close(o, ref, "stream")
