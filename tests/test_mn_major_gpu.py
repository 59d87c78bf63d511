"""GPU parity tests for MN-major operands: a stored as [K][M] and/or b as [K][N], the storage the
reference's harness hands its kernels (1-amd-fp8-mm/amd-fp8-mm-submission.py:283-300 index
`a[k*m + i]`). The tile is loaded as it lies and described to the tensor core as an MN-major
operand; the results must equal the K-major ones bit for bit (same products, same order)."""
import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from amd_developer_challenge_2025_b200.fp8_mm import Fp8MmError, Plan, check_device_status
from amd_developer_challenge_2025_b200.inputs import mn_major
from oracle import fp8_mm_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-3


def run(a, b, a_s, b_s, c, **kw):
    out = pkg.fp8_mm(a, b, a_s, b_s, c, **kw)
    check_device_status(c.device)
    return out


def assert_close(c, ref, what=""):
    ok, excess, max_err = oracle.check(c, ref, RTOL, ATOL)
    assert ok, f"{what}: worst excess over tolerance {excess}, max abs err {max_err}"


LAYOUTS = [(True, False), (False, True), (True, True)]


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS, ids=["a_mn", "b_mn", "both_mn"])
@pytest.mark.parametrize("bn", [64, 128, 192, 256])
def test_every_width_and_layout(bn, a_mn, b_mn):
    """Forced tile widths (b uses 64-byte swizzle boxes at 64 and 192, 128-byte ones at 128 and 256),
    whole tiles and split-K; against the oracle and bit-equal to the K-major run of the same plan."""
    m, n, k = 608, 1104, 1536
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 99, device="cuda")
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    aa = mn_major(a) if a_mn else a
    bb = mn_major(b) if b_mn else b
    assert (aa.stride(0) == 1) == a_mn and (bb.stride(0) == 1) == b_mn
    for split in (1, 3):
        plan = Plan(block_n=bn, cta_pair=-1, split_k=split)
        want = torch.empty_like(c)
        run(a, b, a_s, b_s, want, plan=plan)
        c.fill_(float("nan"))
        run(aa, bb, a_s, b_s, c, plan=plan)
        assert_close(c, ref, f"bn={bn} split={split}")
        assert torch.equal(c.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("m,n,k,seed", [
    (256, 1536, 7168, 8135),
    (2048, 576, 7168, 12346),
    (2048, 7168, 512, 17512),
    (2048, 7168, 256, 5364),
])
def test_named_configs_in_harness_native_storage(m, n, k, seed):
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, seed, device="cuda", layout="mn")
    a_s, b_s = mn_major(a_s), mn_major(b_s)  # the harness stores the scales [K/128][M] as well
    c.fill_(float("nan"))
    out = pkg.custom_kernel((a, b, a_s, b_s, c))
    check_device_status()
    assert out is c
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), f"{m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(16, 64, 128), (144, 80, 256), (1008, 528, 384), (128, 16, 128), (272, 4112, 128)])
def test_ragged_shapes(m, n, k):
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, m + n + k, device="cuda", layout="mn")
    c.fill_(float("nan"))
    run(a, b, a_s, b_s, c)
    assert_close(c, oracle.dequant_matmul(a, b, a_s, b_s), f"{m}x{n}x{k}")


def test_headline_equals_k_major_bits_under_the_same_plan():
    """Same plan, same products, same order: the MN-major run reproduces the K-major bits, for the single-CTA
    plan and for the 256-wide CTA-pair plan (the automatic choice for this shape in either storage)."""
    m, n, k = 8192, 4608, 7168
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 65436, device="cuda")
    am, bm = mn_major(a), mn_major(b)
    assert pkg.describe(m, n, k).cta_pair == 1 and pkg.describe(m, n, k).block_n == 256
    for plan in (Plan(block_n=192, cta_pair=-1, split_k=1), Plan(block_n=256, cta_pair=1, split_k=1), None):
        run(a, b, a_s, b_s, c, plan=plan)
        c2 = torch.full_like(c, float("nan"))
        run(am, bm, a_s, b_s, c2, plan=plan)
        assert torch.equal(c2.view(torch.int16), c.view(torch.int16)), str(plan)
    rows = torch.tensor([0, 127, 128, 4095, 4096, 8191], device="cuda")
    assert_close(c2[rows], oracle.dequant_matmul(a[rows], b, a_s[rows], b_s), "automatic MN-major plan")
    assert torch.isfinite(c2.float()).all()


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS, ids=["a_mn", "b_mn", "both_mn"])
@pytest.mark.parametrize("bn", [192, 256])
def test_cta_pairs_with_mn_major_operands(bn, a_mn, b_mn):
    """CTA pairs take MN-major operands where a paired kernel exists: any a at the 192- and 256-wide tiles, an
    MN-major b at the 256-wide tile only (each CTA's half of the columns must be whole 64-byte boxes). A forced
    pair plan outside that set is refused; the automatic plan falls back to single CTAs."""
    from amd_developer_challenge_2025_b200.fp8_mm import Fp8MmError

    m, n, k = 1104, 1104, 1024   # MN-major storage needs M and N to be multiples of 16 (the pitch)
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 98, device="cuda")
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    aa = mn_major(a) if a_mn else a
    bb = mn_major(b) if b_mn else b
    plan = Plan(block_n=bn, cta_pair=1, split_k=1)
    if b_mn and bn == 192:
        with pytest.raises(Fp8MmError):
            pkg.fp8_mm(aa, bb, a_s, b_s, c, plan=plan)
        check_device_status()
        return
    want = torch.empty_like(c)
    run(a, b, a_s, b_s, want, plan=plan)
    c.fill_(float("nan"))
    run(aa, bb, a_s, b_s, c, plan=plan)
    assert_close(c, ref, f"pair bn={bn}")
    assert torch.equal(c.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("world", [2, 8])
def test_column_shards_of_an_mn_major_b_are_views(world):
    """A column shard of [K][N] storage is a strided view (pitch = the full N): no copy is needed."""
    m, n, k = 512, 4608, 1024
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 77, device="cuda", layout="mn")
    parts = []
    for r in range(world):
        spec = pkg.shard_spec(n, world, r)
        bb, bs = pkg.shard_inputs(b, b_s, spec)
        assert bb.stride() == (1, n)
        cc = torch.empty(m, spec.n_local, dtype=torch.bfloat16, device="cuda")
        run(a, bb, a_s, bs.contiguous(), cc, n_phase=spec.n_phase)
        parts.append(cc)
    assert_close(torch.cat(parts, dim=1), oracle.dequant_matmul(a, b, a_s, b_s), f"world {world}")


def test_layout_errors():
    a, b, a_s, b_s, c = pkg.make_inputs(128, 128, 256, 1, device="cuda", layout="mn")
    with pytest.raises(Fp8MmError):
        pkg.fp8_mm(a, b, a_s, b_s, c, plan=Plan(block_n=128, cta_pair=1))   # no paired kernel at this width
    with pytest.raises(ValueError):
        pkg.fp8_mm(a[::2], b, a_s[::2], b_s, c[::2])                   # neither dimension contiguous
    a24, b24, as24, bs24, c24 = pkg.make_inputs(24, 128, 128, 2, device="cuda", layout="mn")
    with pytest.raises(ValueError):
        pkg.fp8_mm(a24, b24, as24, bs24, c24)                          # pitch 24 is not a multiple of 16
    check_device_status()
