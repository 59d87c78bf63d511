"""GPU parity tests for the grouped launch: G independent block-scaled GEMMs (same N, K) in one kernel,
each group checked against the CPU oracle, and bit-equal to G separate launches of the same plan."""
import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from amd_developer_challenge_2025_b200.fp8_mm import Fp8MmError, Plan, check_device_status
from oracle import fp8_mm_oracle as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-3


def grouped_inputs(g, m, n, k, seed):
    parts = [pkg.make_inputs(m, n, k, seed + i) for i in range(g)]
    a, b, a_s, b_s = (torch.stack([p[j] for p in parts]).cuda() for j in range(4))
    c = torch.full((g, m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    return a, b, a_s, b_s, c


def assert_close(c, ref, what=""):
    ok, excess, max_err = oracle.check(c, ref, RTOL, ATOL)
    assert ok, f"{what}: worst excess over tolerance {excess}, max abs err {max_err}"


@pytest.mark.parametrize("g,m,n,k", [(1, 128, 128, 128), (3, 300, 576, 512), (8, 128, 1536, 256), (5, 1, 64, 128),
                                     (4, 520, 200, 384)])
def test_groups_against_oracle(g, m, n, k):
    a, b, a_s, b_s, c = grouped_inputs(g, m, n, k, 11 * g + m)
    pkg.fp8_mm_grouped(a, b, a_s, b_s, c)
    check_device_status()
    for i in range(g):
        assert_close(c[i], oracle.dequant_matmul(a[i], b[i], a_s[i], b_s[i]), f"group {i} of {g}x{m}x{n}x{k}")


@pytest.mark.parametrize("bn,pair", [(64, -1), (128, -1), (192, -1), (256, -1), (192, 1), (256, 1)])
@pytest.mark.parametrize("store_bufs", [-1, 1, 2])
def test_every_width_equals_separate_launches(bn, pair, store_bufs):
    g, m, n, k = 3, 392, 840, 768
    a, b, a_s, b_s, c = grouped_inputs(g, m, n, k, 5)
    plan = Plan(block_n=bn, cta_pair=pair, split_k=1, store_bufs=store_bufs)
    pkg.fp8_mm_grouped(a, b, a_s, b_s, c, plan=plan)
    check_device_status()
    for i in range(g):
        want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        pkg.fp8_mm(a[i], b[i], a_s[i], b_s[i], want, plan=plan)
        check_device_status()
        assert torch.equal(c[i].view(torch.int16), want.view(torch.int16)), f"group {i}"
    assert_close(c[0], oracle.dequant_matmul(a[0], b[0], a_s[0], b_s[0]), "group 0")


def test_valid_rows_per_group_are_respected():
    """Rows at or past m_valid[g] are never written (NaN sentinel survives); the rows before it are right.
    Covers an empty group, a group cut inside a tile, one cut at a tile edge and a full one."""
    g, m, n, k = 5, 384, 328, 512
    a, b, a_s, b_s, c = grouped_inputs(g, m, n, k, 9)
    valid = [384, 0, 17, 256, 300]
    mv = torch.tensor(valid, dtype=torch.int32, device="cuda")
    for plan in (None, Plan(block_n=128, cta_pair=-1, store_bufs=-1), Plan(block_n=64, cta_pair=-1, store_bufs=2),
                 Plan(block_n=192, cta_pair=1), Plan(block_n=256, cta_pair=1, store_bufs=-1)):
        c.fill_(float("nan"))
        pkg.fp8_mm_grouped(a, b, a_s, b_s, c, m_valid=mv, plan=plan)
        check_device_status()
        for i, v in enumerate(valid):
            assert torch.isnan(c[i, v:].float()).all(), f"group {i}: rows past {v} were written"
            if v:
                assert_close(c[i, :v], oracle.dequant_matmul(a[i, :v], b[i], a_s[i, :v], b_s[i]), f"group {i}")


def test_strided_groups_and_padded_rows():
    """Groups as slices of larger buffers: group pitch and row pitch larger than the dense ones."""
    g, m, n, k = 3, 200, 192, 256
    a, b, a_s, b_s, _ = grouped_inputs(g, m, n, k, 21)
    a_big = torch.zeros(g, m + 56, k + 128, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    a_big[:, :m, :k] = a
    c_big = torch.full((g, m + 8, n + 16), float("nan"), dtype=torch.bfloat16, device="cuda")
    a_s_t = a_s.permute(0, 2, 1).contiguous().permute(0, 2, 1)  # [g][kb][m] storage
    pkg.fp8_mm_grouped(a_big[:, :m, :k], b, a_s_t, b_s, c_big[:, :m, 8:8 + n])
    check_device_status()
    for i in range(g):
        assert_close(c_big[i, :m, 8:8 + n], oracle.dequant_matmul(a[i], b[i], a_s[i], b_s[i]), f"group {i}")
    assert torch.isnan(c_big[:, m:].float()).all() and torch.isnan(c_big[:, :, :8].float()).all()
    assert torch.isnan(c_big[:, :, 8 + n:].float()).all()


def test_moe_sized_problem_matches_separate_launches():
    g, m, n, k = 8, 1024, 2048, 7168
    a, b, a_s, b_s, c = grouped_inputs(g, m, n, k, 77)
    pkg.fp8_mm_grouped(a, b, a_s, b_s, c)
    check_device_status()
    plan = pkg.describe(g * m, n, k)
    for i in (0, 3, 7):
        want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        pkg.fp8_mm(a[i], b[i], a_s[i], b_s[i], want, plan=Plan(block_n=plan.block_n, cta_pair=-1, split_k=1))
        check_device_status()
        assert_close(c[i], want.cpu(), f"group {i} vs single launch")
    rows = torch.tensor([0, 127, 128, 1023])
    assert_close(c[5][rows.cuda()], oracle.dequant_matmul(a[5][rows.cuda()], b[5], a_s[5][rows.cuda()], b_s[5]), "rows")


def test_grouped_errors():
    a, b, a_s, b_s, c = grouped_inputs(2, 128, 128, 128, 1)
    with pytest.raises(ValueError):
        pkg.fp8_mm_grouped(a[0], b, a_s, b_s, c)                               # a not 3-D
    with pytest.raises(ValueError):
        pkg.fp8_mm_grouped(a, b, a_s, b_s, c, plan=Plan(split_k=2))            # no split-K in grouped launches
    with pytest.raises(Fp8MmError):
        pkg.fp8_mm_grouped(a, b, a_s, b_s, c, plan=Plan(block_n=128, cta_pair=1))  # no paired kernel at this width
    with pytest.raises(ValueError):
        pkg.fp8_mm_grouped(a, b, a_s, b_s, c, m_valid=torch.zeros(2, dtype=torch.int64, device="cuda"))
    check_device_status()
