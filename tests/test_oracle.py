"""CPU tests of the oracle: against the reference's own dequantise kernels compiled for the host
(oracle/_ref), against the committed fixtures those kernels produced, against the independent plain-C
restatement, and the two summation orders against each other within the contract's tolerance."""
import glob
import hashlib
import os

import numpy as np
import pytest
import torch

from amd_developer_challenge_2025_b200.inputs import make_inputs
from oracle import c_oracle
from oracle import fp8_mm_oracle as oracle
from oracle import ref_oracle

needs_ref = pytest.mark.skipif(not ref_oracle.available(),
                               reason="neither the reference checkout nor a prebuilt oracle/_ref is present")

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))


def load_case(path):
    z = np.load(path)
    a = torch.from_numpy(z["a"]).view(torch.float8_e4m3fn)
    b = torch.from_numpy(z["b"]).view(torch.float8_e4m3fn)
    a_s = torch.from_numpy(z["a_scale"])
    b_s = torch.from_numpy(z["b_scale"])
    c32 = torch.from_numpy(z["c_fp32"])
    c16 = torch.from_numpy(z["c_bf16_bits"]).view(torch.bfloat16)
    m, n, k, seed, phase = (int(v) for v in z["meta"])
    return a, b, a_s, b_s, c32, c16, (m, n, k, seed, phase)


def sha(t: torch.Tensor) -> bytes:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).digest()


def test_fixtures_exist():
    assert len(CASES) >= 5


def test_e4m3fn_decode_table_all_256_codes():
    """torch's decoder, the C oracle's own decoder and the committed table agree bit for bit."""
    want = np.load(os.path.join(GOLDEN, "e4m3fn_table.npy"))
    got_torch = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    got_c = c_oracle.e4m3fn_table()
    for got in (got_torch, got_c):
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    # e4m3fn landmarks: max 448, smallest subnormal 2^-9, NaN only at 0x7f / 0xff
    assert want[0x7E] == 448.0 and want[0x01] == 2.0 ** -9 and want[0x38] == 1.0
    assert np.isnan(want[0x7F]) and np.isnan(want[0xFF]) and np.isnan(want).sum() == 2


@needs_ref
def test_reference_shim_decodes_e4m3fn_like_torch():
    """The float conversion given to the reference's `(float)src_val` is torch's e4m3fn decode, all 256 codes."""
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    got = ref_oracle.decode_table()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))


# Beside the fixtures: N=576 (five b_scale rows, the last one half used), a ragged everything, and
# one problem at config 0's K.
REF_SHAPES = [(40, 576, 384, 13), (7, 130, 128, 21), (65, 577, 256, 22), (16, 1536, 7168, 23)]


@needs_ref
@pytest.mark.parametrize("m,n,k,seed", REF_SHAPES)
def test_dequantise_equals_reference_kernels_bit_for_bit(m, n, k, seed):
    """oracle.dequant_a / dequant_b against the reference's dqa_kernel / dqb_kernel run on the
    reference's own [k][m] / [k][n] / [k/128][m] / [k/128][ceil(n/128)] storage."""
    a, b, a_s, b_s, _ = make_inputs(m, n, k, seed)
    a_km = ref_oracle.dequant_a_km(a, a_s)
    b_kn = ref_oracle.dequant_b_kn(b, b_s)
    assert torch.equal(oracle.dequant_a(a, a_s).view(torch.int32), a_km.T.contiguous().view(torch.int32))
    assert torch.equal(oracle.dequant_b(b, b_s).view(torch.int32), b_kn.T.contiguous().view(torch.int32))
    # the whole path: the same dequantised bits go into an fp32 matmul on both sides, so the only
    # difference left is the order in which the BLAS adds K products
    got = oracle.dequant_matmul_fp32(a, b, a_s, b_s)
    want = ref_oracle.dequant_matmul_fp32(a, b, a_s, b_s)
    assert (got - want).abs().max() <= 2e-5 * want.abs().max()
    ok, excess, max_err = oracle.check(got.to(torch.bfloat16), want.to(torch.bfloat16))
    assert ok, (excess, max_err)


@needs_ref
def test_reference_kernels_see_every_code():
    """All 256 byte values through the reference's dqa_kernel with scale 1 give the decode table."""
    a = torch.arange(256, dtype=torch.uint8).repeat(128, 1).T.contiguous().view(torch.float8_e4m3fn)  # [256, 128]
    a_s = torch.ones(256, 1)
    got = ref_oracle.dequant_a_km(a, a_s)[0].numpy()  # k = 0: one value per row = per code
    want = np.load(os.path.join(GOLDEN, "e4m3fn_table.npy"))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_dequantise_matches_the_reference_digests_in_the_fixture(path):
    """Runs without the reference: the fixtures carry SHA-256 digests of what the reference's kernels
    produced (in its [k][m] / [k][n] storage); the oracle's dequantised operands must hash the same."""
    z = np.load(path)
    a, b, a_s, b_s, c32, c16, (m, n, k, seed, phase) = load_case(path)
    assert sha(oracle.dequant_a(a, a_s).T) == bytes(z["dq_a_km_sha256"])
    assert sha(oracle.dequant_b(b, b_s, phase).T) == bytes(z["dq_b_kn_sha256"])


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_oracle_reproduces_fixture(path):
    a, b, a_s, b_s, c32, c16, (m, n, k, seed, phase) = load_case(path)
    got = oracle.dequant_matmul(a, b, a_s, b_s, phase)
    ok, excess, max_err = oracle.check(got, c16)
    assert ok, (excess, max_err)
    # bf16 results may differ by one rounding step when BLAS threads change the fp32 sum order
    assert (got.float() - c16.float()).abs().max() <= 2.0 ** -7 * c16.float().abs().max()


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_c_restatement_matches_fixture(path):
    a, b, a_s, b_s, c32, c16, (m, n, k, seed, phase) = load_case(path)
    for fn in (c_oracle.dequant_matmul_fp32, c_oracle.block_order_fp32):
        got = fn(a, b, a_s, b_s, phase)
        ok, excess, max_err = oracle.check(got.to(torch.bfloat16), c16)
        assert ok, (fn.__name__, excess, max_err)
        # fp32 results agree to fp32 summation noise, far inside the bf16 contract
        rel = (got - c32).abs().max() / c32.abs().max()
        assert rel < 1e-4, (fn.__name__, float(rel))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_inputs_reproduce_fixture_bits(path):
    """The generator is deterministic: the fixture's input bytes come back from the seed."""
    a, b, a_s, b_s, c32, c16, (m, n, k, seed, phase) = load_case(path)
    a2, b2, as2, bs2, _ = make_inputs(m, n + phase, k, seed)
    assert torch.equal(a2.view(torch.uint8), a.view(torch.uint8))
    assert torch.equal(b2[phase:].view(torch.uint8), b.view(torch.uint8))
    assert torch.equal(as2, a_s) and torch.equal(bs2, b_s)


@pytest.mark.parametrize("m,n,k", [(64, 256, 1024), (33, 576, 512), (16, 130, 128)])
def test_block_order_equals_dequant_order_within_contract(m, n, k):
    a, b, a_s, b_s, _ = make_inputs(m, n, k, seed=m + n + k)
    ref = oracle.dequant_matmul(a, b, a_s, b_s)
    alt = oracle.block_order_matmul(a, b, a_s, b_s)
    ok, excess, max_err = oracle.check(alt, ref)
    assert ok, (excess, max_err)


def test_b_scale_has_ceil_rows():
    """N=576 uses 5 scale rows, not 4.5 (reference: 1-amd-fp8-mm/amd-fp8-mm-submission.py:75)."""
    a, b, a_s, b_s, c = make_inputs(8, 576, 128, seed=3)
    assert b_s.shape == (5, 1) and a_s.shape == (8, 1) and c.shape == (8, 576)
    # zeroing the 5th row's scale zeroes exactly columns 512..575
    b_s2 = b_s.clone()
    b_s2[4] = 0
    out = oracle.dequant_matmul(a, b, a_s, b_s2).float()
    assert out[:, 512:].abs().max() == 0 and out[:, :512].abs().max() > 0


def test_linearity_in_scales():
    """Doubling a_scale doubles c exactly (power-of-two scaling commutes with every rounding)."""
    a, b, a_s, b_s, _ = make_inputs(16, 128, 256, seed=5)
    c1 = oracle.dequant_matmul(a, b, a_s, b_s).float()
    c2 = oracle.dequant_matmul(a, b, a_s * 2, b_s).float()
    assert torch.equal(c2, c1 * 2)


def test_check_rejects_wrong_and_nonfinite():
    ref = torch.full((4, 4), 10.0, dtype=torch.bfloat16)
    assert oracle.check(ref.clone(), ref)[0]
    bad = ref.clone()
    bad[0, 0] = 10.5
    assert not oracle.check(bad, ref)[0]
    nan = ref.clone()
    nan[1, 1] = float("nan")
    assert not oracle.check(nan, ref)[0]
