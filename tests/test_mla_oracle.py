"""CPU tests of the oracle for the RoPE and scaled-softmax kernels (the custom kernels around the KV
down-projection in the reference's MLA-decode submission)."""
import math

import pytest
import torch

from oracle import mla_oracle

needs_ref = pytest.mark.skipif(not mla_oracle.ref_available(),
                               reason="neither the reference checkout nor a prebuilt oracle/_ref is present")


def bf16_randn(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16)


# (d0, d1, d2, pos): the query call (d0 = bs*nh = 128, one position, d2 = 64 -> the d0=128 kernel), the key call
# (d0 = bs, d1 = past + 1 positions), an odd d0 (the plain kernel), a d2 other than 64
ROPE_CASES = [(128, 1, 64, 4096), (128, 1, 64, 77), (4, 300, 64, 0), (3, 17, 64, 5), (6, 9, 32, 1000), (2, 520, 64, 0)]


@needs_ref
@pytest.mark.parametrize("d0,d1,d2,pos", ROPE_CASES)
def test_rope_restatement_equals_the_reference_kernels_bit_for_bit(d0, d1, d2, pos):
    x = bf16_randn(d0, d1, d2, seed=d0 + d1 + pos)
    want = mla_oracle.rope_3d_ref(x, pos)                  # the launcher's choice of kernel
    got = mla_oracle.rope_3d(x, pos)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # the reference's kernel variants agree with one another wherever they apply
    assert torch.equal(mla_oracle.rope_3d_ref(x, pos, which=1).view(torch.int16), want.view(torch.int16))
    if d0 % 2 == 0:
        assert torch.equal(mla_oracle.rope_3d_ref(x, pos, which=2).view(torch.int16), want.view(torch.int16))


def test_rope_is_a_rotation_up_to_bf16_rounding():
    x = bf16_randn(8, 40, 64, seed=3)
    y = mla_oracle.rope_3d(x, 11).float()
    xf = x.float()
    n_in = (xf[..., :32] ** 2 + xf[..., 32:] ** 2)
    n_out = (y[..., :32] ** 2 + y[..., 32:] ** 2)
    assert torch.allclose(n_out, n_in, rtol=5e-2, atol=5e-2)
    # position 0 of a rope that starts at 0 is the identity (angle 0: cos 1, sin 0)
    assert torch.equal(mla_oracle.rope_3d(x, 0)[:, 0].view(torch.int16), x[:, 0].view(torch.int16))


@pytest.mark.parametrize("bs,nh,sl", [(2, 3, 8), (1, 5, 1000), (2, 2, 4097), (1, 1, 8192), (3, 2, 13)])
def test_softmax_restatement_against_torch(bs, nh, sl):
    qk = (bf16_randn(bs, nh, sl, seed=sl) * 4).to(torch.bfloat16)
    got = mla_oracle.div_softmax(qk, 128, 64).float()
    want = torch.softmax(qk.float() / math.sqrt(192.0), dim=-1)
    # two bf16 roundings (the kept exponential and the result): 2^-8 each, relative
    assert torch.allclose(got, want, rtol=2.0 ** -6, atol=1e-30)
    assert torch.allclose(got.sum(-1), torch.ones(bs, nh), atol=2e-2)
