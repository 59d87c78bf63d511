"""GPU parity of the RoPE and scaled-softmax kernels against the CPU oracle (oracle/mla_oracle.py, whose RoPE is
pinned bit for bit to the reference's own kernels), through the host mirror of the reference's
`module.mla_decode` / `module.div_softmax` calls.

Tolerance. These are floating-point kernels whose results pass through powf / cosf / sinf / expf, where the
device's and the host's libraries may differ in the last fp32 bit; after the bf16 roundings the reference
prescribes, that can move an output by one bf16 step in rare cases. RoPE: every element within one bf16 ulp
of the oracle (2^-7 relative) and at least 99.5 % of them bit-equal. Softmax: |got - want| <= 2^-6 * want
(two bf16 roundings) and rows sum to 1 within 2e-2."""
import math

import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from oracle import mla_oracle

pytestmark = pytest.mark.gpu


def bf16_randn(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16)


def assert_rope_close(got, want):
    g, w = got.float().cpu(), want.float()
    assert torch.isfinite(g).all()
    assert ((g - w).abs() <= 2.0 ** -7 * w.abs() + 1e-6).all(), float((g - w).abs().max())
    equal = (got.cpu().view(torch.int16) == want.view(torch.int16)).float().mean().item()
    assert equal >= 0.995, equal


@pytest.mark.parametrize("d0,d1,d2,pos", [(128, 1, 64, 4096), (128, 1, 64, 77), (4, 300, 64, 0), (3, 17, 64, 5),
                                          (6, 9, 32, 1000), (16, 2049, 64, 0)])
def test_rope_contiguous(d0, d1, d2, pos):
    x = bf16_randn(d0, d1, d2, seed=d0 + d1 + pos)
    dx = x.cuda()
    y = torch.full_like(dx, float("nan"))
    pkg.mla_decode(dx, y, pos, 0, 0, d0, d1, d2, d1 * d2, d2, d1 * d2, d2)
    torch.cuda.synchronize()
    assert_rope_close(y, mla_oracle.rope_3d(x, pos))


def test_rope_unaligned_strides_take_the_scalar_kernel():
    """Rows that do not start on 16-byte boundaries (a column slice at an odd offset, odd row pitch)."""
    d0, d1, d2, pos = 5, 33, 64, 9
    wide = bf16_randn(d0, d1, d2 + 3, seed=4)
    dwide = wide.cuda()
    out = torch.full((d0, d1, d2 + 5), float("nan"), dtype=torch.bfloat16, device="cuda")
    pkg.mla_decode(dwide, out, pos, 1, 3, d0, d1, d2, d1 * (d2 + 3), d2 + 3, d1 * (d2 + 5), d2 + 5)
    torch.cuda.synchronize()
    assert_rope_close(out[:, :, 3:3 + d2], mla_oracle.rope_3d(wide[:, :, 1:1 + d2], pos))
    assert torch.isnan(out[:, :, :3].float()).all() and torch.isnan(out[:, :, 3 + d2:].float()).all()


def test_rope_as_the_reference_calls_it():
    """The two call sites of the reference (3-amd-mla-decode/amd-mla-submission.py:265, 273): the query's rope
    part rotated in place inside [bs*nh, sl, dnope+drope], and the key's rope part gathered out of the KV cache
    [bs, msl, dkv+drope] into a fresh [bs, pl+sl, drope]."""
    bs, nh, sl, pl, msl = 4, 16, 1, 333, 512
    dnope, drope, dkv = 128, 64, 512
    qu = bf16_randn(bs * nh, sl, dnope + drope, seed=1)
    dq = qu.cuda()
    pkg.mla_decode(dq, dq, pl, dnope, dnope, bs * nh, sl, drope, dnope + drope, dnope + drope, dnope + drope,
                   dnope + drope)
    torch.cuda.synchronize()
    want_q = qu.clone()
    want_q[:, :, dnope:] = mla_oracle.rope_3d(qu[:, :, dnope:], pl)
    assert torch.equal(dq[:, :, :dnope].cpu().view(torch.int16), qu[:, :, :dnope].view(torch.int16))  # untouched
    assert_rope_close(dq[:, :, dnope:], want_q[:, :, dnope:])

    cache = bf16_randn(bs, msl, dkv + drope, seed=2)
    dcache = cache.cuda()
    kr = torch.full((bs, pl + sl, drope), float("nan"), dtype=torch.bfloat16, device="cuda")
    pkg.mla_decode(dcache, kr, 0, dkv, 0, bs, pl + sl, drope, msl * (dkv + drope), dkv + drope, (pl + sl) * drope, drope)
    torch.cuda.synchronize()
    assert_rope_close(kr, mla_oracle.rope_3d(cache[:, :pl + sl, dkv:], 0))
    assert torch.equal(dcache.cpu().view(torch.int16), cache.view(torch.int16))   # the cache is only read


@pytest.mark.parametrize("bs,nh,sl", [(2, 3, 8), (1, 5, 1000), (2, 2, 4097), (4, 16, 6145), (1, 2, 8192), (3, 2, 13),
                                      (1, 1, 20000)])
def test_div_softmax(bs, nh, sl):
    qk = (bf16_randn(bs, nh, sl, seed=sl) * 4).to(torch.bfloat16)
    d = qk.cuda()
    out = pkg.div_softmax(d, bs, nh, sl, 128, 64)
    torch.cuda.synchronize()
    assert out is d
    got = d.float().cpu()
    want = mla_oracle.div_softmax(qk, 128, 64).float()
    assert torch.isfinite(got).all()
    assert ((got - want).abs() <= 2.0 ** -6 * want.abs() + 1e-30).all(), float((got - want).abs().max())
    assert torch.allclose(got.sum(-1), torch.ones(bs, nh), atol=2e-2)
    # and against the textbook definition
    ref = torch.softmax(qk.float() / math.sqrt(192.0), dim=-1)
    assert torch.allclose(got, ref, rtol=2.0 ** -6, atol=1e-30)


def test_kv_down_projection_shape_through_the_fp8_gemm():
    """`x @ wDKV.T` of the reference's model (bs rows, N = dkv + drope = 576, K = 7168) as an FP8 block-scaled GEMM."""
    from oracle import fp8_mm_oracle as oracle

    bs, n, k = 128, 576, 7168
    x, w, xs, ws, _ = pkg.make_inputs(bs, n, k, seed=9, device="cuda")
    out = pkg.kv_down_projection_fp8(x, xs, w, ws)
    torch.cuda.synchronize()
    ok, excess, max_err = oracle.check(out, oracle.dequant_matmul(x, w, xs, ws))
    assert ok, (excess, max_err)


def test_bad_arguments_are_refused():
    x = torch.zeros(4, 4, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        pkg.mla_decode(x, x, 0, 0, 0, 4, 4, 63, 256, 64, 256, 64)      # odd d2
    with pytest.raises(ValueError):
        pkg.mla_decode(x, x, 0, 0, 0, 5, 4, 64, 256, 64, 256, 64)      # runs past the tensor
    with pytest.raises(ValueError):
        pkg.div_softmax(x.float(), 4, 4, 64, 128, 64)                  # not bf16
