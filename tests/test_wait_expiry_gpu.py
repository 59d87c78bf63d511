"""A wait inside the kernel runs out, in the allowed form: nothing traps, nothing waits without limit.

The library's self-test entry point launches the plain 64-wide kernel with every mbarrier wait limited
to a few milliseconds and with the copy of one K block left out. The waits that depend on that block
run out, the kernel returns by itself, and the status words say which role gave up. The context stays
usable: the next ordinary launch in the same process passes parity."""
import pytest
import torch

import amd_developer_challenge_2025_b200 as pkg
from amd_developer_challenge_2025_b200.fp8_mm import (Fp8MmDeviceError, _status_words, check_device_status,
                                                      selftest_wait_expiry)
from oracle import fp8_mm_oracle as oracle

pytestmark = pytest.mark.gpu

DEV_WAIT_EXPIRED = 1


def test_expired_wait_is_reported_and_the_context_stays_usable():
    check_device_status()                      # nothing pending from earlier launches
    words = selftest_wait_expiry("cuda", limit_ms=5.0)
    assert words[0] == DEV_WAIT_EXPIRED, words
    role = words[1] >> 8
    # the roles that wait for the missing block: the MMA issuer (0x3xx: operands never land) or the
    # promotion warps (0x4xx: the block's partial never completes); whoever ran out first reports
    assert role in (3, 4), [hex(x) for x in words]
    assert words[2] == 0                       # one tile, one CTA
    # the very next ordinary launch works and is checked against the CPU oracle
    m, n, k = 384, 576, 1024
    a, b, a_s, b_s, c = pkg.make_inputs(m, n, k, 5, device="cuda")
    c.fill_(float("nan"))
    pkg.fp8_mm(a, b, a_s, b_s, c)
    check_device_status()
    ok, excess, max_err = oracle.check(c, oracle.dequant_matmul(a, b, a_s, b_s))
    assert ok, (excess, max_err)


def test_check_device_status_raises_on_a_recorded_expiry():
    """The host side of the report: status words a kernel left behind turn into Fp8MmDeviceError once,
    and are cleared by the check."""
    dev = torch.device("cuda", torch.cuda.current_device())
    st = _status_words(dev)
    st.copy_(torch.tensor([DEV_WAIT_EXPIRED, 0x401, 7, 1], dtype=torch.int32))
    with pytest.raises(Fp8MmDeviceError) as e:
        check_device_status(dev)
    assert "0x401" in str(e.value) and "block=7" in str(e.value)
    check_device_status(dev)                   # cleared: the second check passes
