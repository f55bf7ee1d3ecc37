"""Failure detection on one GPU, without faulting or hanging anything: a cross-rank wait that can
never complete (the "peers" are local buffers nobody writes — ranks that never show up) must give
up after its poll limit, set the context's error word, and leave the context usable. The failure
is made on the host (strictb200_tp_comm_open_absent_peers); the kernel only runs out of polls."""
import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,two_shot", [(2, 0), (2, 1), (8, 1), (4, 0)])
def test_wait_for_absent_ranks_expires_and_is_reported(world, two_shot):
    ctx = sb.Context(0)  # a context of its own: the shared one stays single-rank
    try:
        N.check(N.lib().strictb200_tp_comm_open_absent_peers(ctx.h, world))
        ctx.set_option("tp_two_shot", two_shot)
        ctx.set_option("wait_limit", 20000)
        assert ctx.get_option("wait_limit") == 20000
        M, d, splits = 4, 1024, 2
        rng = np.random.default_rng(0)
        part = rng.standard_normal((splits, M, d)).astype(np.float32)
        dp, dsx, dsw = DV.of(ctx, part), DV.of(ctx, np.ones(M, np.float32)), DV.of(ctx, np.ones(d, np.float32))
        dres, dg, dy = DV.of(ctx, np.zeros((M, d), np.float32)), DV.of(ctx, np.ones(d, np.float32)), DV(ctx, M * d, np.uint16)
        for _ in range(2):  # the second call finds a clean error word and fails the same way
            N.check(N.lib().strictb200_tp_allreduce_rownorm(ctx.h, dp.p, splits, dsx.p, dsw.p, dres.p, dg.p, 1e-6, M, d, dy.p, None, None))
            with pytest.raises(N.KernelException) as e:
                ctx.device_status()
            assert e.value.status == N.ERR_TIMEOUT and "wait expired" in str(e.value)
            assert ctx.device_status() == 0  # reading the word cleared it
        # the context still runs ordinary work
        a = DV.of(ctx, np.arange(1000, dtype=np.float32))
        N.check(N.lib().strictb200_ew_binary(ctx.h, 2, a.p, a.p, a.p, 1000))
        assert np.array_equal(a.to_host(), np.arange(1000, dtype=np.float32) ** 2)
        assert ctx.device_status() == 0
    finally:
        ctx.dispose()


def test_options_are_per_context_and_checked(ctx):
    assert ctx.get_option("pdl") in (0, 1)
    with ctx.option("attn_tc", 2):
        assert ctx.get_option("attn_tc") == 2
        other = sb.Context(0)
        assert other.get_option("attn_tc") == -1
        other.dispose()
    assert ctx.get_option("attn_tc") == -1
    with pytest.raises(ValueError):
        ctx.set_option("no_such_switch", 1)
