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


_FAKE_NCCL_CHILD = r"""
import ctypes, os, sys
import numpy as np
sys.path.insert(0, os.environ["REPO_ROOT"])
import strict_b200 as sb
from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV
fake = ctypes.CDLL(os.environ["STRICTB200_NCCL_LIB"])  # the same object the library dlopens

def tp_context():
    ctx = sb.Context(0)
    uid = np.zeros(128, np.uint8)
    N.check(N.lib().strictb200_tp_unique_id(N.ptr(uid)))
    assert uid[0] == 7                                   # it is the stand-in that answered
    ctx.tp_init(2, 0, N.ptr(uid))
    return ctx

# 1. an asynchronous NCCL error (a peer or a link failed) surfaces at the next synchronise and aborts the communicator
ctx = tp_context()
buf = DV.of(ctx, np.ones(16, np.float32))
N.check(N.lib().strictb200_tp_allreduce_f32(ctx.h, buf.p, 16))
ctx.synchronize()
assert fake.fake_nccl_allreduces() == 1 and fake.fake_nccl_aborts() == 0
fake.fake_nccl_set_async_error(3)
try:
    ctx.synchronize()
    raise SystemExit("the asynchronous error was not reported")
except N.KernelException as e:
    assert e.status == N.ERR_NCCL and "aborted" in str(e), e
assert fake.fake_nccl_aborts() == 1
fake.fake_nccl_set_async_error(0)
try:
    N.check(N.lib().strictb200_tp_allreduce_f32(ctx.h, buf.p, 16))
    raise SystemExit("a collective ran on an aborted communicator")
except N.KernelException as e:
    assert e.status == N.ERR_NCCL
ctx.synchronize()                                        # the context itself still works
ctx.dispose()
assert fake.fake_nccl_destroys() == 0                    # an aborted communicator is not destroyed a second time

# 2. a stream that does not finish within host_timeout_ms: ERR_TIMEOUT and an abort, no endless wait.
#    The slow work is an element-wise program bounded by its step budget; it ends by itself.
ctx = tp_context()
slow = sb.InstructionsToCuda().compile(sb.Method("Slow(a Number) Number", ["\tmutable t = 0", "\tfor 8000", "\t\tt = t + a", "\tt"]))
n = 1 << 21
a, out = DV(ctx, n), DV(ctx, n)
a.zero()
ctx.set_option("host_timeout_ms", 20)
slow.launch(ctx, a, out, n)
try:
    ctx.synchronize()
    timed_out = False
except N.KernelException as e:
    assert e.status == N.ERR_TIMEOUT and "aborted" in str(e), e
    timed_out = True
ctx.set_option("host_timeout_ms", 0)
ctx.synchronize()                                        # without a limit the call waits for the kernel, which ends by itself
assert ctx.device_status() == 0
assert timed_out and fake.fake_nccl_aborts() == 2, (timed_out, fake.fake_nccl_aborts())
ctx.dispose()
print("fake-nccl-ok")
"""


def test_nccl_async_error_and_host_timeout_abort_the_communicator(tmp_path):
    """NCCL is bound with dlopen; a stand-in (tests/fake_nccl.c) injects the failures on the host:
    an asynchronous error code, and a stream that outlasts host_timeout_ms. Both must end the
    synchronising call with an error status and one ncclCommAbort, never with an endless wait."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    so = str(tmp_path / "libfakenccl.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", so, os.path.join(here, "fake_nccl.c")])
    env = dict(os.environ, STRICTB200_NCCL_LIB=so, REPO_ROOT=os.path.dirname(here))
    r = subprocess.run([sys.executable, "-c", _FAKE_NCCL_CHILD], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "fake-nccl-ok" in r.stdout, r.stdout + r.stderr
