"""Failure paths of the multi-GPU entry points, without a GPU and without a second rank.

The library looks NCCL up through a table of function pointers; blum_comm_selftest fills that table (and the
"has the stream finished" query) with host stubs and plays one scenario through the real entry points
(blum_comm_init_rank, blum_allreduce_sum, ...).  No process is killed and no device is touched: a failure is an error
code from a fake of the failing call, or a completion that never comes."""
import ctypes as C
import time

import pytest

from luminal_b200 import _lib


def _play(scenario, timeout_ms=150):
    lib = _lib.load()
    buf = C.create_string_buffer(512)
    t0 = time.perf_counter()
    rc = lib.blum_comm_selftest(scenario, timeout_ms, buf, 512)
    return rc, buf.value.decode(), (time.perf_counter() - t0) * 1e3


def test_failed_init_is_reported_not_fatal():
    rc, msg, _ = _play(1)
    assert rc == _lib.ERR_COMM and "ncclCommInitRank" in msg and "system error" in msg


def test_a_collective_that_returns_an_error():
    rc, msg, _ = _play(2)
    assert rc == _lib.ERR_COMM and "AllReduce" in msg and "internal error" in msg


def test_a_peer_that_never_arrives_is_timed_out_and_the_communicator_aborted():
    rc, msg, ms = _play(3, timeout_ms=200)
    assert rc == _lib.ERR_COMM, (rc, msg)          # ERR_STATE would mean the aborted communicator misbehaved afterwards
    assert "did not complete within 200 ms" in msg and "aborted" in msg
    assert 180 <= ms < 2000                         # waited for the timeout, and not much longer


def test_a_rank_that_never_joins_the_init():
    rc, msg, ms = _play(4, timeout_ms=200)
    assert rc == _lib.ERR_COMM and "did not complete within 200 ms" in msg
    assert 180 <= ms < 2000


def test_healthy_path_through_the_stubs():
    rc, msg, ms = _play(5)
    assert rc == 0 and msg == "" and ms < 150


@pytest.mark.parametrize("bad", [(0, 100), (6, 100), (3, 0)])
def test_selftest_rejects_bad_arguments(bad):
    assert _lib.load().blum_comm_selftest(bad[0], bad[1], None, 0) == _lib.ERR_INVALID
