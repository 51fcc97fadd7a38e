"""CPU tests of the all-reduce protocol: host threads play the ranks. Failures
are injected on the host only (a rank that never joins, a late rank, a dropped
flag, stale epochs); nothing here touches a GPU."""
import numpy as np
import pytest

from gcow_b200.codec import ZfpParams
from gcow_b200.comm import allreduce_oracle, protocol_model


def inputs(calls, P, n, seed=0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((calls, P, n)) * 1e-3).astype(np.float32)


@pytest.mark.parametrize("P", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("rate,variant", [(8, "twoshot"), (4, "twoshot"), (16, "twoshot"), (32, "twoshot"),
                                          (8, "oneshot"), (16, "oneshot")])
def test_model_matches_oracle(P, rate, variant):
    n = 4 * 1000 + 3          # tail block, shards not a multiple of the slice
    xs = inputs(2, P, n, seed=P)
    p = ZfpParams.from_rate(rate, 1)
    shift = {1: 0, 2: 1, 4: 2, 8: 3}.get(P, 0)
    outs, status, failed = protocol_model(xs, p.maxbits, variant, ctas=3, shift=shift)
    assert failed == 0 and not status.any()
    for c in range(2):
        ref = allreduce_oracle(xs[c], p, variant, shift)
        for r in range(P):
            assert np.array_equal(outs[c, r].view(np.uint32), ref.view(np.uint32))


def test_many_calls_reuse_parity_regions():
    xs = inputs(7, 4, 4096, seed=5)
    p = ZfpParams.from_rate(8, 1)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=5, shift=2)
    assert failed == 0
    for c in range(7):
        ref = allreduce_oracle(xs[c], p, "twoshot", 2)
        assert all(np.array_equal(outs[c, r], ref) for r in range(4))


def test_small_message_fewer_blocks_than_ranks():
    xs = inputs(1, 8, 5)
    p = ZfpParams.from_rate(8, 1)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, shift=3)
    assert failed == 0
    ref = allreduce_oracle(xs[0], p, "twoshot", 3)
    assert all(np.array_equal(outs[0, r], ref) for r in range(8))


def test_rank_that_never_joins_times_out_everyone():
    xs = inputs(1, 4, 2048)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, timeout_ms=150, fault_call=0, skip_rank=2)
    assert failed == 3                       # the three live ranks
    for r in (0, 1, 3):
        code, phase, peer = status[r, 0], status[r, 1], status[r, 2]
        assert code == 1                     # time-out, not a hang
        assert (phase, peer) in ((1, 2), (2, 2))   # waiting for rank 2's data or its shard
    assert status[2, 0] == 0


def test_late_rank_within_deadline_is_fine():
    xs = inputs(1, 4, 2048)
    p = ZfpParams.from_rate(8, 1)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, timeout_ms=3000, fault_call=0,
                                          delay_rank=1, delay_ms=200, shift=2)
    assert failed == 0
    ref = allreduce_oracle(xs[0], p, "twoshot", 2)
    assert all(np.array_equal(outs[0, r], ref) for r in range(4))


def test_dropped_flag_is_reported_with_phase_and_peer():
    xs = inputs(1, 4, 2048)
    # rank 1's phase-1 flag towards rank 3 is lost
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, timeout_ms=150, fault_call=0,
                                          drop=(1, 3, 0))
    assert failed == 4                       # rank 3 cannot reduce; nobody gets shard 3
    assert tuple(status[3, :3]) == (1, 1, 1)  # time-out in phase "reduce", waiting for rank 1
    for r in (0, 1, 2):
        assert tuple(status[r, :3]) == (1, 2, 3)  # time-out in phase "gather", waiting for rank 3


def test_stale_epochs_are_never_consumed():
    # flags hold an old epoch value: a correct waiter must ignore them
    xs = inputs(2, 2, 1024)
    p = ZfpParams.from_rate(8, 1)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, shift=1, stale_epoch=41)
    assert failed == 0
    for c in range(2):
        ref = allreduce_oracle(xs[c], p, "twoshot", 1)
        assert np.array_equal(outs[c, 0], ref) and np.array_equal(outs[c, 1], ref)


def test_failure_in_one_call_does_not_poison_the_next():
    xs = inputs(3, 2, 1024)
    p = ZfpParams.from_rate(8, 1)
    outs, status, failed = protocol_model(xs, 32, "twoshot", ctas=2, shift=1, timeout_ms=100,
                                          fault_call=0, drop=(0, 1, 0))
    assert failed == 2
    for c in (1, 2):                          # later calls complete and are exact
        ref = allreduce_oracle(xs[c], p, "twoshot", 1)
        assert np.array_equal(outs[c, 0], ref) and np.array_equal(outs[c, 1], ref)


def test_oracle_error_vs_exact_sum():
    P, n = 8, 1 << 14
    xs = inputs(1, P, n)[0]
    exact = xs.astype(np.float64).sum(0) / P
    for rate, lim in ((8, 2e-4), (16, 1e-6)):
        y = allreduce_oracle(xs, ZfpParams.from_rate(rate, 1), "twoshot", 3)
        assert np.sqrt(np.mean((y - exact) ** 2)) < lim


@pytest.mark.parametrize("P", [1, 2, 3, 8])
@pytest.mark.parametrize("bits,tol", [(16, 1e-2), (32, 1e-3), (64, 1e-6), (128, 1e-4)])
def test_sparse_variant_matches_oracle(P, bits, tol):
    """Fixed accuracy with a bit cap: packed codes plus a bitmap per chunk give what the host model gives at the
    same four parameters, for sizes around the chunk and slice bounds."""
    acc = ZfpParams.from_accuracy(tol)
    p = ZfpParams(1, bits, acc.maxprec, acc.minexp)
    rng = np.random.default_rng(bits + P)
    for n in (1, 7, 1023, 4 * 256 * 3 + 5, 70001):
        xs = (rng.standard_normal((1, P, n)) * 1e-3).astype(np.float32)
        xs[:, :, n // 2:] *= np.float32(1e-5)
        for shift in (0, 2):
            outs, status, failed = protocol_model(xs, bits, "sparse", ctas=3, shift=shift, minexp=acc.minexp)
            assert failed == 0
            want = allreduce_oracle(xs[0], p, "twoshot", shift)
            for r in range(P):
                assert np.array_equal(outs[0, r].view(np.uint32), want.view(np.uint32))


def test_sparse_variant_times_out_like_the_others():
    xs = np.zeros((1, 3, 4096), np.float32)
    outs, status, failed = protocol_model(xs, 32, "sparse", ctas=2, timeout_ms=150, fault_call=0, skip_rank=1, minexp=-10)
    assert failed == 2 and status[0, 0] == 1 and status[2, 0] == 1
