"""Exhaustive interleaving check of the flag-barrier protocol used by the peer-memory kernels."""
from adana_b200.parallel.protocol_model import check


def test_sequence_number_barrier_is_safe_and_live_for_all_interleavings():
    ok, why, n = check(world=2, rounds=3)
    assert ok, why
    ok, why, n = check(world=3, rounds=2)
    assert ok and n > 1000, (why, n)


def test_checker_finds_the_bug_of_a_flag_clearing_variant():
    # clearing one's slots after a barrier loses a fast peer's early arrival for the next one: stuck or unsafe
    ok, why, _ = check(world=2, rounds=2, reset_flags=True)
    assert not ok and why
