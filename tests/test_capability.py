"""The device gate of the path: which compute capability a build may run on.

The expectations are the reference's own (the assertions of `test_compute_cap`,
backends/candle/src/compute_cap.rs:53-110, read as data): they pin the oracle's restatement and
the library's C++ rule, which `create` applies to every device it is given.  No GPU needed.
"""
import pytest

from oracle.capability import compute_cap_matching

# (runtime, compile) pairs the reference asserts to match / not to match
REFERENCE_TRUE = [(75, 75), (80, 80), (86, 86), (89, 89), (90, 90), (120, 120), (121, 121), (121, 120),
                  (86, 80), (89, 80), (89, 86)]
REFERENCE_FALSE = [(75, 80), (75, 86), (75, 89), (75, 90),
                   (80, 75), (80, 86), (80, 89), (80, 90),
                   (86, 75), (86, 89), (86, 90),
                   (89, 75), (89, 90),
                   (90, 75), (90, 80), (90, 86), (90, 89),
                   (100, 75), (100, 80), (100, 86), (100, 89), (100, 90),
                   (120, 75), (120, 80), (120, 86), (120, 89), (120, 90), (120, 100),
                   (121, 75), (121, 80), (121, 86), (121, 89), (121, 90), (121, 100)]


def test_oracle_rule_against_the_reference_assertions():
    for r, c in REFERENCE_TRUE:
        assert compute_cap_matching(r, c), (r, c)
    for r, c in REFERENCE_FALSE:
        assert not compute_cap_matching(r, c), (r, c)


def test_library_rule_against_the_reference_assertions_and_the_oracle(lib):
    f = lib.tei_b200_compute_cap_matching
    for r, c in REFERENCE_TRUE:
        assert f(r, c) == 1, (r, c)
    for r, c in REFERENCE_FALSE:
        assert f(r, c) == 0, (r, c)
    for r in range(60, 131):
        for c in range(60, 131):
            assert bool(f(r, c)) == compute_cap_matching(r, c), (r, c)


def test_this_build_runs_on_sm_100_only(lib):
    cap = lib.tei_b200_compile_compute_cap()
    assert cap == 100
    assert [r for r in range(60, 131) if lib.tei_b200_compute_cap_matching(r, cap)] == [100]
