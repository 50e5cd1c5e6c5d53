"""The library's host-side table normalisation (csrc/tables.hpp, reached through the C ABI without
touching a GPU) against the oracle's, on histograms built to hit every branch: equal counts in
large groups (equal fractions straddling the cut and not), few symbols, one symbol, full alphabet."""
import numpy as np
import pytest

from oracle_lib import Oracle


@pytest.fixture(scope="module")
def chk():
    try:
        import checkers_b200
    except ImportError as e:  # library not built in this checkout
        pytest.skip(str(e))
    return checkers_b200


def histograms(rng):
    for trial in range(1500):
        kind = trial % 6
        h = np.zeros(256, np.uint32)
        if kind == 0:    # near-uniform with many equal counts (mantissa-like)
            h[:] = 4096 + rng.integers(0, int(rng.integers(1, 40)), 256)
        elif kind == 1:  # a few groups of identical counts
            vals = rng.integers(1, 100000, int(rng.integers(1, 6)))
            h[:] = vals[rng.integers(0, vals.size, 256)]
        elif kind == 2:  # few symbols (exponent-like)
            k = int(rng.integers(1, 12))
            idx = rng.choice(256, k, replace=False)
            h[idx] = rng.integers(1, 10 ** int(rng.integers(1, 7)), k)
        elif kind == 3:  # all equal
            h[:int(rng.integers(1, 257))] = int(rng.integers(1, 1000))
        elif kind == 4:  # geometric with ties in the tail
            h[:] = (2.0 ** -(np.arange(256) // int(rng.integers(1, 9)) / 2.0) * 1e6).astype(np.uint32)
        else:            # random sparse
            k = int(rng.integers(1, 257))
            idx = rng.choice(256, k, replace=False)
            h[idx] = rng.integers(1, 5000, k)
        yield h


def test_library_normalize_equals_oracle(chk):
    oracle = Oracle()
    rng = np.random.default_rng(2024)
    n = 0
    for h in histograms(rng):
        for full in (False, True):
            for rep in (False, True):
                a = chk.normalize_histogram(h, full, rep)
                b = oracle.normalize(h, full, repaired=rep)
                assert all(np.array_equal(x, y) for x, y in zip(a[:3], b[:3])) and a[3] == b[3], (n, full, rep)
        n += 1
