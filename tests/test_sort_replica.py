"""sort_replica (csrc/sort_replica.hpp) must leave keys in exactly the order std::sort leaves them in:
the tie order of equal fractions decides which symbols of a frequency table get the rounding slots
(src/ANSCompressor.cpp:469-482 in the Checkers tree).  Also: normalize_tables_kernel, run on the CPU
block emulator, against the host routine on histograms built to hit every branch."""
import ctypes as C

import numpy as np
import pytest

from test_normalize_host import histograms

f64p, i32p, u32p = C.POINTER(C.c_double), C.POINTER(C.c_int32), C.POINTER(C.c_uint32)


def _both(lib, frac):
    frac = np.ascontiguousarray(frac, np.float64)
    a, b = np.zeros(frac.size, np.int32), np.zeros(frac.size, np.int32)
    lib.emu_sort_replica(C.c_size_t(frac.size), frac.ctypes.data_as(f64p), a.ctypes.data_as(i32p))
    lib.emu_std_sort(C.c_size_t(frac.size), frac.ctypes.data_as(f64p), b.ctypes.data_as(i32p))
    return a, b


def test_order_equals_std_sort(emu):
    rng = np.random.default_rng(5)
    for trial in range(20000):
        n = int(rng.integers(1, 257))
        distinct = int(rng.integers(1, [4, 40, 100000][trial % 3]) + 1)
        frac = rng.integers(0, distinct, n) / distinct
        a, b = _both(emu.lib, frac)
        assert np.array_equal(a, b), (trial, n, distinct)


def test_adversarial_inputs_and_heap_sort(emu):
    rng = np.random.default_rng(6)
    for n in (40, 64, 100, 128, 200, 255, 256):
        frac = np.zeros(n, np.float64)
        emu.lib.emu_sort_killer(C.c_size_t(n), frac.ctypes.data_as(f64p))
        for coarse in (1, 3, 7):  # coarser values add ties to the degenerate input
            a, b = _both(emu.lib, np.floor(frac / coarse))
            assert np.array_equal(a, b), (n, coarse)
    for trial in range(5000):
        n = int(rng.integers(1, 257))
        frac = rng.integers(0, int(rng.integers(1, 50)) + 1, n).astype(np.float64)
        a, b = np.zeros(n, np.int32), np.zeros(n, np.int32)
        emu.lib.emu_heap_sort_pair(C.c_size_t(n), frac.ctypes.data_as(f64p), a.ctypes.data_as(i32p), b.ctypes.data_as(i32p))
        assert np.array_equal(a, b), trial


def test_device_normalisation_equals_host(emu, oracle):
    """Every histogram of the host test, all four modes, through normalize_tables_kernel."""
    rng = np.random.default_rng(2024)
    hs = list(histograms(rng))[:600]
    # tensor-like histograms: half zeros, a few exponent values, a flat mantissa byte (the benchmark's shape)
    for i in range(200):
        h = np.zeros(256, np.uint32)
        n = 1 << 20
        h[:] = rng.multinomial(n, np.full(256, 1 / 256))
        e = rng.choice(256, 12, replace=False)
        h[e] += rng.multinomial(n, rng.dirichlet(np.ones(12))).astype(np.uint32)
        h[0] += 2 * n if i % 2 else n
        hs.append(h)
    modes = [(0, False, False), (1, True, False), (3, True, True), (2, False, True)]
    hist = np.ascontiguousarray(np.stack([h for h in hs for _ in modes]), np.uint32)
    flags = np.ascontiguousarray([m[0] for _ in hs for m in modes], np.uint32)
    n = hist.shape[0]
    enc = np.zeros((n, 256, 4), np.uint32)
    freq, cum, sums = np.zeros((n, 256), np.uint32), np.zeros((n, 257), np.uint32), np.zeros(n, np.uint32)
    emu.lib.emu_normalize_tables(C.c_size_t(n), hist.ctypes.data_as(u32p), flags.ctypes.data_as(u32p),
                                 enc.ctypes.data_as(u32p), freq.ctypes.data_as(u32p), cum.ctypes.data_as(u32p),
                                 sums.ctypes.data_as(u32p), C.c_uint32(5))
    k = 0
    for h in hs:
        for _, full, rep in modes:
            nf, cf, _, total = oracle.normalize(h, full, repaired=rep)
            assert np.array_equal(freq[k], nf) and np.array_equal(cum[k], cf) and sums[k] == total, (k, full, rep)
            want = np.zeros((256, 4), np.uint32)
            emu.lib.emu_host_enc_entries(nf.ctypes.data_as(u32p), cf.ctypes.data_as(u32p), want.ctypes.data_as(u32p))
            assert np.array_equal(enc[k], want), k
            k += 1
