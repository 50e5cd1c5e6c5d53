"""Host arithmetic on HyperLogLog sketches (the device side is Context.hll_sketch_all): merge and count, as
in the reference's offline study of shared histograms (scripts/llama-3-8b/experiment_2.py:66-82 in the
Checkers tree).  Both run in the library (C), on 16 KiB per sketch."""
import ctypes as C

import numpy as np

from ._lib import check, lib

_u8p = C.POINTER(C.c_uint8)


def hll_merge(sketches):
    """Union of sketches: element-wise maximum of the registers."""
    out = np.zeros(16384, np.uint8)
    for s in sketches:
        s = np.ascontiguousarray(s, np.uint8)
        if s.size != 16384:
            raise ValueError("a sketch has 16384 registers")
        check(lib.chk_hll_merge(out.ctypes.data_as(_u8p), s.ctypes.data_as(_u8p)))
    return out


def hll_count(sketch):
    """Estimated number of distinct symbols behind a sketch."""
    s = np.ascontiguousarray(sketch, np.uint8)
    if s.size != 16384:
        raise ValueError("a sketch has 16384 registers")
    est = C.c_double()
    check(lib.chk_hll_count(s.ctypes.data_as(_u8p), C.byref(est)))
    return est.value


def histogram_bytes(estimate):
    """What the study charges for a histogram over `estimate` distinct 32-bit symbols."""
    return int(estimate * 8) + 64
