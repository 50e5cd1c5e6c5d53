"""CPU restatement (numpy) of the HyperLogLog sketch the reference's offline study uses to estimate the size
of a cluster's shared 32-bit vocabulary (scripts/llama-3-8b/experiment_2.py:31-85 in the Checkers tree).

Test infrastructure only: the product path is checkers_b200.studies (CUDA).  Pinned by
tests/golden/hll_golden.json, which was written from the reference's own functions.

  registers   : 2^14 bytes                                   (experiment_2.py:31-37)
  hash        : MurmurHash3 fmix32 of the 32-bit symbol       (:48-53)
  index       : top 14 bits of the hash                       (:55)
  rank        : leading zeros of ((hash << 14) | 2^13) + 1, clipped to 1..18, kept by maximum   (:58-63)
  merge       : element-wise maximum                          (:66-68)
  count       : alpha m^2 / sum 2^-reg with the small- and large-range corrections              (:71-82)
"""
import numpy as np

HLL_B = 14
HLL_M = 1 << HLL_B
HLL_ALPHA = 0.7213 / (1.0 + 1.079 / HLL_M)


def symbols_of(raw_bytes, elem_size):
    """The 32-bit symbols of a tensor given as bytes: the element's bit pattern, zero-extended."""
    view = {1: np.uint8, 2: np.uint16, 4: np.uint32}[elem_size]
    return np.ascontiguousarray(raw_bytes).view(view).astype(np.uint32)


def fmix32(h):
    h = h.astype(np.uint32).copy()
    h ^= h >> np.uint32(16)
    h *= np.uint32(0x85EBCA6B)
    h ^= h >> np.uint32(13)
    h *= np.uint32(0xC2B2AE35)
    h ^= h >> np.uint32(16)
    return h


def sketch(symbols):
    regs = np.zeros(HLL_M, np.uint8)
    if symbols.size == 0:
        return regs
    with np.errstate(over="ignore"):
        h = fmix32(symbols)
        idx = (h >> np.uint32(32 - HLL_B)).astype(np.int64)
        w = (h << np.uint32(HLL_B)) | np.uint32(1 << (HLL_B - 1))
    # leading zeros of w (never 0): 32 - bit_length
    lz = 31 - np.floor(np.log2(w.astype(np.float64))).astype(np.int64)
    rho = np.clip(lz + 1, 1, 32 - HLL_B).astype(np.uint8)
    np.maximum.at(regs, idx, rho)
    return regs


def merge(sketches):
    return np.stack(sketches).max(axis=0)


def count(regs):
    z = 1.0 / np.sum(np.exp2(-regs.astype(np.float64)))
    raw = HLL_ALPHA * HLL_M * HLL_M * z
    if raw <= 2.5 * HLL_M:
        v = int(np.sum(regs == 0))
        if v > 0:
            raw = HLL_M * np.log(HLL_M / v)
    elif raw > (1.0 / 30.0) * (2 ** 32):
        raw = -(2 ** 32) * np.log(1.0 - raw / 2 ** 32)
    return float(raw)


def shared_histogram_bytes(est_unique):
    """Bytes of a histogram over `est_unique` 32-bit symbols as the study prices it (experiment_2.py:104, 145)."""
    return int(est_unique * 8) + 64
