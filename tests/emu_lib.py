"""Builds and binds tests/emu/libemu_kernels.so: the library's CUDA kernel source
compiled by g++ behind a one-thread block emulator.  CPU tests use it to check
the kernels' index arithmetic against the oracle; it is never shipped."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EMU_DIR = os.path.join(ROOT, "tests", "emu")
CSRC = os.path.join(ROOT, "checkers_b200", "csrc")
EMU_SO = os.path.join(EMU_DIR, "libemu_kernels.so")

u8p = C.POINTER(C.c_uint8)
u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)


def build_emu():
    srcs = [os.path.join(EMU_DIR, "emu_kernels.cpp"), os.path.join(EMU_DIR, "cuda_emu.hpp"),
            os.path.join(CSRC, "kernels.cuh"), os.path.join(CSRC, "rans_kernels.cuh"),
            os.path.join(CSRC, "tables.hpp")]
    srcs += [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    if not os.path.exists(EMU_SO) or any(os.path.getmtime(EMU_SO) < os.path.getmtime(s) for s in srcs):
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", CSRC, "-I", EMU_DIR, "-shared", "-fPIC", "-w",
                               srcs[0], "-o", EMU_SO])
    return EMU_SO


def aligned(n, align=64, fill=None):
    """uint8 array of n bytes whose data pointer is `align`-byte aligned, with 64 spare bytes after it."""
    raw = np.zeros(n + align + 64, np.uint8)
    off = (-raw.ctypes.data) % align
    a = raw[off:off + n]
    if fill is not None:
        a[:] = fill
    return a


def _p(a, t=u8p):
    return a.ctypes.data_as(t)


class Emu:
    def __init__(self):
        self.lib = C.CDLL(build_emu())
        self.lib.emu_encode.restype = C.c_uint32
        self.lib.emu_stats_out_bytes.restype = C.c_uint32

    def split(self, src, es, spe, grid=3, misalign=0):
        n = src.size
        s = aligned(n + 16)[misalign:misalign + n]
        s[:] = src
        masked = aligned(n)
        side = aligned(n // es * spe if es else 0)
        self.lib.emu_split(_p(s), C.c_uint64(n), C.c_uint32(es), C.c_uint32(spe), _p(masked), _p(side), C.c_uint32(grid))
        return masked, side

    def byte_histogram(self, data, grid=3, misalign=0):
        n = data.size
        s = aligned(n + 16)[misalign:misalign + n]
        s[:] = data
        h = np.zeros(256, np.uint32)
        self.lib.emu_byte_histogram(_p(s), C.c_uint64(n), _p(h, u32p), C.c_uint32(grid))
        return h

    @staticmethod
    def _arrays(tensors):
        n = len(tensors)
        ptrs = (C.c_void_p * n)(*[t.ctypes.data for t in tensors])
        return n, ptrs

    def split_hist(self, tensors, es, spe, need_hist=None, grid=4):
        n, ptrs = self._arrays(tensors)
        nb = np.array([t.size for t in tensors], np.uint64)
        es_a, spe_a = np.array(es, np.uint32), np.array(spe, np.uint32)
        side_total = int(sum(t.size // e * s for t, e, s in zip(tensors, es, spe)))
        side = aligned(side_total)
        hist = np.zeros((n, 256), np.uint32)
        nh = None if need_hist is None else np.array(need_hist, np.uint8)
        self.lib.emu_split_hist(C.c_size_t(n), ptrs, _p(nb, u64p), _p(es_a, u32p), _p(spe_a, u32p),
                                None if nh is None else _p(nh), _p(side), _p(hist, u32p), C.c_uint32(grid))
        return side, hist

    def encode(self, tensors, es, spe, table_idx, nf, cf, grid=3, float_only=False, segments=1):
        n, ptrs = self._arrays(tensors)
        nb = np.array([t.size for t in tensors], np.uint64)
        es_a, spe_a = np.array(es, np.uint32), np.array(spe, np.uint32)
        ti = np.array(table_idx, np.uint32)
        nf = np.ascontiguousarray(nf, np.uint32).reshape(-1, 256)
        cf = np.ascontiguousarray(cf, np.uint32).reshape(-1, 257)
        payload = aligned(int(nb.sum()) + 64)
        poff = np.zeros(n + 1, np.uint64)
        hdrs = np.zeros((n, 256, 4), np.uint32)
        raw = np.zeros(n, np.uint8)
        st = self.lib.emu_encode(C.c_size_t(n), ptrs, _p(nb, u64p), _p(es_a, u32p), _p(spe_a, u32p), _p(ti, u32p),
                                 C.c_size_t(nf.shape[0]), _p(nf, u32p), _p(cf, u32p), _p(payload), _p(poff, u64p),
                                 _p(hdrs, u32p), _p(raw), C.c_uint32(grid), C.c_uint32(int(float_only)), C.c_uint32(segments))
        return payload, poff, hdrs, raw, st

    def encode_fused(self, tensors, es, spe, table_idx, nf, cf, grid=3, float_only=False):
        """The one-kernel path (lanes, zero chain, offsets, gather into a payload heap).  Returns the
        payloads re-packed in tensor order, their offsets, headers and raw flags like encode()."""
        n, ptrs = self._arrays(tensors)
        nb = np.array([t.size for t in tensors], np.uint64)
        es_a, spe_a = np.array(es, np.uint32), np.array(spe, np.uint32)
        ti = np.array(table_idx, np.uint32)
        nf = np.ascontiguousarray(nf, np.uint32).reshape(-1, 256)
        cf = np.ascontiguousarray(cf, np.uint32).reshape(-1, 257)
        heap = aligned(int(nb.sum()) + 32 * n + 64)
        hoff, size = np.zeros(n, np.uint64), np.zeros(n, np.uint64)
        hdrs = np.zeros((n, 256, 4), np.uint32)
        raw = np.zeros(n, np.uint8)
        self.lib.emu_encode_fused(C.c_size_t(n), ptrs, _p(nb, u64p), _p(es_a, u32p), _p(spe_a, u32p), _p(ti, u32p),
                                  C.c_size_t(nf.shape[0]), _p(nf, u32p), _p(cf, u32p), _p(heap), _p(hoff, u64p),
                                  _p(size, u64p), _p(hdrs, u32p), _p(raw), C.c_uint32(grid),
                                  C.c_uint32(int(float_only)))
        assert all(int(o) % 32 == 0 for o in hoff)
        spans = sorted((int(o), int(o) + int(z)) for o, z in zip(hoff, size))
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])), "heap ranges overlap"
        poff = np.zeros(n + 1, np.uint64)
        poff[1:] = np.cumsum(size)
        payload = np.concatenate([heap[int(o):int(o) + int(z)] for o, z in zip(hoff, size)] + [np.zeros(0, np.uint8)])
        return payload, poff, hdrs, raw

    def decode(self, n_bytes, es, spe, table_idx, nf, cf, hdrs, payload, poff, raw, sidecar, check_zero=0, grid=3,
               dst_misalign=0, float_only=False):
        n = len(n_bytes)
        outs = [aligned(int(b) + 16)[dst_misalign:dst_misalign + int(b)] for b in n_bytes]
        ptrs = (C.c_void_p * n)(*[o.ctypes.data for o in outs])
        nb = np.array(n_bytes, np.uint64)
        es_a, spe_a = np.array(es, np.uint32), np.array(spe, np.uint32)
        ti = np.array(table_idx, np.uint32)
        nf = np.ascontiguousarray(nf, np.uint32)
        cf = np.ascontiguousarray(cf, np.uint32)
        hdrs = np.ascontiguousarray(hdrs, np.uint32)
        poff = np.ascontiguousarray(poff, np.uint64)
        raw = np.ascontiguousarray(raw, np.uint8)
        status = np.zeros(n, np.uint32)
        padded = aligned(len(payload) + 128)  # the kernel reads whole 32-byte blocks, up to 63 bytes past the end
        padded[:len(payload)] = np.frombuffer(payload, np.uint8) if not isinstance(payload, np.ndarray) else payload
        payload = padded
        self.lib.emu_decode(C.c_size_t(n), ptrs, _p(nb, u64p), _p(es_a, u32p), _p(spe_a, u32p), _p(ti, u32p),
                            _p(nf, u32p), _p(cf, u32p), _p(hdrs, u32p), _p(payload), _p(poff, u64p), _p(raw),
                            _p(sidecar), C.c_uint32(check_zero), _p(status, u32p), C.c_uint32(grid),
                            C.c_uint32(int(float_only)))
        return outs, status

    def planes(self, tensors, n_elem, es, spe, low_off, plane_off, stride, low, planes, grid=3, merge=False):
        n, ptrs = self._arrays(tensors)
        a = lambda x, t: np.array(x, t)
        ne, e, sp = a(n_elem, np.uint64), a(es, np.uint32), a(spe, np.uint32)
        lo, po, st = a(low_off, np.uint64), a(plane_off, np.uint64), a(stride, np.uint64)
        self.lib.emu_planes(C.c_size_t(n), ptrs, _p(ne, u64p), _p(e, u32p), _p(sp, u32p), _p(lo, u64p), _p(po, u64p),
                            _p(st, u64p), _p(low), _p(planes), C.c_uint32(grid), C.c_uint32(int(merge)))

    def decode_planes(self, planes, dsts, lows, n_elem, payload_off, raw, cf, hdrs, payload, grid=2):
        n = len(dsts)
        dp = (C.c_void_p * n)(*[d.ctypes.data for d in dsts])
        lp = (C.c_void_p * n)(*[l.ctypes.data for l in lows])
        ne = np.array(n_elem, np.uint64)
        po, rw = np.array(payload_off, np.uint64), np.array(raw, np.uint32)
        cf = np.ascontiguousarray(cf, np.uint32)
        hdrs = np.ascontiguousarray(hdrs, np.uint32)
        status = np.zeros(n * planes, np.uint32)
        self.lib.emu_decode_planes(C.c_size_t(n), C.c_uint32(planes), dp, lp, _p(ne, u64p), _p(po, u64p), _p(rw, u32p),
                                   _p(cf, u32p), _p(hdrs, u32p), _p(payload), _p(status, u32p), C.c_uint32(grid))
        return status

    def planes_count(self, tensors, n_elem, es, spe, low_off, plane_off, stride, low, planes, grid=3):
        n, ptrs = self._arrays(tensors)
        a = lambda x, t: np.array(x, t)
        ne, e, sp = a(n_elem, np.uint64), a(es, np.uint32), a(spe, np.uint32)
        lo, po, st = a(low_off, np.uint64), a(plane_off, np.uint64), a(stride, np.uint64)
        hist = np.zeros((int(sum(x - y for x, y in zip(es, spe))), 256), np.uint32)
        self.lib.emu_planes_count(C.c_size_t(n), ptrs, _p(ne, u64p), _p(e, u32p), _p(sp, u32p), _p(lo, u64p), _p(po, u64p),
                                  _p(st, u64p), _p(low), _p(planes), _p(hist, u32p), C.c_uint32(grid))
        return hist

    def model_cost(self, tensors, n_elem, dtypes, capacity, scale_log2, grid=4):
        """vocabulary, largest count, overflow, sum of the quantised counts and bits without the most frequent symbol"""
        n, ptrs = self._arrays(tensors)
        ne, dt = np.array(n_elem, np.uint64), np.array(dtypes, np.uint32)
        out = np.zeros(5, np.float64)
        self.lib.emu_model_cost(C.c_size_t(n), ptrs, _p(ne, u64p), _p(dt, u32p), C.c_uint32(capacity),
                                C.c_double(scale_log2), C.c_uint32(grid), _p(out, C.POINTER(C.c_double)))
        return out

    def hll(self, tensors, n_elem, dtypes, grid=3):
        n, ptrs = self._arrays(tensors)
        ne, dt = np.array(n_elem, np.uint64), np.array(dtypes, np.uint32)
        out = np.zeros((n, 16384), np.uint32)
        self.lib.emu_hll(C.c_size_t(n), ptrs, _p(ne, u64p), _p(dt, u32p), _p(out, u32p), C.c_uint32(grid))
        return out.astype(np.uint8)

    def stats(self, tensors, n_elem, dtypes, bins=256, grid=2, fast=False):
        n, ptrs = self._arrays(tensors)
        ne = np.array(n_elem, np.uint64)
        dt = np.array(dtypes, np.uint32)
        words = self.lib.emu_stats_out_bytes() // 4
        out = np.zeros((n, words), np.uint32)
        fn = self.lib.emu_stats_fast if fast else self.lib.emu_stats
        fn(C.c_size_t(n), ptrs, _p(ne, u64p), _p(dt, u32p), C.c_uint32(bins), _p(out, C.c_void_p), C.c_uint32(grid))
        res = []
        for i in range(n):
            res.append((out[i, :256].copy(), out[i, 256:260].view(np.float32).copy(),
                        out[i, 260:262].view(np.float32).copy(), out[i, 262:267].view(np.float32).copy()))
        return res
