"""ctypes bindings for the CPU oracle (oracle/liboracle.so) and, when it has been
built, the reference-text harness (oracle/_ref/libcheckers_ref.so).

Test infrastructure: imported by tests, by the smoke check and by the CPU
baseline leg of the benchmark only.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libcheckers_ref.so")
REF_REPAIR_CLI = os.path.join(ORACLE_DIR, "_ref", "tensor_group_prefix_mask_repair")

F32, BF16, F16, I8, I32, UNKNOWN = 0, 1, 2, 3, 4, 255
ELEM_SIZE = {F32: 4, BF16: 2, F16: 2, I8: 1, I32: 4}
SIDECAR_PER_ELEM = {F32: 2, BF16: 1, F16: 1, I8: 0, I32: 0}
INT32_MIN = -(2 ** 31)

u8p = C.POINTER(C.c_uint8)
u32p = C.POINTER(C.c_uint32)
f32p = C.POINTER(C.c_float)


def build_oracle(force=False):
    src = os.path.join(ORACLE_DIR, "checkers_oracle.cpp")
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
                               src, "-o", ORACLE_SO])
    return ORACLE_SO


def _p(a, t=u8p):
    return a.ctypes.data_as(t)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


class Oracle:
    """The restatement in oracle/checkers_oracle.cpp."""

    def __init__(self):
        self.lib = C.CDLL(build_oracle())
        L = self.lib
        L.orc_normalize.restype = C.c_uint32
        L.orc_normalize_repaired.restype = C.c_uint32
        L.orc_encode_lane.restype = C.c_uint32
        L.orc_compress_tensor.restype = C.c_size_t
        L.orc_decode_tensor.restype = C.c_int
        L.orc_build_clusters.restype = C.c_int
        L.orc_compress_and_save.restype = C.c_int
        L.orc_load_tensor.restype = C.c_int64
        L.orc_list_tensors.restype = C.c_int64

    def split(self, raw, dtype):
        raw = _u8(raw)
        es, spe = ELEM_SIZE[dtype], SIDECAR_PER_ELEM[dtype]
        n = raw.size // es
        masked = np.empty(n * es, np.uint8)
        side = np.empty(n * spe, np.uint8)
        self.lib.orc_split(_p(raw), C.c_size_t(n), C.c_uint32(es), C.c_uint32(spe), _p(masked), _p(side))
        return masked, side

    def byte_histogram(self, data):
        data = _u8(data)
        h = np.zeros(256, np.uint32)
        self.lib.orc_byte_histogram(_p(data), C.c_size_t(data.size), _p(h, u32p))
        return h

    def normalize(self, hist, full=False, repaired=False):
        hist = np.ascontiguousarray(hist, np.uint32)
        nf, cf, xm = np.zeros(256, np.uint32), np.zeros(257, np.uint32), np.zeros(256, np.uint32)
        fn = self.lib.orc_normalize_repaired if repaired else self.lib.orc_normalize
        s = fn(_p(hist, u32p), C.c_int(int(full)), _p(nf, u32p), _p(cf, u32p), _p(xm, u32p))
        return nf, cf, xm, int(s)

    def compress_tensor(self, data, nf, cf, xm, threads=0):
        data = _u8(data)
        B = data.size
        cap = max(((B + 255) // 256) * 2 * 256, B, 1)
        out = np.empty(cap, np.uint8)
        hdr = np.zeros(1024, np.uint32)
        raw = C.c_int(0)
        sz = self.lib.orc_compress_tensor(_p(data), C.c_size_t(B), _p(nf, u32p), _p(cf, u32p), _p(xm, u32p),
                                          _p(hdr, u32p), _p(out), C.byref(raw), C.c_int(threads))
        return out[:sz].copy(), hdr.reshape(256, 4), bool(raw.value)

    def decode_tensor(self, payload, headers, is_raw, nf, cf, n_bytes, threads=0):
        payload = np.ascontiguousarray(payload, np.uint8)
        headers = np.ascontiguousarray(headers, np.uint32)
        out = np.empty(n_bytes, np.uint8)
        rc = self.lib.orc_decode_tensor(_p(payload), C.c_size_t(payload.size), _p(headers, u32p), C.c_int(int(is_raw)),
                                        _p(nf, u32p), _p(cf, u32p), C.c_size_t(n_bytes), _p(out), C.c_int(threads))
        return rc, out

    def merge(self, masked, side, dtype):
        es, spe = ELEM_SIZE[dtype], SIDECAR_PER_ELEM[dtype]
        n = masked.size // es
        out = np.empty(n * es, np.uint8)
        self.lib.orc_merge(_p(masked), _p(side), C.c_size_t(n), C.c_uint32(es), C.c_uint32(spe), _p(out))
        return out

    def tensor_stats(self, raw, dtype, bins=256):
        raw = _u8(raw)
        n = raw.size // ELEM_SIZE[dtype]
        hist = np.zeros(256, np.uint32)
        mom = np.zeros(4, np.float32)
        mm = np.zeros(2, np.float32)
        self.lib.orc_tensor_stats(_p(raw, C.c_void_p), C.c_size_t(n), C.c_int(dtype), C.c_uint32(bins),
                                  _p(hist, u32p), _p(mom, f32p), _p(mm, f32p))
        return hist, mom, mm

    def build_clusters(self, names, fps):
        n = len(names)
        fps = np.ascontiguousarray(fps, np.float32).reshape(n, 5)
        arr = (C.c_char_p * n)(*[s.encode() for s in names])
        cid = np.zeros(max(n, 1), np.int32)
        anchor = np.full(max(n, 1), -1, np.int32)
        k = self.lib.orc_build_clusters(C.c_size_t(n), arr, _p(fps, f32p), _p(cid, C.POINTER(C.c_int)),
                                        _p(anchor, C.POINTER(C.c_int)))
        return cid[:n].copy(), anchor[:k].copy()

    def compress_and_save(self, names, arrays, dtypes, out_dir, rank=0, cluster_id=None, anchor_names=None,
                          repair_tables=False, threads=0):
        n = len(names)
        keep = [None if a is None else _u8(a) for a in arrays]
        nm = (C.c_char_p * n)(*[s.encode() for s in names])
        ptrs = (C.c_void_p * n)(*[None if a is None or a.size == 0 else a.ctypes.data for a in keep])
        ne = np.array([0 if a is None else a.size // max(ELEM_SIZE.get(d, 1), 1) for a, d in zip(keep, dtypes)],
                      np.uint64)
        dt = np.array(dtypes, np.uint8)
        cid = None if cluster_id is None else np.ascontiguousarray(cluster_id, np.int32)
        an = anchor_names or []
        anc = (C.c_char_p * max(len(an), 1))(*[s.encode() for s in an]) if an else None
        rc = self.lib.orc_compress_and_save(C.c_size_t(n), nm, ptrs, _p(ne, C.POINTER(C.c_uint64)), _p(dt),
                                            None if cid is None else _p(cid, C.POINTER(C.c_int32)),
                                            C.c_int(len(an)), anc, C.c_int(rank), out_dir.encode(),
                                            C.c_int(int(repair_tables)), C.c_int(threads))
        if rc != 0:
            raise RuntimeError(f"orc_compress_and_save rc={rc}")

    def roundtrip_timed(self, arrays, dtypes, threads=0):
        """CPU baseline leg: returns (compress_s, decompress_s, original, payload, sidecar bytes)."""
        n = len(arrays)
        keep = [_u8(a) for a in arrays]
        ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in keep])
        ne = np.array([a.size // ELEM_SIZE[d] for a, d in zip(keep, dtypes)], np.uint64)
        dt = np.array(dtypes, np.uint8)
        secs = (C.c_double * 2)()
        nbytes = (C.c_uint64 * 3)()
        self.lib.orc_roundtrip_timed.restype = C.c_int
        rc = self.lib.orc_roundtrip_timed(C.c_size_t(n), ptrs, _p(ne, C.POINTER(C.c_uint64)), _p(dt), C.c_int(threads),
                                          secs, nbytes)
        if rc != 0:
            raise RuntimeError("oracle round trip did not reproduce its input")
        return secs[0], secs[1], nbytes[0], nbytes[1], nbytes[2]

    def list_tensors(self, d, rank=0):
        n = self.lib.orc_list_tensors(d.encode(), C.c_int(rank), None, C.c_size_t(0))
        if n < 0:
            raise RuntimeError(f"orc_list_tensors rc={n}")
        buf = C.create_string_buffer(int(n) * 256 + 1)
        self.lib.orc_list_tensors(d.encode(), C.c_int(rank), buf, C.c_size_t(n))
        return [buf.raw[i * 256:(i + 1) * 256].split(b"\0")[0].decode() for i in range(int(n))]

    def load_tensor(self, d, name, cap, rank=0):
        out = np.empty(cap, np.uint8)
        rc = self.lib.orc_load_tensor(d.encode(), C.c_int(rank), name.encode(), _p(out), C.c_size_t(cap))
        if rc < 0:
            raise RuntimeError(f"orc_load_tensor({name}) rc={rc}")
        return out[:rc]


class RefShim:
    """Reference function text compiled for the CPU (oracle/_ref)."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        self.lib = C.CDLL(REF_SO)
        self.lib.ref_normalize.restype = C.c_uint32
        self.lib.ref_encode_compact.restype = C.c_size_t
        self.lib.ref_build_clusters.restype = C.c_int

    def split(self, raw, dtype):
        raw = _u8(raw)
        es, spe = ELEM_SIZE[dtype], SIDECAR_PER_ELEM[dtype]
        n = raw.size // es
        masked = np.empty(n * es, np.uint8)
        side = np.empty(n * spe, np.uint8)
        self.lib.ref_split(_p(raw), C.c_size_t(n), C.c_uint32(es), C.c_uint32(spe), _p(masked), _p(side))
        return masked, side

    def byte_histogram(self, data):
        data = _u8(data)
        h = np.zeros(256, np.uint32)
        self.lib.ref_byte_histogram(_p(data), C.c_size_t(data.size), _p(h, u32p))
        return h

    def normalize(self, hist, full=False):
        hist = np.ascontiguousarray(hist, np.uint32)
        nf, cf, xm = np.zeros(256, np.uint32), np.zeros(257, np.uint32), np.zeros(256, np.uint32)
        s = self.lib.ref_normalize(_p(hist, u32p), C.c_int(int(full)), _p(nf, u32p), _p(cf, u32p), _p(xm, u32p))
        return nf, cf, xm, int(s)

    def encode_compact(self, data, nf, cf, xm):
        data = _u8(data)
        B = data.size
        out = np.empty(max(((B + 255) // 256) * 2 * 256, 1), np.uint8)
        hdr = np.zeros(1024, np.uint32)
        sz = self.lib.ref_encode_compact(_p(data), C.c_size_t(B), _p(nf, u32p), _p(cf, u32p), _p(xm, u32p),
                                         _p(hdr, u32p), _p(out))
        return out[:sz].copy(), hdr.reshape(256, 4)

    def tensor_stats(self, raw, dtype, bins=256):
        raw = _u8(raw).copy()
        n = raw.size // ELEM_SIZE[dtype]
        hist = np.zeros(256, np.uint32)
        mom = np.zeros(4, np.float32)
        mm = np.zeros(2, np.float32)
        self.lib.ref_tensor_stats(_p(raw, C.c_void_p), C.c_size_t(n), C.c_int(dtype), C.c_uint32(bins),
                                  _p(hist, u32p), _p(mom, f32p), _p(mm, f32p))
        return hist, mom, mm

    def build_clusters(self, names, fps):
        n = len(names)
        fps = np.ascontiguousarray(fps, np.float32).reshape(n, 5)
        arr = (C.c_char_p * n)(*[s.encode() for s in names])
        cid = np.zeros(max(n, 1), np.int32)
        anchor = np.full(max(n, 1), -1, np.int32)
        k = self.lib.ref_build_clusters(C.c_size_t(n), arr, _p(fps, f32p), _p(cid, C.POINTER(C.c_int)),
                                        _p(anchor, C.POINTER(C.c_int)))
        return cid[:n].copy(), anchor[:k].copy()

    def write_states(self, path, rank, entries):
        """entries: dicts name,dtype,original_bytes,num_elements,owns,anchor,lanes(256x4 u32),payload(u8)."""
        n = len(entries)
        nm = (C.c_char_p * n)(*[e["name"].encode() for e in entries])
        an = (C.c_char_p * n)(*[e["anchor"].encode() for e in entries])
        dt = np.array([e["dtype"] for e in entries], np.uint8)
        ob = np.array([e["original_bytes"] for e in entries], np.uint64)
        ne = np.array([e["num_elements"] for e in entries], np.uint64)
        ow = np.array([e["owns"] for e in entries], np.uint8)
        lanes = np.ascontiguousarray(np.stack([e["lanes"] for e in entries]).astype(np.uint32))
        keep = [np.ascontiguousarray(e["payload"], np.uint8) for e in entries]
        pp = (C.c_void_p * n)(*[k.ctypes.data for k in keep])
        ps = np.array([k.size for k in keep], np.uint64)
        u64p = C.POINTER(C.c_uint64)
        rc = self.lib.ref_write_states(path.encode(), C.c_int(rank), C.c_size_t(n), nm, _p(dt), _p(ob, u64p),
                                       _p(ne, u64p), _p(ow), an, _p(lanes, u32p), pp, _p(ps, u64p))
        assert rc == 0

    def write_mantissa(self, path, rank, entries):
        n = len(entries)
        nm = (C.c_char_p * n)(*[e["name"].encode() for e in entries])
        dt = np.array([e["dtype"] for e in entries], np.uint8)
        ne = np.array([e["num_elements"] for e in entries], np.uint64)
        sp = np.array([e["spe"] for e in entries], np.uint8)
        keep = [np.ascontiguousarray(e["sidecar"], np.uint8) for e in entries]
        pp = (C.c_void_p * n)(*[k.ctypes.data for k in keep])
        ps = np.array([k.size for k in keep], np.uint64)
        u64p = C.POINTER(C.c_uint64)
        rc = self.lib.ref_write_mantissa(path.encode(), C.c_int(rank), C.c_size_t(n), nm, _p(dt), _p(ne, u64p),
                                         _p(sp), pp, _p(ps, u64p))
        assert rc == 0

    def write_tables(self, path, rank, names, nf, cf):
        n = len(names)
        nm = (C.c_char_p * n)(*[s.encode() for s in names])
        nf = np.ascontiguousarray(nf, np.uint32)
        cf = np.ascontiguousarray(cf, np.uint32)
        rc = self.lib.ref_write_tables(path.encode(), C.c_int(rank), C.c_size_t(n), nm, _p(nf, u32p), _p(cf, u32p))
        assert rc == 0


# ---------------------------------------------------------------- synthetic state tensors
def to_bf16_bits(x32):
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    b = np.ascontiguousarray(x32, np.float32).view(np.uint32)
    rounded = b + (np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def synth(kind, n, seed):
    """Seeded synthetic tensors with the distributions the benchmark configs name.
    Returns (uint8 view of the bytes, dtype tag)."""
    rng = np.random.default_rng(seed)
    if kind == "bf16_weight":
        return to_bf16_bits(rng.normal(0, 0.02, n).astype(np.float32)).view(np.uint8), BF16
    if kind == "bf16_norm_gain":
        return to_bf16_bits((1.0 + rng.normal(0, 1e-3, n)).astype(np.float32)).view(np.uint8), BF16
    if kind == "f32_master":
        return rng.normal(0, 0.02, n).astype(np.float32).view(np.uint8), F32
    if kind == "f32_exp_avg":
        return rng.normal(0, 1e-4, n).astype(np.float32).view(np.uint8), F32
    if kind == "f32_exp_avg_sq":
        return (rng.normal(0, 1e-3, n).astype(np.float32) ** 2 + np.float32(1e-12)).view(np.uint8), F32
    if kind == "f32_exp_avg_sq_lognormal":
        return rng.lognormal(-18.0, 2.0, n).astype(np.float32).view(np.uint8), F32
    if kind == "f16_weight":
        return rng.normal(0, 0.02, n).astype(np.float16).view(np.uint8), F16
    if kind == "i8":
        return rng.integers(-128, 128, n, dtype=np.int8).view(np.uint8), I8
    if kind == "i32":
        return rng.integers(-1000, 1000, n, dtype=np.int32).view(np.uint8), I32
    if kind == "f32_uniform_bits":
        return rng.integers(0, 2 ** 32, n, dtype=np.uint32).view(np.uint8), F32
    raise ValueError(kind)
