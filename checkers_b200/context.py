"""Object wrapper over one chk_context (one rank, one GPU)."""
import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import check, lib

_TORCH_DTYPES = None


def _torch_dtype_tag(t):
    """Map a torch dtype to the DataType tag of the file format (the reference's
    parse_dtype, src/api.cpp:887-893, tests "float16" before "bfloat16" and so
    tags bf16 as fp16; tagging it 1 here is deliberate and recorded in the file)."""
    global _TORCH_DTYPES
    import torch
    if _TORCH_DTYPES is None:
        _TORCH_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16,
                         torch.int8: _lib.I8, torch.int32: _lib.I32, torch.uint8: _lib.I8}
    return _TORCH_DTYPES.get(t, _lib.DTYPE_UNKNOWN)


def category_of(name):
    if name.startswith("optimizer.exp_avg_sq::"):
        return _lib.CAT_EXP_AVG_SQ
    if name.startswith("optimizer.exp_avg::"):
        return _lib.CAT_EXP_AVG
    if name.startswith("master_weights::"):
        return _lib.CAT_MASTER
    return _lib.CAT_MODEL


class Context:
    """One rank's registry + compressor.  Tensors are borrowed: keep them alive
    and unchanged until the call that uses them returns."""

    def __init__(self, device=0, rank=0, local_rank=None, workspace_bytes=0):
        """workspace_bytes bounds the encode scratch (0 = one slot per encode team the device can hold)."""
        self._h = C.c_void_p()
        check(lib.chk_context_create_ex(int(device), int(rank), int(rank if local_rank is None else local_rank),
                                        int(workspace_bytes), C.byref(self._h)))
        self.device, self.rank = int(device), int(rank)
        self._keep = []
        self.names = []

    def close(self):
        if self._h:
            lib.chk_context_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- registry
    def reset(self):
        check(lib.chk_reset(self._h))
        self._keep.clear()
        self.names.clear()

    def release_workspace(self):
        """Give the context's device memory back to the device (it is otherwise kept and only grows)."""
        check(lib.chk_release_workspace(self._h))

    def set_histogram_bins(self, bins):
        check(lib.chk_set_histogram_bins(self._h, int(bins)))

    def set_option(self, key, value):
        check(lib.chk_set_option(self._h, key.encode(), int(value)))

    def register_pointer(self, name, ptr, num_elements, dtype, category=None):
        cat = category_of(name) if category is None else category
        check(lib.chk_register_tensor(self._h, name.encode(), C.c_void_p(ptr), int(num_elements), int(dtype), int(cat)))
        self.names.append(name)

    def register_tensor(self, name, tensor, dtype=None):
        """Register a contiguous CUDA torch tensor (kept alive by this object)."""
        if not tensor.is_cuda:
            raise ValueError(f"tensor '{name}' is not on a CUDA device")
        if not tensor.is_contiguous():
            raise ValueError(f"tensor '{name}' is not contiguous")
        tag = _torch_dtype_tag(tensor.dtype) if dtype is None else dtype
        self._keep.append(tensor)
        self.register_pointer(name, tensor.data_ptr() if tensor.numel() else 0, tensor.numel(), tag)

    def tensor_count(self):
        n = C.c_uint64()
        check(lib.chk_tensor_count(self._h, C.byref(n)))
        return n.value

    # ---- analysis
    def analyze(self):
        check(lib.chk_analyze(self._h))

    # ---- vocabulary sketches (the reference's offline study of shared histograms)
    def hll_sketch_all(self):
        """One HyperLogLog sketch (2^14 registers over the 32-bit symbols) per registered tensor, on the device."""
        check(lib.chk_hll_sketch_all(self._h))

    def hll_sketch(self, index):
        regs = np.zeros(16384, np.uint8)
        check(lib.chk_hll_get(self._h, int(index), regs.ctypes.data_as(C.POINTER(C.c_uint8))))
        return regs

    def shared_model_cost(self, indices):
        """(stream bytes, vocabulary size) of the registered tensors `indices` coded under one shared model over
        their 32-bit symbols, as the reference's study prices it; one index = the tensor's own model."""
        idx = np.ascontiguousarray(indices, dtype=np.uint64)
        b, v = C.c_double(), C.c_uint64()
        check(lib.chk_shared_model_cost(self._h, idx.ctypes.data_as(C.POINTER(C.c_uint64)), idx.size, C.byref(b),
                                        C.byref(v)))
        return b.value, v.value

    def shared_vocabulary_report(self):
        """(bytes of per-tensor histograms, bytes with one histogram per current cluster), as the study prices them."""
        a, b = C.c_uint64(), C.c_uint64()
        check(lib.chk_shared_vocabulary_report(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def tensor_stats(self, index):
        hist = np.zeros(256, np.uint32)
        mom, mm, fp = np.zeros(4, np.float32), np.zeros(2, np.float32), np.zeros(5, np.float32)
        f32p = C.POINTER(C.c_float)
        check(lib.chk_get_tensor_stats(self._h, int(index), hist.ctypes.data_as(C.POINTER(C.c_uint32)),
                                       mom.ctypes.data_as(f32p), mm.ctypes.data_as(f32p), fp.ctypes.data_as(f32p)))
        return hist, mom, mm, fp

    def cluster_ids(self):
        n = self.tensor_count()
        ids = np.zeros(max(n, 1), np.int32)
        k = C.c_int32()
        check(lib.chk_get_cluster_ids(self._h, ids.ctypes.data_as(C.POINTER(C.c_int32)), n, C.byref(k)))
        return ids[:n].copy(), k.value

    def cluster_anchor(self, cluster):
        buf = C.create_string_buffer(256)
        check(lib.chk_get_cluster_anchor(self._h, int(cluster), buf))
        return buf.value.decode()

    def set_cluster_info(self, names, ids, anchor_names):
        n = len(names)
        nm = (C.c_char_p * max(n, 1))(*[s.encode() for s in names])
        idv = (C.c_int32 * max(n, 1))(*[int(i) for i in ids])
        k = len(anchor_names)
        an = (C.c_char_p * max(k, 1))(*[s.encode() for s in anchor_names])
        check(lib.chk_set_cluster_info(self._h, n, nm, idv, k, an))

    # ---- codec
    def compress_and_save(self, output_dir):
        check(lib.chk_compress_and_save(self._h, os.fspath(output_dir).encode()))

    def compress(self, host_images=False):
        check(lib.chk_compress(self._h, 1 if host_images else 0))

    def image(self, which):
        """The file image (0 states, 1 mantissa, 2 tables) as a uint8 numpy view
        of pinned host memory owned by the context (valid until the next compress)."""
        p, n = C.c_void_p(), C.c_uint64()
        check(lib.chk_get_image(self._h, int(which), C.byref(p), C.byref(n)))
        if n.value == 0:
            return np.zeros(0, np.uint8)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,))

    def summary(self):
        s = _lib.Summary()
        check(lib.chk_get_summary(self._h, C.byref(s)))
        return {k: getattr(s, k) for k, _ in _lib.Summary._fields_}

    def table_report(self):
        """(tables of the last compression, how many of them do not sum to 4096 and cannot be decoded)."""
        n, bad = C.c_uint64(), C.c_uint64()
        check(lib.chk_get_table_report(self._h, C.byref(n), C.byref(bad)))
        return n.value, bad.value

    def load_and_decompress(self, input_dir):
        check(lib.chk_load_and_decompress(self._h, os.fspath(input_dir).encode()))
        return self.restored_count()

    def decompress_images(self, states, mantissa, tables):
        a = [np.ascontiguousarray(x, np.uint8) for x in (states, mantissa, tables)]
        check(lib.chk_decompress_images(self._h, a[0].ctypes.data, a[0].size, a[1].ctypes.data, a[1].size,
                                        a[2].ctypes.data, a[2].size))
        return self.restored_count()

    def decompress_resident(self, dst_ptrs=None):
        if dst_ptrs is None:
            check(lib.chk_decompress_resident(self._h, None))
        else:
            # one pointer per registered tensor (0 = skip); a uint64 numpy array is passed as is
            arr = np.ascontiguousarray(dst_ptrs, dtype=np.uint64)
            check(lib.chk_decompress_resident(self._h, arr.ctypes.data_as(C.POINTER(C.c_void_p))))
        return self.restored_count()

    def restored_count(self):
        n = C.c_uint64()
        check(lib.chk_restored_count(self._h, C.byref(n)))
        return n.value

    # ---- stages
    def split(self, src_ptr, num_elements, dtype, masked_ptr, sidecar_ptr):
        check(lib.chk_split(self._h, C.c_void_p(src_ptr), int(num_elements), int(dtype), C.c_void_p(masked_ptr),
                            C.c_void_p(sidecar_ptr)))

    def merge(self, masked_ptr, sidecar_ptr, num_elements, dtype, out_ptr):
        check(lib.chk_merge(self._h, C.c_void_p(masked_ptr), C.c_void_p(sidecar_ptr), int(num_elements), int(dtype),
                            C.c_void_p(out_ptr)))

    def byte_histogram(self, ptr, n_bytes):
        h = np.zeros(256, np.uint32)
        check(lib.chk_byte_histogram(self._h, C.c_void_p(ptr), int(n_bytes), h.ctypes.data_as(C.POINTER(C.c_uint32))))
        return h

    def timing(self, key):
        v = C.c_double()
        check(lib.chk_get_timing(self._h, key.encode(), C.byref(v)))
        return v.value

    def stream_handle(self):
        """cudaStream_t of this context as an integer (usable with torch.cuda.ExternalStream)."""
        p = C.c_void_p()
        check(lib.chk_get_stream(self._h, C.byref(p)))
        return p.value or 0

    def kernel_launches(self):
        n = C.c_uint64()
        check(lib.chk_kernel_launches(self._h, C.byref(n)))
        return n.value


STATIC_MAX_TENSOR_BYTES = 4 << 20


def encode_tensor_static(src_ptr, num_elements, dtype, norm_freq, cum_freq, payload_ptr, lane_headers_ptr, stream=0):
    """Encode one tensor using only the fixed scratch region built into the library:
    nothing is allocated on the device or in pinned memory, so it is safe where the
    allocator must not be touched (HBM full at checkpoint time, memory owned by another
    framework).  Limited to STATIC_MAX_TENSOR_BYTES per tensor; calls on one GPU must
    not overlap.  Returns (payload_size, is_raw)."""
    nf = np.ascontiguousarray(norm_freq, np.uint32)
    cf = np.ascontiguousarray(cum_freq, np.uint32)
    size, raw = C.c_uint64(), C.c_int()
    u32p = C.POINTER(C.c_uint32)
    check(lib.chk_encode_tensor_static(C.c_void_p(src_ptr), int(num_elements), int(dtype), nf.ctypes.data_as(u32p),
                                       cf.ctypes.data_as(u32p), C.c_void_p(payload_ptr), C.c_void_p(lane_headers_ptr),
                                       C.byref(size), C.byref(raw), C.c_void_p(stream)))
    return size.value, bool(raw.value)


def normalize_histogram(hist, ensure_full_alphabet=False, repair=False):
    """Host table normalisation (no device involved).  Returns (norm_freq, cum_freq, x_max, sum)."""
    hist = np.ascontiguousarray(hist, np.uint32)
    nf, cf, xm = np.zeros(256, np.uint32), np.zeros(257, np.uint32), np.zeros(256, np.uint32)
    s = C.c_uint32()
    u32p = C.POINTER(C.c_uint32)
    check(lib.chk_normalize_histogram(hist.ctypes.data_as(u32p), int(ensure_full_alphabet), int(repair),
                                      nf.ctypes.data_as(u32p), cf.ctypes.data_as(u32p), xm.ctypes.data_as(u32p),
                                      C.byref(s)))
    return nf, cf, xm, s.value
