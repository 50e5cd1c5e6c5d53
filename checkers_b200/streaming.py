"""Chunked compression of HOST-resident state with overlapped copies: the Python face of the
chk_stream_* entry points (include/checkers_b200.h).

For state that does not live in (or does not fit into) HBM -- the 70B-class checkpoints streamed
through a GPU in ~1 GiB pieces -- the rank's tensors are cut into consecutive parts; a few device
staging buffers and contexts ("slots") are shared by all parts, and the library keeps the three
engines of the GPU busy at once: while part k is being compressed, part k+1 is on its way
host->device and the file images of part k-1 are on their way device->host (PCIe is full duplex).
Restore runs the same way in the other direction.  The loop over parts, its threads, streams and
events live in the C++ library; this module only hands over pointers.

Each part is a complete triple of reference-format files
(<dir>/part_<k>/rank_<r>_states.ansc, mantissa/..., tables/...), so every part can be read on its
own by anything that reads the reference's layout.  The reference has no counterpart: it compresses
device-resident tensors one by one under a global mutex (src/ANSCompressor.cpp:1204-1280 in the
Checkers tree) and never reads them back.
"""
import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import check, lib


class HostTensor:
    """One named tensor in (preferably pinned) host memory: a contiguous torch CPU tensor."""

    def __init__(self, name, tensor, dtype_tag):
        if tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"'{name}' must be a contiguous CPU tensor")
        self.name, self.tensor, self.dtype = name, tensor, int(dtype_tag)
        self.nbytes = tensor.numel() * tensor.element_size()
        self.numel = self.nbytes // _lib.ELEM_SIZE[self.dtype]


class _Part:
    def __init__(self, index, items):
        self.index, self.items = index, items
        self.nbytes = sum(t.nbytes for t in items)


def plan_chunks(sizes, chunk_bytes):
    """Cut a sequence of tensor sizes (bytes) into consecutive chunks of at most chunk_bytes;
    a tensor larger than that gets a chunk of its own.  Returns a list of index lists.
    (The library cuts the same way; this copy serves planning without a GPU.)"""
    chunks, cur, cur_bytes = [], [], 0
    for i, n in enumerate(sizes):
        if cur and cur_bytes + n > chunk_bytes:
            chunks.append(cur)
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += n
    if cur:
        chunks.append(cur)
    return chunks


def staging_offsets(sizes, align=256):
    """Offsets of a chunk's tensors inside its staging buffer (each aligned) and the buffer size."""
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + align - 1) & ~(align - 1)
    return offs, total


class ChunkedHostPipeline:
    """Fixed set of host tensors <-> compressed parts, through a few device staging slots.

    pipeline = ChunkedHostPipeline(host_tensors, device=0, rank=0, chunk_bytes=1 << 30)
    pipeline.compress()            # parts now sit in pinned host memory (pipeline.images(k))
    pipeline.save(directory)       # optional: write every part's three files
    pipeline.restore(out_tensors)  # decode the parts back into host tensors
    """

    def __init__(self, host_tensors, device=0, rank=0, chunk_bytes=1 << 30, workers=3, options=None):
        """options: library options (as Context.set_option) for every context of the pipeline, e.g.
        {"format_version": 3}."""
        self.tensors = list(host_tensors)
        self.device, self.rank = int(device), int(rank)
        self._h = C.c_void_p()
        check(lib.chk_stream_create(self.device, self.rank, int(chunk_bytes), max(1, min(int(workers), 8)),
                                    C.byref(self._h)))
        for key, value in (options or {}).items():
            check(lib.chk_stream_set_option(self._h, str(key).encode(), int(value)))
        for t in self.tensors:
            check(lib.chk_stream_add_tensor(self._h, t.name.encode(), C.c_void_p(t.tensor.data_ptr()), t.numel, t.dtype))
        n = C.c_uint64()
        check(lib.chk_stream_part_count(self._h, C.byref(n)))
        self.chunks = []
        for k in range(n.value):
            first, cnt = C.c_uint64(), C.c_uint64()
            check(lib.chk_stream_part_info(self._h, k, C.byref(first), C.byref(cnt)))
            self.chunks.append(_Part(k, self.tensors[first.value:first.value + cnt.value]))

    def compress(self):
        """Host tensors -> per-part file images in pinned host memory."""
        check(lib.chk_stream_compress(self._h))

    def images(self, k):
        """The three file images of part k as uint8 numpy views (valid until the next compress)."""
        out = []
        for which in range(3):
            p, n = C.c_void_p(), C.c_uint64()
            check(lib.chk_stream_get_image(self._h, int(k), which, C.byref(p), C.byref(n)))
            out.append(np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,)) if n.value
                       else np.zeros(0, np.uint8))
        return out

    def summary(self):
        s = _lib.Summary()
        check(lib.chk_stream_get_summary(self._h, C.byref(s)))
        return {k: getattr(s, k) for k, _ in _lib.Summary._fields_}

    def save(self, directory):
        """Write every part as a reference-format file triple under directory/part_<k>/."""
        check(lib.chk_stream_save(self._h, os.fspath(directory).encode()))
        return len(self.chunks)

    def load(self, directory):
        """Read the parts written by save() back (restore() then decodes them)."""
        check(lib.chk_stream_load(self._h, os.fspath(directory).encode()))

    def restore(self, out_tensors=None):
        """Parts (as left by compress() or load()) -> out_tensors: CPU tensors in the order of the
        inputs (None: back into the input tensors)."""
        if out_tensors is None:
            check(lib.chk_stream_restore(self._h, None))
            return
        outs = list(out_tensors)
        if len(outs) != len(self.tensors):
            raise ValueError("one output tensor per input tensor")
        arr = (C.c_void_p * max(len(outs), 1))(*[o.data_ptr() for o in outs])
        check(lib.chk_stream_restore(self._h, arr))

    def timing(self, key):
        v = C.c_double()
        check(lib.chk_stream_get_timing(self._h, key.encode(), C.byref(v)))
        return v.value

    def close(self):
        if self._h:
            lib.chk_stream_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
