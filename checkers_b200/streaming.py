"""Chunked compression of HOST-resident state with overlapped copies.

For state that does not live in (or does not fit into) HBM -- the 70B-class
checkpoints streamed through a GPU in ~1 GiB pieces -- the rank's tensors are
cut into chunks; every chunk owns a device staging buffer and a context, and
host threads keep the three engines of the GPU busy at once: while chunk k is
being compressed, chunk k+1 is on its way host->device and the file images of
chunk k-1 are on their way device->host (PCIe is full duplex).  Restore runs
the same way in the other direction.

Each chunk produces a complete triple of reference-format files
(<dir>/part_<k>/rank_<r>_states.ansc, mantissa/..., tables/...), so every
part can be read on its own by anything that reads the reference's layout.
The reference has no counterpart: it compresses device-resident tensors one
by one under a global mutex (src/ANSCompressor.cpp:1204-1280 in the Checkers
tree) and never reads them back.
"""
import os
import threading

from . import _lib
from .context import Context


class HostTensor:
    """One named tensor in pinned host memory (a torch CPU tensor, contiguous)."""

    def __init__(self, name, tensor, dtype_tag):
        if tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"'{name}' must be a contiguous CPU tensor")
        self.name, self.tensor, self.dtype = name, tensor, int(dtype_tag)
        self.nbytes = tensor.numel() * tensor.element_size()
        self.numel = self.nbytes // _lib.ELEM_SIZE[self.dtype]


class _Chunk:
    def __init__(self, index):
        self.index, self.items, self.nbytes = index, [], 0
        self.ctx = self.dev = self.ready = None


def plan_chunks(sizes, chunk_bytes):
    """Cut a sequence of tensor sizes (bytes) into consecutive chunks of at most chunk_bytes;
    a tensor larger than that gets a chunk of its own.  Returns a list of index lists."""
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
    """Fixed set of host tensors <-> compressed parts, through per-chunk device buffers.

    pipeline = ChunkedHostPipeline(host_tensors, device=0, rank=0, chunk_bytes=1 << 30)
    pipeline.compress()            # parts now sit in pinned host memory (pipeline.images(k))
    pipeline.save(directory)       # optional: write every part's three files
    pipeline.restore(out_tensors)  # decode the parts back into host tensors
    """

    def __init__(self, host_tensors, device=0, rank=0, chunk_bytes=1 << 30, workers=2):
        import torch
        self.torch, self.device, self.rank, self.workers = torch, int(device), int(rank), max(1, int(workers))
        self.dev = torch.device("cuda", self.device)
        host_tensors = list(host_tensors)
        self.chunks = []
        for idx in plan_chunks([ht.nbytes for ht in host_tensors], chunk_bytes):
            ch = _Chunk(len(self.chunks))
            ch.items = [host_tensors[i] for i in idx]
            ch.nbytes = sum(ht.nbytes for ht in ch.items)
            self.chunks.append(ch)
        self.copy_in = torch.cuda.Stream(device=self.dev)
        self.copy_out = torch.cuda.Stream(device=self.dev)
        for ch in self.chunks:
            # one staging allocation per chunk; every tensor starts on a 256-byte boundary
            offs, total = staging_offsets([ht.nbytes for ht in ch.items])
            ch.dev = torch.empty(max(total, 1), dtype=torch.uint8, device=self.dev)
            ch.views = [ch.dev[o:o + ht.nbytes] for o, ht in zip(offs, ch.items)]
            ch.ctx = Context(device=self.device, rank=self.rank)
            for ht, v in zip(ch.items, ch.views):
                ch.ctx.register_pointer(ht.name, v.data_ptr(), ht.numel, ht.dtype)
            ch.ready = torch.cuda.Event()
        torch.cuda.synchronize(self.dev)

    # ------------------------------------------------------------------ helpers
    def _run_workers(self, fn):
        """fn(chunk) for every chunk, chunk k on worker k % workers, in order within a worker."""
        errors = []

        def loop(w):
            try:
                self.torch.cuda.set_device(self.dev)
                for ch in self.chunks[w::self.workers]:
                    fn(ch)
            except BaseException as e:  # noqa: BLE001 - re-raised on the calling thread
                errors.append(e)

        threads = [threading.Thread(target=loop, args=(w,)) for w in range(self.workers)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]

    # ------------------------------------------------------------------ compress
    def compress(self):
        """Host tensors -> per-chunk file images in pinned host memory."""
        torch = self.torch
        with torch.cuda.stream(self.copy_in):
            for ch in self.chunks:
                for ht, v in zip(ch.items, ch.views):
                    v.copy_(ht.tensor.view(torch.uint8).reshape(-1), non_blocking=True)
                ch.ready.record(self.copy_in)

        def work(ch):
            ch.ready.synchronize()              # this chunk's bytes are on the device
            ch.ctx.compress(host_images=True)   # kernels + device->host copy of the three images

        self._run_workers(work)

    def images(self, k):
        return [self.chunks[k].ctx.image(i) for i in range(3)]

    def summary(self):
        keys = ("n_tensors", "n_tables", "states_bytes", "mantissa_bytes", "dict_bytes", "original_bytes")
        tot = dict.fromkeys(keys, 0)
        for ch in self.chunks:
            s = ch.ctx.summary()
            for k in keys:
                tot[k] += s[k]
        return tot

    def save(self, directory):
        """Write every part as a reference-format file triple under directory/part_<k>/."""
        tag = f"rank_{max(self.rank, 0)}"
        for ch in self.chunks:
            base = os.path.join(directory, f"part_{ch.index:04d}")
            os.makedirs(os.path.join(base, "mantissa"), exist_ok=True)
            os.makedirs(os.path.join(base, "tables"), exist_ok=True)
            st, mt, dc = (ch.ctx.image(i) for i in range(3))
            st.tofile(os.path.join(base, f"{tag}_states.ansc"))
            mt.tofile(os.path.join(base, "mantissa", f"{tag}_mantissa.mant"))
            dc.tofile(os.path.join(base, "tables", f"{tag}_tables.dict"))
        return len(self.chunks)

    # ------------------------------------------------------------------ restore
    def restore(self, out_tensors):
        """Parts (as left by compress()) -> out_tensors: CPU tensors in the order of the inputs."""
        torch = self.torch
        outs = iter(out_tensors)
        targets = {ch.index: [next(outs) for _ in ch.items] for ch in self.chunks}

        def work(ch):
            ch.ctx.decompress_images(*[ch.ctx.image(i) for i in range(3)])  # host->device copy + decode
            with torch.cuda.stream(self.copy_out):                          # restored bytes back to the host
                for v, o in zip(ch.views, targets[ch.index]):
                    o.view(torch.uint8).reshape(-1).copy_(v, non_blocking=True)

        self._run_workers(work)
        self.copy_out.synchronize()

    def close(self):
        for ch in self.chunks:
            ch.ctx.close()
