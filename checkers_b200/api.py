"""Drop-in front end with the reference module's three functions.

`checkers_py` (src/python_bindings.cpp:17-35 in the Checkers tree) exposes
    initialize_context(model_engine, optimizer=None, histogram_bins=256, background_threads=1)
    analyze_tensors()
    compress_and_save(output_path)
backed by one process-wide registry, called in that order
(examples/FSDP_ZeRO3/train_llama3.py:235-264).  The same names, argument
defaults, call-order rule and error behaviour (exceptions, plus a
"[CHECKERS CRITICAL ERROR]" line on stderr) are kept here; the work is done by
libcheckers_b200.so through its C ABI.  Added beside them, because the
reference has no reader: load_and_decompress(input_path), and register_tensors()
for callers that already hold (name, tensor) pairs and no DeepSpeed engine.
"""
import os
import sys

from . import _lib
from .context import Context, category_of

_ctx = None          # the process-wide context (MemoryManager::instance() in the reference)
_initialized = False


def _env_rank(obj, attr, env):
    v = getattr(obj, attr, None)
    if callable(v):
        v = v()
    if v is None:
        v = os.environ.get(env)
    try:
        return int(v)
    except (TypeError, ValueError):
        return 0


def _fail(where, exc):
    sys.stderr.write(f"[CHECKERS CRITICAL ERROR] {where}{exc}\n")
    raise exc


def current_context():
    return _ctx


def _named_state_tensors(model_engine, optimizer):
    """(name, tensor) pairs in the reference's naming scheme for a plain module +
    Adam-style optimizer: '<p>', 'optimizer.exp_avg::<p>', 'optimizer.exp_avg_sq::<p>'
    (src/api.cpp:583-653 uses the same prefixes for ZeRO-3 flat slices)."""
    if isinstance(model_engine, dict):
        return list(model_engine.items())
    if isinstance(model_engine, (list, tuple)):
        return list(model_engine)
    module = getattr(model_engine, "module", model_engine)
    out = []
    params = list(module.named_parameters())
    opt = optimizer if optimizer is not None else getattr(model_engine, "optimizer", None)
    base = getattr(opt, "optimizer", opt)
    state = getattr(base, "state", None) or {}
    for name, p in params:
        out.append((name, p.data))
        st = state.get(p, None)
        if st:
            if "exp_avg" in st:
                out.append((f"optimizer.exp_avg::{name}", st["exp_avg"]))
            if "exp_avg_sq" in st:
                out.append((f"optimizer.exp_avg_sq::{name}", st["exp_avg_sq"]))
    return out


def initialize_context(model_engine, optimizer=None, histogram_bins=256, background_threads=1):
    """Registers the rank's tensors.  `model_engine` may be an engine/module with
    named_parameters(), or a dict / list of (name, CUDA tensor) pairs.
    `background_threads` is accepted for signature compatibility; registration
    here is a metadata push and needs no worker threads."""
    global _ctx, _initialized
    try:
        if histogram_bins == 0:
            raise RuntimeError("histogram_bins must be greater than zero")
        if background_threads == 0:
            raise RuntimeError("background_threads must be greater than zero")
        rank = _env_rank(model_engine, "global_rank", "RANK")
        local_rank = _env_rank(model_engine, "local_rank", "LOCAL_RANK")
        pairs = _named_state_tensors(model_engine, optimizer)
        device = None
        for _, t in pairs:
            if getattr(t, "is_cuda", False):
                device = t.device.index
                break
        if device is None:
            import torch
            device = torch.cuda.current_device()
        if _ctx is not None:
            _ctx.close()
        _ctx = Context(device=device, rank=rank, local_rank=local_rank)
        _ctx.set_histogram_bins(histogram_bins)
        for name, t in pairs:
            if not getattr(t, "is_cuda", False):
                continue  # no local device storage on this rank
            _ctx.register_tensor(name, t.contiguous() if not t.is_contiguous() else t)
        _initialized = True
    except Exception as e:  # noqa: BLE001 - mirror the reference: report, then re-raise
        _fail("", e)


def register_tensors(pairs, rank=None, device=None, histogram_bins=256):
    """DeepSpeed-free registration: pairs of (name, contiguous CUDA tensor)."""
    initialize_context(list(pairs), None, histogram_bins, 1)
    if rank is not None:
        _ctx.rank = rank


def analyze_tensors():
    try:
        if not _initialized or _ctx is None:
            raise RuntimeError("Context not initialized: MemoryManager logger is null.")
        if _ctx.tensor_count() == 0:
            return
        _ctx.analyze()
    except Exception as e:  # noqa: BLE001
        _fail("", e)


def compress_and_save(output_path):
    try:
        if not _initialized or _ctx is None:
            raise RuntimeError("Context not initialized: call initialize_context first.")
        _ctx.compress_and_save(output_path)
    except Exception as e:  # noqa: BLE001
        _fail("compress_and_save: ", e)


def load_and_decompress(input_path):
    """Restore every registered tensor found in the checkpoint at input_path
    into its registered storage.  Returns the number of tensors restored."""
    try:
        if not _initialized or _ctx is None:
            raise RuntimeError("Context not initialized: call initialize_context first.")
        return _ctx.load_and_decompress(input_path)
    except Exception as e:  # noqa: BLE001
        _fail("load_and_decompress: ", e)
