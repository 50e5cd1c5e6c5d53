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


def _master_of(optimizer):
    """Map id(model parameter) -> fp32 master tensor for the usual mixed-precision wrappers.

    The reference reads DeepSpeed ZeRO-3's flat fp32 partitions (src/api.cpp:416-685, submitted as
    'master_weights::<p>', :614-625).  Without DeepSpeed the same state sits in one of a few shapes:
    a `master_params` / `master_weights` dict keyed by parameter, parallel lists of low-precision and
    fp32 parameter groups (apex FP16_Optimizer: fp16_groups + fp32_from_fp16_groups; Megatron:
    float16_groups + fp32_from_float16_groups; DeepSpeed stages 1-2: bit16_groups +
    single_partition_of_fp32_groups is flat and is NOT handled here), or a `main_param` attribute on
    the parameter itself."""
    out = {}
    for holder in (optimizer, getattr(optimizer, "optimizer", None)):
        if holder is None:
            continue
        for attr in ("master_params", "master_weights"):
            d = getattr(holder, attr, None)
            if isinstance(d, dict):
                for k, v in d.items():
                    out[id(k)] = v
        for lo, hi in (("fp16_groups", "fp32_from_fp16_groups"), ("float16_groups", "fp32_from_float16_groups"),
                       ("bit16_groups", "fp32_groups")):
            g_lo, g_hi = getattr(holder, lo, None), getattr(holder, hi, None)
            if g_lo is None or g_hi is None:
                continue
            for grp_lo, grp_hi in zip(g_lo, g_hi):
                for p_lo, p_hi in zip(grp_lo, grp_hi):
                    out[id(p_lo)] = p_hi
    return out


def _named_state_tensors(model_engine, optimizer):
    """(name, tensor) pairs in the reference's naming scheme and per-parameter order
    (src/api.cpp:583-653): '<p>', 'master_weights::<p>', 'optimizer.exp_avg::<p>',
    'optimizer.exp_avg_sq::<p>', for a plain module (or an engine with .module) and an
    Adam-style optimizer, with or without fp32 master copies.

    Every parameter the module holds on this rank is tracked.  (The reference's ZeRO-3 walk keeps
    only the parameters whose index falls into the rank's "territory", :543-573, although every
    rank holds a slice of every parameter -- so most of each rank's state is never saved.  There
    is no such filter here: what is local is registered.)"""
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
    masters = _master_of(opt) if opt is not None else {}
    for name, p in params:
        out.append((name, p.data))
        master = masters.get(id(p), getattr(p, "main_param", None))
        if master is not None:
            out.append((f"master_weights::{name}", master.data if hasattr(master, "data") else master))
        st = None
        for key in (master, p):  # Adam state is keyed by whichever tensor the optimizer steps
            if key is not None:
                try:
                    st = state.get(key, None)
                except TypeError:
                    st = None
                if st:
                    break
        if st:
            if "exp_avg" in st:
                out.append((f"optimizer.exp_avg::{name}", st["exp_avg"]))
            if "exp_avg_sq" in st:
                out.append((f"optimizer.exp_avg_sq::{name}", st["exp_avg_sq"]))
    return out


_log_file = None


def _log(line):
    """One line of the per-rank log, in the reference's place and spelling:
    ./logs/<run id>/rank_<r>/checkers.log (src/logging.cpp:105-160), '[TIMING] key=value'
    (src/api.cpp:1017-1020, 1240-1246, 1293; src/ANSCompressor.cpp:1397-1399)."""
    global _log_file
    if os.environ.get("CHECKERS_LOG", "1") == "0" or _ctx is None:
        return
    try:
        if _log_file is None:
            run_id = os.environ.get("CHECKERS_LOG_RUN_ID") or f"run_{os.getpid()}"
            d = os.path.join(os.environ.get("CHECKERS_LOG_DIR", "logs"), run_id, f"rank_{max(_ctx.rank, 0)}")
            os.makedirs(d, exist_ok=True)
            _log_file = open(os.path.join(d, "checkers.log"), "a", buffering=1)
        _log_file.write(line + "\n")
    except OSError:
        pass  # logging never fails a checkpoint


def _timing(key, ms):
    _log(f"[TIMING] {key}={ms:.6f}")


def initialize_context(model_engine, optimizer=None, histogram_bins=256, background_threads=1, *,
                       shared_tables="reference", analysis_mode="reference", container_version=2):
    """Registers the rank's tensors.  `model_engine` may be an engine/module with
    named_parameters(), or a dict / list of (name, CUDA tensor) pairs.
    `background_threads` is accepted for signature compatibility; registration
    here is a metadata push and needs no worker threads.

    shared_tables (an addition): what to do when analyze_tensors() has grouped tensors into clusters
    whose shared table the reference's normalisation leaves undecodable (every bf16 cluster):
    "reference" refuses to write such files (compress_and_save raises), "reference_bytes" writes the
    reference's exact, unrestorable bytes, "repair" renormalises shared tables so they decode.

    container_version (an addition): 2 = the reference's files (default); 3 = the byte-plane container (about a
    fifth smaller on optimizer state, not readable by the reference's layout; load_and_decompress of the same
    context reads what it wrote).

    analysis_mode (an addition): "reference" computes the statistics of analyze_tensors() in the
    reference's order of float additions (bit-identical results, one thread block per tensor); "fast"
    spreads every tensor over the whole device and sums in double: minimum, maximum and the value
    histogram are the same, the moments differ by the rounding error of the reference's float sums,
    so a cluster boundary can fall differently."""
    global _ctx, _initialized, _log_file
    import time
    t0 = time.perf_counter()
    try:
        if histogram_bins == 0:
            raise RuntimeError("histogram_bins must be greater than zero")
        if background_threads == 0:
            raise RuntimeError("background_threads must be greater than zero")
        if shared_tables not in ("reference", "reference_bytes", "repair"):
            raise RuntimeError("shared_tables must be 'reference', 'reference_bytes' or 'repair'")
        if analysis_mode not in ("reference", "fast"):
            raise RuntimeError("analysis_mode must be 'reference' or 'fast'")
        if container_version not in (2, 3):
            raise RuntimeError("container_version must be 2 or 3")
        rank = _env_rank(model_engine, "global_rank", "RANK")
        local_rank = _env_rank(model_engine, "local_rank", "LOCAL_RANK")
        t1 = time.perf_counter()
        pairs = _named_state_tensors(model_engine, optimizer)
        t2 = time.perf_counter()
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
        if _log_file is not None:
            _log_file.close()
            _log_file = None
        _ctx = Context(device=device, rank=rank, local_rank=local_rank)
        _ctx.set_histogram_bins(histogram_bins)
        _ctx.set_option("repair_tables", int(shared_tables == "repair"))
        _ctx.set_option("allow_undecodable", int(shared_tables == "reference_bytes"))
        _ctx.set_option("fast_stats", int(analysis_mode == "fast"))
        _ctx.set_option("format_version", int(container_version))
        for name, t in pairs:
            if not getattr(t, "is_cuda", False):
                continue  # no local device storage on this rank
            _ctx.register_tensor(name, t.contiguous() if not t.is_contiguous() else t)
        _initialized = True
        t3 = time.perf_counter()
        _timing("setup_ms", (t1 - t0) * 1e3)
        _timing("discovery_ms", (t2 - t1) * 1e3)
        _timing("flush_ms", (t3 - t2) * 1e3)
        _timing("total_ms", (t3 - t0) * 1e3)
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
        import time
        t0 = time.perf_counter()
        _ctx.analyze()
        _timing("analyze_histograms_ms", _ctx.timing("analyze_stats_ms"))   # statistics, value histograms, fingerprints: one kernel
        _timing("analyze_knn_clusters_ms", _ctx.timing("analyze_cluster_ms"))
        _timing("analyze_total_ms", (time.perf_counter() - t0) * 1e3)
    except Exception as e:  # noqa: BLE001
        _fail("", e)


def compress_and_save(output_path):
    try:
        if not _initialized or _ctx is None:
            raise RuntimeError("Context not initialized: call initialize_context first.")
        import time
        t0 = time.perf_counter()
        _ctx.compress_and_save(output_path)
        _timing("compress_and_save_total_ms", _ctx.timing("compress_total_ms") + _ctx.timing("io_ms"))
        _timing("compress_computation_ms", _ctx.timing("compress_device_ms"))
        _timing("compress_io_ms", _ctx.timing("io_ms"))
        _timing("compress_and_save_wall_ms", (time.perf_counter() - t0) * 1e3)
        s = _ctx.summary()
        _log(f"[ANS][rank={max(_ctx.rank, 0)}][summary] tensors={s['n_tensors']} tables={s['n_tables']} "
             f"original_bytes={s['original_bytes']} ans_bytes={s['states_bytes']} sidecar_bytes={s['mantissa_bytes']} "
             f"disk_ratio={s['original_bytes'] / max(s['states_bytes'] + s['mantissa_bytes'] + s['dict_bytes'], 1):.6f}")
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
