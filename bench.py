#!/usr/bin/env python3
"""Benchmark of the checkpoint-compression hot path on B200.

    python bench.py --gpus N --steps K --warmup W              (N == 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1)
    python bench.py --impl reference ...                        (CPU arm: the oracle port on all host threads)

Workload ("llama3-8b-zero3-shard"): the ZeRO-3 state of Llama-3-8B (291 tensors,
8 030 261 248 parameters; bf16 weight, fp32 master, fp32 exp_avg, fp32 exp_avg_sq
per parameter = 14 B/param) cut by flat parameter index into `--world-shards`
(8) equal shards; every rank holds ONE shard (14.05 GB) in HBM, registered in
chunks of `--chunk-elems` (1 Mi) elements, so per-GPU work is fixed as N grows
(weak scaling) and N = 8 is the whole model.  Values are synthetic, seeded, with
the distributions the benchmark config names.

A step = compress the shard (low-byte split + histograms, tables, 256-lane rANS
encode and gather into the file layout) and restore it (decode + merge) with
all data resident in HBM.  value = shard bytes / step time, summed over ranks,
timed with CUDA events on the library's stream, max over ranks.

e2e = the same work for a slice of the shard that starts and ends in pinned host
memory, through the chk_stream_* entry points (checkers_b200.streaming): every
input byte is copied host->device, the three file images of every part
device->host, then the images host->device and the restored tensors
device->host, all inside the timed region (wall clock between device
synchronisations, max over ranks).  The same slice size is used at every N.

parity = outside the timed region, the first tensors of the shard (the ones the
cpu_baseline leg times) are compressed to file images once more and compared byte
for byte with the files the CPU oracle writes for the same tensors.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

LLAMA3_8B = dict(hidden=4096, layers=32, inter=14336, q_heads=32, kv_heads=8, head_dim=128, vocab=128256)
LLAMA3_70B = dict(hidden=8192, layers=80, inter=28672, q_heads=64, kv_heads=8, head_dim=128, vocab=128256)
PARAMS_8B = 8030261248
# DRAM read + write bytes per byte of tensor, from one ncu capture of each kernel on a 939.5 MB slice of this
# workload (1024 tensors of 256 Ki elements); the traffic of a launch grows in proportion to the tensor bytes
NCU_DRAM_BYTES_PER_TENSOR_BYTE = {"rans_encode_fused_kernel": (1.350e9 + 0.810e9) / 939.5e6,
                                  "rans_decode_kernel": (0.905e9 + 0.902e9) / 939.5e6}


def llama_params(cfg):
    """(name, numel, is_norm_gain) in flat order."""
    h, i = cfg["hidden"], cfg["inter"]
    q, kv = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    out = [("model.embed_tokens.weight", cfg["vocab"] * h, False)]
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}."
        out += [(p + "self_attn.q_proj.weight", q * h, False), (p + "self_attn.k_proj.weight", kv * h, False),
                (p + "self_attn.v_proj.weight", kv * h, False), (p + "self_attn.o_proj.weight", h * q, False),
                (p + "mlp.gate_proj.weight", i * h, False), (p + "mlp.up_proj.weight", i * h, False),
                (p + "mlp.down_proj.weight", h * i, False), (p + "input_layernorm.weight", h, True),
                (p + "post_attention_layernorm.weight", h, True)]
    out += [("model.norm.weight", h, True), ("lm_head.weight", cfg["vocab"] * h, False)]
    return out


def shard_pieces(cfg, shard, world_shards, chunk_elems, limit_elems=None):
    """Chunks (param name, offset inside the shard, numel, is_norm) of one flat-index shard."""
    params = llama_params(cfg)
    total = sum(n for _, n, _ in params)
    lo, hi = shard * total // world_shards, (shard + 1) * total // world_shards
    if limit_elems:
        hi = min(hi, lo + limit_elems)
    pieces, pos = [], 0
    for name, n, is_norm in params:
        a, b = max(pos, lo), min(pos + n, hi)
        k = 0
        while a < b:
            c = min(chunk_elems, b - a)
            pieces.append((f"{name}@{a - pos}", a - lo, c, is_norm))
            a += c
            k += 1
        pos += n
    return pieces, hi - lo, total


STATE_KINDS = (("", "bf16"), ("master_weights::", "f32"), ("optimizer.exp_avg::", "f32"),
               ("optimizer.exp_avg_sq::", "f32"))


def make_shard_on_device(torch, pieces, n_elems, seed, device):
    """Four flat device buffers holding the shard's states."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    master = torch.empty(n_elems, dtype=torch.float32, device=device)
    master.normal_(0.0, 0.02, generator=g)
    for _, off, n, is_norm in pieces:
        if is_norm:
            master[off:off + n].normal_(0.0, 1e-3, generator=g).add_(1.0)
    weight = master.to(torch.bfloat16)
    exp_avg = torch.empty(n_elems, dtype=torch.float32, device=device).normal_(0.0, 1e-4, generator=g)
    exp_avg_sq = torch.empty(n_elems, dtype=torch.float32, device=device).normal_(-18.0, 2.0, generator=g).exp_()
    return [weight, master, exp_avg, exp_avg_sq]


def make_shard_on_host(pieces, n_elems, seed):
    """Same distributions with numpy, for the CPU arm."""
    from oracle_lib import to_bf16_bits
    rng = np.random.default_rng(seed)
    master = rng.normal(0.0, 0.02, n_elems).astype(np.float32)
    for _, off, n, is_norm in pieces:
        if is_norm:
            master[off:off + n] = (1.0 + rng.normal(0.0, 1e-3, n)).astype(np.float32)
    weight = to_bf16_bits(master)
    exp_avg = rng.normal(0.0, 1e-4, n_elems).astype(np.float32)
    exp_avg_sq = np.exp(rng.normal(-18.0, 2.0, n_elems)).astype(np.float32)
    return [weight, master, exp_avg, exp_avg_sq]


def bind_to_gpu_cpus(torch, local_rank):
    """With several ranks on a box, keep this rank's threads -- and so the pinned host memory they touch first -- on
    the CPUs next to its GPU (read from NVML; nothing is changed on the GPU).  Returns the CPU count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def pcie_rates(torch, pinned, device):
    """Plain copies of one pinned host buffer: host->device, device->host, and both at once (GB/s each way)."""
    nbytes = pinned.numel() * pinned.element_size()
    up = torch.empty_like(pinned, device=device)
    down_src = torch.empty_like(pinned, device=device)
    down = torch.empty_like(pinned).pin_memory()
    s1, s2 = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def run(do_up, do_down):
        best = None
        for _ in range(3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if do_up:
                with torch.cuda.stream(s1):
                    up.copy_(pinned, non_blocking=True)
            if do_down:
                with torch.cuda.stream(s2):
                    down.copy_(down_src, non_blocking=True)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return nbytes / best / 1e9

    return {"h2d_gbs": round(run(True, False), 1), "d2h_gbs": round(run(False, True), 1),
            "both_directions_gbs_each": round(run(True, True), 1), "copy_bytes": nbytes}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def wait_first(self, timeout=10.0):
        """Block until the first sample has arrived (nvidia-smi takes a while to start on a box with many GPUs)."""
        t0 = time.time()
        while self.proc and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.02)

    def mark(self):
        return len(self.lines)

    def stop(self, first=0, last=None):
        """Summary of the samples with index in [first, last]; when the window was shorter than the
        sampling interval, the sample before it and the one after it are used."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        lo = max(first - 1, 0)
        hi = len(self.lines) if last is None else min(last + 1, len(self.lines))
        for ln in self.lines[lo:max(hi, lo + 1)]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_arm(args, rank, world):
    """--impl reference: the oracle port (CPU restatement of the reference kernels;
    the reference has no CPU build of this path) on all host threads."""
    if rank != 0:
        return
    from oracle_lib import BF16, F32, Oracle
    o = Oracle()
    threads = os.cpu_count() or 1
    pieces, n_elems, _ = shard_pieces(LLAMA3_8B, 0, args.world_shards, args.chunk_elems,
                                      limit_elems=args.cpu_sample_elems)
    bufs = make_shard_on_host(pieces, n_elems, args.seed)
    arrays, dtypes = [], []
    for _, off, n, _ in pieces:
        for b, dt in zip(bufs, (BF16, F32, F32, F32)):
            arrays.append(b[off:off + n])
            dtypes.append(dt)
    times = []
    for step in range(args.warmup + args.steps):
        c, d, orig, pay, side = o.roundtrip_timed(arrays, dtypes, threads)
        if step >= args.warmup:
            times.append(c + d)
    t = float(np.mean(times))
    value = orig / t / 1e9
    sample = f"{orig / 2**20:.0f} MiB of shard 0 ({len(arrays)} tensors of <= {args.chunk_elems} elements) per step"
    line = {"impl": "reference", "metric": "compress+decompress GB/s", "value": value, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "llama3-8b-zero3-shard", "world_shards": args.world_shards,
                       "chunk_elems": args.chunk_elems, "bytes_per_step": int(orig)},
            "ratio": orig / (pay + side) if pay + side else None,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def host_stream_70b(args, torch):
    """Llama-3-70B ZeRO-3 state, shard 0 of 8 (123 GB per rank at 14 B per parameter): the first --c4-elems
    parameters of it, resident in pinned host memory, through the chunked host pipeline in 1 GiB parts."""
    from checkers_b200.streaming import ChunkedHostPipeline, HostTensor
    dev = torch.device("cuda", torch.cuda.current_device())
    import checkers_b200 as chk
    pieces, n_elems, total = shard_pieces(LLAMA3_70B, 0, 8, args.chunk_elems, limit_elems=args.c4_elems)
    bufs = make_shard_on_device(torch, pieces, n_elems, 70, dev)
    h_in = [torch.empty(n_elems, dtype=b.dtype).pin_memory() for b in bufs]
    h_out = [torch.empty(n_elems, dtype=b.dtype).pin_memory() for b in bufs]
    for h, b in zip(h_in, bufs):
        h.copy_(b)
    del bufs
    torch.cuda.empty_cache()
    tags = (chk.BF16, chk.F32, chk.F32, chk.F32)
    tensors, targets = [], []
    for name, off, n, _ in pieces:
        for (prefix, _), hi, ho, tag in zip(STATE_KINDS, h_in, h_out, tags):
            tensors.append(HostTensor(prefix + name, hi[off:off + n], tag))
            targets.append(ho[off:off + n])
    nbytes = sum(h.numel() * h.element_size() for h in h_in)

    def run(version):
        pipe = ChunkedHostPipeline(tensors, device=dev.index, rank=0, chunk_bytes=1 << 30, workers=3,
                                   options={"format_version": version})
        best_c = best_r = None
        for it in range(3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            pipe.compress()
            t1 = time.perf_counter()
            pipe.restore(targets)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            if it:
                best_c = t1 - t0 if best_c is None else min(best_c, t1 - t0)
                best_r = t2 - t1 if best_r is None else min(best_r, t2 - t1)
        for h, g in zip(h_in, h_out):
            assert torch.equal(h.view(torch.uint8), g.view(torch.uint8)), "70B-shaped host round trip is not lossless"
        s, parts = pipe.summary(), len(pipe.chunks)
        pipe.close()
        return best_c, best_r, s, parts

    c3, r3, s3, _ = run(3)
    best_c, best_r, s, n_parts = run(2)
    res = {"what": "Llama-3-70B shapes, shard 0 of 8 (123 GB per rank), first %d Mi parameters = %.2f GiB from pinned host "
                   "memory in 1 GiB parts over 3 staging slots, tensors of <= %d elements" % (n_elems >> 20, nbytes / 2**30, args.chunk_elems),
           "shard_bytes_full": total // 8 * 14, "sample_bytes": nbytes, "parts": n_parts,
           "compress_s": best_c, "restore_s": best_r, "compress_gbs": nbytes / best_c / 1e9,
           "restore_gbs": nbytes / best_r / 1e9, "compress_plus_restore_gbs": nbytes / (best_c + best_r) / 1e9,
           "ratio": s["original_bytes"] / (s["states_bytes"] + s["mantissa_bytes"] + s["dict_bytes"]),
           "full_shard_estimate_s": (best_c + best_r) * (total // 8 * 14) / nbytes,
           "container_version_3": {"compress_gbs": nbytes / c3 / 1e9, "restore_gbs": nbytes / r3 / 1e9,
                                   "compress_plus_restore_gbs": nbytes / (c3 + r3) / 1e9,
                                   "ratio": s3["original_bytes"] / (s3["states_bytes"] + s3["mantissa_bytes"] + s3["dict_bytes"])}}
    return res


def extras(args, torch, chk, ctx, shard_bytes, peak):
    """Numbers outside the headline step (flag --extras, second JSON line): the per-stage codec sweep of the
    microbenchmark configuration, the per-shard statistics pass, the Re-Pair tool against the reference's CLI."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best

    # ---- container version 3 (opt-in experiment; before the analysis below groups tensors into clusters): every high byte plane coded with its own table, same coder
    def one_format():
        best_c = best_d = None
        for _ in range(3):
            ctx.compress(host_images=False)
            cm, sm = ctx.timing("compress_device_ms"), ctx.timing("plane_split_ms")
            s = ctx.summary()
            t0 = time.perf_counter()
            ctx.decompress_resident(None)       # restores in place: the registered tensors are their own targets
            torch.cuda.synchronize()
            dm = (time.perf_counter() - t0) * 1e3
            best_c = cm if best_c is None else min(best_c, cm)
            best_d = dm if best_d is None else min(best_d, dm)
        total = s["states_bytes"] + s["mantissa_bytes"] + s["dict_bytes"]
        return {"compress_device_ms": best_c, "restore_call_ms": best_d, "ratio_all_files": s["original_bytes"] / total,
                "files_bytes": total, "plane_split_ms": sm, "plane_merge_ms": ctx.timing("plane_merge_ms")}

    v2 = one_format()
    ctx.set_option("format_version", 3)
    v3 = one_format()
    ctx.set_option("format_version", 2)
    out["format_v3"] = {"what": "the benchmark shard through container version 2 (the reference's) and version 3 (byte planes "
                                "with a table each); restore_call_ms is host wall time of the call, device-resident",
                        "v2": v2, "v3": v3}

    # ---- host-resident state in 1 GiB pieces (70B shapes): a bounded sample of shard 0 of 8 from pinned host memory
    out["host_stream_70b"] = host_stream_70b(args, torch)

    # ---- statistics of the resident shard: two passes over every tensor (src/TensorAnalyzer.cpp:64-198)
    def analyze_ms():
        ctx.analyze()
        ms = ctx.timing("analyze_stats_ms")
        for _ in range(2):
            ctx.analyze()
            ms = min(ms, ctx.timing("analyze_stats_ms"))
        return {"ms": ms, "algorithmic_bytes": 2 * shard_bytes, "gbs": 2 * shard_bytes / ms / 1e6,
                "frac_of_hbm_peak": 2 * shard_bytes / ms / 1e6 / peak}

    out["analyze"] = {"reference_order": dict(analyze_ms(), kernel="tensor_stats_kernel"),
                      "cluster_ms": ctx.timing("analyze_cluster_ms"), "tensors": ctx.tensor_count()}
    ctx.set_option("fast_stats", 1)
    out["analyze"]["fast"] = dict(analyze_ms(), kernel="stats_fast_pass1/2_kernel (sums in double, order-free)")
    ctx.set_option("fast_stats", 0)

    # ---- the offline study of shared histograms: one HyperLogLog sketch per tensor, union per cluster of the analysis above
    ctx.hll_sketch_all()
    hll_ms = ctx.timing("hll_sketch_ms")
    ctx.hll_sketch_all()
    hll_ms = min(hll_ms, ctx.timing("hll_sketch_ms"))
    own, shared = ctx.shared_vocabulary_report()
    out["shared_vocabulary"] = {"kernel": "hll_sketch_kernel", "ms": hll_ms, "gbs": shard_bytes / hll_ms / 1e6,
                                "frac_of_hbm_peak": shard_bytes / hll_ms / 1e6 / peak,
                                "per_tensor_histogram_bytes": own, "shared_histogram_bytes": shared,
                                "ratio": shared / own if own else None}

    # ---- codec microbenchmark configuration: 1 GiB fp32 ~ N(0, 1e-3) and 1 GiB bf16 ~ N(0, 0.02), seed 1, 4 MiB chunks
    g = torch.Generator(device=dev).manual_seed(1)
    chunk = 4 << 20
    sweep = {}
    for tag, dt, es, make in (("fp32", chk.F32, 4, lambda: torch.randn(256 << 20, generator=g, device=dev) * 1e-3),
                              ("bf16", chk.BF16, 2,
                               lambda: (torch.randn(512 << 20, generator=g, device=dev) * 0.02).to(torch.bfloat16))):
        x = make()
        B = x.numel() * x.element_size()
        n_chunks = B // chunk
        masked = torch.empty(B, dtype=torch.uint8, device=dev)
        side = torch.empty(B // 2, dtype=torch.uint8, device=dev)
        back = torch.empty(B, dtype=torch.uint8, device=dev)
        c = chk.Context(device=dev.index)
        torch.cuda.synchronize()
        res = {}
        # bit-pack only: tensor -> masked copy + packed low bytes (2.5 B moved per byte), and back (2.5 B)
        t = timed(lambda: c.split(x.data_ptr(), x.numel(), dt, masked.data_ptr(), side.data_ptr()))
        res["split_only_encode"] = {"ms": t * 1e3, "gbs": B / t / 1e9, "algorithmic_bytes": 2.5 * B}
        t = timed(lambda: c.merge(masked.data_ptr(), side.data_ptr(), x.numel(), dt, back.data_ptr()))
        res["split_only_decode"] = {"ms": t * 1e3, "gbs": B / t / 1e9, "algorithmic_bytes": 2.5 * B}
        assert torch.equal(back, x.view(torch.uint8))
        # entropy coding only: the masked buffer as byte tensors (all 256 lanes are real chains, zeros included)
        ca = chk.Context(device=dev.index)
        dst = []
        for k in range(n_chunks):
            ca.register_pointer(f"m.{k}", masked.data_ptr() + k * chunk, chunk, chk.I8)
            dst.append(back.data_ptr() + k * chunk)
        dst = np.asarray(dst, dtype=np.uint64)
        enc, dec = [], []
        for _ in range(3):
            ca.compress(host_images=False)
            enc.append(ca.timing("compress_device_ms"))
            ca.decompress_resident(dst)
            dec.append(ca.timing("decode_ms"))
        sa = ca.summary()
        pay = sa["states_bytes"] - 16 - 4648 * sa["n_tensors"]
        res["ans_only_encode"] = {"ms": min(enc), "gbs": B / min(enc) / 1e6, "algorithmic_bytes": 2 * B + pay,
                                  "note": "counting pass + encode: the tensors are read twice (1 GiB exceeds L2)"}
        res["ans_only_decode"] = {"ms": min(dec), "gbs": B / min(dec) / 1e6, "algorithmic_bytes": B + pay}
        assert torch.equal(back, masked)
        ca.close()
        # full pipeline on the float tensor
        cf = chk.Context(device=dev.index)
        dst = []
        for k in range(n_chunks):
            cf.register_pointer(f"t.{k}", x.data_ptr() + k * chunk, chunk // es, dt)
            dst.append(back.data_ptr() + k * chunk)
        dst = np.asarray(dst, dtype=np.uint64)
        enc, dec = [], []
        for _ in range(3):
            cf.compress(host_images=False)
            enc.append(cf.timing("compress_device_ms"))
            cf.decompress_resident(dst)
            dec.append(cf.timing("decode_ms"))
        sf = cf.summary()
        pay = sf["states_bytes"] - 16 - 4648 * sf["n_tensors"]
        sidecar = sf["mantissa_bytes"] - 16 - 288 * sf["n_tensors"]
        res["full_encode"] = {"ms": min(enc), "gbs": B / min(enc) / 1e6, "algorithmic_bytes": B + sidecar + pay}
        res["full_decode"] = {"ms": min(dec), "gbs": B / min(dec) / 1e6, "algorithmic_bytes": B + sidecar + pay}
        res["ratio"] = sf["original_bytes"] / (sf["states_bytes"] + sf["mantissa_bytes"] + sf["dict_bytes"])
        assert torch.equal(back, x.view(torch.uint8))
        cf.close()
        c.close()
        for v in res.values():
            if isinstance(v, dict):
                v["frac_of_hbm_peak"] = v["algorithmic_bytes"] / (v["ms"] * 1e-3) / 1e9 / peak
        sweep[tag] = res
        del x, masked, side, back
        torch.cuda.empty_cache()
    out["stage_sweep"] = {"config": "1 GiB fp32 ~ N(0,1e-3) and 1 GiB bf16 ~ N(0,0.02), seed 1, 4 MiB chunks (256 tensors each)",
                          "peak_gbs": peak, **sweep}

    # ---- prefix-mask Re-Pair: seconds per export for groups of 2^16 .. 2^22 elements, against the reference CLI
    import shutil
    import tempfile
    from checkers_b200 import repair
    from oracle_lib import REF_REPAIR_CLI, synth
    rep = []
    for lg in (16, 18, 20, 22):
        root = tempfile.mkdtemp(prefix="chk_repair_")
        try:
            os.makedirs(os.path.join(root, "analysis", "plots"))
            os.makedirs(os.path.join(root, "tensors"))
            manifest = ["tensor_key,layer,category,state_type,numel,dtype,file"]
            for layer in range(3):
                raw, _ = synth("f32_master", 1 << lg, 300 + layer)
                rel = f"tensors/master_mlp.up_{layer}.bin"
                raw.tofile(os.path.join(root, rel))
                manifest.append(f"master.mlp.up.{layer},{layer},mlp.up,master,{1 << lg},float32,{rel}")
            groups = ["state_type,category,group_id,n_layers,layers,representative_layer,c6,c7,c8,c9",
                      'master,mlp.up,0,3,"0 1 2",1,0,0,0,0']
            open(os.path.join(root, "manifest.csv"), "w").write("\n".join(manifest) + "\n")
            open(os.path.join(root, "analysis", "plots", "grouping_summary.csv"), "w").write("\n".join(groups) + "\n")
            with open(os.devnull, "w") as null:
                old = sys.stdout
                sys.stdout = null
                try:
                    repair.main([root])          # the first call pays for the workspace
                    t0 = time.perf_counter()
                    repair.main([root])
                    ours = time.perf_counter() - t0
                finally:
                    sys.stdout = old
            theirs = None
            if os.path.exists(REF_REPAIR_CLI):
                t0 = time.perf_counter()
                subprocess.check_call([REF_REPAIR_CLI, root], stdout=subprocess.DEVNULL)
                theirs = time.perf_counter() - t0
            rep.append({"elements_per_tensor": 1 << lg, "tensors": 3, "seconds": ours, "reference_cli_seconds": theirs})
        finally:
            shutil.rmtree(root, ignore_errors=True)
    out["repair"] = {"what": "python -m checkers_b200.repair on one group of three fp32 tensors, default arguments, "
                             "file reading and report writing included; reference = its own CLI, single-threaded, same box",
                     "groups": rep}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--world-shards", type=int, default=8, help="flat-index shards of the model; one per rank")
    ap.add_argument("--chunk-elems", type=int, default=1 << 20, help="elements per registered tensor")
    ap.add_argument("--limit-elems", type=int, default=0, help="use only this many parameters of the shard (tests)")
    ap.add_argument("--e2e-elems", type=int, default=256 << 20,
                    help="parameters per GPU in the host-buffer end-to-end leg (14 bytes each; the same at every N)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--c4-elems", type=int, default=512 << 20,
                    help="--extras: parameters of the 70B-shaped shard streamed from host memory (14 bytes each)")
    ap.add_argument("--e2e-workers", type=int, default=4, help="staging slots (and host threads) of the chunk pipeline")
    ap.add_argument("--e2e-chunk-bytes", type=int, default=512 << 20,
                    help="tensor bytes per chunk of the host-buffer pipeline")
    ap.add_argument("--cpu-sample-elems", type=int, default=32 << 20, help="parameters in the timed CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--analyze-only", action="store_true",
                    help="run only the statistics pass over the shard (for profiling) and print its time")
    ap.add_argument("--extras", action="store_true",
                    help="after the headline line, print a second JSON line: per-stage codec sweep, statistics pass, Re-Pair")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--opt", action="append", default=[], help="library option key=value (chk_set_option)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        cpu_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import checkers_b200 as chk
    from checkers_b200 import manifest

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa = bind_to_gpu_cpus(torch, local_rank) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    shard = rank % args.world_shards
    pieces, n_elems, total_params = shard_pieces(LLAMA3_8B, shard, args.world_shards, args.chunk_elems,
                                                 limit_elems=args.limit_elems or None)
    assert total_params == PARAMS_8B
    bufs = make_shard_on_device(torch, pieces, n_elems, args.seed * 1000 + shard, device)
    outs = [torch.empty_like(b) for b in bufs]
    tags = (chk.BF16, chk.F32, chk.F32, chk.F32)

    ctx = chk.Context(device=local_rank, rank=rank, local_rank=local_rank)
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    for kv in args.opt:
        k, v = kv.split("=")
        ctx.set_option(k, int(v))
    dst = []
    for name, off, n, _ in pieces:
        for (prefix, _), b, o, tag in zip(STATE_KINDS, bufs, outs, tags):
            es = b.element_size()
            ctx.register_pointer(prefix + name, b.data_ptr() + off * es, n, tag)
            dst.append(o.data_ptr() + off * es)
    dst = np.asarray(dst, dtype=np.uint64)
    shard_bytes = sum(b.numel() * b.element_size() for b in bufs)
    torch.cuda.synchronize()

    if args.analyze_only:
        ms = []
        for _ in range(3):
            ctx.analyze()
            ms.append(ctx.timing("analyze_stats_ms"))
        print(json.dumps({"analyze_stats_ms": min(ms), "bytes": shard_bytes, "gbs_of_2B": 2 * shard_bytes / min(ms) / 1e6}))
        return

    lib_stream = torch.cuda.ExternalStream(ctx.stream_handle(), device=device)

    def step():
        ctx.compress(host_images=False)
        s = ctx.summary()
        pending = manifest.start_gather(s, device=device) if world > 1 else None   # sizes of all ranks for the manifest
        ctx.decompress_resident(dst)
        if pending is not None:
            pending.result()
        return s

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        summ = step()
    # the restored bytes must equal the inputs (checked once, outside the timed region)
    barrier()
    for b, o in zip(bufs, outs):
        assert torch.equal(b.view(torch.uint8), o.view(torch.uint8)), "round trip is not lossless"

    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
    except Exception:
        gpu_id = str(local_rank)
    sampler = ClockSampler(gpu_id)
    sampler.start()
    sampler.wait_first()
    barrier()
    launches0 = ctx.kernel_launches()
    mark0 = sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    enc_ms, dec_ms, split_ms, table_ms, cwall_ms, dwall_ms = [], [], [], [], [], []
    e0.record(lib_stream)
    for _ in range(args.steps):
        summ = step()
        enc_ms.append(ctx.timing("encode_ms"))
        dec_ms.append(ctx.timing("decode_ms"))
        split_ms.append(ctx.timing("split_hist_ms"))
        table_ms.append(ctx.timing("table_ms"))
        cwall_ms.append(ctx.timing("compress_total_ms"))
        dwall_ms.append(ctx.timing("decompress_total_ms"))
    e1.record(lib_stream)
    barrier()
    clocks = sampler.stop(mark0, sampler.mark())
    launches = ctx.kernel_launches() - launches0
    elapsed_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = shard_bytes * world / (ms_per_step * 1e-3) / 1e9

    # ---- end-to-end leg through the C ABI with HOST buffers (pinned), copies timed
    e_elems = min(args.e2e_elems, n_elems)
    e_pieces = [(nm, off, min(n, e_elems - off), nrm) for nm, off, n, nrm in pieces if off < e_elems]
    h_in = [torch.empty(e_elems, dtype=b.dtype).pin_memory() for b in bufs]
    h_out = [torch.empty(e_elems, dtype=b.dtype).pin_memory() for b in bufs]
    for h, b in zip(h_in, bufs):
        h.copy_(b[:e_elems])
    from checkers_b200.streaming import ChunkedHostPipeline, HostTensor
    h_tensors, h_targets = [], []
    for name, off, n, _ in e_pieces:
        for (prefix, _), hi, ho, tag in zip(STATE_KINDS, h_in, h_out, tags):
            h_tensors.append(HostTensor(prefix + name, hi[off:off + n], tag))
            h_targets.append(ho[off:off + n])
    pipe = ChunkedHostPipeline(h_tensors, device=local_rank, rank=rank, chunk_bytes=args.e2e_chunk_bytes,
                               workers=args.e2e_workers)
    e2e_keys = ("compress_h2d_ms", "compress_kernel_ms", "compress_d2h_ms", "compress_wall_ms", "restore_h2d_ms",
                "restore_kernel_ms", "restore_d2h_ms", "restore_wall_ms")
    e_bytes = sum(h.numel() * h.element_size() for h in h_in)
    img_bytes = 0

    def e2e_step():
        nonlocal img_bytes
        pipe.compress()              # H2D of every chunk, kernels, D2H of each chunk's three file images
        s = pipe.summary()
        img_bytes = s["states_bytes"] + s["mantissa_bytes"] + s["dict_bytes"]
        pipe.restore(h_targets)      # H2D of the images, decode, D2H of the restored tensors
        torch.cuda.synchronize()

    e2e_step()
    for h, g in zip(h_in, h_out):
        assert torch.equal(h.view(torch.uint8), g.view(torch.uint8)), "end-to-end round trip is not lossless"
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    own_s = (time.perf_counter() - t0) / args.e2e_steps   # this rank's own steps (each ends with a device synchronise)
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    e2e_rank_ms = [round(own_s * 1e3, 1)]
    if world > 1:
        t = torch.tensor([e2e_s, own_s], dtype=torch.float64, device=device)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        e2e_rank_ms = [round(float(x[1].item()) * 1e3, 1) for x in every]
        e2e_s = max(float(x[0].item()) for x in every)
    e2e_value = e_bytes * world / e2e_s / 1e9
    e2e_engines = {k: round(pipe.timing(k), 2) for k in e2e_keys}   # last step, this rank: busy time per engine
    pipe.close()
    # the link's own rates: rank 0 alone (the other ranks wait), then all ranks at once (slowest rank counts)
    barrier()
    pcie = pcie_rates(torch, h_in[1], device) if rank == 0 else None
    barrier()
    if world > 1:
        mine = pcie_rates(torch, h_in[1], device)
        t = torch.tensor([mine["h2d_gbs"], mine["d2h_gbs"], mine["both_directions_gbs_each"]], dtype=torch.float64,
                         device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if pcie:
            pcie["all_ranks_at_once_min"] = {"h2d_gbs": round(float(t[0]), 1), "d2h_gbs": round(float(t[1]), 1),
                                             "both_directions_gbs_each": round(float(t[2]), 1)}
    if pcie:
        if world > 1:
            pcie["both_directions_gbs_each"] = pcie["all_ranks_at_once_min"]["both_directions_gbs_each"]
        # every step moves h2d_bytes up and d2h_bytes down; with both directions busy the link cannot do better than
        floor_s = max(e_bytes + img_bytes, img_bytes + e_bytes) / (pcie["both_directions_gbs_each"] * 1e9)
        pcie["link_floor_ms_per_step"] = round(floor_s * 1e3, 2)
        pcie["measured_ms_per_step"] = round(e2e_s * 1e3, 2)
        pcie["link_fraction"] = round(floor_s / e2e_s, 3)

    # ---- parity of the benchmark's own tensors with the CPU oracle (outside every timed region)
    parity = None
    if rank == 0 and not args.no_cpu_baseline:
        import tempfile
        from oracle_lib import BF16, F32, Oracle
        p_elems = min(args.cpu_sample_elems, n_elems)
        pctx = chk.Context(device=local_rank, rank=rank, local_rank=local_rank)
        p_names, p_host, p_dtypes = [], [], []
        host = [b[:p_elems].cpu() for b in bufs]
        for name, off, n, _ in pieces:
            if off >= p_elems:
                break
            n = min(n, p_elems - off)
            for (prefix, _), b, hb, tag, dt in zip(STATE_KINDS, bufs, host, tags, (BF16, F32, F32, F32)):
                pctx.register_pointer(prefix + name, b.data_ptr() + off * b.element_size(), n, tag)
                p_names.append(prefix + name)
                a = hb[off:off + n]
                p_host.append((a.view(torch.int16) if dt == BF16 else a).numpy())
                p_dtypes.append(dt)
        pctx.compress(host_images=True)
        with tempfile.TemporaryDirectory() as tmp:
            Oracle().compress_and_save(p_names, p_host, p_dtypes, tmp, rank=rank, threads=os.cpu_count() or 1)
            same = True
            for which, rel in enumerate((f"rank_{rank}_states.ansc", f"mantissa/rank_{rank}_mantissa.mant",
                                         f"tables/rank_{rank}_tables.dict")):
                same = same and np.array_equal(pctx.image(which), np.fromfile(os.path.join(tmp, rel), np.uint8))
        pctx.close()
        parity = {"files_identical": bool(same), "tensors": len(p_names), "against": "CPU oracle, same tensors"}
        assert same, "the file images of the benchmark shard differ from the CPU oracle's"

    # ---- roofline of the dominant kernel (rANS encode): algorithmic bytes = B read + c*B written
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak, peak_kind = 6650.0, "fallback"
    if os.path.exists(peaks_path):
        try:
            peak, peak_kind = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    payload_bytes = summ["states_bytes"] - 16 - 4648 * summ["n_tensors"]
    sidecar_bytes = summ["mantissa_bytes"] - 16
    # algorithmic bytes per launch: the fused encode reads the tensors and writes the payload once (its scratch
    # round trip and gather are its own overhead and show in `traffic`); decode reads payload + low bytes and
    # writes the tensors; counting reads the tensors and writes the low bytes
    kernels = {"rans_encode_fused_kernel": (float(np.mean(enc_ms)), shard_bytes + payload_bytes),
               "rans_decode_kernel": (float(np.mean(dec_ms)), shard_bytes + payload_bytes + sidecar_bytes),
               "split_hist_kernel": (float(np.mean(split_ms)), shard_bytes + sidecar_bytes)}
    dom = max(("rans_encode_fused_kernel", "rans_decode_kernel"), key=lambda k: kernels[k][0])
    dom_ms, dom_bytes = kernels[dom]
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": achieved / peak,
                # DRAM bytes of one launch: ncu dram__bytes_read + write on a 939.5 MB slice, scaled by tensor bytes
                "traffic": shard_bytes * NCU_DRAM_BYTES_PER_TENSOR_BYTE[dom],
                "per_kernel_ms": {k: v[0] for k, v in kernels.items()},
                "per_kernel_algorithmic_gbs": {k: (v[1] / (v[0] * 1e-3) / 1e9 if v[0] > 0 else None)
                                               for k, v in kernels.items()},
                "note": "compress = counting, then one kernel that encodes every tensor and gathers its lanes; tables are "
                        "built on the device while the next piece is counted (table_exposed_ms is what that did not hide)",
                "table_exposed_ms": float(np.mean(table_ms)),
                "compress_call_ms": float(np.mean(cwall_ms)), "restore_call_ms": float(np.mean(dwall_ms)),
                # DRAM bytes per tensor byte of the whole compress call: the counting pass streams (read 1, write the
                # low bytes), the fused kernel's figure is the ncu one above; against one read, one low-byte write and
                # one payload write if the tables were known beforehand and a lane's length before it ends
                "compress_dram_bytes_per_tensor_byte": {
                    "counting": (shard_bytes + sidecar_bytes) / shard_bytes,
                    "fused_encode_ncu": NCU_DRAM_BYTES_PER_TENSOR_BYTE["rans_encode_fused_kernel"],
                    "total": (shard_bytes + sidecar_bytes) / shard_bytes
                    + NCU_DRAM_BYTES_PER_TENSOR_BYTE["rans_encode_fused_kernel"],
                    "single_pass_ideal": (shard_bytes + sidecar_bytes + payload_bytes) / shard_bytes}}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle_lib import BF16, F32, Oracle
        o = Oracle()
        threads = os.cpu_count() or 1
        c_elems = min(args.cpu_sample_elems, n_elems)
        arrays, dtypes = [], []
        host = [b[:c_elems].cpu() for b in bufs]
        for _, off, n, _ in pieces:
            if off >= c_elems:
                break
            n = min(n, c_elems - off)
            for hb, dt in zip(host, (BF16, F32, F32, F32)):
                a = hb[off:off + n]
                arrays.append((a.view(torch.int16) if dt == BF16 else a).numpy())
                dtypes.append(dt)
        c, d, orig, pay, side = o.roundtrip_timed(arrays, dtypes, threads)
        cpu_baseline = {"value": orig / (c + d) / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                        "sample": f"first {orig / 2**20:.0f} MiB of the shard ({len(arrays)} tensors), one pass: "
                                  f"compress {c:.2f} s + restore {d:.2f} s",
                        "compress_gbs": orig / c / 1e9, "decompress_gbs": orig / d / 1e9}

    if rank == 0:
        compressed = summ["states_bytes"] + summ["mantissa_bytes"] + summ["dict_bytes"]
        line = {"metric": "compress+decompress GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": {"workload": "llama3-8b-zero3-shard", "world_shards": args.world_shards,
                           "shard_bytes_per_gpu": int(shard_bytes), "tensors_per_gpu": int(summ["n_tensors"]),
                           "chunk_elems": args.chunk_elems, "tables": "singleton (per tensor)",
                           "l2": "inputs (14 GB) exceed L2; no flush needed"},
                "ratio": summ["original_bytes"] / compressed,
                "compress_gbs_per_gpu": shard_bytes / np.mean(cwall_ms) / 1e6,
                "decompress_gbs_per_gpu": shard_bytes / np.mean(dwall_ms) / 1e6,
                "hbm_frac_of_step": (2 * (shard_bytes + payload_bytes + sidecar_bytes)) / (ms_per_step * 1e-3) / 1e9
                / peak,
                "roofline": roofline, "cpu_baseline": cpu_baseline, "parity": parity,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(e_bytes + img_bytes),
                        "d2h_bytes_per_step": int(img_bytes + e_bytes), "steps": args.e2e_steps,
                        "sample": f"{e_bytes / 2**30:.2f} GiB of the shard per GPU from pinned host buffers: "
                                  f"in {len(pipe.chunks)} parts over {args.e2e_workers} staging slots with copies and "
                                  "kernels overlapped: H2D, compress, D2H of the file images; then H2D of the images, "
                                  "restore, D2H",
                        "engine_busy_ms_rank0_last_step": e2e_engines, "pcie_rank0": pcie,
                        "cpus_bound_rank0": numa, "ms_per_step_by_rank": e2e_rank_ms},
                "gpu_launches": int(launches), "clocks": clocks}
        print(json.dumps(line), flush=True)
    if args.extras and rank == 0 and world == 1:
        del outs, h_in, h_out
        torch.cuda.empty_cache()
        print(json.dumps({"extras": extras(args, torch, chk, ctx, shard_bytes, peak)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
