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
encode, compaction into the file layout) and restore it (decode + merge) with
all data resident in HBM.  value = shard bytes / step time, summed over ranks,
timed with CUDA events on the library's stream, max over ranks.

e2e = the same work for a slice of the shard that starts and ends in pinned host
memory, through checkers_b200.streaming.ChunkedHostPipeline: every input byte is
copied host->device, the three file images of every chunk device->host, then the
images host->device and the restored tensors device->host, all inside the timed
region (wall clock between device synchronisations, max over ranks).
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
PARAMS_8B = 8030261248
# measured once under ncu (see profiles/): DRAM read+write bytes per byte of tensor processed
NCU_DRAM_BYTES_PER_TENSOR_BYTE = {"rans_encode_kernel": (1.013e9 + 0.426e9) / 939.5e6,
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--world-shards", type=int, default=8, help="flat-index shards of the model; one per rank")
    ap.add_argument("--chunk-elems", type=int, default=1 << 20, help="elements per registered tensor")
    ap.add_argument("--limit-elems", type=int, default=0, help="use only this many parameters of the shard (tests)")
    ap.add_argument("--e2e-elems", type=int, default=0,
                    help="parameters in the host-buffer end-to-end leg (default: 256 Mi on one GPU, 128 Mi per GPU on several, "
                         "to bound pinned host memory)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--e2e-workers", type=int, default=4, help="host threads driving chunks of the pipeline")
    ap.add_argument("--e2e-chunk-bytes", type=int, default=256 << 20,
                    help="tensor bytes per chunk of the host-buffer pipeline")
    ap.add_argument("--cpu-sample-elems", type=int, default=32 << 20, help="parameters in the timed CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    enc_ms, dec_ms, split_ms, compact_ms, table_ms, cwall_ms, dwall_ms = [], [], [], [], [], [], []
    e0.record(lib_stream)
    for _ in range(args.steps):
        summ = step()
        enc_ms.append(ctx.timing("encode_ms"))
        dec_ms.append(ctx.timing("decode_ms"))
        split_ms.append(ctx.timing("split_hist_ms"))
        compact_ms.append(ctx.timing("compact_ms"))
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
    e_elems = min(args.e2e_elems or ((256 << 20) if world == 1 else (128 << 20)), n_elems)
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
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = e_bytes * world / e2e_s / 1e9

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
    kernels = {"rans_encode_kernel": (float(np.mean(enc_ms)), shard_bytes + payload_bytes),
               "rans_decode_kernel": (float(np.mean(dec_ms)), shard_bytes + payload_bytes + sidecar_bytes),
               "split_hist_kernel": (float(np.mean(split_ms)), shard_bytes + sidecar_bytes),
               "scan+compact": (float(np.mean(compact_ms)), 2 * payload_bytes)}
    dom = max(("rans_encode_kernel", "rans_decode_kernel"), key=lambda k: kernels[k][0])
    dom_ms, dom_bytes = kernels[dom]
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": achieved / peak,
                # DRAM bytes of one launch: ncu dram__bytes_read+write on a 939.5 MB case (profiles/
                # rans_kernels_llama3_shard.md), scaled by tensor bytes (traffic grows in proportion)
                "traffic": shard_bytes * NCU_DRAM_BYTES_PER_TENSOR_BYTE[dom],
                "per_kernel_ms": {k: v[0] for k, v in kernels.items()},
                "per_kernel_algorithmic_gbs": {k: (v[1] / (v[0] * 1e-3) / 1e9 if v[0] > 0 else None)
                                               for k, v in kernels.items()},
                "note": "compress runs as a pipeline: counting, encode grids and compaction of neighbouring segments "
                        "overlap, so their times are spans measured while sharing the device and add up to more "
                        "than compress_call_ms; decode runs alone",
                "host_table_ms": float(np.mean(table_ms)),
                "compress_call_ms": float(np.mean(cwall_ms)), "restore_call_ms": float(np.mean(dwall_ms))}

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
                "roofline": roofline, "cpu_baseline": cpu_baseline,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(e_bytes + img_bytes),
                        "d2h_bytes_per_step": int(img_bytes + e_bytes), "steps": args.e2e_steps,
                        "sample": f"{e_bytes / 2**30:.2f} GiB of the shard per GPU from pinned host buffers: "
                                  f"in {len(pipe.chunks)} chunks with copies and kernels overlapped: H2D, compress, D2H of "
                                  "the file images; then H2D of the images, restore, D2H"},
                "gpu_launches": int(launches), "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
