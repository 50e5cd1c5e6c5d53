"""Checkpoint manifest across ranks.

Every rank compresses its own shard into its own three files; nothing is
exchanged on the data path.  The only collective is one all-gather of six
64-bit totals per rank (chk_summary), from which rank 0 writes
<dir>/manifest.json with per-rank sizes and running offsets.  The reference has
no manifest (each rank just writes rank_<r>_* files,
src/ANSCompressor.cpp:1374-1377 in the Checkers tree); this file is an addition
next to them and never changes their bytes.
"""
import json
import os

FIELDS = ("n_tensors", "n_tables", "states_bytes", "mantissa_bytes", "dict_bytes", "original_bytes")


def gather_summaries(summary, group=None, device=None):
    """All-gather this rank's summary dict.  Uses torch.distributed when it is
    initialised (NCCL on GPUs, gloo on CPU); a single process returns [summary]."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return [dict(summary)]
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                             if backend == "nccl" else torch.device("cpu"))
    mine = torch.tensor([int(summary[k]) for k in FIELDS], dtype=torch.int64, device=dev)
    if backend == "nccl":
        out = torch.empty(world * len(FIELDS), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(out, mine, group=group)
        rows = out.view(world, len(FIELDS)).cpu().tolist()
    else:
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine, group=group)
        rows = [p.tolist() for p in parts]
    return [dict(zip(FIELDS, r)) for r in rows]


class PendingGather:
    """An all-gather of summaries that runs in the background (start_gather); result() waits for it."""

    def __init__(self, rows=None, work=None, out=None, world=1):
        self._rows, self._work, self._out, self._world = rows, work, out, world

    def result(self):
        if self._rows is None:
            self._work.wait()
            self._rows = self._out.view(self._world, len(FIELDS)).cpu().tolist()
        return [dict(zip(FIELDS, r)) for r in self._rows]


def start_gather(summary, group=None, device=None):
    """gather_summaries without waiting: the collective is queued (NCCL: asynchronously, on the
    process group's own stream) and the caller goes on, e.g. restores or writes its files, before
    it asks for result().  A rank is then not held up by the others between the two calls."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_backend(group) != "nccl":
        return PendingGather(rows=[[int(s[k]) for k in FIELDS] for s in gather_summaries(summary, group, device)])
    world = dist.get_world_size(group)
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    mine = torch.tensor([int(summary[k]) for k in FIELDS], dtype=torch.int64, device=dev)
    out = torch.empty(world * len(FIELDS), dtype=torch.int64, device=dev)
    work = dist.all_gather_into_tensor(out, mine, group=group, async_op=True)
    return PendingGather(work=work, out=out, world=world)


def build_manifest(summaries):
    """Per-rank sizes plus exclusive running offsets, and the totals."""
    ranks, run = [], {k: 0 for k in FIELDS}
    for r, s in enumerate(summaries):
        entry = {"rank": r, "files": {"states": f"rank_{r}_states.ansc",
                                      "mantissa": f"mantissa/rank_{r}_mantissa.mant",
                                      "tables": f"tables/rank_{r}_tables.dict"}}
        for k in FIELDS:
            entry[k] = int(s[k])
            entry[k + "_offset"] = run[k]
            run[k] += int(s[k])
        ranks.append(entry)
    compressed = run["states_bytes"] + run["mantissa_bytes"] + run["dict_bytes"]
    return {"format": "checkers-manifest", "version": 1, "world_size": len(summaries), "ranks": ranks,
            "totals": dict(run, compressed_bytes=compressed,
                           ratio=(run["original_bytes"] / compressed) if compressed else 0.0)}


def write_manifest(output_dir, manifest):
    path = os.path.join(output_dir, "manifest.json")
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(manifest, f, indent=1)
    os.replace(tmp, path)
    return path
