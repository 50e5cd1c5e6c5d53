"""Checkpoint manifest across ranks.

Every rank compresses its own shard into its own three files; nothing is
exchanged on the data path.  The only collective is one all-gather of a fixed
record per rank -- six 64-bit totals (chk_summary) and, optionally, the SHA-256
of the rank's three files -- from which rank 0 writes <dir>/manifest.json with
per-rank sizes, running offsets and digests.  The reference has no manifest and
no reader (each rank just writes rank_<r>_* files,
src/ANSCompressor.cpp:1374-1377 in the Checkers tree); this file is an addition
next to them and never changes their bytes.
"""
import hashlib
import json
import os

FIELDS = ("n_tensors", "n_tables", "states_bytes", "mantissa_bytes", "dict_bytes", "original_bytes")
FILES = ("states", "mantissa", "tables")
_DIGEST_WORDS = 4 * len(FILES)          # three SHA-256 values as 64-bit words
ROW_WORDS = len(FIELDS) + _DIGEST_WORDS


def rank_files(rank):
    return {"states": f"rank_{rank}_states.ansc", "mantissa": f"mantissa/rank_{rank}_mantissa.mant",
            "tables": f"tables/rank_{rank}_tables.dict"}


def file_digests(output_dir, rank):
    """SHA-256 (hex) of the three files rank `rank` wrote under output_dir."""
    out = {}
    for key, rel in rank_files(rank).items():
        h = hashlib.sha256()
        with open(os.path.join(output_dir, rel), "rb") as f:
            for block in iter(lambda: f.read(1 << 22), b""):
                h.update(block)
        out[key] = h.hexdigest()
    return out


def _row(summary):
    """Summary dict (+ optional "digests") -> ROW_WORDS signed 64-bit integers."""
    words = [int(summary[k]) for k in FIELDS]
    raw = b"".join(bytes.fromhex(summary["digests"][k]) for k in FILES) if summary.get("digests") else bytes(96)
    words += [int.from_bytes(raw[i:i + 8], "little", signed=True) for i in range(0, 96, 8)]
    return words


def _unrow(words):
    s = dict(zip(FIELDS, (int(w) for w in words[:len(FIELDS)])))
    raw = b"".join(int(w).to_bytes(8, "little", signed=True) for w in words[len(FIELDS):ROW_WORDS])
    if any(raw):
        s["digests"] = {k: raw[32 * i:32 * i + 32].hex() for i, k in enumerate(FILES)}
    return s


def gather_summaries(summary, group=None, device=None):
    """All-gather this rank's summary dict.  Uses torch.distributed when it is
    initialised (NCCL on GPUs, gloo on CPU); a single process returns [summary]."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return [_unrow(_row(summary))]
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                             if backend == "nccl" else torch.device("cpu"))
    mine = torch.tensor(_row(summary), dtype=torch.int64, device=dev)
    if backend == "nccl":
        out = torch.empty(world * ROW_WORDS, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(out, mine, group=group)
        rows = out.view(world, ROW_WORDS).cpu().tolist()
    else:
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine, group=group)
        rows = [p.tolist() for p in parts]
    return [_unrow(r) for r in rows]


class PendingGather:
    """An all-gather of summaries that runs in the background (start_gather); result() waits for it."""

    def __init__(self, rows=None, work=None, out=None, world=1):
        self._rows, self._work, self._out, self._world = rows, work, out, world

    def result(self):
        if self._rows is None:
            self._work.wait()
            self._rows = self._out.view(self._world, ROW_WORDS).cpu().tolist()
        return [_unrow(r) for r in self._rows]


def start_gather(summary, group=None, device=None):
    """gather_summaries without waiting: the collective is queued (NCCL: asynchronously, on the
    process group's own stream) and the caller goes on, e.g. restores or writes its files, before
    it asks for result().  A rank is then not held up by the others between the two calls."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_backend(group) != "nccl":
        return PendingGather(rows=[_row(s) for s in gather_summaries(summary, group, device)])
    world = dist.get_world_size(group)
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    mine = torch.tensor(_row(summary), dtype=torch.int64, device=dev)
    out = torch.empty(world * ROW_WORDS, dtype=torch.int64, device=dev)
    work = dist.all_gather_into_tensor(out, mine, group=group, async_op=True)
    return PendingGather(work=work, out=out, world=world)


def build_manifest(summaries):
    """Per-rank sizes plus exclusive running offsets (and file digests where given), and the totals."""
    ranks, run = [], {k: 0 for k in FIELDS}
    for r, s in enumerate(summaries):
        entry = {"rank": r, "files": rank_files(r)}
        for k in FIELDS:
            entry[k] = int(s[k])
            entry[k + "_offset"] = run[k]
            run[k] += int(s[k])
        if s.get("digests"):
            entry["sha256"] = dict(s["digests"])
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


def verify_manifest(output_dir, ranks=None):
    """Check the files under output_dir against manifest.json: sizes always, SHA-256 where the
    manifest has it.  `ranks` limits the check to the files this process can see.  Returns a list
    of problems (empty = all good); a reader calls this before it restores."""
    with open(os.path.join(output_dir, "manifest.json")) as f:
        m = json.load(f)
    size_key = {"states": "states_bytes", "mantissa": "mantissa_bytes", "tables": "dict_bytes"}
    problems = []
    for entry in m["ranks"]:
        r = entry["rank"]
        if ranks is not None and r not in ranks:
            continue
        digests = None
        for key, rel in entry["files"].items():
            path = os.path.join(output_dir, rel)
            if not os.path.exists(path):
                problems.append(f"rank {r}: {rel} is missing")
                continue
            if os.path.getsize(path) != entry[size_key[key]]:
                problems.append(f"rank {r}: {rel} has {os.path.getsize(path)} bytes, manifest says {entry[size_key[key]]}")
                continue
            if "sha256" in entry:
                digests = digests or file_digests(output_dir, r)
                if digests[key] != entry["sha256"][key]:
                    problems.append(f"rank {r}: {rel} does not match its SHA-256")
    return problems
