"""Multi-rank manifest over gloo (world size 2, CPU): each rank contributes its six totals, rank 0
writes manifest.json.  The per-rank summaries come from files the oracle writes, so no GPU is needed."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import numpy as np, torch.distributed as dist
    from oracle_lib import Oracle, synth, ELEM_SIZE
    from checkers_b200 import manifest
    rank, world, out = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), sys.argv[1]
    dist.init_process_group("gloo")
    o = Oracle()
    names, arrays, dtypes = [], [], []
    for i, kind in enumerate(("bf16_weight", "f32_master", "f32_exp_avg")):
        raw, dt = synth(kind, 3000 + 500 * rank, 10 * rank + i)
        names.append(f"p{{i}}"); arrays.append(raw); dtypes.append(dt)
    o.compress_and_save(names, arrays, dtypes, out, rank=rank)
    size = lambda rel: os.path.getsize(os.path.join(out, rel))
    summary = dict(n_tensors=3, n_tables=3, states_bytes=size(f"rank_{{rank}}_states.ansc"),
                   mantissa_bytes=size(f"mantissa/rank_{{rank}}_mantissa.mant"),
                   dict_bytes=size(f"tables/rank_{{rank}}_tables.dict"),
                   original_bytes=sum(a.size for a in arrays), digests=manifest.file_digests(out, rank))
    rows = manifest.gather_summaries(summary)
    assert len(rows) == world and rows[rank] == summary
    assert manifest.start_gather(summary).result() == rows   # the non-blocking form gives the same rows
    if rank == 0:
        manifest.write_manifest(out, manifest.build_manifest(rows))
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_ranks_write_one_manifest(tmp_path):
    out = str(tmp_path / "ckpt")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29571", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), out], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(2)]
    logs = [p.communicate(timeout=240)[0].decode() for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    m = json.load(open(os.path.join(out, "manifest.json")))
    assert m["world_size"] == 2 and len(m["ranks"]) == 2
    r0, r1 = m["ranks"]
    assert r0["states_bytes_offset"] == 0 and r1["states_bytes_offset"] == r0["states_bytes"]
    assert r1["original_bytes_offset"] == r0["original_bytes"]
    for r in (r0, r1):
        for key, rel in r["files"].items():
            assert os.path.getsize(os.path.join(out, rel)) == r[{"states": "states_bytes", "mantissa": "mantissa_bytes",
                                                                  "tables": "dict_bytes"}[key]]
    from checkers_b200 import manifest
    assert manifest.verify_manifest(out) == []
    assert all(len(r["sha256"][k]) == 64 for r in (r0, r1) for k in ("states", "mantissa", "tables"))
    victim = os.path.join(out, r1["files"]["mantissa"])
    blob = bytearray(open(victim, "rb").read())
    blob[len(blob) // 2] ^= 1
    open(victim, "wb").write(bytes(blob))
    problems = manifest.verify_manifest(out)
    assert len(problems) == 1 and "rank 1" in problems[0] and "SHA-256" in problems[0]
    assert manifest.verify_manifest(out, ranks=[0]) == []
    t = m["totals"]
    assert t["original_bytes"] == r0["original_bytes"] + r1["original_bytes"]
    assert t["compressed_bytes"] == sum(r[k] for r in (r0, r1) for k in ("states_bytes", "mantissa_bytes", "dict_bytes"))


def test_single_process_manifest():
    from checkers_b200 import manifest
    rows = manifest.gather_summaries(dict(n_tensors=1, n_tables=1, states_bytes=10, mantissa_bytes=5, dict_bytes=3,
                                          original_bytes=20))
    m = manifest.build_manifest(rows)
    assert m["world_size"] == 1 and m["totals"]["compressed_bytes"] == 18 and abs(m["totals"]["ratio"] - 20 / 18) < 1e-12
