"""Writes tests/golden/xe_golden.json from the reference's own shared-model study functions.

Run where the Checkers tree is available (CHECKERS_REFERENCE=<path>):  python tests/golden/make_xe_golden.py
Inputs are seeded synthetic tensors (tests/oracle_lib.synth).  Per group: the stream bytes and vocabulary size of
cluster_cost_worker over tensor_stats_worker's summaries; per tensor: its own-model stream and model bytes."""
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import ELEM_SIZE, synth  # noqa: E402

TENSORS = [("f32_master", 60000, 11), ("f32_master", 50001, 12), ("f32_exp_avg", 40000, 13), ("bf16_weight", 300000, 14),
           ("bf16_weight", 200001, 15), ("i8", 5000, 16), ("f32_exp_avg_sq_lognormal", 30000, 17), ("f32_master", 1, 18)]
GROUPS = [[0, 1], [0, 1, 2], [3, 4], [3, 4, 5], [6], [7], [0, 1, 2, 3, 4, 5, 6, 7]]


def symbols(i):
    kind, n, seed = TENSORS[i]
    raw, dt = synth(kind, n, seed)
    return raw.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[ELEM_SIZE[dt]]).astype(np.uint32)


def main():
    ref = os.environ.get("CHECKERS_REFERENCE", "")
    path = os.path.join(ref, "scripts", "llama-3-8b", "experiment_2_1.py")
    if not os.path.exists(path):
        raise SystemExit("set CHECKERS_REFERENCE to the Checkers tree")
    spec = importlib.util.spec_from_file_location("checkers_experiment_2_1", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    stats = [mod.tensor_stats_worker(symbols(i)) for i in range(len(TENSORS))]
    out = {"tensors": [{"kind": k, "n": n, "seed": s, "own_stream_bytes": st["xe_stream_bytes"],
                        "own_model_bytes": st["per_tensor_model_bytes"]}
                       for (k, n, s), st in zip(TENSORS, stats)], "groups": []}
    for g in GROUPS:
        b, v = mod.cluster_cost_worker((len(out["groups"]), [{"vocab": stats[i]["vocab"], "counts": stats[i]["counts"]} for i in g]))
        out["groups"].append({"members": g, "stream_bytes": b, "vocabulary": v})
    with open(os.path.join(HERE, "xe_golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", len(out["groups"]), "groups")


if __name__ == "__main__":
    main()
