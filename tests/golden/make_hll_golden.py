"""Writes tests/golden/hll_golden.json from the reference's own HyperLogLog functions.

Run where the Checkers tree is available (CHECKERS_REFERENCE=<path>):  python tests/golden/make_hll_golden.py
The inputs are seeded synthetic tensors (tests/oracle_lib.synth); the file keeps, per case, the SHA-256 of the
16384 registers, a few register values and the cardinality estimate, and for the union of all cases the same."""
import hashlib
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import ELEM_SIZE, synth  # noqa: E402

CASES = [("f32_master", 200000, 1), ("f32_exp_avg", 65537, 2), ("f32_exp_avg_sq_lognormal", 300001, 3),
         ("bf16_weight", 500000, 4), ("i8", 4096, 5), ("i32", 70000, 6), ("f32_master", 1, 7), ("f16_weight", 33333, 8)]


def main():
    ref = os.environ.get("CHECKERS_REFERENCE", "")
    path = os.path.join(ref, "scripts", "llama-3-8b", "experiment_2.py")
    if not os.path.exists(path):
        raise SystemExit("set CHECKERS_REFERENCE to the Checkers tree")
    spec = importlib.util.spec_from_file_location("checkers_experiment_2", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out, all_regs = {"cases": []}, []
    for kind, n, seed in CASES:
        raw, dt = synth(kind, n, seed)
        es = ELEM_SIZE[dt]
        sym = raw.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[es]).astype(np.uint32)
        regs = mod.hll_create()
        mod.hll_add_uint32(regs, sym)
        all_regs.append(regs)
        out["cases"].append({"kind": kind, "n": n, "seed": seed, "sha256": hashlib.sha256(regs.tobytes()).hexdigest(),
                             "first_registers": [int(x) for x in regs[:32]], "estimate": mod.hll_count(regs),
                             "exact_unique": int(np.unique(sym).size)})
    merged = mod.hll_merge(all_regs)
    out["union"] = {"sha256": hashlib.sha256(merged.tobytes()).hexdigest(), "estimate": mod.hll_count(merged)}
    with open(os.path.join(HERE, "hll_golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", len(out["cases"]), "cases")


if __name__ == "__main__":
    main()
