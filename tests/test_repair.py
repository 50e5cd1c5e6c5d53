"""Prefix-mask Re-Pair estimator.

CPU: the device kernels (emulated) against plain Python restatements of the reference's pair count
and left-to-right rewrite (src/tensor_group_prefix_mask_repair.cpp:373-421).
GPU: the command-line front end against the reference's own CLI (oracle/_ref, compiled unmodified
from the reference tree) on synthetic export directories; all report columns except the timings
must be identical.  Where the reference binary is absent the committed reports under
tests/golden/repair/ (written by that binary for the same seeded inputs) are used instead."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle_lib import REF_REPAIR_CLI, synth

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "repair")
u32p = C.POINTER(C.c_uint32)


def py_apply(tokens, lhs, rhs, new):
    out, i, n = [], 0, len(tokens)
    while i < n:
        if i + 1 < n and tokens[i] == lhs and tokens[i + 1] == rhs:
            out.append(new)
            i += 2
        else:
            out.append(tokens[i])
            i += 1
    return out


def test_pair_table_and_rewrite_emulated(emu):
    rng = np.random.default_rng(3)
    seqs = [rng.integers(0, 4, 5000), rng.integers(0, 300, 3000), np.zeros(2049, np.int64), np.array([7]),
            np.array([1, 1, 1, 2, 1, 1, 1, 1, 2, 2, 2]), rng.integers(0, 2, 1025)]
    for s in seqs:
        t = np.ascontiguousarray(s, np.uint32)
        n = t.size
        keys, counts, first = np.zeros(max(n, 1), np.uint64), np.zeros(max(n, 1), np.uint32), np.zeros(max(n, 1), np.uint32)
        best = np.zeros(4, np.uint32)
        d = emu.lib.emu_repair_count(t.ctypes.data_as(u32p), n, keys.ctypes.data_as(C.POINTER(C.c_uint64)),
                                     counts.ctypes.data_as(u32p), first.ctypes.data_as(u32p), best.ctypes.data_as(u32p), 3)
        want = {}
        for i in range(n - 1):
            k = (int(t[i]) << 32) | int(t[i + 1])
            c, f = want.get(k, (0, i))
            want[k] = (c + 1, f)
        got = {int(keys[i]): (int(counts[i]), int(first[i])) for i in range(d)}
        assert got == want and best[2] == 0
        if want:
            m = max(c for c, _ in want.values())
            assert best[0] == m and best[1] == sum(1 for c, _ in want.values() if c == m)
        # rewrite under a few rules, including lhs == rhs
        vals = sorted(set(int(x) for x in t))[:3]
        for lhs in vals:
            for rhs in vals:
                out = np.zeros(max(n, 1), np.uint32)
                m = emu.lib.emu_repair_apply(t.ctypes.data_as(u32p), n, lhs, rhs, 0x80000005, out.ctypes.data_as(u32p), 2)
                ref = py_apply([int(x) for x in t], lhs, rhs, 0x80000005)
                assert m == len(ref) and [int(x) for x in out[:m]] == ref, (lhs, rhs)
    raw, _ = synth("f32_master", 1000, 1)
    tok = np.zeros(1000, np.uint32)
    emu.lib.emu_repair_mask(raw.ctypes.data_as(C.POINTER(C.c_uint8)), C.c_uint64(1000), 4, 23, tok.ctypes.data_as(u32p), 2)
    assert np.array_equal(tok, raw.view(np.uint32) >> 23)
    raw, _ = synth("bf16_weight", 1000, 1)
    emu.lib.emu_repair_mask(raw.ctypes.data_as(C.POINTER(C.c_uint8)), C.c_uint64(1000), 2, 7, tok.ctypes.data_as(u32p), 2)
    assert np.array_equal(tok, raw.view(np.uint16).astype(np.uint32) >> 7)


# ---------------------------------------------------------------- synthetic export directories
def make_export(root, seed=0):
    """Groups of same-dtype tensors with sizes 2^16..2^19 (log-uniform), as config 3 describes."""
    rng = np.random.default_rng(seed)
    os.makedirs(os.path.join(root, "analysis", "plots"), exist_ok=True)
    os.makedirs(os.path.join(root, "tensors"), exist_ok=True)
    manifest = ["tensor_key,layer,category,state_type,numel,dtype,file"]
    groups = ["state_type,category,group_id,n_layers,layers,representative_layer,c6,c7,c8,c9"]
    spec = [("weights", "mlp.up", "bfloat16", "bf16_weight"), ("master", "mlp.up", "float32", "f32_master"),
            ("exp_avg_sq", "attn.q", "float32", "f32_exp_avg_sq_lognormal"), ("weights", "norm", "float16", "f16_weight")]
    layer = 0
    for gi, (state, cat, dtype, kind) in enumerate(spec):
        layers = []
        for _ in range(3):
            n = int(2 ** rng.uniform(16, 19))
            raw, _ = synth(kind, n, seed * 100 + layer)
            rel = f"tensors/{state}_{cat}_{layer}.bin"
            raw.tofile(os.path.join(root, rel))
            manifest.append(f"{state}.{cat}.{layer},{layer},{cat},{state},{n},{dtype},{rel}")
            layers.append(layer)
            layer += 1
        groups.append(f'{state},{cat},{gi},{len(layers)},"{" ".join(map(str, layers))}",{layers[1]},0,0,0,0')
    open(os.path.join(root, "manifest.csv"), "w").write("\n".join(manifest) + "\n")
    open(os.path.join(root, "analysis", "plots", "grouping_summary.csv"), "w").write("\n".join(groups) + "\n")


def strip_times(path):
    """Report text without its timing fields."""
    out = []
    for line in open(path).read().splitlines():
        if path.endswith(".csv"):
            line = ",".join(line.split(",")[:-1])  # time_ms / total_time_ms is the last column
        out.append(line)
    return out


REPORTS = ("tensor_prefix_mask_repair.csv", "group_prefix_mask_repair.csv", "checkpoint_prefix_mask_repair_summary.txt")
VARIANTS = [("default", []), ("bits8", ["--masked-mantissa-bits", "8"]), ("bits16_rules7", ["--masked-mantissa-bits", "16",
                                                                                          "--max-rules", "7"])]


@pytest.mark.gpu
@pytest.mark.parametrize("tag,extra", VARIANTS)
def test_cli_matches_reference(tmp_path, tag, extra):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from checkers_b200 import repair
    ours = str(tmp_path / "ours")
    make_export(ours, seed=1)
    assert repair.main([ours] + extra) == 0
    if os.path.exists(REF_REPAIR_CLI):
        theirs = str(tmp_path / "theirs")
        make_export(theirs, seed=1)
        subprocess.check_call([REF_REPAIR_CLI, theirs] + extra, stdout=subprocess.DEVNULL)
        ref_dir = os.path.join(theirs, "prefix_mask_repair")
    else:
        ref_dir = os.path.join(GOLD, tag)
    for r in REPORTS:
        assert strip_times(os.path.join(ours, "prefix_mask_repair", r)) == strip_times(os.path.join(ref_dir, r)), (tag, r)


def test_golden_reports_match_reference_cli(tmp_path):
    """Keeps tests/golden/repair in step with the reference binary wherever that binary exists."""
    if not os.path.exists(REF_REPAIR_CLI):
        pytest.skip("oracle/_ref not built")
    for tag, extra in VARIANTS:
        d = str(tmp_path / tag)
        make_export(d, seed=1)
        subprocess.check_call([REF_REPAIR_CLI, d] + extra, stdout=subprocess.DEVNULL)
        for r in REPORTS:
            gold = os.path.join(GOLD, tag, r)
            if os.environ.get("CHK_WRITE_GOLDEN"):
                os.makedirs(os.path.dirname(gold), exist_ok=True)
                shutil.copy(os.path.join(d, "prefix_mask_repair", r), gold)
            assert strip_times(os.path.join(d, "prefix_mask_repair", r)) == strip_times(gold), (tag, r)


@pytest.mark.gpu
def test_cli_large_group_matches_reference(tmp_path):
    """A group at the upper end of the restore configuration's range (2^22 elements) next to a small one."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(REF_REPAIR_CLI):
        pytest.skip("oracle/_ref not built: no reference output for this size")
    from checkers_b200 import repair

    def export(root):
        os.makedirs(os.path.join(root, "analysis", "plots"), exist_ok=True)
        os.makedirs(os.path.join(root, "tensors"), exist_ok=True)
        manifest = ["tensor_key,layer,category,state_type,numel,dtype,file"]
        for layer, (n, kind, dtype) in enumerate([(1 << 22, "f32_master", "float32"), (1 << 16, "f32_master", "float32")]):
            raw, _ = synth(kind, n, 900 + layer)
            rel = f"tensors/master_mlp.up_{layer}.bin"
            raw.tofile(os.path.join(root, rel))
            manifest.append(f"master.mlp.up.{layer},{layer},mlp.up,master,{n},{dtype},{rel}")
        groups = ["state_type,category,group_id,n_layers,layers,representative_layer,c6,c7,c8,c9",
                  'master,mlp.up,0,2,"0 1",0,0,0,0,0']
        open(os.path.join(root, "manifest.csv"), "w").write("\n".join(manifest) + "\n")
        open(os.path.join(root, "analysis", "plots", "grouping_summary.csv"), "w").write("\n".join(groups) + "\n")

    extra = ["--max-rules", "6"]
    ours, theirs = str(tmp_path / "ours"), str(tmp_path / "theirs")
    export(ours)
    export(theirs)
    assert repair.main([ours] + extra) == 0
    subprocess.check_call([REF_REPAIR_CLI, theirs] + extra, stdout=subprocess.DEVNULL)
    for r in REPORTS:
        assert strip_times(os.path.join(ours, "prefix_mask_repair", r)) == \
            strip_times(os.path.join(theirs, "prefix_mask_repair", r)), r
