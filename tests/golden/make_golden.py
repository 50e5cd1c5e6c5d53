#!/usr/bin/env python3
"""Regenerates tests/golden/golden.npz from the REFERENCE'S OWN function text
(oracle/_ref/libcheckers_ref.so, built by oracle/build_ref.py where the reference tree exists).

Vectors (all inputs are reproducible from the seeds below via oracle_lib.synth):
  tab_*     histogram -> (norm_freq, cum_freq) for random and adversarial histograms, both alphabet modes
  lane_*    tiny tensors -> compacted lane bytes + (final_state, byte_count) per lane
  stats_*   tensor -> value histogram, moments, min/max
  clus_*    fingerprints -> cluster ids and anchors
  file_sha  SHA-256 of the three files the reference writers emit for a seeded multi-tensor rank
Run: python tests/golden/make_golden.py
"""
import hashlib
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import ELEM_SIZE, SIDECAR_PER_ELEM, Oracle, RefShim, synth  # noqa: E402

LANE_CASES = [("i8", 1), ("i8", 255), ("i8", 256), ("i8", 257), ("i8", 65537), ("bf16_weight", 2048),
              ("f32_master", 1024), ("f32_exp_avg_sq_lognormal", 777), ("f16_weight", 1500), ("bf16_norm_gain", 4096)]
STATS_CASES = [("bf16_weight", 5000), ("f32_master", 4099), ("f16_weight", 2048), ("i8", 300), ("i32", 1000),
               ("f32_exp_avg_sq", 256)]
FILE_CASES = [("layers.0.w", "bf16_weight", 3000), ("master_weights::layers.0.w", "f32_master", 3000),
              ("optimizer.exp_avg::layers.0.w", "f32_exp_avg", 3000),
              ("optimizer.exp_avg_sq::layers.0.w", "f32_exp_avg_sq", 3000), ("ints", "i8", 700), ("n" * 300, "i32", 513)]


def histograms():
    rng = np.random.default_rng(2024)
    hs = [np.zeros(256, np.uint32), np.ones(256, np.uint32)]
    h = np.zeros(256, np.uint32); h[7] = 1; hs.append(h)
    h = np.zeros(256, np.uint32); h[0] = 2 ** 31; h[255] = 1; hs.append(h)
    h = np.ones(256, np.uint32); h[0] = 10 ** 6; hs.append(h)
    h = np.zeros(256, np.uint32); h[:20] = 5; hs.append(h)
    h = np.zeros(256, np.uint32); h[[0, 60, 61, 188, 189]] = [524288, 200000, 60000, 200001, 59999]; hs.append(h)
    for _ in range(25):
        k = int(rng.integers(1, 257))
        h = np.zeros(256, np.uint32)
        h[rng.choice(256, k, replace=False)] = rng.integers(1, 10 ** int(rng.integers(1, 8)), k)
        hs.append(h)
    return np.stack(hs)


def main():
    if not RefShim.available():
        raise SystemExit("oracle/_ref is not built: run python oracle/build_ref.py first")
    ref, orc = RefShim(), Oracle()
    out = {}
    hs = histograms()
    out["tab_hist"] = hs
    for full in (0, 1):
        res = [ref.normalize(h, bool(full)) for h in hs]
        out[f"tab_nf_{full}"] = np.stack([r[0] for r in res])
        out[f"tab_cf_{full}"] = np.stack([r[1] for r in res])
    for i, (kind, n) in enumerate(LANE_CASES):
        raw, dt = synth(kind, n, 100 + i)
        m = ref.split(raw, dt)[0] if SIDECAR_PER_ELEM[dt] else raw
        t = ref.normalize(ref.byte_histogram(m), False)
        payload, hdr = ref.encode_compact(m, *t[:3])
        out[f"lane_{i}_payload"] = payload
        out[f"lane_{i}_hdr"] = hdr[:, :2].copy()
    for i, (kind, n) in enumerate(STATS_CASES):
        raw, dt = synth(kind, n, 200 + i)
        h, mom, mm = ref.tensor_stats(raw, dt)
        out[f"stats_{i}_hist"], out[f"stats_{i}_mom"], out[f"stats_{i}_mm"] = h, mom, mm
    rng = np.random.default_rng(7)
    names = [f"{p}layers.{l}.w" for l in range(10) for p in ("", "master_weights::", "optimizer.exp_avg::")]
    fps = (rng.normal(0, 1, (len(names), 5)) * [1e-5, 1e-6, 1e-2, 1e-2, 1e-2] + [0, 4e-4, 0, 3, 0.2]).astype(np.float32)
    cid, anchors = ref.build_clusters(names, fps)
    out["clus_fps"], out["clus_id"], out["clus_anchor"] = fps, cid, anchors
    # files: records computed by the oracle (validated against the reference text above), bytes by the reference writers
    st, mt, tb = [], [], ([], [], [])
    for i, (nm, kind, n) in enumerate(FILE_CASES):
        raw, dt = synth(kind, n, 300 + i)
        m, s = orc.split(raw, dt) if SIDECAR_PER_ELEM[dt] else (raw, None)
        nf, cf, xm, _ = ref.normalize(ref.byte_histogram(m), False)
        p, hd, _ = orc.compress_tensor(m, nf, cf, xm)
        st.append(dict(name=nm, dtype=dt, original_bytes=raw.size, num_elements=raw.size // ELEM_SIZE[dt], owns=1,
                       anchor="", lanes=hd, payload=p))
        if s is not None:
            mt.append(dict(name=nm, dtype=dt, num_elements=raw.size // ELEM_SIZE[dt], spe=SIDECAR_PER_ELEM[dt], sidecar=s))
        tb[0].append(nm); tb[1].append(nf); tb[2].append(cf)
    with tempfile.TemporaryDirectory() as d:
        ref.write_states(os.path.join(d, "s"), 2, st)
        ref.write_mantissa(os.path.join(d, "m"), 2, mt)
        ref.write_tables(os.path.join(d, "t"), 2, tb[0], np.stack(tb[1]), np.stack(tb[2]))
        out["file_sha"] = np.array([hashlib.sha256(open(os.path.join(d, k), "rb").read()).hexdigest() for k in "smt"])
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    main()
