"""Committed golden vectors (tests/golden/golden.npz, generated from the reference's own function
text by tests/golden/make_golden.py).  The oracle must reproduce them on any machine; the CUDA
library must reproduce the file hashes through its C ABI on a GPU."""
import hashlib
import os

import numpy as np
import pytest

from oracle_lib import ELEM_SIZE, SIDECAR_PER_ELEM, synth

HERE = os.path.dirname(os.path.abspath(__file__))
import sys
sys.path.insert(0, os.path.join(HERE, "golden"))
from make_golden import FILE_CASES, LANE_CASES, STATS_CASES  # noqa: E402

G = np.load(os.path.join(HERE, "golden", "golden.npz"))


def test_tables(oracle):
    for full in (0, 1):
        for h, nf, cf in zip(G["tab_hist"], G[f"tab_nf_{full}"], G[f"tab_cf_{full}"]):
            a = oracle.normalize(h, bool(full))
            assert np.array_equal(a[0], nf) and np.array_equal(a[1], cf)
    import checkers_b200 as chk   # the library's own host normaliser
    for full in (0, 1):
        for h, nf, cf in zip(G["tab_hist"], G[f"tab_nf_{full}"], G[f"tab_cf_{full}"]):
            a = chk.normalize_histogram(h, bool(full))
            assert np.array_equal(a[0], nf) and np.array_equal(a[1], cf)


def test_lane_streams(oracle, emu):
    from emu_lib import aligned
    for i, (kind, n) in enumerate(LANE_CASES):
        raw, dt = synth(kind, n, 100 + i)
        m = oracle.split(raw, dt)[0] if SIDECAR_PER_ELEM[dt] else raw
        t = oracle.normalize(oracle.byte_histogram(m), False)
        p, hd, is_raw = oracle.compress_tensor(m, *t[:3])
        gold_p, gold_h = G[f"lane_{i}_payload"], G[f"lane_{i}_hdr"]
        if is_raw:
            assert int(gold_h[:, 1].sum()) >= m.size
        else:
            assert np.array_equal(p, gold_p) and np.array_equal(hd[:, :2], gold_h), (kind, n)
        # and the CUDA kernels (emulated) on the same input
        a = aligned(raw.size); a[:] = raw
        payload, poff, hdrs, rawf, _ = emu.encode([a], [ELEM_SIZE[dt]], [SIDECAR_PER_ELEM[dt]], [0], t[0], t[1])
        if not rawf[0]:
            assert np.array_equal(payload[:int(poff[1])], gold_p) and np.array_equal(hdrs[0][:, :2], gold_h), (kind, n)


def test_stats(oracle):
    for i, (kind, n) in enumerate(STATS_CASES):
        raw, dt = synth(kind, n, 200 + i)
        h, mom, mm = oracle.tensor_stats(raw, dt)
        assert np.array_equal(h, G[f"stats_{i}_hist"])
        assert np.array_equal(mom.view(np.uint32), G[f"stats_{i}_mom"].view(np.uint32))
        assert np.array_equal(mm.view(np.uint32), G[f"stats_{i}_mm"].view(np.uint32))


def test_clusters(oracle):
    names = [f"{p}layers.{l}.w" for l in range(10) for p in ("", "master_weights::", "optimizer.exp_avg::")]
    cid, anchors = oracle.build_clusters(names, G["clus_fps"])
    assert np.array_equal(cid, G["clus_id"]) and np.array_equal(anchors, G["clus_anchor"])


def _file_inputs():
    names, arrays, dtypes = [], [], []
    for i, (nm, kind, n) in enumerate(FILE_CASES):
        raw, dt = synth(kind, n, 300 + i)
        names.append(nm); arrays.append(raw); dtypes.append(dt)
    return names, arrays, dtypes


def _sha(d, rank):
    rel = (f"rank_{rank}_states.ansc", f"mantissa/rank_{rank}_mantissa.mant", f"tables/rank_{rank}_tables.dict")
    return [hashlib.sha256(open(os.path.join(d, r), "rb").read()).hexdigest() for r in rel]


def test_files_oracle(oracle, tmp_path):
    names, arrays, dtypes = _file_inputs()
    oracle.compress_and_save(names, arrays, dtypes, str(tmp_path), rank=2)
    assert _sha(str(tmp_path), 2) == list(G["file_sha"])


@pytest.mark.gpu
def test_files_gpu(tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200 as chk
    names, arrays, dtypes = _file_inputs()
    dev = [torch.from_numpy(a.copy()).cuda() for a in arrays]
    torch.cuda.synchronize()
    ctx = chk.Context(device=0, rank=2)
    for n, t, dt in zip(names, dev, dtypes):
        ctx.register_pointer(n, t.data_ptr(), t.numel() // ELEM_SIZE[dt], dt)
    ctx.compress_and_save(str(tmp_path))
    assert _sha(str(tmp_path), 2) == list(G["file_sha"])
    ctx.close()
