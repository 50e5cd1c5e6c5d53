"""Pins the oracle restatement to the reference's own function text.

oracle/_ref/libcheckers_ref.so is built by oracle/build_ref.py from function
bodies cut out of the reference tree (kernels run on a CPU block emulator).
Every comparison here is bit-exact.  Skipped where that build is absent."""
import numpy as np
import pytest

from oracle_lib import ELEM_SIZE, SIDECAR_PER_ELEM, synth

CASES = [("bf16_weight", 8192), ("f32_master", 4096), ("f32_exp_avg", 2048), ("f32_exp_avg_sq", 2501),
         ("f32_exp_avg_sq_lognormal", 1500), ("bf16_norm_gain", 4097), ("f16_weight", 3000), ("i8", 1000), ("i32", 777),
         ("f32_uniform_bits", 3000), ("bf16_weight", 3), ("f32_master", 1), ("i8", 255), ("i8", 256), ("i8", 257)]


@pytest.mark.parametrize("kind,n", CASES)
def test_split_hist_table_encode(oracle, ref, kind, n):
    raw, dt = synth(kind, n, 0)
    if SIDECAR_PER_ELEM[dt]:
        m1, s1 = oracle.split(raw, dt)
        m2, s2 = ref.split(raw, dt)
        assert np.array_equal(m1, m2) and np.array_equal(s1, s2)
    else:
        m1 = raw
    h1, h2 = oracle.byte_histogram(m1), ref.byte_histogram(m1)
    assert np.array_equal(h1, h2)
    for full in (False, True):
        t1, t2 = oracle.normalize(h1, full), ref.normalize(h1, full)
        assert all(np.array_equal(a, b) for a, b in zip(t1[:3], t2[:3])) and t1[3] == t2[3]
        p1, hd1, raw1 = oracle.compress_tensor(m1, *t1[:3])
        p2, hd2 = ref.encode_compact(m1, *t2[:3])
        total = int(hd2[:, 1].sum())
        assert raw1 == (total >= m1.size)  # passthrough rule of compress_tensor
        if not raw1:
            assert np.array_equal(p1, p2)
            assert np.array_equal(hd1[:, :2], hd2[:, :2])  # final_state, byte_count
            assert np.array_equal(hd1[:, 2], np.concatenate([[0], np.cumsum(hd2[:-1, 1])]).astype(np.uint32))
        if t1[3] == 4096:
            rc, dec = oracle.decode_tensor(p1, hd1, raw1, t1[0], t1[1], m1.size)
            assert rc == 0 and np.array_equal(dec, m1)


def test_normalize_random_and_adversarial(oracle, ref):
    rng = np.random.default_rng(1)
    hists = [np.zeros(256, np.uint32), np.ones(256, np.uint32), np.full(256, 2 ** 24 - 1, np.uint32)]
    h = np.zeros(256, np.uint32); h[7] = 1; hists.append(h)
    h = np.zeros(256, np.uint32); h[0] = 2 ** 31; h[255] = 1; hists.append(h)
    h = np.ones(256, np.uint32); h[0] = 10 ** 6; hists.append(h)           # many ties at the minimum
    h = np.zeros(256, np.uint32); h[:20] = 5; hists.append(h)              # all fractions equal
    for _ in range(120):
        k = int(rng.integers(1, 257))
        h = np.zeros(256, np.uint32)
        h[rng.choice(256, k, replace=False)] = rng.integers(1, 10 ** int(rng.integers(1, 8)), k)
        hists.append(h)
    for h in hists:
        for full in (False, True):
            a, b = oracle.normalize(h, full), ref.normalize(h, full)
            assert all(np.array_equal(x, y) for x, y in zip(a[:3], b[:3])), (h, full)


@pytest.mark.parametrize("kind,n", [("bf16_weight", 5000), ("f32_master", 4099), ("f16_weight", 2048), ("i8", 300),
                                    ("i32", 1000), ("bf16_norm_gain", 513), ("f32_exp_avg_sq", 256)])
def test_tensor_stats(oracle, ref, kind, n):
    raw, dt = synth(kind, n, 3)
    for bins in (256, 64, 4096):
        a, b = oracle.tensor_stats(raw, dt, bins), ref.tensor_stats(raw, dt, bins)
        assert np.array_equal(a[0], b[0])
        assert np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))
        assert np.array_equal(a[2].view(np.uint32), b[2].view(np.uint32))


def test_clusters(oracle, ref):
    rng = np.random.default_rng(5)
    names, fps = [], []
    for l in range(12):
        for prefix, scale in (("", 1.0), ("master_weights::", 1.0), ("optimizer.exp_avg::", 1e-2),
                              ("optimizer.exp_avg_sq::", 1e-4)):
            names.append(f"{prefix}layers.{l}.w")
            base = np.array([0.0, 4e-4, 0.0, 3.0, 0.2]) * scale
            jitter = rng.normal(0, 1, 5) * np.array([1e-5, 1e-6, 1e-2, 1e-2, 1e-2]) * (5 if l % 4 == 0 else 1)
            fps.append(base + jitter)
    fps = np.array(fps, np.float32)
    c1, a1 = oracle.build_clusters(names, fps)
    c2, a2 = ref.build_clusters(names, fps)
    assert np.array_equal(c1, c2) and np.array_equal(a1, a2)
    assert len(a1) >= 1
    # degenerate inputs
    for nm, fp in (([], np.zeros((0, 5), np.float32)), (["only"], np.zeros((1, 5), np.float32)),
                   (["a", "b", "c"], np.zeros((3, 5), np.float32))):
        x, y = oracle.build_clusters(nm, fp), ref.build_clusters(nm, fp)
        assert np.array_equal(x[0], y[0]) and np.array_equal(x[1], y[1])


def test_file_writers(oracle, ref, tmp_path):
    """The oracle's three files equal what the reference's writers emit for the same records."""
    import os
    kinds = [("w.0", "bf16_weight", 3000), ("master_weights::w.0", "f32_master", 2000), ("ints", "i8", 700),
             ("x" * 300, "f32_exp_avg", 513)]
    names, arrays, dtypes = [], [], []
    for i, (nm, kind, n) in enumerate(kinds):
        raw, dt = synth(kind, n, i)
        names.append(nm); arrays.append(raw); dtypes.append(dt)
    d = str(tmp_path / "o")
    oracle.compress_and_save(names, arrays, dtypes, d, rank=5)
    st, mt, tb = [], [], ([], [], [])
    for nm, raw, dt in zip(names, arrays, dtypes):
        m, s = oracle.split(raw, dt) if SIDECAR_PER_ELEM[dt] else (raw, None)
        nf, cf, xm, _ = oracle.normalize(oracle.byte_histogram(m), False)
        p, hd, _ = oracle.compress_tensor(m, nf, cf, xm)
        st.append(dict(name=nm, dtype=dt, original_bytes=raw.size, num_elements=raw.size // ELEM_SIZE[dt], owns=1,
                       anchor="", lanes=hd, payload=p))
        if s is not None:
            mt.append(dict(name=nm, dtype=dt, num_elements=raw.size // ELEM_SIZE[dt], spe=SIDECAR_PER_ELEM[dt], sidecar=s))
        tb[0].append(nm); tb[1].append(nf); tb[2].append(cf)
    r = str(tmp_path / "r")
    os.makedirs(r)
    ref.write_states(os.path.join(r, "s"), 5, st)
    ref.write_mantissa(os.path.join(r, "m"), 5, mt)
    ref.write_tables(os.path.join(r, "t"), 5, tb[0], np.stack(tb[1]), np.stack(tb[2]))
    assert open(os.path.join(r, "s"), "rb").read() == open(os.path.join(d, "rank_5_states.ansc"), "rb").read()
    assert open(os.path.join(r, "m"), "rb").read() == open(os.path.join(d, "mantissa/rank_5_mantissa.mant"), "rb").read()
    assert open(os.path.join(r, "t"), "rb").read() == open(os.path.join(d, "tables/rank_5_tables.dict"), "rb").read()
