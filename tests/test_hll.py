"""HyperLogLog sketches (the reference's offline study of shared histograms, scripts/llama-3-8b/experiment_2.py):
the numpy oracle against golden values written from the reference's own functions, the CUDA kernel's source
under the block emulator against the oracle, the library's host arithmetic (merge, count) against the oracle,
and -- on a GPU -- the batched device sketches and the shared-vocabulary report."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))
import hll_oracle as H  # noqa: E402
from oracle_lib import ELEM_SIZE, synth  # noqa: E402

GOLDEN = json.load(open(os.path.join(HERE, "golden", "hll_golden.json")))


def _case(c):
    raw, dt = synth(c["kind"], c["n"], c["seed"])
    return raw, dt


def test_oracle_matches_reference_golden():
    regs = []
    for c in GOLDEN["cases"]:
        raw, dt = _case(c)
        r = H.sketch(H.symbols_of(raw, ELEM_SIZE[dt]))
        assert hashlib.sha256(r.tobytes()).hexdigest() == c["sha256"], c["kind"]
        assert [int(x) for x in r[:32]] == c["first_registers"]
        assert H.count(r) == c["estimate"]
        assert abs(c["estimate"] - c["exact_unique"]) <= 0.03 * c["exact_unique"] + 2
        regs.append(r)
    u = H.merge(regs)
    assert hashlib.sha256(u.tobytes()).hexdigest() == GOLDEN["union"]["sha256"]
    assert H.count(u) == GOLDEN["union"]["estimate"]


def test_kernel_source_under_emulator(emu):
    cases = [c for c in GOLDEN["cases"] if c["n"] <= 70000] + [{"kind": "bf16_weight", "n": 140001, "seed": 9}]
    for shift in (0, 1):   # aligned / off a 16-byte boundary
        tensors, n_elem, dts, want = [], [], [], []
        for c in cases:
            raw, dt = _case(c)
            buf = np.zeros(raw.size + 64, np.uint8)
            off = (-buf.ctypes.data) % 64 + shift * ELEM_SIZE[dt]
            a = buf[off:off + raw.size]
            a[:] = raw
            tensors.append(a); n_elem.append(raw.size // ELEM_SIZE[dt]); dts.append(dt)
            want.append(H.sketch(H.symbols_of(raw, ELEM_SIZE[dt])))
        got = emu.hll(tensors, n_elem, dts, grid=5)
        for g, w, c in zip(got, want, cases):
            assert np.array_equal(g, w), c


def test_library_merge_and_count():
    from checkers_b200 import studies
    regs = []
    for c in GOLDEN["cases"]:
        raw, dt = _case(c)
        r = H.sketch(H.symbols_of(raw, ELEM_SIZE[dt]))
        assert studies.hll_count(r) == c["estimate"]
        regs.append(r)
    u = studies.hll_merge(regs)
    assert np.array_equal(u, H.merge(regs))
    assert studies.hll_count(u) == GOLDEN["union"]["estimate"]
    assert studies.hll_count(np.zeros(16384, np.uint8)) == 0.0
    assert studies.histogram_bytes(10.5) == H.shared_histogram_bytes(10.5)


@pytest.mark.gpu
def test_device_sketches_and_report():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200 as chk
    from checkers_b200 import studies
    cases = GOLDEN["cases"] + [{"kind": "f32_master", "n": 1 << 21, "seed": 31}, {"kind": "f32_master", "n": 1 << 21, "seed": 32}]
    ctx = chk.Context(device=0)
    host, dev = [], []
    for i, c in enumerate(cases):
        raw, dt = _case(c)
        t = torch.from_numpy(raw.copy()).cuda()
        host.append((raw, dt)); dev.append(t)
        name = ("optimizer.exp_avg::w." if i >= len(GOLDEN["cases"]) else "t.") + str(i)
        ctx.register_pointer(name, t.data_ptr(), raw.size // ELEM_SIZE[dt], dt)
    ctx.hll_sketch_all()
    sk = []
    for i, (raw, dt) in enumerate(host):
        want = H.sketch(H.symbols_of(raw, ELEM_SIZE[dt]))
        got = ctx.hll_sketch(i)
        assert np.array_equal(got, want), cases[i]
        sk.append(got)
    for c, s in zip(GOLDEN["cases"], sk):
        assert studies.hll_count(s) == c["estimate"]
    # no clusters: sharing changes nothing
    own, shared = ctx.shared_vocabulary_report()
    assert own == shared == sum(H.shared_histogram_bytes(H.count(s)) for s in sk)
    # the two large tensors in one cluster: one histogram over their union
    n = len(cases)
    names = [("optimizer.exp_avg::w." if i >= len(GOLDEN["cases"]) else "t.") + str(i) for i in range(n)]
    ids = [-1] * (n - 2) + [0, 0]
    ctx.set_cluster_info(names, ids, [names[n - 2]])
    own2, shared2 = ctx.shared_vocabulary_report()
    union = H.shared_histogram_bytes(H.count(H.merge(sk[-2:])))
    assert own2 == own
    assert shared2 == own - sum(H.shared_histogram_bytes(H.count(s)) for s in sk[-2:]) + union
    ctx.close()
    # more tensors than one batch of the sketch pass holds
    big = torch.arange(9000 * 16, dtype=torch.int32, device="cuda")
    ctx = chk.Context(device=0)
    for i in range(9000):
        ctx.register_pointer(f"s{i}", big.data_ptr() + i * 64, 16, chk.I32)
    ctx.hll_sketch_all()
    for i in (0, 8191, 8192, 8999):
        want = H.sketch(np.arange(i * 16, i * 16 + 16, dtype=np.uint32))
        assert np.array_equal(ctx.hll_sketch(i), want), i
    ctx.close()
