"""Cost of a shared 32-bit model (the reference's offline study, scripts/llama-3-8b/experiment_2_1.py): the numpy
oracle against golden values written from the reference's own functions, the CUDA kernels' source under the block
emulator against the oracle, and -- on a GPU -- Context.shared_model_cost.  Tolerance: 1e-9 relative on the
stream bytes (sums of doubles in another order); vocabulary sizes are exact."""
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))
sys.path.insert(0, os.path.join(HERE, "golden"))
import xe_oracle as X  # noqa: E402
from make_xe_golden import TENSORS, symbols  # noqa: E402
from oracle_lib import ELEM_SIZE, synth  # noqa: E402

GOLDEN = json.load(open(os.path.join(HERE, "golden", "xe_golden.json")))
REL = 1e-9


def test_oracle_matches_reference_golden():
    for grp in GOLDEN["groups"]:
        b, v = X.shared_model_cost([symbols(i) for i in grp["members"]])
        assert v == grp["vocabulary"]
        assert abs(b - grp["stream_bytes"]) <= REL * max(1.0, grp["stream_bytes"])
    for i, t in enumerate(GOLDEN["tensors"]):
        b, v = X.shared_model_cost([symbols(i)])
        assert v * 8 == t["own_model_bytes"]
        assert abs(b - t["own_stream_bytes"]) <= REL * max(1.0, t["own_stream_bytes"])


def test_kernel_source_under_emulator(emu):
    for grp in GOLDEN["groups"][:5]:
        raws = [synth(*TENSORS[i]) for i in grp["members"]]
        tensors = [r for r, _ in raws]
        n_elem = [r.size // ELEM_SIZE[dt] for r, dt in raws]
        total = sum(n_elem)
        cap = 1024
        while cap < 2 * total:
            cap *= 2
        v = grp["vocabulary"]
        p = max(14, int(np.ceil(np.log2(max(v, 2)))) + 1)
        vocab, c_max, overflow, norm_sum, bits = emu.model_cost(tensors, n_elem, [dt for _, dt in raws], cap, p)
        assert overflow == 0 and int(vocab) == v
        scale = float(1 << p)
        norm_max = max(np.floor(c_max * (scale / total)), 1.0)
        norm_max = max(norm_max + scale - (norm_sum + norm_max), 1.0)
        got = (bits + c_max * np.log2(scale / norm_max)) / 8.0
        assert abs(got - grp["stream_bytes"]) <= REL * max(1.0, grp["stream_bytes"]), (got, grp)


@pytest.mark.gpu
def test_device_shared_model_cost():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200 as chk
    ctx = chk.Context(device=0)
    keep = []
    for i, (kind, n, seed) in enumerate(TENSORS):
        raw, dt = synth(kind, n, seed)
        t = torch.from_numpy(raw.copy()).cuda()
        keep.append(t)
        ctx.register_pointer(f"t{i}", t.data_ptr(), raw.size // ELEM_SIZE[dt], dt)
    for grp in GOLDEN["groups"]:
        b, v = ctx.shared_model_cost(grp["members"])
        assert v == grp["vocabulary"], grp
        assert abs(b - grp["stream_bytes"]) <= REL * max(1.0, grp["stream_bytes"]), (b, grp)
    for i, t in enumerate(GOLDEN["tensors"]):
        b, v = ctx.shared_model_cost([i])
        assert v * 8 == t["own_model_bytes"]
        assert abs(b - t["own_stream_bytes"]) <= REL * max(1.0, t["own_stream_bytes"])
    assert ctx.shared_model_cost([]) == (0.0, 0)
    with pytest.raises(chk.CheckersError):
        ctx.shared_model_cost([99])
    ctx.close()
