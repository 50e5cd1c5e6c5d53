"""Chunked host pipeline (checkers_b200/streaming.py) on the GPU: every part it
writes must be the file triple the oracle produces for that chunk's tensors,
and restore must return the input bytes."""
import os

import numpy as np
import pytest

from oracle_lib import BF16, F32, synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

KINDS = [("bf16_weight", BF16), ("f32_master", F32), ("f32_exp_avg", F32), ("f32_exp_avg_sq", F32)]


def read_part(d, rank):
    out = []
    for rel in (f"rank_{rank}_states.ansc", f"mantissa/rank_{rank}_mantissa.mant", f"tables/rank_{rank}_tables.dict"):
        with open(os.path.join(d, rel), "rb") as f:
            out.append(f.read())
    return out


@pytest.mark.parametrize("workers", [1, 2, 3])
def test_parts_match_oracle_and_round_trip(oracle, tmp_path, workers):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from checkers_b200.streaming import ChunkedHostPipeline, HostTensor

    sizes = [70001, 4096, 262144, 1, 33333, 100000, 65536]
    host, tensors, outs = [], [], []
    for i, n in enumerate(sizes):
        for j, (kind, dt) in enumerate(KINDS):
            raw, dt2 = synth(kind, n, 100 * i + j)
            assert dt2 == dt
            t = torch.from_numpy(raw.view(np.uint8).copy()).pin_memory()
            host.append(raw.view(np.uint8).copy())
            tensors.append(HostTensor(f"{kind}::layer{i}", t, dt))
            outs.append(torch.zeros_like(t).pin_memory())
    pipe = ChunkedHostPipeline(tensors, device=0, rank=2, chunk_bytes=1 << 20, workers=workers)
    assert len(pipe.chunks) >= 3
    assert sum(len(ch.items) for ch in pipe.chunks) == len(tensors)
    for _ in range(2):  # the second pass reuses every context and staging buffer
        pipe.compress()
    assert pipe.save(str(tmp_path / "gpu")) == len(pipe.chunks)

    k = 0
    for ch in pipe.chunks:
        m = len(ch.items)
        ref_dir = str(tmp_path / f"cpu_{ch.index}")
        oracle.compress_and_save([t.name for t in ch.items], host[k:k + m], [t.dtype for t in ch.items], ref_dir, rank=2)
        got = read_part(str(tmp_path / "gpu" / f"part_{ch.index:04d}"), 2)
        for a, b, what in zip(got, read_part(ref_dir, 2), ("states", "mantissa", "tables")):
            assert a == b, f"part {ch.index}: {what} file differs from the oracle's"
        k += m
    s = pipe.summary()
    assert s["n_tensors"] == len(tensors) and s["original_bytes"] == sum(h.size for h in host)

    pipe.restore(outs)
    for o, h, t in zip(outs, host, tensors):
        assert np.array_equal(o.numpy(), h), t.name
    pipe.close()


def test_pipeline_with_container_version3(tmp_path):
    """The host pipeline with every context set to container version 3: smaller parts, lossless through memory
    and through files."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from checkers_b200.streaming import ChunkedHostPipeline, HostTensor
    from oracle_lib import synth
    tensors, outs = [], []
    for i in range(24):
        kind = ("bf16_weight", "f32_master", "f32_exp_avg", "f32_exp_avg_sq_lognormal")[i % 4]
        # a few large tensors: their copy to the device takes milliseconds, and the kernels must wait for it
        raw, dt = synth(kind, (3 << 20) + 5 if i in (1, 2, 9) else 100000 + 17 * i, 500 + i)
        t = torch.from_numpy(raw.copy()).pin_memory()
        tensors.append(HostTensor(f"optimizer.exp_avg::w.{i}" if i % 4 == 2 else f"w.{i}", t, dt))
        outs.append(torch.zeros_like(t).pin_memory())
    sizes = {}
    for version in (2, 3):
        pipe = ChunkedHostPipeline(tensors, device=0, rank=0, chunk_bytes=2 << 20, workers=3,
                                   options={"format_version": version})
        pipe.compress()
        s = pipe.summary()
        sizes[version] = s["states_bytes"] + s["mantissa_bytes"]
        for o in outs:
            o.zero_()
        pipe.restore(outs)
        for t, o in zip(tensors, outs):
            assert torch.equal(t.tensor, o), (version, t.name)
        d = str(tmp_path / f"v{version}")
        pipe.save(d)
        pipe.close()
        again = ChunkedHostPipeline(tensors, device=0, rank=0, chunk_bytes=2 << 20, workers=2,
                                    options={"format_version": version})
        again.load(d)
        for o in outs:
            o.zero_()
        again.restore(outs)
        for t, o in zip(tensors, outs):
            assert torch.equal(t.tensor, o), (version, t.name, "from files")
        again.close()
    assert sizes[3] < 0.93 * sizes[2]
