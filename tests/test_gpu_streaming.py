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


def test_pipeline_with_tensors_sliced_from_one_buffer():
    """Tensors that are slices of one pinned buffer (moved by merged copies): registered out of address order, with
    gaps, one of them twice, odd sizes; restored into slices of another buffer laid out differently."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from checkers_b200.streaming import ChunkedHostPipeline, HostTensor
    from oracle_lib import synth, ELEM_SIZE
    rng = np.random.default_rng(8)
    specs = [("bf16_weight", 200001), ("f32_master", 150000), ("f32_exp_avg", 99999), ("i8", 12345), ("bf16_weight", 64),
             ("f32_exp_avg_sq_lognormal", 300000), ("f16_weight", 77777)]
    raws = [synth(k, n, 900 + i) for i, (k, n) in enumerate(specs)]
    total = sum(r.size for r, _ in raws)
    src = torch.zeros(total + 4096, dtype=torch.uint8).pin_memory()
    dst = torch.zeros(2 * total + 8192, dtype=torch.uint8).pin_memory()
    offs, at = [], 0
    for i, (r, dt) in enumerate(raws):
        at += 0 if i % 2 else 3 * ELEM_SIZE[dt]          # every second tensor follows its neighbour without a gap
        at = (at + ELEM_SIZE[dt] - 1) // ELEM_SIZE[dt] * ELEM_SIZE[dt]
        offs.append(at)
        src[at:at + r.size] = torch.from_numpy(r.copy())
        at += r.size
    order = [3, 0, 6, 1, 5, 2, 4, 1]                      # out of address order; tensor 1 twice
    tensors, targets, want = [], [], []
    d_at = 0
    for j, i in enumerate(order):
        r, dt = raws[i]
        tensors.append(HostTensor(f"t{j}.{i}", src[offs[i]:offs[i] + r.size], dt))
        d_at = (d_at + 7) // 8 * 8 + (8 if j % 3 == 0 else 0)
        targets.append(dst[d_at:d_at + r.size])
        d_at += r.size
        want.append(torch.from_numpy(r.copy()))
    for chunk in (1 << 20, 300000):
        pipe = ChunkedHostPipeline(tensors, device=0, rank=0, chunk_bytes=chunk, workers=3)
        pipe.compress()
        dst.zero_()
        pipe.restore(targets)
        for t, w, ht in zip(targets, want, tensors):
            assert torch.equal(t, w), (chunk, ht.name)
        pipe.close()
