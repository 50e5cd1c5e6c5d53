"""Host-side planning of the chunked pipeline (no GPU): chunk cuts and staging offsets."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_plan_functions():
    # streaming.py imports the CUDA library through the package; only its two pure functions are needed here
    src = open(os.path.join(ROOT, "checkers_b200", "streaming.py")).read()
    ns = {}
    start = src.index("def plan_chunks")
    end = src.index("class ChunkedHostPipeline")
    exec(compile(src[start:end], "streaming_plan", "exec"), ns)
    return ns["plan_chunks"], ns["staging_offsets"]


def test_plan_chunks_partitions_in_order():
    plan_chunks, _ = load_plan_functions()
    rng = np.random.default_rng(0)
    for trial in range(200):
        sizes = [int(x) for x in rng.integers(0, 5000, int(rng.integers(0, 40)))]
        cap = int(rng.integers(1, 8000))
        chunks = plan_chunks(sizes, cap)
        flat = [i for c in chunks for i in c]
        assert flat == list(range(len(sizes)))           # every tensor once, order kept
        for c in chunks:
            assert c                                      # no empty chunk
            total = sum(sizes[i] for i in c)
            assert total <= cap or len(c) == 1            # over the cap only when one tensor alone is
        for a, b in zip(chunks, chunks[1:]):              # greedy: the next tensor did not fit
            assert sum(sizes[i] for i in a) + sizes[b[0]] > cap
    assert plan_chunks([], 10) == []
    assert plan_chunks([100], 10) == [[0]]


def test_staging_offsets_are_aligned_and_disjoint():
    _, staging_offsets = load_plan_functions()
    sizes = [1, 255, 256, 257, 0, 4096, 3]
    offs, total = staging_offsets(sizes)
    assert all(o % 256 == 0 for o in offs)
    for (o, n), o2 in zip(zip(offs, sizes), offs[1:] + [total]):
        assert o + n <= o2
    assert total % 256 == 0
