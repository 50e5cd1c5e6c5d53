"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bit-exact everywhere: integer/byte work, and the float statistics too (the
kernel keeps the reference's accumulation order and fuses nothing)."""
import os

import numpy as np
import pytest

from oracle_lib import (BF16, ELEM_SIZE, F16, F32, I8, I32, SIDECAR_PER_ELEM, UNKNOWN, Oracle, synth)

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def chk():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200
    return checkers_b200


def dev_bytes(arr, misalign=0):
    """uint8 device tensor holding arr's bytes, optionally starting `misalign` bytes into its allocation."""
    a = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    buf = torch.zeros(a.size + misalign + 64, dtype=torch.uint8, device="cuda")
    view = buf[misalign:misalign + a.size]
    view.copy_(torch.from_numpy(a.copy()))
    torch.cuda.synchronize()  # the library works on its own stream
    return view


def read_files(d, rank=0):
    out = []
    for rel in (f"rank_{rank}_states.ansc", f"mantissa/rank_{rank}_mantissa.mant", f"tables/rank_{rank}_tables.dict"):
        with open(os.path.join(d, rel), "rb") as f:
            out.append(f.read())
    return out


MIXED = [  # (name, kind, elements, misalign bytes)
    ("layers.0.w", "bf16_weight", 262144, 0),
    ("master_weights::layers.0.w", "f32_master", 262144, 0),
    ("optimizer.exp_avg::layers.0.w", "f32_exp_avg", 262144, 0),
    ("optimizer.exp_avg_sq::layers.0.w", "f32_exp_avg_sq", 262144, 0),
    ("layers.0.norm", "bf16_norm_gain", 4096, 0),
    ("odd.bf16", "bf16_weight", 70001, 0),
    ("odd.f32", "f32_master", 10001, 0),
    ("tiny.1", "f32_master", 1, 0),
    ("tiny.3", "bf16_weight", 3, 0),
    ("sub256", "i8", 255, 0),
    ("exact256", "i8", 256, 0),
    ("plus1", "i8", 257, 0),
    ("bytes.65537", "i8", 65537, 0),
    ("int32.t", "i32", 5000, 0),
    ("half.t", "f16_weight", 33000, 0),
    ("noise.f32", "f32_uniform_bits", 20000, 0),
    ("misaligned.f32", "f32_master", 30000, 4),
    ("misaligned.bf16", "bf16_weight", 30001, 2),
    ("lognormal", "f32_exp_avg_sq_lognormal", 100000, 0),
]


def make_mixed(seed=0):
    names, host, dev, dtypes = [], [], [], []
    for i, (name, kind, n, mis) in enumerate(MIXED):
        raw, dt = synth(kind, n, seed * 1000 + i)
        names.append(name)
        host.append(raw.copy())
        dev.append(dev_bytes(raw, mis))
        dtypes.append(dt)
    return names, host, dev, dtypes


def register_all(ctx, names, dev, dtypes):
    for n, t, dt in zip(names, dev, dtypes):
        ctx.register_pointer(n, t.data_ptr(), t.numel() // ELEM_SIZE[dt], dt)


def test_stage_split_and_histogram(chk, oracle):
    ctx = chk.Context(device=0)
    for kind, n in [("bf16_weight", 100003), ("f32_master", 65536), ("f16_weight", 4097)]:
        raw, dt = synth(kind, n, 7)
        src = dev_bytes(raw)
        masked = torch.zeros(raw.size + 64, dtype=torch.uint8, device="cuda")
        side = torch.zeros(n * SIDECAR_PER_ELEM[dt] + 64, dtype=torch.uint8, device="cuda")
        ctx.split(src.data_ptr(), n, dt, masked.data_ptr(), side.data_ptr())
        m_ref, s_ref = oracle.split(raw, dt)
        assert np.array_equal(masked[:raw.size].cpu().numpy(), m_ref)
        assert np.array_equal(side[:s_ref.size].cpu().numpy(), s_ref)
        h = ctx.byte_histogram(masked.data_ptr(), raw.size)
        assert np.array_equal(h, oracle.byte_histogram(m_ref))
        # misaligned source for the histogram
        h2 = ctx.byte_histogram(masked.data_ptr() + 3, raw.size - 3)
        assert np.array_equal(h2, oracle.byte_histogram(m_ref[3:]))
    ctx.close()


def test_normalize_matches_oracle(chk, oracle):
    rng = np.random.default_rng(3)
    for trial in range(200):
        k = int(rng.integers(1, 257))
        hist = np.zeros(256, np.uint32)
        idx = rng.choice(256, k, replace=False)
        hist[idx] = rng.integers(1, 10 ** int(rng.integers(1, 7)), k)
        for full in (False, True):
            for rep in (False, True):
                a = chk.normalize_histogram(hist, full, rep)
                b = oracle.normalize(hist, full, repaired=rep)
                assert all(np.array_equal(x, y) for x, y in zip(a[:3], b[:3])) and a[3] == b[3]


def test_files_identical_to_oracle_singletons(chk, oracle, tmp_path):
    names, host, dev, dtypes = make_mixed()
    # entries the reference drops: null pointer, zero elements, unknown dtype
    ctx = chk.Context(device=0, rank=3)
    ctx.register_pointer("null.ptr", 0, 100, F32)
    register_all(ctx, names, dev, dtypes)
    ctx.register_pointer("zero.elems", dev[0].data_ptr(), 0, F32)
    ctx.register_pointer("unknown.dtype", dev[0].data_ptr(), 16, UNKNOWN)
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    ctx.compress_and_save(out_gpu)
    oracle.compress_and_save(["null.ptr"] + names + ["zero.elems", "unknown.dtype"],
                             [None] + host + [np.zeros(0, np.uint8), host[0][:16]],
                             [F32] + dtypes + [F32, UNKNOWN], out_cpu, rank=3)
    for a, b, what in zip(read_files(out_gpu, 3), read_files(out_cpu, 3), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    s = ctx.summary()
    assert s["n_tensors"] == len(names) and s["states_bytes"] == len(read_files(out_gpu, 3)[0])

    # restore into fresh buffers through the files
    ctx2 = chk.Context(device=0, rank=3)
    outs = [torch.zeros(t.numel() + 64, dtype=torch.uint8, device="cuda") for t in dev]
    for n, o, t, dt in zip(names, outs, dev, dtypes):
        ctx2.register_pointer(n, o.data_ptr(), t.numel() // ELEM_SIZE[dt], dt)
    ctx2.set_option("verify_zero_lanes", 1)
    assert ctx2.load_and_decompress(out_gpu) == len(names)
    for o, h, n in zip(outs, host, names):
        assert np.array_equal(o[:h.size].cpu().numpy(), h), n
        assert int(o[h.size:].sum()) == 0, f"{n}: wrote past the tensor"
    # and the oracle's reader accepts the GPU-written files
    for n, h in zip(names, host):
        assert np.array_equal(oracle.load_tensor(out_gpu, n, h.size, rank=3), h), n
    ctx.close()
    ctx2.close()


def test_restore_misaligned_targets(chk, oracle, tmp_path):
    names, host, dev, dtypes = make_mixed(seed=2)
    out_cpu = str(tmp_path / "cpu")
    oracle.compress_and_save(names, host, dtypes, out_cpu, rank=0)  # files written by the oracle
    ctx = chk.Context(device=0, rank=0)
    outs = []
    for k, (n, h, dt) in enumerate(zip(names, host, dtypes)):
        mis = (k % 4) * ELEM_SIZE[dt]
        buf = torch.zeros(h.size + mis + 64, dtype=torch.uint8, device="cuda")
        outs.append((buf, mis))
        ctx.register_pointer(n, buf.data_ptr() + mis, h.size // ELEM_SIZE[dt], dt)
    assert ctx.load_and_decompress(out_cpu) == len(names)
    for (buf, mis), h, n in zip(outs, host, names):
        got = buf.cpu().numpy()
        assert np.array_equal(got[mis:mis + h.size], h), n
        assert got[:mis].sum() == 0 and got[mis + h.size:].sum() == 0, f"{n}: wrote outside the tensor"
    ctx.close()


def _cluster_setup(oracle, names, host, dtypes):
    fps = []
    for h, dt in zip(host, dtypes):
        _, mom, mm = oracle.tensor_stats(h, dt)
        fps.append([mom[0], mom[1], mom[2], mom[3], np.float32(mm[1] - mm[0])])
    cid, anchors = oracle.build_clusters(names, np.array(fps, np.float32))
    return cid, [names[a] for a in anchors]


def make_state(n_layers=6, n=32768, seed=11):
    names, host, dtypes = [], [], []
    for l in range(n_layers):
        p = f"model.layers.{l}.mlp.weight"
        for prefix, kind in (("", "bf16_weight"), ("master_weights::", "f32_master"),
                             ("optimizer.exp_avg::", "f32_exp_avg"), ("optimizer.exp_avg_sq::", "f32_exp_avg_sq")):
            raw, dt = synth(kind, n + 17 * l if l % 2 else n, seed * 100 + len(names))
            names.append(prefix + p)
            host.append(raw.copy())
            dtypes.append(dt)
    return names, host, dtypes


@pytest.mark.parametrize("repair", [False, True])
def test_files_identical_with_clusters(chk, oracle, tmp_path, repair):
    names, host, dtypes = make_state()
    dev = [dev_bytes(h) for h in host]
    cid, anchors = _cluster_setup(oracle, names, host, dtypes)
    assert len(anchors) >= 1, "test data should produce at least one cluster"
    ctx = chk.Context(device=0, rank=1)
    register_all(ctx, names, dev, dtypes)
    ctx.set_cluster_info(names, cid, anchors)
    ctx.set_option("repair_tables", int(repair))
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    if not repair:
        # reference-exact shared tables for bf16 data do not sum to 4096: nothing is written unless asked for
        with pytest.raises(chk.CheckersError) as ei:
            ctx.compress_and_save(out_gpu)
        assert ei.value.code == -6 and not os.path.exists(os.path.join(out_gpu, "rank_1_states.ansc"))
        n_tab, n_bad = ctx.table_report()
        assert 0 < n_bad <= n_tab
        ctx.set_option("allow_undecodable", 1)
    ctx.compress_and_save(out_gpu)
    if repair:
        assert ctx.table_report()[1] == 0
    oracle.compress_and_save(names, host, dtypes, out_cpu, rank=1, cluster_id=cid, anchor_names=anchors,
                             repair_tables=repair)
    for a, b, what in zip(read_files(out_gpu, 1), read_files(out_cpu, 1), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's (repair={repair})"
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    ctx2 = chk.Context(device=0, rank=1)
    for n, o, h, dt in zip(names, outs, host, dtypes):
        ctx2.register_pointer(n, o.data_ptr(), h.size // ELEM_SIZE[dt], dt)
    if repair:
        assert ctx2.load_and_decompress(out_gpu) == len(names)
        for o, h, n in zip(outs, host, names):
            assert np.array_equal(o.cpu().numpy(), h), n
    else:
        # The reference's shared tables for bf16 data do not sum to 4096: such
        # streams are written identically but refused by the reader.
        dict_bytes = read_files(out_gpu, 1)[2]
        n_tab = int(np.frombuffer(dict_bytes[12:16], np.uint32)[0])
        sums = [int(np.frombuffer(dict_bytes[16 + i * 2308 + 1280 + 1024:16 + i * 2308 + 1284 + 1024], np.uint32)[0])
                for i in range(n_tab)]
        if any(s != 4096 for s in sums):
            with pytest.raises(chk.CheckersError) as ei:
                ctx2.load_and_decompress(out_gpu)
            assert ei.value.code == -4
        else:
            assert ctx2.load_and_decompress(out_gpu) == len(names)
    ctx.close()
    ctx2.close()


def test_analysis_matches_oracle(chk, oracle):
    names, host, dtypes = make_state(n_layers=5, n=20000, seed=5)
    names += ["ints.i8", "ints.i32", "half"]
    for kind in ("i8", "i32", "f16_weight"):
        raw, dt = synth(kind, 9999, 77)
        host.append(raw.copy())
        dtypes.append(dt)
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0)
    register_all(ctx, names, dev, dtypes)
    ctx.analyze()
    fps = []
    for i, (h, dt) in enumerate(zip(host, dtypes)):
        hist, mom, mm, fp = ctx.tensor_stats(i)
        h_ref, mom_ref, mm_ref = oracle.tensor_stats(h, dt)
        assert np.array_equal(hist, h_ref), names[i]
        assert np.array_equal(mom.view(np.uint32), mom_ref.view(np.uint32)), (names[i], mom, mom_ref)
        assert np.array_equal(mm.view(np.uint32), mm_ref.view(np.uint32)), names[i]
        fps.append(fp)
    cid_ref, anchors_ref = oracle.build_clusters(names, np.array(fps, np.float32))
    cid, k = ctx.cluster_ids()
    assert np.array_equal(cid, cid_ref) and k == len(anchors_ref)
    for c in range(k):
        assert ctx.cluster_anchor(c) == names[anchors_ref[c]]
    # histogram_bins below 256 narrows the value histogram
    ctx.set_histogram_bins(64)
    ctx.analyze()
    hist, _, _, _ = ctx.tensor_stats(0)
    h_ref, _, _ = oracle.tensor_stats(host[0], dtypes[0], bins=64)
    assert np.array_equal(hist, h_ref)
    ctx.close()


def test_config0_three_tensors_split_in_64(chk, oracle, tmp_path):
    """The reference-scale CPU case: 3 x 16 Mi elements, each cut into 64 tensors of 256 Ki."""
    per, parts = 262144, 64
    kinds = [("w.{}", "bf16_weight"), ("optimizer.exp_avg::w.{}", "f32_exp_avg"),
             ("optimizer.exp_avg_sq::w.{}", "f32_exp_avg_sq")]
    names, host, dtypes = [], [], []
    for fmt, kind in kinds:
        raw, dt = synth(kind, per * parts, 0)
        es = ELEM_SIZE[dt]
        for i in range(parts):
            names.append(fmt.format(i))
            host.append(raw[i * per * es:(i + 1) * per * es].copy())
            dtypes.append(dt)
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0)
    register_all(ctx, names, dev, dtypes)
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    ctx.compress_and_save(out_gpu)
    oracle.compress_and_save(names, host, dtypes, out_cpu)
    for a, b, what in zip(read_files(out_gpu), read_files(out_cpu), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    # device-resident round trip into separate buffers
    ctx.compress(host_images=False)
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
    for o, d in zip(outs, dev):
        assert torch.equal(o, d)
    # in-memory images equal the files
    ctx.compress(host_images=True)
    for k, b in enumerate(read_files(out_gpu)):
        assert ctx.image(k).tobytes() == b
    ctx.close()


def test_error_paths(chk, tmp_path):
    ctx = chk.Context(device=0)
    with pytest.raises(chk.CheckersError):
        ctx.decompress_resident()  # nothing compressed yet
    with pytest.raises(chk.CheckersError):
        ctx.load_and_decompress(str(tmp_path / "missing"))
    with pytest.raises(chk.CheckersError):
        ctx.set_option("no_such_option", 1)
    # empty registry: directories only, no files
    out = str(tmp_path / "empty")
    ctx.compress_and_save(out)
    assert os.path.isdir(os.path.join(out, "mantissa")) and not os.path.exists(os.path.join(out, "rank_0_states.ansc"))
    # corrupted file
    raw, dt = synth("f32_master", 5000, 1)
    t = dev_bytes(raw)
    ctx.register_pointer("a", t.data_ptr(), 5000, dt)
    good = str(tmp_path / "good")
    ctx.compress_and_save(good)
    p = os.path.join(good, "rank_0_states.ansc")
    data = bytearray(open(p, "rb").read())
    data[0] ^= 0xFF
    open(p, "wb").write(bytes(data))
    with pytest.raises(chk.CheckersError) as ei:
        ctx.load_and_decompress(good)
    assert ei.value.code == -4
    data[0] ^= 0xFF
    # flip a payload byte: the lane's end-state / length check must catch it
    data[-100] ^= 0x55
    open(p, "wb").write(bytes(data))
    try:
        ctx.load_and_decompress(good)
        changed = not np.array_equal(t.cpu().numpy(), raw)
        assert changed, "a corrupted payload decoded to the original bytes"
    except chk.CheckersError as e:
        assert e.code == -5
    ctx.close()


def test_front_end_api(chk, oracle, tmp_path):
    names, host, dtypes = make_state(n_layers=2, n=8192, seed=9)
    tensors = {}
    for n, h, dt in zip(names, host, dtypes):
        t = torch.from_numpy(h.copy()).cuda()
        tensors[n] = t.view(torch.bfloat16) if dt == BF16 else t.view(torch.float32)
    with pytest.raises(RuntimeError):
        chk.initialize_context(tensors, histogram_bins=0)
    # reference-exact bytes even where a cluster's shared table is not decodable (compared with the oracle below)
    chk.initialize_context(tensors, None, 256, 1, shared_tables="reference_bytes")
    chk.analyze_tensors()
    out = str(tmp_path / "out")
    chk.compress_and_save(out)
    ctx = chk.current_context()
    cid, k = ctx.cluster_ids()
    anchors = [ctx.cluster_anchor(c) for c in range(k)]
    out_cpu = str(tmp_path / "cpu")
    oracle.compress_and_save(names, host, dtypes, out_cpu, cluster_id=cid, anchor_names=anchors)
    for a, b in zip(read_files(out), read_files(out_cpu)):
        assert a == b


def test_segmented_pipeline_matches_oracle(chk, oracle, tmp_path):
    """Batches of 512 tensors or more are compressed as a pipeline over segments: the files must not
    depend on the cut (1, 3, 8 segments) and must equal the oracle's."""
    rng = np.random.default_rng(11)
    kinds = ["bf16_weight", "f32_master", "f32_exp_avg", "f32_exp_avg_sq", "f16_weight"]
    names, host, dev, dtypes = [], [], [], []
    for i in range(640):
        kind = kinds[i % len(kinds)]
        n = int(rng.integers(1, 6000)) if i % 7 else int(rng.integers(20000, 60000))
        raw, dt = synth(kind, n, 5000 + i)
        names.append(f"{kind}::{i}")
        host.append(raw.copy())
        dev.append(dev_bytes(raw))
        dtypes.append(dt)
    out_cpu = str(tmp_path / "cpu")
    oracle.compress_and_save(names, host, dtypes, out_cpu, rank=0)
    ref = read_files(out_cpu, 0)
    for segments in (3, 1, 8):
        ctx = chk.Context(device=0, rank=0)
        ctx.set_option("segments", segments)
        register_all(ctx, names, dev, dtypes)
        out_gpu = str(tmp_path / f"gpu{segments}")
        ctx.compress_and_save(out_gpu)
        for a, b, what in zip(read_files(out_gpu, 0), ref, ("states", "mantissa", "tables")):
            assert a == b, f"{segments} segments: {what} file differs from the oracle's"
        # and back, from the device-resident result of the same call
        outs = [torch.zeros(t.numel() + 64, dtype=torch.uint8, device="cuda") for t in dev]
        assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
        torch.cuda.synchronize()
        for o, h, n in zip(outs, host, names):
            assert np.array_equal(o[:h.view(np.uint8).size].cpu().numpy(), h.view(np.uint8).reshape(-1)), n
        ctx.close()


def test_codec_microbenchmark_config_full_size(chk, oracle, tmp_path):
    """The codec microbenchmark configuration at its full size -- a 1 GiB fp32 tensor ~ N(0, 1e-3) and a 1 GiB
    bf16 tensor ~ N(0, 0.02), seed 1, in 4 MiB chunks -- checked through size-independent properties: the
    full pipeline round-trips losslessly, split-only recombines to the source, entropy-coding-only (the same
    bytes registered as int8, no low-byte split) round-trips, and sampled chunks equal the oracle's files."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x32 = torch.randn(256 << 20, generator=g, device="cuda", dtype=torch.float32) * 1e-3
    xbf = (torch.randn(512 << 20, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    o32, obf = torch.zeros_like(x32), torch.zeros_like(xbf)
    torch.cuda.synchronize()
    chunk = 4 << 20
    ctx = chk.Context(device=0)
    dst = []
    for k in range(256):
        ctx.register_pointer(f"fp32.{k}", x32.data_ptr() + k * chunk, chunk // 4, F32)
        dst.append(o32.data_ptr() + k * chunk)
    for k in range(256):
        ctx.register_pointer(f"bf16.{k}", xbf.data_ptr() + k * chunk, chunk // 2, BF16)
        dst.append(obf.data_ptr() + k * chunk)
    ctx.compress()
    s = ctx.summary()
    assert s["n_tensors"] == 512 and s["original_bytes"] == 2 << 30
    compressed = s["states_bytes"] + s["mantissa_bytes"] + s["dict_bytes"]
    assert compressed < s["original_bytes"]                      # Gaussian data: the exponent bytes compress
    assert ctx.decompress_resident(dst) == 512
    torch.cuda.synchronize()
    assert torch.equal(x32.view(torch.uint8), o32.view(torch.uint8))
    assert torch.equal(xbf.view(torch.uint8), obf.view(torch.uint8))
    ctx.close()

    # split only: masked | low bytes is the source again
    for t, dt, es in ((x32, F32, 4), (xbf, BF16, 2)):
        n = chunk // es
        masked = torch.zeros(chunk, dtype=torch.uint8, device="cuda")
        side = torch.zeros(chunk // 2, dtype=torch.uint8, device="cuda")
        c2 = chk.Context(device=0)
        c2.split(t.data_ptr() + 3 * chunk, n, dt, masked.data_ptr(), side.data_ptr())
        torch.cuda.synchronize()
        src = t.view(torch.uint8)[3 * chunk:4 * chunk].view(n, es)
        m, sd = masked.view(n, es), side.view(n, es // 2)
        assert torch.equal(m[:, es // 2:], src[:, es // 2:]) and int(m[:, :es // 2].max()) == 0
        assert torch.equal(sd, src[:, :es // 2])
        c2.close()

    # entropy coding only: the fp32 bytes as int8 tensors (no split), first 64 MiB
    c3 = chk.Context(device=0)
    o8 = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    for k in range(16):
        c3.register_pointer(f"bytes.{k}", x32.data_ptr() + k * chunk, chunk, I8)
    c3.compress()
    assert c3.decompress_resident([o8.data_ptr() + k * chunk for k in range(16)]) == 16
    torch.cuda.synchronize()
    assert torch.equal(o8, x32.view(torch.uint8)[:64 << 20])
    c3.close()

    # sampled chunks against the oracle, file for file
    names, host, dev, dtypes = [], [], [], []
    for t, dt, tag in ((x32, F32, "fp32"), (xbf, BF16, "bf16")):
        for k in (0, 255):
            piece = t.view(torch.uint8)[k * chunk:(k + 1) * chunk]
            names.append(f"{tag}.{k}")
            host.append(piece.cpu().numpy().copy())
            dev.append(piece)
            dtypes.append(dt)
    c4 = chk.Context(device=0)
    register_all(c4, names, dev, dtypes)
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    c4.compress_and_save(out_gpu)
    oracle.compress_and_save(names, host, dtypes, out_cpu)
    for a, b, what in zip(read_files(out_gpu), read_files(out_cpu), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    c4.close()


def test_segmented_pipeline_with_shared_tables(chk, oracle, tmp_path):
    """Cluster members borrow their anchor's table across pipeline segments (the anchor's table is built
    on another stream, segments earlier): files equal the oracle's and restore, for 1 and 4 segments."""
    names, host, dtypes = make_state(n_layers=140, n=3000, seed=21)   # 560 tensors
    dev = [dev_bytes(h) for h in host]
    cid, anchors = _cluster_setup(oracle, names, host, dtypes)
    assert len(anchors) >= 1
    out_cpu = str(tmp_path / "cpu")
    oracle.compress_and_save(names, host, dtypes, out_cpu, cluster_id=cid, anchor_names=anchors, repair_tables=True)
    ref = read_files(out_cpu)
    for segments in (4, 1):
        ctx = chk.Context(device=0)
        register_all(ctx, names, dev, dtypes)
        ctx.set_cluster_info(names, cid, anchors)
        ctx.set_option("repair_tables", 1)
        ctx.set_option("segments", segments)
        out_gpu = str(tmp_path / f"gpu{segments}")
        ctx.compress_and_save(out_gpu)
        for a, b, what in zip(read_files(out_gpu), ref, ("states", "mantissa", "tables")):
            assert a == b, f"{segments} segments: {what} file differs from the oracle's"
        ctx.close()
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    ctx2 = chk.Context(device=0)
    for n, o, h, dt in zip(names, outs, host, dtypes):
        ctx2.register_pointer(n, o.data_ptr(), h.size // ELEM_SIZE[dt], dt)
    assert ctx2.load_and_decompress(out_gpu) == len(names)
    for o, h, n in zip(outs, host, names):
        assert np.array_equal(o.cpu().numpy(), h), n
    ctx2.close()
