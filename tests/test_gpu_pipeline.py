"""GPU tests of what surrounds the kernels: the benchmark's own tensor shapes against the oracle, the
workspace bound, raw-passthrough float tensors through a borrowed table, parameter discovery on a
module + optimizer, the `checkers_py` module name with the reference example's call sequence, the
[TIMING] log.  All through the C ABI; files bit-exact."""
import os
import types

import numpy as np
import pytest

from oracle_lib import BF16, ELEM_SIZE, F32, I8, Oracle, synth
from test_gpu_codec import chk, dev_bytes, read_files, register_all  # noqa: F401  (chk is a fixture)

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _bench_slice(shard, world_shards, chunk_elems, seed):
    """A flat-index slice of the benchmark's Llama-3-8B state, built like bench.py builds its CPU sample."""
    import bench
    pieces, n_elems, _ = bench.shard_pieces(bench.LLAMA3_8B, shard, world_shards, chunk_elems)
    bufs = bench.make_shard_on_host(pieces, n_elems, seed)
    names, host, dtypes = [], [], []
    for name, off, n, _ in pieces:
        for (prefix, _), b, dt in zip(bench.STATE_KINDS, bufs, (BF16, F32, F32, F32)):
            names.append(prefix + name)
            host.append(np.ascontiguousarray(b[off:off + n]).view(np.uint8).reshape(-1).copy())
            dtypes.append(dt)
    return pieces, names, host, dtypes


def test_benchmark_slice_matches_oracle(chk, oracle, tmp_path):
    """Pieces of 1 Mi elements at shard position: the end of a down_proj, both RMSNorm gains of the layer
    (1 + N(0, 1e-3): every bf16 value is 1.0) and the start of the next q_proj, with the lognormal
    exp_avg_sq the benchmark uses."""
    pieces, names, host, dtypes = _bench_slice(189, 2048, 1 << 20, 7)
    assert any(p[3] for p in pieces) and len({p[0].split("@")[0] for p in pieces}) >= 3
    assert max(p[2] for p in pieces) == 1 << 20
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0, rank=3)
    register_all(ctx, names, dev, dtypes)
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    ctx.compress_and_save(out_gpu)
    oracle.compress_and_save(names, host, dtypes, out_cpu, rank=3)
    for a, b, what in zip(read_files(out_gpu, 3), read_files(out_cpu, 3), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
    torch.cuda.synchronize()
    for o, h, n in zip(outs, host, names):
        assert np.array_equal(o.cpu().numpy(), h), n
    ctx.close()


def test_workspace_bound(chk, oracle, tmp_path):
    """A deliberately small workspace: fewer encode teams, the same files; below one slot: refused."""
    rng = np.random.default_rng(3)
    kinds = ["bf16_weight", "f32_master", "f32_exp_avg", "f32_exp_avg_sq_lognormal", "i8"]
    names, host, dev, dtypes = [], [], [], []
    for i in range(600):
        raw, dt = synth(kinds[i % len(kinds)], int(rng.integers(1, 30000)), 900 + i)
        names.append(f"t{i}")
        host.append(raw.copy())
        dev.append(dev_bytes(raw))
        dtypes.append(dt)
    out_cpu = str(tmp_path / "cpu")
    oracle.compress_and_save(names, host, dtypes, out_cpu)
    ref = read_files(out_cpu)
    slot = 256 * 2 * ((30000 * 4 + 255) // 256 + 16)      # an upper estimate of one team's scratch slot
    teams_seen = []
    for ws in (0, 3 * slot):
        ctx = chk.Context(device=0, workspace_bytes=ws)
        register_all(ctx, names, dev, dtypes)
        out_gpu = str(tmp_path / f"gpu{ws}")
        ctx.compress_and_save(out_gpu)
        for a, b, what in zip(read_files(out_gpu), ref, ("states", "mantissa", "tables")):
            assert a == b, f"workspace {ws}: {what} file differs from the oracle's"
        teams_seen.append(ctx.timing("encode_teams"))
        if ws:
            assert ctx.timing("workspace_mb") * 2 ** 20 <= ws
        ctx.close()
    assert 1 <= teams_seen[1] < teams_seen[0] and teams_seen[1] <= 8   # my slot estimate is generous
    ctx = chk.Context(device=0, workspace_bytes=4096)
    register_all(ctx, names, dev, dtypes)
    with pytest.raises(chk.CheckersError) as ei:
        ctx.compress(host_images=False)
    assert ei.value.code == -7
    ctx.set_option("workspace_bytes", 0)     # the option lifts the bound again
    ctx.compress(host_images=False)
    ctx.close()


def test_raw_passthrough_float_through_borrowed_table(chk, oracle, tmp_path):
    """Float tensors that borrow the table of an anchor whose bytes are nearly all one value: every other byte,
    the zeroed low bytes included, costs 12 bits, the streams come out larger than the tensor, and the passthrough
    rule stores the masked bytes raw; restoring such a tensor merges them with its sidecar."""
    specs = [("a.w", None, 50000), ("b.w", "f32_uniform_bits", 40000), ("c.w", "bf16_weight", 777),
             ("d.w", "f32_uniform_bits", 255), ("e.w", "f32_master", 30000)]
    names, host, dtypes = [], [], []
    for i, (n, kind, cnt) in enumerate(specs):
        if kind is None:
            raw, dt = np.full(cnt, 0x55, np.uint8), I8
            raw[::97] = 0x56
        else:
            raw, dt = synth(kind, cnt, 70 + i)
        names.append(n)
        host.append(raw.copy())
        dtypes.append(dt)
    dev = [dev_bytes(h) for h in host]
    cid, anchors = [0, 0, 0, 0, -1], ["a.w"]
    ctx = chk.Context(device=0)
    register_all(ctx, names, dev, dtypes)
    ctx.set_cluster_info(names, cid, anchors)
    ctx.set_option("repair_tables", 1)
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    ctx.compress_and_save(out_gpu)
    oracle.compress_and_save(names, host, dtypes, out_cpu, cluster_id=cid, anchor_names=anchors, repair_tables=True)
    st = read_files(out_gpu)[0]
    for a, b, what in zip(read_files(out_gpu), read_files(out_cpu), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    assert all(st[16 + k * 4648 + 257] == 1 for k in (1, 2, 3)), "the float members must be stored raw"
    for source in ("resident", "files"):
        outs = [torch.zeros(h.size + 8, dtype=torch.uint8, device="cuda") for h in host]
        if source == "resident":
            assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
        else:
            ctx2 = chk.Context(device=0)
            for n, o, h, dt in zip(names, outs, host, dtypes):
                ctx2.register_pointer(n, o.data_ptr(), h.size // ELEM_SIZE[dt], dt)
            assert ctx2.load_and_decompress(out_gpu) == len(names)
            ctx2.close()
        torch.cuda.synchronize()
        for o, h, n in zip(outs, host, names):
            got = o.cpu().numpy()
            assert np.array_equal(got[:h.size], h) and not got[h.size:].any(), (source, n)
    ctx.close()


class _MasterAdam(torch.optim.Adam):
    """Adam over fp32 master copies of bf16 parameters, apex FP16_Optimizer style."""

    def __init__(self, params):
        self.fp16_groups = [list(params)]
        self.fp32_from_fp16_groups = [[p.detach().clone().float().requires_grad_(True) for p in self.fp16_groups[0]]]
        super().__init__(self.fp32_from_fp16_groups[0], lr=1e-2)

    def step_from(self):
        for lo, hi in zip(self.fp16_groups[0], self.fp32_from_fp16_groups[0]):
            hi.grad = lo.grad.float()
        self.step()
        for lo, hi in zip(self.fp16_groups[0], self.fp32_from_fp16_groups[0]):
            lo.data.copy_(hi.data)


def _train_one_step(module, opt, master):
    x = torch.randn(16, 64, device="cuda", dtype=next(module.parameters()).dtype)
    module(x).float().pow(2).mean().backward()
    if master:
        opt.step_from()
    else:
        opt.step()


@pytest.mark.parametrize("master", [False, True])
def test_discovery_on_module_and_optimizer(chk, oracle, tmp_path, master):
    """initialize_context(module, optimizer): weight, (master copy,) exp_avg, exp_avg_sq per parameter, in the
    reference's order and names; files equal the oracle's over the same tensors; restore brings them back."""
    torch.manual_seed(5)
    module = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.LayerNorm(128), torch.nn.Linear(128, 64)).cuda()
    if master:
        module = module.bfloat16()
        opt = _MasterAdam(module.parameters())
    else:
        opt = torch.optim.Adam(module.parameters(), lr=1e-2)
    _train_one_step(module, opt, master)
    torch.cuda.synchronize()
    chk.initialize_context(module, opt, 256, 1)
    ctx = chk.current_context()
    per_param = 4 if master else 3
    assert ctx.tensor_count() == per_param * len(list(module.parameters()))
    want = []
    for name, _ in module.named_parameters():
        want += [name] + (["master_weights::" + name] if master else []) + \
                ["optimizer.exp_avg::" + name, "optimizer.exp_avg_sq::" + name]
    assert ctx.names == want
    pairs = chk.api._named_state_tensors(module, opt)
    host = [t.detach().contiguous().view(torch.uint8).reshape(-1).cpu().numpy().copy() for _, t in pairs]
    dtypes = [BF16 if t.dtype == torch.bfloat16 else F32 for _, t in pairs]
    out_gpu, out_cpu = str(tmp_path / "gpu"), str(tmp_path / "cpu")
    chk.compress_and_save(out_gpu)       # no analyze_tensors(): every tensor owns its table
    oracle.compress_and_save([n for n, _ in pairs], host, dtypes, out_cpu)
    for a, b, what in zip(read_files(out_gpu), read_files(out_cpu), ("states", "mantissa", "tables")):
        assert a == b, f"{what} file differs from the oracle's"
    for _, t in pairs:
        t.detach().zero_()
    assert chk.load_and_decompress(out_gpu) == len(pairs)
    torch.cuda.synchronize()
    for (n, t), h in zip(pairs, host):
        assert np.array_equal(t.detach().view(torch.uint8).reshape(-1).cpu().numpy(), h), n


def test_checkers_py_call_sequence_and_timing_log(tmp_path, monkeypatch):
    """`import checkers_py` and the call sequence of the reference's training script
    (examples/FSDP_ZeRO3/train_llama3.py:235-264) on a stand-in engine object."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    monkeypatch.setenv("CHECKERS_LOG_DIR", str(tmp_path / "logs"))
    monkeypatch.setenv("CHECKERS_LOG_RUN_ID", "t1")
    import checkers_py
    torch.manual_seed(1)
    module = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.Linear(64, 64)).cuda()
    optimizer = torch.optim.Adam(module.parameters())
    _train_one_step(module, optimizer, False)
    engine = types.SimpleNamespace(module=module, optimizer=optimizer, global_rank=2, local_rank=0, global_steps=1)
    # the script's own call, plus the one added keyword: tiny bias tensors that get clustered would otherwise hit
    # the reference's undecodable shared tables, which compress_and_save refuses to write
    checkers_py.initialize_context(engine, optimizer, histogram_bins=4096, background_threads=4, shared_tables="repair")
    checkers_py.analyze_tensors()
    out = str(tmp_path / "ckpt")
    checkers_py.compress_and_save(out)
    assert os.path.exists(os.path.join(out, "rank_2_states.ansc"))
    assert os.path.exists(os.path.join(out, "mantissa", "rank_2_mantissa.mant"))
    assert os.path.exists(os.path.join(out, "tables", "rank_2_tables.dict"))
    log = open(tmp_path / "logs" / "t1" / "rank_2" / "checkers.log").read()
    for key in ("setup_ms", "discovery_ms", "flush_ms", "total_ms", "analyze_histograms_ms", "analyze_knn_clusters_ms",
                "analyze_total_ms", "compress_and_save_total_ms", "compress_computation_ms", "compress_io_ms",
                "compress_and_save_wall_ms"):
        assert f"[TIMING] {key}=" in log, key
    before = [p.detach().clone() for p in module.parameters()]
    for p in module.parameters():
        p.data.zero_()
    assert checkers_py.load_and_decompress(out) == 3 * len(before)
    torch.cuda.synchronize()
    for p, b in zip(module.parameters(), before):
        assert torch.equal(p.detach(), b)
    # the same through the byte-plane container
    checkers_py.initialize_context(engine, optimizer, histogram_bins=4096, background_threads=4, container_version=3)
    out3 = str(tmp_path / "ckpt3")
    checkers_py.compress_and_save(out3)
    v2 = sum(os.path.getsize(os.path.join(out, r)) for r in ("rank_2_states.ansc", "mantissa/rank_2_mantissa.mant"))
    v3 = sum(os.path.getsize(os.path.join(out3, r)) for r in ("rank_2_states.ansc", "mantissa/rank_2_mantissa.mant"))
    for p in module.parameters():
        p.data.zero_()
    assert checkers_py.load_and_decompress(out3) == 3 * len(before)
    torch.cuda.synchronize()
    for p, b in zip(module.parameters(), before):
        assert torch.equal(p.detach(), b)
    assert v3 < v2 * 1.6   # tiny tensors: twice the index entries; the payload is what shrinks on real sizes


def test_fast_statistics_against_oracle(chk, oracle):
    """analysis in the order-free mode: minimum, maximum and value histogram identical to the reference-order
    statistics, moments within the rounding error of the reference's float sums; large and unaligned tensors."""
    cases = [("bf16_weight", 3_000_001), ("f32_master", 1 << 20), ("f32_exp_avg_sq_lognormal", 700_003),
             ("bf16_norm_gain", 4096), ("i8", 1_000_000), ("i32", 65_537), ("f16_weight", 250_000), ("f32_exp_avg", 1)]
    host, dts, dev, views = [], [], [], []
    for i, (kind, n) in enumerate(cases):
        raw, dt = synth(kind, n, 300 + i)
        host.append(raw)
        dts.append(dt)
        buf = torch.zeros(raw.size + 64, dtype=torch.uint8, device="cuda")
        off = ELEM_SIZE[dt] if i % 3 == 2 else 0      # every third tensor starts off a 16-byte boundary
        buf[off:off + raw.size] = torch.from_numpy(raw.copy()).cuda()
        dev.append(buf)
        views.append(buf.data_ptr() + off)
    ctx = chk.Context(device=0)
    ctx.set_option("fast_stats", 1)
    for i, (raw, dt) in enumerate(zip(host, dts)):
        ctx.register_pointer(f"t{i}", views[i], raw.size // ELEM_SIZE[dt], dt)
    for bins in (256, 100):
        ctx.set_histogram_bins(bins)
        ctx.analyze()
        first = [ctx.tensor_stats(i) for i in range(len(host))]
        ctx.analyze()
        for i, (raw, dt) in enumerate(zip(host, dts)):
            hist, mom, mm, fp = ctx.tensor_stats(i)
            h_ref, mom_ref, mm_ref = oracle.tensor_stats(raw, dt, bins=bins)
            assert np.array_equal(hist, h_ref), i
            assert np.array_equal(mm.view(np.uint32), mm_ref.view(np.uint32)), i
            spread = max(abs(float(mm_ref[0])), abs(float(mm_ref[1])), 1e-30)
            assert abs(float(mom[0]) - float(mom_ref[0])) <= 1e-5 * spread, (i, mom, mom_ref)
            assert abs(float(mom[1]) - float(mom_ref[1])) <= 1e-4 * abs(float(mom_ref[1])) + 1e-12, (i, mom, mom_ref)
            assert abs(float(mom[2]) - float(mom_ref[2])) <= 1e-3 * max(1.0, abs(float(mom_ref[2]))), (i, mom, mom_ref)
            assert abs(float(mom[3]) - float(mom_ref[3])) <= 1e-3 * max(1.0, abs(float(mom_ref[3]))), (i, mom, mom_ref)
            # the same numbers on every run
            for a, b in zip(first[i], (hist, mom, mm, fp)):
                assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), i
    ctx.close()


def _v3_expected(oracle, names, host, dtypes, tmp_path, rank):
    """What container version 3 must write, from the version-2 oracle: states / tables = the oracle's files for the
    byte planes as 8-bit tensors (integer tensors as they are); mantissa = its file for the original tensors."""
    from oracle_lib import SIDECAR_PER_ELEM
    p_names, p_host, p_dt = [], [], []
    for name, raw, dt in zip(names, host, dtypes):
        es, spe = ELEM_SIZE[dt], SIDECAR_PER_ELEM[dt]
        if spe == 0:
            p_names.append(name); p_host.append(raw); p_dt.append(dt)
            continue
        m = raw.reshape(-1, es)
        for k in range(spe, es):
            p_names.append(f"{name}#b{k}"); p_host.append(np.ascontiguousarray(m[:, k])); p_dt.append(I8)
    d_planes, d_orig = str(tmp_path / "o_planes"), str(tmp_path / "o_orig")
    oracle.compress_and_save(p_names, p_host, p_dt, d_planes, rank=rank)
    oracle.compress_and_save(names, host, dtypes, d_orig, rank=rank)
    st, _, dc = read_files(d_planes, rank)
    _, mt, _ = read_files(d_orig, rank)

    def v3(b):
        b = bytearray(b)
        b[4:8] = (3).to_bytes(4, "little")
        return bytes(b)
    return v3(st), v3(mt), v3(dc)


def test_container_version3_byte_planes(chk, oracle, tmp_path):
    """Opt-in container version 3: every high byte plane of a float tensor coded as an 8-bit tensor of its own.
    Files equal what the version-2 oracle writes for those planes; restore from the device-resident result and
    from files is lossless; the result is smaller than version 2's; version 2 is unaffected by the switch."""
    names, host, dtypes = make_state_v3()
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0, rank=2)
    register_all(ctx, names, dev, dtypes)
    out2 = str(tmp_path / "v2")
    ctx.compress_and_save(out2)
    v2_files = read_files(out2, 2)
    v2_total = sum(len(f) for f in v2_files)

    ctx.set_option("format_version", 3)
    out3 = str(tmp_path / "v3")
    ctx.compress_and_save(out3)
    got = read_files(out3, 2)
    want = _v3_expected(oracle, names, host, dtypes, tmp_path, 2)
    for g, w, what in zip(got, want, ("states", "mantissa", "tables")):
        assert g == w, f"{what} file differs from the oracle's files of the planes"
    s = ctx.summary()
    assert s["states_bytes"] + s["mantissa_bytes"] + s["dict_bytes"] == sum(len(f) for f in got)
    assert s["original_bytes"] == sum(h.size for h in host)
    v3_payload = s["states_bytes"] + s["mantissa_bytes"]
    assert v3_payload < 0.93 * (len(v2_files[0]) + len(v2_files[1])), (v3_payload, v2_total)

    # device-resident round trip into separate buffers
    ctx.compress(host_images=False)
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
    for o, d in zip(outs, dev):
        assert torch.equal(o, d)
    # from the files, into a fresh context with fresh tensors
    fresh = [torch.zeros_like(d) for d in dev]
    ctx2 = chk.Context(device=0, rank=2)
    register_all(ctx2, names, fresh, dtypes)
    ctx2.set_option("format_version", 3)
    assert ctx2.load_and_decompress(out3) == len(names)
    for f, d in zip(fresh, dev):
        assert torch.equal(f, d)
    # a version-2 reader refuses the files, and the other way round
    ctx2.set_option("format_version", 2)
    with pytest.raises(chk.CheckersError):
        ctx2.load_and_decompress(out3)
    ctx2.set_option("format_version", 3)
    with pytest.raises(chk.CheckersError):
        ctx2.load_and_decompress(out2)
    # back to version 2: the same bytes as before
    ctx.set_option("format_version", 2)
    out2b = str(tmp_path / "v2b")
    ctx.compress_and_save(out2b)
    assert read_files(out2b, 2) == v2_files
    ctx.close(); ctx2.close()


def make_state_v3():
    kinds = [("model.embed.weight", "bf16_weight", 300001), ("master_weights::model.embed.weight", "f32_master", 300001),
             ("optimizer.exp_avg::model.embed.weight", "f32_exp_avg", 300001),
             ("optimizer.exp_avg_sq::model.embed.weight", "f32_exp_avg_sq_lognormal", 300001),
             ("model.norm.weight", "bf16_norm_gain", 4096), ("half.w", "f16_weight", 70000), ("tiny", "f32_master", 1),
             ("ints.i8", "i8", 50000), ("ints.i32", "i32", 12345), ("model.q.weight", "bf16_weight", 1 << 20),
             ("master_weights::model.q.weight", "f32_master", 1 << 20)]
    names, host, dtypes = [], [], []
    for i, (name, kind, n) in enumerate(kinds):
        raw, dt = synth(kind, n, 900 + i)
        names.append(name); host.append(raw.copy()); dtypes.append(dt)
    return names, host, dtypes


def test_short_decode_table_option(chk):
    """decode_zero_skip: float tensors decode through the short slot table, integer and raw-passthrough tensors
    through the full one (two launches); the restored bytes are the inputs, zeros in value lanes included."""
    names, host, dtypes = make_state_v3()
    rng = np.random.default_rng(3)
    for h, dt in zip(host, dtypes):
        if dt in (F32, BF16) and h.size > 100000:
            v = h.reshape(-1, ELEM_SIZE[dt])
            v[rng.random(v.shape[0]) < 0.25] = 0
    names.append("noise.i8"); host.append(rng.integers(0, 256, 1 << 18, dtype=np.uint8)); dtypes.append(I8)
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0)
    register_all(ctx, names, dev, dtypes)
    ctx.set_option("decode_zero_skip", 1)
    ctx.set_option("verify_zero_lanes", 1)
    ctx.compress(host_images=True)
    images = [ctx.image(k).copy() for k in range(3)]
    launches = ctx.kernel_launches()
    outs = [torch.zeros(h.size, dtype=torch.uint8, device="cuda") for h in host]
    assert ctx.decompress_resident([o.data_ptr() for o in outs]) == len(names)
    assert ctx.kernel_launches() - launches >= 2
    for o, d in zip(outs, dev):
        assert torch.equal(o, d)
    fresh = [torch.zeros_like(d) for d in dev]
    ctx2 = chk.Context(device=0)
    register_all(ctx2, names, fresh, dtypes)
    ctx2.set_option("decode_zero_skip", 1)
    assert ctx2.decompress_images(*images) == len(names)
    for f, d in zip(fresh, dev):
        assert torch.equal(f, d)
    ctx.close(); ctx2.close()


def test_release_workspace_returns_device_memory(chk, tmp_path):
    """The context keeps its buffers from call to call; release_workspace gives them back to the device, the host
    images stay, and the next compress works as before."""
    names, host, dtypes = make_state_v3()
    dev = [dev_bytes(h) for h in host]
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    ctx = chk.Context(device=0)
    register_all(ctx, names, dev, dtypes)
    free0 = torch.cuda.mem_get_info()[0]
    ctx.compress(host_images=True)
    first = [ctx.image(k).copy() for k in range(3)]
    held = free0 - torch.cuda.mem_get_info()[0]
    assert held > sum(h.size for h in host) // 2          # sidecar section, payload heap, scratch ...
    ctx.release_workspace()
    assert free0 - torch.cuda.mem_get_info()[0] <= 4 << 20, "device memory was not given back"
    assert all(np.array_equal(ctx.image(k), first[k]) for k in range(3))
    with pytest.raises(chk.CheckersError):
        ctx.decompress_resident([d.data_ptr() for d in dev])     # the resident result went with the buffers
    ctx.compress(host_images=True)
    assert all(np.array_equal(ctx.image(k), first[k]) for k in range(3))
    ctx.set_option("format_version", 3)
    ctx.compress(host_images=False)
    ctx.release_workspace()
    assert free0 - torch.cuda.mem_get_info()[0] <= 4 << 20
    ctx.close()


@pytest.mark.parametrize("fused", [1, 0])
def test_container_version3_float_only_restore_paths(chk, oracle, tmp_path, fused):
    """Float tensors only: restore decodes the planes straight into whole elements (one kernel, no plane buffers);
    with the switch off, planes are decoded to memory and merged.  Both from the device-resident result and from
    files, into misaligned targets too; an incompressible plane (stored raw) among them."""
    names, host, dtypes = [], [], []
    for n_, h_, d_ in zip(*make_state_v3()):
        if d_ in (F32, BF16) or n_ == "half.w":
            names.append(n_); host.append(h_); dtypes.append(d_)
    rng = np.random.default_rng(11)
    noise = host[1].copy().reshape(-1, 4)            # fp32: make the lower high byte uniform -> that plane is stored raw
    noise[:, 2] = rng.permutation(np.tile(np.arange(256, dtype=np.uint8), noise.shape[0] // 256 + 1)[:noise.shape[0]])
    names.append("noise.f32"); host.append(noise.reshape(-1).copy()); dtypes.append(F32)
    dev = [dev_bytes(h) for h in host]
    ctx = chk.Context(device=0, rank=1)
    register_all(ctx, names, dev, dtypes)
    ctx.set_option("format_version", 3)
    ctx.set_option("v3_fused_decode", fused)
    out = str(tmp_path / "v3")
    ctx.compress_and_save(out)
    # targets off a 16-byte boundary for every second tensor
    bufs = [torch.zeros(h.size + 32, dtype=torch.uint8, device="cuda") for h in host]
    targets = [b[(2 if i % 2 else 0):][:h.size] for i, (b, h) in enumerate(zip(bufs, host))]
    assert ctx.decompress_resident([t.data_ptr() for t in targets]) == len(names)
    for t, d in zip(targets, dev):
        assert torch.equal(t, d)
    fresh = [torch.zeros_like(d) for d in dev]
    ctx2 = chk.Context(device=0, rank=1)
    register_all(ctx2, names, fresh, dtypes)
    ctx2.set_option("format_version", 3)
    ctx2.set_option("v3_fused_decode", fused)
    assert ctx2.load_and_decompress(out) == len(names)
    for f, d in zip(fresh, dev):
        assert torch.equal(f, d)
    # a damaged stream is reported, not restored silently
    st_path = os.path.join(out, "rank_1_states.ansc")
    blob = bytearray(open(st_path, "rb").read())
    blob[-100] ^= 0x5A
    open(st_path, "wb").write(bytes(blob))
    with pytest.raises(chk.CheckersError):
        ctx2.load_and_decompress(out)
    ctx.close(); ctx2.close()
