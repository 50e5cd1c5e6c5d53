"""The allocation-free encode entry point against the CPU oracle and the regular pipeline.

Some callers cannot allocate when they compress (HBM is full at checkpoint
time, or another framework owns the allocator); chk_encode_tensor_static keeps
all of its working memory in a fixed region inside the library.  Here it is
called through the C ABI twice in a row -- so the second call starts on the
first call's leftovers -- and must reproduce, byte for byte, the payload, lane
headers and passthrough flag that the oracle and the regular entry point give
for the same tensor and table; the device's free memory must be the same after
the calls as before.  Collected last on purpose."""
import numpy as np
import pytest

from oracle_lib import ELEM_SIZE, SIDECAR_PER_ELEM, I8, synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _regular(chk, raw, dt, name):
    """Payload, headers, raw flag and table of one tensor from the pooled pipeline."""
    t = torch.from_numpy(raw.copy()).cuda()
    torch.cuda.synchronize()
    ctx = chk.Context(device=0)
    ctx.register_pointer(name, t.data_ptr(), raw.size // ELEM_SIZE[dt], dt)
    ctx.compress(host_images=True)
    st, dc = ctx.image(0).copy(), ctx.image(2).copy()
    ctx.close()
    entry = st[16:16 + 4648]
    is_raw = bool(entry[257])
    size = int(entry[288:296].view(np.uint64)[0])
    headers = entry[552:552 + 4096].view(np.uint32).reshape(256, 4).copy()
    payload = st[16 + 4648:16 + 4648 + size].copy()
    nf = dc[16 + 256:16 + 256 + 1024].view(np.uint32).copy()
    cf = dc[16 + 1280:16 + 1280 + 1028].view(np.uint32).copy()
    return t, payload, headers, is_raw, nf, cf


def _cases():
    rng = np.random.default_rng(77)
    out = [("f32_master", 1 << 20), ("bf16_weight", 300001), ("i8", 70000), ("f32_exp_avg_sq_lognormal", 4099),
           ("f32_master", 1), ("bf16_weight", 1), ("i8", 1), ("i8", 255), ("bf16_weight", 127)]
    cases = [synth(kind, n, 40 + i) for i, (kind, n) in enumerate(out)]
    # uniform bytes up to the limit: every symbol costs 8 bits and more, so the passthrough rule stores the tensor raw
    cases.append((rng.integers(0, 256, 4 << 20, dtype=np.uint8), I8))
    cases.append((rng.integers(0, 256, 65537, dtype=np.uint8), I8))
    return cases


def test_static_scratch_encode_matches_oracle_and_pipeline(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200 as chk
    cases = _cases()
    # warm everything the comparison itself allocates, then take the reading the calls are held to
    out = torch.full(((4 << 20) + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    hdr = torch.zeros(1024, dtype=torch.int32, device="cuda")
    saw_raw = False
    for round_ in range(2):  # two passes over the cases: every call sees stale scratch from the one before
        for i, (raw, dt) in enumerate(cases):
            n = raw.size // ELEM_SIZE[dt]
            t, payload, headers, is_raw, nf, cf = _regular(chk, raw, dt, f"t{i}")
            masked = oracle.split(raw, dt)[0] if SIDECAR_PER_ELEM[dt] else raw
            o_nf, o_cf, o_xm, _ = oracle.normalize(oracle.byte_histogram(masked), False)
            o_payload, o_headers, o_raw = oracle.compress_tensor(masked, o_nf, o_cf, o_xm)
            assert np.array_equal(nf, o_nf) and np.array_equal(cf, o_cf)
            out.fill_(0xEE)
            hdr.zero_()
            torch.cuda.synchronize()
            size, raw_flag = chk.encode_tensor_static(t.data_ptr(), n, dt, o_nf, o_cf, out.data_ptr(), hdr.data_ptr())
            # (the first launch of a kernel variant in a process makes the driver load its code; from then on
            # nothing about the device's memory may change)
            free0 = torch.cuda.mem_get_info()[0]
            size2, raw_flag2 = chk.encode_tensor_static(t.data_ptr(), n, dt, o_nf, o_cf, out.data_ptr(), hdr.data_ptr())
            assert torch.cuda.mem_get_info()[0] == free0, "the call changed the device's free memory"
            assert (size, raw_flag) == (size2, raw_flag2)
            got, got_hdr = out[:size].cpu().numpy(), hdr.cpu().numpy().view(np.uint32).reshape(256, 4)
            assert raw_flag == o_raw == is_raw and size == o_payload.size == payload.size, (i, round_)
            assert np.array_equal(got, o_payload) and np.array_equal(got, payload), (i, round_)
            assert np.array_equal(got_hdr, o_headers) and np.array_equal(got_hdr, headers), (i, round_)
            assert int((out[size:] != 0xEE).sum()) == 0, "wrote past the payload"
            saw_raw = saw_raw or raw_flag
    assert saw_raw, "the passthrough case was not exercised"
    nf, cf = o_nf, o_cf
    # beyond the fixed limit: refused, nothing touched
    big = torch.zeros(chk.STATIC_MAX_TENSOR_BYTES + 4, dtype=torch.uint8, device="cuda")
    with pytest.raises(chk.CheckersError) as ei:
        chk.encode_tensor_static(big.data_ptr(), big.numel() // 4, chk.F32, nf, cf, big.data_ptr(), hdr.data_ptr())
    assert ei.value.code == -7
    # a table that is not a table: refused before anything is launched
    bad = cf.copy()
    bad[100] += 1
    with pytest.raises(chk.CheckersError) as ei:
        chk.encode_tensor_static(t.data_ptr(), 1, chk.I8, nf, bad, out.data_ptr(), hdr.data_ptr())
    assert ei.value.code == -1
    too_big = nf.copy()
    too_big[3] = 5000
    with pytest.raises(chk.CheckersError):
        chk.encode_tensor_static(t.data_ptr(), 1, chk.I8, too_big, cf, out.data_ptr(), hdr.data_ptr())
