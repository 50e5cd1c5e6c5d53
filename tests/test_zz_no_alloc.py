"""The allocation-free encode entry point against the regular pipeline.

Some callers cannot allocate when they compress (HBM is full at checkpoint
time, or another framework owns the allocator); chk_encode_tensor_static keeps
all of its working memory in a fixed region inside the library.  Here it is
called through the C ABI twice in a row -- so the second call starts on the
first call's leftovers -- and must reproduce the regular entry point's payload,
lane headers and passthrough flag byte for byte.  Collected last on purpose."""
import numpy as np
import pytest

from oracle_lib import ELEM_SIZE, synth

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


def test_static_scratch_encode_matches_pipeline():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import checkers_b200 as chk
    cases = [("f32_master", 1 << 20), ("bf16_weight", 300001), ("i8", 70000), ("f32_exp_avg_sq_lognormal", 4099)]
    for round_ in range(2):  # two passes over the cases: every call sees stale scratch from the one before
        for i, (kind, n) in enumerate(cases):
            raw, dt = synth(kind, n, 40 + i)
            t, payload, headers, is_raw, nf, cf = _regular(chk, raw, dt, f"t{i}")
            out = torch.full((raw.size + 64,), 0xEE, dtype=torch.uint8, device="cuda")
            hdr = torch.zeros(1024, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            size, raw_flag = chk.encode_tensor_static(t.data_ptr(), n, dt, nf, cf, out.data_ptr(), hdr.data_ptr())
            assert raw_flag == is_raw and size == payload.size, (kind, round_)
            assert np.array_equal(out[:size].cpu().numpy(), payload), (kind, round_)
            assert int((out[size:] != 0xEE).sum()) == 0, "wrote past the payload"
            assert np.array_equal(hdr.cpu().numpy().view(np.uint32).reshape(256, 4), headers), (kind, round_)
    # beyond the fixed limit: refused, nothing touched
    big = torch.zeros(chk.STATIC_MAX_TENSOR_BYTES + 4, dtype=torch.uint8, device="cuda")
    with pytest.raises(chk.CheckersError) as ei:
        chk.encode_tensor_static(big.data_ptr(), big.numel() // 4, chk.F32, nf, cf, big.data_ptr(), hdr.data_ptr())
    assert ei.value.code == -7
