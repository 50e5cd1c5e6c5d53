"""The library's CUDA kernels, compiled by g++ behind the block emulator
(tests/emu), against the oracle: checks index arithmetic, ring buffers, tails,
misalignment and the shared symbol-0 chain without a GPU.  Bit-exact."""
import numpy as np
import pytest

from emu_lib import aligned
from oracle_lib import ELEM_SIZE, SIDECAR_PER_ELEM, synth

CASES = [("bf16_weight", 40000), ("f32_master", 20000), ("f32_exp_avg_sq", 10001), ("i8", 1000), ("bf16_norm_gain", 4097),
         ("f32_uniform_bits", 9000), ("i32", 777), ("f16_weight", 70001), ("bf16_weight", 3), ("f32_master", 1),
         ("i8", 255), ("i8", 256), ("i8", 257), ("bf16_weight", 2048 + 64), ("f32_master", 64 * 9 + 3)]


def make(cases, seed, misalign=None):
    tensors, es, spe, dts = [], [], [], []
    for i, (kind, n) in enumerate(cases):
        raw, dt = synth(kind, n, seed + i)
        m = 0 if misalign is None else misalign[i % len(misalign)] * ELEM_SIZE[dt]
        a = aligned(raw.size + 64)[m:m + raw.size]
        a[:] = raw
        tensors.append(a); es.append(ELEM_SIZE[dt]); spe.append(SIDECAR_PER_ELEM[dt]); dts.append(dt)
    return tensors, es, spe, dts


@pytest.mark.parametrize("misalign", [None, [1, 0, 3, 2]])
def test_split_hist_encode_decode(emu, oracle, misalign):
    tensors, es, spe, dts = make(CASES, 1, misalign)
    side, hist = emu.split_hist(tensors, es, spe)
    off, tabs, masked_all = 0, [], []
    for i, a in enumerate(tensors):
        m, s = (oracle.split(a, dts[i]) if spe[i] else (a.copy(), np.zeros(0, np.uint8)))
        assert np.array_equal(side[off:off + s.size], s), i
        off += s.size
        h = oracle.byte_histogram(m)
        hh = hist[i].copy()
        hh[0] += a.size // es[i] * spe[i]
        assert np.array_equal(hh, h), i
        tabs.append(oracle.normalize(h, False))
        masked_all.append(m)
    nf, cf = np.stack([t[0] for t in tabs]), np.stack([t[1] for t in tabs])
    payload, poff, hdrs, raw, st = emu.encode(tensors, es, spe, list(range(len(tensors))), nf, cf)
    assert st == 0
    for i in range(len(tensors)):
        p, hd, r = oracle.compress_tensor(masked_all[i], *tabs[i][:3])
        got = payload[int(poff[i]):int(poff[i + 1])]
        assert bool(raw[i]) == r, i
        assert np.array_equal(got, p), i
        assert np.array_equal(hdrs[i], hd), i
    # cut into segments that go through their own launches on offset pointers (the compress
    # pipeline of the library): same payload, offsets and headers whatever the cut
    for segments in (2, 3, len(tensors)):
        p2, o2, h2, r2, st2 = emu.encode(tensors, es, spe, list(range(len(tensors))), nf, cf, segments=segments)
        assert st2 == 0 and np.array_equal(o2, poff) and np.array_equal(h2, hdrs) and np.array_equal(r2, raw)
        assert np.array_equal(p2[:int(poff[-1])], payload[:int(poff[-1])]), segments
    # the one-kernel path (lanes, zero chain, offsets and gather inside the team) gives the same bytes
    for grid in (1, 4):
        p3, o3, h3, r3 = emu.encode_fused(tensors, es, spe, list(range(len(tensors))), nf, cf, grid=grid)
        assert np.array_equal(o3, poff) and np.array_equal(h3, hdrs) and np.array_equal(r3, raw)
        assert np.array_equal(p3[:int(poff[-1])], payload[:int(poff[-1])]), grid
    for dst_mis in (0, 4):
        outs, status = emu.decode([a.size for a in tensors], es, spe, list(range(len(tensors))), nf, cf, hdrs, payload,
                                  poff, raw, side, check_zero=1, dst_misalign=dst_mis)
        assert not status.any()
        for o, a in zip(outs, tensors):
            assert np.array_equal(o, a)


def test_float_only_kernel_variants(emu, oracle):
    """The kernel builds used for float-only batches (two chains per thread, no escape test)."""
    cases = [("bf16_weight", 50000), ("f32_master", 30000), ("f16_weight", 8191), ("f32_exp_avg_sq_lognormal", 2049),
             ("bf16_norm_gain", 130), ("f32_master", 63)]
    tensors, es, spe, dts = make(cases, 21)
    side, hist = emu.split_hist(tensors, es, spe)
    tabs, masked = [], []
    for a, d in zip(tensors, dts):
        m, _ = oracle.split(a, d)
        masked.append(m)
        tabs.append(oracle.normalize(oracle.byte_histogram(m), False))
    nf, cf = np.stack([t[0] for t in tabs]), np.stack([t[1] for t in tabs])
    payload, poff, hdrs, raw, _ = emu.encode(tensors, es, spe, list(range(len(tensors))), nf, cf, float_only=True)
    for i in range(len(tensors)):
        p, hd, r = oracle.compress_tensor(masked[i], *tabs[i][:3])
        assert bool(raw[i]) == r and np.array_equal(payload[int(poff[i]):int(poff[i + 1])], p), i
        assert np.array_equal(hdrs[i], hd), i
    p3, o3, h3, r3 = emu.encode_fused(tensors, es, spe, list(range(len(tensors))), nf, cf, float_only=True)
    assert np.array_equal(o3, poff) and np.array_equal(h3, hdrs) and np.array_equal(r3, raw)
    assert np.array_equal(p3[:int(poff[-1])], payload[:int(poff[-1])])
    outs, status = emu.decode([a.size for a in tensors], es, spe, list(range(len(tensors))), nf, cf, hdrs, payload,
                              poff, raw, side, check_zero=1, float_only=True)
    assert not status.any()
    for o, a in zip(outs, tensors):
        assert np.array_equal(o, a)


def test_shared_and_degenerate_tables(emu, oracle):
    """Members encoded with an anchor's full-alphabet table (incl. tables that do not sum
    to 4096, and symbols the table lacks), and a passthrough tensor."""
    tensors, es, spe, dts = make([("bf16_weight", 30000), ("bf16_weight", 20000), ("f32_master", 5000),
                                  ("i8", 3000), ("f32_uniform_bits", 3000)], 9)
    masked = [oracle.split(a, d)[0] if s else a.copy() for a, d, s in zip(tensors, dts, spe)]
    t_anchor = oracle.normalize(oracle.byte_histogram(masked[0]), True)      # sums past 4096
    t_f32 = oracle.normalize(oracle.byte_histogram(masked[2]), True, repaired=True)
    hist_few = np.zeros(256, np.uint32); hist_few[:4] = [100, 50, 20, 3]     # lacks most symbols -> escapes
    t_few = oracle.normalize(hist_few, False)
    hist_skew = np.ones(256, np.uint32); hist_skew[0] = 10 ** 6                # every other symbol costs 12 bits
    t_noise = oracle.normalize(hist_skew, False)
    tabs = [t_anchor, t_f32, t_few, t_noise]
    table_idx = [0, 0, 1, 3, 2]
    nf, cf = np.stack([t[0] for t in tabs]), np.stack([t[1] for t in tabs])
    payload, poff, hdrs, raw, st = emu.encode(tensors, es, spe, table_idx, nf, cf)
    for i in range(len(tensors)):
        p, hd, r = oracle.compress_tensor(masked[i], *tabs[table_idx[i]][:3])
        assert bool(raw[i]) == r, i
        assert np.array_equal(payload[int(poff[i]):int(poff[i + 1])], p), i
        assert np.array_equal(hdrs[i], hd), i
    assert raw[3] == 1  # random bytes under a skewed table expand: the passthrough rule stores them raw
    side = emu.split_hist(tensors, es, spe)[0]
    outs, status = emu.decode([a.size for a in tensors[2:4]], es[2:4], spe[2:4], [1, 3], nf, cf, hdrs[2:4],
                              payload, poff[2:4], raw[2:4], side[50000:])
    assert not status.any()
    assert np.array_equal(outs[0], tensors[2])       # repaired shared table decodes
    assert np.array_equal(outs[1], tensors[3])       # raw passthrough restores


def test_stage_kernels(emu, oracle):
    for kind, n, mis in [("bf16_weight", 10007, 0), ("f32_master", 4099, 0), ("f16_weight", 4000, 2), ("f32_master", 512, 4)]:
        raw, dt = synth(kind, n, 3)
        m, s = emu.split(raw, ELEM_SIZE[dt], SIDECAR_PER_ELEM[dt], misalign=mis)
        m_ref, s_ref = oracle.split(raw, dt)
        assert np.array_equal(m, m_ref) and np.array_equal(s, s_ref)
        import ctypes as C
        u8p = C.POINTER(C.c_uint8)
        for shift in (0, 1):  # aligned (vector path) and not
            mm, ss, oo = aligned(m.size + 16)[shift:shift + m.size], aligned(s.size + 16)[shift:shift + s.size], aligned(m.size + 16)[shift:shift + m.size]
            mm[:], ss[:] = m_ref, s_ref
            emu.lib.emu_merge(mm.ctypes.data_as(u8p), ss.ctypes.data_as(u8p), C.c_uint64(m.size), C.c_uint32(ELEM_SIZE[dt]),
                              C.c_uint32(SIDECAR_PER_ELEM[dt]), oo.ctypes.data_as(u8p), C.c_uint32(2))
            assert np.array_equal(oo, raw), (kind, shift)
        assert np.array_equal(emu.byte_histogram(m_ref, misalign=mis + 1), oracle.byte_histogram(m_ref))


def _assert_fast_stats(got, want_hist, want_mom, want_mm):
    """The order-free statistics against the reference-order ones: what does not depend on the order is
    identical, the rest agrees to the rounding error of the reference's float chains."""
    hist, mom, mm, fp = got
    assert np.array_equal(hist, want_hist)
    assert np.array_equal(mm.view(np.uint32), want_mm.view(np.uint32))
    spread = max(abs(float(want_mm[0])), abs(float(want_mm[1])), 1e-30)
    assert abs(float(mom[0]) - float(want_mom[0])) <= 1e-5 * spread                      # mean
    assert abs(float(mom[1]) - float(want_mom[1])) <= 1e-4 * abs(float(want_mom[1])) + 1e-12   # variance
    assert abs(float(mom[2]) - float(want_mom[2])) <= 1e-3 * max(1.0, abs(float(want_mom[2])))  # skewness
    assert abs(float(mom[3]) - float(want_mom[3])) <= 1e-3 * max(1.0, abs(float(want_mom[3])))  # kurtosis
    assert np.array_equal(fp[:4].view(np.uint32), mom.view(np.uint32))
    assert fp[4] == np.float32(want_mm[1] - want_mm[0])


def test_fast_stats_kernels(emu, oracle):
    cases = [("bf16_weight", 70001), ("f32_master", 40000), ("f16_weight", 2048), ("i8", 300), ("i32", 1000),
             ("bf16_norm_gain", 513), ("f32_exp_avg_sq_lognormal", 33000), ("f32_master", 1), ("i8", 140000)]
    for mis in (None, [1]):   # 16-byte loads possible / not
        tensors, es, spe, dts = make(cases, 4, mis)
        for bins, grid in ((256, 3), (64, 64)):
            res = emu.stats(tensors, [a.size // e for a, e in zip(tensors, es)], dts, bins=bins, grid=grid, fast=True)
            for i, a in enumerate(tensors):
                h, mom, mm = oracle.tensor_stats(a, dts[i], bins)
                _assert_fast_stats(res[i], h, mom, mm)


def test_stats_kernel(emu, oracle):
    cases = [("bf16_weight", 5000), ("f32_master", 4099), ("f16_weight", 2048), ("i8", 300), ("i32", 1000),
             ("bf16_norm_gain", 513), ("f32_exp_avg_sq", 256), ("f32_master", 1), ("f32_exp_avg_sq_lognormal", 9000)]
    tensors, es, spe, dts = make(cases, 4)
    for bins in (256, 64):
        res = emu.stats(tensors, [a.size // e for a, e in zip(tensors, es)], dts, bins=bins)
        for i, a in enumerate(tensors):
            h, mom, mm = oracle.tensor_stats(a, dts[i], bins)
            assert np.array_equal(res[i][0], h), i
            assert np.array_equal(res[i][1].view(np.uint32), mom.view(np.uint32)), i
            assert np.array_equal(res[i][2].view(np.uint32), mm.view(np.uint32)), i
            assert res[i][3][4] == np.float32(mm[1] - mm[0])


@pytest.mark.parametrize("misalign", [None, [1, 0, 2]])
def test_plane_split_and_merge(emu, misalign):
    """Byte planes of container version 3: low bytes element-major, every high byte a plane of its own; the
    merge restores the tensor.  16-byte path, ragged tails and unaligned tensors."""
    cases = [("f32_master", 20000), ("bf16_weight", 70001), ("f16_weight", 4099), ("f32_exp_avg", 3), ("bf16_weight", 1),
             ("f32_exp_avg_sq", 8192 + 16)]
    tensors, es, spe, dts = make(cases, 9, misalign)
    n_elem = [a.size // e for a, e in zip(tensors, es)]
    low_off, plane_off, stride = [], [], []
    lo = po = 0
    for n, e, sp in zip(n_elem, es, spe):
        low_off.append(lo); plane_off.append(po); stride.append((n + 31) & ~31)
        lo += n * sp
        po += stride[-1] * (e - sp)
    low, planes = aligned(lo + 64), aligned(po + 64)
    low[:] = 0xAA; planes[:] = 0xBB
    emu.planes(tensors, n_elem, es, spe, low_off, plane_off, stride, low, planes)
    for i, a in enumerate(tensors):
        m = a.reshape(n_elem[i], es[i])
        assert np.array_equal(low[low_off[i]:low_off[i] + n_elem[i] * spe[i]], m[:, :spe[i]].reshape(-1)), i
        for k in range(es[i] - spe[i]):
            p0 = plane_off[i] + k * stride[i]
            assert np.array_equal(planes[p0:p0 + n_elem[i]], m[:, spe[i] + k]), (i, k)
            assert np.all(planes[p0 + n_elem[i]:p0 + stride[i]] == 0xBB), (i, k)
    assert np.all(low[lo:] == 0xAA)
    # the same split with the planes' byte histograms counted in the pass
    low2, planes2 = aligned(lo + 64), aligned(po + 64)
    hist = emu.planes_count(tensors, n_elem, es, spe, low_off, plane_off, stride, low2, planes2, grid=4)
    assert np.array_equal(low2[:lo], low[:lo])
    row = 0
    for i, a in enumerate(tensors):
        m = a.reshape(n_elem[i], es[i])
        for k in range(es[i] - spe[i]):
            p0 = plane_off[i] + k * stride[i]
            assert np.array_equal(planes2[p0:p0 + n_elem[i]], m[:, spe[i] + k]), (i, k)
            assert np.array_equal(hist[row], np.bincount(m[:, spe[i] + k], minlength=256)), (i, k)
            row += 1
    outs = []
    for a in tensors:
        off = (a.ctypes.data & 15)
        o = aligned(a.size + 64)[off:off + a.size]
        o[:] = 0
        outs.append(o)
    emu.planes(outs, n_elem, es, spe, low_off, plane_off, stride, low, planes, grid=5, merge=True)
    for a, o in zip(tensors, outs):
        assert np.array_equal(a, o)


def test_short_decode_table_with_zeros_in_value_lanes(emu, oracle):
    """The decoder's short slot table leaves out the slots that symbol 0 owns; value lanes that do see zeros
    (tensors with exact 0.0 entries: all four bytes zero) must decode through its entry 0."""
    rng = np.random.default_rng(5)
    tensors, es, spe, dts = make([("f32_master", 30000), ("bf16_weight", 50001)], 12)
    for a, e in zip(tensors, es):
        v = a.reshape(-1, e)
        v[rng.random(v.shape[0]) < 0.3] = 0      # 30 % exact zeros
    side, hist = emu.split_hist(tensors, es, spe)
    tabs, masked_all, off, sides = [], [], 0, []
    for i, a in enumerate(tensors):
        m, s = oracle.split(a, dts[i])
        tabs.append(oracle.normalize(oracle.byte_histogram(m), False))
        assert tabs[-1][0][0] >= 2048      # symbol 0 owns at least half of the slots: the short table is used
        masked_all.append(m)
    nf = np.concatenate([t[0] for t in tabs]).astype(np.uint32)
    cf = np.concatenate([t[1] for t in tabs]).astype(np.uint32)
    payloads, hdrs, raws = [], [], []
    for m, t in zip(masked_all, tabs):
        p, h, r = oracle.compress_tensor(m, t[0], t[1], t[2])
        payloads.append(p); hdrs.append(h); raws.append(r)
    poff = np.cumsum([0] + [p.size for p in payloads])[:-1].astype(np.uint64)
    payload = np.concatenate(payloads + [np.zeros(64, np.uint8)])
    outs, status = emu.decode([a.size for a in tensors], es, spe, list(range(len(tensors))), nf, cf,
                              np.concatenate(hdrs).astype(np.uint32), payload, poff, np.array(raws, np.uint8), side,
                              check_zero=1, float_only=True)
    assert not status.any()
    for a, o in zip(tensors, outs):
        assert np.array_equal(a, o)


@pytest.mark.parametrize("kind,es", [("f32_master", 4), ("bf16_weight", 2), ("f32_exp_avg_sq_lognormal", 4)])
def test_plane_decoder_writes_whole_elements(emu, oracle, kind, es):
    """Container version 3 restore without a merge pass: every plane compressed by the oracle as an 8-bit tensor,
    the team decodes the planes of a tensor side by side and writes whole elements; sizes with full groups of
    8 rows, leftover rows, a partial row, next to nothing; one plane stored raw (uniform bytes)."""
    rng = np.random.default_rng(3)
    planes = es // 2
    sizes = [8 * 256 * 3 + 5 * 256 + 77, 4096, 255, 1, 256 * 9]
    dsts, lows, want, n_elem, poff, raws, cfs, hdrs, payloads = [], [], [], [], [], [], [], [], []
    at = 0
    for gi, n in enumerate(sizes):
        raw, dt = synth(kind, n, 70 + gi)
        m = raw.reshape(n, es).copy()
        if gi == 1:
            flat = np.tile(np.arange(256, dtype=np.uint8), n // 256)        # every value equally often: incompressible
            rng.shuffle(flat)
            m[:, es - 2 if planes == 2 else es - 1] = flat
        want.append(m.reshape(-1).copy())
        low = aligned(n * (es // 2) + 16)[:n * (es // 2)]
        low[:] = m[:, :es // 2].reshape(-1)
        lows.append(low)
        dsts.append(aligned(n * es + 16)[:n * es])
        n_elem.append(n)
        for p in range(planes):
            plane = np.ascontiguousarray(m[:, es // 2 + p])
            nf, cf, xm, _ = oracle.normalize(oracle.byte_histogram(plane), False)
            pay, h, is_raw = oracle.compress_tensor(plane, nf, cf, xm)
            pad = (-at) % 32
            payloads.append(np.zeros(pad, np.uint8)); at += pad
            poff.append(at); raws.append(int(is_raw)); cfs.append(cf); hdrs.append(h); payloads.append(pay)
            at += pay.size
    assert any(raws), "the raw-plane case is not exercised"
    payload = np.concatenate(payloads + [np.zeros(64, np.uint8)])
    for d in dsts:
        d[:] = 0xEE
    status = emu.decode_planes(planes, dsts, lows, n_elem, poff, raws, np.concatenate(cfs), np.concatenate(hdrs), payload)
    assert not status.any()
    for d, w in zip(dsts, want):
        assert np.array_equal(d, w)
