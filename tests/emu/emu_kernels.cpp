// emu_kernels.cpp -- the library's kernel source run on the CPU block emulator.
// Test-only: lets the CPU suite check every kernel's index arithmetic against
// the oracle.  Build: g++ -std=c++17 -O1 -I checkers_b200/csrc -shared -fPIC.
#include "cuda_emu.hpp"
//
#include "kernels.cuh"
#include "tables.hpp"

#include <vector>

using namespace chk;

namespace {
struct Batch {
    std::vector<TensorDesc> descs;
    std::vector<uint32_t> tile_start;
    unsigned long long sidecar_total = 0, scratch_total = 0, bytes_total = 0;
};

Batch make_batch(size_t n, const uint8_t* const* srcs, uint8_t* const* dsts, const uint64_t* n_bytes,
                 const uint32_t* es, const uint32_t* spe, const uint32_t* table_idx, const uint8_t* need_hist) {
    Batch b;
    b.descs.resize(n);
    b.tile_start.resize(n + 1);
    b.tile_start[0] = 0;
    for (size_t i = 0; i < n; ++i) {
        TensorDesc& d = b.descs[i];
        std::memset(&d, 0, sizeof(d));
        d.src = srcs ? srcs[i] : nullptr;
        d.dst = dsts ? dsts[i] : nullptr;
        d.n_bytes = n_bytes[i];
        d.es = es[i];
        d.spe = spe[i];
        d.table_idx = table_idx ? table_idx[i] : (uint32_t)i;
        d.sidecar_off = b.sidecar_total;
        d.scratch_off = b.scratch_total;
        const unsigned long long c_max = (d.n_bytes + 255) / 256;
        d.chunk_stride = (uint32_t)((2 * c_max + 31) & ~31ull);
        d.flags = 0;
        if (!need_hist || need_hist[i]) d.flags |= kFlagNeedHist;
        const uintptr_t p = (uintptr_t)(srcs ? (const void*)srcs[i] : (const void*)dsts[i]);
        if ((p & 15) == 0 && (d.sidecar_off & 15) == 0) d.flags |= kFlagAligned;
        b.sidecar_total += (d.n_bytes / d.es) * d.spe;
        b.scratch_total += (d.spe * 2 == d.es ? 129ull : 256ull) * d.chunk_stride;
        b.bytes_total += d.n_bytes;
        b.tile_start[i + 1] = b.tile_start[i] + (uint32_t)((d.n_bytes + kSplitTileBytes - 1) / kSplitTileBytes);
    }
    return b;
}
}  // namespace

extern "C" {

void emu_split(const uint8_t* src, uint64_t n_bytes, uint32_t es, uint32_t spe, uint8_t* masked, uint8_t* sidecar,
               uint32_t grid) {
    const uint32_t vec = ((uintptr_t)src & 15) == 0 && ((uintptr_t)masked & 15) == 0 && ((uintptr_t)sidecar & 15) == 0;
    emu::launch(grid, 256, 0, [&] { split_kernel(src, n_bytes, es, spe, masked, sidecar, vec); });
}

void emu_merge(const uint8_t* masked, const uint8_t* sidecar, uint64_t n_bytes, uint32_t es, uint32_t spe, uint8_t* out,
               uint32_t grid) {
    const uint32_t vec = ((uintptr_t)masked & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)sidecar & 7) == 0;
    emu::launch(grid, 256, 0, [&] { merge_kernel(masked, sidecar, n_bytes, es, spe, out, vec); });
}

void emu_byte_histogram(const uint8_t* data, uint64_t n, uint32_t* hist, uint32_t grid) {
    std::memset(hist, 0, 1024);
    emu::launch(grid, 256, 0, [&] { byte_histogram_kernel(data, n, hist); });
}

// sidecar_out: concatenated low bytes; hist_out: n*256 counters (without the zeroed bytes)
void emu_split_hist(size_t n, const uint8_t* const* srcs, const uint64_t* n_bytes, const uint32_t* es,
                    const uint32_t* spe, const uint8_t* need_hist, uint8_t* sidecar_out, uint32_t* hist_out,
                    uint32_t grid) {
    Batch b = make_batch(n, srcs, nullptr, n_bytes, es, spe, nullptr, need_hist);
    std::memset(hist_out, 0, n * 1024);
    const uint32_t total = b.tile_start[n];
    emu::launch(grid, 256, 0, [&] {
        split_hist_kernel(b.descs.data(), b.tile_start.data(), (uint32_t)n, 0u, total, sidecar_out, hist_out);
    });
}

// Full encode: lanes -> lane scan -> tensor scan -> compaction.
// payload_off_out has n+1 entries; hdrs_out n*1024 words; raw_out n bytes.
uint32_t emu_encode(size_t n, const uint8_t* const* srcs, const uint64_t* n_bytes, const uint32_t* es,
                    const uint32_t* spe, const uint32_t* table_idx, size_t n_tables, const uint32_t* nf,
                    const uint32_t* cf, uint8_t* payload_out, uint64_t* payload_off_out, uint32_t* hdrs_out,
                    uint8_t* raw_out, uint32_t grid, uint32_t float_only, uint32_t segments) {
    Batch b = make_batch(n, srcs, nullptr, n_bytes, es, spe, table_idx, nullptr);
    std::vector<EncEntry> enc(n_tables * 256);
    for (size_t t = 0; t < n_tables; ++t) {
        FreqTable ft;
        std::memcpy(ft.norm_freq, nf + t * 256, 1024);
        std::memcpy(ft.cum_freq, cf + t * 257, 1028);
        build_enc_entries(ft, &enc[t * 256]);
    }
    std::vector<uint8_t> scratch(b.scratch_total + 64, 0xAA);
    // keep lane regions 16-byte aligned like the device allocation
    uint8_t* scr = (uint8_t*)(((uintptr_t)scratch.data() + 15) & ~(uintptr_t)15);
    std::vector<LaneHeader> hdrs(n * 256);
    std::vector<unsigned long long> lsrc(n * 256);
    std::vector<uint32_t> loff(n * 256);
    // The batch runs as `segments` consecutive ranges, each through its own launches on offset
    // pointers, the way the library's compress pipeline does; any cut must give the same bytes.
    std::vector<unsigned long long> psize(n), poff(n + 1);
    uint32_t status = 0;
    if (segments < 1) segments = 1;
    std::vector<uint32_t> order(n);
    std::vector<uint32_t> tickets(segments, 0);
    for (uint32_t g = 0; g < segments; ++g) {
        const size_t a = n * g / segments, e = n * (g + 1) / segments, m = e - a;
        if (m == 0) continue;
        for (size_t i = 0; i < m; ++i) order[a + i] = (uint32_t)(m - 1 - i);  // any permutation must give the same result
        TensorDesc* descs = b.descs.data() + a;
        LaneHeader* hd = hdrs.data() + a * 256;
        unsigned long long* ls = lsrc.data() + a * 256;
        uint32_t* lo = loff.data() + a * 256;
        emu::launch((unsigned)((m + 31) / 32), 32, 0, [&] { zero_lane_kernel(descs, enc.data(), scr, hd, ls, (uint32_t)m); });
        if (float_only)  // the variant the pipeline uses for float-only batches without missing symbols
            emu::launch(grid, kTeam, sizeof(EncSmem<2>), [&] {
                rans_encode_kernel<false, false>(descs, enc.data(), scr, hd, ls, order.data() + a, &tickets[g], (uint32_t)m);
            });
        else
            emu::launch(grid, kTeam, sizeof(EncSmem<4>), [&] {
                rans_encode_kernel<true, true>(descs, enc.data(), scr, hd, ls, order.data() + a, &tickets[g], (uint32_t)m);
            });
        emu::launch(grid, 256, 0, [&] { lane_scan_kernel(descs, hd, psize.data() + a, lo, (uint32_t)m); });
        emu::launch(1, 1024, 0, [&] {
            tensor_scan_kernel(descs, psize.data() + a, poff.data() + a, (uint32_t)m, a ? poff.data() + a : nullptr);
        });
        emu::launch(grid, 256, 0, [&] { compact_kernel(descs, hd, ls, lo, scr, payload_out, (uint32_t)m); });
    }
    for (size_t i = 0; i <= n; ++i) payload_off_out[i] = poff[i];
    std::memcpy(hdrs_out, hdrs.data(), n * 4096);
    for (size_t i = 0; i < n; ++i) raw_out[i] = (b.descs[i].flags & kFlagRaw) ? 1 : 0;
    return status;
}

// The same through rans_encode_fused_kernel (one launch: lanes, zero chain, offsets, gather).
// The device payload is a heap: heap_off_out[i] / size_out[i] say where tensor i's payload is.
void emu_encode_fused(size_t n, const uint8_t* const* srcs, const uint64_t* n_bytes, const uint32_t* es,
                      const uint32_t* spe, const uint32_t* table_idx, size_t n_tables, const uint32_t* nf,
                      const uint32_t* cf, uint8_t* heap_out, uint64_t* heap_off_out, uint64_t* size_out,
                      uint32_t* hdrs_out, uint8_t* raw_out, uint32_t grid, uint32_t float_only) {
    Batch b = make_batch(n, srcs, nullptr, n_bytes, es, spe, table_idx, nullptr);
    std::vector<EncEntry> enc(n_tables * 256);
    for (size_t t = 0; t < n_tables; ++t) {
        FreqTable ft;
        std::memcpy(ft.norm_freq, nf + t * 256, 1024);
        std::memcpy(ft.cum_freq, cf + t * 257, 1028);
        build_enc_entries(ft, &enc[t * 256]);
    }
    unsigned long long slot_bytes = 0;
    for (size_t i = 0; i < n; ++i) {
        const unsigned long long need = (b.descs[i].spe * 2 == b.descs[i].es ? 129ull : 256ull) * b.descs[i].chunk_stride;
        if (need > slot_bytes) slot_bytes = need;
    }
    slot_bytes = (slot_bytes + 255) & ~255ull;
    std::vector<uint8_t> scratch(slot_bytes * grid + 64, 0xAA);
    uint8_t* scr = (uint8_t*)(((uintptr_t)scratch.data() + 31) & ~(uintptr_t)31);
    std::vector<LaneHeader> hdrs(n * 256);
    std::vector<unsigned long long> psize(n, 0);
    std::vector<uint32_t> order(n);
    for (size_t i = 0; i < n; ++i) order[i] = (uint32_t)((i * 7 + 3) % n);  // any permutation must give the same result
    if (n % 7 == 0) for (size_t i = 0; i < n; ++i) order[i] = (uint32_t)(n - 1 - i);
    unsigned long long cursor = 0;
    uint32_t ticket = 0;
    // shared symbol-0 chains: deliberately few slots, so that some tensors fall back to computing their own
    uint32_t max_stride = 0;
    for (size_t i = 0; i < n; ++i) max_stride = std::max(max_stride, b.descs[i].chunk_stride);
    const uint32_t z_slots = 2;
    std::vector<ZeroSlot> zslots(z_slots);
    std::memset(zslots.data(), 0, z_slots * sizeof(ZeroSlot));
    std::vector<uint8_t> zregions((size_t)z_slots * max_stride + 64, 0xBB);
    std::vector<int32_t> zslot_of(n, -7);
    emu::launch((unsigned)n, 32, 0, [&] {
        zero_chain_kernel(b.descs.data(), enc.data(), zslots.data(), z_slots, zregions.data(), max_stride, zslot_of.data(),
                          (uint32_t)n);
    });
    FusedParams fp{};
    fp.descs = b.descs.data();
    fp.tables = enc.data();
    fp.scratch = scr;
    fp.slot_bytes = slot_bytes;
    fp.zero_slots = zslots.data();
    fp.zero_regions = zregions.data();
    fp.zero_slot_of = zslot_of.data();
    fp.zero_region_stride = max_stride;
    fp.n_tensors = (uint32_t)n;
    fp.hdrs = hdrs.data();
    fp.payload = heap_out;
    fp.payload_size = psize.data();
    fp.heap_cursor = &cursor;
    fp.order = order.data();
    fp.ticket = &ticket;
    if (float_only)
        emu::launch(grid, kTeam, sizeof(EncSmem<2>), [&] { rans_encode_fused_kernel<false>(fp); });
    else
        emu::launch(grid, kTeam, sizeof(EncSmem<4>), [&] { rans_encode_fused_kernel<true>(fp); });
    for (size_t i = 0; i < n; ++i) {
        heap_off_out[i] = b.descs[i].payload_off;
        size_out[i] = psize[i];
        raw_out[i] = (b.descs[i].flags & kFlagRaw) ? 1 : 0;
    }
    std::memcpy(hdrs_out, hdrs.data(), n * 4096);
}

// payload must be readable 64 bytes past its end and 16-byte aligned.
void emu_decode(size_t n, uint8_t* const* dsts, const uint64_t* n_bytes, const uint32_t* es, const uint32_t* spe,
                const uint32_t* table_idx, const uint32_t* nf, const uint32_t* cf, const uint32_t* hdrs,
                const uint8_t* payload, const uint64_t* payload_off, const uint8_t* raw, const uint8_t* sidecar,
                uint32_t check_zero_lanes, uint32_t* status_out, uint32_t grid, uint32_t float_only) {
    Batch b = make_batch(n, nullptr, dsts, n_bytes, es, spe, table_idx, nullptr);
    for (size_t i = 0; i < n; ++i) {
        b.descs[i].payload_off = payload_off[i];
        if (raw[i]) b.descs[i].flags |= kFlagRaw;
    }
    std::memset(status_out, 0, n * 4);
    // as the library's host side does: float tensors whose table qualifies go to the short-table kernel
    std::vector<uint32_t> short_order, full_order;
    bool any_int = false;
    for (size_t k = 0; k < n; ++k) {
        const uint32_t i = (uint32_t)(n - 1 - k);
        const bool is_float = spe[i] * 2 == es[i];
        if (float_only && is_float && !raw[i] && zero_skip_fits(nf[(size_t)table_idx[i] * 256]))
            short_order.push_back(i);
        else {
            full_order.push_back(i);
            any_int = any_int || !is_float;
        }
    }
    uint32_t ticket[2] = {0, 0};
    if (!short_order.empty())
        emu::launch(grid, kTeam, kDecSmemBytes[0][1], [&] {
            rans_decode_kernel<false, true>(b.descs.data(), nf, cf, (const LaneHeader*)hdrs, payload, sidecar,
                                            short_order.data(), &ticket[0], (uint32_t)short_order.size(), check_zero_lanes,
                                            status_out);
        });
    if (full_order.empty()) return;
    if (any_int)
        emu::launch(grid, kTeam, kDecSmemBytes[1][0], [&] {
            rans_decode_kernel<true, false>(b.descs.data(), nf, cf, (const LaneHeader*)hdrs, payload, sidecar,
                                            full_order.data(), &ticket[1], (uint32_t)full_order.size(), check_zero_lanes,
                                            status_out);
        });
    else
        emu::launch(grid, kTeam, kDecSmemBytes[0][0], [&] {
            rans_decode_kernel<false, false>(b.descs.data(), nf, cf, (const LaneHeader*)hdrs, payload, sidecar,
                                             full_order.data(), &ticket[1], (uint32_t)full_order.size(), check_zero_lanes,
                                             status_out);
        });
}

// outs: n * sizeof(StatsOut)/4 words
void emu_stats(size_t n, const void* const* ptrs, const uint64_t* n_elem, const uint32_t* dtype, uint32_t bins,
               void* outs, uint32_t grid) {
    std::vector<StatsDesc> d(n);
    for (size_t i = 0; i < n; ++i) d[i] = StatsDesc{ptrs[i], n_elem[i], dtype[i], bins};
    std::memset(outs, 0, n * sizeof(StatsOut));
    emu::launch(grid, 256, 0, [&] { tensor_stats_kernel(d.data(), (StatsOut*)outs, (uint32_t)n); });
}

// the order-free variant: same outputs, four launches
void emu_stats_fast(size_t n, const void* const* ptrs, const uint64_t* n_elem, const uint32_t* dtype, uint32_t bins,
                    void* outs, uint32_t grid) {
    std::vector<StatsDesc> d(n);
    std::vector<uint32_t> tile_start(n + 1);
    uint32_t tiles = 0;
    for (size_t i = 0; i < n; ++i) {
        d[i] = StatsDesc{ptrs[i], n_elem[i], dtype[i], bins};
        tile_start[i] = tiles;
        const uint64_t bytes = n_elem[i] * stats_elem_size(dtype[i]);
        if (ptrs[i] && n_elem[i]) tiles += (uint32_t)((bytes + kStatsTileBytes - 1) / kStatsTileBytes);
    }
    tile_start[n] = tiles;
    std::memset(outs, 0, n * sizeof(StatsOut));
    if (!tiles) return;
    std::vector<StatsPart1> p1(tiles);
    std::vector<StatsPart2> p2(tiles);
    std::vector<StatsMid> mids(n);
    if (grid > tiles) grid = tiles;
    emu::launch(grid, 256, 0, [&] { stats_fast_pass1_kernel(d.data(), tile_start.data(), (uint32_t)n, tiles, p1.data()); });
    emu::launch((uint32_t)n, 256, 0, [&] {
        stats_fast_reduce1_kernel(d.data(), tile_start.data(), p1.data(), mids.data(), (StatsOut*)outs, (uint32_t)n);
    });
    emu::launch(grid, 256, 0, [&] {
        stats_fast_pass2_kernel(d.data(), tile_start.data(), (uint32_t)n, tiles, mids.data(), p2.data(), (StatsOut*)outs);
    });
    emu::launch((uint32_t)n, 256, 0, [&] {
        stats_fast_reduce2_kernel(d.data(), tile_start.data(), p2.data(), (StatsOut*)outs, (uint32_t)n);
    });
}

// byte planes: split n tensors into low bytes + planes, or merge them back (merge != 0: `tensors` are written)
void emu_planes(size_t n, void* const* tensors, const uint64_t* n_elem, const uint32_t* es, const uint32_t* spe,
                const uint64_t* low_off, const uint64_t* plane_off, const uint64_t* stride, uint8_t* low, uint8_t* planes,
                uint32_t grid, uint32_t merge) {
    std::vector<PlaneDesc> d(n);
    std::vector<uint32_t> ts(n + 1);
    uint32_t tiles = 0;
    for (size_t i = 0; i < n; ++i) {
        d[i] = PlaneDesc{};
        d[i].tensor = (uint8_t*)tensors[i];
        d[i].n_elem = n_elem[i];
        d[i].low_off = low_off[i];
        d[i].plane_off = plane_off[i];
        d[i].plane_stride = stride[i];
        d[i].es = es[i];
        d[i].spe = spe[i];
        d[i].vector_ok = ((uintptr_t)tensors[i] & 15) == 0 && (low_off[i] & 15) == 0 && ((uintptr_t)low & 15) == 0 &&
                         ((uintptr_t)planes & 15) == 0;
        ts[i] = tiles;
        tiles += (uint32_t)((n_elem[i] * es[i] + kPlaneTileBytes - 1) / kPlaneTileBytes);
    }
    ts[n] = tiles;
    if (!tiles) return;
    if (grid > tiles) grid = tiles;
    if (merge)
        emu::launch(grid, 256, 0, [&] { plane_merge_kernel(d.data(), ts.data(), (uint32_t)n, tiles, low, planes); });
    else
        emu::launch(grid, 256, 0, [&] { plane_split_kernel(d.data(), ts.data(), (uint32_t)n, tiles, low, planes); });
}

// the split that also counts every plane's bytes: hist = 256 counters per plane, planes numbered through the tensors
void emu_planes_count(size_t n, void* const* tensors, const uint64_t* n_elem, const uint32_t* es, const uint32_t* spe,
                      const uint64_t* low_off, const uint64_t* plane_off, const uint64_t* stride, uint8_t* low,
                      uint8_t* planes, uint32_t* hist, uint32_t grid) {
    std::vector<PlaneDesc> d(n);
    std::vector<uint32_t> ts(n + 1);
    uint32_t tiles = 0, row = 0;
    for (size_t i = 0; i < n; ++i) {
        d[i] = PlaneDesc{};
        d[i].tensor = (uint8_t*)tensors[i];
        d[i].n_elem = n_elem[i];
        d[i].low_off = low_off[i];
        d[i].plane_off = plane_off[i];
        d[i].plane_stride = stride[i];
        d[i].es = es[i];
        d[i].spe = spe[i];
        d[i].vector_ok = ((uintptr_t)tensors[i] & 15) == 0 && (low_off[i] & 15) == 0 && ((uintptr_t)low & 15) == 0 &&
                         ((uintptr_t)planes & 15) == 0;
        d[i].hist_row = row;
        row += es[i] - spe[i];
        ts[i] = tiles;
        tiles += (uint32_t)((n_elem[i] * es[i] + kPlaneTileBytes - 1) / kPlaneTileBytes);
    }
    ts[n] = tiles;
    std::memset(hist, 0, (size_t)row * 1024);
    if (!tiles) return;
    if (grid > tiles) grid = tiles;
    emu::launch(grid, 256, kPlaneCountSmem, [&] {
        plane_split_count_kernel(d.data(), ts.data(), (uint32_t)n, tiles, low, planes, hist);
    });
}

// HyperLogLog sketches of n tensors: regs_out n x 16384 words
void emu_hll(size_t n, const void* const* ptrs, const uint64_t* n_elem, const uint32_t* dtype, uint32_t* regs_out,
             uint32_t grid) {
    std::vector<StatsDesc> d(n);
    std::vector<uint32_t> tile_start(n + 1);
    uint32_t tiles = 0;
    for (size_t i = 0; i < n; ++i) {
        d[i] = StatsDesc{ptrs[i], n_elem[i], dtype[i], 0};
        tile_start[i] = tiles;
        if (ptrs[i] && n_elem[i])
            tiles += (uint32_t)((n_elem[i] * stats_elem_size(dtype[i]) + kHllTileBytes - 1) / kHllTileBytes);
    }
    tile_start[n] = tiles;
    std::memset(regs_out, 0, n * kHllRegs * 4);
    if (!tiles) return;
    if (grid > tiles) grid = tiles;
    emu::launch(grid, 256, kHllRegs * 4, [&] { hll_sketch_kernel(d.data(), tile_start.data(), (uint32_t)n, tiles, regs_out); });
}

// shared-model cost: the three kernels over n tensors; out = {vocabulary, packed best, overflow, norm sum, bits}
void emu_model_cost(size_t n, const void* const* ptrs, const uint64_t* n_elem, const uint32_t* dtype, uint32_t capacity,
                    double factor_scale_log2, uint32_t grid, double* out) {
    std::vector<StatsDesc> d(n);
    std::vector<uint32_t> tile_start(n + 1);
    uint32_t tiles = 0;
    uint64_t symbols = 0;
    for (size_t i = 0; i < n; ++i) {
        d[i] = StatsDesc{ptrs[i], n_elem[i], dtype[i], 0};
        tile_start[i] = tiles;
        tiles += (uint32_t)((n_elem[i] * stats_elem_size(dtype[i]) + kHllTileBytes - 1) / kHllTileBytes);
        symbols += n_elem[i];
    }
    tile_start[n] = tiles;
    std::vector<unsigned long long> keys(capacity, 0), head(8, 0);
    std::vector<uint32_t> counts(capacity, 0);
    uint32_t g1 = grid > tiles ? tiles : grid;
    emu::launch(g1, 256, 0, [&] {
        symbol_count_kernel(d.data(), tile_start.data(), (uint32_t)n, tiles, keys.data(), counts.data(), capacity - 1,
                            (uint32_t*)&head[2]);
    });
    emu::launch(grid, 256, 0, [&] { model_scan_kernel(keys.data(), counts.data(), capacity, head.data()); });
    const double scale = std::ldexp(1.0, (int)factor_scale_log2), factor = scale / (double)symbols;
    const unsigned long long max_key = kSymUsed | (0xFFFFFFFFull - (head[1] & 0xFFFFFFFFull));
    std::vector<double> partial(2 * grid, 0.0);
    emu::launch(grid, 256, 0, [&] { model_cost_kernel(keys.data(), counts.data(), capacity, factor, scale, max_key, partial.data()); });
    out[0] = (double)head[0];
    out[1] = (double)(head[1] >> 32);
    out[2] = (double)(uint32_t)head[2];
    out[3] = out[4] = 0.0;
    for (uint32_t b = 0; b < grid; ++b) {
        out[3] += partial[2 * b];
        out[4] += partial[2 * b + 1];
    }
}

// container version 3 restore without a merge pass: n groups of `planes` planes each (1: 2-byte elements, 2: 4-byte)
// item arrays are indexed [group * planes + plane]
void emu_decode_planes(size_t n, uint32_t planes, uint8_t* const* dsts, const uint8_t* const* lows, const uint64_t* n_elem,
                       const uint64_t* payload_off, const uint32_t* raw, const uint32_t* cf, const uint32_t* hdrs,
                       const uint8_t* payload, uint32_t* status_out, uint32_t grid) {
    std::vector<PlaneGroup> g(n);
    std::vector<uint32_t> order(n);
    for (size_t i = 0; i < n; ++i) {
        g[i] = PlaneGroup{};
        g[i].dst = dsts[i];
        g[i].low = lows[i];
        g[i].n_elem = n_elem[i];
        for (uint32_t p = 0; p < planes; ++p) {
            const uint32_t k = (uint32_t)(i * planes + p);
            g[i].plane[p] = PlaneItem{payload_off[k], k, k, raw[k], k};
        }
        order[i] = (uint32_t)(n - 1 - i);
    }
    std::memset(status_out, 0, n * planes * 4);
    uint32_t ticket = 0;
    if (planes == 2)
        emu::launch(grid, 2 * kTeam, sizeof(PlaneDecSmem<2>), [&] {
            rans_decode_planes_kernel<2>(g.data(), cf, (const LaneHeader*)hdrs, payload, order.data(), &ticket, (uint32_t)n, status_out);
        });
    else
        emu::launch(grid, kTeam, sizeof(PlaneDecSmem<1>), [&] {
            rans_decode_planes_kernel<1>(g.data(), cf, (const LaneHeader*)hdrs, payload, order.data(), &ticket, (uint32_t)n, status_out);
        });
}

// the host routine the device kernel must agree with
void emu_host_enc_entries(const uint32_t* nf, const uint32_t* cf, uint32_t* enc_out) {
    FreqTable ft;
    std::memcpy(ft.norm_freq, nf, 1024);
    std::memcpy(ft.cum_freq, cf, 1028);
    build_enc_entries(ft, (EncEntry*)enc_out);
}

// normalize_tables_kernel over n histograms (taken as they are: the descriptors carry no low bytes).
// enc_out n*256*4 words, freq_out n*256, cum_out n*257, sums_out n.
void emu_normalize_tables(size_t n, const uint32_t* hist, const uint32_t* flags, uint32_t* enc_out, uint32_t* freq_out,
                          uint32_t* cum_out, uint32_t* sums_out, uint32_t grid) {
    std::vector<TensorDesc> descs(n);
    std::vector<TableJob> jobs(n);
    for (size_t i = 0; i < n; ++i) {
        std::memset(&descs[i], 0, sizeof(TensorDesc));
        descs[i].es = 1;
        jobs[i].owner = (uint32_t)i;
        jobs[i].flags = flags[i];
    }
    emu::launch(grid, 256, 0, [&] {
        normalize_tables_kernel(jobs.data(), descs.data(), hist, (EncEntry*)enc_out, freq_out, cum_out, sums_out, (uint32_t)n);
    });
}

// sort_replica and the library routine it reproduces, on the same keys (symbols 0..n-1 in input order).
void emu_sort_replica(size_t n, const double* frac, int32_t* sym_out) {
    std::vector<FracKey> k(n);
    for (size_t i = 0; i < n; ++i) k[i] = FracKey{frac[i], (int32_t)i, 0};
    sort_replica(k.data(), (int)n);
    for (size_t i = 0; i < n; ++i) sym_out[i] = k[i].sym;
}
void emu_std_sort(size_t n, const double* frac, int32_t* sym_out) {
    std::vector<FracKey> k(n);
    for (size_t i = 0; i < n; ++i) k[i] = FracKey{frac[i], (int32_t)i, 0};
    std::sort(k.begin(), k.end(), [](const FracKey& a, const FracKey& b) { return a.frac > b.frac; });
    for (size_t i = 0; i < n; ++i) sym_out[i] = k[i].sym;
}
void emu_heap_sort_pair(size_t n, const double* frac, int32_t* replica_out, int32_t* std_out) {
    std::vector<FracKey> a(n), b;
    for (size_t i = 0; i < n; ++i) a[i] = FracKey{frac[i], (int32_t)i, 0};
    b = a;
    sr_heap_sort(a.data(), a.data() + n);
    std::partial_sort(b.begin(), b.end(), b.end(), [](const FracKey& x, const FracKey& y) { return x.frac > y.frac; });
    for (size_t i = 0; i < n; ++i) {
        replica_out[i] = a[i].sym;
        std_out[i] = b[i].sym;
    }
}
// An input on which the library's quicksort degenerates (M. D. McIlroy's adversary: the
// comparator fixes values while std::sort runs), so the depth limit and the heap sort are reached.
void emu_sort_killer(size_t n, double* frac_out) {
    std::vector<double> val(n);
    const double gas = 1e18;
    int nsolid = 0, candidate = 0;
    std::vector<int> idx(n);
    for (size_t i = 0; i < n; ++i) {
        idx[i] = (int)i;
        val[i] = gas;
    }
    auto cmp = [&](int x, int y) {
        if (val[x] == gas && val[y] == gas) {
            if (x == candidate) val[x] = nsolid++; else val[y] = nsolid++;
        }
        if (val[x] == gas) candidate = x; else if (val[y] == gas) candidate = y;
        return val[x] > val[y];
    };
    std::sort(idx.begin(), idx.end(), cmp);
    for (size_t i = 0; i < n; ++i) frac_out[i] = val[i] == gas ? (double)nsolid : val[i];
}

uint32_t emu_stats_out_bytes() { return (uint32_t)sizeof(StatsOut); }

}  // extern "C"

// ---------------------------------------------------------------- Re-Pair kernels
#include "repair_kernels.cuh"

extern "C" {

// Pair table of a token sequence: returns the number of occupied slots; keys/counts/first get the
// occupied entries (capacity n), best[0] the largest count, best[1] how many keys reach it.
uint32_t emu_repair_count(const uint32_t* tokens, uint32_t n, unsigned long long* keys_out, uint32_t* counts_out,
                          uint32_t* first_out, uint32_t* best, uint32_t grid) {
    using namespace chkrp;
    uint32_t cap = 1024;
    while (cap < 2ull * n) cap <<= 1;
    std::vector<unsigned long long> keys(cap, kEmptyKey), tie_keys(8);
    std::vector<uint32_t> counts(cap, 0), first(cap, 0xFFFFFFFFu), tie_first(8);
    uint32_t small[4] = {0, 0, 0, 0};
    emu::launch(grid, 256, 0, [&] { pair_count_kernel(tokens, n, keys.data(), counts.data(), first.data(), cap - 1, small + 2); });
    emu::launch(grid, 256, 0, [&] { pair_max_kernel(counts.data(), cap, small); });
    emu::launch(grid, 256, 0, [&] {
        pair_ties_kernel(keys.data(), counts.data(), first.data(), cap, small, tie_keys.data(), tie_first.data());
    });
    emu::launch(grid, 256, 0, [&] {
        pair_dump_kernel(keys.data(), counts.data(), first.data(), cap, small + 3, keys_out, counts_out, first_out);
    });
    best[0] = small[0];
    best[1] = small[1];
    best[2] = small[2];
    return small[3];
}

// One rule application; returns the new length.
uint32_t emu_repair_apply(const uint32_t* tokens, uint32_t n, uint32_t lhs, uint32_t rhs, uint32_t new_sym,
                          uint32_t* out, uint32_t grid) {
    using namespace chkrp;
    if (!n) return 0;
    const uint32_t nb = (n + kScanBlock - 1) / kScanBlock;
    std::vector<uint32_t> mark(n), run_start(n, 0xDEADBEEF), keep(n), pos(n), blocks(nb + 8);
    auto scan = [&](int op, const uint32_t* in, uint32_t* o) {
        if (op == 0) {
            emu::launch(nb, 256, 0, [&] { scan_reduce_kernel<0>(in, n, blocks.data()); });
            emu::launch(1, 256, 0, [&] { scan_blocks_kernel<0>(blocks.data(), nb); });
            emu::launch(nb, 256, 0, [&] { scan_apply_kernel<0>(in, n, blocks.data(), o); });
        } else {
            emu::launch(nb, 256, 0, [&] { scan_reduce_kernel<1>(in, n, blocks.data()); });
            emu::launch(1, 256, 0, [&] { scan_blocks_kernel<1>(blocks.data(), nb); });
            emu::launch(nb, 256, 0, [&] { scan_apply_kernel<1>(in, n, blocks.data(), o); });
        }
    };
    if (lhs == rhs) {
        emu::launch(grid, 256, 0, [&] { run_mark_kernel(tokens, n, lhs, mark.data()); });
        scan(1, mark.data(), run_start.data());
    }
    emu::launch(grid, 256, 0, [&] { rule_flags_kernel(tokens, n, lhs, rhs, run_start.data(), keep.data()); });
    scan(0, keep.data(), pos.data());
    emu::launch(grid, 256, 0, [&] {
        rule_scatter_kernel(tokens, n, lhs, rhs, new_sym, run_start.data(), keep.data(), pos.data(), out);
    });
    return blocks[nb];
}

void emu_repair_mask(const uint8_t* raw, uint64_t n, uint32_t storage_bytes, uint32_t masked_bits, uint32_t* tokens,
                     uint32_t grid) {
    emu::launch(grid, 256, 0, [&] { chkrp::mask_words_kernel(raw, n, storage_bytes, masked_bits, tokens); });
}

}  // extern "C"
