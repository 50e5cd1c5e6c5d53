// engine.cu -- host side of libcheckers_b200.so: context, registry, the batched
// compress / restore pipelines, analysis, file images, and the C ABI declared
// in include/checkers_b200.h.  Device code is in kernels.cuh.
//
// How the reference's per-tensor, mutex-serialised loop
// (ANSCompressor::compress_and_save_all, src/ANSCompressor.cpp:1014-1401 in the
// Checkers tree: >= 8 stream syncs and 3 device-to-host copies per tensor) is
// re-shaped here: all tensors of a rank go through each stage together --
//   split_hist_kernel         low bytes -> final .mant data layout, histograms; in a few pieces
//   normalize_tables_kernel   frequency tables and encode entries of a piece, on the device,
//   zero_chain_kernel         while the next piece is counted (a second stream)
//   rans_encode_fused_kernel  one persistent grid of 64-thread teams, one tensor at a time each,
//                             largest first: lanes, lane offsets, passthrough rule, headers and
//                             the gather of the lanes into a payload heap
// with ONE host synchronisation per checkpoint; the payload of each tensor is then copied
// to its place in the .ansc image (file order) and the other two images by a large copy each.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <cstddef>
#include <algorithm>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/checkers_b200.h"
#include "clusters.hpp"
#include "kernels.cuh"
#include "tables.hpp"

namespace chk {

// ------------------------------------------------------------------ errors
struct Error {
    int code;
    std::string msg;
};
static thread_local std::string g_last_error;

#define CHK_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess)                                                                      \
            throw Error{CHK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)};          \
    } while (0)

static inline uint32_t elem_size(uint8_t dt) {
    switch (dt) {
        case CHK_F32: return 4;
        case CHK_BF16: return 2;
        case CHK_F16: return 2;
        case CHK_I8: return 1;
        case CHK_I32: return 4;
        default: return 0;
    }
}
static inline uint32_t sidecar_per_elem(uint8_t dt) {
    switch (dt) {
        case CHK_BF16:
        case CHK_F16: return 1;
        case CHK_F32: return 2;
        default: return 0;
    }
}

// ------------------------------------------------------------------ file layout constants
constexpr uint32_t kStatesMagic = 0x414E5343u, kStatesVersion = 2;
constexpr uint32_t kMantMagic = 0x4D414E54u, kMantVersion = 2;
constexpr uint32_t kDictMagic = 0x44494354u, kDictVersion = 1;
constexpr size_t kStatesEntry = 4648, kMantEntry = 288, kDictEntry = 2308, kFileHeader = 16;

// ------------------------------------------------------------------ buffers
struct DevBuf {
    void* p = nullptr;
    size_t cap = 0;
};
struct PinBuf {
    void* p = nullptr;
    size_t cap = 0;
    size_t size = 0;
};

struct Tensor {
    std::string name;
    void* ptr;
    uint64_t n_elem;
    uint8_t dtype, category;
    bool hot = false;  // an 8-bit plane whose bytes take few values (container version 3): counted in the spread bins
};

struct WorkItem {
    size_t idx;  // registry index
    uint64_t bytes;
    uint32_t es, spe;
    bool owns;
    int table;  // table index in .dict order
    std::string anchor_name;
};

struct Context {
    int device = 0, rank = 0, local_rank = 0;
    cudaStream_t stream = nullptr;
    cudaMemPool_t pool = nullptr;
    cudaEvent_t ev[8] = {};
    std::vector<Tensor> tensors;
    uint32_t histogram_bins = 256;

    bool have_clusters = false;
    ClusterMap clusters;
    std::vector<StatsOut> stats;
    std::vector<uint8_t> hll;     // one 2^14-register sketch per registered tensor (chk_hll_sketch_all)

    bool repair_tables = false, verify_zero_lanes = false, allow_undecodable = false;
    bool fast_stats = false;      // statistics with order-free sums over the whole device (see stats_kernels.cuh)
    bool precounted = false;      // the caller filled d_hist (one row per work item) itself: compress() does not count
    bool v3_fused_decode = true;  // container version 3: decode planes straight into whole elements (no merge pass)
    bool skip_decode = false;     // decompress_images stops after parsing and uploading: the caller decodes (format_v3.inc)
    std::vector<TensorDesc> last_run;       // with skip_decode: the parsed entries, in upload order (lane headers k at k * 4096)
    std::vector<size_t> last_run_tensor;    // and the registry index of each
    int format_version = 2;       // 2: the reference's container; 3: byte planes with a table each (format_v3.inc)
    uint32_t file_version[3] = {kStatesVersion, kMantVersion, kDictVersion};  // written to and expected in the headers
    struct V3State* v3 = nullptr;
    uint64_t registry_epoch = 0;  // changes whenever the registered tensors change
    bool decode_zero_skip = false; // float tensors whose table allows it are decoded with the short slot table (measured slower)

    // device buffers (grow-only, from the context's pool)
    DevBuf d_descs, d_tiles, d_hist, d_sidecar, d_scratch, d_hdrs, d_order, d_ticket, d_psize, d_zslots, d_zregions, d_zslot_of, d_jobs, d_sums, d_stats_part, d_stats_mid, d_poff, d_fileorder, d_hll32, d_hll8, d_symkeys, d_symcounts,
        d_payload, d_enc, d_freq, d_cum, d_status, d_stats_desc, d_stats_out;
    cudaStream_t side_stream = nullptr;
    std::vector<cudaEvent_t> ev_count, ev_tab;
    int segments = 4;             // launches the counting of a batch is cut into (tables of a piece are built under the next)
    uint64_t workspace_bytes = 0; // bound on the encode scratch (0 = one slot for every team the device can hold)
    int encode_teams_per_sm = 0;  // cap on resident encode teams per SM and launch (0 = as many as fit)
    int decode_teams_per_sm = 0;  // same for the decode grid
    int sm_count = 0;
    // pinned host staging
    PinBuf h_hdrs, h_poff, h_psize, h_descs, h_status, h_jobs, h_sums, h_freq, h_cum, h_stats, h_order, h_tiles;
    PinBuf img[3];  // states, mantissa, tables
    // Where the next compress builds its file images instead of img[] (caller-owned pinned memory of
    // at least the worst-case sizes); the chunked host pipeline keeps one set per part this way.
    void* img_ext[3] = {nullptr, nullptr, nullptr};
    size_t img_ext_cap[3] = {0, 0, 0};
    bool blocking_sync = false;
    cudaEvent_t ev_block = nullptr;

    // result of the last compression
    std::vector<WorkItem> work;
    size_t n_tables = 0;
    std::vector<uint32_t> table_sums;  // per table of the last compression: 4096 when decodable
    uint64_t undecodable_tables = 0;
    std::vector<TensorDesc> descs;  // host copy, payload_off / flags filled in
    bool have_resident = false, have_images = false;
    chk_summary summary{};
    uint64_t restored = 0;

    std::map<std::string, double> timing;
    uint64_t launches = 0;
};

// container version 3 (format_v3.inc, at the end of this file)
static void v3_compress(Context* c, bool host_images);
static void v3_decompress_resident(Context* c, void* const* dst);
static void v3_decompress_images(Context* c, const uint8_t* st, size_t st_n, const uint8_t* mt, size_t mt_n,
                                 const uint8_t* dc, size_t dc_n);
static const void* v3_image_ptr(const Context* c, int k);
static size_t v3_image_size(const Context* c, int k);
static void v3_destroy(Context* c);

static void dev_ensure(Context* c, DevBuf& b, size_t bytes) {
    bytes = (bytes + 255) & ~(size_t)255;
    if (bytes == 0) bytes = 256;
    if (b.cap >= bytes) return;
    if (b.p) CHK_CUDA(cudaFreeAsync(b.p, c->stream));
    b.p = nullptr;
    b.cap = 0;
    // grow with some slack so near-equal batches reuse the allocation
    const size_t want = bytes + bytes / 16;
    CHK_CUDA(cudaMallocFromPoolAsync(&b.p, want, c->pool, c->stream));
    b.cap = want;
}
static void pin_ensure(PinBuf& b, size_t bytes) {
    b.size = bytes;
    if (bytes == 0) bytes = 16;
    if (b.cap >= bytes) return;
    if (b.p) cudaFreeHost(b.p);
    b.p = nullptr;
    b.cap = 0;
    const size_t want = bytes + bytes / 16;
    // mapped: the control kernels below read and write this memory directly
    CHK_CUDA(cudaHostAlloc(&b.p, want, cudaHostAllocMapped | cudaHostAllocPortable));
    b.cap = want;
}

// Waits for a stream.  A context that is one of several driven by host threads at once (the chunked
// host pipeline) sleeps on a blocking event instead of spinning on a core.
static void sync_stream(Context* c, cudaStream_t s);

static double ms_between(cudaEvent_t a, cudaEvent_t b) {
    float ms = 0;
    cudaEventElapsedTime(&ms, a, b);
    return ms;
}
static double wall_ms(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

// Control data (descriptors, histograms, offsets, status words) moves between pinned host
// memory and the device through these kernels, not through the copy engines.  A copy engine
// serves transfers in submission order across all streams, so a few KB of control data would
// wait behind every bulk transfer that a pipelined caller (several contexts, chunked
// host-resident state) has queued; a kernel that loads or stores the pinned pages directly
// does not queue there.
__global__ void control_copy_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, size_t n_words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
}
__global__ void control_fill_kernel(uint32_t* __restrict__ dst, size_t n_words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = 0u;
}
static uint32_t control_grid(size_t n_words) {
    const size_t blocks = (n_words + 255) / 256;
    return (uint32_t)(blocks < 592 ? (blocks ? blocks : 1) : 592);
}
// bytes must be a multiple of 4; one side is device memory, the other pinned (mapped) host memory
static void control_copy(Context* c, void* dst, const void* src, size_t bytes, cudaStream_t s) {
    if (bytes == 0) return;
    control_copy_kernel<<<control_grid(bytes / 4), 256, 0, s>>>(static_cast<uint32_t*>(dst),
                                                                static_cast<const uint32_t*>(src), bytes / 4);
    CHK_CUDA(cudaGetLastError());
    c->launches++;
}
static void control_zero(Context* c, void* dst, size_t bytes, cudaStream_t s) {
    if (bytes == 0) return;
    control_fill_kernel<<<control_grid(bytes / 4), 256, 0, s>>>(static_cast<uint32_t*>(dst), bytes / 4);
    CHK_CUDA(cudaGetLastError());
    c->launches++;
}

static void sync_stream(Context* c, cudaStream_t s) {
    if (!c->blocking_sync) {
        CHK_CUDA(cudaStreamSynchronize(s));
        return;
    }
    if (!c->ev_block) CHK_CUDA(cudaEventCreateWithFlags(&c->ev_block, cudaEventBlockingSync | cudaEventDisableTiming));
    CHK_CUDA(cudaEventRecord(c->ev_block, s));
    CHK_CUDA(cudaEventSynchronize(c->ev_block));
}

// The buffer image k of the next compress is built in: the caller's, if one was installed, else the context's own.
static uint8_t* image_buffer(Context* c, int k, size_t bytes) {
    if (c->img_ext[k]) {
        if (bytes > c->img_ext_cap[k])
            throw Error{CHK_ERR_CAPACITY, "file image " + std::to_string(k) + " needs " + std::to_string(bytes) +
                                              " bytes, the buffer provided holds " + std::to_string(c->img_ext_cap[k])};
        c->img[k].size = bytes;
        return static_cast<uint8_t*>(c->img_ext[k]);
    }
    pin_ensure(c->img[k], bytes);
    return static_cast<uint8_t*>(c->img[k].p);
}
static const void* image_ptr(const Context* c, int k) {
    if (c->format_version == 3 && k != 1) return v3_image_ptr(c, k);
    return c->img_ext[k] ? c->img_ext[k] : c->img[k].p;
}
static size_t image_size(const Context* c, int k) {
    if (c->format_version == 3 && k != 1) return v3_image_size(c, k);
    return c->img[k].size;
}

// ------------------------------------------------------------------ work list
// Order, ownership and sharing rules of compress_and_save_all
// (src/ANSCompressor.cpp:1056-1078, :1210, :1239-1261, :1352-1371).
static void build_work(Context* c) {
    c->work.clear();
    std::unordered_map<int, bool> seen;
    std::unordered_map<int, int> cluster_table;
    int n_tables = 0;
    for (size_t i = 0; i < c->tensors.size(); ++i) {
        const Tensor& t = c->tensors[i];
        if (!t.ptr || t.n_elem == 0) continue;
        int cid = -1;
        if (c->have_clusters) {
            auto it = c->clusters.tensor_to_cluster.find(t.name);
            if (it != c->clusters.tensor_to_cluster.end()) cid = it->second;
        }
        const bool single = cid == -1;
        bool anchor = false;
        if (!single && !seen[cid]) {
            seen[cid] = true;
            anchor = true;
        }
        const uint32_t es = elem_size(t.dtype);
        const uint64_t bytes = t.n_elem * es;
        if (bytes == 0) continue;  // unknown dtype: never produces a result (:1133)
        WorkItem w;
        w.idx = i;
        w.bytes = bytes;
        w.es = es;
        w.spe = sidecar_per_elem(t.dtype);
        w.owns = anchor || single;
        if (w.owns) {
            w.table = n_tables++;
            if (!single) cluster_table[cid] = w.table;
        } else {
            auto it = cluster_table.find(cid);
            if (it == cluster_table.end()) continue;  // its anchor produced no table (the reference waits forever)
            w.table = it->second;
            auto an = c->clusters.cluster_anchor.find(cid);
            if (an != c->clusters.cluster_anchor.end()) w.anchor_name = an->second;
        }
        if (bytes >= (1ull << 32))
            throw Error{CHK_ERR_CAPACITY, "tensor '" + t.name + "' is 4 GiB or larger; lane offsets are 32-bit"};
        c->work.push_back(std::move(w));
    }
    // whether a table is built with the full alphabet: owner that is a cluster anchor
    c->n_tables = (size_t)n_tables;
}

static bool is_cluster_anchor(const Context* c, const WorkItem& w) {
    if (!w.owns || !c->have_clusters) return false;
    auto it = c->clusters.tensor_to_cluster.find(c->tensors[w.idx].name);
    return it != c->clusters.tensor_to_cluster.end() && it->second != -1;
}

static void put_name(uint8_t* dst, const std::string& s) {
    std::memset(dst, 0, 256);
    std::memcpy(dst, s.data(), s.size() < 255 ? s.size() : 255);
}
template <typename T>
static void put(uint8_t* dst, T v) {
    std::memcpy(dst, &v, sizeof(T));
}
template <typename T>
static T get(const uint8_t* src) {
    T v;
    std::memcpy(&v, src, sizeof(T));
    return v;
}
static std::string get_name(const uint8_t* p) {
    size_t n = 0;
    while (n < 256 && p[n]) ++n;
    return std::string(reinterpret_cast<const char*>(p), n);
}

// Largest-first processing order of a batch plus a zeroed ticket counter for
// the persistent encode / decode kernels.
template <typename SizeFn>
static void upload_order(Context* c, size_t W, SizeFn&& size_of) {
    std::vector<uint32_t> order(W);
    for (size_t i = 0; i < W; ++i) order[i] = (uint32_t)i;
    std::stable_sort(order.begin(), order.end(),
                     [&](uint32_t a, uint32_t b) { return size_of(a) > size_of(b); });
    pin_ensure(c->h_order, W * 4);
    std::memcpy(c->h_order.p, order.data(), W * 4);
    dev_ensure(c, c->d_order, W * 4);
    dev_ensure(c, c->d_ticket, 256);
    control_copy(c, c->d_order.p, c->h_order.p, W * 4, c->stream);
    control_zero(c, c->d_ticket.p, 256, c->stream);
}

// blocking: a host thread that waits for the event sleeps instead of spinning on a core
static void ensure_events(std::vector<cudaEvent_t>& v, size_t n, bool timing, bool blocking = false) {
    while (v.size() < n) {
        cudaEvent_t e = nullptr;
        CHK_CUDA(cudaEventCreateWithFlags(&e, (timing ? cudaEventDefault : cudaEventDisableTiming) |
                                                  (blocking ? cudaEventBlockingSync : 0)));
        v.push_back(e);
    }
}

// Grid of a persistent team kernel: as many teams as fit on the device at once.
static uint32_t persistent_grid(Context* c, const void* kernel, size_t smem, size_t W, int cap_per_sm = 0) {
    int per_sm = 0;
    CHK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, (int)kTeam, smem));
    if (cap_per_sm > 0 && per_sm > cap_per_sm) per_sm = cap_per_sm;
    if (per_sm < 1) per_sm = 1;
    const size_t cap = (size_t)per_sm * (size_t)(c->sm_count > 0 ? c->sm_count : 1);
    return (uint32_t)(W < cap ? W : cap);
}

// ------------------------------------------------------------------ compress
// The whole call is queued in one go -- the host never waits in between:
//   count stream   split_hist_kernel over the batch, in a few launches ("segments")
//   table stream   normalize_tables_kernel for each of those pieces as soon as it is counted, so
//                  only the tables of the last piece are not hidden under the counting
//   count stream   one persistent rans_encode_fused_kernel for the whole batch: lanes, symbol-0
//                  chains, lane and tensor offsets, headers and the gather into the data-section
//                  layout, tensor by tensor inside the teams.  Its scratch is one slot per
//                  resident team; a workspace bound simply means fewer teams.
// Counting and encoding contend for the same units of an SM (shared-memory atomics against table
// lookups): run side by side they only take turns, so they run one after the other, while the
// memory-bound gather of finished tensors hides under the issue-bound chains of the others.
static void compress(Context* c, bool host_images) {
    if (c->format_version == 3) return v3_compress(c, host_images);
    const auto t_total = std::chrono::steady_clock::now();
    CHK_CUDA(cudaSetDevice(c->device));
    c->have_resident = c->have_images = false;
    c->summary = chk_summary{};
    c->undecodable_tables = 0;
    build_work(c);
    const size_t W = c->work.size();
    const size_t T = c->n_tables;
    cudaStream_t s = c->stream;

    c->descs.assign(W, TensorDesc{});
    pin_ensure(c->h_tiles, (W + 1) * 4);
    uint32_t* tile_start = static_cast<uint32_t*>(c->h_tiles.p);
    tile_start[0] = 0;
    unsigned long long sidecar_total = 0, bytes_total = 0, slot_bytes = 0;
    uint32_t max_stride = 0;
    size_t n_sidecars = 0;
    bool any_member = false, any_int = false;
    for (size_t i = 0; i < W; ++i) {
        const WorkItem& w = c->work[i];
        TensorDesc& d = c->descs[i];
        d.src = static_cast<const uint8_t*>(c->tensors[w.idx].ptr);
        d.dst = nullptr;
        d.n_bytes = w.bytes;
        d.es = w.es;
        d.spe = w.spe;
        d.table_idx = (uint32_t)w.table;
        d.sidecar_off = sidecar_total;
        d.scratch_off = 0;  // lanes go to the slot of whichever team encodes the tensor
        const unsigned long long c_max = (w.bytes + 255) / 256;
        d.chunk_stride = (uint32_t)((2 * c_max + 31) & ~31ull);
        d.flags = w.owns ? kFlagNeedHist : 0u;
        if (c->tensors[w.idx].hot) d.flags |= kFlagHotBins;
        if ((reinterpret_cast<uintptr_t>(d.src) & 15) == 0 && (sidecar_total & 15) == 0) d.flags |= kFlagAligned;
        sidecar_total += (unsigned long long)c->tensors[w.idx].n_elem * w.spe;
        // value-lane regions, plus one shared region for the lanes that only see zeroed bytes
        const unsigned long long need = (w.spe * 2 == w.es ? 129ull : 256ull) * d.chunk_stride;
        if (need > slot_bytes) slot_bytes = need;
        if (d.chunk_stride > max_stride) max_stride = d.chunk_stride;
        bytes_total += w.bytes;
        n_sidecars += w.spe > 0;
        any_member = any_member || !w.owns;
        any_int = any_int || w.spe * 2 != w.es;
        tile_start[i + 1] = tile_start[i] + (uint32_t)((w.bytes + kSplitTileBytes - 1) / kSplitTileBytes);
    }

    if (W == 0) {
        c->have_resident = true;
        c->table_sums.clear();
        if (host_images) {
            const uint32_t magic[3] = {kStatesMagic, kMantMagic, kDictMagic};
            const uint32_t* ver = c->file_version;
            for (int k = 0; k < 3; ++k) {
                uint8_t* p = image_buffer(c, k, kFileHeader);
                put<uint32_t>(p, magic[k]);
                put<uint32_t>(p + 4, ver[k]);
                put<uint32_t>(p + 8, (uint32_t)(c->rank < 0 ? 0 : c->rank));
                put<uint32_t>(p + 12, 0);
            }
            c->have_images = true;
            c->summary.states_bytes = c->summary.mantissa_bytes = c->summary.dict_bytes = kFileHeader;
        }
        return;
    }

    // ---- the encode grid and its scratch: one slot (the largest tensor's lane regions) per team
    slot_bytes = (slot_bytes + 255) & ~255ull;
    auto kernel = any_int ? rans_encode_fused_kernel<true> : rans_encode_fused_kernel<false>;
    const size_t smem = any_int ? sizeof(EncSmem<4>) : sizeof(EncSmem<2>);
    uint32_t teams = persistent_grid(c, reinterpret_cast<const void*>(kernel), smem, W, c->encode_teams_per_sm);
    if (c->workspace_bytes) {
        const unsigned long long fit = c->workspace_bytes / slot_bytes;
        if (fit == 0)
            throw Error{CHK_ERR_CAPACITY, "workspace of " + std::to_string(c->workspace_bytes) + " bytes is smaller than the " +
                                              std::to_string(slot_bytes) + " bytes of encode scratch the largest tensor needs"};
        if (fit < teams) teams = (uint32_t)fit;
    }

    // ---- pieces the batch is counted in (equal bytes; a small batch is one piece).  The tables of a piece are
    // built while the next piece is counted, so a piece must take about as long to count as the tables of the
    // one before take to build: a small last piece (1/16 of the bytes) exposed more table time, not less.
    const size_t n_seg = W >= 512 && !c->precounted ? (size_t)c->segments : 1;
    std::vector<size_t> seg_end;
    {
        unsigned long long acc = 0;
        for (size_t i = 0; i < W; ++i) {
            acc += c->descs[i].n_bytes;
            if (seg_end.size() + 1 < n_seg && acc * n_seg >= bytes_total * (seg_end.size() + 1)) seg_end.push_back(i + 1);
        }
        if (!seg_end.empty() && seg_end.back() == W) seg_end.pop_back();
        seg_end.push_back(W);
    }
    const size_t n_win = seg_end.size();

    dev_ensure(c, c->d_descs, W * sizeof(TensorDesc));
    dev_ensure(c, c->d_tiles, (W + 1) * 4);
    dev_ensure(c, c->d_hist, W * 1024);
    dev_ensure(c, c->d_sidecar, sidecar_total + 64);
    dev_ensure(c, c->d_scratch, (unsigned long long)teams * slot_bytes + 64);
    // the batch's distinct symbol-0 chains (a handful: see zero_chain_kernel)
    const uint32_t z_slots = (uint32_t)(n_sidecars < 64 ? (n_sidecars ? n_sidecars : 1) : 64);
    dev_ensure(c, c->d_zslots, z_slots * sizeof(ZeroSlot));
    dev_ensure(c, c->d_zregions, (unsigned long long)z_slots * max_stride + 64);
    dev_ensure(c, c->d_zslot_of, W * 4);
    dev_ensure(c, c->d_hdrs, W * 4096);
    dev_ensure(c, c->d_ticket, 256);
    dev_ensure(c, c->d_order, W * 4);
    dev_ensure(c, c->d_psize, W * 8);
    dev_ensure(c, c->d_payload, bytes_total + (unsigned long long)kPayloadAlign * W + 64);  // a heap: every range starts on a sector
    dev_ensure(c, c->d_enc, T * 256 * sizeof(EncEntry));
    dev_ensure(c, c->d_freq, T * 256 * 4);
    dev_ensure(c, c->d_cum, T * 257 * 4);
    dev_ensure(c, c->d_jobs, T * sizeof(TableJob));
    dev_ensure(c, c->d_sums, T * 4);
    pin_ensure(c->h_hdrs, host_images ? W * 4096 : 0);
    pin_ensure(c->h_poff, (W + 1) * 8);
    pin_ensure(c->h_psize, W * 8);
    pin_ensure(c->h_order, W * 4);
    pin_ensure(c->h_descs, W * sizeof(TensorDesc));
    pin_ensure(c->h_jobs, T * sizeof(TableJob));
    pin_ensure(c->h_sums, T * 4 + 4);
    const bool want_tables = host_images || any_member;
    pin_ensure(c->h_freq, want_tables ? T * 256 * 4 : 0);
    pin_ensure(c->h_cum, host_images ? T * 257 * 4 : 0);

    std::memcpy(c->h_descs.p, c->descs.data(), W * sizeof(TensorDesc));
    {
        TableJob* jobs = static_cast<TableJob*>(c->h_jobs.p);
        for (size_t i = 0; i < W; ++i) {
            const WorkItem& w = c->work[i];
            if (!w.owns) continue;
            const bool full = is_cluster_anchor(c, w);
            jobs[w.table].owner = (uint32_t)i;
            jobs[w.table].flags = (full ? kTableFullAlphabet : 0u) | (full && c->repair_tables ? kTableRepair : 0u);
        }
        // largest tensors first, so the persistent grid drains the batch without a ragged last wave
        uint32_t* ord = static_cast<uint32_t*>(c->h_order.p);
        for (size_t i = 0; i < W; ++i) ord[i] = (uint32_t)i;
        std::stable_sort(ord, ord + W, [&](uint32_t x, uint32_t y) { return c->descs[x].n_bytes > c->descs[y].n_bytes; });
    }
    ensure_events(c->ev_count, n_win, true);
    ensure_events(c->ev_tab, n_win, true);

    c->timing["prepare_ms"] = wall_ms(t_total);
    CHK_CUDA(cudaEventRecord(c->ev[0], s));
    control_copy(c, c->d_descs.p, c->h_descs.p, W * sizeof(TensorDesc), s);
    control_copy(c, c->d_tiles.p, c->h_tiles.p, (W + 1) * 4, s);
    control_copy(c, c->d_jobs.p, c->h_jobs.p, T * sizeof(TableJob), s);
    control_copy(c, c->d_order.p, c->h_order.p, W * 4, s);
    if (!c->precounted) control_zero(c, c->d_hist.p, W * 1024, s);
    control_zero(c, c->d_ticket.p, 256, s);  // word 0: ticket counter; words 2-3: the 64-bit heap cursor
    control_zero(c, c->d_zslots.p, z_slots * sizeof(ZeroSlot), s);

    const uint32_t sms = (uint32_t)(c->sm_count > 0 ? c->sm_count : 1);
    size_t tab_done = 0;
    for (size_t g = 0, a = 0; g < n_win; ++g) {
        const size_t b = seg_end[g], n = b - a;
        const uint32_t tiles = tile_start[b] - tile_start[a];
        const uint32_t grid1 = tiles < sms * 8u ? tiles : sms * 8u;
        if (!c->precounted) {
            split_hist_kernel<<<grid1, 256, 0, s>>>(static_cast<const TensorDesc*>(c->d_descs.p) + a,
                                                    static_cast<const uint32_t*>(c->d_tiles.p) + a, (uint32_t)n, tile_start[a],
                                                    tiles, static_cast<uint8_t*>(c->d_sidecar.p),
                                                    static_cast<uint32_t*>(c->d_hist.p) + a * 256);
            CHK_CUDA(cudaGetLastError());
            c->launches++;
        }
        CHK_CUDA(cudaEventRecord(c->ev_count[g], s));
        // tables owned inside this piece: table numbers follow the work order, so they are a range
        size_t tab_hi = tab_done;
        for (size_t i = a; i < b; ++i)
            if (c->work[i].owns) tab_hi = (size_t)c->work[i].table + 1;
        CHK_CUDA(cudaStreamWaitEvent(c->side_stream, c->ev_count[g], 0));
        if (tab_hi > tab_done) {
            const size_t t0 = tab_done, nt = tab_hi - tab_done;
            // a job's owner index counts from the start of the batch: whole-batch descriptor and histogram arrays
            normalize_tables_kernel<<<(uint32_t)(nt < sms * 8u ? nt : sms * 8u), 256, 0, c->side_stream>>>(
                static_cast<const TableJob*>(c->d_jobs.p) + t0, static_cast<const TensorDesc*>(c->d_descs.p),
                static_cast<const uint32_t*>(c->d_hist.p), static_cast<EncEntry*>(c->d_enc.p) + t0 * 256,
                static_cast<uint32_t*>(c->d_freq.p) + t0 * 256, static_cast<uint32_t*>(c->d_cum.p) + t0 * 257,
                static_cast<uint32_t*>(c->d_sums.p) + t0, (uint32_t)nt);
            CHK_CUDA(cudaGetLastError());
            c->launches++;
            tab_done = tab_hi;
        }
        // the symbol-0 chains this piece needs and the batch does not have yet
        zero_chain_kernel<<<(uint32_t)n, 32, 0, c->side_stream>>>(
            static_cast<const TensorDesc*>(c->d_descs.p) + a, static_cast<const EncEntry*>(c->d_enc.p),
            static_cast<ZeroSlot*>(c->d_zslots.p), z_slots, static_cast<uint8_t*>(c->d_zregions.p), max_stride,
            static_cast<int32_t*>(c->d_zslot_of.p) + a, (uint32_t)n);
        CHK_CUDA(cudaGetLastError());
        c->launches++;
        CHK_CUDA(cudaEventRecord(c->ev_tab[g], c->side_stream));
        a = b;
    }
    CHK_CUDA(cudaStreamWaitEvent(s, c->ev_tab[n_win - 1], 0));  // the table stream is in order: all tables are complete
    CHK_CUDA(cudaEventRecord(c->ev[1], s));
    uint32_t* const ticket = static_cast<uint32_t*>(c->d_ticket.p);
    FusedParams fp{};
    fp.descs = static_cast<TensorDesc*>(c->d_descs.p);
    fp.tables = static_cast<const EncEntry*>(c->d_enc.p);
    fp.scratch = static_cast<uint8_t*>(c->d_scratch.p);
    fp.slot_bytes = slot_bytes;
    fp.zero_slots = static_cast<const ZeroSlot*>(c->d_zslots.p);
    fp.zero_regions = static_cast<const uint8_t*>(c->d_zregions.p);
    fp.zero_slot_of = static_cast<const int32_t*>(c->d_zslot_of.p);
    fp.zero_region_stride = max_stride;
    fp.n_tensors = (uint32_t)W;
    fp.hdrs = static_cast<LaneHeader*>(c->d_hdrs.p);
    fp.payload = static_cast<uint8_t*>(c->d_payload.p);
    fp.payload_size = static_cast<unsigned long long*>(c->d_psize.p);
    fp.heap_cursor = reinterpret_cast<unsigned long long*>(ticket + 2);
    fp.order = static_cast<const uint32_t*>(c->d_order.p);
    fp.ticket = ticket;
    kernel<<<teams, kTeam, smem, s>>>(fp);
    CHK_CUDA(cudaGetLastError());
    c->launches++;
    CHK_CUDA(cudaEventRecord(c->ev[2], s));
    c->timing["enqueue_ms"] = wall_ms(t_total);

    control_copy(c, c->h_psize.p, c->d_psize.p, W * 8, s);
    control_copy(c, c->h_descs.p, c->d_descs.p, W * sizeof(TensorDesc), s);
    control_copy(c, c->h_sums.p, c->d_sums.p, T * 4, s);
    if (host_images) control_copy(c, c->h_hdrs.p, c->d_hdrs.p, W * 4096, s);
    if (want_tables) control_copy(c, c->h_freq.p, c->d_freq.p, T * 256 * 4, s);
    if (host_images) control_copy(c, c->h_cum.p, c->d_cum.p, T * 257 * 4, s);
    sync_stream(c, s);

    c->timing["split_hist_ms"] = ms_between(c->ev[0], c->ev_count[n_win - 1]);
    c->timing["table_ms"] = ms_between(c->ev_count[n_win - 1], c->ev[1]);  // what the counting did not hide
    c->timing["encode_ms"] = ms_between(c->ev[1], c->ev[2]);                // lanes, offsets and gather
    c->timing["compact_ms"] = 0.0;                                          // part of the encode kernel
    c->timing["device_span_ms"] = ms_between(c->ev[0], c->ev[2]);
    c->timing["compress_device_ms"] = c->timing["device_span_ms"];
    c->timing["encode_teams"] = (double)teams;
    c->timing["workspace_mb"] = (double)((unsigned long long)teams * slot_bytes) / 1048576.0;
    c->timing["to_sync_ms"] = wall_ms(t_total);

    // descriptors come back with each tensor's place in the payload heap and its raw flag; the file wants
    // the payloads in index order, so the offsets written there are the running sum of the sizes
    std::memcpy(c->descs.data(), c->h_descs.p, W * sizeof(TensorDesc));
    const unsigned long long* psize = static_cast<const unsigned long long*>(c->h_psize.p);
    unsigned long long* poff = static_cast<unsigned long long*>(c->h_poff.p);
    poff[0] = 0;
    for (size_t i = 0; i < W; ++i) poff[i + 1] = poff[i] + psize[i];
    const unsigned long long payload_total = poff[W];
    const uint32_t* sums = static_cast<const uint32_t*>(c->h_sums.p);
    c->table_sums.assign(sums, sums + T);
    for (size_t t = 0; t < T; ++t) c->undecodable_tables += sums[t] != kM;
    if (any_member) {
        // the encode grids ran without the test for symbols missing from a borrowed table
        const uint32_t* fq = static_cast<const uint32_t*>(c->h_freq.p);
        for (size_t i = 0; i < W; ++i) {
            if (c->work[i].owns) continue;
            const uint32_t* f = fq + (size_t)c->work[i].table * 256;
            for (int sy = 0; sy < 256; ++sy)
                if (f[sy] == 0)
                    throw Error{CHK_ERR_INVALID, "internal: shared table of '" + c->tensors[c->work[i].idx].name +
                                                     "' lacks a symbol; shared tables must cover the full alphabet"};
        }
    }
    c->have_resident = true;

    c->summary.n_tensors = W;
    c->summary.n_tables = T;
    c->summary.original_bytes = bytes_total;
    c->summary.states_bytes = kFileHeader + W * kStatesEntry + payload_total;
    c->summary.mantissa_bytes = kFileHeader + n_sidecars * kMantEntry + sidecar_total;
    c->summary.dict_bytes = kFileHeader + T * kDictEntry;

    if (host_images) {
        const uint32_t rank_u = (uint32_t)(c->rank < 0 ? 0 : c->rank);
        CHK_CUDA(cudaEventRecord(c->ev[5], s));
        // states image (write_rank_states_file, src/ANSCompressor.cpp:751-816)
        uint8_t* st = image_buffer(c, 0, c->summary.states_bytes);
        const size_t st_data = kFileHeader + W * kStatesEntry;
        // heap order -> file order on the device, then the data section in one copy
        if (payload_total) {
            dev_ensure(c, c->d_poff, (W + 1) * 8);
            dev_ensure(c, c->d_fileorder, payload_total + 64);
            control_copy(c, c->d_poff.p, c->h_poff.p, (W + 1) * 8, s);
            const size_t cap = (size_t)(c->sm_count > 0 ? c->sm_count : 1) * 8;
            order_payload_kernel<<<(uint32_t)(W < cap ? W : cap), 256, 0, s>>>(
                static_cast<const TensorDesc*>(c->d_descs.p), static_cast<const unsigned long long*>(c->d_psize.p),
                static_cast<const unsigned long long*>(c->d_poff.p), static_cast<const uint8_t*>(c->d_payload.p),
                static_cast<uint8_t*>(c->d_fileorder.p), (uint32_t)W);
            CHK_CUDA(cudaGetLastError());
            c->launches++;
            CHK_CUDA(cudaMemcpyAsync(st + st_data, c->d_fileorder.p, payload_total, cudaMemcpyDeviceToHost, s));
        }
        // mantissa image (write_rank_mantissa_file, :839-887)
        uint8_t* mt = image_buffer(c, 1, c->summary.mantissa_bytes);
        const size_t mt_data = kFileHeader + n_sidecars * kMantEntry;
        if (sidecar_total)
            CHK_CUDA(cudaMemcpyAsync(mt + mt_data, c->d_sidecar.p, sidecar_total, cudaMemcpyDeviceToHost, s));
        // tables image (write_rank_tables_file, :903-931)
        uint8_t* dc = image_buffer(c, 2, c->summary.dict_bytes);

        put<uint32_t>(st, kStatesMagic);
        put<uint32_t>(st + 4, c->file_version[0]);
        put<uint32_t>(st + 8, rank_u);
        put<uint32_t>(st + 12, (uint32_t)W);
        put<uint32_t>(mt, kMantMagic);
        put<uint32_t>(mt + 4, c->file_version[1]);
        put<uint32_t>(mt + 8, rank_u);
        put<uint32_t>(mt + 12, (uint32_t)n_sidecars);
        put<uint32_t>(dc, kDictMagic);
        put<uint32_t>(dc + 4, c->file_version[2]);
        put<uint32_t>(dc + 8, rank_u);
        put<uint32_t>(dc + 12, (uint32_t)T);

        const LaneHeader* hdrs = static_cast<const LaneHeader*>(c->h_hdrs.p);
        const uint32_t* h_freq = static_cast<const uint32_t*>(c->h_freq.p);
        const uint32_t* h_cum = static_cast<const uint32_t*>(c->h_cum.p);
        size_t m_i = 0;
        for (size_t i = 0; i < W; ++i) {
            const WorkItem& w = c->work[i];
            const Tensor& t = c->tensors[w.idx];
            uint8_t* e = st + kFileHeader + i * kStatesEntry;
            put_name(e, t.name);
            const LaneHeader* lh = hdrs + i * 256;
            bool is_raw = lh[0].byte_count == (uint32_t)w.bytes;  // derived from the lane pattern (:787-789)
            for (int l = 1; l < 256 && is_raw; ++l) is_raw = lh[l].byte_count == 0;
            e[256] = t.dtype;
            e[257] = is_raw ? 1 : 0;
            e[258] = w.owns ? 1 : 0;
            std::memset(e + 259, 0, 5);
            put<uint64_t>(e + 264, w.bytes);
            put<uint64_t>(e + 272, t.n_elem);
            put<uint64_t>(e + 280, poff[i]);
            put<uint64_t>(e + 288, poff[i + 1] - poff[i]);
            put_name(e + 296, w.anchor_name);
            std::memcpy(e + 552, lh, 4096);
            if (w.spe) {
                uint8_t* m = mt + kFileHeader + m_i * kMantEntry;
                put_name(m, t.name);
                m[256] = t.dtype;
                m[257] = (uint8_t)w.spe;
                std::memset(m + 258, 0, 6);
                put<uint64_t>(m + 264, t.n_elem);
                put<uint64_t>(m + 272, c->descs[i].sidecar_off);
                put<uint64_t>(m + 280, t.n_elem * w.spe);
                ++m_i;
            }
            if (w.owns) {
                uint8_t* d = dc + kFileHeader + (size_t)w.table * kDictEntry;
                put_name(d, t.name);
                std::memcpy(d + 256, h_freq + (size_t)w.table * 256, 1024);
                std::memcpy(d + 1280, h_cum + (size_t)w.table * 257, 1028);
            }
        }
        CHK_CUDA(cudaEventRecord(c->ev[6], s));
        sync_stream(c, s);
        c->timing["d2h_ms"] = ms_between(c->ev[5], c->ev[6]);
        c->have_images = true;
    }
    c->timing["compress_total_ms"] = wall_ms(t_total);
}

static void write_file(const std::string& path, const void* p, size_t n) {
    std::FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) throw Error{CHK_ERR_IO, "cannot open for write: " + path};
    const size_t w = n ? std::fwrite(p, 1, n, f) : 0;
    const int rc = std::fclose(f);
    if (w != n || rc != 0) throw Error{CHK_ERR_IO, "short write: " + path};
}

static void rank_paths(const Context* c, const std::string& dir, std::string out[3]) {
    const std::string tag = "rank_" + std::to_string(c->rank < 0 ? 0 : c->rank);
    out[0] = dir + "/" + tag + "_states.ansc";
    out[1] = dir + "/mantissa/" + tag + "_mantissa.mant";
    out[2] = dir + "/tables/" + tag + "_tables.dict";
}

static void compress_and_save(Context* c, const std::string& dir) {
    namespace fs = std::filesystem;
    std::error_code ec;
    fs::create_directories(dir, ec);
    fs::create_directories(dir + "/mantissa", ec);
    fs::create_directories(dir + "/tables", ec);
    if (ec) throw Error{CHK_ERR_IO, "cannot create output directories under " + dir};
    if (c->tensors.empty()) return;  // nothing registered: directories only (src/ANSCompressor.cpp:1026-1029)
    compress(c, true);
    if (c->undecodable_tables && !c->allow_undecodable)
        throw Error{CHK_ERR_UNDECODABLE,
                    std::to_string(c->undecodable_tables) + " of " + std::to_string(c->n_tables) +
                        " tables do not sum to 4096 (the reference's single take-back pass on a shared full-alphabet "
                        "table): the files could not be restored and were not written.  Set \"repair_tables\" for decodable "
                        "shared tables, \"allow_undecodable\" for the reference's bytes, or compress without clusters."};
    const auto t0 = std::chrono::steady_clock::now();
    std::string paths[3];
    rank_paths(c, dir, paths);
    for (int k = 0; k < 3; ++k) write_file(paths[k], image_ptr(c, k), image_size(c, k));
    c->timing["io_ms"] = wall_ms(t0);
}

// ------------------------------------------------------------------ restore
static void run_decode(Context* c, size_t W, const uint8_t* d_payload, const uint8_t* d_sidecar,
                       const uint32_t* d_freq, const uint32_t* d_cum, const LaneHeader* d_hdrs,
                       const std::vector<size_t>& tensor_of) {
    cudaStream_t s = c->stream;
    dev_ensure(c, c->d_status, W * 4 + 256);
    pin_ensure(c->h_status, W * 4 + 256);
    control_zero(c, c->d_status.p, W * 4, s);
    // Two launches at most.  With option "decode_zero_skip", floating-point tensors whose table gives symbol 0
    // half of the slots (all of them, as a rule) go to the kernel with the short table, of which more teams fit an
    // SM; integer tensors -- four chains per thread, larger rings -- and whatever does not qualify go to the
    // full-table kernel.  Off by default: on a B200 the two extra instructions per symbol cost more than the
    // added teams bring (9.8 ms against 9.6 ms for the 14 GB benchmark shard).
    const TensorDesc* hd = static_cast<const TensorDesc*>(c->h_descs.p);
    std::vector<uint32_t> order(W);
    for (size_t i = 0; i < W; ++i) order[i] = (uint32_t)i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return hd[a].n_bytes > hd[b].n_bytes; });
    auto short_table = [&](uint32_t i) {
        return c->decode_zero_skip && hd[i].spe * 2 == hd[i].es && (hd[i].flags & kFlagZeroSkip) && !(hd[i].flags & kFlagRaw);
    };
    const size_t n_short = (size_t)(std::stable_partition(order.begin(), order.end(), short_table) - order.begin());
    bool any_int = false;
    for (size_t k = n_short; k < W && !any_int; ++k) any_int = hd[order[k]].spe * 2 != hd[order[k]].es;
    pin_ensure(c->h_order, W * 4);
    std::memcpy(c->h_order.p, order.data(), W * 4);
    dev_ensure(c, c->d_order, W * 4);
    dev_ensure(c, c->d_ticket, 256);
    control_copy(c, c->d_order.p, c->h_order.p, W * 4, s);
    control_zero(c, c->d_ticket.p, 256, s);
    CHK_CUDA(cudaEventRecord(c->ev[1], s));
    auto launch = [&](auto kernel, uint32_t smem, size_t first, size_t n, uint32_t ticket_word) {
        if (!n) return;
        const uint32_t grid = persistent_grid(c, reinterpret_cast<const void*>(kernel), smem, n, c->decode_teams_per_sm);
        kernel<<<grid, kTeam, smem, s>>>(static_cast<const TensorDesc*>(c->d_descs.p), d_freq, d_cum, d_hdrs, d_payload,
                                         d_sidecar, static_cast<const uint32_t*>(c->d_order.p) + first,
                                         static_cast<uint32_t*>(c->d_ticket.p) + ticket_word, (uint32_t)n,
                                         c->verify_zero_lanes ? 1u : 0u, static_cast<uint32_t*>(c->d_status.p));
        CHK_CUDA(cudaGetLastError());
        c->launches++;
    };
    launch(rans_decode_kernel<false, true>, kDecSmemBytes[0][1], 0, n_short, 0);
    if (any_int)
        launch(rans_decode_kernel<true, false>, kDecSmemBytes[1][0], n_short, W - n_short, 8);
    else
        launch(rans_decode_kernel<false, false>, kDecSmemBytes[0][0], n_short, W - n_short, 8);
    CHK_CUDA(cudaEventRecord(c->ev[2], s));
    control_copy(c, c->h_status.p, c->d_status.p, W * 4, s);
    CHK_CUDA(cudaEventRecord(c->ev[4], s));
    sync_stream(c, s);
    c->timing["decode_ms"] = ms_between(c->ev[1], c->ev[2]);
    c->timing["decode_tail_ms"] = ms_between(c->ev[2], c->ev[4]);
    const uint32_t* st = static_cast<const uint32_t*>(c->h_status.p);
    for (size_t i = 0; i < W; ++i)
        if (st[i])
            throw Error{CHK_ERR_DECODE, "tensor '" + c->tensors[tensor_of[i]].name + "' failed its stream check (" +
                                            ((st[i] & kErrEndState) ? "end state " : "") +
                                            ((st[i] & kErrEndPointer) ? "stream length" : "") + ")"};
    c->restored = W;
}

static void decompress_resident(Context* c, void* const* dst) {
    if (c->format_version == 3) return v3_decompress_resident(c, dst);
    const auto t_total = std::chrono::steady_clock::now();
    CHK_CUDA(cudaSetDevice(c->device));
    if (!c->have_resident) throw Error{CHK_ERR_INVALID, "no device-resident compressed state: call chk_compress first"};
    c->restored = 0;
    std::vector<TensorDesc> run;
    std::vector<size_t> src_index;
    std::vector<size_t> tensor_of;
    // which tables leave room for the short decode table: the frequency of symbol 0 of each (4 bytes per table)
    std::vector<uint32_t> f0;
    if (c->decode_zero_skip && c->n_tables) {
        f0.resize(c->n_tables);
        CHK_CUDA(cudaMemcpy2DAsync(f0.data(), 4, c->d_freq.p, 1024, 4, c->n_tables, cudaMemcpyDeviceToHost, c->stream));
        sync_stream(c, c->stream);
    }
    for (size_t i = 0; i < c->work.size(); ++i) {
        const WorkItem& w = c->work[i];
        void* target = dst ? dst[w.idx] : c->tensors[w.idx].ptr;
        if (!target) continue;
        TensorDesc d = c->descs[i];
        if (!(d.flags & kFlagRaw) && c->table_sums[w.table] != kM)
            throw Error{CHK_ERR_FORMAT, "table of '" + c->tensors[w.idx].name + "' sums to " +
                                            std::to_string(c->table_sums[w.table]) +
                                            ", not 4096: the stream cannot be decoded"};
        d.dst = static_cast<uint8_t*>(target);
        d.src = nullptr;
        d.flags &= ~(kFlagAligned | kFlagZeroSkip);
        if (!f0.empty() && zero_skip_fits(f0[w.table])) d.flags |= kFlagZeroSkip;
        if ((reinterpret_cast<uintptr_t>(target) & 15) == 0 && (d.sidecar_off & 15) == 0) d.flags |= kFlagAligned;
        run.push_back(d);
        src_index.push_back(i);
        tensor_of.push_back(w.idx);
    }
    const size_t W = run.size();
    if (W == 0) return;
    // lane headers of the selected tensors must be contiguous per descriptor index
    const bool all = W == c->work.size();
    if (!all) throw Error{CHK_ERR_INVALID, "chk_decompress_resident: partial restore is not supported; pass all targets"};
    pin_ensure(c->h_descs, W * sizeof(TensorDesc));
    std::memcpy(c->h_descs.p, run.data(), W * sizeof(TensorDesc));
    dev_ensure(c, c->d_descs, W * sizeof(TensorDesc));
    control_copy(c, c->d_descs.p, c->h_descs.p, W * sizeof(TensorDesc), c->stream);
    run_decode(c, W, static_cast<const uint8_t*>(c->d_payload.p), static_cast<const uint8_t*>(c->d_sidecar.p),
               static_cast<const uint32_t*>(c->d_freq.p), static_cast<const uint32_t*>(c->d_cum.p),
               static_cast<const LaneHeader*>(c->d_hdrs.p), tensor_of);
    c->timing["decompress_total_ms"] = wall_ms(t_total);
}

static void decompress_images(Context* c, const uint8_t* st, size_t st_n, const uint8_t* mt, size_t mt_n,
                              const uint8_t* dc, size_t dc_n) {
    if (c->format_version == 3) return v3_decompress_images(c, st, st_n, mt, mt_n, dc, dc_n);
    c->last_run.clear();
    c->last_run_tensor.clear();
    const auto t_total = std::chrono::steady_clock::now();
    CHK_CUDA(cudaSetDevice(c->device));
    c->restored = 0;
    c->have_resident = false;  // device buffers are about to be reused
    if (st_n < kFileHeader || get<uint32_t>(st) != kStatesMagic || get<uint32_t>(st + 4) != c->file_version[0])
        throw Error{CHK_ERR_FORMAT, "states file: bad magic or version"};
    if (mt_n < kFileHeader || get<uint32_t>(mt) != kMantMagic || get<uint32_t>(mt + 4) != c->file_version[1])
        throw Error{CHK_ERR_FORMAT, "mantissa file: bad magic or version"};
    if (dc_n < kFileHeader || get<uint32_t>(dc) != kDictMagic || get<uint32_t>(dc + 4) != c->file_version[2])
        throw Error{CHK_ERR_FORMAT, "tables file: bad magic or version"};
    const size_t n_st = get<uint32_t>(st + 12), n_mt = get<uint32_t>(mt + 12), n_dc = get<uint32_t>(dc + 12);
    const size_t st_data = kFileHeader + n_st * kStatesEntry;
    const size_t mt_data = kFileHeader + n_mt * kMantEntry;
    if (st_n < st_data) throw Error{CHK_ERR_FORMAT, "states file: truncated index"};
    if (mt_n < mt_data) throw Error{CHK_ERR_FORMAT, "mantissa file: truncated index"};
    if (dc_n < kFileHeader + n_dc * kDictEntry) throw Error{CHK_ERR_FORMAT, "tables file: truncated"};
    const size_t payload_total = st_n - st_data, sidecar_total = mt_n - mt_data;

    std::unordered_map<std::string, size_t> reg, side, tab;
    for (size_t i = 0; i < c->tensors.size(); ++i) reg.emplace(c->tensors[i].name, i);
    for (size_t i = 0; i < n_mt; ++i) side.emplace(get_name(mt + kFileHeader + i * kMantEntry), i);
    for (size_t i = 0; i < n_dc; ++i) tab.emplace(get_name(dc + kFileHeader + i * kDictEntry), i);

    std::vector<TensorDesc> run;
    std::vector<size_t> entry_of;
    std::vector<size_t> tensor_of;
    for (size_t i = 0; i < n_st; ++i) {
        const uint8_t* e = st + kFileHeader + i * kStatesEntry;
        const std::string name = get_name(e);
        auto r = reg.find(name);
        if (r == reg.end()) continue;
        const Tensor& t = c->tensors[r->second];
        if (!t.ptr) continue;
        const uint8_t dtype = e[256];
        const bool is_raw = e[257] != 0, owns = e[258] != 0;
        const uint64_t bytes = get<uint64_t>(e + 264), n_elem = get<uint64_t>(e + 272);
        const uint64_t off = get<uint64_t>(e + 280), size = get<uint64_t>(e + 288);
        const uint32_t es = elem_size(dtype), spe = sidecar_per_elem(dtype);
        if (es == 0 || n_elem > UINT64_MAX / es || bytes != n_elem * es || bytes >= (1ull << 32))
            throw Error{CHK_ERR_FORMAT, "entry '" + name + "': inconsistent sizes"};
        if (t.dtype != dtype || t.n_elem != n_elem)
            throw Error{CHK_ERR_INVALID, "tensor '" + name + "': registered dtype/size differs from the checkpoint"};
        if (size > payload_total || off > payload_total - size)
            throw Error{CHK_ERR_FORMAT, "entry '" + name + "': payload out of range"};
        if (is_raw && size != bytes) throw Error{CHK_ERR_FORMAT, "entry '" + name + "': raw payload size mismatch"};
        TensorDesc d{};
        d.dst = static_cast<uint8_t*>(t.ptr);
        d.n_bytes = bytes;
        d.es = es;
        d.spe = spe;
        d.payload_off = off;
        d.flags = is_raw ? kFlagRaw : 0u;
        if (!is_raw) {
            const std::string key = owns ? name : get_name(e + 296);
            auto tb = tab.find(key);
            if (tb == tab.end()) throw Error{CHK_ERR_FORMAT, "entry '" + name + "': table '" + key + "' not in tables file"};
            d.table_idx = (uint32_t)tb->second;
            const uint8_t* te = dc + kFileHeader + tb->second * kDictEntry;
            if (zero_skip_fits(get<uint32_t>(te + 256))) d.flags |= kFlagZeroSkip;  // frequency of symbol 0
            const uint32_t sum = get<uint32_t>(te + 1280 + 256 * 4);
            if (sum != kM)
                throw Error{CHK_ERR_FORMAT, "table '" + key + "' sums to " + std::to_string(sum) +
                                                ", not 4096: the stream cannot be decoded"};
            // lane ranges must lie inside this tensor's payload
            const LaneHeader* lh = reinterpret_cast<const LaneHeader*>(e + 552);
            for (int l = 0; l < 256; ++l) {
                LaneHeader h;
                std::memcpy(&h, lh + l, sizeof(h));
                if ((uint64_t)h.buf_offset + h.byte_count > size)
                    throw Error{CHK_ERR_FORMAT, "entry '" + name + "': lane " + std::to_string(l) + " out of range"};
            }
        }
        if (spe) {
            auto sd = side.find(name);
            if (sd == side.end()) throw Error{CHK_ERR_FORMAT, "entry '" + name + "': no sidecar in mantissa file"};
            const uint8_t* m = mt + kFileHeader + sd->second * kMantEntry;
            const uint64_t moff = get<uint64_t>(m + 272), msz = get<uint64_t>(m + 280);
            if (msz != n_elem * spe || msz > sidecar_total || moff > sidecar_total - msz)
                throw Error{CHK_ERR_FORMAT, "entry '" + name + "': sidecar out of range"};
            d.sidecar_off = moff;
        }
        if ((reinterpret_cast<uintptr_t>(d.dst) & 15) == 0 && (d.sidecar_off & 15) == 0) d.flags |= kFlagAligned;
        run.push_back(d);
        entry_of.push_back(i);
        tensor_of.push_back(r->second);
    }
    const size_t W = run.size();
    if (W == 0) return;

    cudaStream_t s = c->stream;
    dev_ensure(c, c->d_descs, W * sizeof(TensorDesc));
    dev_ensure(c, c->d_payload, payload_total + 64);
    dev_ensure(c, c->d_sidecar, sidecar_total + 64);
    dev_ensure(c, c->d_hdrs, W * 4096);
    dev_ensure(c, c->d_freq, n_dc * 256 * 4 + 4);
    dev_ensure(c, c->d_cum, n_dc * 257 * 4 + 4);
    pin_ensure(c->h_descs, W * sizeof(TensorDesc));
    std::memcpy(c->h_descs.p, run.data(), W * sizeof(TensorDesc));

    c->timing["parse_ms"] = wall_ms(t_total);
    CHK_CUDA(cudaEventRecord(c->ev[0], s));
    control_copy(c, c->d_descs.p, c->h_descs.p, W * sizeof(TensorDesc), s);
    // index data first, so it does not queue behind this call's own bulk copies
    // lane headers: one strided copy per run of consecutive entries
    for (size_t k = 0; k < W;) {
        size_t j = k + 1;
        while (j < W && entry_of[j] == entry_of[j - 1] + 1) ++j;
        CHK_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(c->d_hdrs.p) + k * 4096, 4096,
                                   st + kFileHeader + entry_of[k] * kStatesEntry + 552, kStatesEntry, 4096, j - k,
                                   cudaMemcpyHostToDevice, s));
        k = j;
    }
    if (n_dc) {
        CHK_CUDA(cudaMemcpy2DAsync(c->d_freq.p, 1024, dc + kFileHeader + 256, kDictEntry, 1024, n_dc,
                                   cudaMemcpyHostToDevice, s));
        CHK_CUDA(cudaMemcpy2DAsync(c->d_cum.p, 1028, dc + kFileHeader + 1280, kDictEntry, 1028, n_dc,
                                   cudaMemcpyHostToDevice, s));
    }
    if (payload_total) CHK_CUDA(cudaMemcpyAsync(c->d_payload.p, st + st_data, payload_total, cudaMemcpyHostToDevice, s));
    if (sidecar_total) CHK_CUDA(cudaMemcpyAsync(c->d_sidecar.p, mt + mt_data, sidecar_total, cudaMemcpyHostToDevice, s));
    CHK_CUDA(cudaEventRecord(c->ev[3], s));
    if (c->skip_decode) {
        c->last_run = run;
        c->last_run_tensor = tensor_of;
        return;
    }
    run_decode(c, W, static_cast<const uint8_t*>(c->d_payload.p), static_cast<const uint8_t*>(c->d_sidecar.p),
               static_cast<const uint32_t*>(c->d_freq.p), static_cast<const uint32_t*>(c->d_cum.p),
               static_cast<const LaneHeader*>(c->d_hdrs.p), tensor_of);
    c->timing["h2d_ms"] = ms_between(c->ev[0], c->ev[3]);
    c->timing["decode_wait_ms"] = ms_between(c->ev[3], c->ev[1]);
    c->timing["decompress_total_ms"] = wall_ms(t_total);
}

static void read_file(const std::string& path, PinBuf& out) {
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) throw Error{CHK_ERR_IO, "cannot open: " + path};
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (n < 0) {
        std::fclose(f);
        throw Error{CHK_ERR_IO, "cannot size: " + path};
    }
    pin_ensure(out, (size_t)n);
    const size_t r = n ? std::fread(out.p, 1, (size_t)n, f) : 0;
    std::fclose(f);
    if (r != (size_t)n) throw Error{CHK_ERR_IO, "short read: " + path};
}

static void load_and_decompress(Context* c, const std::string& dir) {
    const auto t0 = std::chrono::steady_clock::now();
    std::string paths[3];
    rank_paths(c, dir, paths);
    for (int k = 0; k < 3; ++k) read_file(paths[k], c->img[k]);
    c->have_images = false;
    c->timing["io_ms"] = wall_ms(t0);
    decompress_images(c, static_cast<const uint8_t*>(c->img[0].p), c->img[0].size,
                      static_cast<const uint8_t*>(c->img[1].p), c->img[1].size,
                      static_cast<const uint8_t*>(c->img[2].p), c->img[2].size);
}

// ------------------------------------------------------------------ analysis
static void analyze(Context* c) {
    CHK_CUDA(cudaSetDevice(c->device));
    const size_t N = c->tensors.size();
    c->stats.assign(N, StatsOut{});
    if (N == 0) return;
    cudaStream_t s = c->stream;
    std::vector<StatsDesc> d(N);
    for (size_t i = 0; i < N; ++i) {
        const Tensor& t = c->tensors[i];
        d[i] = StatsDesc{elem_size(t.dtype) ? t.ptr : nullptr, t.n_elem, t.dtype, c->histogram_bins};
    }
    dev_ensure(c, c->d_stats_desc, N * sizeof(StatsDesc));
    dev_ensure(c, c->d_stats_out, N * sizeof(StatsOut));
    pin_ensure(c->h_stats, N * sizeof(StatsOut));
    CHK_CUDA(cudaMemcpyAsync(c->d_stats_desc.p, d.data(), N * sizeof(StatsDesc), cudaMemcpyHostToDevice, s));
    CHK_CUDA(cudaMemsetAsync(c->d_stats_out.p, 0, N * sizeof(StatsOut), s));
    CHK_CUDA(cudaEventRecord(c->ev[0], s));
    if (!c->fast_stats) {
        const size_t cap = (size_t)(c->sm_count > 0 ? c->sm_count : 1) * 64;
        const uint32_t grid = (uint32_t)(N < cap ? N : cap);
        tensor_stats_kernel<<<grid, 256, 0, s>>>(static_cast<const StatsDesc*>(c->d_stats_desc.p),
                                                 static_cast<StatsOut*>(c->d_stats_out.p), (uint32_t)N);
        CHK_CUDA(cudaGetLastError());
        c->launches++;
    } else {
        // the order-free variant: tiles of all tensors over the whole device, two passes
        pin_ensure(c->h_tiles, (N + 1) * 4);
        uint32_t* tile_start = static_cast<uint32_t*>(c->h_tiles.p);
        unsigned long long tiles = 0;
        for (size_t i = 0; i < N; ++i) {
            tile_start[i] = (uint32_t)tiles;
            if (d[i].ptr && d[i].n) tiles += (d[i].n * elem_size(c->tensors[i].dtype) + kStatsTileBytes - 1) / kStatsTileBytes;
            if (tiles > 0xFFFFFFFFull) throw Error{CHK_ERR_CAPACITY, "too many statistics tiles in one batch"};
        }
        tile_start[N] = (uint32_t)tiles;
        if (tiles) {
            dev_ensure(c, c->d_tiles, (N + 1) * 4);
            dev_ensure(c, c->d_stats_part, (size_t)tiles * (sizeof(StatsPart1) + sizeof(StatsPart2)));
            dev_ensure(c, c->d_stats_mid, N * sizeof(StatsMid));
            control_copy(c, c->d_tiles.p, c->h_tiles.p, (N + 1) * 4, s);
            auto* p1 = static_cast<StatsPart1*>(c->d_stats_part.p);
            auto* p2 = reinterpret_cast<StatsPart2*>(p1 + tiles);
            const auto* dd = static_cast<const StatsDesc*>(c->d_stats_desc.p);
            const auto* ts = static_cast<const uint32_t*>(c->d_tiles.p);
            auto* mids = static_cast<StatsMid*>(c->d_stats_mid.p);
            auto* outs = static_cast<StatsOut*>(c->d_stats_out.p);
            const unsigned long long cap = (unsigned long long)(c->sm_count > 0 ? c->sm_count : 1) * 8;
            const uint32_t grid = (uint32_t)(tiles < cap ? tiles : cap);
            stats_fast_pass1_kernel<<<grid, 256, 0, s>>>(dd, ts, (uint32_t)N, (uint32_t)tiles, p1);
            stats_fast_reduce1_kernel<<<(uint32_t)N, 256, 0, s>>>(dd, ts, p1, mids, outs, (uint32_t)N);
            stats_fast_pass2_kernel<<<grid, 256, 0, s>>>(dd, ts, (uint32_t)N, (uint32_t)tiles, mids, p2, outs);
            stats_fast_reduce2_kernel<<<(uint32_t)N, 256, 0, s>>>(dd, ts, p2, outs, (uint32_t)N);
            CHK_CUDA(cudaGetLastError());
            c->launches += 4;
        }
    }
    CHK_CUDA(cudaEventRecord(c->ev[1], s));
    CHK_CUDA(cudaMemcpyAsync(c->h_stats.p, c->d_stats_out.p, N * sizeof(StatsOut), cudaMemcpyDeviceToHost, s));
    sync_stream(c, s);
    c->timing["analyze_stats_ms"] = ms_between(c->ev[0], c->ev[1]);
    std::memcpy(c->stats.data(), c->h_stats.p, N * sizeof(StatsOut));

    const auto t0 = std::chrono::steady_clock::now();
    std::vector<std::string> names(N);
    std::vector<float> fps(N * 5);
    for (size_t i = 0; i < N; ++i) {
        names[i] = c->tensors[i].name;
        std::memcpy(&fps[i * 5], c->stats[i].fingerprint, 20);
    }
    c->clusters = build_clusters(names, fps);
    c->have_clusters = true;
    c->timing["analyze_cluster_ms"] = wall_ms(t0);
}

// ------------------------------------------------------------------ vocabulary sketches (offline study)
// One HyperLogLog sketch per registered tensor, all in one pass (study_kernels.cuh).
static void hll_sketch_all(Context* c) {
    CHK_CUDA(cudaSetDevice(c->device));
    const size_t N = c->tensors.size();
    c->hll.assign(N * (size_t)kHllRegs, 0);
    if (N == 0) return;
    cudaStream_t s = c->stream;
    const uint32_t smem = kHllRegs * 4;
    CHK_CUDA(cudaFuncSetAttribute(hll_sketch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned long long cap = (unsigned long long)(c->sm_count > 0 ? c->sm_count : 1) * 3;
    double ms = 0.0;
    // batches of at most kBatch tensors: the registers of a batch take 80 KiB per tensor on the device
    constexpr size_t kBatch = 8192;
    for (size_t first = 0; first < N; first += kBatch) {
        const size_t n = std::min(kBatch, N - first);
        std::vector<StatsDesc> d(n);
        pin_ensure(c->h_tiles, (n + 1) * 4);
        uint32_t* tile_start = static_cast<uint32_t*>(c->h_tiles.p);
        unsigned long long tiles = 0;
        for (size_t i = 0; i < n; ++i) {
            const Tensor& t = c->tensors[first + i];
            const uint32_t es = elem_size(t.dtype);
            d[i] = StatsDesc{es ? t.ptr : nullptr, t.n_elem, t.dtype, 0};
            tile_start[i] = (uint32_t)tiles;
            if (d[i].ptr && d[i].n) tiles += (d[i].n * es + kHllTileBytes - 1) / kHllTileBytes;
            if (tiles > 0xFFFFFFFFull) throw Error{CHK_ERR_CAPACITY, "too many tiles in one batch"};
        }
        tile_start[n] = (uint32_t)tiles;
        if (!tiles) continue;
        const unsigned long long regs = (unsigned long long)n * kHllRegs;
        dev_ensure(c, c->d_stats_desc, n * sizeof(StatsDesc));
        dev_ensure(c, c->d_tiles, (n + 1) * 4);
        dev_ensure(c, c->d_hll32, regs * 4);
        dev_ensure(c, c->d_hll8, regs);
        CHK_CUDA(cudaMemcpyAsync(c->d_stats_desc.p, d.data(), n * sizeof(StatsDesc), cudaMemcpyHostToDevice, s));
        control_copy(c, c->d_tiles.p, c->h_tiles.p, (n + 1) * 4, s);
        CHK_CUDA(cudaMemsetAsync(c->d_hll32.p, 0, regs * 4, s));
        CHK_CUDA(cudaEventRecord(c->ev[0], s));
        hll_sketch_kernel<<<(uint32_t)(tiles < cap ? tiles : cap), 256, smem, s>>>(
            static_cast<const StatsDesc*>(c->d_stats_desc.p), static_cast<const uint32_t*>(c->d_tiles.p), (uint32_t)n,
            (uint32_t)tiles, static_cast<uint32_t*>(c->d_hll32.p));
        hll_pack_kernel<<<(uint32_t)cap, 256, 0, s>>>(static_cast<const uint32_t*>(c->d_hll32.p),
                                                      static_cast<uint8_t*>(c->d_hll8.p), regs);
        CHK_CUDA(cudaGetLastError());
        c->launches += 2;
        CHK_CUDA(cudaEventRecord(c->ev[1], s));
        CHK_CUDA(cudaMemcpyAsync(c->hll.data() + first * kHllRegs, c->d_hll8.p, regs, cudaMemcpyDeviceToHost, s));
        sync_stream(c, s);  // the descriptors on the host stack and the pinned tile table are reused by the next batch
        ms += ms_between(c->ev[0], c->ev[1]);
    }
    c->timing["hll_sketch_ms"] = ms;
}

// Bytes of the group's tensors coded under one shared 32-bit model, and the size of the model's vocabulary
// (cluster_cost_worker, scripts/llama-3-8b/experiment_2_1.py:273-330; a group of one tensor gives the own-model
// figures of tensor_stats_worker, :129-184).
static void shared_model_cost(Context* c, const uint64_t* index, size_t n, double* stream_bytes, uint64_t* vocab) {
    CHK_CUDA(cudaSetDevice(c->device));
    *stream_bytes = 0.0;
    *vocab = 0;
    cudaStream_t s = c->stream;
    std::vector<StatsDesc> d;
    std::vector<uint32_t> tiles_before;
    unsigned long long tiles = 0, symbols = 0;
    for (size_t k = 0; k < n; ++k) {
        if (index[k] >= c->tensors.size()) throw Error{CHK_ERR_INVALID, "tensor index out of range"};
        const Tensor& t = c->tensors[index[k]];
        const uint32_t es = elem_size(t.dtype);
        if (!t.ptr || !t.n_elem || !es) continue;
        d.push_back(StatsDesc{t.ptr, t.n_elem, t.dtype, 0});
        tiles_before.push_back((uint32_t)tiles);
        tiles += (t.n_elem * es + kHllTileBytes - 1) / kHllTileBytes;
        symbols += t.n_elem;
        if (tiles > 0xFFFFFFFFull) throw Error{CHK_ERR_CAPACITY, "too many tiles in one group"};
    }
    if (!symbols) return;
    tiles_before.push_back((uint32_t)tiles);
    // a table with at least twice as many slots as there are symbols (all of them may be distinct)
    unsigned long long capacity = 1024;
    while (capacity < 2 * symbols) capacity <<= 1;
    if (capacity > (1ull << 31)) throw Error{CHK_ERR_CAPACITY, "group too large for the symbol table (2^30 symbols at most)"};
    const size_t N = d.size();
    const uint32_t blocks = (uint32_t)(c->sm_count > 0 ? c->sm_count : 1) * 8;
    dev_ensure(c, c->d_stats_desc, N * sizeof(StatsDesc));
    dev_ensure(c, c->d_tiles, (N + 1) * 4);
    dev_ensure(c, c->d_symkeys, capacity * 8);
    dev_ensure(c, c->d_symcounts, capacity * 4);
    dev_ensure(c, c->d_stats_part, 64 + (size_t)blocks * 16);
    CHK_CUDA(cudaMemcpyAsync(c->d_stats_desc.p, d.data(), N * sizeof(StatsDesc), cudaMemcpyHostToDevice, s));
    CHK_CUDA(cudaMemcpyAsync(c->d_tiles.p, tiles_before.data(), (N + 1) * 4, cudaMemcpyHostToDevice, s));
    CHK_CUDA(cudaMemsetAsync(c->d_symkeys.p, 0, capacity * 8, s));
    CHK_CUDA(cudaMemsetAsync(c->d_symcounts.p, 0, capacity * 4, s));
    CHK_CUDA(cudaMemsetAsync(c->d_stats_part.p, 0, 64, s));
    auto* keys = static_cast<unsigned long long*>(c->d_symkeys.p);
    auto* counts = static_cast<uint32_t*>(c->d_symcounts.p);
    auto* head = static_cast<unsigned long long*>(c->d_stats_part.p);  // [0] vocabulary, [1] best, [2] overflow
    auto* partial = reinterpret_cast<double*>(head + 8);
    CHK_CUDA(cudaEventRecord(c->ev[0], s));
    symbol_count_kernel<<<(uint32_t)(tiles < blocks ? tiles : blocks), 256, 0, s>>>(
        static_cast<const StatsDesc*>(c->d_stats_desc.p), static_cast<const uint32_t*>(c->d_tiles.p), (uint32_t)N,
        (uint32_t)tiles, keys, counts, (uint32_t)(capacity - 1), reinterpret_cast<uint32_t*>(head + 2));
    model_scan_kernel<<<blocks, 256, 0, s>>>(keys, counts, (uint32_t)capacity, head);
    CHK_CUDA(cudaGetLastError());
    unsigned long long h[3] = {};
    CHK_CUDA(cudaMemcpyAsync(h, head, sizeof(h), cudaMemcpyDeviceToHost, s));
    sync_stream(c, s);
    if (h[2]) throw Error{CHK_ERR_CAPACITY, "internal: symbol table overflow"};
    const unsigned long long n_vocab = h[0];
    const double c_max = (double)(h[1] >> 32);
    const unsigned long long max_key = kSymUsed | (0xFFFFFFFFull - (h[1] & 0xFFFFFFFFull));
    // _build_model (:52-75): scale = 2^p > 2 * vocabulary, p >= 14; norm = max(floor(count * scale / total), 1);
    // the drift goes onto the most frequent symbol
    int p = 14;
    {
        int need = 1;
        while ((1ull << need) < (n_vocab > 2 ? n_vocab : 2)) ++need;  // ceil(log2(max(n_vocab, 2)))
        if (need + 1 > p) p = need + 1;
    }
    const double scale = std::ldexp(1.0, p);
    const double factor = scale / (double)symbols;
    model_cost_kernel<<<blocks, 256, 0, s>>>(keys, counts, (uint32_t)capacity, factor, scale, max_key, partial);
    CHK_CUDA(cudaGetLastError());
    CHK_CUDA(cudaEventRecord(c->ev[1], s));
    std::vector<double> part((size_t)blocks * 2);
    CHK_CUDA(cudaMemcpyAsync(part.data(), partial, part.size() * 8, cudaMemcpyDeviceToHost, s));
    sync_stream(c, s);
    c->launches += 3;
    double norm_sum = 0.0, bits = 0.0;
    for (uint32_t b = 0; b < blocks; ++b) {
        norm_sum += part[2 * b];
        bits += part[2 * b + 1];
    }
    double norm_max = std::floor(c_max * factor);
    if (norm_max < 1.0) norm_max = 1.0;
    norm_max += scale - (norm_sum + norm_max);
    if (norm_max < 1.0) norm_max = 1.0;
    bits += c_max * std::log2(scale / norm_max);
    *stream_bytes = bits / 8.0;
    *vocab = n_vocab;
    c->timing["model_cost_ms"] = ms_between(c->ev[0], c->ev[1]);
}

// Cardinality estimate of one sketch: alpha m^2 / sum 2^-register with the small- and large-range corrections
// (scripts/llama-3-8b/experiment_2.py:71-82).  The sum is formed over the 19 possible register values, which is
// exact in double, as is numpy's pairwise sum of the same powers of two.
static double hll_count(const uint8_t* regs) {
    unsigned long long by_value[64] = {};
    for (uint32_t i = 0; i < kHllRegs; ++i) by_value[regs[i] & 63]++;
    double sum = 0.0;
    for (int k = 0; k < 64; ++k) sum += (double)by_value[k] * std::ldexp(1.0, -k);
    const double m = (double)kHllRegs;
    const double alpha = 0.7213 / (1.0 + 1.079 / m);
    double raw = alpha * m * m * (1.0 / sum);
    if (raw <= 2.5 * m) {
        if (by_value[0] > 0) raw = m * std::log(m / (double)by_value[0]);
    } else if (raw > (1.0 / 30.0) * 4294967296.0) {
        raw = -4294967296.0 * std::log(1.0 - raw / 4294967296.0);
    }
    return raw;
}

}  // namespace chk

// ====================================================================== C ABI
using namespace chk;
struct chk_context : chk::Context {};

#define CHK_API_BEGIN try {
#define CHK_API_END                                   \
    }                                                 \
    catch (const chk::Error& e) {                     \
        chk::g_last_error = e.msg;                    \
        return e.code;                                \
    }                                                 \
    catch (const std::exception& e) {                 \
        chk::g_last_error = e.what();                 \
        return CHK_ERR_INVALID;                       \
    }                                                 \
    return CHK_OK;

#define CHK_REQUIRE(cond, msg) \
    if (!(cond)) throw chk::Error { CHK_ERR_INVALID, msg }

extern "C" {

const char* chk_last_error(void) { return chk::g_last_error.c_str(); }

int chk_context_create(int device, int rank, int local_rank, chk_context** out) {
    return chk_context_create_ex(device, rank, local_rank, 0, out);
}

int chk_context_create_ex(int device, int rank, int local_rank, uint64_t workspace_bytes, chk_context** out) {
    CHK_API_BEGIN
    CHK_REQUIRE(out, "out is NULL");
    int n = 0;
    CHK_CUDA(cudaGetDeviceCount(&n));
    CHK_REQUIRE(device >= 0 && device < n, "no such CUDA device");
    CHK_CUDA(cudaSetDevice(device));
    auto* c = new chk_context();
    c->device = device;
    c->rank = rank;
    c->local_rank = local_rank;
    c->workspace_bytes = workspace_bytes;
    try {
        // the counting stream gets the highest priority: its blocks go first whenever an SM has room,
        // so the encode teams of earlier segments do not hold up the tables of later ones
        int prio_lo = 0, prio_hi = 0;
        CHK_CUDA(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));
        CHK_CUDA(cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, prio_hi));
        CHK_CUDA(cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking));
        CHK_CUDA(cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device));
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        CHK_CUDA(cudaMemPoolCreate(&c->pool, &props));
        uint64_t keep = UINT64_MAX;
        CHK_CUDA(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &keep));
        for (auto& e : c->ev) CHK_CUDA(cudaEventCreate(&e));
    } catch (...) {
        delete c;
        throw;
    }
    *out = c;
    CHK_API_END
}

// Every device buffer of the context back to its pool, and the pool's memory back to the device.
static void release_device_buffers(chk_context* c) {
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->side_stream) cudaStreamSynchronize(c->side_stream);
    DevBuf* bufs[] = {&c->d_descs, &c->d_tiles, &c->d_hist, &c->d_sidecar, &c->d_scratch, &c->d_hdrs,
                      &c->d_order, &c->d_ticket, &c->d_psize, &c->d_zslots, &c->d_zregions, &c->d_zslot_of, &c->d_jobs, &c->d_sums, &c->d_payload, &c->d_enc,
                      &c->d_freq, &c->d_cum, &c->d_status, &c->d_stats_desc, &c->d_stats_out, &c->d_stats_part, &c->d_stats_mid, &c->d_poff, &c->d_fileorder, &c->d_hll32, &c->d_hll8, &c->d_symkeys, &c->d_symcounts};
    for (DevBuf* b : bufs) {
        if (b->p) cudaFreeAsync(b->p, c->stream);
        b->p = nullptr;
        b->cap = 0;
    }
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->pool) cudaMemPoolTrimTo(c->pool, 0);
}

int chk_release_workspace(chk_context* c) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    CHK_CUDA(cudaSetDevice(c->device));
    v3_destroy(c);
    release_device_buffers(c);
    c->have_resident = false;  // the device-resident result lived in those buffers; host images stay
    CHK_API_END
}

int chk_context_destroy(chk_context* c) {
    CHK_API_BEGIN
    if (!c) return CHK_OK;
    cudaSetDevice(c->device);
    v3_destroy(c);
    release_device_buffers(c);
    PinBuf* pins[] = {&c->h_hdrs, &c->h_poff, &c->h_psize, &c->h_descs, &c->h_status, &c->h_jobs, &c->h_sums, &c->h_freq, &c->h_cum, &c->h_stats, &c->h_order, &c->h_tiles,
                      &c->img[0], &c->img[1], &c->img[2]};
    for (PinBuf* b : pins)
        if (b->p) cudaFreeHost(b->p);
    for (auto& e : c->ev)
        if (e) cudaEventDestroy(e);
    if (c->ev_block) cudaEventDestroy(c->ev_block);
    for (auto* v : {&c->ev_count, &c->ev_tab})
        for (auto& e : *v)
            if (e) cudaEventDestroy(e);
    if (c->pool) cudaMemPoolDestroy(c->pool);
    if (c->side_stream) cudaStreamDestroy(c->side_stream);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    CHK_API_END
}

int chk_reset(chk_context* c) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    c->tensors.clear();
    c->registry_epoch++;
    c->clusters = ClusterMap{};
    c->have_clusters = false;
    c->stats.clear();
    c->work.clear();
    c->n_tables = 0;
    c->table_sums.clear();
    c->undecodable_tables = 0;
    c->descs.clear();
    c->have_resident = c->have_images = false;
    c->summary = chk_summary{};
    c->restored = 0;
    CHK_API_END
}

int chk_set_histogram_bins(chk_context* c, uint32_t bins) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    c->histogram_bins = bins;
    CHK_API_END
}

int chk_register_tensor(chk_context* c, const char* name, const void* ptr, uint64_t n, uint8_t dtype, uint8_t cat) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && name, "context or name is NULL");
    c->tensors.push_back(Tensor{name, const_cast<void*>(ptr), n, dtype, cat});
    c->have_resident = false;
    c->registry_epoch++;
    CHK_API_END
}

int chk_tensor_count(chk_context* c, uint64_t* count) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && count, "NULL argument");
    *count = c->tensors.size();
    CHK_API_END
}

int chk_set_option(chk_context* c, const char* key, int64_t value) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && key, "NULL argument");
    const std::string k(key);
    if (k == "repair_tables")
        c->repair_tables = value != 0;
    else if (k == "verify_zero_lanes")
        c->verify_zero_lanes = value != 0;
    else if (k == "fast_stats")
        c->fast_stats = value != 0;
    else if (k == "v3_fused_decode")
        c->v3_fused_decode = value != 0;
    else if (k == "format_version") {
        if (value != 2 && value != 3) throw chk::Error{CHK_ERR_INVALID, "format_version must be 2 or 3"};
        if (c->format_version != (int)value) c->have_resident = c->have_images = false;
        c->format_version = (int)value;
    }
    else if (k == "allow_undecodable")
        c->allow_undecodable = value != 0;

    else if (k == "workspace_bytes") {
        if (value < 0) throw chk::Error{CHK_ERR_INVALID, "workspace_bytes must not be negative (0 = no bound)"};
        c->workspace_bytes = (uint64_t)value;
    }
    else if (k == "decode_zero_skip")
        c->decode_zero_skip = value != 0;
    else if (k == "segments") {
        if (value < 1 || value > 8) throw chk::Error{CHK_ERR_INVALID, "segments must be 1..8"};
        c->segments = (int)value;
    } else if (k == "encode_teams_per_sm") {
        if (value < 0 || value > 64) throw chk::Error{CHK_ERR_INVALID, "encode_teams_per_sm must be 0..64 (0 = as many as fit)"};
        c->encode_teams_per_sm = (int)value;
    } else if (k == "decode_teams_per_sm") {
        if (value < 0 || value > 64) throw chk::Error{CHK_ERR_INVALID, "decode_teams_per_sm must be 0..64 (0 = as many as fit)"};
        c->decode_teams_per_sm = (int)value;
    } else
        throw chk::Error{CHK_ERR_INVALID, "unknown option: " + k};
    CHK_API_END
}

int chk_analyze(chk_context* c) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    analyze(c);
    CHK_API_END
}

int chk_shared_model_cost(chk_context* c, const uint64_t* index, uint64_t n, double* stream_bytes, uint64_t* vocabulary) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && (index || n == 0) && stream_bytes && vocabulary, "NULL argument");
    shared_model_cost(c, index, (size_t)n, stream_bytes, vocabulary);
    CHK_API_END
}

int chk_hll_sketch_all(chk_context* c) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    hll_sketch_all(c);
    CHK_API_END
}

int chk_hll_get(chk_context* c, uint64_t index, uint8_t regs[16384]) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && regs, "NULL argument");
    CHK_REQUIRE((index + 1) * (uint64_t)kHllRegs <= c->hll.size(), "no sketch for this tensor: call chk_hll_sketch_all");
    std::memcpy(regs, c->hll.data() + index * kHllRegs, kHllRegs);
    CHK_API_END
}

int chk_hll_merge(uint8_t acc[16384], const uint8_t other[16384]) {
    CHK_API_BEGIN
    CHK_REQUIRE(acc && other, "NULL argument");
    for (uint32_t i = 0; i < kHllRegs; ++i) acc[i] = acc[i] > other[i] ? acc[i] : other[i];
    CHK_API_END
}

int chk_hll_count(const uint8_t regs[16384], double* estimate) {
    CHK_API_BEGIN
    CHK_REQUIRE(regs && estimate, "NULL argument");
    *estimate = hll_count(regs);
    CHK_API_END
}

// Bytes of per-tensor histograms against histograms shared inside the current clusters, as the study prices
// them: 8 bytes per distinct 32-bit symbol + 64 (scripts/llama-3-8b/experiment_2.py:104, 145, 440-470).
int chk_shared_vocabulary_report(chk_context* c, uint64_t* per_tensor_bytes, uint64_t* shared_bytes) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && per_tensor_bytes && shared_bytes, "NULL argument");
    const size_t N = c->tensors.size();
    CHK_REQUIRE(c->hll.size() == N * (size_t)kHllRegs, "no sketches: call chk_hll_sketch_all");
    uint64_t own = 0, shared = 0;
    std::map<int, std::vector<uint8_t>> unions;
    for (size_t i = 0; i < N; ++i) {
        const Tensor& t = c->tensors[i];
        if (!t.ptr || t.n_elem == 0 || elem_size(t.dtype) == 0) continue;
        const uint8_t* r = c->hll.data() + i * kHllRegs;
        const uint64_t mine = (uint64_t)(hll_count(r) * 8.0) + 64;
        own += mine;
        int cid = -1;
        if (c->have_clusters) {
            auto it = c->clusters.tensor_to_cluster.find(t.name);
            if (it != c->clusters.tensor_to_cluster.end()) cid = it->second;
        }
        if (cid < 0) {
            shared += mine;
            continue;
        }
        auto& u = unions[cid];
        if (u.empty()) u.assign(kHllRegs, 0);
        for (uint32_t k = 0; k < kHllRegs; ++k) u[k] = u[k] > r[k] ? u[k] : r[k];
    }
    for (const auto& kv : unions) shared += (uint64_t)(hll_count(kv.second.data()) * 8.0) + 64;
    *per_tensor_bytes = own;
    *shared_bytes = shared;
    CHK_API_END
}

int chk_get_tensor_stats(chk_context* c, uint64_t i, uint32_t hist[256], float moments[4], float minmax[2],
                         float fingerprint[5]) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    CHK_REQUIRE(i < c->stats.size(), "no statistics for that index: call chk_analyze first");
    const StatsOut& o = c->stats[i];
    if (hist) std::memcpy(hist, o.hist, 1024);
    if (moments) std::memcpy(moments, o.moments, 16);
    if (minmax) std::memcpy(minmax, o.minmax, 8);
    if (fingerprint) std::memcpy(fingerprint, o.fingerprint, 20);
    CHK_API_END
}

int chk_get_cluster_ids(chk_context* c, int32_t* ids, uint64_t cap, int32_t* n_clusters) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    CHK_REQUIRE(cap >= c->tensors.size() || !ids, "capacity too small");
    if (ids)
        for (size_t i = 0; i < c->tensors.size(); ++i) {
            auto it = c->clusters.tensor_to_cluster.find(c->tensors[i].name);
            ids[i] = (c->have_clusters && it != c->clusters.tensor_to_cluster.end()) ? it->second : -1;
        }
    if (n_clusters) *n_clusters = c->have_clusters ? c->clusters.n_clusters : 0;
    CHK_API_END
}

int chk_get_cluster_anchor(chk_context* c, int32_t cluster, char name_out[256]) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && name_out, "NULL argument");
    auto it = c->clusters.cluster_anchor.find(cluster);
    CHK_REQUIRE(c->have_clusters && it != c->clusters.cluster_anchor.end(), "no such cluster");
    std::memset(name_out, 0, 256);
    std::strncpy(name_out, it->second.c_str(), 255);
    CHK_API_END
}

int chk_set_cluster_info(chk_context* c, uint64_t n, const char* const* names, const int32_t* ids, int32_t n_clusters,
                         const char* const* anchors) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    CHK_REQUIRE(n == 0 || (names && ids), "names/ids are NULL");
    ClusterMap m;
    for (uint64_t i = 0; i < n; ++i) m.tensor_to_cluster[names[i]] = ids[i] < 0 ? -1 : ids[i];
    for (int32_t k = 0; k < n_clusters; ++k)
        if (anchors && anchors[k]) m.cluster_anchor[k] = anchors[k];
    m.n_clusters = n_clusters;
    c->clusters = std::move(m);
    c->have_clusters = true;
    CHK_API_END
}

int chk_compress_and_save(chk_context* c, const char* dir) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && dir, "NULL argument");
    compress_and_save(c, dir);
    CHK_API_END
}

int chk_compress(chk_context* c, int host_images) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    compress(c, host_images != 0);
    CHK_API_END
}

int chk_get_image(chk_context* c, int which, const void** data, uint64_t* size) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && data && size, "NULL argument");
    CHK_REQUIRE(which >= 0 && which < 3, "which must be 0, 1 or 2");
    CHK_REQUIRE(c->have_images, "no host images: call chk_compress(ctx, 1) first");
    *data = image_ptr(c, which);
    *size = image_size(c, which);
    CHK_API_END
}

int chk_get_table_report(chk_context* c, uint64_t* n_tables, uint64_t* n_undecodable) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    if (n_tables) *n_tables = c->n_tables;
    if (n_undecodable) *n_undecodable = c->undecodable_tables;
    CHK_API_END
}

int chk_get_summary(chk_context* c, chk_summary* out) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && out, "NULL argument");
    *out = c->summary;
    CHK_API_END
}

int chk_load_and_decompress(chk_context* c, const char* dir) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && dir, "NULL argument");
    load_and_decompress(c, dir);
    CHK_API_END
}

int chk_decompress_images(chk_context* c, const void* st, uint64_t st_n, const void* mt, uint64_t mt_n, const void* dc,
                          uint64_t dc_n) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && st && mt && dc, "NULL argument");
    decompress_images(c, static_cast<const uint8_t*>(st), st_n, static_cast<const uint8_t*>(mt), mt_n,
                      static_cast<const uint8_t*>(dc), dc_n);
    CHK_API_END
}

int chk_decompress_resident(chk_context* c, void* const* dst) {
    CHK_API_BEGIN
    CHK_REQUIRE(c, "context is NULL");
    decompress_resident(c, dst);
    CHK_API_END
}

int chk_restored_count(chk_context* c, uint64_t* count) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && count, "NULL argument");
    *count = c->restored;
    CHK_API_END
}

int chk_split(chk_context* c, const void* d_src, uint64_t n_elem, uint8_t dtype, void* d_masked, void* d_sidecar) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && d_src && d_masked, "NULL argument");
    const uint32_t es = elem_size(dtype), spe = sidecar_per_elem(dtype);
    CHK_REQUIRE(es && spe, "dtype has no low-byte split");
    CHK_REQUIRE(d_sidecar, "sidecar is NULL");
    if (n_elem == 0) return CHK_OK;
    CHK_CUDA(cudaSetDevice(c->device));
    const unsigned long long nb = n_elem * es;
    const uint32_t vec = ((reinterpret_cast<uintptr_t>(d_src) | reinterpret_cast<uintptr_t>(d_masked)) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(d_sidecar) & 7) == 0;
    const unsigned long long want = (nb / 16 + 255) / 256 + 1;
    const unsigned long long cap = (unsigned long long)(c->sm_count > 0 ? c->sm_count : 1) * 16;
    const uint32_t grid = (uint32_t)(want < cap ? want : cap);
    split_kernel<<<grid, 256, 0, c->stream>>>(static_cast<const uint8_t*>(d_src), nb, es, spe,
                                              static_cast<uint8_t*>(d_masked), static_cast<uint8_t*>(d_sidecar), vec);
    CHK_CUDA(cudaGetLastError());
    c->launches++;
    CHK_CUDA(cudaStreamSynchronize(c->stream));
    CHK_API_END
}

int chk_merge(chk_context* c, const void* d_masked, const void* d_sidecar, uint64_t n_elem, uint8_t dtype, void* d_out) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && d_masked && d_sidecar && d_out, "NULL argument");
    const uint32_t es = elem_size(dtype), spe = sidecar_per_elem(dtype);
    CHK_REQUIRE(es && spe, "dtype has no low-byte split");
    if (n_elem == 0) return CHK_OK;
    CHK_CUDA(cudaSetDevice(c->device));
    const unsigned long long nb = n_elem * es;
    const uint32_t vec = ((reinterpret_cast<uintptr_t>(d_masked) | reinterpret_cast<uintptr_t>(d_out)) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(d_sidecar) & 7) == 0;
    const unsigned long long want = (nb / 16 + 255) / 256 + 1;
    const unsigned long long cap = (unsigned long long)(c->sm_count > 0 ? c->sm_count : 1) * 16;
    merge_kernel<<<(uint32_t)(want < cap ? want : cap), 256, 0, c->stream>>>(
        static_cast<const uint8_t*>(d_masked), static_cast<const uint8_t*>(d_sidecar), nb, es, spe,
        static_cast<uint8_t*>(d_out), vec);
    CHK_CUDA(cudaGetLastError());
    c->launches++;
    sync_stream(c, c->stream);
    CHK_API_END
}

int chk_byte_histogram(chk_context* c, const void* d_data, uint64_t n_bytes, uint32_t hist_out[256]) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && hist_out, "NULL argument");
    std::memset(hist_out, 0, 1024);
    if (n_bytes == 0) return CHK_OK;
    CHK_REQUIRE(d_data, "data is NULL");
    CHK_CUDA(cudaSetDevice(c->device));
    dev_ensure(c, c->d_hist, 1024);
    CHK_CUDA(cudaMemsetAsync(c->d_hist.p, 0, 1024, c->stream));
    const unsigned long long want = (n_bytes / 16 + 255) / 256 + 1;
    const unsigned long long cap = (unsigned long long)(c->sm_count > 0 ? c->sm_count : 1) * 8;
    const uint32_t grid = (uint32_t)(want < cap ? want : cap);
    byte_histogram_kernel<<<grid, 256, 0, c->stream>>>(static_cast<const uint8_t*>(d_data), n_bytes,
                                                       static_cast<uint32_t*>(c->d_hist.p));
    CHK_CUDA(cudaGetLastError());
    c->launches++;
    CHK_CUDA(cudaMemcpyAsync(hist_out, c->d_hist.p, 1024, cudaMemcpyDeviceToHost, c->stream));
    CHK_CUDA(cudaStreamSynchronize(c->stream));
    CHK_API_END
}

int chk_normalize_histogram(const uint32_t hist[256], int full, int repair, uint32_t norm_freq[256],
                            uint32_t cum_freq[257], uint32_t x_max[256], uint32_t* sum_out) {
    CHK_API_BEGIN
    CHK_REQUIRE(hist && norm_freq && cum_freq, "NULL argument");
    FreqTable t;
    normalize_histogram(hist, full != 0, repair != 0, t);
    std::memcpy(norm_freq, t.norm_freq, 1024);
    std::memcpy(cum_freq, t.cum_freq, 1028);
    if (x_max)
        for (int s = 0; s < 256; ++s) x_max[s] = t.norm_freq[s] << 19;
    if (sum_out) *sum_out = t.sum;
    CHK_API_END
}

int chk_get_timing(chk_context* c, const char* key, double* ms) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && key && ms, "NULL argument");
    auto it = c->timing.find(key);
    *ms = it == c->timing.end() ? 0.0 : it->second;
    CHK_API_END
}

int chk_get_stream(chk_context* c, void** stream_out) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && stream_out, "NULL argument");
    *stream_out = c->stream;
    CHK_API_END
}

int chk_kernel_launches(chk_context* c, uint64_t* count) {
    CHK_API_BEGIN
    CHK_REQUIRE(c && count, "NULL argument");
    *count = c->launches;
    CHK_API_END
}

}  // extern "C"

#include "host_stream.inc"
#include "format_v3.inc"

// ====================================================================== encode without allocating
// chk_encode_tensor_static: the rANS encode of ONE tensor whose working memory
// (lane scratch regions, offset tables, the uploaded frequency table, the
// ticket counter) lives in a fixed device array that is part of the library
// image, so the call performs no device or pinned-host allocation at all.
//
// Who needs it: code that compresses state at the moment device memory is
// fullest or is owned by someone else -- a checkpoint hook that fires at the
// peak of a training step, a process whose whole HBM is held by another
// framework's caching allocator, a serving loop that may not block on the
// allocator.  For those callers cudaMalloc can fail, synchronise the device or
// fragment a pool; a fixed region cannot.
//
// The price: every GPU that loads this library carries kStaticScratchBytes
// (about 8.3 MiB) until the process exits, tensors are limited to
// CHK_STATIC_MAX_TENSOR_BYTES, all calls on a device share the one region
// (calls that overlap on the GPU would corrupt each other -- issue them on one
// stream or order them yourself), and the region keeps the previous call's
// contents (the call clears the few words that must start at zero).
namespace chk {

constexpr unsigned long long kStaticMaxTensorBytes = CHK_STATIC_MAX_TENSOR_BYTES;
constexpr uint32_t kStaticChunkStride = (uint32_t)(2 * ((kStaticMaxTensorBytes + 255) / 256));  // bytes per lane

struct StaticScratch {
    TensorDesc desc;
    uint32_t order[4];
    uint32_t ticket[4];
    unsigned long long payload_size[2];
    unsigned long long payload_off[2];
    EncEntry enc[256];
    unsigned long long lane_src[256];
    uint32_t lane_off[256];
    alignas(256) uint8_t lanes[256ull * kStaticChunkStride + 256];  // lane regions are written 16 bytes at a time
};
constexpr size_t kStaticScratchBytes = sizeof(StaticScratch);
static_assert(offsetof(StaticScratch, lanes) % 16 == 0 && offsetof(StaticScratch, lane_src) % 8 == 0 &&
                  offsetof(StaticScratch, payload_size) % 8 == 0,
              "static scratch members must keep their natural alignment");

// In host code this name is only a handle for cudaGetSymbolAddress; the device
// address it stands for is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_static_mutex;
static unsigned char* g_static_addr[64] = {};  // per device ordinal

// First call on a device: resolve the array's device address with that device current.
static unsigned char* static_scratch_for_current_device() {
    int dev = -1;
    CHK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) throw Error{CHK_ERR_INVALID, "device ordinal out of range for the static scratch table"};
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_addr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            throw Error{CHK_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e)};
        g_static_addr[dev] = static_cast<unsigned char*>(p);
    }
    return g_static_addr[dev];
}

}  // namespace chk

extern "C" int chk_encode_tensor_static(const void* d_src, uint64_t num_elements, uint8_t dtype,
                                        const uint32_t norm_freq[256], const uint32_t cum_freq[257],
                                        void* d_payload, void* d_lane_headers, uint64_t* payload_size_out,
                                        int* is_raw_out, void* stream) {
    CHK_API_BEGIN
    CHK_REQUIRE(d_src && norm_freq && cum_freq && d_payload && d_lane_headers && payload_size_out, "NULL argument");
    const uint32_t es = elem_size(dtype), spe = sidecar_per_elem(dtype);
    CHK_REQUIRE(es != 0, "unknown dtype");
    CHK_REQUIRE(num_elements != 0, "empty tensor");
    const unsigned long long bytes = (unsigned long long)num_elements * es;
    if (bytes > kStaticMaxTensorBytes)
        throw chk::Error{CHK_ERR_CAPACITY, "tensor of " + std::to_string(bytes) + " bytes exceeds the fixed scratch limit of " +
                                               std::to_string(kStaticMaxTensorBytes) + " bytes (CHK_STATIC_MAX_TENSOR_BYTES)"};
    unsigned char* base = static_scratch_for_current_device();
    StaticScratch* dev = reinterpret_cast<StaticScratch*>(base);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // host-side image of the small header part (desc .. enc); lives on this stack frame only
    struct Head {
        TensorDesc desc;
        uint32_t order[4];
        uint32_t ticket[4];
        unsigned long long payload_size[2];
        unsigned long long payload_off[2];
        EncEntry enc[256];
    } head;
    static_assert(offsetof(StaticScratch, lane_src) == sizeof(Head), "header layout");
    std::memset(&head, 0, sizeof(head));  // order[0] = 0, ticket = 0, sizes = 0
    const unsigned long long c_max = (bytes + 255) / 256;
    head.desc.src = static_cast<const uint8_t*>(d_src);
    head.desc.n_bytes = bytes;
    head.desc.es = es;
    head.desc.spe = spe;
    head.desc.table_idx = 0;
    head.desc.scratch_off = offsetof(StaticScratch, lanes);
    head.desc.chunk_stride = (uint32_t)((2 * c_max + 31) & ~31ull);
    CHK_REQUIRE(cum_freq[0] == 0, "cum_freq[0] must be 0");
    for (int i = 0; i < 256; ++i) {
        CHK_REQUIRE(norm_freq[i] <= kM, "norm_freq above 4096");
        CHK_REQUIRE(cum_freq[i + 1] == cum_freq[i] + norm_freq[i], "cum_freq is not the running sum of norm_freq");
    }
    FreqTable ft;
    std::memcpy(ft.norm_freq, norm_freq, 1024);
    std::memcpy(ft.cum_freq, cum_freq, 1028);
    ft.sum = cum_freq[256];
    build_enc_entries(ft, head.enc);
    bool escape = false;
    for (int i = 0; i < 256 && !escape; ++i) escape = norm_freq[i] == 0;

    // pageable source: the runtime stages it before returning, so the stack frame may go away
    CHK_CUDA(cudaMemcpyAsync(base, &head, sizeof(head), cudaMemcpyHostToDevice, s));
    const bool ints = spe * 2 != es;
    zero_lane_kernel<<<1, 32, 0, s>>>(&dev->desc, dev->enc, base, static_cast<LaneHeader*>(d_lane_headers), dev->lane_src,
                                      1u);
    CHK_CUDA(cudaGetLastError());
    auto kernel = ints ? (escape ? rans_encode_kernel<true, true> : rans_encode_kernel<true, false>)
                       : (escape ? rans_encode_kernel<false, true> : rans_encode_kernel<false, false>);
    kernel<<<1, kTeam, ints ? sizeof(EncSmem<4>) : sizeof(EncSmem<2>), s>>>(
        &dev->desc, dev->enc, base, static_cast<LaneHeader*>(d_lane_headers), dev->lane_src, dev->order, dev->ticket, 1u);
    CHK_CUDA(cudaGetLastError());
    lane_scan_kernel<<<1, 256, 0, s>>>(&dev->desc, static_cast<LaneHeader*>(d_lane_headers), dev->payload_size,
                                       dev->lane_off, 1u);
    CHK_CUDA(cudaGetLastError());
    tensor_scan_kernel<<<1, 1024, 0, s>>>(&dev->desc, dev->payload_size, dev->payload_off, 1u, nullptr);
    CHK_CUDA(cudaGetLastError());
    compact_kernel<<<32, 256, 0, s>>>(&dev->desc, static_cast<const LaneHeader*>(d_lane_headers), dev->lane_src,
                                      dev->lane_off, base, static_cast<uint8_t*>(d_payload), 1u);
    CHK_CUDA(cudaGetLastError());
    struct {
        unsigned long long size;
        TensorDesc desc;
    } back;
    CHK_CUDA(cudaMemcpyAsync(&back.size, dev->payload_size, 8, cudaMemcpyDeviceToHost, s));
    CHK_CUDA(cudaMemcpyAsync(&back.desc, &dev->desc, sizeof(TensorDesc), cudaMemcpyDeviceToHost, s));
    CHK_CUDA(cudaStreamSynchronize(s));
    *payload_size_out = back.size;
    if (is_raw_out) *is_raw_out = (back.desc.flags & kFlagRaw) ? 1 : 0;
    CHK_API_END
}
