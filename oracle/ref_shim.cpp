// ref_shim.cpp -- CPU harness around function bodies cut out of the Checkers
// reference by oracle/build_ref.py.  TEST INFRASTRUCTURE ONLY.
//
// The *.inc files included below do not exist in this repository: build_ref.py
// writes them to a temporary directory from the reference tree and deletes
// them after compiling.  This file supplies what those bodies need to run on a
// CPU: a one-OS-thread emulation of a CUDA thread block (each CUDA thread is a
// ucontext fiber, __syncthreads() yields to the next fiber), stand-ins for
// half/bfloat16, and stub owner classes exposing only the members the cut
// functions touch.  Single-threaded by design; meant for small inputs.
#include <ucontext.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <new>
#include <numeric>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

// ---------------------------------------------------------------- block emulator
struct Idx3 {
    unsigned x = 0, y = 0, z = 0;
};
struct dim3 {
    unsigned x, y, z;
    dim3(unsigned a = 1, unsigned b = 1, unsigned c = 1) : x(a), y(b), z(c) {}
};
static Idx3 threadIdx, blockIdx;
static dim3 blockDim, gridDim;

namespace emu {
constexpr size_t kStack = 256 * 1024;
struct Fiber {
    ucontext_t ctx;
    char* stack = nullptr;  // from a pool that is allocated once and reused by every block
    bool done = false;
};
// Fiber stacks are not zeroed and never freed: blocks run one after another and reuse them.
static char* fiber_stack(unsigned t) {
    static std::vector<char*> pool;
    while (pool.size() <= t) pool.push_back(static_cast<char*>(std::malloc(kStack)));
    return pool[t];
}
static ucontext_t g_main;
static std::vector<Fiber>* g_fibers = nullptr;
static unsigned g_cur = 0;
static std::function<void()>* g_body = nullptr;

static void trampoline() {
    (*g_body)();
    (*g_fibers)[g_cur].done = true;
    swapcontext(&(*g_fibers)[g_cur].ctx, &g_main);
}
static void yield() { swapcontext(&(*g_fibers)[g_cur].ctx, &g_main); }

static void run_block(unsigned nthreads, std::function<void()> body) {
    std::vector<Fiber> fibers(nthreads);
    g_fibers = &fibers;
    g_body = &body;
    for (unsigned t = 0; t < nthreads; ++t) {
        Fiber& f = fibers[t];
        f.stack = fiber_stack(t);
        getcontext(&f.ctx);
        f.ctx.uc_stack.ss_sp = f.stack;
        f.ctx.uc_stack.ss_size = kStack;
        f.ctx.uc_link = &g_main;
        makecontext(&f.ctx, trampoline, 0);
    }
    bool live = true;
    while (live) {  // one sweep == "run every thread to its next barrier"
        live = false;
        for (unsigned t = 0; t < nthreads; ++t) {
            if (fibers[t].done) continue;
            g_cur = t;
            threadIdx.x = t;
            swapcontext(&g_main, &fibers[t].ctx);
            live |= !fibers[t].done;
        }
    }
    g_fibers = nullptr;
    g_body = nullptr;
}

template <typename F>
static void launch(unsigned grid, unsigned block, F&& kernel_call) {
    gridDim = dim3(grid);
    blockDim = dim3(block);
    for (unsigned b = 0; b < grid; ++b) {
        blockIdx.x = b;
        run_block(block, kernel_call);
    }
}
}  // namespace emu

static inline void __syncthreads() { emu::yield(); }
template <typename T>
static inline T atomicAdd(T* p, T v) {
    T old = *p;
    *p = old + v;
    return old;
}
using std::max;
using std::min;

#define __global__
#define __device__
#define __forceinline__ inline
#define __shared__ static

// 16-bit float stand-ins (bit containers; conversions are exact)
struct half {
    uint16_t bits;
};
struct __nv_bfloat16 {
    uint16_t bits;
};
static inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31;
    int e = (h >> 10) & 31;
    uint32_t m = h & 1023;
    uint32_t out;
    if (e == 31)
        out = sign | 0x7F800000u | (m << 13);
    else if (e == 0) {
        if (!m)
            out = sign;
        else {
            e = 1;
            while (!(m & 1024)) {
                m <<= 1;
                --e;
            }
            out = sign | ((uint32_t)(e + 112) << 23) | ((m & 1023) << 13);
        }
    } else
        out = sign | ((uint32_t)(e + 112) << 23) | (m << 13);
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}
template <typename T>
static inline float to_float(T v) {
    return static_cast<float>(v);
}
template <>
inline float to_float(half v) {
    return half_to_float(v.bits);
}
template <>
inline float to_float(__nv_bfloat16 v) {
    uint32_t b = (uint32_t)v.bits << 16;
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}

// ---------------------------------------------------------------- reference text
namespace checkers {

#include "types.inc"

class RankLogger {
  public:
    void log_message(const std::string&) {}
    int global_rank() const { return 0; }
};

struct Fingerprint {
    double values[5];
};

class MemoryManager {
  public:
    static MemoryManager& instance() {
        static MemoryManager m;
        return m;
    }
    const std::vector<Fingerprint>& get_fingerprints() const { return fps; }
    const std::string& get_name_from_index(size_t i) const { return names[i]; }
    void set_cluster_info(ClusterInfo ci) { info = std::move(ci); }
    std::vector<Fingerprint> fps;
    std::vector<std::string> names;
    ClusterInfo info;
};

#include "kernels.inc"

#define __CUDACC__ 1
#include "stats.inc"
#undef __CUDACC__

class ANSCompressor {
  public:
#include "member_types.inc"
    ANSFreqTable normalize_histogram(const uint32_t h_raw_hist[256], bool ensure_full_alphabet = false) const;
    void write_rank_states_file(const std::string& path, int rank, const std::vector<CompressedTensor>& cts) const;
    void write_rank_mantissa_file(const std::string& path, int rank, const std::vector<SidecarEntry>& sidecars) const;
    void write_rank_tables_file(const std::string& path, int rank, const std::vector<TableEntry>& tables) const;
};

#include "host.inc"

class TensorAnalyzer {
  public:
    using gpuStream_t = void*;
    std::shared_ptr<RankLogger> m_logger;
    void build_knn_clusters(DeviceTensorRecord* d_records, size_t N, int K, gpuStream_t stream);
};

#include "cluster.inc"

}  // namespace checkers

// ---------------------------------------------------------------- C entry points
using namespace checkers;

extern "C" {

void ref_split(const uint8_t* src, size_t n_elem, uint32_t es, uint32_t spe, uint8_t* masked, uint8_t* sidecar) {
    if (!n_elem) return;
    const unsigned grid = (unsigned)((n_elem + 255) / 256);
    emu::launch(grid, 256, [&] { extract_mantissa_kernel(src, masked, sidecar, n_elem, es, spe); });
}

void ref_byte_histogram(const uint8_t* data, size_t n, uint32_t hist[256]) {
    std::memset(hist, 0, 1024);
    if (!n) return;
    const unsigned grid = (unsigned)std::min<size_t>((n + 255) / 256, 4096);
    emu::launch(grid, 256, [&] { byte_histogram_kernel(data, n, hist); });
}

// The reference fills its 4096-entry decode tables up to cum_freq[256]; when
// its table sums past 4096 those writes run off the struct.  The result is
// therefore built inside a padded arena so the stray writes stay in memory this
// harness owns.
struct PaddedTable {
    alignas(64) unsigned char room[sizeof(ANSFreqTable) + (8 << 20)];
};

uint32_t ref_normalize(const uint32_t hist[256], int full, uint32_t nf[256], uint32_t cf[257], uint32_t xm[256]) {
    static PaddedTable arena;
    ANSCompressor c;
    ANSFreqTable* t = new (arena.room) ANSFreqTable(c.normalize_histogram(hist, full != 0));
    std::memcpy(nf, t->norm_freq, 1024);
    std::memcpy(cf, t->cum_freq, 1028);
    std::memcpy(xm, t->x_max, 1024);
    uint32_t s = 0;
    for (int i = 0; i < 256; ++i) s += nf[i];
    return s;
}

// Lanes + CPU prefix sum + compaction exactly as compress_tensor drives them;
// the passthrough decision is left to the caller (it is host logic of
// compress_tensor, which cannot be cut out).  Returns total compressed bytes.
size_t ref_encode_compact(const uint8_t* data, size_t n, const uint32_t nf[256], const uint32_t cf[257],
                          const uint32_t xm[256], uint32_t headers_out[1024], uint8_t* compact_out) {
    if (!n) return 0;
    const size_t max_chunk = ((n + 255) / 256) * 2;
    std::vector<uint8_t> enc(256 * max_chunk);
    std::vector<ANSStreamHeader> hdr(256);
    emu::launch(1, 256, [&] { rans_encode_kernel(data, n, nf, cf, xm, enc.data(), hdr.data(), max_chunk); });
    uint32_t off[257];
    off[0] = 0;
    for (int t = 0; t < 256; ++t) off[t + 1] = off[t] + hdr[t].byte_count;
    emu::launch(256, 256, [&] { compact_streams_kernel(enc.data(), hdr.data(), compact_out, off, max_chunk); });
    std::memcpy(headers_out, hdr.data(), 4096);
    return off[256];
}

void ref_tensor_stats(void* data, size_t n, int dtype, uint32_t bins, uint32_t* hist, float moments[4],
                      float minmax[2]) {
    DeviceTensorRecord rec{};
    rec.d_ptr = data;
    rec.d_histogram = hist;
    rec.d_raw_moments = moments;
    rec.d_minmax = minmax;
    rec.num_elements = n;
    rec.histogram_bins = bins;
    rec.data_type = (uint8_t)dtype;
    emu::launch(1, 256, [&] { tensor_stats_kernel(&rec, 1); });
}

int ref_build_clusters(size_t n, const char* const* names, const float* fps, int* cluster_id, int* anchor_index) {
    MemoryManager& m = MemoryManager::instance();
    m.fps.resize(n);
    m.names.resize(n);
    m.info = ClusterInfo{};
    for (size_t i = 0; i < n; ++i) {
        m.names[i] = names[i];
        for (int d = 0; d < 5; ++d) m.fps[i].values[d] = (double)fps[i * 5 + d];
    }
    TensorAnalyzer a;
    a.m_logger = std::make_shared<RankLogger>();
    a.build_knn_clusters(nullptr, n, 4, nullptr);
    int n_clusters = 0;
    for (size_t i = 0; i < n; ++i) {
        auto it = m.info.tensor_to_cluster.find(m.names[i]);
        cluster_id[i] = it == m.info.tensor_to_cluster.end() ? -1 : it->second;
        n_clusters = std::max(n_clusters, cluster_id[i] + 1);
    }
    for (int c = 0; c < n_clusters; ++c) {
        anchor_index[c] = -1;
        auto it = m.info.cluster_anchor.find(c);
        if (it == m.info.cluster_anchor.end()) continue;
        for (size_t i = 0; i < n; ++i)
            if (m.names[i] == it->second) {
                anchor_index[c] = (int)i;
                break;
            }
    }
    return n_clusters;
}

// Writers.  lanes: n*1024 uint32 (final_state, byte_count, buf_offset, pad).
int ref_write_states(const char* path, int rank, size_t n, const char* const* names, const uint8_t* dtypes,
                     const uint64_t* original_bytes, const uint64_t* num_elements, const uint8_t* owns,
                     const char* const* anchors, const uint32_t* lanes, const uint8_t* const* payload,
                     const uint64_t* payload_size) {
    std::vector<CompressedTensor> cts(n);
    for (size_t i = 0; i < n; ++i) {
        cts[i].name = names[i];
        cts[i].dtype = (DataType)dtypes[i];
        cts[i].original_bytes = original_bytes[i];
        cts[i].num_elements = num_elements[i];
        cts[i].owns_table = owns[i] != 0;
        cts[i].anchor_name = anchors[i] ? anchors[i] : "";
        std::memcpy(cts[i].streams, lanes + i * 1024, 4096);
        cts[i].data.assign(payload[i], payload[i] + payload_size[i]);
    }
    try {
        ANSCompressor().write_rank_states_file(path, rank, cts);
    } catch (...) {
        return -1;
    }
    return 0;
}

int ref_write_mantissa(const char* path, int rank, size_t n, const char* const* names, const uint8_t* dtypes,
                       const uint64_t* num_elements, const uint8_t* spe, const uint8_t* const* data,
                       const uint64_t* size) {
    std::vector<ANSCompressor::SidecarEntry> v(n);
    for (size_t i = 0; i < n; ++i) {
        v[i].name = names[i];
        v[i].dtype = (DataType)dtypes[i];
        v[i].n_elements = num_elements[i];
        v[i].si.bytes_per_elem = spe[i];
        v[i].si.data.assign(data[i], data[i] + size[i]);
    }
    try {
        ANSCompressor().write_rank_mantissa_file(path, rank, v);
    } catch (...) {
        return -1;
    }
    return 0;
}

int ref_write_tables(const char* path, int rank, size_t n, const char* const* names, const uint32_t* nf,
                     const uint32_t* cf) {
    std::vector<ANSCompressor::TableEntry> v(n);
    for (size_t i = 0; i < n; ++i) {
        v[i].anchor_name = names[i];
        std::memset(&v[i].table, 0, sizeof(ANSFreqTable));
        std::memcpy(v[i].table.norm_freq, nf + i * 256, 1024);
        std::memcpy(v[i].table.cum_freq, cf + i * 257, 1028);
    }
    try {
        ANSCompressor().write_rank_tables_file(path, rank, v);
    } catch (...) {
        return -1;
    }
    return 0;
}

}  // extern "C"
