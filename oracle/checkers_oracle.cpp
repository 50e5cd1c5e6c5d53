// checkers_oracle.cpp -- CPU restatement of the Checkers checkpoint-compression
// path.  TEST INFRASTRUCTURE ONLY (see checkers_oracle.h).  Build:
//   g++ -std=c++17 -O2 -ffp-contract=off -fopenmp -fPIC -shared
// -ffp-contract=off matters: the statistics below must not be fused.
#include "checkers_oracle.h"

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <map>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr uint32_t kLanes = ORC_LANES;
constexpr uint32_t kM = ORC_M;
constexpr uint32_t kL = ORC_L;
constexpr uint32_t kNormBase = (kL >> ORC_SCALE_BITS) << 8;  // 2^19, ANSCompressor.hpp:54

int clamp_threads(int n) {
#ifdef _OPENMP
    if (n <= 0) n = omp_get_max_threads();
#else
    n = 1;
#endif
    return n < 1 ? 1 : n;
}

// Shared body of the two normalisers.  `repeat_fix` = false follows
// src/ANSCompressor.cpp:416-503 literally.
uint32_t normalize_impl(const uint32_t hist[256], bool full, bool repeat_fix,
                        uint32_t nf[256], uint32_t cf[257], uint32_t xm[256]) {
    std::memset(nf, 0, 256 * sizeof(uint32_t));
    std::memset(cf, 0, 257 * sizeof(uint32_t));
    std::memset(xm, 0, 256 * sizeof(uint32_t));

    uint64_t total = 0;
    int distinct = 0;
    for (int s = 0; s < 256; ++s) {
        total += hist[s];
        distinct += hist[s] > 0;
    }
    if ((full ? 256 : distinct) == 0) {  // :432-441 -- everything on symbol 0
        nf[0] = kM;
        for (int s = 1; s <= 256; ++s) cf[s] = kM;
        xm[0] = kNormBase * kM;
        return kM;
    }

    // :448-456 proportional floor with a minimum of one slot
    uint32_t slots[256] = {};
    uint32_t assigned = 0;
    for (int s = 0; s < 256; ++s) {
        if (!full && hist[s] == 0) continue;
        uint32_t v = total > 0 ? (uint32_t)((uint64_t)std::max(hist[s], 1u) * kM / total) : 0u;
        if (v == 0) v = 1;
        slots[s] = v;
        assigned += v;
    }

    // :459-471 order by fractional part, descending, with std::sort (unstable:
    // the tie order of libstdc++'s introsort is part of the result).
    struct Frac {
        int sym;
        double frac;
    };
    std::vector<Frac> order;
    order.reserve(256);
    for (int s = 0; s < 256; ++s) {
        if (slots[s] == 0) continue;
        double exact = total > 0 ? ((double)std::max(hist[s], 1u) * kM / (double)total) : 1.0;
        order.push_back({s, exact - (double)(int)exact});
    }
    std::sort(order.begin(), order.end(), [](const Frac& a, const Frac& b) { return a.frac > b.frac; });

    if (assigned < kM) {  // :473-476
        uint32_t rem = kM - assigned;
        for (size_t k = 0; k < order.size() && rem; ++k, --rem) slots[order[k].sym]++;
    } else if (assigned > kM) {  // :477-482 one reverse pass in the reference
        uint32_t rem = assigned - kM;
        do {
            uint32_t before = rem;
            for (int k = (int)order.size() - 1; k >= 0 && rem; --k) {
                if (slots[order[k].sym] > 1) {
                    slots[order[k].sym]--;
                    --rem;
                }
            }
            if (rem == before) break;  // nothing left to take
        } while (repeat_fix && rem);
    }

    uint32_t sum = 0;
    for (int s = 0; s < 256; ++s) {
        nf[s] = slots[s];
        cf[s + 1] = cf[s] + slots[s];
        xm[s] = slots[s] ? kNormBase * slots[s] : 0u;  // :493-494
        sum += slots[s];
    }
    return sum;
}

inline float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FF;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal half -> normal float
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline float load_as_float(const void* p, size_t i, int dtype) {
    switch (dtype) {
        case ORC_F32:
            return ((const float*)p)[i];
        case ORC_BF16: {
            uint32_t b = (uint32_t)((const uint16_t*)p)[i] << 16;
            float f;
            std::memcpy(&f, &b, 4);
            return f;
        }
        case ORC_F16:
            return half_bits_to_float(((const uint16_t*)p)[i]);
        case ORC_I8:
            return (float)((const int8_t*)p)[i];
        case ORC_I32:
            return (float)((const int32_t*)p)[i];
        default:
            return 0.0f;
    }
}

struct FileEntry {
    std::string name;
    uint8_t dtype = 0, is_raw = 0, owns = 0;
    uint64_t original_bytes = 0, num_elements = 0, data_offset = 0, data_size = 0;
    std::string anchor;
    orc_lane_header lanes[256];
};

void put_name(std::ofstream& f, const std::string& s) {
    char buf[256] = {};
    std::strncpy(buf, s.c_str(), 255);
    f.write(buf, 256);
}
template <typename T>
void put(std::ofstream& f, const T& v) {
    f.write(reinterpret_cast<const char*>(&v), sizeof(T));
}

bool read_all(const std::string& path, std::vector<uint8_t>& out) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) return false;
    std::streamsize n = f.tellg();
    f.seekg(0);
    out.resize((size_t)n);
    return n == 0 || (bool)f.read(reinterpret_cast<char*>(out.data()), n);
}

std::string cstr256(const uint8_t* p) {
    size_t n = 0;
    while (n < 256 && p[n]) ++n;
    return std::string(reinterpret_cast<const char*>(p), n);
}

}  // namespace

extern "C" {

uint32_t orc_elem_size(int dtype) {
    switch (dtype) {
        case ORC_F32: return 4;
        case ORC_BF16: return 2;
        case ORC_F16: return 2;
        case ORC_I8: return 1;
        case ORC_I32: return 4;
        default: return 0;
    }
}

uint32_t orc_sidecar_per_elem(int dtype) {
    switch (dtype) {
        case ORC_F16:
        case ORC_BF16: return 1;
        case ORC_F32: return 2;
        default: return 0;
    }
}

void orc_split(const uint8_t* src, size_t n_elem, uint32_t es, uint32_t spe, uint8_t* masked,
               uint8_t* sidecar) {
    for (size_t i = 0; i < n_elem; ++i) {
        for (uint32_t j = 0; j < es; ++j) masked[i * es + j] = j < spe ? 0 : src[i * es + j];
        for (uint32_t j = 0; j < spe; ++j) sidecar[i * spe + j] = src[i * es + j];
    }
}

void orc_byte_histogram(const uint8_t* data, size_t n_bytes, uint32_t hist[256]) {
    std::memset(hist, 0, 256 * sizeof(uint32_t));
    for (size_t i = 0; i < n_bytes; ++i) hist[data[i]]++;
}

uint32_t orc_normalize(const uint32_t hist[256], int full, uint32_t nf[256], uint32_t cf[257],
                       uint32_t xm[256]) {
    return normalize_impl(hist, full != 0, false, nf, cf, xm);
}

uint32_t orc_normalize_repaired(const uint32_t hist[256], int full, uint32_t nf[256],
                                uint32_t cf[257], uint32_t xm[256]) {
    return normalize_impl(hist, full != 0, true, nf, cf, xm);
}

uint32_t orc_encode_lane(const uint8_t* data, size_t n_bytes, uint32_t lane, const uint32_t nf[256],
                         const uint32_t cf[257], const uint32_t xm[256], uint8_t* region,
                         size_t max_chunk, uint32_t* final_state) {
    // symbols of this lane: lane, lane+256, ... (src/ANSCompressor.cpp:168)
    const size_t count = n_bytes > lane ? (n_bytes - lane + kLanes - 1) / kLanes : 0;
    uint8_t* const end = region + max_chunk;
    uint8_t* w = end;
    uint32_t x = kL;
    for (size_t k = count; k-- > 0;) {  // last symbol first (:178)
        const uint8_t s = data[(size_t)lane + k * kLanes];
        const uint32_t f = nf[s];
        if (f == 0) {  // symbol missing from the table: raw escape byte (:185-192)
            if (w > region) *--w = s;
            continue;
        }
        while (x >= xm[s]) {  // :195-199
            if (w <= region) {
                w = region;
                break;
            }
            *--w = (uint8_t)(x & 0xFF);
            x >>= 8;
        }
        x = ((x / f) << ORC_SCALE_BITS) + cf[s] + (x % f);  // :202
    }
    *final_state = x;
    return (uint32_t)(end - w);
}

size_t orc_compress_tensor(const uint8_t* data, size_t n_bytes, const uint32_t nf[256],
                           const uint32_t cf[257], const uint32_t xm[256],
                           orc_lane_header headers[256], uint8_t* out, int* is_raw, int n_threads) {
    *is_raw = 0;
    std::memset(headers, 0, 256 * sizeof(orc_lane_header));
    if (n_bytes == 0) return 0;
    const size_t max_chunk = ((n_bytes + kLanes - 1) / kLanes) * 2;  // :590
    std::vector<uint8_t> scratch(kLanes * max_chunk);
    const int nt = clamp_threads(n_threads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int t = 0; t < (int)kLanes; ++t) {
        uint32_t st;
        uint32_t cnt = orc_encode_lane(data, n_bytes, (uint32_t)t, nf, cf, xm,
                                       scratch.data() + (size_t)t * max_chunk, max_chunk, &st);
        headers[t].final_state = st;
        headers[t].byte_count = cnt;
        headers[t].buf_offset = (uint32_t)(max_chunk - cnt);
        headers[t].pad = 0;
    }
    // :647-651 prefix sum, :225-238 gather, :686-691 offsets become compact offsets
    uint32_t off = 0;
    for (uint32_t t = 0; t < kLanes; ++t) {
        std::memcpy(out + off, scratch.data() + (size_t)t * max_chunk + headers[t].buf_offset,
                    headers[t].byte_count);
        headers[t].buf_offset = off;
        off += headers[t].byte_count;
    }
    const size_t total = off;
    if (total >= n_bytes) {  // :695-713 raw passthrough of the codec input
        std::memcpy(out, data, n_bytes);
        std::memset(headers, 0, 256 * sizeof(orc_lane_header));
        headers[0].byte_count = (uint32_t)n_bytes;
        *is_raw = 1;
        return n_bytes;
    }
    return total;
}

int orc_decode_tensor(const uint8_t* payload, size_t payload_size, const orc_lane_header headers[256],
                      int is_raw, const uint32_t nf[256], const uint32_t cf[257], size_t n_bytes,
                      uint8_t* masked_out, int n_threads) {
    if (is_raw) {
        if (payload_size < n_bytes) return -4;
        std::memcpy(masked_out, payload, n_bytes);
        return 0;
    }
    if (cf[256] != kM) return -1;
    // slot -> symbol (the table the reference builds at :492-500)
    std::vector<uint8_t> slot_sym(kM);
    for (int s = 0; s < 256; ++s)
        for (uint32_t j = cf[s]; j < cf[s + 1]; ++j) slot_sym[j] = (uint8_t)s;
    int rc = 0;
    const int nt = clamp_threads(n_threads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int t = 0; t < (int)kLanes; ++t) {
        const size_t count = n_bytes > (size_t)t ? (n_bytes - t + kLanes - 1) / kLanes : 0;
        const orc_lane_header& h = headers[t];
        if ((size_t)h.buf_offset + h.byte_count > payload_size) {
#pragma omp critical
            rc = -4;
            continue;
        }
        const uint8_t* p = payload + h.buf_offset;
        const uint8_t* const end = p + h.byte_count;
        uint32_t x = h.final_state;
        bool short_read = false;
        for (size_t k = 0; k < count; ++k) {
            const uint32_t slot = x & (kM - 1);
            const uint8_t s = slot_sym[slot];
            masked_out[(size_t)t + k * kLanes] = s;
            x = nf[s] * (x >> ORC_SCALE_BITS) + slot - cf[s];
            while (x < kL) {
                if (p >= end) {
                    short_read = true;
                    break;
                }
                x = (x << 8) | *p++;
            }
            if (short_read) break;
        }
        if (short_read || p != end) {
#pragma omp critical
            if (rc == 0 || rc == -2) rc = -3;
        } else if (x != kL) {
#pragma omp critical
            if (rc == 0) rc = -2;
        }
    }
    return rc;
}

void orc_merge(const uint8_t* masked, const uint8_t* sidecar, size_t n_elem, uint32_t es, uint32_t spe,
               uint8_t* out) {
    for (size_t i = 0; i < n_elem; ++i)
        for (uint32_t j = 0; j < es; ++j)
            out[i * es + j] = j < spe ? (uint8_t)(masked[i * es + j] | sidecar[i * spe + j]) : masked[i * es + j];
}

void orc_tensor_stats(const void* data, size_t n, int dtype, uint32_t bins_in, uint32_t hist[256],
                      float moments[4], float minmax[2]) {
    const uint32_t bins = bins_in < 256u ? bins_in : 256u;  // TensorAnalyzer.cpp:73
    std::memset(hist, 0, 256 * sizeof(uint32_t));
    moments[0] = moments[1] = moments[2] = moments[3] = 0.f;
    minmax[0] = minmax[1] = 0.f;
    if (!data || n == 0) return;
    constexpr int T = 256;  // block size of the reference launch (:303)
    float rmin[T], rmax[T], rsum[T];
    for (int t = 0; t < T; ++t) {  // pass 1, :86-95
        float lo = 1e37f, hi = -1e37f, sum = 0.f;
        for (size_t i = t; i < n; i += T) {
            float x = load_as_float(data, i, dtype);
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
            sum += x;
        }
        rmin[t] = lo;
        rmax[t] = hi;
        rsum[t] = sum;
    }
    for (int s = T / 2; s > 0; s >>= 1)  // :102-109
        for (int t = 0; t < s; ++t) {
            rmin[t] = fminf(rmin[t], rmin[t + s]);
            rmax[t] = fmaxf(rmax[t], rmax[t + s]);
            rsum[t] += rsum[t + s];
        }
    const float vmin = rmin[0], vmax = rmax[0];
    const float mean = rsum[0] / (float)n;
    const float range = vmax - vmin;
    const float scale = range > 1e-9f ? ((float)bins - 1.0f) / range : 0.0f;  // :120

    float a2[T], a3[T], a4[T];
    for (int t = 0; t < T; ++t) {  // pass 2, :127-143
        float m2 = 0.f, m3 = 0.f, m4 = 0.f;
        for (size_t i = t; i < n; i += T) {
            float x = load_as_float(data, i, dtype);
            if (range > 1e-9f) {
                int b = (int)((x - vmin) * scale);
                b = std::max(0, std::min(b, (int)(bins - 1)));
                hist[b]++;
            } else if (bins > 0) {
                hist[0]++;
            }
            float d = x - mean;
            float d2 = d * d;
            m2 += d2;
            m3 += d2 * d;
            m4 += d2 * d2;
        }
        a2[t] = m2;
        a3[t] = m3;
        a4[t] = m4;
    }
    for (int s = T / 2; s > 0; s >>= 1)  // :151-158
        for (int t = 0; t < s; ++t) {
            a2[t] += a2[t + s];
            a3[t] += a3[t + s];
            a4[t] += a4[t + s];
        }
    const float M2 = a2[0] / (float)n, M3 = a3[0] / (float)n, M4 = a4[0] / (float)n;
    float skew = 0.f, kurt = 0.f;
    if (M2 > 1e-9f) {  // :173-177
        float sd = sqrtf(M2);
        skew = M3 / (M2 * sd);
        kurt = M4 / (M2 * M2);
    }
    moments[0] = mean;
    moments[1] = M2;
    moments[2] = skew;
    moments[3] = kurt;
    minmax[0] = vmin;
    minmax[1] = vmax;
}

int orc_build_clusters(size_t n, const char* const* names, const float* fps, int* cluster_id,
                       int* anchor_index) {
    auto category_of = [](const std::string& nm) -> std::string {  // TensorAnalyzer.cpp:455-460
        if (nm.rfind("optimizer.exp_avg_sq::", 0) == 0) return "exp_avg_sq";
        if (nm.rfind("optimizer.exp_avg::", 0) == 0) return "exp_avg";
        if (nm.rfind("master_weights::", 0) == 0) return "master_weights";
        return "model_state";
    };
    std::map<std::string, std::vector<size_t>> by_cat;
    for (size_t i = 0; i < n; ++i) {
        by_cat[category_of(names[i])].push_back(i);
        cluster_id[i] = -1;
    }
    struct UF {  // :468-479
        std::vector<int> p, r;
        explicit UF(int m) : p(m), r(m, 0) { std::iota(p.begin(), p.end(), 0); }
        int find(int x) { return p[x] == x ? x : p[x] = find(p[x]); }
        void unite(int a, int b) {
            a = find(a);
            b = find(b);
            if (a == b) return;
            if (r[a] < r[b]) std::swap(a, b);
            p[b] = a;
            if (r[a] == r[b]) ++r[a];
        }
    };
    int next_id = 0;
    for (const auto& kv : by_cat) {
        const std::vector<size_t>& idx = kv.second;
        const int m = (int)idx.size();
        if (m == 0) continue;
        auto F = [&](int a, int d) -> double { return (double)fps[idx[a] * 5 + d]; };
        double mu[5] = {}, sd[5] = {};
        for (int a = 0; a < m; ++a)
            for (int d = 0; d < 5; ++d) mu[d] += F(a, d);
        for (int d = 0; d < 5; ++d) mu[d] /= m;
        for (int a = 0; a < m; ++a)
            for (int d = 0; d < 5; ++d) {
                double df = F(a, d) - mu[d];
                sd[d] += df * df;
            }
        for (int d = 0; d < 5; ++d) sd[d] = (sd[d] / m < 1e-30) ? 1.0 : std::sqrt(sd[d] / m);
        auto dist = [&](int a, int b) -> double {
            double s = 0;
            for (int d = 0; d < 5; ++d) {
                double df = (F(a, d) - F(b, d)) / sd[d];
                s += df * df;
            }
            return std::sqrt(s);
        };
        std::vector<double> all;
        all.reserve((size_t)m * (m - 1) / 2);
        for (int a = 0; a < m; ++a)
            for (int b = a + 1; b < m; ++b) all.push_back(dist(a, b));
        double thr = 0.0;
        if (!all.empty()) {
            std::sort(all.begin(), all.end());
            thr = all[all.size() / 4];  // lower quartile, :532
        }
        UF uf(m);
        for (int a = 0; a < m; ++a)
            for (int b = a + 1; b < m; ++b)
                if (dist(a, b) < thr) uf.unite(a, b);
        std::map<int, std::vector<int>> groups;
        for (int a = 0; a < m; ++a) groups[uf.find(a)].push_back(a);
        for (const auto& g : groups) {
            if (g.second.size() >= 2) {
                anchor_index[next_id] = (int)idx[g.second[0]];
                for (int local : g.second) cluster_id[idx[local]] = next_id;
                ++next_id;
            }
        }
    }
    return next_id;
}

int orc_compress_and_save(size_t n, const char* const* names, const void* const* data,
                          const uint64_t* num_elements, const uint8_t* dtypes, const int32_t* cluster_id,
                          int n_clusters, const char* const* anchor_names, int rank, const char* out_dir,
                          int repair_tables, int n_threads) {
    namespace fs = std::filesystem;
    const std::string out(out_dir);
    std::error_code ec;
    fs::create_directories(out, ec);
    fs::create_directories(out + "/mantissa", ec);
    fs::create_directories(out + "/tables", ec);
    if (n == 0) return 0;  // src/ANSCompressor.cpp:1026-1029: nothing written

    struct Work {
        size_t idx;
        size_t bytes;
        bool anchor, single;
        int cid;
    };
    std::vector<Work> work;  // :1056-1078
    std::unordered_map<int, bool> seen;
    for (size_t i = 0; i < n; ++i) {
        if (!data[i] || num_elements[i] == 0) continue;
        int cid = cluster_id ? cluster_id[i] : -1;
        if (cid == INT32_MIN) cid = -1;
        const bool single = cid == -1;
        bool anchor = false;
        if (!single && !seen[cid]) {
            seen[cid] = true;
            anchor = true;
        }
        work.push_back({i, (size_t)num_elements[i] * orc_elem_size(dtypes[i]), anchor, single, cid});
    }

    struct Table {
        uint32_t nf[256], cf[257], xm[256];
    };
    struct Result {
        bool valid = false, owns = false;
        std::string anchor;
        Table table;
        orc_lane_header lanes[256];
        std::vector<uint8_t> payload, sidecar;
        uint32_t spe = 0;
    };
    std::vector<Result> res(work.size());
    std::unordered_map<int, Table> cluster_tables;
    const int nt = clamp_threads(n_threads);

    // Owners first so members always find their anchor's table (the reference
    // reaches the same tables through a wait loop, :1250-1258).
    for (int phase = 0; phase < 2; ++phase) {
        for (size_t w = 0; w < work.size(); ++w) {
            const Work& it = work[w];
            const bool owns = it.anchor || it.single;
            if ((phase == 0) != owns) continue;
            if (it.bytes == 0) continue;  // unknown dtype, :1133
            Result& r = res[w];
            const int dt = dtypes[it.idx];
            const uint32_t es = orc_elem_size(dt), spe = orc_sidecar_per_elem(dt);
            const uint8_t* src = (const uint8_t*)data[it.idx];
            std::vector<uint8_t> masked;
            const uint8_t* codec_in = src;
            if (spe) {
                masked.resize(it.bytes);
                r.sidecar.resize((size_t)num_elements[it.idx] * spe);
                orc_split(src, num_elements[it.idx], es, spe, masked.data(), r.sidecar.data());
                codec_in = masked.data();
            }
            r.spe = spe;
            if (owns) {
                uint32_t h[256];
                orc_byte_histogram(codec_in, it.bytes, h);
                const bool full = !it.single;  // :1239
                if (full && repair_tables)
                    orc_normalize_repaired(h, 1, r.table.nf, r.table.cf, r.table.xm);
                else
                    orc_normalize(h, full, r.table.nf, r.table.cf, r.table.xm);
                if (!it.single) cluster_tables[it.cid] = r.table;
            } else {
                auto f = cluster_tables.find(it.cid);
                if (f == cluster_tables.end()) continue;  // anchor skipped: the reference would hang
                r.table = f->second;
                if (it.cid >= 0 && it.cid < n_clusters && anchor_names && anchor_names[it.cid])
                    r.anchor = anchor_names[it.cid];  // :1259-1261
            }
            r.owns = owns;
            const size_t cap = std::max(((it.bytes + 255) / 256) * 2 * 256, it.bytes);
            r.payload.resize(cap);
            int raw = 0;
            size_t sz = orc_compress_tensor(codec_in, it.bytes, r.table.nf, r.table.cf, r.table.xm, r.lanes,
                                            r.payload.data(), &raw, nt);
            r.payload.resize(sz);
            r.valid = true;
        }
    }

    const uint32_t rank_u = (uint32_t)(rank < 0 ? 0 : rank);
    const std::string tag = "rank_" + std::to_string(rank < 0 ? 0 : rank);
    size_t n_valid = 0, n_side = 0, n_tab = 0;
    for (auto& r : res) {
        n_valid += r.valid;
        n_side += r.valid && r.spe > 0;
        n_tab += r.valid && r.owns;
    }
    {  // states file, :751-816
        std::ofstream f(out + "/" + tag + "_states.ansc", std::ios::binary | std::ios::trunc);
        if (!f) return -1;
        put(f, (uint32_t)0x414E5343u);
        put(f, (uint32_t)2u);
        put(f, rank_u);
        put(f, (uint32_t)n_valid);
        uint64_t off = 0;
        for (size_t w = 0; w < work.size(); ++w) {
            const Result& r = res[w];
            if (!r.valid) continue;
            const Work& it = work[w];
            put_name(f, names[it.idx]);
            bool is_raw = r.lanes[0].byte_count == (uint32_t)it.bytes;  // :787-789
            for (int t = 1; t < 256 && is_raw; ++t) is_raw &= r.lanes[t].byte_count == 0;
            put(f, (uint8_t)dtypes[it.idx]);
            put(f, (uint8_t)(is_raw ? 1 : 0));
            put(f, (uint8_t)(r.owns ? 1 : 0));
            const uint8_t pad5[5] = {};
            f.write((const char*)pad5, 5);
            put(f, (uint64_t)it.bytes);
            put(f, (uint64_t)num_elements[it.idx]);
            put(f, off);
            put(f, (uint64_t)r.payload.size());
            put_name(f, r.anchor);
            f.write((const char*)r.lanes, sizeof(r.lanes));
            off += r.payload.size();
        }
        for (const Result& r : res)
            if (r.valid) f.write((const char*)r.payload.data(), (std::streamsize)r.payload.size());
    }
    {  // mantissa file, :839-887
        std::ofstream f(out + "/mantissa/" + tag + "_mantissa.mant", std::ios::binary | std::ios::trunc);
        if (!f) return -1;
        put(f, (uint32_t)0x4D414E54u);
        put(f, (uint32_t)2u);
        put(f, rank_u);
        put(f, (uint32_t)n_side);
        uint64_t off = 0;
        for (size_t w = 0; w < work.size(); ++w) {
            const Result& r = res[w];
            if (!r.valid || r.spe == 0) continue;
            const Work& it = work[w];
            put_name(f, names[it.idx]);
            put(f, (uint8_t)dtypes[it.idx]);
            put(f, (uint8_t)r.spe);
            const uint8_t pad6[6] = {};
            f.write((const char*)pad6, 6);
            put(f, (uint64_t)num_elements[it.idx]);
            put(f, off);
            put(f, (uint64_t)r.sidecar.size());
            off += r.sidecar.size();
        }
        for (const Result& r : res)
            if (r.valid && r.spe) f.write((const char*)r.sidecar.data(), (std::streamsize)r.sidecar.size());
    }
    {  // tables file, :903-931
        std::ofstream f(out + "/tables/" + tag + "_tables.dict", std::ios::binary | std::ios::trunc);
        if (!f) return -1;
        put(f, (uint32_t)0x44494354u);
        put(f, (uint32_t)1u);
        put(f, rank_u);
        put(f, (uint32_t)n_tab);
        for (size_t w = 0; w < work.size(); ++w) {
            const Result& r = res[w];
            if (!r.valid || !r.owns) continue;
            put_name(f, names[work[w].idx]);
            f.write((const char*)r.table.nf, 256 * 4);
            f.write((const char*)r.table.cf, 257 * 4);
        }
    }
    return 0;
}

static int parse_states(const std::vector<uint8_t>& buf, std::vector<FileEntry>& out, size_t& data_base) {
    if (buf.size() < 16) return -11;
    uint32_t magic, ver, rk, cnt;
    std::memcpy(&magic, &buf[0], 4);
    std::memcpy(&ver, &buf[4], 4);
    std::memcpy(&rk, &buf[8], 4);
    std::memcpy(&cnt, &buf[12], 4);
    if (magic != 0x414E5343u || ver != 2) return -11;
    constexpr size_t E = 4648;
    if (buf.size() < 16 + (size_t)cnt * E) return -11;
    out.resize(cnt);
    for (uint32_t i = 0; i < cnt; ++i) {
        const uint8_t* p = &buf[16 + (size_t)i * E];
        FileEntry& e = out[i];
        e.name = cstr256(p);
        e.dtype = p[256];
        e.is_raw = p[257];
        e.owns = p[258];
        std::memcpy(&e.original_bytes, p + 264, 8);
        std::memcpy(&e.num_elements, p + 272, 8);
        std::memcpy(&e.data_offset, p + 280, 8);
        std::memcpy(&e.data_size, p + 288, 8);
        e.anchor = cstr256(p + 296);
        std::memcpy(e.lanes, p + 552, sizeof(e.lanes));
    }
    data_base = 16 + (size_t)cnt * E;
    return 0;
}

int64_t orc_list_tensors(const char* dir, int rank, char* names_out, size_t n_cap) {
    std::vector<uint8_t> buf;
    const std::string tag = "rank_" + std::to_string(rank < 0 ? 0 : rank);
    if (!read_all(std::string(dir) + "/" + tag + "_states.ansc", buf)) return -11;
    std::vector<FileEntry> ents;
    size_t base;
    int rc = parse_states(buf, ents, base);
    if (rc) return rc;
    if (names_out)
        for (size_t i = 0; i < ents.size() && i < n_cap; ++i) {
            std::memset(names_out + i * 256, 0, 256);
            std::strncpy(names_out + i * 256, ents[i].name.c_str(), 255);
        }
    return (int64_t)ents.size();
}

int64_t orc_load_tensor(const char* dir, int rank, const char* name, uint8_t* out, size_t out_cap) {
    const std::string d(dir);
    const std::string tag = "rank_" + std::to_string(rank < 0 ? 0 : rank);
    std::vector<uint8_t> st, mt, dc;
    if (!read_all(d + "/" + tag + "_states.ansc", st)) return -11;
    if (!read_all(d + "/mantissa/" + tag + "_mantissa.mant", mt)) return -11;
    if (!read_all(d + "/tables/" + tag + "_tables.dict", dc)) return -11;
    std::vector<FileEntry> ents;
    size_t base;
    int rc = parse_states(st, ents, base);
    if (rc) return rc;
    const FileEntry* e = nullptr;
    for (const auto& x : ents)
        if (x.name == name) {
            e = &x;
            break;
        }
    if (!e) return -10;
    if (e->original_bytes > out_cap) return -12;
    if (base + e->data_offset + e->data_size > st.size()) return -11;

    // table: own name for owners, anchor_name otherwise
    const std::string key = e->owns ? e->name : e->anchor;
    if (dc.size() < 16) return -11;
    uint32_t ntab;
    std::memcpy(&ntab, &dc[12], 4);
    const uint32_t *nf = nullptr, *cf = nullptr;
    std::vector<uint32_t> tbl(513);
    for (uint32_t i = 0; i < ntab; ++i) {
        const size_t o = 16 + (size_t)i * 2308;
        if (o + 2308 > dc.size()) return -11;
        if (cstr256(&dc[o]) == key) {
            std::memcpy(tbl.data(), &dc[o + 256], 513 * 4);
            nf = tbl.data();
            cf = tbl.data() + 256;
            break;
        }
    }
    if (!nf && !e->is_raw) return -11;
    std::vector<uint8_t> masked(e->original_bytes);
    rc = orc_decode_tensor(&st[base + e->data_offset], e->data_size, e->lanes, e->is_raw, nf ? nf : tbl.data(),
                           cf ? cf : tbl.data() + 256, e->original_bytes, masked.data(), 0);
    if (rc) return rc;

    const uint32_t es = orc_elem_size(e->dtype), spe = orc_sidecar_per_elem(e->dtype);
    if (spe == 0) {
        std::memcpy(out, masked.data(), masked.size());
        return (int64_t)masked.size();
    }
    if (mt.size() < 16) return -11;
    uint32_t nm;
    std::memcpy(&nm, &mt[12], 4);
    const size_t mbase = 16 + (size_t)nm * 288;
    for (uint32_t i = 0; i < nm; ++i) {
        const size_t o = 16 + (size_t)i * 288;
        if (o + 288 > mt.size()) return -11;
        if (cstr256(&mt[o]) == e->name) {
            uint64_t doff, dsz;
            std::memcpy(&doff, &mt[o + 272], 8);
            std::memcpy(&dsz, &mt[o + 280], 8);
            if (mbase + doff + dsz > mt.size() || dsz != e->num_elements * spe) return -11;
            orc_merge(masked.data(), &mt[mbase + doff], e->num_elements, es, spe, out);
            return (int64_t)masked.size();
        }
    }
    return -11;
}

int orc_roundtrip_timed(size_t n, const void* const* data, const uint64_t* num_elements, const uint8_t* dtypes,
                        int n_threads, double seconds_out[2], uint64_t bytes_out[3]) {
    struct Item {
        std::vector<uint8_t> payload, sidecar;
        orc_lane_header lanes[256];
        uint32_t nf[256], cf[257], xm[256];
        int raw = 0;
    };
    std::vector<Item> items(n);
    const int nt = clamp_threads(n_threads);
    uint64_t orig = 0, pay = 0, side = 0;
    int bad = 0;
    auto now = [] {
#ifdef _OPENMP
        return omp_get_wtime();
#else
        return (double)clock() / CLOCKS_PER_SEC;
#endif
    };
    const double t0 = now();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt) reduction(+ : orig, pay, side)
    for (long i = 0; i < (long)n; ++i) {
        Item& it = items[i];
        const int dt = dtypes[i];
        const uint32_t es = orc_elem_size(dt), spe = orc_sidecar_per_elem(dt);
        const size_t B = (size_t)num_elements[i] * es;
        const uint8_t* src = (const uint8_t*)data[i];
        std::vector<uint8_t> masked;
        const uint8_t* in = src;
        if (spe) {
            masked.resize(B);
            it.sidecar.resize((size_t)num_elements[i] * spe);
            orc_split(src, num_elements[i], es, spe, masked.data(), it.sidecar.data());
            in = masked.data();
        }
        uint32_t h[256];
        orc_byte_histogram(in, B, h);
        orc_normalize(h, 0, it.nf, it.cf, it.xm);
        it.payload.resize(std::max(((B + 255) / 256) * 2 * 256, B));
        size_t sz = orc_compress_tensor(in, B, it.nf, it.cf, it.xm, it.lanes, it.payload.data(), &it.raw, 1);
        it.payload.resize(sz);
        orig += B;
        pay += sz;
        side += it.sidecar.size();
    }
    const double t1 = now();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt) reduction(+ : bad)
    for (long i = 0; i < (long)n; ++i) {
        Item& it = items[i];
        const int dt = dtypes[i];
        const uint32_t es = orc_elem_size(dt), spe = orc_sidecar_per_elem(dt);
        const size_t B = (size_t)num_elements[i] * es;
        std::vector<uint8_t> masked(B), out(B);
        int rc = orc_decode_tensor(it.payload.data(), it.payload.size(), it.lanes, it.raw, it.nf, it.cf, B,
                                   masked.data(), 1);
        if (spe)
            orc_merge(masked.data(), it.sidecar.data(), num_elements[i], es, spe, out.data());
        else
            out.swap(masked);
        if (rc != 0 || std::memcmp(out.data(), data[i], B) != 0) bad += 1;
    }
    const double t2 = now();
    seconds_out[0] = t1 - t0;
    seconds_out[1] = t2 - t1;
    bytes_out[0] = orig;
    bytes_out[1] = pay;
    bytes_out[2] = side;
    return bad ? -1 : 0;
}

}  // extern "C"
