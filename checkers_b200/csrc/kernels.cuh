// kernels.cuh -- device code of the checkpoint-compression path (sm_100a).
//
// One header so the same source is compiled twice: by nvcc into the shipped
// library, and by g++ behind a single-thread block emulator in the CPU test
// suite (CHK_CPU_EMULATION), where it is compared against the oracle without
// a GPU.  The emulated build is a test of the index arithmetic only; the
// library has no CPU path.
//
// Reference behaviour each kernel reproduces (paths inside the Checkers tree):
//   split_hist_kernel / split_kernel   src/ANSCompressor.cpp:258-279 (+ :109-126 fused)
//   byte_histogram_kernel              src/ANSCompressor.cpp:109-126
//   rans_encode_kernel                 src/ANSCompressor.cpp:154-211
//   lane_scan_kernel, tensor_scan_kernel, compact_kernel
//                                      src/ANSCompressor.cpp:647-651, :225-238, :686-713
//   rans_decode_kernel                 inverse of :154-211 (the reference ships no decoder)
//   tensor_stats_kernel                src/TensorAnalyzer.cpp:64-198
#pragma once
#include <stdint.h>

namespace chk {

constexpr uint32_t kLanes = 256;
constexpr uint32_t kScaleBits = 12;
constexpr uint32_t kM = 1u << kScaleBits;
constexpr uint32_t kL = 1u << 23;

// Entries of the decoder's short slot table, and whether a table (by its frequency of symbol 0) can use it:
// see the decode section of rans_kernels.cuh.
constexpr uint32_t kZsEntries = 2176;
__host__ __device__ inline bool zero_skip_fits(uint32_t f0) { return (f0 < 2048u ? f0 : 2048u) + kZsEntries >= kM + 1u; }

enum : uint32_t {
    kFlagNeedHist = 1u,   // this tensor owns a table: count its bytes
    kFlagAligned = 2u,    // tensor, sidecar slice and decode target allow 16-byte vectors
    kFlagRaw = 4u,        // payload is the masked tensor itself (passthrough rule)
    kFlagZeroSkip = 16u,  // symbol 0 owns so many slots of the tensor's table that the short decode table fits
    kFlagHotBins = 8u,    // an 8-bit tensor whose bytes take few values (a sign/exponent plane): count in the spread bins
};

enum : uint32_t {
    kErrEndState = 2u,         // a decoded lane did not end in state 2^23
    kErrEndPointer = 4u,       // a decoded lane did not consume exactly byte_count bytes
};

// One work item (a registered tensor that is neither null nor empty).
struct TensorDesc {
    const uint8_t* src;             // tensor bytes to compress (borrowed)
    uint8_t* dst;                   // where decompression writes the tensor (borrowed)
    unsigned long long n_bytes;     // num_elements * elem_size
    unsigned long long sidecar_off; // start of this tensor's low bytes in the sidecar section
    unsigned long long scratch_off; // start of this tensor's 256 lane regions in encode scratch
    unsigned long long payload_off; // start of this tensor's payload in the data section
    uint32_t es;                    // element size in bytes
    uint32_t spe;                   // low bytes per element that bypass the codec
    uint32_t table_idx;             // which frequency table encodes/decodes it
    uint32_t chunk_stride;          // bytes of scratch per lane (multiple of 32)
    uint32_t flags;
    uint32_t pad_;
};

// On-disk lane header (include/checkers/ANSCompressor.hpp:79-84).
struct LaneHeader {
    uint32_t final_state;
    uint32_t byte_count;
    uint32_t buf_offset;
    uint32_t pad;
};

// Encode table entry for one symbol.  x / freq is done as a multiply-high:
// with s = ceil(log2 freq) and rcp = ceil(2^(31+s) / freq), floor(x / freq) ==
// umulhi(x, rcp) >> (s - 1) for every x < 2^31 (the error term rcp*freq - 2^(31+s)
// is below freq <= 2^s, so x * err < 2^(31+s)).  freq == 1 uses rcp = 2^32-1,
// which yields x - 1, and folds the missing 4095 into `bias`.
// The new state is x + q * cmpl + bias with cmpl = 4096 - freq, bias = cum_freq.
// This is the layout in global memory; an encode team packs its table into
// 8-byte entries in shared memory (see EncSmem).  freq == 0 marks a symbol that
// is not in the table.
struct EncEntry {
    uint32_t rcp;
    uint32_t freq_shift;  // freq[0:16) | shift[16:32)
    uint32_t bias;
    uint32_t cmpl;
};

#ifdef CHK_CPU_EMULATION
#define CHK_SHARED static
#define CHK_DYN_SMEM(p) \
    unsigned char* p = (unsigned char*)(((uintptr_t)emu::g_dyn_smem.data() + 127) & ~(uintptr_t)127)
#else
#define CHK_SHARED __shared__
#define CHK_DYN_SMEM(p)                                            \
    extern __shared__ __align__(128) unsigned char chk_dyn_smem_[]; \
    unsigned char* p = chk_dyn_smem_
#endif

__device__ __forceinline__ uint4 ld_global_v4(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// ------------------------------------------------------------------ split + histogram
#ifndef CHK_SPLIT_TILE
#define CHK_SPLIT_TILE 32768
#endif
constexpr uint32_t kSplitTileBytes = CHK_SPLIT_TILE;
constexpr int kSplitLoads = kSplitTileBytes / (256 * 16);  // 16-byte loads per thread and tile

// Count one byte value in this warp's private bins.
__device__ __forceinline__ void bin_add(uint32_t* wh, uint32_t b) { atomicAdd(&wh[b], 1u); }

// Sign-and-exponent bytes take only a handful of values, so a warp's 32 lanes
// would pile onto the same few counters.  They are counted in a second set of
// bins kept in kHotCopies copies (a lane uses copy lane % kHotCopies), laid out
// so that the values that occur together -- neighbouring exponents, either
// sign -- and the copies all fall into different shared-memory banks:
//   slot(b) = 2 * (b & 127) + (b >> 7)      neighbours 2 apart, the sign 1 apart
//   copy c starts kHotStride = 264 (= 8 mod 32) counters after copy c - 1
constexpr uint32_t kHotCopies = 4;
constexpr uint32_t kHotStride = 264;
constexpr uint32_t kHotWords = kHotCopies * kHotStride;
__device__ __forceinline__ uint32_t hot_slot(uint32_t b) { return ((b & 127u) << 1) | (b >> 7); }
__device__ __forceinline__ void bin_add_hot(uint32_t* hot_copy, uint32_t b) { atomicAdd(&hot_copy[hot_slot(b)], 1u); }

// One byte at tensor offset `off`: low bytes go to the sidecar, the rest are counted.
__device__ __forceinline__ void split_one_byte(const TensorDesc& d, unsigned long long off, uint8_t* sidecar,
                                               uint32_t* wh, bool count) {
    const uint8_t v = d.src[off];
    const uint32_t j = (uint32_t)(off % d.es);
    if (j < d.spe) {
        if (sidecar) sidecar[d.sidecar_off + (off / d.es) * d.spe + j] = v;
    } else if (count) {
        bin_add(wh, v);
    }
}

// Fused row-1 + row-2 pass over all tensors of a batch: writes each tensor's
// packed low bytes straight into its slice of the sidecar section and counts
// the bytes the codec will see, except the zeroed ones (num_elements*spe are
// added to bin 0 where the tables are built).  The masked copy is never
// materialised.  With sidecar == nullptr the pass only counts.
// Tiles are handed to CTAs in contiguous ranges so a CTA mostly stays inside
// one tensor and merges its bins into global memory once per tensor.
__global__ void __launch_bounds__(256) split_hist_kernel(const TensorDesc* __restrict__ descs,
                                                         const uint32_t* __restrict__ tile_start,
                                                         uint32_t n_tensors, uint32_t tile_base,
                                                         uint32_t total_tiles, uint8_t* __restrict__ sidecar,
                                                         uint32_t* __restrict__ hist) {
    CHK_SHARED uint32_t wh[8][256];
    CHK_SHARED uint32_t hot[8][kHotWords];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (uint32_t i = tid; i < 8 * 256; i += 256) (&wh[0][0])[i] = 0;
    for (uint32_t i = tid; i < 8 * kHotWords; i += 256) (&hot[0][0])[i] = 0;
    __syncthreads();

    // `descs`, `tile_start` and `hist` point at the first tensor of this launch's range;
    // tile_start holds running totals over the whole batch, tile_base = tile_start[0]
    const uint32_t t0 = tile_base + (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = tile_base + (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;

    // tensor holding tile t0: last index with tile_start[i] <= t0
    uint32_t lo = 0, hi = n_tensors;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (tile_start[mid] <= t0) lo = mid; else hi = mid;
    }
    uint32_t cur = lo;

    auto flush = [&](uint32_t tensor) {
        __syncthreads();
        uint32_t s = 0;
        const uint32_t hs = hot_slot(tid);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            s += wh[w][tid];
            wh[w][tid] = 0;
#pragma unroll
            for (uint32_t c = 0; c < kHotCopies; ++c) {
                s += hot[w][c * kHotStride + hs];
                hot[w][c * kHotStride + hs] = 0;
            }
        }
        if (s && (descs[tensor].flags & kFlagNeedHist)) atomicAdd(&hist[(size_t)tensor * 256 + tid], s);
        __syncthreads();
    };

    for (uint32_t tile = t0; tile < t1; ++tile) {
        while (tile >= tile_start[cur + 1]) {
            flush(cur);
            ++cur;
        }
        const TensorDesc d = descs[cur];
        const unsigned long long base = (unsigned long long)(tile - tile_start[cur]) * kSplitTileBytes;
        const uint32_t nb = (uint32_t)((d.n_bytes - base) < kSplitTileBytes ? (d.n_bytes - base) : kSplitTileBytes);
        const bool count = (d.flags & kFlagNeedHist) != 0;
        if (!count && !sidecar) continue;  // nothing to do for a tensor that borrows its table
        uint32_t* mine = wh[warp];
        uint32_t* mine_hot = hot[warp] + (lane % kHotCopies) * kHotStride;

        if ((d.flags & kFlagAligned) && (d.es == 4 || d.es == 2) && d.spe * 2 == d.es) {
            const uint32_t nvec = nb >> 4;
            // a whole tile (kSplitLoads independent 16-byte loads per thread) is in flight before any of it is used
            const uint32_t iters = (nvec + 255) >> 8;
            for (uint32_t it0 = 0; it0 < iters; it0 += kSplitLoads) {
                uint4 q[kSplitLoads];
                bool ok[kSplitLoads];
#pragma unroll
                for (int u = 0; u < kSplitLoads; ++u) {
                    const uint32_t v = (it0 + u) * 256 + tid;
                    ok[u] = v < nvec;
                    q[u] = make_uint4(0, 0, 0, 0);
                    if (ok[u]) q[u] = ld_global_v4(d.src + base + (size_t)v * 16);
                }
#pragma unroll
                for (int u = 0; u < kSplitLoads; ++u) {
                    if (!ok[u]) continue;
                    const uint32_t v = (it0 + u) * 256 + tid;
                    const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
                    uint2 s2;
                    if (d.es == 4) {
                        s2.x = __byte_perm(w[0], w[1], 0x5410);
                        s2.y = __byte_perm(w[2], w[3], 0x5410);
                    } else {
                        s2.x = __byte_perm(w[0], w[1], 0x6420);
                        s2.y = __byte_perm(w[2], w[3], 0x6420);
                    }
                    if (sidecar) *reinterpret_cast<uint2*>(sidecar + d.sidecar_off + ((base + (size_t)v * 16) >> 1)) = s2;
                    if (count) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (d.es == 4)
                                bin_add(mine, (w[k] >> 16) & 0xFF);
                            else
                                bin_add_hot(mine_hot, (w[k] >> 8) & 0xFF);
                            bin_add_hot(mine_hot, w[k] >> 24);
                        }
                    }
                }
            }
            for (uint32_t i = (nvec << 4) + tid; i < nb; i += 256) split_one_byte(d, base + i, sidecar, mine, count);
        } else if ((d.flags & kFlagAligned) && d.spe == 0) {
            const uint32_t nvec = nb >> 4;
            if (count) {
                for (uint32_t v = tid; v < nvec; v += 256) {
                    const uint4 q = ld_global_v4(d.src + base + (size_t)v * 16);
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                    if (d.flags & kFlagHotBins) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            bin_add_hot(mine_hot, w[k] & 0xFF);
                            bin_add_hot(mine_hot, (w[k] >> 8) & 0xFF);
                            bin_add_hot(mine_hot, (w[k] >> 16) & 0xFF);
                            bin_add_hot(mine_hot, w[k] >> 24);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            bin_add(mine, w[k] & 0xFF);
                            bin_add(mine, (w[k] >> 8) & 0xFF);
                            bin_add(mine, (w[k] >> 16) & 0xFF);
                            bin_add(mine, w[k] >> 24);
                        }
                    }
                }
                for (uint32_t i = (nvec << 4) + tid; i < nb; i += 256) bin_add(mine, d.src[base + i]);
            }
        } else {
            for (uint32_t i = tid; i < nb; i += 256) split_one_byte(d, base + i, sidecar, mine, count);
        }
    }
    flush(cur);
}

// Stand-alone row 1: masked copy + packed low bytes of one tensor.
__global__ void __launch_bounds__(256) split_kernel(const uint8_t* __restrict__ src, unsigned long long n_bytes,
                                                    uint32_t es, uint32_t spe, uint8_t* __restrict__ masked,
                                                    uint8_t* __restrict__ sidecar, uint32_t vector_ok) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    const unsigned long long gid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long body = 0;
    if (vector_ok && spe * 2 == es && (es == 4 || es == 2)) {
        const unsigned long long nvec = n_bytes >> 4;
        body = nvec << 4;
        for (unsigned long long v = gid; v < nvec; v += stride) {
            const uint4 q = ld_global_v4(src + v * 16);
            uint4 m;
            uint2 s;
            if (es == 4) {
                m = make_uint4(q.x & 0xFFFF0000u, q.y & 0xFFFF0000u, q.z & 0xFFFF0000u, q.w & 0xFFFF0000u);
                s.x = __byte_perm(q.x, q.y, 0x5410);
                s.y = __byte_perm(q.z, q.w, 0x5410);
            } else {
                m = make_uint4(q.x & 0xFF00FF00u, q.y & 0xFF00FF00u, q.z & 0xFF00FF00u, q.w & 0xFF00FF00u);
                s.x = __byte_perm(q.x, q.y, 0x6420);
                s.y = __byte_perm(q.z, q.w, 0x6420);
            }
            *reinterpret_cast<uint4*>(masked + v * 16) = m;
            *reinterpret_cast<uint2*>(sidecar + v * 8) = s;
        }
    }
    for (unsigned long long i = body + gid; i < n_bytes; i += stride) {
        const uint32_t j = (uint32_t)(i % es);
        const uint8_t v = src[i];
        if (j < spe) {
            masked[i] = 0;
            sidecar[(i / es) * spe + j] = v;
        } else {
            masked[i] = v;
        }
    }
}

// Stand-alone inverse of row 1: tensor = masked | low bytes (include/checkers/ANSCompressor.hpp:170).
// The restore path does this inside the decode kernel; this stage exists for the per-stage sweep.
__global__ void __launch_bounds__(256) merge_kernel(const uint8_t* __restrict__ masked, const uint8_t* __restrict__ sidecar,
                                                    unsigned long long n_bytes, uint32_t es, uint32_t spe,
                                                    uint8_t* __restrict__ out, uint32_t vector_ok) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    const unsigned long long gid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long body = 0;
    if (vector_ok && spe * 2 == es && (es == 4 || es == 2)) {
        const unsigned long long nvec = n_bytes >> 4;
        body = nvec << 4;
        for (unsigned long long v = gid; v < nvec; v += stride) {
            const uint4 m = ld_global_v4(masked + v * 16);
            const uint2 s = *reinterpret_cast<const uint2*>(sidecar + v * 8);
            uint4 o;
            if (es == 4) {
                o = make_uint4(m.x | (s.x & 0xFFFFu), m.y | (s.x >> 16), m.z | (s.y & 0xFFFFu), m.w | (s.y >> 16));
            } else {
                o = make_uint4(m.x | __byte_perm(s.x, 0u, 0x4140), m.y | __byte_perm(s.x, 0u, 0x4342),
                               m.z | __byte_perm(s.y, 0u, 0x4140), m.w | __byte_perm(s.y, 0u, 0x4342));
            }
            *reinterpret_cast<uint4*>(out + v * 16) = o;
        }
    }
    for (unsigned long long i = body + gid; i < n_bytes; i += stride) {
        const uint32_t j = (uint32_t)(i % es);
        out[i] = j < spe ? sidecar[(i / es) * spe + j] : masked[i];
    }
}

// Stand-alone row 2: 256-bin histogram of a byte buffer (hist must start at zero).
__global__ void __launch_bounds__(256) byte_histogram_kernel(const uint8_t* __restrict__ data,
                                                             unsigned long long n_bytes,
                                                             uint32_t* __restrict__ hist) {
    CHK_SHARED uint32_t wh[8][256];
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid; i < 8 * 256; i += 256) (&wh[0][0])[i] = 0;
    __syncthreads();
    uint32_t* mine = wh[warp];
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    const unsigned long long gid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long body = 0;
    if ((reinterpret_cast<uintptr_t>(data) & 15) == 0) {
        const unsigned long long nvec = n_bytes >> 4;
        body = nvec << 4;
        for (unsigned long long v = gid; v < nvec; v += stride) {
            const uint4 q = ld_global_v4(data + v * 16);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                bin_add(mine, w[k] & 0xFF);
                bin_add(mine, (w[k] >> 8) & 0xFF);
                bin_add(mine, (w[k] >> 16) & 0xFF);
                bin_add(mine, w[k] >> 24);
            }
        }
    }
    for (unsigned long long i = body + gid; i < n_bytes; i += stride) bin_add(mine, data[i]);
    __syncthreads();
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += wh[w][tid];
    if (s) atomicAdd(&hist[tid], s);
}

}  // namespace chk

#include "rans_kernels.cuh"
#include "table_kernels.cuh"

namespace chk {

// ------------------------------------------------------------------ statistics
__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    const uint32_t sign = (h >> 15) << 31;
    uint32_t e = (h >> 10) & 31u, m = h & 1023u;
    uint32_t bits;
    if (e == 31u) {
        bits = sign | 0x7F800000u | (m << 13);
    } else if (e == 0u) {
        if (m == 0u) {
            bits = sign;
        } else {
            int sh = 0;
            while (!(m & 1024u)) {
                m <<= 1;
                ++sh;
            }
            bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
        }
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    return __uint_as_float(bits);
}

__device__ __forceinline__ float load_value(const void* p, unsigned long long i, uint32_t dtype) {
    switch (dtype) {
        case 0: return reinterpret_cast<const float*>(p)[i];
        case 1: return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p)[i] << 16);
        case 2: return half_bits_to_float(reinterpret_cast<const uint16_t*>(p)[i]);
        case 3: return (float)reinterpret_cast<const int8_t*>(p)[i];
        case 4: return (float)reinterpret_cast<const int32_t*>(p)[i];
        default: return 0.0f;
    }
}

struct StatsDesc {
    const void* ptr;
    unsigned long long n;
    uint32_t dtype;
    uint32_t bins;
};
struct StatsOut {
    uint32_t hist[256];
    float moments[4];  // mean, variance, skewness, kurtosis
    float minmax[2];
    float fingerprint[5];  // mean, variance, skewness, kurtosis, max - min
    float pad_;
};

template <int DT>
__device__ __forceinline__ float load_value_t(const void* p, unsigned long long i) {
    if (DT == 0) return reinterpret_cast<const float*>(p)[i];
    if (DT == 1) return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p)[i] << 16);
    if (DT == 2) return half_bits_to_float(reinterpret_cast<const uint16_t*>(p)[i]);
    if (DT == 3) return (float)reinterpret_cast<const int8_t*>(p)[i];
    return (float)reinterpret_cast<const int32_t*>(p)[i];
}

constexpr int kStatsAhead = 8;  // loads a thread has in flight before it uses the first

// Value histogram bin (src/TensorAnalyzer.cpp:139-146): float arithmetic, nothing fused.
__device__ __forceinline__ int stats_bin(float x, float vmin, float scale, int bins, bool wide) {
    if (!wide) return 0;
    int b = (int)__fmul_rn(__fsub_rn(x, vmin), scale);
    return max(0, min(b, bins - 1));
}

// Counts go to the warp's private bins, and equal consecutive bins of a thread are
// added in one go: a skewed tensor (second moments: nearly everything in bin 0)
// would otherwise serialise 32 lanes on one counter.
struct BinRun {
    int cur = -1;
    uint32_t run = 0;
    __device__ __forceinline__ void add(uint32_t* wh, int b) {
        if (b == cur) {
            ++run;
        } else {
            if (run) atomicAdd(&wh[cur], run);
            cur = b;
            run = 1;
        }
    }
    __device__ __forceinline__ void flush(uint32_t* wh) {
        if (run) atomicAdd(&wh[cur], run);
        cur = -1;
        run = 0;
    }
};

// The two passes of one tensor in the reference's order: thread t takes elements
// t, t+256, ... one after the other (kStatsAhead of them are loaded before the first
// is used; the order of the arithmetic is unchanged).
template <int DT>
__device__ __forceinline__ void stats_pass1(const void* p, unsigned long long n, uint32_t t, float& lo, float& hi,
                                            float& sum) {
    unsigned long long i = t;
    for (; i + (unsigned long long)(kStatsAhead - 1) * 256 < n; i += (unsigned long long)kStatsAhead * 256) {
        float v[kStatsAhead];
#pragma unroll
        for (int k = 0; k < kStatsAhead; ++k) v[k] = load_value_t<DT>(p, i + (unsigned long long)k * 256);
#pragma unroll
        for (int k = 0; k < kStatsAhead; ++k) {
            lo = fminf(lo, v[k]);
            hi = fmaxf(hi, v[k]);
            sum = __fadd_rn(sum, v[k]);
        }
    }
    for (; i < n; i += 256) {
        const float x = load_value_t<DT>(p, i);
        lo = fminf(lo, x);
        hi = fmaxf(hi, x);
        sum = __fadd_rn(sum, x);
    }
}

template <int DT>
__device__ __forceinline__ void stats_pass2(const void* p, unsigned long long n, uint32_t t, float vmin, float mean,
                                            float scale, int bins, bool wide, uint32_t* wh, float& m2, float& m3,
                                            float& m4) {
    BinRun br;
    auto one = [&](float x) {
        if (bins > 0) br.add(wh, stats_bin(x, vmin, scale, bins, wide));
        const float dd = __fsub_rn(x, mean);
        const float d2 = __fmul_rn(dd, dd);
        m2 = __fadd_rn(m2, d2);
        m3 = __fadd_rn(m3, __fmul_rn(d2, dd));
        m4 = __fadd_rn(m4, __fmul_rn(d2, d2));
    };
    unsigned long long i = t;
    for (; i + (unsigned long long)(kStatsAhead - 1) * 256 < n; i += (unsigned long long)kStatsAhead * 256) {
        float v[kStatsAhead];
#pragma unroll
        for (int k = 0; k < kStatsAhead; ++k) v[k] = load_value_t<DT>(p, i + (unsigned long long)k * 256);
#pragma unroll
        for (int k = 0; k < kStatsAhead; ++k) one(v[k]);
    }
    for (; i < n; i += 256) one(load_value_t<DT>(p, i));
    br.flush(wh);
}

// One CTA per tensor, 256 threads, two passes, all in float and in the
// reference's order: thread t accumulates elements t, t+256, ... one after the
// other, the 256 partials are combined by the same halving tree, and no
// multiply-add is fused, so the results are reproducible bit for bit.
__global__ void __launch_bounds__(256) tensor_stats_kernel(const StatsDesc* __restrict__ descs,
                                                           StatsOut* __restrict__ outs, uint32_t n_tensors) {
    CHK_SHARED float ra[256], rb[256], rc[256];
    CHK_SHARED uint32_t s_hist[8 * 256];
    CHK_SHARED float s_min, s_max, s_mean;
    const uint32_t t = threadIdx.x;
    uint32_t* const wh = s_hist + (t >> 5) * 256;
    for (uint32_t ti = blockIdx.x; ti < n_tensors; ti += gridDim.x) {
        const StatsDesc d = descs[ti];
        StatsOut& o = outs[ti];
        const uint32_t bins = d.bins < 256u ? d.bins : 256u;
        if (!d.ptr || d.n == 0 || d.dtype > 4u) continue;
        for (uint32_t k = t; k < 8 * 256; k += 256) s_hist[k] = 0;

        float lo = 1e37f, hi = -1e37f, sum = 0.0f;
        switch (d.dtype) {
            case 0: stats_pass1<0>(d.ptr, d.n, t, lo, hi, sum); break;
            case 1: stats_pass1<1>(d.ptr, d.n, t, lo, hi, sum); break;
            case 2: stats_pass1<2>(d.ptr, d.n, t, lo, hi, sum); break;
            case 3: stats_pass1<3>(d.ptr, d.n, t, lo, hi, sum); break;
            default: stats_pass1<4>(d.ptr, d.n, t, lo, hi, sum); break;
        }
        ra[t] = lo;
        rb[t] = hi;
        rc[t] = sum;
        __syncthreads();
        for (uint32_t s = 128; s > 0; s >>= 1) {
            if (t < s) {
                ra[t] = fminf(ra[t], ra[t + s]);
                rb[t] = fmaxf(rb[t], rb[t + s]);
                rc[t] = __fadd_rn(rc[t], rc[t + s]);
            }
            __syncthreads();
        }
        if (t == 0) {
            s_min = ra[0];
            s_max = rb[0];
            s_mean = __fdiv_rn(rc[0], (float)d.n);
        }
        __syncthreads();
        const float vmin = s_min, mean = s_mean;
        const float range = __fsub_rn(s_max, vmin);
        const bool wide = range > 1e-9f;
        const float scale = wide ? __fdiv_rn(__fsub_rn((float)bins, 1.0f), range) : 0.0f;

        float m2 = 0.0f, m3 = 0.0f, m4 = 0.0f;
        switch (d.dtype) {
            case 0: stats_pass2<0>(d.ptr, d.n, t, vmin, mean, scale, (int)bins, wide, wh, m2, m3, m4); break;
            case 1: stats_pass2<1>(d.ptr, d.n, t, vmin, mean, scale, (int)bins, wide, wh, m2, m3, m4); break;
            case 2: stats_pass2<2>(d.ptr, d.n, t, vmin, mean, scale, (int)bins, wide, wh, m2, m3, m4); break;
            case 3: stats_pass2<3>(d.ptr, d.n, t, vmin, mean, scale, (int)bins, wide, wh, m2, m3, m4); break;
            default: stats_pass2<4>(d.ptr, d.n, t, vmin, mean, scale, (int)bins, wide, wh, m2, m3, m4); break;
        }
        __syncthreads();
        ra[t] = m2;
        rb[t] = m3;
        rc[t] = m4;
        __syncthreads();
        for (uint32_t s = 128; s > 0; s >>= 1) {
            if (t < s) {
                ra[t] = __fadd_rn(ra[t], ra[t + s]);
                rb[t] = __fadd_rn(rb[t], rb[t + s]);
                rc[t] = __fadd_rn(rc[t], rc[t + s]);
            }
            __syncthreads();
        }
        {
            uint32_t cnt = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) cnt += s_hist[w * 256 + t];
            o.hist[t] = t < bins ? cnt : 0u;
        }
        if (t == 0) {
            const float nf = (float)d.n;
            const float M2 = __fdiv_rn(ra[0], nf), M3 = __fdiv_rn(rb[0], nf), M4 = __fdiv_rn(rc[0], nf);
            float skew = 0.0f, kurt = 0.0f;
            if (M2 > 1e-9f) {
                const float sd = __fsqrt_rn(M2);
                skew = __fdiv_rn(M3, __fmul_rn(M2, sd));
                kurt = __fdiv_rn(M4, __fmul_rn(M2, M2));
            }
            o.moments[0] = mean;
            o.moments[1] = M2;
            o.moments[2] = skew;
            o.moments[3] = kurt;
            o.minmax[0] = vmin;
            o.minmax[1] = s_max;
            o.fingerprint[0] = mean;
            o.fingerprint[1] = M2;
            o.fingerprint[2] = skew;
            o.fingerprint[3] = kurt;
            o.fingerprint[4] = __fsub_rn(s_max, vmin);
        }
        __syncthreads();
    }
}

}  // namespace chk

#include "stats_kernels.cuh"
#include "plane_kernels.cuh"
#include "study_kernels.cuh"
