// plane_kernels.cuh -- byte planes of floating-point tensors, for container version 3
// (included by kernels.cuh).
//
// Version 2 -- the reference's format (src/ANSCompressor.cpp:258-279, :393-411 in the
// Checkers tree) -- codes the bytes of a tensor that are not "low bytes" as ONE
// stream under ONE table that was counted over the whole masked tensor: the zeroed
// low bytes take half of the table's probability mass (one extra bit for every real
// symbol), and for 4-byte elements the sign/exponent byte and the top mantissa byte
// share a table although their distributions have nothing in common.  Version 3
// keeps every piece of version 2 (the 256-lane coder, the table normalisation, the
// three files and their entry layouts) and only changes WHAT is handed to it: each
// high byte of the elements becomes a byte plane of its own, coded as an
// independent 8-bit tensor with its own table; the low bytes stay raw.
//
//   plane_split_kernel   tensor -> low bytes (element-major, as in the .mant data section)
//                                  + (es - spe) planes of n bytes, plane-major
//   plane_merge_kernel   the inverse
#pragma once

namespace chk {

constexpr uint32_t kPlaneTileBytes = 32768;  // of tensor bytes

struct PlaneDesc {
    uint8_t* tensor;               // split: source; merge: destination
    unsigned long long n_elem;
    unsigned long long low_off;    // this tensor's low bytes in the low-byte section
    unsigned long long plane_off;  // its first plane in the plane section
    unsigned long long plane_stride;  // bytes from one plane to the next (>= n_elem, multiple of 32)
    uint32_t es, spe;
    uint32_t vector_ok;            // tensor, low_off and plane_off allow 16-byte vectors
    uint32_t hist_row;             // split with counting: row (256 counters) of the first plane's byte histogram
};

// Byte counters of the planes a block is working on: plane k of the current tensor in bins[k], each warp its
// own copy; the top plane (sign / exponent bytes: a handful of values) in the bank-spread copies of
// split_hist_kernel.  Null when the pass does not count.
struct PlaneBins {
    uint32_t (*wh)[8][256];   // [plane][warp][value]
    uint32_t (*hot)[kHotWords];  // [warp][copies]
};

// One element of the general path (any element size, any alignment).
template <bool kMerge>
__device__ __forceinline__ void plane_one(const PlaneDesc& d, unsigned long long e, uint8_t* low, uint8_t* planes,
                                          const PlaneBins* bins = nullptr) {
    for (uint32_t j = 0; j < d.es; ++j) {
        uint8_t* side = j < d.spe ? low + d.low_off + e * d.spe + j
                                  : planes + d.plane_off + (unsigned long long)(j - d.spe) * d.plane_stride + e;
        if (kMerge) {
            d.tensor[e * d.es + j] = *side;
        } else {
            const uint8_t v = d.tensor[e * d.es + j];
            *side = v;
            if (bins && j >= d.spe) {
                const uint32_t warp = threadIdx.x >> 5;
                if (j + 1 == d.es)
                    bin_add_hot(bins->hot[warp] + (threadIdx.x % kHotCopies) * kHotStride, v);
                else
                    bin_add(bins->wh[j - d.spe][warp], v);
            }
        }
    }
}

// tile_start[i] = tiles before tensor i (n + 1 entries); a persistent grid walks contiguous ranges of tiles.
template <bool kMerge, bool kCount = false>
__device__ __forceinline__ void plane_pass(const PlaneDesc* __restrict__ descs, const uint32_t* __restrict__ tile_start,
                                           uint32_t n_tensors, uint32_t total_tiles, uint8_t* __restrict__ low,
                                           uint8_t* __restrict__ planes, uint32_t* __restrict__ hist = nullptr,
                                           unsigned char* smem = nullptr) {
    const uint32_t tid = threadIdx.x;
    PlaneBins bins{};
    if (kCount) {  // shared memory: one set of warp-private bins (the plane below the top one) + the spread copies
        bins.wh = reinterpret_cast<uint32_t(*)[8][256]>(smem);
        bins.hot = reinterpret_cast<uint32_t(*)[kHotWords]>(smem + sizeof(uint32_t) * 8 * 256);
        for (uint32_t i = tid; i < 8 * 256 + 8 * kHotWords; i += 256) reinterpret_cast<uint32_t*>(smem)[i] = 0;
        __syncthreads();
    }
    // counters of this block for tensor ti -> its planes' rows; cleared for the next tensor
    auto flush = [&](uint32_t ti) {
        __syncthreads();
        const PlaneDesc fd = descs[ti];
        const uint32_t n_planes = fd.es - fd.spe;
        uint32_t top = 0, mid = 0;
        const uint32_t hs = hot_slot(tid);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            mid += bins.wh[0][w][tid];
            bins.wh[0][w][tid] = 0;
#pragma unroll
            for (uint32_t c = 0; c < kHotCopies; ++c) {
                top += bins.hot[w][c * kHotStride + hs];
                bins.hot[w][c * kHotStride + hs] = 0;
            }
        }
        if (top) atomicAdd(&hist[(size_t)(fd.hist_row + n_planes - 1) * 256 + tid], top);
        if (mid && n_planes > 1) atomicAdd(&hist[(size_t)fd.hist_row * 256 + tid], mid);
        __syncthreads();
    };
    const uint32_t t0 = (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;
    uint32_t lo = 0, hi = n_tensors;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (tile_start[mid] <= t0) lo = mid; else hi = mid;
    }
    uint32_t cur = lo;
    for (uint32_t tile = t0; tile < t1; ++tile) {
        if (tile >= tile_start[cur + 1]) {
            if (kCount) flush(cur);
            while (tile >= tile_start[cur + 1]) ++cur;
        }
        const PlaneDesc d = descs[cur];
        const unsigned long long base = (unsigned long long)(tile - tile_start[cur]) * kPlaneTileBytes;
        const unsigned long long total = d.n_elem * d.es;
        const uint32_t nb = (uint32_t)((total - base) < kPlaneTileBytes ? (total - base) : kPlaneTileBytes);
        uint32_t done = 0;  // bytes of this tile handled by the vector path
        if (d.vector_ok && d.spe * 2 == d.es && (d.es == 4 || d.es == 2)) {
            const uint32_t nvec = nb >> 4;
            done = nvec << 4;
            uint8_t* const lowp = low + d.low_off + (base >> 1);
            if (d.es == 4) {
                uint8_t* const p2 = planes + d.plane_off + (base >> 2);
                uint8_t* const p3 = p2 + d.plane_stride;
                for (uint32_t v0 = 0; v0 < nvec; v0 += 4 * 256) {
                    if (!kMerge) {
                        uint4 q[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v < nvec) q[u] = ld_global_v4(d.tensor + base + (size_t)v * 16);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v >= nvec) continue;
                            uint2 l;
                            l.x = __byte_perm(q[u].x, q[u].y, 0x5410);
                            l.y = __byte_perm(q[u].z, q[u].w, 0x5410);
                            const uint32_t a = __byte_perm(q[u].x, q[u].y, 0x7362);  // byte 2 of elements 0, 1, then byte 3
                            const uint32_t b = __byte_perm(q[u].z, q[u].w, 0x7362);  // the same of elements 2, 3
                            const uint32_t w2 = __byte_perm(a, b, 0x5410), w3 = __byte_perm(a, b, 0x7632);
                            *reinterpret_cast<uint2*>(lowp + (size_t)v * 8) = l;
                            *reinterpret_cast<uint32_t*>(p2 + (size_t)v * 4) = w2;
                            *reinterpret_cast<uint32_t*>(p3 + (size_t)v * 4) = w3;
                            if (kCount) {
                                uint32_t* mine = bins.wh[0][tid >> 5];
                                uint32_t* mine_hot = bins.hot[tid >> 5] + (tid % kHotCopies) * kHotStride;
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    bin_add(mine, (w2 >> (8 * k)) & 0xFFu);
                                    bin_add_hot(mine_hot, (w3 >> (8 * k)) & 0xFFu);
                                }
                            }
                        }
                    } else {
                        uint2 l[4];
                        uint32_t w2[4], w3[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v < nvec) {
                                l[u] = *reinterpret_cast<const uint2*>(lowp + (size_t)v * 8);
                                w2[u] = *reinterpret_cast<const uint32_t*>(p2 + (size_t)v * 4);
                                w3[u] = *reinterpret_cast<const uint32_t*>(p3 + (size_t)v * 4);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v >= nvec) continue;
                            const uint32_t h01 = __byte_perm(w2[u], w3[u], 0x5140);  // b2 b3 of element 0, then of element 1
                            const uint32_t h23 = __byte_perm(w2[u], w3[u], 0x7362);
                            uint4 q;
                            q.x = __byte_perm(l[u].x, h01, 0x5410);
                            q.y = __byte_perm(l[u].x, h01, 0x7632);
                            q.z = __byte_perm(l[u].y, h23, 0x5410);
                            q.w = __byte_perm(l[u].y, h23, 0x7632);
                            *reinterpret_cast<uint4*>(d.tensor + base + (size_t)v * 16) = q;
                        }
                    }
                }
            } else {
                uint8_t* const p1 = planes + d.plane_off + (base >> 1);
                for (uint32_t v0 = 0; v0 < nvec; v0 += 4 * 256) {
                    if (!kMerge) {
                        uint4 q[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v < nvec) q[u] = ld_global_v4(d.tensor + base + (size_t)v * 16);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v >= nvec) continue;
                            uint2 l, h;
                            l.x = __byte_perm(q[u].x, q[u].y, 0x6420);
                            l.y = __byte_perm(q[u].z, q[u].w, 0x6420);
                            h.x = __byte_perm(q[u].x, q[u].y, 0x7531);
                            h.y = __byte_perm(q[u].z, q[u].w, 0x7531);
                            *reinterpret_cast<uint2*>(lowp + (size_t)v * 8) = l;
                            *reinterpret_cast<uint2*>(p1 + (size_t)v * 8) = h;
                            if (kCount) {
                                uint32_t* mine_hot = bins.hot[tid >> 5] + (tid % kHotCopies) * kHotStride;
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    bin_add_hot(mine_hot, (h.x >> (8 * k)) & 0xFFu);
                                    bin_add_hot(mine_hot, (h.y >> (8 * k)) & 0xFFu);
                                }
                            }
                        }
                    } else {
                        uint2 l[4], h[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v < nvec) {
                                l[u] = *reinterpret_cast<const uint2*>(lowp + (size_t)v * 8);
                                h[u] = *reinterpret_cast<const uint2*>(p1 + (size_t)v * 8);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t v = v0 + u * 256 + tid;
                            if (v >= nvec) continue;
                            uint4 q;
                            q.x = __byte_perm(l[u].x, h[u].x, 0x5140);
                            q.y = __byte_perm(l[u].x, h[u].x, 0x7362);
                            q.z = __byte_perm(l[u].y, h[u].y, 0x5140);
                            q.w = __byte_perm(l[u].y, h[u].y, 0x7362);
                            *reinterpret_cast<uint4*>(d.tensor + base + (size_t)v * 16) = q;
                        }
                    }
                }
            }
        }
        // what the vector path left: whole elements (tiles and 16-byte groups end on element boundaries)
        const unsigned long long e0 = (base + done) / d.es, e1 = (base + nb) / d.es;
        for (unsigned long long e = e0 + tid; e < e1; e += 256) plane_one<kMerge>(d, e, low, planes, kCount ? &bins : nullptr);
    }
    if (kCount) flush(cur);
}

__global__ void __launch_bounds__(256) plane_split_kernel(const PlaneDesc* __restrict__ descs,
                                                          const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                          uint32_t total_tiles, uint8_t* __restrict__ low,
                                                          uint8_t* __restrict__ planes) {
    plane_pass<false>(descs, tile_start, n_tensors, total_tiles, low, planes);
}

// The split with the byte histogram of every plane counted in the same pass (hist: 256 counters per plane,
// zeroed by the caller): what split_hist_kernel would count if the planes were read again as 8-bit tensors.
// Element sizes with more than two high bytes are not supported here (the caller falls back).
constexpr uint32_t kPlaneCountSmem = sizeof(uint32_t) * (8 * 256 + 8 * kHotWords);
__global__ void __launch_bounds__(256) plane_split_count_kernel(const PlaneDesc* __restrict__ descs,
                                                                const uint32_t* __restrict__ tile_start,
                                                                uint32_t n_tensors, uint32_t total_tiles,
                                                                uint8_t* __restrict__ low, uint8_t* __restrict__ planes,
                                                                uint32_t* __restrict__ hist) {
    CHK_DYN_SMEM(smem);
    plane_pass<false, true>(descs, tile_start, n_tensors, total_tiles, low, planes, hist, smem);
}

__global__ void __launch_bounds__(256) plane_merge_kernel(const PlaneDesc* __restrict__ descs,
                                                          const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                          uint32_t total_tiles, uint8_t* __restrict__ low,
                                                          uint8_t* __restrict__ planes) {
    plane_pass<true>(descs, tile_start, n_tensors, total_tiles, low, planes);
}

}  // namespace chk
