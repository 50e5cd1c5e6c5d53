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
    uint32_t pad_;
};

// One element of the general path (any element size, any alignment).
template <bool kMerge>
__device__ __forceinline__ void plane_one(const PlaneDesc& d, unsigned long long e, uint8_t* low, uint8_t* planes) {
    for (uint32_t j = 0; j < d.es; ++j) {
        uint8_t* side = j < d.spe ? low + d.low_off + e * d.spe + j
                                  : planes + d.plane_off + (unsigned long long)(j - d.spe) * d.plane_stride + e;
        if (kMerge) d.tensor[e * d.es + j] = *side; else *side = d.tensor[e * d.es + j];
    }
}

// tile_start[i] = tiles before tensor i (n + 1 entries); a persistent grid walks contiguous ranges of tiles.
template <bool kMerge>
__device__ __forceinline__ void plane_pass(const PlaneDesc* __restrict__ descs, const uint32_t* __restrict__ tile_start,
                                           uint32_t n_tensors, uint32_t total_tiles, uint8_t* __restrict__ low,
                                           uint8_t* __restrict__ planes) {
    const uint32_t tid = threadIdx.x;
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
        while (tile >= tile_start[cur + 1]) ++cur;
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
                            *reinterpret_cast<uint2*>(lowp + (size_t)v * 8) = l;
                            *reinterpret_cast<uint32_t*>(p2 + (size_t)v * 4) = __byte_perm(a, b, 0x5410);
                            *reinterpret_cast<uint32_t*>(p3 + (size_t)v * 4) = __byte_perm(a, b, 0x7632);
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
        for (unsigned long long e = e0 + tid; e < e1; e += 256) plane_one<kMerge>(d, e, low, planes);
    }
}

__global__ void __launch_bounds__(256) plane_split_kernel(const PlaneDesc* __restrict__ descs,
                                                          const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                          uint32_t total_tiles, uint8_t* __restrict__ low,
                                                          uint8_t* __restrict__ planes) {
    plane_pass<false>(descs, tile_start, n_tensors, total_tiles, low, planes);
}

__global__ void __launch_bounds__(256) plane_merge_kernel(const PlaneDesc* __restrict__ descs,
                                                          const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                          uint32_t total_tiles, uint8_t* __restrict__ low,
                                                          uint8_t* __restrict__ planes) {
    plane_pass<true>(descs, tile_start, n_tensors, total_tiles, low, planes);
}

}  // namespace chk
