// stats_kernels.cuh -- the fast variant of the tensor statistics (included by kernels.cuh).
//
// tensor_stats_kernel keeps the reference's order of floating-point additions
// (src/TensorAnalyzer.cpp:64-198 in the Checkers tree: 256 strided chains per
// tensor, combined by a halving tree), which ties one tensor to one block of 256
// threads.  The kernels here give up that order -- and nothing else -- to use the
// whole device on every tensor:
//   * tensors are cut into tiles of kStatsTileBytes; a persistent grid walks the
//     tiles of the batch with 16-byte loads, kStatsAhead of them in flight per thread;
//   * minimum, maximum and the value histogram are exact (they do not depend on
//     the order; the bin of a value is computed with the reference's float
//     operations from the exact minimum and maximum);
//   * a thread sums its share of one tile (128 to 512 values) in float; from there
//     on everything is double and combined in a fixed order (per-tile partials,
//     then one block per tensor), so results repeat from run to run on the same
//     device; mean, variance, skewness and kurtosis differ from the reference's
//     float chains by the rounding error of those chains.
#pragma once

namespace chk {

constexpr uint32_t kStatsTileBytes = 131072;

struct StatsPart1 {
    float lo, hi;
    double sum;
};
struct StatsPart2 {
    double m2, m3, m4;
};
struct StatsMid {  // what the second pass needs from the first
    float vmin, vmax, mean, scale;
};

__device__ __forceinline__ uint32_t stats_elem_size(uint32_t dtype) {
    return dtype == 0u || dtype == 4u ? 4u : (dtype == 3u ? 1u : 2u);
}

// The values held by 16 bytes of a tensor, in any order.
template <int DT, typename F>
__device__ __forceinline__ void stats_unpack(const uint4& v, F&& f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (DT == 0) {
            f(__uint_as_float(w[k]));
        } else if (DT == 1) {
            f(__uint_as_float(w[k] << 16));
            f(__uint_as_float(w[k] & 0xFFFF0000u));
        } else if (DT == 2) {
            f(half_bits_to_float((uint16_t)(w[k] & 0xFFFFu)));
            f(half_bits_to_float((uint16_t)(w[k] >> 16)));
        } else if (DT == 3) {
#pragma unroll
            for (int b = 0; b < 4; ++b) f((float)(int8_t)(w[k] >> (8 * b)));
        } else {
            f((float)(int32_t)w[k]);
        }
    }
}

// Every value of one tile to `f`: 16-byte loads where the tensor allows them.
template <int DT, typename F>
__device__ __forceinline__ void stats_tile(const uint8_t* base, uint32_t nbytes, bool aligned, uint32_t t, F&& f) {
    constexpr uint32_t es = DT == 0 || DT == 4 ? 4 : (DT == 3 ? 1 : 2);
    if (aligned) {
        const uint32_t nvec = nbytes >> 4;
        const uint4* vp = reinterpret_cast<const uint4*>(base);
        uint32_t i = t;
        for (; i + (kStatsAhead - 1) * 256u < nvec; i += kStatsAhead * 256u) {
            uint4 v[kStatsAhead];
#pragma unroll
            for (int k = 0; k < kStatsAhead; ++k) v[k] = vp[i + (uint32_t)k * 256u];
#pragma unroll
            for (int k = 0; k < kStatsAhead; ++k) stats_unpack<DT>(v[k], f);
        }
        for (; i < nvec; i += 256u) stats_unpack<DT>(vp[i], f);
        const uint32_t done = nvec << 4;
        for (uint32_t e = t; e < (nbytes - done) / es; e += 256u) f(load_value_t<DT>(base + done, e));
    } else {
        for (uint32_t e = t; e < nbytes / es; e += 256u) f(load_value_t<DT>(base, e));
    }
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// The tensor that holds tile t0: last index with tile_start[i] <= t0.
__device__ __forceinline__ uint32_t stats_tensor_of(const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                    uint32_t t0) {
    uint32_t lo = 0, hi = n_tensors;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (tile_start[mid] <= t0) lo = mid; else hi = mid;
    }
    return lo;
}

// Pass 1: per tile, minimum, maximum and sum.  tile_start[i] = tiles before tensor i (n_tensors + 1 entries).
__global__ void __launch_bounds__(256) stats_fast_pass1_kernel(const StatsDesc* __restrict__ descs,
                                                               const uint32_t* __restrict__ tile_start,
                                                               uint32_t n_tensors, uint32_t total_tiles,
                                                               StatsPart1* __restrict__ parts) {
    CHK_SHARED float s_lo[8], s_hi[8];
    CHK_SHARED double s_sum[8];
    const uint32_t t = threadIdx.x;
    const uint32_t t0 = (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;
    uint32_t cur = stats_tensor_of(tile_start, n_tensors, t0);
    for (uint32_t tile = t0; tile < t1; ++tile) {
        while (tile >= tile_start[cur + 1]) ++cur;
        const StatsDesc d = descs[cur];
        const uint32_t es = stats_elem_size(d.dtype);
        const unsigned long long off = (unsigned long long)(tile - tile_start[cur]) * kStatsTileBytes;
        const unsigned long long left = d.n * es - off;
        const uint32_t nbytes = left < kStatsTileBytes ? (uint32_t)left : kStatsTileBytes;
        const uint8_t* base = static_cast<const uint8_t*>(d.ptr) + off;
        const bool aligned = (reinterpret_cast<uintptr_t>(d.ptr) & 15u) == 0;
        float lo = 1e37f, hi = -1e37f, fsum = 0.0f;
        auto f = [&](float x) {
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
            fsum += x;
        };
        switch (d.dtype) {
            case 0: stats_tile<0>(base, nbytes, aligned, t, f); break;
            case 1: stats_tile<1>(base, nbytes, aligned, t, f); break;
            case 2: stats_tile<2>(base, nbytes, aligned, t, f); break;
            case 3: stats_tile<3>(base, nbytes, aligned, t, f); break;
            default: stats_tile<4>(base, nbytes, aligned, t, f); break;
        }
        lo = warp_min(lo);
        hi = warp_max(hi);
        const double sum = warp_sum((double)fsum);
        if ((t & 31u) == 0) {
            s_lo[t >> 5] = lo;
            s_hi[t >> 5] = hi;
            s_sum[t >> 5] = sum;
        }
        __syncthreads();
        if (t == 0) {
            StatsPart1 p{s_lo[0], s_hi[0], s_sum[0]};
            for (int w = 1; w < 8; ++w) {
                p.lo = fminf(p.lo, s_lo[w]);
                p.hi = fmaxf(p.hi, s_hi[w]);
                p.sum += s_sum[w];
            }
            parts[tile] = p;
        }
        __syncthreads();
    }
}

// One block per tensor: the tile partials of pass 1 in a fixed order -> minimum, maximum, mean, bin scale.
__global__ void __launch_bounds__(256) stats_fast_reduce1_kernel(const StatsDesc* __restrict__ descs,
                                                                 const uint32_t* __restrict__ tile_start,
                                                                 const StatsPart1* __restrict__ parts,
                                                                 StatsMid* __restrict__ mids,
                                                                 StatsOut* __restrict__ outs, uint32_t n_tensors) {
    CHK_SHARED float s_lo[8], s_hi[8];
    CHK_SHARED double s_sum[8];
    const uint32_t t = threadIdx.x, ti = blockIdx.x;
    if (ti >= n_tensors) return;
    const uint32_t a = tile_start[ti], b = tile_start[ti + 1];
    if (a == b) return;
    float lo = 1e37f, hi = -1e37f;
    double sum = 0.0;
    for (uint32_t k = a + t; k < b; k += 256u) {
        const StatsPart1 p = parts[k];
        lo = fminf(lo, p.lo);
        hi = fmaxf(hi, p.hi);
        sum += p.sum;
    }
    lo = warp_min(lo);
    hi = warp_max(hi);
    sum = warp_sum(sum);
    if ((t & 31u) == 0) {
        s_lo[t >> 5] = lo;
        s_hi[t >> 5] = hi;
        s_sum[t >> 5] = sum;
    }
    __syncthreads();
    if (t == 0) {
        for (int w = 1; w < 8; ++w) {
            lo = fminf(lo, s_lo[w]);
            hi = fmaxf(hi, s_hi[w]);
            sum += s_sum[w];
        }
        const StatsDesc d = descs[ti];
        const uint32_t bins = d.bins < 256u ? d.bins : 256u;
        const float range = __fsub_rn(hi, lo);
        StatsMid m;
        m.vmin = lo;
        m.vmax = hi;
        m.mean = (float)(sum / (double)d.n);
        m.scale = range > 1e-9f ? __fdiv_rn(__fsub_rn((float)bins, 1.0f), range) : 0.0f;
        mids[ti] = m;
        StatsOut& o = outs[ti];
        o.moments[0] = o.fingerprint[0] = m.mean;
        o.minmax[0] = lo;
        o.minmax[1] = hi;
        o.fingerprint[4] = range;
    }
}

// Pass 2: value histogram (exact) and the central power sums about the reported mean, per tile.
__global__ void __launch_bounds__(256) stats_fast_pass2_kernel(const StatsDesc* __restrict__ descs,
                                                               const uint32_t* __restrict__ tile_start,
                                                               uint32_t n_tensors, uint32_t total_tiles,
                                                               const StatsMid* __restrict__ mids,
                                                               StatsPart2* __restrict__ parts,
                                                               StatsOut* __restrict__ outs) {
    CHK_SHARED uint32_t s_hist[8 * 256];
    CHK_SHARED double s_m[3][8];
    const uint32_t t = threadIdx.x;
    uint32_t* const wh = s_hist + (t >> 5) * 256;
    const uint32_t t0 = (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;
    for (uint32_t k = t; k < 8 * 256; k += 256) s_hist[k] = 0;
    __syncthreads();
    uint32_t cur = stats_tensor_of(tile_start, n_tensors, t0);
    auto flush = [&](uint32_t ti) {  // this block's counts of tensor ti -> global, bins cleared for the next tensor
        __syncthreads();
        uint32_t cnt = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            cnt += s_hist[w * 256 + t];
            s_hist[w * 256 + t] = 0;
        }
        if (cnt) atomicAdd(&outs[ti].hist[t], cnt);
        __syncthreads();
    };
    for (uint32_t tile = t0; tile < t1; ++tile) {
        if (tile >= tile_start[cur + 1]) {
            flush(cur);
            while (tile >= tile_start[cur + 1]) ++cur;
        }
        const StatsDesc d = descs[cur];
        const StatsMid m = mids[cur];
        const int bins = (int)(d.bins < 256u ? d.bins : 256u);
        const bool wide = __fsub_rn(m.vmax, m.vmin) > 1e-9f;
        const uint32_t es = stats_elem_size(d.dtype);
        const unsigned long long off = (unsigned long long)(tile - tile_start[cur]) * kStatsTileBytes;
        const unsigned long long left = d.n * es - off;
        const uint32_t nbytes = left < kStatsTileBytes ? (uint32_t)left : kStatsTileBytes;
        const uint8_t* base = static_cast<const uint8_t*>(d.ptr) + off;
        const bool aligned = (reinterpret_cast<uintptr_t>(d.ptr) & 15u) == 0;
        const float mean = m.mean;
        float f2 = 0.0f, f3 = 0.0f, f4 = 0.0f;
        BinRun br;
        auto f = [&](float x) {
            if (bins > 0) br.add(wh, stats_bin(x, m.vmin, m.scale, bins, wide));
            const float dd = x - mean;
            const float d2 = dd * dd;
            f2 += d2;
            f3 += d2 * dd;
            f4 += d2 * d2;
        };
        switch (d.dtype) {
            case 0: stats_tile<0>(base, nbytes, aligned, t, f); break;
            case 1: stats_tile<1>(base, nbytes, aligned, t, f); break;
            case 2: stats_tile<2>(base, nbytes, aligned, t, f); break;
            case 3: stats_tile<3>(base, nbytes, aligned, t, f); break;
            default: stats_tile<4>(base, nbytes, aligned, t, f); break;
        }
        br.flush(wh);
        const double m2 = warp_sum((double)f2), m3 = warp_sum((double)f3), m4 = warp_sum((double)f4);
        if ((t & 31u) == 0) {
            s_m[0][t >> 5] = m2;
            s_m[1][t >> 5] = m3;
            s_m[2][t >> 5] = m4;
        }
        __syncthreads();
        if (t == 0) {
            StatsPart2 p{s_m[0][0], s_m[1][0], s_m[2][0]};
            for (int w = 1; w < 8; ++w) {
                p.m2 += s_m[0][w];
                p.m3 += s_m[1][w];
                p.m4 += s_m[2][w];
            }
            parts[tile] = p;
        }
        __syncthreads();
    }
    flush(cur);
}

// One block per tensor: the tile partials of pass 2 in a fixed order -> variance, skewness, kurtosis.
__global__ void __launch_bounds__(256) stats_fast_reduce2_kernel(const StatsDesc* __restrict__ descs,
                                                                 const uint32_t* __restrict__ tile_start,
                                                                 const StatsPart2* __restrict__ parts,
                                                                 StatsOut* __restrict__ outs, uint32_t n_tensors) {
    CHK_SHARED double s_m[3][8];
    const uint32_t t = threadIdx.x, ti = blockIdx.x;
    if (ti >= n_tensors) return;
    const uint32_t a = tile_start[ti], b = tile_start[ti + 1];
    if (a == b) return;
    double m2 = 0.0, m3 = 0.0, m4 = 0.0;
    for (uint32_t k = a + t; k < b; k += 256u) {
        const StatsPart2 p = parts[k];
        m2 += p.m2;
        m3 += p.m3;
        m4 += p.m4;
    }
    m2 = warp_sum(m2);
    m3 = warp_sum(m3);
    m4 = warp_sum(m4);
    if ((t & 31u) == 0) {
        s_m[0][t >> 5] = m2;
        s_m[1][t >> 5] = m3;
        s_m[2][t >> 5] = m4;
    }
    __syncthreads();
    if (t == 0) {
        for (int w = 1; w < 8; ++w) {
            m2 += s_m[0][w];
            m3 += s_m[1][w];
            m4 += s_m[2][w];
        }
        const double n = (double)descs[ti].n;
        const double M2 = m2 / n, M3 = m3 / n, M4 = m4 / n;
        const float var = (float)M2;
        float skew = 0.0f, kurt = 0.0f;
        if (var > 1e-9f) {
            skew = (float)(M3 / (M2 * sqrt(M2)));
            kurt = (float)(M4 / (M2 * M2));
        }
        StatsOut& o = outs[ti];
        o.moments[1] = o.fingerprint[1] = var;
        o.moments[2] = o.fingerprint[2] = skew;
        o.moments[3] = o.fingerprint[3] = kurt;
    }
}

}  // namespace chk
