// study_kernels.cuh -- HyperLogLog sketches of tensors' 32-bit symbols (included by kernels.cuh).
//
// The reference's offline study (scripts/llama-3-8b/experiment_2.py:31-85 in the Checkers tree, numpy on the
// host) estimates how large a histogram SHARED by a cluster of tensors would be: one 2^14-register sketch per
// tensor, the union of a cluster = the element-wise maximum of its sketches, the cardinality from the
// registers.  Here the sketches of all tensors of a batch are taken in one pass over the data:
//   symbol   : the element's bit pattern, zero-extended to 32 bits
//   hash     : MurmurHash3 fmix32                                  (:48-53)
//   register : top 14 bits of the hash                             (:55)
//   rank     : leading zeros of ((hash << 14) | 2^13) + 1, clipped to 18   (:58-63), kept by maximum
// A block keeps a whole sketch in shared memory (2^14 words) and merges it into the tensor's global registers
// when it moves on to another tensor.  Merge and count are 16 KB of host arithmetic per sketch.
#pragma once

namespace chk {

constexpr uint32_t kHllBits = 14;
constexpr uint32_t kHllRegs = 1u << kHllBits;
constexpr uint32_t kHllTileBytes = 131072;

__device__ __forceinline__ uint32_t hll_fmix32(uint32_t h) {
    h ^= h >> 16;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    h *= 0xC2B2AE35u;
    h ^= h >> 16;
    return h;
}

__device__ __forceinline__ void hll_add(uint32_t* regs, uint32_t symbol) {
    const uint32_t h = hll_fmix32(symbol);
    const uint32_t w = (h << kHllBits) | (1u << (kHllBits - 1));
    const uint32_t lz = (uint32_t)__clz((int)w) + 1u;   // at most 19 (the guard bit), clipped to 32 - 14 as the study does
    const uint32_t rho = lz < 32u - kHllBits ? lz : 32u - kHllBits;
    uint32_t* r = regs + (h >> (32 - kHllBits));
    if (*r < rho) atomicMax(r, rho);  // most additions do not raise the register: read first
}

// descs[i].ptr / n / dtype as for the statistics; tile_start[i] = tiles of kHllTileBytes before tensor i;
// regs: n_tensors x kHllRegs words, zeroed by the caller.
__global__ void __launch_bounds__(256) hll_sketch_kernel(const StatsDesc* __restrict__ descs,
                                                         const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                         uint32_t total_tiles, uint32_t* __restrict__ regs) {
    CHK_DYN_SMEM(smem);
    uint32_t* s_regs = reinterpret_cast<uint32_t*>(smem);
    const uint32_t t = threadIdx.x;
    const uint32_t t0 = (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;
    for (uint32_t k = t; k < kHllRegs; k += 256) s_regs[k] = 0;
    __syncthreads();
    uint32_t cur = stats_tensor_of(tile_start, n_tensors, t0);
    auto flush = [&](uint32_t ti) {
        __syncthreads();
        uint32_t* g = regs + (size_t)ti * kHllRegs;
        for (uint32_t k = t; k < kHllRegs; k += 256) {
            const uint32_t v = s_regs[k];
            if (v) atomicMax(&g[k], v);
            s_regs[k] = 0;
        }
        __syncthreads();
    };
    for (uint32_t tile = t0; tile < t1; ++tile) {
        if (tile >= tile_start[cur + 1]) {
            flush(cur);
            while (tile >= tile_start[cur + 1]) ++cur;
        }
        const StatsDesc d = descs[cur];
        const uint32_t es = stats_elem_size(d.dtype);
        const unsigned long long off = (unsigned long long)(tile - tile_start[cur]) * kHllTileBytes;
        const unsigned long long left = d.n * es - off;
        const uint32_t nbytes = left < kHllTileBytes ? (uint32_t)left : kHllTileBytes;
        const uint8_t* base = static_cast<const uint8_t*>(d.ptr) + off;
        auto add_vec = [&](const uint4& v) {  // the symbols held by 16 bytes of the tensor
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (es == 4) {
                    hll_add(s_regs, w[k]);
                } else if (es == 2) {
                    hll_add(s_regs, w[k] & 0xFFFFu);
                    hll_add(s_regs, w[k] >> 16);
                } else {
#pragma unroll
                    for (int b = 0; b < 4; ++b) hll_add(s_regs, (w[k] >> (8 * b)) & 0xFFu);
                }
            }
        };
        uint32_t done = 0;
        if ((reinterpret_cast<uintptr_t>(d.ptr) & 15u) == 0) {
            const uint32_t nvec = nbytes >> 4;
            const uint4* vp = reinterpret_cast<const uint4*>(base);
            uint32_t i = t;
            for (; i + (kStatsAhead - 1) * 256u < nvec; i += kStatsAhead * 256u) {  // kStatsAhead loads in flight per thread
                uint4 v[kStatsAhead];
#pragma unroll
                for (int k = 0; k < kStatsAhead; ++k) v[k] = vp[i + (uint32_t)k * 256u];
#pragma unroll
                for (int k = 0; k < kStatsAhead; ++k) add_vec(v[k]);
            }
            for (; i < nvec; i += 256u) add_vec(vp[i]);
            done = nvec << 4;
        }
        // what is left (or everything, for a tensor that does not start on a 16-byte boundary): element by element
        for (uint32_t e = done / es + t; e < nbytes / es; e += 256) {
            const uint8_t* p = base + (size_t)e * es;
            uint32_t sym = p[0];
            if (es >= 2) sym |= (uint32_t)p[1] << 8;
            if (es == 4) sym |= ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
            hll_add(s_regs, sym);
        }
    }
    flush(cur);
}

// registers as bytes, as the host keeps them
__global__ void __launch_bounds__(256) hll_pack_kernel(const uint32_t* __restrict__ regs, uint8_t* __restrict__ out,
                                                       unsigned long long n) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = (uint8_t)regs[i];
}

}  // namespace chk

// ------------------------------------------------------------------ cost of a shared 32-bit model
// The reference's second study (scripts/llama-3-8b/experiment_2_1.py:52-75, 217-330) prices a group of tensors
// coded under ONE model over their 32-bit symbols: the group's symbol counts are quantised to a power-of-two
// scale (every symbol at least 1, the rounding drift onto the most frequent symbol) and every occurrence of a
// symbol costs log2(scale / norm[symbol]) bits.  Summed over the tensors of the group that is
// sum over the group's vocabulary of count * log2(scale / norm), so one table of symbol counts is all it needs:
//   symbol_count_kernel   open-addressing table of (symbol, count) over all tensors of the group
//   model_scan_kernel     vocabulary size, the largest count (smallest symbol among equals, as argmax over the
//                         sorted vocabulary picks it)
//   model_cost_kernel     sum of the quantised counts and of count * log2(scale / norm), per block
namespace chk {

constexpr unsigned long long kSymUsed = 1ull << 32;  // a stored key is the symbol with this bit set; 0 = free

__device__ __forceinline__ void symbol_insert(unsigned long long* keys, uint32_t* counts, uint32_t mask, uint32_t sym,
                                              uint32_t* overflow) {
    const unsigned long long key = kSymUsed | sym;
    uint32_t slot = hll_fmix32(sym) & mask;
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        unsigned long long prev = keys[slot];
        if (prev == 0ull) prev = atomicCAS(&keys[slot], 0ull, key);
        if (prev == 0ull || prev == key) {
            atomicAdd(&counts[slot], 1u);
            return;
        }
        slot = (slot + 1) & mask;
    }
    atomicAdd(overflow, 1u);
}

__global__ void __launch_bounds__(256) symbol_count_kernel(const StatsDesc* __restrict__ descs,
                                                           const uint32_t* __restrict__ tile_start, uint32_t n_tensors,
                                                           uint32_t total_tiles, unsigned long long* __restrict__ keys,
                                                           uint32_t* __restrict__ counts, uint32_t mask,
                                                           uint32_t* __restrict__ overflow) {
    const uint32_t t = threadIdx.x;
    const uint32_t t0 = (uint32_t)((unsigned long long)total_tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)total_tiles * (blockIdx.x + 1) / gridDim.x);
    if (t0 >= t1) return;
    uint32_t cur = stats_tensor_of(tile_start, n_tensors, t0);
    for (uint32_t tile = t0; tile < t1; ++tile) {
        while (tile >= tile_start[cur + 1]) ++cur;
        const StatsDesc d = descs[cur];
        const uint32_t es = stats_elem_size(d.dtype);
        const unsigned long long off = (unsigned long long)(tile - tile_start[cur]) * kHllTileBytes;
        const unsigned long long left = d.n * es - off;
        const uint32_t nbytes = left < kHllTileBytes ? (uint32_t)left : kHllTileBytes;
        const uint8_t* base = static_cast<const uint8_t*>(d.ptr) + off;
        for (uint32_t e = t; e < nbytes / es; e += 256) {
            const uint8_t* p = base + (size_t)e * es;
            uint32_t sym = p[0];
            if (es >= 2) sym |= (uint32_t)p[1] << 8;
            if (es == 4) sym |= ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
            symbol_insert(keys, counts, mask, sym, overflow);
        }
    }
}

// out[0] = vocabulary size; out[1] = largest count << 32 | (2^32 - 1 - its smallest symbol)
__global__ void __launch_bounds__(256) model_scan_kernel(const unsigned long long* __restrict__ keys,
                                                         const uint32_t* __restrict__ counts, uint32_t capacity,
                                                         unsigned long long* __restrict__ out) {
    unsigned long long used = 0, best = 0;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += stride) {
        const unsigned long long k = keys[i];
        if (!k) continue;
        ++used;
        const unsigned long long cand = ((unsigned long long)counts[i] << 32) | (0xFFFFFFFFull - (k & 0xFFFFFFFFull));
        best = cand > best ? cand : best;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        used += __shfl_xor_sync(0xffffffffu, used, m);
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, m);
        best = o > best ? o : best;
    }
    if ((threadIdx.x & 31) == 0) {
        if (used) atomicAdd(&out[0], used);
        if (best) atomicMax(&out[1], best);
    }
}

// Per block: sum of norm = max(floor(count * factor), 1) and of count * log2(scale / norm), the most frequent
// symbol left out (the host adds it with the rounding drift).  partial[2 * block], partial[2 * block + 1].
__global__ void __launch_bounds__(256) model_cost_kernel(const unsigned long long* __restrict__ keys,
                                                         const uint32_t* __restrict__ counts, uint32_t capacity,
                                                         double factor, double scale, unsigned long long skip_key,
                                                         double* __restrict__ partial) {
    CHK_SHARED double s_a[8], s_b[8];
    double norm_sum = 0.0, bits = 0.0;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += stride) {
        const unsigned long long k = keys[i];
        if (!k || k == skip_key) continue;
        const double c = (double)counts[i];
        double norm = floor(c * factor);
        norm = norm < 1.0 ? 1.0 : norm;
        norm_sum += norm;
        bits += c * log2(scale / norm);
    }
    norm_sum = warp_sum(norm_sum);
    bits = warp_sum(bits);
    if ((threadIdx.x & 31) == 0) {
        s_a[threadIdx.x >> 5] = norm_sum;
        s_b[threadIdx.x >> 5] = bits;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            norm_sum += s_a[w];
            bits += s_b[w];
        }
        partial[2 * blockIdx.x] = norm_sum;
        partial[2 * blockIdx.x + 1] = bits;
    }
}

}  // namespace chk
