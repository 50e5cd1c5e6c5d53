// repair_kernels.cuh -- device side of the prefix-mask Re-Pair size estimator.
//
// Reference behaviour (src/tensor_group_prefix_mask_repair.cpp in the Checkers
// tree, a single-threaded CPU tool): mask the low mantissa bits of every word
// (:328-352), then up to max_rules times count every adjacent token pair, pick
// the most frequent one (:373-401) and rewrite the sequence left to right,
// replacing non-overlapping occurrences by a new symbol (:403-421).
//
// Here tokens are 32-bit ids (masked word >> masked_bits for words, kRuleBase + r
// for rule r); a pair is the 64-bit key (lhs << 32 | rhs).
//   pair_count_kernel   open-addressing hash table of (key, count, first index);
//                       lanes of a warp that hold the same key add once
//   pair_max_kernel / pair_ties_kernel   largest count, how many keys reach it
//   rule_flags_kernel + scan kernels + rule_scatter_kernel   the rewrite as a
//                       data-parallel stream compaction (a run of equal symbols
//                       under a rule (a,a) is paired from its start, as the
//                       sequential scan does)
// Included by repair.cu and by the CPU emulator build of the test suite.
#pragma once
#include <stdint.h>

namespace chkrp {

constexpr uint32_t kRuleBase = 0x80000000u;  // ids of rule symbols start here
constexpr unsigned long long kEmptyKey = 0xFFFFFFFFFFFFFFFFull;
constexpr uint32_t kScanBlock = 1024;        // elements per block in the scan passes (256 threads x 4)

#ifdef CHK_CPU_EMULATION
#define CHKRP_SHARED static
#else
#define CHKRP_SHARED __shared__
#endif

// words: little-endian storage of the tensor (2 or 4 bytes per element) -> token ids
__global__ void __launch_bounds__(256) mask_words_kernel(const uint8_t* __restrict__ raw, unsigned long long n,
                                                         uint32_t storage_bytes, uint32_t masked_bits,
                                                         uint32_t* __restrict__ tokens) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t w;
        if (storage_bytes == 4)
            w = (uint32_t)raw[4 * i] | ((uint32_t)raw[4 * i + 1] << 8) | ((uint32_t)raw[4 * i + 2] << 16) |
                ((uint32_t)raw[4 * i + 3] << 24);
        else
            w = (uint32_t)raw[2 * i] | ((uint32_t)raw[2 * i + 1] << 8);
        tokens[i] = w >> masked_bits;
    }
}

__device__ __forceinline__ uint32_t pair_hash(unsigned long long key) {
    key ^= key >> 33;
    key *= 0xff51afd7ed558ccdull;
    key ^= key >> 33;
    key *= 0xc4ceb9fe1a85ec53ull;
    key ^= key >> 33;
    return (uint32_t)key;
}

// keys must be preset to kEmptyKey, counts to 0, first to 0xFFFFFFFF; capacity is a power of two > n.
__global__ void __launch_bounds__(256) pair_count_kernel(const uint32_t* __restrict__ tokens, uint32_t n,
                                                         unsigned long long* __restrict__ keys,
                                                         uint32_t* __restrict__ counts, uint32_t* __restrict__ first,
                                                         uint32_t capacity_mask, uint32_t* __restrict__ overflow) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t stride = gridDim.x * blockDim.x;
    const uint32_t n_pairs = n > 0 ? n - 1 : 0;
    // uniform trip count so every lane reaches the warp vote
    const uint32_t iters = (n_pairs + stride - 1) / stride;
    for (uint32_t it = 0; it < iters; ++it) {
        const uint32_t i = it * stride + blockIdx.x * blockDim.x + threadIdx.x;
        const bool ok = i < n_pairs;
        const unsigned long long key =
            ok ? (((unsigned long long)tokens[i] << 32) | tokens[i + 1]) : (kEmptyKey - 1 - lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (!ok || lane != (uint32_t)(__ffs(peers) - 1)) continue;  // one lane per distinct key of the warp
        // lowest index among the peers is this lane's (peers are in index order)
        uint32_t slot = pair_hash(key) & capacity_mask;
        bool placed = false;
        for (uint32_t probe = 0; probe <= capacity_mask; ++probe) {
            const unsigned long long prev = atomicCAS(&keys[slot], kEmptyKey, key);
            if (prev == kEmptyKey || prev == key) {
                atomicAdd(&counts[slot], (uint32_t)__popc(peers));
                atomicMin(&first[slot], i);
                placed = true;
                break;
            }
            slot = (slot + 1) & capacity_mask;
        }
        if (!placed) atomicAdd(overflow, 1u);
    }
}

// out[0] = largest count
__global__ void __launch_bounds__(256) pair_max_kernel(const uint32_t* __restrict__ counts, uint32_t capacity,
                                                       uint32_t* __restrict__ out) {
    CHKRP_SHARED uint32_t red[256];
    uint32_t m = 0;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x)
        m = counts[i] > m ? counts[i] : m;
    red[threadIdx.x] = m;
    __syncthreads();
    for (uint32_t s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s && red[threadIdx.x + s] > red[threadIdx.x]) red[threadIdx.x] = red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) atomicMax(&out[0], red[0]);
}

// out[1] = number of keys whose count equals out[0]; the first 8 of them land in tie_keys / tie_first
__global__ void __launch_bounds__(256) pair_ties_kernel(const unsigned long long* __restrict__ keys,
                                                        const uint32_t* __restrict__ counts,
                                                        const uint32_t* __restrict__ first, uint32_t capacity,
                                                        uint32_t* __restrict__ out,
                                                        unsigned long long* __restrict__ tie_keys,
                                                        uint32_t* __restrict__ tie_first) {
    const uint32_t best = out[0];
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x) {
        if (best && counts[i] == best && keys[i] != kEmptyKey) {
            const uint32_t pos = atomicAdd(&out[1], 1u);
            if (pos < 8) {
                tie_keys[pos] = keys[i];
                tie_first[pos] = first[i];
            }
        }
    }
}

// Compacts the occupied slots (key, first index) for the host-side tie break.
__global__ void __launch_bounds__(256) pair_dump_kernel(const unsigned long long* __restrict__ keys,
                                                        const uint32_t* __restrict__ counts,
                                                        const uint32_t* __restrict__ first, uint32_t capacity,
                                                        uint32_t* __restrict__ n_out,
                                                        unsigned long long* __restrict__ keys_out,
                                                        uint32_t* __restrict__ counts_out,
                                                        uint32_t* __restrict__ first_out) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x) {
        if (keys[i] != kEmptyKey) {
            const uint32_t pos = atomicAdd(n_out, 1u);
            keys_out[pos] = keys[i];
            counts_out[pos] = counts[i];
            first_out[pos] = first[i];
        }
    }
}

// ---- rule application ------------------------------------------------------------------------
// run_mark[i]: for a rule (a, a) the index just past the last non-a token at or before i (else 0);
// its running maximum is the start of the run of a's that i belongs to.
__global__ void __launch_bounds__(256) run_mark_kernel(const uint32_t* __restrict__ tokens, uint32_t n, uint32_t sym,
                                                       uint32_t* __restrict__ mark) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        mark[i] = tokens[i] != sym ? i + 1 : 0u;
}

// Generic three-pass scan over 32-bit values: op 0 = sum (exclusive result), op 1 = max (inclusive result).
template <int OP>
__device__ __forceinline__ uint32_t scan_op(uint32_t a, uint32_t b) {
    return OP == 0 ? a + b : (a > b ? a : b);
}

template <int OP>
__global__ void __launch_bounds__(256) scan_reduce_kernel(const uint32_t* __restrict__ in, uint32_t n,
                                                          uint32_t* __restrict__ block_out) {
    CHKRP_SHARED uint32_t red[256];
    const uint32_t base = blockIdx.x * kScanBlock;
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t i = base + threadIdx.x * 4 + k;
        if (i < n) acc = scan_op<OP>(acc, in[i]);
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (uint32_t s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] = scan_op<OP>(red[threadIdx.x], red[threadIdx.x + s]);
        __syncthreads();
    }
    if (threadIdx.x == 0) block_out[blockIdx.x] = red[0];
}

// one block: exclusive scan of the block totals in place; total -> block_vals[n_blocks]
template <int OP>
__global__ void __launch_bounds__(256) scan_blocks_kernel(uint32_t* __restrict__ block_vals, uint32_t n_blocks) {
    CHKRP_SHARED uint32_t part[256];
    const uint32_t per = (n_blocks + 255) / 256;
    const uint32_t lo = threadIdx.x * per < n_blocks ? threadIdx.x * per : n_blocks;
    const uint32_t hi = lo + per < n_blocks ? lo + per : n_blocks;
    uint32_t acc = 0;
    for (uint32_t i = lo; i < hi; ++i) acc = scan_op<OP>(acc, block_vals[i]);
    part[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t t = 0; t < 256; ++t) {
            const uint32_t v = part[t];
            part[t] = run;
            run = scan_op<OP>(run, v);
        }
        block_vals[n_blocks] = run;
    }
    __syncthreads();
    uint32_t run = part[threadIdx.x];
    for (uint32_t i = lo; i < hi; ++i) {
        const uint32_t v = block_vals[i];
        block_vals[i] = run;
        run = scan_op<OP>(run, v);
    }
}

// final pass: out[i] = exclusive sum (OP 0) or inclusive max (OP 1) of in[0..i]
template <int OP>
__global__ void __launch_bounds__(256) scan_apply_kernel(const uint32_t* __restrict__ in, uint32_t n,
                                                         const uint32_t* __restrict__ block_vals,
                                                         uint32_t* __restrict__ out) {
    CHKRP_SHARED uint32_t part[256];
    const uint32_t base = blockIdx.x * kScanBlock;
    uint32_t v[4];
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t i = base + threadIdx.x * 4 + k;
        v[k] = i < n ? in[i] : 0u;
        acc = scan_op<OP>(acc, v[k]);
    }
    part[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = block_vals[blockIdx.x];
        for (uint32_t t = 0; t < 256; ++t) {
            const uint32_t x = part[t];
            part[t] = run;
            run = scan_op<OP>(run, x);
        }
    }
    __syncthreads();
    uint32_t run = part[threadIdx.x];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t i = base + threadIdx.x * 4 + k;
        if (i < n) {
            if (OP == 0) {
                out[i] = run;
                run += v[k];
            } else {
                run = run > v[k] ? run : v[k];
                out[i] = run;
            }
        }
    }
}

// keep[i] = 1 unless token i is the second half of a replaced pair.  run_start is only read when lhs == rhs.
__device__ __forceinline__ bool pair_taken(const uint32_t* tokens, uint32_t n, uint32_t i, uint32_t lhs, uint32_t rhs,
                                           const uint32_t* run_start) {
    if (i + 1 >= n || tokens[i] != lhs || tokens[i + 1] != rhs) return false;
    if (lhs != rhs) return true;
    return ((i - run_start[i]) & 1u) == 0;  // pairs are formed from the start of the run
}

__global__ void __launch_bounds__(256) rule_flags_kernel(const uint32_t* __restrict__ tokens, uint32_t n, uint32_t lhs,
                                                         uint32_t rhs, const uint32_t* __restrict__ run_start,
                                                         uint32_t* __restrict__ keep) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        keep[i] = (i > 0 && pair_taken(tokens, n, i - 1, lhs, rhs, run_start)) ? 0u : 1u;
}

__global__ void __launch_bounds__(256) rule_scatter_kernel(const uint32_t* __restrict__ tokens, uint32_t n,
                                                           uint32_t lhs, uint32_t rhs, uint32_t new_sym,
                                                           const uint32_t* __restrict__ run_start,
                                                           const uint32_t* __restrict__ keep,
                                                           const uint32_t* __restrict__ pos,
                                                           uint32_t* __restrict__ out) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        if (keep[i]) out[pos[i]] = pair_taken(tokens, n, i, lhs, rhs, run_start) ? new_sym : tokens[i];
}

}  // namespace chkrp
