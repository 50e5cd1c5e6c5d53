// table_kernels.cuh -- histogram -> 12-bit frequency table on the device.
//
// normalize_tables_kernel is ANSCompressor::normalize_histogram
// (src/ANSCompressor.cpp:416-503 in the Checkers tree) for a whole batch of
// tables, one CTA of 256 threads (one per symbol) per table, followed by what
// build_enc_entries (tables.hpp) derives from the result.  With it the
// histograms never leave the device and the compress pipeline needs no host
// step between counting and encoding.
//
// The reference hands out (or takes back) rounding slots in the order
// std::sort leaves the symbols in when sorted by the fractional part of their
// ideal share.  When slots are handed out only the SET of the first `rem`
// symbols matters, and that set does not depend on the order of equal
// fractions unless a group of equal fractions straddles position `rem`: each
// thread counts the fractions above and not below its own and decides for
// itself.  Only the straddling case, and the case where slots are taken back
// (which walks the order from its end, skipping symbols that hold one slot),
// need the order itself; one thread then runs sort_replica -- the library's
// algorithm restated move for move -- and applies the reference's loops.
#pragma once
#include "sort_replica.hpp"

namespace chk {

enum : uint32_t {
    kTableFullAlphabet = 1u,  // every symbol gets at least one slot (tables shared by a cluster)
    kTableRepair = 2u,        // repeat the take-back pass until the sum is 4096 (opt-in deviation)
};

// Which work item owns table t and how it is built.
struct TableJob {
    uint32_t owner;  // index of the owning tensor in the batch (histogram row)
    uint32_t flags;  // kTable*
};

struct NormSmem {
    FracKey keys[256];
    double frac[256];
    uint32_t slots[256];
    uint32_t warp_a[8], warp_b[8];
    unsigned long long warp_c[8];
    uint32_t n_keys, assigned, need_sort;
    unsigned long long total;
};

// Sums over the 256 threads of a CTA (all threads get the result).
__device__ __forceinline__ uint32_t block_sum256(uint32_t v, uint32_t* warp_part) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();  // warp_part may still be read from a previous use
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += warp_part[w];
    return s;
}
__device__ __forceinline__ unsigned long long block_sum256_u64(unsigned long long v, unsigned long long* warp_part) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long s = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += warp_part[w];
    return s;
}
// Exclusive prefix sum over the 256 threads; *total_out receives the sum.
__device__ __forceinline__ uint32_t block_scan256(uint32_t v, uint32_t* warp_part, uint32_t* total_out) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_part[warp] = inc;
    __syncthreads();
    uint32_t before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        if ((uint32_t)w < warp) before += warp_part[w];
        total += warp_part[w];
    }
    *total_out = total;
    return before + inc - v;
}

// The encode entry of one symbol (same arithmetic as build_enc_entries in tables.hpp).
__device__ __forceinline__ EncEntry make_enc_entry(uint32_t f, uint32_t c) {
    EncEntry e;
    e.rcp = e.freq_shift = e.bias = e.cmpl = 0;
    if (f == 1) {
        e.rcp = 0xFFFFFFFFu;
        e.freq_shift = 1u;
        e.bias = c + (kM - 1);
        e.cmpl = kM - 1;
    } else if (f > 1) {
        uint32_t sh = 0;
        while ((1u << sh) < f) ++sh;
        const unsigned long long num = 1ull << (31 + sh);
        e.rcp = (uint32_t)((num + f - 1) / f);
        e.freq_shift = f | ((sh - 1) << 16);
        e.bias = c;
        e.cmpl = kM - f;
    }
    return e;
}

// hist: [batch tensors][256] counts of the codec-input bytes EXCEPT the zeroed low bytes
// (split_hist_kernel's output); the kernel adds those to bin 0 from the descriptor.
// Outputs for table t (t counts from the first table of this launch): freq[t][256],
// cum[t][257], enc[t][256], sums[t] (4096 for a decodable table).
__global__ void __launch_bounds__(256) normalize_tables_kernel(const TableJob* __restrict__ jobs,
                                                               const TensorDesc* __restrict__ descs,
                                                               const uint32_t* __restrict__ hist,
                                                               EncEntry* __restrict__ enc, uint32_t* __restrict__ freq,
                                                               uint32_t* __restrict__ cum, uint32_t* __restrict__ sums,
                                                               uint32_t n_tables) {
    CHK_SHARED NormSmem sm;
    const uint32_t s = threadIdx.x;
    for (uint32_t t = blockIdx.x; t < n_tables; t += gridDim.x) {
        const TableJob job = jobs[t];
        const TensorDesc d = descs[job.owner];
        const bool full = (job.flags & kTableFullAlphabet) != 0;
        uint32_t h = hist[(size_t)job.owner * 256 + s];
        if (s == 0 && d.es) h += (uint32_t)(d.n_bytes / d.es * d.spe);  // the zeroed low bytes are codec input too
        const unsigned long long total = block_sum256_u64(h, sm.warp_c);
        const uint32_t distinct = block_sum256(h ? 1u : 0u, sm.warp_a);
        uint32_t slot = 0;
        if ((full ? 256u : distinct) == 0) {
            slot = s == 0 ? kM : 0u;  // empty input: all mass on symbol 0 (:432-441)
        } else {
            const bool present = full || h != 0;
            const uint32_t hc = h > 1u ? h : 1u;
            if (present) {
                const uint32_t v = total ? (uint32_t)(((unsigned long long)hc * kM) / total) : 0u;
                slot = v ? v : 1u;
            }
            const double exact = total ? ((double)hc * (double)kM / (double)total) : 1.0;
            const double fr = exact - (double)(int)exact;
            const uint32_t assigned = block_sum256(slot, sm.warp_a);
            const uint32_t n_keys = block_sum256(present ? 1u : 0u, sm.warp_b);
            bool need_sort = assigned > kM;
            if (assigned < kM) {
                const uint32_t rem = kM - assigned;
                if (rem >= n_keys) {
                    slot += present ? 1u : 0u;
                } else {
                    __syncthreads();
                    sm.frac[s] = present ? fr : -1.0;  // real fractions are never negative
                    __syncthreads();
                    uint32_t greater = 0, not_less = 0;
                    for (uint32_t k = 0; k < 256; ++k) {
                        const double o = sm.frac[k];
                        greater += o > fr;
                        not_less += o >= fr;
                    }
                    const bool in = present && not_less <= rem;    // among the first rem whatever the tie order
                    const bool out = !present || greater >= rem;   // behind them whatever the tie order
                    need_sort = block_sum256((!in && !out) ? 1u : 0u, sm.warp_a) != 0;
                    if (!need_sort) slot += in ? 1u : 0u;
                }
            }
            if (need_sort) {
                // keys in symbol order, exactly the vector the reference sorts
                uint32_t n_tot;
                const uint32_t pos = block_scan256(present ? 1u : 0u, sm.warp_a, &n_tot);
                __syncthreads();
                sm.slots[s] = slot;
                if (present) {
                    FracKey key;
                    key.frac = fr;
                    key.sym = (int32_t)s;
                    key.pad_ = 0;
                    sm.keys[pos] = key;
                }
                __syncthreads();
                if (s == 0) {
                    sort_replica(sm.keys, (int)n_tot);
                    if (assigned < kM) {
                        uint32_t rem = kM - assigned;
                        for (uint32_t k = 0; k < n_tot && rem; ++k, --rem) sm.slots[sm.keys[k].sym]++;
                    } else {
                        uint32_t rem = assigned - kM;
                        for (;;) {
                            const uint32_t before = rem;
                            for (int k = (int)n_tot - 1; k >= 0 && rem; --k)
                                if (sm.slots[sm.keys[k].sym] > 1) {
                                    sm.slots[sm.keys[k].sym]--;
                                    --rem;
                                }
                            if (!(job.flags & kTableRepair) || rem == 0 || rem == before) break;
                        }
                    }
                }
                __syncthreads();
                slot = sm.slots[s];
            }
        }
        uint32_t sum;
        const uint32_t c = block_scan256(slot, sm.warp_b, &sum);
        freq[(size_t)t * 256 + s] = slot;
        cum[(size_t)t * 257 + s] = c;
        if (s == 255) {
            cum[(size_t)t * 257 + 256] = c + slot;
            sums[t] = sum;
        }
        enc[(size_t)t * 256 + s] = make_enc_entry(slot, c);
        __syncthreads();
    }
}

}  // namespace chk
