// repair.cu -- host side of the prefix-mask Re-Pair estimator (C ABI: chk_repair_*).
//
// Drives the kernels of repair_kernels.cuh the way build_shared_grammar /
// apply_existing_grammar drive their loops in the reference
// (src/tensor_group_prefix_mask_repair.cpp:423-463 in the Checkers tree).
//
// Tie order.  The reference picks the most frequent pair by iterating a
// std::unordered_map and keeping the first entry whose count is strictly larger
// (:389-395), so among pairs with equal counts the winner is whichever the map
// yields first.  The map's order depends only on the bucket count
// (reserve(tokens.size())), the hash, and the order in which distinct keys were
// first inserted.  When the device finds more than one pair at the maximum, the
// distinct pairs are brought to the host with their first positions, inserted
// in that order into a map built exactly like the reference's, and the map is
// walked the same way; otherwise the host is not involved.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/checkers_b200.h"
#include "repair_kernels.cuh"

namespace chkrp {

struct Error {
    int code;
    std::string msg;
};
static thread_local std::string g_err;

#define RP_CUDA(call)                                                                        \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) throw Error{CHK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)}; \
    } while (0)

struct Dev {
    void* p = nullptr;
    ~Dev() {
        if (p) cudaFree(p);
    }
    template <typename T>
    T* as() const {
        return static_cast<T*>(p);
    }
    void alloc(size_t bytes) { RP_CUDA(cudaMalloc(&p, bytes ? bytes : 16)); }
};

// symbol value the reference would hold for a token id
static inline uint64_t symbol_of(uint32_t id, uint32_t masked_bits) {
    return id < kRuleBase ? ((uint64_t)id << masked_bits) : ((1ull << 63) + (uint64_t)(id - kRuleBase));
}

struct PairKey {
    uint64_t lhs, rhs;
    bool operator==(const PairKey& o) const { return lhs == o.lhs && rhs == o.rhs; }
};
struct PairKeyHash {  // same mixing as the reference's PairKeyHash (:363-371)
    size_t operator()(const PairKey& k) const {
        const size_t a = std::hash<uint64_t>{}(k.lhs), b = std::hash<uint64_t>{}(k.rhs);
        return a ^ (b + 0x9e3779b97f4a7c15ull + (a << 6u) + (a >> 2u));
    }
};

// Device working set of one call.  One instance per device is kept for the life of the process and
// only grows, so a run over many tensors does not pay an allocation per tensor.
struct Workspace {
    uint32_t n_cap = 0, capacity = 0;
    size_t raw_cap = 0;
    bool ready = false;
    Dev tok_a, tok_b, mark, run_start, keep, pos, blocks, keys, counts, first, small, tie_keys, tie_first, dump_keys,
        dump_counts, dump_first, raw;
    cudaStream_t s = nullptr;
    ~Workspace() {
        if (s) cudaStreamDestroy(s);
    }
    void release() {
        Dev* all[] = {&tok_a, &tok_b, &mark, &run_start, &keep, &pos, &blocks, &keys, &counts, &first, &small, &tie_keys,
                      &tie_first, &dump_keys, &dump_counts, &dump_first, &raw};
        for (Dev* d : all) {
            if (d->p) cudaFree(d->p);
            d->p = nullptr;
        }
    }
    void init(uint32_t n, size_t raw_bytes) {
        if (ready && n <= n_cap && raw_bytes <= raw_cap) {
            capacity = 1024;  // table sized for THIS tensor: the hash mask must match what is cleared
            while (capacity < 2ull * n) capacity <<= 1;
            return;
        }
        release();
        n_cap = n;
        raw_cap = raw_bytes;
        capacity = 1024;
        while (capacity < 2ull * n) capacity <<= 1;
        if (!s) RP_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        ready = true;
        const size_t nb = (size_t)(n ? n : 1) * 4;
        tok_a.alloc(nb);
        tok_b.alloc(nb);
        mark.alloc(nb);
        run_start.alloc(nb);
        keep.alloc(nb);
        pos.alloc(nb);
        blocks.alloc(((size_t)n / kScanBlock + 8) * 4);
        keys.alloc((size_t)capacity * 8);
        counts.alloc((size_t)capacity * 4);
        first.alloc((size_t)capacity * 4);
        small.alloc(64);
        tie_keys.alloc(64);
        tie_first.alloc(32);
        raw.alloc(raw_bytes);
    }
};

template <int OP>
static void scan(Workspace& w, const uint32_t* in, uint32_t n, uint32_t* out) {
    const uint32_t nb = (n + kScanBlock - 1) / kScanBlock;
    scan_reduce_kernel<OP><<<nb, 256, 0, w.s>>>(in, n, w.blocks.as<uint32_t>());
    scan_blocks_kernel<OP><<<1, 256, 0, w.s>>>(w.blocks.as<uint32_t>(), nb);
    scan_apply_kernel<OP><<<nb, 256, 0, w.s>>>(in, n, w.blocks.as<uint32_t>(), out);
    RP_CUDA(cudaGetLastError());
}

static uint32_t grid_for(uint32_t n) {
    const uint32_t g = (n + 255) / 256;
    return g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g);
}

// Rewrites `in` (n tokens) under rule (lhs, rhs) -> new_sym into `out`; returns the new length.
static uint32_t apply_rule(Workspace& w, const uint32_t* in, uint32_t n, uint32_t lhs, uint32_t rhs, uint32_t new_sym,
                           uint32_t* out) {
    if (n == 0) return 0;
    const uint32_t g = grid_for(n);
    if (lhs == rhs) {
        run_mark_kernel<<<g, 256, 0, w.s>>>(in, n, lhs, w.mark.as<uint32_t>());
        scan<1>(w, w.mark.as<uint32_t>(), n, w.run_start.as<uint32_t>());
    }
    rule_flags_kernel<<<g, 256, 0, w.s>>>(in, n, lhs, rhs, w.run_start.as<uint32_t>(), w.keep.as<uint32_t>());
    scan<0>(w, w.keep.as<uint32_t>(), n, w.pos.as<uint32_t>());
    rule_scatter_kernel<<<g, 256, 0, w.s>>>(in, n, lhs, rhs, new_sym, w.run_start.as<uint32_t>(),
                                            w.keep.as<uint32_t>(), w.pos.as<uint32_t>(), out);
    RP_CUDA(cudaGetLastError());
    uint32_t total = 0;  // scan_blocks leaves the grand total after the last block value
    const uint32_t nb = (n + kScanBlock - 1) / kScanBlock;
    RP_CUDA(cudaMemcpyAsync(&total, w.blocks.as<uint32_t>() + nb, 4, cudaMemcpyDeviceToHost, w.s));
    RP_CUDA(cudaStreamSynchronize(w.s));
    return total;
}

static void upload_tokens(Workspace& w, const void* h_raw, uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits) {
    if (numel == 0) return;
    RP_CUDA(cudaMemcpyAsync(w.raw.p, h_raw, numel * storage_bytes, cudaMemcpyHostToDevice, w.s));
    mask_words_kernel<<<grid_for((uint32_t)numel), 256, 0, w.s>>>(w.raw.as<uint8_t>(), numel, storage_bytes, masked_bits,
                                                                  w.tok_a.as<uint32_t>());
    RP_CUDA(cudaGetLastError());
}

static Workspace& workspace_for(int device) {
    static Workspace* per_device[64] = {};
    if (device < 0 || device >= 64) throw Error{CHK_ERR_INVALID, "device ordinal out of range"};
    if (!per_device[device]) per_device[device] = new Workspace();
    return *per_device[device];
}

static void check_args(uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits) {
    if (storage_bytes != 2 && storage_bytes != 4) throw Error{CHK_ERR_INVALID, "storage_bytes must be 2 or 4"};
    if (masked_bits > storage_bytes * 8) throw Error{CHK_ERR_INVALID, "masked_bits exceeds the word width"};
    if (storage_bytes * 8 - masked_bits > 31)
        throw Error{CHK_ERR_CAPACITY, "at least one bit of a 32-bit word must be masked (token ids are 31-bit)"};
    if (numel >= (1ull << 31)) throw Error{CHK_ERR_CAPACITY, "tensor too long for 32-bit token positions"};
}

}  // namespace chkrp

using namespace chkrp;

#define RP_BEGIN try {
#define RP_END                       \
    }                                \
    catch (const chkrp::Error& e) {  \
        chkrp::g_err = e.msg;        \
        return e.code;               \
    }                                \
    catch (const std::exception& e) {\
        chkrp::g_err = e.what();     \
        return CHK_ERR_INVALID;      \
    }                                \
    return CHK_OK;

extern "C" {

const char* chk_repair_last_error(void) { return chkrp::g_err.c_str(); }

int chk_repair_build(int device, const void* h_raw, uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits,
                     uint32_t max_rules, uint32_t* rule_lhs, uint32_t* rule_rhs, uint64_t* rule_freq,
                     uint32_t* n_rules_out, uint64_t* tokens_out, uint64_t* max_pair_frequency_out,
                     uint64_t* tie_rounds_out) {
    RP_BEGIN
    if (!h_raw && numel) throw Error{CHK_ERR_INVALID, "NULL tensor"};
    if (!n_rules_out || !tokens_out) throw Error{CHK_ERR_INVALID, "NULL output"};
    check_args(numel, storage_bytes, masked_bits);
    RP_CUDA(cudaSetDevice(device));
    Workspace& w = workspace_for(device);
    w.init((uint32_t)numel, numel * storage_bytes);
    upload_tokens(w, h_raw, numel, storage_bytes, masked_bits);
    uint32_t* cur = w.tok_a.as<uint32_t>();
    uint32_t* nxt = w.tok_b.as<uint32_t>();
    uint32_t n = (uint32_t)numel, n_rules = 0;
    uint64_t max_freq = 0, tie_rounds = 0;
    for (uint32_t r = 0; r < max_rules; ++r) {
        if (n < 2) break;
        RP_CUDA(cudaMemsetAsync(w.keys.p, 0xFF, (size_t)w.capacity * 8, w.s));
        RP_CUDA(cudaMemsetAsync(w.counts.p, 0, (size_t)w.capacity * 4, w.s));
        RP_CUDA(cudaMemsetAsync(w.first.p, 0xFF, (size_t)w.capacity * 4, w.s));
        RP_CUDA(cudaMemsetAsync(w.small.p, 0, 64, w.s));
        uint32_t* small = w.small.as<uint32_t>();  // [0] best, [1] ties, [2] overflow, [3] dump count
        pair_count_kernel<<<grid_for(n), 256, 0, w.s>>>(cur, n, w.keys.as<unsigned long long>(), w.counts.as<uint32_t>(),
                                                        w.first.as<uint32_t>(), w.capacity - 1, small + 2);
        pair_max_kernel<<<grid_for(w.capacity), 256, 0, w.s>>>(w.counts.as<uint32_t>(), w.capacity, small);
        pair_ties_kernel<<<grid_for(w.capacity), 256, 0, w.s>>>(w.keys.as<unsigned long long>(), w.counts.as<uint32_t>(),
                                                                w.first.as<uint32_t>(), w.capacity, small,
                                                                w.tie_keys.as<unsigned long long>(),
                                                                w.tie_first.as<uint32_t>());
        RP_CUDA(cudaGetLastError());
        uint32_t h_small[4];
        unsigned long long h_tie_keys[8];
        RP_CUDA(cudaMemcpyAsync(h_small, small, 16, cudaMemcpyDeviceToHost, w.s));
        RP_CUDA(cudaMemcpyAsync(h_tie_keys, w.tie_keys.p, 64, cudaMemcpyDeviceToHost, w.s));
        RP_CUDA(cudaStreamSynchronize(w.s));
        if (h_small[2]) throw Error{CHK_ERR_CAPACITY, "pair table overflow"};
        const uint32_t best = h_small[0];
        if (best > max_freq) max_freq = best;
        if (best < 2) break;  // k_min_rule_frequency
        unsigned long long key = h_tie_keys[0];
        if (h_small[1] > 1) {
            // several pairs share the maximum: replay the reference's map to see which it meets first
            ++tie_rounds;
            if (!w.dump_keys.p) {
                w.dump_keys.alloc((size_t)w.n_cap * 8 + 8);
                w.dump_counts.alloc((size_t)w.n_cap * 4 + 4);
                w.dump_first.alloc((size_t)w.n_cap * 4 + 4);
            }
            pair_dump_kernel<<<grid_for(w.capacity), 256, 0, w.s>>>(
                w.keys.as<unsigned long long>(), w.counts.as<uint32_t>(), w.first.as<uint32_t>(), w.capacity, small + 3,
                w.dump_keys.as<unsigned long long>(), w.dump_counts.as<uint32_t>(), w.dump_first.as<uint32_t>());
            RP_CUDA(cudaGetLastError());
            uint32_t d = 0;
            RP_CUDA(cudaMemcpyAsync(&d, small + 3, 4, cudaMemcpyDeviceToHost, w.s));
            RP_CUDA(cudaStreamSynchronize(w.s));
            std::vector<unsigned long long> hk(d);
            std::vector<uint32_t> hc(d), hf(d);
            RP_CUDA(cudaMemcpy(hk.data(), w.dump_keys.p, (size_t)d * 8, cudaMemcpyDeviceToHost));
            RP_CUDA(cudaMemcpy(hc.data(), w.dump_counts.p, (size_t)d * 4, cudaMemcpyDeviceToHost));
            RP_CUDA(cudaMemcpy(hf.data(), w.dump_first.p, (size_t)d * 4, cudaMemcpyDeviceToHost));
            std::vector<uint32_t> order(d);
            for (uint32_t i = 0; i < d; ++i) order[i] = i;
            std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return hf[a] < hf[b]; });
            std::unordered_map<PairKey, size_t, PairKeyHash> counts;
            counts.reserve(n);
            std::unordered_map<PairKey, unsigned long long, PairKeyHash> back;  // symbol pair -> id key
            back.reserve(d);
            for (uint32_t i : order) {
                const PairKey pk{symbol_of((uint32_t)(hk[i] >> 32), masked_bits), symbol_of((uint32_t)hk[i], masked_bits)};
                counts[pk] = hc[i];
                back[pk] = hk[i];
            }
            size_t best_count = 0;
            PairKey best_pair{};
            for (const auto& kv : counts)
                if (kv.second > best_count) {
                    best_count = kv.second;
                    best_pair = kv.first;
                }
            key = back[best_pair];
        }
        const uint32_t lhs = (uint32_t)(key >> 32), rhs = (uint32_t)key, sym = kRuleBase + n_rules;
        const uint32_t m = apply_rule(w, cur, n, lhs, rhs, sym, nxt);
        if (m >= n) break;  // no shrink: the rule is not kept (:440-443)
        std::swap(cur, nxt);
        n = m;
        if (rule_lhs) rule_lhs[n_rules] = lhs;
        if (rule_rhs) rule_rhs[n_rules] = rhs;
        if (rule_freq) rule_freq[n_rules] = best;
        ++n_rules;
    }
    *n_rules_out = n_rules;
    *tokens_out = n;
    if (max_pair_frequency_out) *max_pair_frequency_out = max_freq;
    if (tie_rounds_out) *tie_rounds_out = tie_rounds;
    RP_END
}

int chk_repair_apply(int device, const void* h_raw, uint64_t numel, uint32_t storage_bytes, uint32_t masked_bits,
                     const uint32_t* rule_lhs, const uint32_t* rule_rhs, uint32_t n_rules, uint64_t* tokens_out) {
    RP_BEGIN
    if ((!h_raw && numel) || !tokens_out) throw Error{CHK_ERR_INVALID, "NULL argument"};
    if (n_rules && (!rule_lhs || !rule_rhs)) throw Error{CHK_ERR_INVALID, "NULL rules"};
    check_args(numel, storage_bytes, masked_bits);
    RP_CUDA(cudaSetDevice(device));
    Workspace& w = workspace_for(device);
    w.init((uint32_t)numel, numel * storage_bytes);
    upload_tokens(w, h_raw, numel, storage_bytes, masked_bits);
    uint32_t* cur = w.tok_a.as<uint32_t>();
    uint32_t* nxt = w.tok_b.as<uint32_t>();
    uint32_t n = (uint32_t)numel;
    for (uint32_t r = 0; r < n_rules; ++r) {
        n = apply_rule(w, cur, n, rule_lhs[r], rule_rhs[r], kRuleBase + r, nxt);
        std::swap(cur, nxt);
    }
    RP_CUDA(cudaStreamSynchronize(w.s));
    *tokens_out = n;
    RP_END
}

}  // extern "C"
