// tables.hpp -- host side of the entropy model: histogram -> 12-bit frequency
// table, and the per-symbol encode entries the kernels consume.
//
// normalize_histogram reproduces ANSCompressor::normalize_histogram
// (src/ANSCompressor.cpp:416-503 in the Checkers tree) including its use of
// std::sort on the fractional parts: the sort is unstable, equal fractions are
// common, and the resulting order decides which symbols receive the rounding
// remainder, so the same library call on the same input order is part of the
// bitstream contract.  That is why this step stays on the host.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <functional>
#include <vector>

#include "kernels.cuh"

namespace chk {

struct FreqTable {
    uint32_t norm_freq[256];
    uint32_t cum_freq[257];
    uint32_t sum;  // 4096 for a decodable table
};

// floor(num / den) for num < 2^44, den < 2^40: a double estimate (off by at most one) put right
// with one multiplication, instead of a 64-bit division per symbol.
inline uint32_t floor_div(uint64_t num, uint64_t den, double inv_den) {
    uint64_t q = (uint64_t)((double)num * inv_den);
    if (q * den > num) --q;
    else if ((q + 1) * den <= num) ++q;
    return (uint32_t)q;
}

// `repair` = false is the reference behaviour (a single decrement pass when the
// minimum-one-slot rule over-assigns, which can leave the sum above 4096 for
// full-alphabet tables of low-entropy data).  `repair` = true repeats the pass
// until the sum is 4096; it is an opt-in deviation that keeps shared tables
// decodable.
inline void normalize_histogram(const uint32_t hist[256], bool ensure_full_alphabet, bool repair, FreqTable& out) {
    std::memset(&out, 0, sizeof(out));
    uint64_t total = 0;
    int distinct = 0;
    for (int s = 0; s < 256; ++s) {
        total += hist[s];
        if (hist[s]) ++distinct;
    }
    if ((ensure_full_alphabet ? 256 : distinct) == 0) {
        out.norm_freq[0] = kM;
        for (int s = 1; s <= 256; ++s) out.cum_freq[s] = kM;
        out.sum = kM;
        return;
    }
    uint32_t slots[256] = {};
    uint32_t assigned = 0;
    const double inv_total = total ? 1.0 / (double)total : 0.0;
    for (int s = 0; s < 256; ++s) {
        if (!ensure_full_alphabet && hist[s] == 0) continue;
        uint32_t v = total ? floor_div((uint64_t)std::max(hist[s], 1u) * kM, total, inv_total) : 0u;
        slots[s] = v ? v : 1u;
        assigned += slots[s];
    }
    struct Key {
        int sym;
        double frac;
    };
    Key keys[256];
    size_t n_keys = 0;
    for (int s = 0; s < 256; ++s) {
        if (!slots[s]) continue;
        const double exact = total ? ((double)std::max(hist[s], 1u) * kM / (double)total) : 1.0;
        keys[n_keys++] = {s, exact - (double)(int)exact};
    }
    // The order is only consulted when slots have to be handed out or taken back, and when they
    // are handed out only the SET of the first `rem` keys matters.  That set is the same for
    // every correct sort unless equal fractions straddle position `rem`; so it is found by
    // selection (about a fifth of the sort's cost), and the sort itself -- whose tie order is
    // part of the format -- only runs when the straddling case occurs.
    auto by_frac = [](const Key& a, const Key& b) { return a.frac > b.frac; };
    if (assigned < kM) {
        uint32_t rem = kM - assigned;
        if (rem >= n_keys) {
            for (size_t k = 0; k < n_keys; ++k) slots[keys[k].sym]++;
        } else {
            double fr[256];
            for (size_t k = 0; k < n_keys; ++k) fr[k] = keys[k].frac;
            std::nth_element(fr, fr + (rem - 1), fr + n_keys, std::greater<double>());
            const double t = fr[rem - 1];  // the rem-th largest fraction
            size_t n_ge = 0;
            for (size_t k = 0; k < n_keys; ++k) n_ge += keys[k].frac >= t;
            if (n_ge == rem) {
                for (size_t k = 0; k < n_keys; ++k)
                    if (keys[k].frac >= t) slots[keys[k].sym]++;
            } else {
                std::sort(keys, keys + n_keys, by_frac);
                for (size_t k = 0; k < n_keys && rem; ++k, --rem) slots[keys[k].sym]++;
            }
        }
    } else if (assigned > kM) {
        std::sort(keys, keys + n_keys, by_frac);
        uint32_t rem = assigned - kM;
        for (;;) {
            const uint32_t before = rem;
            for (int k = (int)n_keys - 1; k >= 0 && rem; --k)
                if (slots[keys[k].sym] > 1) {
                    slots[keys[k].sym]--;
                    --rem;
                }
            if (!repair || rem == 0 || rem == before) break;
        }
    }
    for (int s = 0; s < 256; ++s) {
        out.norm_freq[s] = slots[s];
        out.cum_freq[s + 1] = out.cum_freq[s] + slots[s];
    }
    out.sum = out.cum_freq[256];
}

// Encode entries (see EncEntry in kernels.cuh for the arithmetic they support).
inline void build_enc_entries(const FreqTable& t, EncEntry out[256]) {
    for (int s = 0; s < 256; ++s) {
        const uint32_t f = t.norm_freq[s], cum = t.cum_freq[s];
        EncEntry e{0, 0, 0, 0};
        if (f == 1) {
            e.rcp = 0xFFFFFFFFu;
            e.freq_shift = 1u;
            e.bias = cum + (kM - 1);
            e.cmpl = kM - 1;
        } else if (f > 1) {
            uint32_t sh = 0;
            while ((1u << sh) < f) ++sh;  // ceil(log2 f) >= 1
            const uint64_t num = 1ull << (31 + sh);
            e.rcp = (uint32_t)((num + f - 1) / f);
            e.freq_shift = f | ((sh - 1) << 16);
            e.bias = cum;
            e.cmpl = kM - f;
        }
        out[s] = e;
    }
}

}  // namespace chk
