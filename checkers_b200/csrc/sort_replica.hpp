// sort_replica.hpp -- the order std::sort produces, reproduced step by step.
//
// ANSCompressor::normalize_histogram (src/ANSCompressor.cpp:469-471 in the
// Checkers tree) orders the symbols of a table by the fractional part of their
// ideal slot count with std::sort, which is not stable: where fractions are
// equal (equal byte counts are common) the order -- and with it which symbols
// receive or give up a rounding slot -- is whatever the library's algorithm
// leaves behind.  To normalise tables on the GPU with the same result, the
// algorithm itself is restated here: the introsort of GNU libstdc++ (median of
// three to the front, unguarded Hoare partition, recursion depth 2*floor(log2 n),
// heap sort below that depth, ranges of 16 or fewer left to one final insertion
// sort), with every comparison and every move in the same sequence.  The code
// is plain C++ that compiles for the host and for the device;
// tests/test_sort_replica.py checks it against std::sort itself, ties,
// adversarial inputs and the heap-sort fallback included.
#pragma once
#include <stdint.h>

#ifndef CHK_HD
#if defined(__CUDACC__) && !defined(CHK_CPU_EMULATION)
#define CHK_HD __host__ __device__
#else
#define CHK_HD
#endif
#endif

namespace chk {

// One sortable record: a symbol and the fractional part it is ordered by
// (descending).  Equal fractions compare equal whatever the symbols are.
struct FracKey {
    double frac;
    int32_t sym;
    int32_t pad_;
};

CHK_HD inline bool frac_before(const FracKey& a, const FracKey& b) { return a.frac > b.frac; }

CHK_HD inline void sr_swap(FracKey& a, FracKey& b) {
    const FracKey t = a;
    a = b;
    b = t;
}

CHK_HD inline void sr_linear_insert(FracKey* last) {  // *last moves left until its predecessor is not after it
    const FracKey val = *last;
    FracKey* next = last - 1;
    while (frac_before(val, *next)) {
        *last = *next;
        last = next;
        --next;
    }
    *last = val;
}

CHK_HD inline void sr_insertion_sort(FracKey* first, FracKey* last) {
    if (first == last) return;
    for (FracKey* i = first + 1; i != last; ++i) {
        if (frac_before(*i, *first)) {  // new front element: shift the whole prefix right by one
            const FracKey val = *i;
            for (FracKey* p = i; p != first; --p) *p = *(p - 1);
            *first = val;
        } else {
            sr_linear_insert(i);
        }
    }
}

CHK_HD inline void sr_adjust_heap(FracKey* first, long hole, long len, FracKey value) {
    const long top = hole;
    long child = hole;
    while (child < (len - 1) / 2) {
        child = 2 * (child + 1);
        if (frac_before(first[child], first[child - 1])) --child;
        first[hole] = first[child];
        hole = child;
    }
    if ((len & 1) == 0 && child == (len - 2) / 2) {
        child = 2 * (child + 1);
        first[hole] = first[child - 1];
        hole = child - 1;
    }
    long parent = (hole - 1) / 2;  // sift the value back up
    while (hole > top && frac_before(first[parent], value)) {
        first[hole] = first[parent];
        hole = parent;
        parent = (hole - 1) / 2;
    }
    first[hole] = value;
}

// What the library falls back to when a range has used up its recursion depth.
CHK_HD inline void sr_heap_sort(FracKey* first, FracKey* last) {
    const long len = last - first;
    if (len >= 2) {
        for (long parent = (len - 2) / 2;; --parent) {
            sr_adjust_heap(first, parent, len, first[parent]);
            if (parent == 0) break;
        }
    }
    while (last - first > 1) {
        --last;
        const FracKey value = *last;
        *last = *first;
        sr_adjust_heap(first, 0, last - first, value);
    }
}

CHK_HD inline void sr_median_to_first(FracKey* result, FracKey* a, FracKey* b, FracKey* c) {
    if (frac_before(*a, *b)) {
        if (frac_before(*b, *c)) sr_swap(*result, *b);
        else if (frac_before(*a, *c)) sr_swap(*result, *c);
        else sr_swap(*result, *a);
    } else if (frac_before(*a, *c)) {
        sr_swap(*result, *a);
    } else if (frac_before(*b, *c)) {
        sr_swap(*result, *c);
    } else {
        sr_swap(*result, *b);
    }
}

CHK_HD inline FracKey* sr_partition(FracKey* first, FracKey* last, const FracKey* pivot) {
    for (;;) {
        while (frac_before(*first, *pivot)) ++first;
        --last;
        while (frac_before(*pivot, *last)) --last;
        if (!(first < last)) return first;
        sr_swap(*first, *last);
        ++first;
    }
}

// keys[0..n) into the order std::sort(keys, keys + n, by descending frac) leaves them in.
// n <= 256.  The sub-ranges the library handles by recursion are independent of one
// another, so they are kept on a small explicit stack instead.
CHK_HD inline void sort_replica(FracKey* keys, int n) {
    if (n <= 1) return;
    int lg = 0;
    while ((1 << (lg + 1)) <= n) ++lg;
    struct Range {
        int16_t first, last, depth;
    };
    Range stack[40];
    int sp = 0;
    stack[sp++] = Range{0, (int16_t)n, (int16_t)(2 * lg)};
    while (sp) {
        const Range r = stack[--sp];
        FracKey* first = keys + r.first;
        FracKey* last = keys + r.last;
        int depth = r.depth;
        while (last - first > 16) {
            if (depth == 0) {
                sr_heap_sort(first, last);
                break;
            }
            --depth;
            FracKey* mid = first + (last - first) / 2;
            sr_median_to_first(first, first + 1, mid, last - 1);
            FracKey* cut = sr_partition(first + 1, last, first);
            if (last - cut > 16) stack[sp++] = Range{(int16_t)(cut - keys), (int16_t)(last - keys), (int16_t)depth};
            last = cut;
        }
    }
    if (n > 16) {
        sr_insertion_sort(keys, keys + 16);
        for (FracKey* i = keys + 16; i != keys + n; ++i) sr_linear_insert(i);
    } else {
        sr_insertion_sort(keys, keys + n);
    }
}

}  // namespace chk
