// cuda_emu.hpp -- run CUDA kernel source on one CPU thread, for tests only.
//
// The library's kernels live in checkers_b200/csrc/kernels.cuh.  This header
// lets a plain g++ build include that file: every CUDA thread of a block is a
// ucontext fiber, __syncthreads() and the warp collectives yield until all
// participants arrived, and the asynchronous-copy wrappers become memcpy.  It
// exists so index arithmetic, ring buffers and barrier placement can be
// checked against the oracle without a GPU.  It is slow, single-threaded and
// never part of the shipped library.
#pragma once
#include <ucontext.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <vector>

#define CHK_CPU_EMULATION 1
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __launch_bounds__(...)
#define __align__(n) alignas(n)

struct emu_idx3 {
    unsigned x = 0, y = 0, z = 0;
};
struct dim3 {
    unsigned x, y, z;
    dim3(unsigned a = 1, unsigned b = 1, unsigned c = 1) : x(a), y(b), z(c) {}
};
struct uint2 {
    unsigned x, y;
};
struct alignas(16) uint4 {
    unsigned x, y, z, w;
};
struct alignas(16) float4 {
    float x, y, z, w;
};
static inline uint2 make_uint2(unsigned a, unsigned b) { return uint2{a, b}; }
static inline uint4 make_uint4(unsigned a, unsigned b, unsigned c, unsigned d) { return uint4{a, b, c, d}; }

static emu_idx3 threadIdx, blockIdx;
static dim3 blockDim, gridDim;

namespace emu {
constexpr size_t kStack = 128 * 1024;
struct Fiber {
    ucontext_t ctx;
    char* stack = nullptr;  // from a pool that is allocated once and reused by every block
    bool done = false;
};
// Fiber stacks are not zeroed and never freed: blocks run one after another and reuse them.
static char* fiber_stack(unsigned t) {
    static std::vector<char*> pool;
    while (pool.size() <= t) pool.push_back(static_cast<char*>(std::malloc(kStack)));
    return pool[t];
}
static ucontext_t g_main;
static std::vector<Fiber>* g_fibers = nullptr;
static unsigned g_cur = 0;
static std::function<void()>* g_body = nullptr;
static std::vector<unsigned char> g_dyn_smem;

// warp collectives: per-warp mailbox, generation-stamped
struct WarpBox {
    unsigned long long val[32];
    unsigned arrived = 0;
    unsigned gen = 0;
    unsigned long long result[32];
};
static std::vector<WarpBox> g_warp;

// block barrier: released when every fiber that is still running has arrived
static unsigned g_live = 0, g_bar_arrived = 0, g_bar_gen = 0;
static inline void yield() { swapcontext(&(*g_fibers)[g_cur].ctx, &g_main); }
static inline void barrier_release_if_full() {
    if (g_bar_arrived && g_bar_arrived == g_live) {
        g_bar_arrived = 0;
        ++g_bar_gen;
    }
}
static inline void block_barrier() {
    const unsigned gen = g_bar_gen;
    ++g_bar_arrived;
    barrier_release_if_full();
    while (g_bar_gen == gen) yield();
}
static void trampoline() {
    (*g_body)();
    (*g_fibers)[g_cur].done = true;
    --g_live;
    barrier_release_if_full();
    swapcontext(&(*g_fibers)[g_cur].ctx, &g_main);
}

static void run_block(unsigned nthreads, std::function<void()> body) {
    std::vector<Fiber> fibers(nthreads);
    g_fibers = &fibers;
    g_body = &body;
    g_warp.assign((nthreads + 31) / 32, WarpBox{});
    g_live = nthreads;
    g_bar_arrived = 0;
    for (unsigned t = 0; t < nthreads; ++t) {
        Fiber& f = fibers[t];
        f.stack = fiber_stack(t);
        getcontext(&f.ctx);
        f.ctx.uc_stack.ss_sp = f.stack;
        f.ctx.uc_stack.ss_size = kStack;
        f.ctx.uc_link = &g_main;
        makecontext(&f.ctx, trampoline, 0);
    }
    bool live = true;
    while (live) {
        live = false;
        for (unsigned t = 0; t < nthreads; ++t) {
            if (fibers[t].done) continue;
            g_cur = t;
            threadIdx.x = t;
            swapcontext(&g_main, &fibers[t].ctx);
            live |= !fibers[t].done;
        }
    }
    g_fibers = nullptr;
    g_body = nullptr;
}

template <typename F>
static void launch(unsigned grid, unsigned block, size_t dyn_smem, F&& call) {
    gridDim = dim3(grid);
    blockDim = dim3(block);
    g_dyn_smem.assign(dyn_smem + 256, 0);
    for (unsigned b = 0; b < grid; ++b) {
        blockIdx.x = b;
        run_block(block, call);
    }
}

// Whole-warp collective over all 32 lanes (kernels here always use the full mask).
template <typename Fn>
static unsigned long long warp_collective(unsigned long long v, Fn&& combine) {
    const unsigned t = g_cur, w = t / 32, l = t % 32;
    WarpBox& box = g_warp[w];
    const unsigned my_gen = box.gen;
    box.val[l] = v;
    const unsigned want = std::min(32u, blockDim.x - w * 32);
    if (++box.arrived == want) {
        for (unsigned i = 0; i < want; ++i) box.result[i] = combine(box.val, want, i);
        box.arrived = 0;
        box.gen++;
    } else {
        while (box.gen == my_gen) yield();
    }
    return box.result[l];
}
}  // namespace emu

static inline void __syncthreads() { emu::block_barrier(); }
static inline void __syncwarp(unsigned = 0xffffffffu) {}
static inline void __threadfence() {}

static inline unsigned __match_any_sync(unsigned, unsigned v) {
    return (unsigned)emu::warp_collective(v, [](const unsigned long long* a, unsigned n, unsigned me) {
        unsigned long long m = 0;
        for (unsigned i = 0; i < n; ++i)
            if (a[i] == a[me]) m |= 1ull << i;
        return m;
    });
}
static inline unsigned __match_any_sync(unsigned, unsigned long long v) {
    return (unsigned)emu::warp_collective(v, [](const unsigned long long* a, unsigned n, unsigned me) {
        unsigned long long m = 0;
        for (unsigned i = 0; i < n; ++i)
            if (a[i] == a[me]) m |= 1ull << i;
        return m;
    });
}
static inline unsigned long long atomicCAS(unsigned long long* p, unsigned long long cmp, unsigned long long val) {
    const unsigned long long old = *p;
    if (old == cmp) *p = val;
    return old;
}
static inline unsigned atomicMin(unsigned* p, unsigned v) {
    const unsigned old = *p;
    *p = std::min(old, v);
    return old;
}
static inline unsigned __ballot_sync(unsigned, int p) {
    return (unsigned)emu::warp_collective(p ? 1 : 0, [](const unsigned long long* a, unsigned n, unsigned) {
        unsigned long long m = 0;
        for (unsigned i = 0; i < n; ++i)
            if (a[i]) m |= 1ull << i;
        return m;
    });
}
template <typename T>
static inline T __shfl_up_sync(unsigned, T v, unsigned delta) {
    static_assert(sizeof(T) <= 8, "");
    unsigned long long raw = 0;
    std::memcpy(&raw, &v, sizeof(T));
    unsigned long long r = emu::warp_collective(raw, [delta](const unsigned long long* a, unsigned, unsigned me) {
        return me >= delta ? a[me - delta] : a[me];
    });
    T out;
    std::memcpy(&out, &r, sizeof(T));
    return out;
}
template <typename T>
static inline T __shfl_sync(unsigned, T v, int src) {
    unsigned long long raw = 0;
    std::memcpy(&raw, &v, sizeof(T));
    unsigned long long r = emu::warp_collective(raw, [src](const unsigned long long* a, unsigned n, unsigned) {
        return a[(unsigned)src % n];
    });
    T out;
    std::memcpy(&out, &r, sizeof(T));
    return out;
}
template <typename T>
static inline T __shfl_xor_sync(unsigned, T v, int mask) {
    unsigned long long raw = 0;
    std::memcpy(&raw, &v, sizeof(T));
    unsigned long long r = emu::warp_collective(raw, [mask](const unsigned long long* a, unsigned n, unsigned me) {
        return a[(me ^ (unsigned)mask) % n];
    });
    T out;
    std::memcpy(&out, &r, sizeof(T));
    return out;
}

template <typename T>
static inline T atomicAdd(T* p, T v) {
    T old = *p;
    *p = old + v;
    return old;
}
static inline unsigned atomicOr(unsigned* p, unsigned v) {
    unsigned old = *p;
    *p = old | v;
    return old;
}
static inline unsigned long long atomicMax(unsigned long long* p, unsigned long long v) {
    unsigned long long old = *p;
    *p = std::max(old, v);
    return old;
}
static inline unsigned atomicMax(unsigned* p, unsigned v) {
    unsigned old = *p;
    *p = std::max(old, v);
    return old;
}
static inline unsigned __umulhi(unsigned a, unsigned b) { return (unsigned)(((unsigned long long)a * b) >> 32); }
static inline int __popc(unsigned v) { return __builtin_popcount(v); }
static inline int __ffs(unsigned v) { return __builtin_ffs((int)v); }
static inline int __clz(int v) { return v ? __builtin_clz((unsigned)v) : 32; }
static inline unsigned __funnelshift_r(unsigned lo, unsigned hi, unsigned sh) {
    unsigned long long v = ((unsigned long long)hi << 32) | lo;
    return (unsigned)(v >> (sh & 31));
}
static inline unsigned __funnelshift_l(unsigned lo, unsigned hi, unsigned sh) {
    unsigned long long v = ((unsigned long long)hi << 32) | lo;
    return (unsigned)((v << (sh & 31)) >> 32);
}
static inline unsigned __byte_perm(unsigned a, unsigned b, unsigned s) {
    unsigned long long v = ((unsigned long long)b << 32) | a;
    unsigned r = 0;
    for (int i = 0; i < 4; ++i) {
        unsigned sel = (s >> (4 * i)) & 0xF;
        unsigned byte = (unsigned)(v >> (8 * (sel & 7))) & 0xFF;
        if (sel & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        r |= byte << (8 * i);
    }
    return r;
}
static inline float __fadd_rn(float a, float b) { return a + b; }
static inline float __fsub_rn(float a, float b) { return a - b; }
static inline float __fmul_rn(float a, float b) { return a * b; }
static inline float __fdiv_rn(float a, float b) { return a / b; }
static inline float __fsqrt_rn(float a) { return sqrtf(a); }
static inline float __uint_as_float(unsigned u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static inline unsigned __float_as_uint(float f) {
    unsigned u;
    std::memcpy(&u, &f, 4);
    return u;
}
using std::max;
using std::min;
