// rans_kernels.cuh -- 256-lane rANS encode / decode and the payload layout
// kernels.  Included by kernels.cuh (which provides the shared types).
//
// Thread mapping.  A tensor is 256 interleaved lanes: lane t owns bytes t,
// t+256, ...  (src/ANSCompressor.cpp:154-211 in the Checkers tree).  A team of
// 64 threads works on one tensor; thread j owns the four lanes 4j..4j+3, i.e.
// one aligned 32-bit word of every 256-byte row, so a warp reads or writes 128
// contiguous bytes per row with no staging.  Of those four lanes only the ones
// that carry codec input are real chains:
//     fp32      bytes 2,3 of each word     2 chains per thread
//     bf16/fp16 bytes 1,3 of each word     2 chains per thread
//     int8/32   all four bytes             4 chains per thread
// The remaining lanes only ever see the zeroed low bytes.  Every such lane of a
// tensor encodes the same symbol-0 sequence, so that sequence is produced once
// per tensor (zero_lane_kernel) and shared: a lane with one symbol fewer owns a
// suffix of the same byte string.  The independent chains of a thread give the
// scheduler instruction-level parallelism across the serial state updates.
#pragma once

#include <type_traits>

namespace chk {

constexpr uint32_t kTeam = 64;  // threads per tensor

// Byte of the thread's 32-bit row word that chain k encodes.  NV = chains per
// thread; B0 = byte of the first chain when NV == 2 (2 for fp32, 1 for bf16/fp16).
template <int NV, int B0>
__device__ __forceinline__ constexpr uint32_t chain_byte(int k) {
    return NV == 4 ? (uint32_t)k : (k == 0 ? (uint32_t)B0 : 3u);
}

// Shared memory of one encode team: table (256 x 8 B) + a 64-byte output ring
// per chain (two 32-byte blocks).  Ring words are interleaved across the team
// (word slot s of thread j's chain k sits at byte k*4096 + s*256 + j*4 of the
// ring area), so a warp never has a bank conflict on it whatever the lanes'
// positions are.
constexpr uint32_t kEncRingSlots = 16;                          // words per chain
constexpr uint32_t kEncRingBytes = kEncRingSlots * kTeam * 4;   // ring area of one chain index
constexpr uint32_t kEncSlotMask = (kEncRingSlots - 1) * 256u;   // the slot bits of a ring offset
template <int NV>
struct EncSmem {
    uint2 tab[256];  // per symbol: rcp | freq << 19 + bias << 5 + shift
    uint32_t ring[NV * kEncRingSlots * kTeam];
};

// Output side of one chain.  Emitted bytes are first collected in a 64-bit
// register pair (newest byte lowest); every two steps a completed 4-byte word
// moves to the shared-memory ring, and every eight steps a completed 32-byte
// block -- one whole DRAM sector, so the L2 never has to merge or fill a
// partly written one -- moves from the ring to the lane's scratch region.
// Streams grow downward in memory, so the oldest byte of a word is its most
// significant one and ring slots are filled from the top of a block (slot 7 or
// 15) downward.  Everything is kept as running offsets so that a step costs no
// address arithmetic beyond one add.
struct EncOut {
    uint32_t lo, hi;   // pending bytes, newest in lo[7:0]
    uint32_t cnt8;     // pending bits (8 per byte; below 32 after a word check)
    uint32_t soff;     // byte offset in the ring area of the slot the next word goes to
    uint32_t foff;     // byte offset in the ring area of the block (8 slots) that is flushed next
    uint32_t wleft;    // words in the ring that are not in global memory yet
    uint32_t gpos;     // byte position in the lane region the next 32-byte block goes to
};

__device__ __forceinline__ void enc_emit(EncOut& o, uint32_t v) {  // append byte v[7:0]
    o.hi = __byte_perm(o.hi, o.lo, 0x2107);
    o.lo = __byte_perm(o.lo, v, 0x2104);
    o.cnt8 += 8;
}

// One encode step of one chain: renormalise (at most two bytes, low byte first)
// and advance the state.  The two conditional byte emissions are written as
// predicated instructions, not branches: in a warp some lane nearly always
// emits, so a branch would only add its own overhead and a divergent re-issue.
// kEscape = true adds the test for symbols that are missing from the table
// (raw escape byte, state untouched); the host proves when there are none.
// Table entry: 8 bytes, so a warp's random lookups cost half the shared-memory wavefronts of a
// 16-byte entry (the lookups are what the kernel is bound by).  e.x = reciprocal, e.y = freq in bits
// 19..31 (so e.y with its low 19 bits cleared is freq * 2^19, the renormalisation bound), bias in bits
// 5..17, the shift count in bits 0..3 (bit 4 is zero: a funnel shift by e.y shifts by just that count).
template <bool kEscape>
__device__ __forceinline__ void enc_step(uint32_t sym, const uint2* tab, uint32_t& x, EncOut& o) {
    const uint2 e = tab[sym];
    if (kEscape && e.y == 0) {
        enc_emit(o, sym);
        return;
    }
    const uint32_t xmax = e.y & 0xFFF80000u;  // freq * 2^19
#ifdef CHK_CPU_EMULATION
    if (x >= xmax) {
        enc_emit(o, x);
        x >>= 8;
    }
    if (x >= xmax) {  // a second byte needs freq < 16
        enc_emit(o, x);
        x >>= 8;
    }
#else
    asm("{\n\t.reg .pred p;\n\t"
        "setp.hs.u32 p, %0, %4;\n\t"
        "@p prmt.b32 %1, %1, %2, 0x2107;\n\t"
        "@p prmt.b32 %2, %2, %0, 0x2104;\n\t"
        "@p add.u32 %3, %3, 8;\n\t"
        "@p shr.u32 %0, %0, 8;\n\t"
        "setp.hs.u32 p, %0, %4;\n\t"
        "@p prmt.b32 %1, %1, %2, 0x2107;\n\t"
        "@p prmt.b32 %2, %2, %0, 0x2104;\n\t"
        "@p add.u32 %3, %3, 8;\n\t"
        "@p shr.u32 %0, %0, 8;\n\t}"
        : "+r"(x), "+r"(o.hi), "+r"(o.lo), "+r"(o.cnt8)
        : "r"(xmax));
#endif
    const uint32_t q = __funnelshift_r(__umulhi(x, e.x), 0u, e.y);  // shift count: the low 5 bits of e.y
    x = x + q * (kM - (e.y >> 19)) + ((e.y >> 5) & 0x1FFFu);
}

// After at most two steps (4 new bytes, fewer than 8 pending): move one word to the ring.
__device__ __forceinline__ void enc_word(EncOut& o, uint8_t* ring) {
    // the oldest four pending bytes; the funnel shift takes its count modulo 32 = cnt8 - 32
    const uint32_t w = __funnelshift_r(o.lo, o.hi, o.cnt8);
    if (o.cnt8 >= 32) {
        *reinterpret_cast<uint32_t*>(ring + o.soff) = w;
        o.soff = (o.soff & ~kEncSlotMask) | ((o.soff - 256u) & kEncSlotMask);  // next slot down, wrapping inside the ring
        ++o.wleft;
    }
    o.cnt8 &= 31u;
}

// After at most eight steps (16 new bytes in the ring, at most 28 + 16 unflushed): move the
// one 32-byte block that may have completed to the lane's scratch region.
__device__ __forceinline__ void enc_block(EncOut& o, const uint8_t* ring, uint8_t* region) {
    if (o.wleft >= 8) {
        const uint8_t* b = ring + o.foff;
        uint4 v0, v1;
        v0.x = *reinterpret_cast<const uint32_t*>(b);
        v0.y = *reinterpret_cast<const uint32_t*>(b + 256);
        v0.z = *reinterpret_cast<const uint32_t*>(b + 512);
        v0.w = *reinterpret_cast<const uint32_t*>(b + 768);
        v1.x = *reinterpret_cast<const uint32_t*>(b + 1024);
        v1.y = *reinterpret_cast<const uint32_t*>(b + 1280);
        v1.z = *reinterpret_cast<const uint32_t*>(b + 1536);
        v1.w = *reinterpret_cast<const uint32_t*>(b + 1792);
        *reinterpret_cast<uint4*>(region + o.gpos) = v0;
        *reinterpret_cast<uint4*>(region + o.gpos + 16) = v1;
        o.gpos -= 32;
        o.foff ^= 2048u;
        o.wleft -= 8;
    }
}

__device__ __forceinline__ uint32_t load_row_word(const uint8_t* p, bool aligned4) {
    if (aligned4) return *reinterpret_cast<const uint32_t*>(p);
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// The value lanes of one tensor, encoded by the team into lane regions of d.chunk_stride bytes
// each starting at `regions` (chain k of thread j uses region j*NV + k).  Returns each chain's
// final state and the lowest byte position of its stream inside its region.  Ends without a
// barrier: the caller synchronises before the table and ring are reused.
template <int NV, int B0, bool kEscape>
__device__ __forceinline__ void encode_lanes(const TensorDesc& d, const EncEntry* __restrict__ tables,
                                             uint8_t* __restrict__ regions, unsigned char* smem_raw,
                                             uint32_t (&x_out)[NV], uint32_t (&low_out)[NV]) {
    EncSmem<NV>* sm = reinterpret_cast<EncSmem<NV>*>(smem_raw);
    uint8_t* const ring = reinterpret_cast<uint8_t*>(sm->ring);
    const uint32_t j = threadIdx.x;
    const unsigned long long B = d.n_bytes;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const EncEntry e = tables[(size_t)d.table_idx * 256 + j * 4 + i];
        sm->tab[j * 4 + i] = make_uint2(e.rcp, ((e.freq_shift & 0xFFFFu) << 19) | (e.bias << 5) | (e.freq_shift >> 16));
    }
    __syncthreads();

    const uint32_t S = d.chunk_stride;  // multiple of 32
    uint32_t x[NV];
    EncOut out[NV];
    uint8_t* region[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        x[k] = kL;
        out[k].lo = out[k].hi = 0;
        out[k].cnt8 = 0;
        const uint32_t s0 = ((S >> 2) - 1u) & (kEncRingSlots - 1);  // slot of the first word: the top of its block
        out[k].soff = (uint32_t)k * kEncRingBytes + s0 * 256u + j * 4u;
        out[k].foff = (uint32_t)k * kEncRingBytes + (s0 >> 3) * 2048u + j * 4u;
        out[k].wleft = 0;
        out[k].gpos = S - 32u;
        region[k] = regions + (size_t)(j * NV + k) * S;
    }

    const unsigned long long full_rows = B >> 8;
    const uint32_t tail = (uint32_t)(B & 255);
    const bool aligned4 = (reinterpret_cast<uintptr_t>(d.src) & 3) == 0;
    const uint8_t* col = d.src + 4 * j;
    // One row for all chains of the thread, then (every second row) the word check.
    auto row = [&](uint32_t w, bool word_check) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            enc_step<kEscape>((w >> (8 * chain_byte<NV, B0>(k))) & 0xFF, sm->tab, x[k], out[k]);
            if (word_check) enc_word(out[k], ring);
        }
    };

    // the last, partial row (symbols of the highest index come first)
    if (tail) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const uint32_t t = 4 * j + chain_byte<NV, B0>(k);
            if (t < tail) enc_step<kEscape>(d.src[(full_rows << 8) + t], sm->tab, x[k], out[k]);
            enc_word(out[k], ring);
        }
    }
    // rows above the last multiple of 8, one at a time: with the partial row at most 8 steps
    unsigned long long r = full_rows;
    const uint32_t odd = (uint32_t)(full_rows & 7);
    for (uint32_t u = 0; u < odd; ++u) {
        --r;
        row(load_row_word(col + (r << 8), aligned4), true);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) enc_block(out[k], ring, region[k]);

    // full groups of 8 rows, highest first.  The words of the NEXT group are
    // requested before the current group's dependent chains run, so the memory
    // latency hides behind 8 * NV chain steps.
    uint32_t nxt[8];
    if (r >= 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) nxt[u] = load_row_word(col + ((r - 8 + u) << 8), aligned4);
    }
    while (r >= 8) {
        r -= 8;
        uint32_t w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = nxt[u];
        if (r >= 8) {
#pragma unroll
            for (int u = 0; u < 8; ++u) nxt[u] = load_row_word(col + ((r - 8 + u) << 8), aligned4);
        }
#pragma unroll
        for (int u = 7; u >= 0; --u) row(w[u], (u & 1) == 0);
#pragma unroll
        for (int k = 0; k < NV; ++k) enc_block(out[k], ring, region[k]);
    }

    // what is still pending: up to 3 bytes in registers, up to 7 words in the ring
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        EncOut& o = out[k];
        // word i of the unfinished block (oldest first) sits in slot 7 - i of it and belongs at gpos + 4 * (7 - i)
        for (uint32_t i = 0; i < o.wleft; ++i) {
            const uint32_t sl = 7u - i;
            *reinterpret_cast<uint32_t*>(region[k] + o.gpos + 4u * sl) =
                *reinterpret_cast<const uint32_t*>(ring + o.foff + 256u * sl);
        }
        const uint32_t top = o.gpos + 32u - 4u * o.wleft;  // lowest byte position written as a whole word
        const uint32_t cnt = o.cnt8 >> 3;
        for (uint32_t i = 0; i < cnt; ++i)  // oldest pending byte sits highest in memory
            region[k][top - 1 - i] = (uint8_t)(o.lo >> ((cnt - 1 - i) * 8));
        x_out[k] = x[k];
        low_out[k] = top - cnt;  // final lowest byte position of the stream
    }
}

// Stand-alone stage: lanes to scratch, provisional headers and byte locations to global memory
// (offsets and the gather follow in lane_scan_kernel / tensor_scan_kernel / compact_kernel).
template <int NV, int B0, bool kEscape>
__device__ __forceinline__ void encode_tensor(const TensorDesc& d, uint32_t ti, const EncEntry* __restrict__ tables,
                                              uint8_t* __restrict__ scratch, LaneHeader* __restrict__ hdrs,
                                              unsigned long long* __restrict__ lane_src, unsigned char* smem_raw) {
    uint32_t x[NV], low[NV];
    encode_lanes<NV, B0, kEscape>(d, tables, scratch + d.scratch_off, smem_raw, x, low);
    const uint32_t j = threadIdx.x;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const uint32_t t = 4 * j + chain_byte<NV, B0>(k);
        LaneHeader h;
        h.final_state = x[k];
        h.byte_count = d.chunk_stride - low[k];
        h.buf_offset = 0;
        h.pad = 0;
        hdrs[(size_t)ti * kLanes + t] = h;
        lane_src[(size_t)ti * kLanes + t] = d.scratch_off + (unsigned long long)(j * NV + k) * d.chunk_stride + low[k];
    }
    __syncthreads();  // table and ring are reused by the next tensor
}

// One team (CTA of 64 threads) per tensor.  kInts = false is the build for
// batches of float tensors only (two chains per thread, fewer registers, more
// resident teams); the host picks the variant per batch.
// Work is handed out through a ticket counter in the order given by `order`
// (largest tensors first), so a persistent grid of resident teams drains the
// batch without a ragged last wave.
__device__ __forceinline__ uint32_t next_ticket(uint32_t* ticket, uint32_t* slot) {
    if (threadIdx.x == 0) *slot = atomicAdd(ticket, 1u);
    __syncthreads();
    return *slot;  // every thread reads it before the next barrier, which precedes the next write
}

template <bool kInts, bool kEscape>
__global__ void __launch_bounds__(kTeam) rans_encode_kernel(const TensorDesc* __restrict__ descs,
                                                            const EncEntry* __restrict__ tables,
                                                            uint8_t* __restrict__ scratch,
                                                            LaneHeader* __restrict__ hdrs,
                                                            unsigned long long* __restrict__ lane_src,
                                                            const uint32_t* __restrict__ order,
                                                            uint32_t* __restrict__ ticket, uint32_t n_tensors) {
    CHK_DYN_SMEM(smem);
    CHK_SHARED uint32_t s_ticket;
    for (;;) {
        const uint32_t tk = next_ticket(ticket, &s_ticket);
        if (tk >= n_tensors) break;
        const uint32_t ti = order[tk];
        const TensorDesc d = descs[ti];
        if (d.es == 4 && d.spe == 2)
            encode_tensor<2, 2, kEscape>(d, ti, tables, scratch, hdrs, lane_src, smem);
        else if (d.es == 2 && d.spe == 1)
            encode_tensor<2, 1, kEscape>(d, ti, tables, scratch, hdrs, lane_src, smem);
        else if (kInts)
            encode_tensor<4, 0, kEscape>(d, ti, tables, scratch, hdrs, lane_src, smem);
        else
            __syncthreads();  // keep the barrier count uniform
    }
}

// The symbol-0 chain of every tensor that has zeroed low bytes: one thread per
// tensor, c_max steps, bytes written downward from the top of the tensor's zero
// region (the region after its value-lane regions).  The same thread then fills
// in the header and byte location of each of the tensor's zero lanes: a lane
// with c_max symbols owns the whole string, one with c_max-1 owns its suffix.
// Runs next to the value-lane kernel (it touches different lanes and regions).
struct ZeroChain {
    uint32_t state0, nbytes0;  // after c_max symbols
    uint32_t state1, nbytes1;  // after c_max - 1 symbols (a suffix of the same byte string)
};
// Encodes c_max zeros with table entry e, bytes written downward from region + stride
// (a multiple of 4; region 4-byte aligned).  One thread, one dependent chain: emitted bytes are
// collected four at a time so that the chain is not held up by a store per byte.
__device__ __forceinline__ ZeroChain zero_chain(const EncEntry e, uint8_t* __restrict__ region, uint32_t stride,
                                                unsigned long long c_max) {
    const uint32_t f = e.freq_shift & 0xFFFFu, sh = e.freq_shift >> 16, xmax = e.freq_shift << 19;
    ZeroChain z;
    if (f == 0) {  // symbol 0 is not in the table: every zero is a raw escape byte and the state never moves
        for (unsigned long long i = 0; i < c_max; ++i) region[stride - 1 - i] = 0;
        z.state0 = z.state1 = kL;
        z.nbytes0 = (uint32_t)c_max;
        z.nbytes1 = c_max ? (uint32_t)c_max - 1u : 0u;
        return z;
    }
    uint32_t x = kL, acc = 0, nacc = 0, emitted = 0;
    uint8_t* wp = region + stride;  // the next word goes below this
    // One step.  This thread's time is one chain of dependent operations (compare, shift, multiply-high,
    // shift, multiply-add), so nothing in it may branch: with freq >= 16 a symbol emits at most one byte
    // and everything conditional is a predicated instruction.
    auto step = [&]() {
#ifndef CHK_CPU_EMULATION
        if (f >= 16) {
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t.reg .u32 t;\n\t"
                "setp.hs.u32 p, %0, %5;\n\t"
                "@p prmt.b32 %1, %0, %1, 0x6540;\n\t"  // acc = acc << 8 | low byte of x: the newest byte is the lowest in memory
                "@p shr.u32 %0, %0, 8;\n\t"
                "@p add.u32 %2, %2, 1;\n\t"
                "@p add.u32 %3, %3, 1;\n\t"
                "setp.eq.u32 q, %3, 4;\n\t"
                "@q sub.u64 %4, %4, 4;\n\t"
                "@q st.global.u32 [%4], %1;\n\t"
                "@q mov.u32 %3, 0;\n\t"
                "mul.hi.u32 t, %0, %6;\n\t"
                "shr.u32 t, t, %7;\n\t"
                "mad.lo.u32 %0, t, %8, %0;\n\t"
                "add.u32 %0, %0, %9;\n\t}"
                : "+r"(x), "+r"(acc), "+r"(emitted), "+r"(nacc), "+l"(wp)
                : "r"(xmax), "r"(e.rcp), "r"(sh), "r"(e.cmpl), "r"(e.bias)
                : "memory");
            return;
        }
#endif
#pragma unroll
        for (int r = 0; r < 2; ++r) {  // at most two bytes per symbol
            if (x >= xmax) {
                acc = (acc << 8) | (x & 0xFFu);  // the newest byte is the lowest in memory
                x >>= 8;
                ++emitted;
                if (++nacc == 4) {
                    wp -= 4;
                    *reinterpret_cast<uint32_t*>(wp) = acc;
                    nacc = 0;
                }
            }
        }
        const uint32_t q = __umulhi(x, e.rcp) >> sh;
        x = x + q * e.cmpl + e.bias;
    };
    const uint32_t n1 = c_max ? (uint32_t)(c_max - 1) : 0u;  // c_max < 2^24: a tensor is smaller than 4 GiB
    uint32_t i = 0;
    for (; i + 4 <= n1; i += 4) {
        step();
        step();
        step();
        step();
    }
    for (; i < n1; ++i) step();
    z.state1 = c_max ? x : kL;
    z.nbytes1 = emitted;
    if (c_max) step();
    z.state0 = x;
    z.nbytes0 = emitted;
    for (uint32_t k = 0; k < nacc; ++k) (wp - nacc)[k] = (uint8_t)(acc >> (8 * k));  // up to three bytes left
    return z;
}

__global__ void __launch_bounds__(32) zero_lane_kernel(const TensorDesc* __restrict__ descs,
                                                        const EncEntry* __restrict__ tables,
                                                        uint8_t* __restrict__ scratch,
                                                        LaneHeader* __restrict__ hdrs,
                                                        unsigned long long* __restrict__ lane_src,
                                                        uint32_t n_tensors) {
    const uint32_t ti = blockIdx.x * blockDim.x + threadIdx.x;
    if (ti >= n_tensors) return;
    const TensorDesc d = descs[ti];
    if (d.spe * 2 != d.es) return;  // integer tensors have no zeroed bytes
    const unsigned long long zbase = d.scratch_off + (unsigned long long)kTeam * 2 * d.chunk_stride;
    const unsigned long long c_max = (d.n_bytes + kLanes - 1) / kLanes;
    const ZeroChain z = zero_chain(tables[(size_t)d.table_idx * 256], scratch + zbase, d.chunk_stride, c_max);
    for (uint32_t t = 0; t < kLanes; ++t) {
        if ((t % d.es) >= d.spe) continue;
        const unsigned long long cnt = d.n_bytes > t ? (d.n_bytes - t + kLanes - 1) / kLanes : 0;
        LaneHeader h;
        h.buf_offset = 0;
        h.pad = 0;
        h.final_state = cnt == 0 ? kL : (cnt == c_max ? z.state0 : z.state1);
        h.byte_count = cnt == 0 ? 0u : (cnt == c_max ? z.nbytes0 : z.nbytes1);
        hdrs[(size_t)ti * kLanes + t] = h;
        lane_src[(size_t)ti * kLanes + t] = zbase + d.chunk_stride - h.byte_count;
    }
}

// ------------------------------------------------------------------ offsets and compaction
// Per tensor: exclusive prefix sum of the 256 lane byte counts
// (src/ANSCompressor.cpp:647-651), the passthrough decision total >= n_bytes
// (:695-713) and the final on-disk lane headers (:686-691).
__global__ void __launch_bounds__(256) lane_scan_kernel(TensorDesc* __restrict__ descs,
                                                        LaneHeader* __restrict__ hdrs,
                                                        unsigned long long* __restrict__ payload_size,
                                                        uint32_t* __restrict__ lane_off, uint32_t n_tensors) {
    CHK_SHARED uint32_t warp_tot[8];
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (uint32_t ti = blockIdx.x; ti < n_tensors; ti += gridDim.x) {
        LaneHeader h = hdrs[(size_t)ti * kLanes + t];
        uint32_t v = h.byte_count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= (uint32_t)o) v += n;
        }
        if (lane == 31) warp_tot[warp] = v;
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            if ((uint32_t)w < warp) before += warp_tot[w];
            total += warp_tot[w];
        }
        const uint32_t excl = before + v - h.byte_count;
        const unsigned long long B = descs[ti].n_bytes;
        const bool raw = (unsigned long long)total >= B;
        lane_off[(size_t)ti * kLanes + t] = excl;
        if (raw) {
            h.final_state = 0;
            h.byte_count = t == 0 ? (uint32_t)B : 0u;
            h.buf_offset = 0;
        } else {
            h.buf_offset = excl;
        }
        h.pad = 0;
        hdrs[(size_t)ti * kLanes + t] = h;
        if (t == 0) {
            payload_size[ti] = raw ? B : (unsigned long long)total;
            if (raw) descs[ti].flags |= kFlagRaw; else descs[ti].flags &= ~kFlagRaw;
        }
        __syncthreads();
    }
}

// Exclusive prefix sum of the per-tensor payload sizes (one CTA); total in out[n].
// A batch scanned in several launches chains them: `start` points at the total the
// previous launch left (its out[n], which is this launch's out[0]); null starts at 0.
__global__ void __launch_bounds__(1024) tensor_scan_kernel(TensorDesc* __restrict__ descs,
                                                           const unsigned long long* __restrict__ payload_size,
                                                           unsigned long long* __restrict__ payload_off,
                                                           uint32_t n_tensors, const unsigned long long* start) {
    CHK_SHARED unsigned long long part[1024];
    const uint32_t t = threadIdx.x;
    const unsigned long long first = start ? *start : 0ull;
    __syncthreads();  // everyone has read the start before out[0] is rewritten
    const uint32_t per = (n_tensors + 1023) / 1024;
    const uint32_t lo = t * per < n_tensors ? t * per : n_tensors;
    const uint32_t hi = lo + per < n_tensors ? lo + per : n_tensors;
    unsigned long long s = 0;
    for (uint32_t i = lo; i < hi; ++i) s += payload_size[i];
    part[t] = s;
    __syncthreads();
    if (t == 0) {
        unsigned long long run = first;
        for (uint32_t i = 0; i < 1024; ++i) {
            const unsigned long long v = part[i];
            part[i] = run;
            run += v;
        }
        payload_off[n_tensors] = run;
    }
    __syncthreads();
    unsigned long long run = part[t];
    for (uint32_t i = lo; i < hi; ++i) {
        payload_off[i] = run;
        descs[i].payload_off = run;
        run += payload_size[i];
    }
}

// One warp copies cnt bytes from s to o (neither aligned): 16 bytes per thread per step once the
// destination is aligned (funnel-shifted source words), kPieces pieces per thread in flight so a
// warp keeps kPieces x 512 bytes on their way.
template <int kPieces>
__device__ __forceinline__ void warp_copy(uint8_t* __restrict__ o, const uint8_t* __restrict__ s, uint32_t cnt,
                                          uint32_t lane) {
    uint32_t head = (uint32_t)((16 - (reinterpret_cast<uintptr_t>(o) & 15)) & 15);
    if (head > cnt) head = cnt;
    if (lane < head) o[lane] = s[lane];
    const uint32_t nvec = (cnt - head) >> 4;
    const uint8_t* sv = s + head;
    uint8_t* ov = o + head;
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(sv) & 3);
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(sv - mis);
    for (uint32_t v0 = lane; v0 < nvec; v0 += 32 * kPieces) {
        uint32_t a[kPieces][5];
#pragma unroll
        for (int u = 0; u < kPieces; ++u) {
            const uint32_t v = v0 + 32 * u;
            if (v < nvec) {
#pragma unroll
                for (int i = 0; i < 4; ++i) a[u][i] = sw[v * 4 + i];
                a[u][4] = mis ? sw[v * 4 + 4] : 0u;
            }
        }
#pragma unroll
        for (int u = 0; u < kPieces; ++u) {
            const uint32_t v = v0 + 32 * u;
            if (v < nvec) {
                uint4 r;
                r.x = __funnelshift_r(a[u][0], a[u][1], mis * 8);
                r.y = __funnelshift_r(a[u][1], a[u][2], mis * 8);
                r.z = __funnelshift_r(a[u][2], a[u][3], mis * 8);
                r.w = __funnelshift_r(a[u][3], a[u][4], mis * 8);
                *reinterpret_cast<uint4*>(ov + (size_t)v * 16) = r;
            }
        }
    }
    for (uint32_t i = head + (nvec << 4) + lane; i < cnt; i += 32) o[i] = s[i];
}

// Gather (src/ANSCompressor.cpp:225-238): one warp per (tensor, lane) moves that
// lane's bytes from scratch to their place in the data section, 16 bytes per
// thread per step once the destination is aligned.  A passthrough tensor instead
// has its masked bytes written, each warp taking 1/256 of the tensor.
__global__ void __launch_bounds__(256) compact_kernel(const TensorDesc* __restrict__ descs,
                                                      const LaneHeader* __restrict__ hdrs,
                                                      const unsigned long long* __restrict__ lane_src,
                                                      const uint32_t* __restrict__ lane_off,
                                                      const uint8_t* __restrict__ scratch,
                                                      uint8_t* __restrict__ payload, uint32_t n_tensors) {
    const uint32_t lane = threadIdx.x & 31;
    const unsigned long long warps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;
    const unsigned long long total = (unsigned long long)n_tensors * kLanes;
    for (unsigned long long w = (((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); w < total;
         w += warps) {
        const uint32_t ti = (uint32_t)(w >> 8), t = (uint32_t)(w & 255);
        const TensorDesc d = descs[ti];
        uint8_t* out = payload + d.payload_off;
        if (d.flags & kFlagRaw) {
            const unsigned long long per = (d.n_bytes + kLanes - 1) / kLanes;
            const unsigned long long a = per * t;
            const unsigned long long b = a + per < d.n_bytes ? a + per : d.n_bytes;
            for (unsigned long long i = a + lane; i < b; i += 32)
                out[i] = (i % d.es) < d.spe ? (uint8_t)0 : d.src[i];
            continue;
        }
        warp_copy<4>(out + lane_off[(size_t)ti * kLanes + t], scratch + lane_src[(size_t)ti * kLanes + t],
                  hdrs[(size_t)ti * kLanes + t].byte_count, lane);
    }
}

// Heap order -> file order.  The fused encode kernel hands out payload space in the order tensors finish;
// the data section of the states file wants them in index order (src/ANSCompressor.cpp:751-816).  One block
// per tensor at a time, its warps taking 8 KiB pieces in turn, so the host receives the whole data section
// in one device-to-host copy instead of one per tensor.
__global__ void __launch_bounds__(256) order_payload_kernel(const TensorDesc* __restrict__ descs,
                                                            const unsigned long long* __restrict__ size,
                                                            const unsigned long long* __restrict__ file_off,
                                                            const uint8_t* __restrict__ heap, uint8_t* __restrict__ out,
                                                            uint32_t n_tensors) {
    constexpr unsigned long long kPiece = 8192;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t ti = blockIdx.x; ti < n_tensors; ti += gridDim.x) {
        const unsigned long long n = size[ti];
        const uint8_t* src = heap + descs[ti].payload_off;
        uint8_t* dst = out + file_off[ti];
        for (unsigned long long at = warp * kPiece; at < n; at += 8 * kPiece)
            warp_copy<4>(dst + at, src + at, (uint32_t)(n - at < kPiece ? n - at : kPiece), lane);
    }
}

// ------------------------------------------------------------------ shared symbol-0 chains of a batch
// The symbol-0 chain of a tensor depends on nothing but the table entry of symbol 0 and the
// number of symbols per lane.  Half of a float tensor's codec input is zeroed bytes, so that
// entry is the same (frequency 2048, give or take one) for nearly every tensor of a checkpoint,
// and a batch of thousands of tensors has a handful of distinct chains.  zero_chain_kernel
// computes each distinct chain once: one warp per tensor, lane 0 looks its key up in a small
// open-addressing table (an atomicCAS on the key claims a free slot), the first to claim a slot
// computes the chain into the slot's region, every tensor records its slot; nothing waits.  A chain is
// 16384 dependent steps for a 4 MiB tensor -- about a millisecond for one thread however it is
// written -- which is why it is taken out of the encode teams' path.  Tensors that find the
// table full get slot -1 and their team computes the chain itself.
struct ZeroSlot {
    // c_max << 32 | frequency and shift of symbol 0 (top bit set; 0 = free).  Symbol 0 is the first symbol, so
    // its cumulative frequency is 0 and the rest of its table entry follows from the frequency.
    unsigned long long key;
    ZeroChain chain;
};

__global__ void __launch_bounds__(32) zero_chain_kernel(const TensorDesc* __restrict__ descs,
                                                        const EncEntry* __restrict__ tables,
                                                        ZeroSlot* __restrict__ slots, uint32_t n_slots,
                                                        uint8_t* __restrict__ regions, uint32_t region_stride,
                                                        int32_t* __restrict__ slot_of, uint32_t n_tensors) {
    const uint32_t ti = blockIdx.x;
    if (ti >= n_tensors || threadIdx.x != 0) return;
    const TensorDesc d = descs[ti];
    if (d.spe * 2 != d.es) {  // integer tensors have no zeroed bytes
        slot_of[ti] = -1;
        return;
    }
    const EncEntry e = tables[(size_t)d.table_idx * 256];
    const unsigned long long c_max = (d.n_bytes + kLanes - 1) / kLanes;
    const unsigned long long key = (c_max << 32) | e.freq_shift | (1ull << 63);  // never 0
    uint32_t h = (uint32_t)((key * 0x9E3779B97F4A7C15ull) >> 40) % n_slots;
    int32_t found = -1;
    for (uint32_t probe = 0; probe < n_slots && found < 0; ++probe, h = h + 1 == n_slots ? 0 : h + 1) {
        const unsigned long long prev = atomicCAS(&slots[h].key, 0ull, key);
        if (prev == 0ull) {  // claimed: this thread computes the chain (nobody reads it before the kernel has ended)
            slots[h].chain = zero_chain(e, regions + (size_t)h * region_stride, d.chunk_stride, c_max);
            found = (int32_t)h;
        } else if (prev == key) {
            found = (int32_t)h;
        }
    }
    slot_of[ti] = found;
}

// ------------------------------------------------------------------ encode + offsets + gather in one kernel
// rans_encode_fused_kernel does for each tensor what rans_encode_kernel, zero_lane_kernel,
// lane_scan_kernel and compact_kernel do for a batch, inside the team that encodes it: value
// lanes into the team's OWN scratch slot (one slot per resident team, reused from tensor to
// tensor, so the scratch a batch needs is teams x largest tensor instead of the whole batch),
// the shared symbol-0 chain, the prefix sum of the 256 lane lengths
// (src/ANSCompressor.cpp:647-651), the passthrough rule and final headers (:686-713), and the
// gather of the lanes into one contiguous payload (:225-238).
//
// Where that payload goes: the data section of the file wants the tensors in index order, so
// the place of tensor i depends on the sizes of all tensors before it -- which other teams are
// still producing.  Waiting for them would make the teams march in step (every team of a wave
// waiting for the slowest one before any gathers).  Instead the device payload is a heap: a team
// takes the next free range with one atomic add, records it in the descriptor, and gathers at
// once, while the other teams of its SM keep the issue slots busy with their chains -- which is
// how the memory-bound gather hides under the issue-bound encoding.  The decoder follows the
// descriptors, so it does not care about the order; the file order is restored where the
// payloads leave the device (one copy per tensor into its place in the file image).
constexpr uint32_t kPayloadAlign = 32;  // heap ranges start on a DRAM sector

struct FusedInfo {  // per tensor, overlaid on the ring area once the lanes are encoded
    uint32_t cnt[kLanes];   // bytes of lane t
    uint32_t src[kLanes];   // where they start: offset in the team's scratch slot, or (top bit set) in the shared zero chain
    uint32_t dst[kLanes];   // where they go, relative to the tensor's payload
    uint32_t fin[kLanes];   // final state of lane t
    uint32_t warp_tot[2];
    unsigned long long payload_off;
    ZeroChain zero;
};

constexpr uint32_t kSrcSharedChain = 0x80000000u;

#ifdef CHK_CPU_EMULATION
#define CHK_NOINLINE
#else
#define CHK_NOINLINE __noinline__
#endif

// Everything after the value lanes of a tensor are in the team's slot (their lengths, positions and final
// states already in `info`).  Kept out of line so that its registers do not add to those of the encode loop.
// Everything the one-kernel path needs, passed as one kernel parameter: it stays in the constant
// bank and is read where it is used instead of being carried in registers through the encode loop.
struct FusedParams {
    TensorDesc* descs;
    const EncEntry* tables;
    uint8_t* scratch;                  // one slot of slot_bytes per team
    unsigned long long slot_bytes;
    const ZeroSlot* zero_slots;        // the batch's shared symbol-0 chains (zero_chain_kernel)
    const uint8_t* zero_regions;
    const int32_t* zero_slot_of;       // may be null: every team then computes its own chain
    uint32_t zero_region_stride;
    uint32_t n_tensors;
    LaneHeader* hdrs;
    uint8_t* payload;                  // the payload heap
    unsigned long long* payload_size;  // per tensor
    unsigned long long* heap_cursor;
    const uint32_t* order;
    uint32_t* ticket;
};

// Everything after the value lanes of a tensor are in the team's slot (their lengths, positions and final
// states already in `info`).  Kept out of line so that its registers do not add to those of the encode loop.
__device__ CHK_NOINLINE void finish_tensor(const FusedParams& P, uint32_t ti, bool floats, uint8_t* __restrict__ slot,
                                           FusedInfo* info) {
    const TensorDesc d = P.descs[ti];
    const uint32_t j = threadIdx.x, lane = j & 31, warp = j >> 5;
    const uint32_t S = d.chunk_stride;
    const unsigned long long B = d.n_bytes;
    const uint8_t* shared_chain = nullptr;
    if (floats) {
        // the symbol-0 chain that all lanes of zeroed low bytes share: from the batch's cache, or (cache full)
        // computed here by one thread into the region after the value lanes
        uint32_t zbase = 2u * kTeam * S;
        const unsigned long long c_max = (B + kLanes - 1) / kLanes;
        const int32_t zs = P.zero_slot_of ? P.zero_slot_of[ti] : -1;
        if (zs >= 0) {
            if (j == 0) info->zero = P.zero_slots[zs].chain;
            shared_chain = P.zero_regions + (size_t)zs * P.zero_region_stride;
            zbase = kSrcSharedChain;
        } else if (j == 0) {
            info->zero = zero_chain(P.tables[(size_t)d.table_idx * 256], slot + zbase, S, c_max);
        }
        __syncthreads();
        const ZeroChain z = info->zero;
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            const uint32_t t = 4 * j + b;
            if ((t % d.es) >= d.spe) continue;  // a value lane
            const unsigned long long n = B > t ? (B - t + kLanes - 1) / kLanes : 0;
            const uint32_t c = n == 0 ? 0u : (n == c_max ? z.nbytes0 : z.nbytes1);
            info->cnt[t] = c;
            info->fin[t] = n == 0 ? kL : (n == c_max ? z.state0 : z.state1);
            info->src[t] = zbase + S - c;
        }
    }

    // ---- the prefix sum of the lane lengths, the passthrough decision, the final headers
    uint32_t cnt[4];
#pragma unroll
    for (uint32_t b = 0; b < 4; ++b) cnt[b] = info->cnt[4 * j + b];
    const uint32_t mine = cnt[0] + cnt[1] + cnt[2] + cnt[3];
    uint32_t inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += n;
    }
    if (lane == 31) info->warp_tot[warp] = inc;
    __syncthreads();
    const uint32_t total = info->warp_tot[0] + info->warp_tot[1];
    uint32_t off = (warp ? info->warp_tot[0] : 0u) + inc - mine;
    const bool raw = (unsigned long long)total >= B;
    const unsigned long long size = raw ? B : (unsigned long long)total;
    if (j == 0) {  // the tensor's range of the payload heap
        const unsigned long long at = atomicAdd(P.heap_cursor, (size + kPayloadAlign - 1) & ~(unsigned long long)(kPayloadAlign - 1));
        info->payload_off = at;
        P.payload_size[ti] = size;
        P.descs[ti].payload_off = at;
        P.descs[ti].flags = raw ? (d.flags | kFlagRaw) : (d.flags & ~kFlagRaw);
    }
#pragma unroll
    for (uint32_t b = 0; b < 4; ++b) {
        const uint32_t t = 4 * j + b;
        LaneHeader h;
        h.pad = 0;
        if (raw) {
            h.final_state = 0;
            h.byte_count = t == 0 ? (uint32_t)B : 0u;
            h.buf_offset = 0;
        } else {
            h.final_state = info->fin[t];
            h.byte_count = cnt[b];
            h.buf_offset = off;
        }
        P.hdrs[(size_t)ti * kLanes + t] = h;
        info->dst[t] = off;
        off += cnt[b];
    }
    __syncthreads();

    // ---- gather: lanes side by side in lane order, or the masked tensor itself
    uint8_t* out = P.payload + info->payload_off;
    if (raw) {
        for (unsigned long long i = j; i < B; i += kTeam) out[i] = (i % d.es) < d.spe ? (uint8_t)0 : d.src[i];
    } else {
        for (uint32_t t = warp; t < kLanes; t += 2) {
            const uint32_t sr = info->src[t];
            warp_copy<4>(out + info->dst[t], (sr & kSrcSharedChain) ? shared_chain + (sr & ~kSrcSharedChain) : slot + sr,
                         info->cnt[t], lane);
        }
    }
    __syncthreads();  // table and lane table are reused by the next tensor
}

template <int NV, int B0>
__device__ __forceinline__ void encode_tensor_fused(const FusedParams& P, uint32_t ti, uint8_t* __restrict__ slot,
                                                    unsigned char* smem_raw) {
    const uint32_t j = threadIdx.x;
    uint32_t x[NV], low[NV];
    uint32_t S;
    {
        const TensorDesc d = P.descs[ti];
        S = d.chunk_stride;
        encode_lanes<NV, B0, false>(d, P.tables, slot, smem_raw, x, low);
    }
    __syncthreads();  // the ring is free: its area now holds the per-tensor lane table
    FusedInfo* info = reinterpret_cast<FusedInfo*>(reinterpret_cast<EncSmem<NV>*>(smem_raw)->ring);
    static_assert(sizeof(FusedInfo) <= sizeof(uint32_t) * 2 * kEncRingSlots * kTeam, "lane table must fit the ring area");
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const uint32_t t = 4 * j + chain_byte<NV, B0>(k);
        info->cnt[t] = S - low[k];
        info->fin[t] = x[k];
        info->src[t] = (j * NV + (uint32_t)k) * S + low[k];
    }
    __syncthreads();
    finish_tensor(P, ti, NV == 2, slot, info);
}

// One team per tensor.  Tensors are handed out through a ticket counter in the order given by
// P.order (largest first), so the persistent grid drains the batch without a ragged last wave.
// Teams per SM the register allocation is held to: 12 (80 registers) for the two-chain float path; 8 (128
// registers instead of the 158 the four-chain path takes when left alone: 10.45 -> 9.8 ms for the 8-bit planes
// of the benchmark shard).
#ifndef CHK_ENC_MINBLOCKS
#define CHK_ENC_MINBLOCKS 12
#endif
#ifndef CHK_ENC_INT_MINBLOCKS
#define CHK_ENC_INT_MINBLOCKS 8
#endif
#ifdef CHK_CPU_EMULATION
#define CHK_GRID_CONSTANT
#else
#define CHK_GRID_CONSTANT __grid_constant__
#endif
template <bool kInts>
__global__ void __launch_bounds__(kTeam, kInts ? CHK_ENC_INT_MINBLOCKS : CHK_ENC_MINBLOCKS) rans_encode_fused_kernel(
    const CHK_GRID_CONSTANT FusedParams P) {
    CHK_DYN_SMEM(smem);
    CHK_SHARED uint32_t s_ticket;
    uint8_t* const slot = P.scratch + (unsigned long long)blockIdx.x * P.slot_bytes;
    for (;;) {
        const uint32_t tk = next_ticket(P.ticket, &s_ticket);
        if (tk >= P.n_tensors) break;
        const uint32_t ti = P.order[tk];
        const uint32_t es = P.descs[ti].es, spe = P.descs[ti].spe;
        if (es == 4 && spe == 2)
            encode_tensor_fused<2, 2>(P, ti, slot, smem);
        else if (es == 2 && spe == 1)
            encode_tensor_fused<2, 1>(P, ti, slot, smem);
        else if (kInts)
            encode_tensor_fused<4, 0>(P, ti, slot, smem);
        else
            __syncthreads();  // keep the barrier count uniform
    }
}

// ------------------------------------------------------------------ rANS decode
// The slot table: slot -> symbol[0:8) | (freq-1)[8:20) | (slot - cum[symbol])[20:32), 16 KiB per tensor.
// Two shapes, chosen per launch by the ZS template flag:
//   full      : one entry per slot.
//   zero-skip : for tensors whose symbol 0 owns the first `skip` >= kM - kZsEntries + 1 slots -- every
//               floating-point tensor: its zeroed low bytes are half of what the table was counted over, while
//               the lanes that are decoded here hardly ever see a zero -- all of those slots share entry 0 and
//               the table is about half as long, so more teams fit an SM.  With s1 = skip - 1 and
//               m = max(slot, s1) the entry is dtab[m - s1], and the state needs slot - m added (entry 0 holds
//               offset s1, so a slot below skip gets f0 * (x >> 12) + slot as it must).  Two more integer
//               instructions per symbol, no extra load.
constexpr uint32_t kRingWords = 17;
template <int NV, bool ZS>
struct DecSmem {
    uint32_t dtab[ZS ? kZsEntries : kM];
    // 64-byte input ring per chain (two 32-byte blocks) plus a 17th word that repeats word 0,
    // so the word after any ring word is the next one without a wrap.  The rings of a warp are
    // interleaved word by word (word w of lane l at [w * 32 + l]): every lane stays in its own
    // shared-memory bank wherever its read position is, so neither the reads (each lane at a
    // different, data-dependent position) nor the block stores ever conflict.
    uint32_t ring[NV * kTeam * kRingWords];
    uint32_t cum[260];
};
// shared memory per team: [chains per thread: 2 = float tensors only, 4 = integers present][table shape]
constexpr uint32_t kDecSmemBytes[2][2] = {{(uint32_t)sizeof(DecSmem<2, false>), (uint32_t)sizeof(DecSmem<2, true>)},
                                          {(uint32_t)sizeof(DecSmem<4, false>), (uint32_t)sizeof(DecSmem<4, true>)}};


__device__ __forceinline__ void prefetch_l2(const void* p) {
#ifndef CHK_CPU_EMULATION
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
#else
    (void)p;
#endif
}

struct DecChain {
    uint32_t x;
    uint32_t rel;      // read position relative to blk0 * 32
    uint32_t rel_end;  // where a valid stream ends
    uint32_t loaded;   // 32-byte blocks requested so far
    uint32_t max_blocks;
    unsigned long long blk0;
    uint4 pend0, pend1;  // block requested at the previous check, not yet in the ring
    bool has_pend;
};

// A lane reads its stream forward in aligned 32-byte blocks -- one DRAM sector each, so the
// scattered requests of a warp's lanes are as few as they can be -- into a ring of two.
// The next block is REQUESTED at the first check point after the read position has entered
// the newer of the two blocks, and is only moved into the ring (over the older one) at the
// following check point, 8 symbols later, so the load latency hides behind decode work.  A
// group of 8 symbols consumes at most 16 bytes, so more than 16 unread bytes are in the
// ring at the request and the new block is in place before they run out.
// A valid stream never needs bytes past its own end; a damaged one could run ahead, so
// requests stop one block after the lane's last byte (the lane then decodes stale bytes
// and fails its end check).
__device__ __forceinline__ void dec_request(DecChain& c, const uint8_t* __restrict__ payload) {
    if (c.loaded < c.max_blocks) {
        const uint8_t* src = payload + (c.blk0 + c.loaded) * 32;
        c.pend0 = ld_global_v4(src);
        c.pend1 = ld_global_v4(src + 16);
        c.has_pend = true;
        // start the block after this one on its way from DRAM to L2: by the time it is
        // requested (some 36 symbols from now) the request is a short L2 hit
        if (c.loaded + 1 < c.max_blocks) prefetch_l2(src + 32);
    }
    ++c.loaded;
}
// ring_words: this lane's ring word 0; its word w is at ring_words[w * 32]
__device__ __forceinline__ void dec_commit(DecChain& c, uint32_t* ring_words) {
    if (c.has_pend) {
        const uint32_t r = ((c.loaded - 1) & 1) * 8;
        ring_words[(r + 0) * 32] = c.pend0.x;
        ring_words[(r + 1) * 32] = c.pend0.y;
        ring_words[(r + 2) * 32] = c.pend0.z;
        ring_words[(r + 3) * 32] = c.pend0.w;
        ring_words[(r + 4) * 32] = c.pend1.x;
        ring_words[(r + 5) * 32] = c.pend1.y;
        ring_words[(r + 6) * 32] = c.pend1.z;
        ring_words[(r + 7) * 32] = c.pend1.w;
        if (r == 0) ring_words[16 * 32] = c.pend0.x;  // word 0 again behind word 15
        c.has_pend = false;
    }
}

// acc with its byte P replaced by the low byte of v
__device__ __forceinline__ uint32_t put_byte(uint32_t acc, uint32_t v, uint32_t P) {
    const uint32_t sel = P == 0 ? 0x3214u : P == 1 ? 0x3240u : P == 2 ? 0x3410u : 0x4210u;  // folds once unrolled
    return __byte_perm(acc, v, sel);
}

// One decode step: look the slot up, step the state back, and pull in 0, 1 or 2
// stream bytes without branching: the two candidate bytes are placed at the top
// of a word and funnel-shifted into the state by 0, 8 or 16 bits.  Returns the
// table entry (symbol in its low byte).
template <bool ZS>
__device__ __forceinline__ uint32_t dec_step(DecChain& c, const uint32_t* dtab, int s1, const uint8_t* ring_bytes) {
    const uint32_t slot = c.x & (kM - 1);
    const uint32_t xs = c.x >> kScaleBits;
    uint32_t x, sym;
    if (ZS) {
        const int m = max((int)slot, s1);
        const uint32_t e = dtab[m - s1];
        sym = e;
        x = ((e >> 8) & 0xFFFu) * xs + xs + ((e >> 20) + (slot - (uint32_t)m));
    } else {
        const uint32_t e = dtab[slot];
        sym = e;
        x = ((e >> 8) & 0xFFFu) * xs + xs + (e >> 20);
    }
    // the two stream bytes at the read position: the ring word that holds the first one and its
    // successor (two conflict-free loads), shifted down by the position inside the word
    const uint32_t* rw = reinterpret_cast<const uint32_t*>(ring_bytes + ((c.rel << 5) & 0x780u));  // word (rel >> 2) & 15
    const uint32_t pair = __funnelshift_r(rw[0], rw[32], c.rel << 3);  // shift count is taken mod 32: 8 * (rel & 3)
    const uint32_t top = __byte_perm(pair, 0u, 0x0144);  // first byte to bits 31..24, second to bits 23..16
    // bytes to pull in: 0 for x >= 2^23, 1 for x >= 2^15, else 2 (a valid state is never below 2^11)
    const uint32_t t = (uint32_t)__clz((int)x) - 1u;
    c.x = __funnelshift_l(top, x, t & 24u);
    c.rel += t >> 3;
    return sym;
}

template <int NV, int B0, bool ZS>
__device__ __forceinline__ void decode_tensor(const TensorDesc& d, uint32_t ti,
                                              const uint32_t* __restrict__ freq_tables,
                                              const uint32_t* __restrict__ cum_tables,
                                              const LaneHeader* __restrict__ hdrs,
                                              const uint8_t* __restrict__ payload,
                                              const uint8_t* __restrict__ sidecar, uint32_t check_zero_lanes,
                                              uint32_t* __restrict__ status, unsigned char* smem_raw) {
    DecSmem<NV, ZS>* sm = reinterpret_cast<DecSmem<NV, ZS>*>(smem_raw);
    const uint32_t j = threadIdx.x;
    const unsigned long long B = d.n_bytes;

    // ---- slot table
    (void)freq_tables;  // frequencies are differences of the prefix sums
    const uint32_t* cq = cum_tables + (size_t)d.table_idx * 257;
    for (uint32_t i = j; i < 257; i += kTeam) sm->cum[i] = cq[i];
    __syncthreads();
    // zero-skip: slots below `skip` (all symbol 0) share entry 0; the host sends only tensors that fit
    const uint32_t f0 = sm->cum[1];
    const uint32_t skip = ZS ? (f0 < 2048u ? f0 : 2048u) : 0u;
    const int s1 = (int)skip - 1;
    for (uint32_t slot = skip + j; slot < kM; slot += kTeam) {
        uint32_t lo = 0, hi = 256;  // last s with cum[s] <= slot
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (sm->cum[mid] <= slot) lo = mid; else hi = mid;
        }
        const uint32_t e = lo | ((sm->cum[lo + 1] - sm->cum[lo] - 1) << 8) | ((slot - sm->cum[lo]) << 20);
        if (ZS) {
            if (slot - (uint32_t)s1 < kZsEntries) sm->dtab[slot - (uint32_t)s1] = e;
        } else {
            sm->dtab[slot] = e;
        }
    }
    if (ZS && j == 0 && skip) sm->dtab[0] = ((f0 - 1u) << 8) | ((uint32_t)s1 << 20);

    DecChain ch[NV];
    uint32_t* ringw[NV];
    const uint8_t* ringb[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const uint32_t t = 4 * j + chain_byte<NV, B0>(k);
        const LaneHeader h = hdrs[(size_t)ti * kLanes + t];
        const unsigned long long p_abs = d.payload_off + h.buf_offset;
        ch[k].x = h.final_state;
        ch[k].blk0 = p_abs >> 5;
        ch[k].rel = (uint32_t)(p_abs & 31);
        ch[k].rel_end = ch[k].rel + h.byte_count;
        ch[k].max_blocks = ((ch[k].rel_end + 31) >> 5) + 1;
        ch[k].loaded = 0;
        ch[k].has_pend = false;
        ringw[k] = sm->ring + (size_t)(k * (kTeam / 32) + (j >> 5)) * (kRingWords * 32) + (j & 31);
        ringb[k] = reinterpret_cast<const uint8_t*>(ringw[k]);
        if (B > t) {  // the lane has symbols: start with both blocks of the ring filled
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                dec_request(ch[k], payload);
                dec_commit(ch[k], ringw[k]);
            }
        }
    }
    __syncthreads();  // table complete

    const unsigned long long full_rows = B >> 8;
    const uint32_t tail = (uint32_t)(B & 255);
    const bool dst4 = (reinterpret_cast<uintptr_t>(d.dst) & 3) == 0;
    const bool side2 = NV == 2 && ((reinterpret_cast<uintptr_t>(sidecar) + d.sidecar_off) & 1) == 0;
    uint8_t* col = d.dst + 4 * j;

    // low bytes of the word of row r: fp32 -> element 64r+j (2 bytes); bf16 -> elements 128r+2j, +1
    auto side_word = [&](unsigned long long r) -> uint32_t {
        if (NV == 4) return 0u;
        const uint8_t* sp = sidecar + d.sidecar_off + (r << 7) + 2 * j;
        const uint32_t s = side2 ? (uint32_t)*reinterpret_cast<const uint16_t*>(sp)
                                 : ((uint32_t)sp[0] | ((uint32_t)sp[1] << 8));
        return B0 == 2 ? s : ((s & 0xFFu) | ((s & 0xFF00u) << 8));
    };
    auto store_word = [&](unsigned long long r, uint32_t w) {
        uint8_t* p = col + (r << 8);
        if (dst4) {
            *reinterpret_cast<uint32_t*>(p) = w;
        } else {
            p[0] = (uint8_t)w;
            p[1] = (uint8_t)(w >> 8);
            p[2] = (uint8_t)(w >> 16);
            p[3] = (uint8_t)(w >> 24);
        }
    };

    unsigned long long r = 0;
    uint32_t side_next[8];
    if (8 <= full_rows) {
#pragma unroll
        for (int u = 0; u < 8; ++u) side_next[u] = side_word(u);
    }
    while (r + 8 <= full_rows) {
        uint32_t side[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) side[u] = side_next[u];
        if (r + 16 <= full_rows) {  // low bytes of the next group, requested ahead of use
#pragma unroll
            for (int u = 0; u < 8; ++u) side_next[u] = side_word(r + 8 + u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            uint32_t acc = side[u];
#pragma unroll
            for (int k = 0; k < NV; ++k) acc = put_byte(acc, dec_step<ZS>(ch[k], sm->dtab, s1, ringb[k]), chain_byte<NV, B0>(k));
            store_word(r + u, acc);
        }
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            dec_commit(ch[k], ringw[k]);
            // reading from the newer block: the older one can be replaced
            if (ch[k].rel >= (ch[k].loaded - 1) * 32) dec_request(ch[k], payload);
        }
        r += 8;
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) dec_commit(ch[k], ringw[k]);
    // remaining full rows and the partial row: at most 8 steps per chain
    for (; r < full_rows; ++r) {
        uint32_t acc = side_word(r);
#pragma unroll
        for (int k = 0; k < NV; ++k) acc = put_byte(acc, dec_step<ZS>(ch[k], sm->dtab, s1, ringb[k]), chain_byte<NV, B0>(k));
        store_word(r, acc);
    }
    if (tail) {
        uint32_t acc = 0;
#pragma unroll
        for (int k = 0; k < NV; ++k)
            if (4 * j + chain_byte<NV, B0>(k) < tail) acc = put_byte(acc, dec_step<ZS>(ch[k], sm->dtab, s1, ringb[k]), chain_byte<NV, B0>(k));
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            const uint32_t t = 4 * j + b;
            if (t >= tail) continue;
            const unsigned long long gi = (full_rows << 8) + t;
            const uint32_t jb = (uint32_t)(gi % d.es);
            d.dst[gi] = jb < d.spe ? sidecar[d.sidecar_off + (gi / d.es) * d.spe + jb] : (uint8_t)(acc >> (8 * b));
        }
    }

    uint32_t err = 0;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        if (ch[k].x != kL) err |= kErrEndState;
        if (ch[k].rel != ch[k].rel_end) err |= kErrEndPointer;
    }
    if (NV == 2 && check_zero_lanes) {
        // optional: replay the lanes that only carry zeroed bytes and check their end state
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            if (b == (uint32_t)B0 || b == 3u) continue;
            const uint32_t t = 4 * j + b;
            const unsigned long long n = B > t ? (B - t + kLanes - 1) / kLanes : 0;
            const LaneHeader h = hdrs[(size_t)ti * kLanes + t];
            const uint8_t* p = payload + d.payload_off + h.buf_offset;
            const uint8_t* const end = p + h.byte_count;
            uint32_t x = h.final_state;
            bool bad = false;
            for (unsigned long long i = 0; i < n && !bad; ++i) {
                const uint32_t slot = x & (kM - 1);
                const int m = ZS ? max((int)slot, s1) : (int)slot;
                const uint32_t e = sm->dtab[ZS ? m - s1 : (int)slot];
                if (e & 0xFFu) bad = true;  // must decode to symbol 0
                x = (((e >> 8) & 0xFFFu) + 1u) * (x >> kScaleBits) + (e >> 20) + (slot - (uint32_t)m);
                while (x < kL && !bad) {
                    if (p >= end) bad = true; else x = (x << 8) | *p++;
                }
            }
            if (bad || p != end) err |= kErrEndPointer;
            if (x != kL) err |= kErrEndState;
        }
    }
    if (err) atomicOr(&status[ti], err);
    __syncthreads();  // table and rings are reused by the next tensor
}

// One team (CTA of 64 threads) per tensor.  Each thread rebuilds one 32-bit word
// of every row from its decoded bytes and the sidecar and stores it directly.
// kInts as for the encoder; ZS selects the table shape.
#ifndef CHK_DEC_MINBLOCKS
#define CHK_DEC_MINBLOCKS 1
#endif
#ifndef CHK_DEC_ZS_MINBLOCKS
#define CHK_DEC_ZS_MINBLOCKS 10
#endif
template <bool kInts, bool ZS>
__global__ void __launch_bounds__(kTeam, ZS ? CHK_DEC_ZS_MINBLOCKS : CHK_DEC_MINBLOCKS) rans_decode_kernel(const TensorDesc* __restrict__ descs,
                                                            const uint32_t* __restrict__ freq_tables,  // [T][256]
                                                            const uint32_t* __restrict__ cum_tables,   // [T][257]
                                                            const LaneHeader* __restrict__ hdrs,
                                                            const uint8_t* __restrict__ payload,
                                                            const uint8_t* __restrict__ sidecar,
                                                            const uint32_t* __restrict__ order,
                                                            uint32_t* __restrict__ ticket, uint32_t n_tensors,
                                                            uint32_t check_zero_lanes,
                                                            uint32_t* __restrict__ status /* per tensor */) {
    CHK_DYN_SMEM(smem);
    CHK_SHARED uint32_t s_ticket;
    for (;;) {
        const uint32_t tk = next_ticket(ticket, &s_ticket);
        if (tk >= n_tensors) break;
        const uint32_t ti = order[tk];
        const TensorDesc d = descs[ti];
        if (d.flags & kFlagRaw) {  // payload is the masked tensor
            const uint8_t* in = payload + d.payload_off;
            for (unsigned long long i = threadIdx.x; i < d.n_bytes; i += kTeam) {
                const uint32_t jb = (uint32_t)(i % d.es);
                d.dst[i] = jb < d.spe ? sidecar[d.sidecar_off + (i / d.es) * d.spe + jb] : in[i];
            }
            __syncthreads();  // s_ticket may be rewritten only after everyone has read it
            continue;
        }
        if (d.es == 4 && d.spe == 2)
            decode_tensor<2, 2, ZS>(d, ti, freq_tables, cum_tables, hdrs, payload, sidecar, check_zero_lanes, status, smem);
        else if (d.es == 2 && d.spe == 1)
            decode_tensor<2, 1, ZS>(d, ti, freq_tables, cum_tables, hdrs, payload, sidecar, check_zero_lanes, status, smem);
        else if (kInts)
            decode_tensor<4, 0, ZS>(d, ti, freq_tables, cum_tables, hdrs, payload, sidecar, check_zero_lanes, status, smem);
        else
            __syncthreads();
    }
}

}  // namespace chk

// ------------------------------------------------------------------ container version 3: planes -> whole elements
// A floating-point tensor of container version 3 is stored as one 8-bit stream per high byte plane plus raw low
// bytes (plane_kernels.cuh).  rans_decode_planes_kernel restores it without writing the planes to memory.  A team
// has 64 threads per plane (kPlanes = 2: 4-byte elements, 1: 2-byte elements); a thread decodes four
// neighbouring lanes 4c..4c+3 of its plane exactly as the 8-bit path of rans_decode_kernel does.  With two planes
// the threads of a warp are split 16 + 16: lane l and lane l + 16 hold the two high bytes of the SAME four
// elements, swap their words with one shuffle per row, and each writes two whole elements (its own low bytes,
// both high bytes) -- no barrier and no shared-memory staging inside the loop, stores coalesced.  A plane
// stored raw (passthrough rule) is read instead of decoded.
namespace chk {

struct PlaneItem {                  // one stored plane
    unsigned long long payload_off; // start of its payload in the payload section
    uint32_t hdr_index;             // its lane headers are hdrs[hdr_index * 256 ...]
    uint32_t table_idx;
    uint32_t raw;                   // payload is the plane itself
    uint32_t status_index;          // where a failed stream check is recorded
};
struct PlaneGroup {                 // one tensor
    uint8_t* dst;
    const uint8_t* low;             // its low bytes (n * spe)
    unsigned long long n_elem;
    PlaneItem plane[2];             // [0] the lower plane, [kPlanes - 1] the sign/exponent plane
};

template <int kPlanes>
struct PlaneDecSmem {
    uint32_t dtab[kPlanes][kM];
    uint32_t ring[4 * kPlanes * kTeam * kRingWords];  // per chain index and warp: 17 words x 32 lanes, interleaved
    uint32_t cum[kPlanes][260];
};

template <int kPlanes>
__device__ __forceinline__ void decode_plane_group(const PlaneGroup& g, const uint32_t* __restrict__ cum_tables,
                                                   const LaneHeader* __restrict__ hdrs,
                                                   const uint8_t* __restrict__ payload, uint32_t* __restrict__ status,
                                                   unsigned char* smem_raw) {
    constexpr uint32_t kThreads = kPlanes * kTeam;
    constexpr uint32_t kWarps = kThreads / 32;
    constexpr uint32_t ES = kPlanes * 2;         // element size: low bytes and high bytes are half each
    PlaneDecSmem<kPlanes>* sm = reinterpret_cast<PlaneDecSmem<kPlanes>*>(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // plane of this thread and its column c: it decodes lanes 4c .. 4c+3 of that plane
    const uint32_t h = kPlanes == 2 ? lane >> 4 : 0u;
    const uint32_t c = kPlanes == 2 ? (warp << 4) | (lane & 15u) : tid;
    const PlaneItem it = g.plane[h];
    const unsigned long long B = g.n_elem;       // bytes of a plane

    // ---- the slot tables (threads t, t + kThreads, ... of the team build both)
    for (uint32_t p = 0; p < (uint32_t)kPlanes; ++p) {
        if (g.plane[p].raw) continue;
        const uint32_t* cq = cum_tables + (size_t)g.plane[p].table_idx * 257;
        for (uint32_t i = tid; i < 257; i += kThreads) sm->cum[p][i] = cq[i];
    }
    __syncthreads();
    for (uint32_t p = 0; p < (uint32_t)kPlanes; ++p) {
        if (g.plane[p].raw) continue;
        for (uint32_t slot = tid; slot < kM; slot += kThreads) {
            uint32_t lo = 0, hi = 256;  // last s with cum[s] <= slot
            while (hi - lo > 1) {
                const uint32_t mid = (lo + hi) >> 1;
                if (sm->cum[p][mid] <= slot) lo = mid; else hi = mid;
            }
            sm->dtab[p][slot] = lo | ((sm->cum[p][lo + 1] - sm->cum[p][lo] - 1) << 8) | ((slot - sm->cum[p][lo]) << 20);
        }
    }

    DecChain ch[4];
    uint32_t* ringw[4];
    const uint8_t* ringb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t t = 4 * c + k;
        LaneHeader lh{kL, 0, 0, 0};
        if (!it.raw) lh = hdrs[(size_t)it.hdr_index * kLanes + t];
        const unsigned long long p_abs = it.payload_off + lh.buf_offset;
        ch[k].x = lh.final_state;
        ch[k].blk0 = p_abs >> 5;
        ch[k].rel = (uint32_t)(p_abs & 31);
        ch[k].rel_end = ch[k].rel + lh.byte_count;
        ch[k].max_blocks = ((ch[k].rel_end + 31) >> 5) + 1;
        ch[k].loaded = 0;
        ch[k].has_pend = false;
        ringw[k] = sm->ring + (size_t)(k * kWarps + warp) * (kRingWords * 32) + lane;
        ringb[k] = reinterpret_cast<const uint8_t*>(ringw[k]);
        if (!it.raw && B > t) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                dec_request(ch[k], payload);
                dec_commit(ch[k], ringw[k]);
            }
        }
    }
    __syncthreads();  // tables complete

    const unsigned long long full_rows = B >> 8;
    const uint32_t tail = (uint32_t)(B & 255);
    const uint32_t* const dtab = sm->dtab[h];
    const uint8_t* raw_col = payload + it.payload_off + 4 * c;  // a raw plane: the thread's word of every row
    const bool raw4 = (reinterpret_cast<uintptr_t>(raw_col) & 3) == 0;
    const bool dst_ok = (reinterpret_cast<uintptr_t>(g.dst) & 7) == 0, low_ok = (reinterpret_cast<uintptr_t>(g.low) & 3) == 0;
    // the elements this thread writes in a row: two planes -> 4c + 2h, 4c + 2h + 1; one plane -> 4c .. 4c + 3
    const uint32_t e0 = kPlanes == 2 ? 4 * c + 2 * h : 4 * c;

    // the four bytes of this thread's plane in row r (kRaw: the plane may be a stored-raw one)
    auto row_word = [&](unsigned long long r, auto may_be_raw) -> uint32_t {
        if (decltype(may_be_raw)::value && it.raw) return load_row_word(raw_col + (r << 8), raw4);
        uint32_t acc = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc = put_byte(acc, dec_step<false>(ch[k], dtab, 0, ringb[k]), k);
        return acc;
    };
    // the low bytes of the thread's elements in row r: four bytes either way
    auto low_word = [&](unsigned long long r) -> uint32_t {
        const uint8_t* lp = g.low + ((r << 8) + e0) * (ES / 2);
        return low_ok ? *reinterpret_cast<const uint32_t*>(lp)
                      : ((uint32_t)lp[0] | ((uint32_t)lp[1] << 8) | ((uint32_t)lp[2] << 16) | ((uint32_t)lp[3] << 24));
    };
    // whole elements of row r from the thread's plane word, its partner's, and the low bytes: 8 bytes
    auto assemble = [&](uint32_t w, uint32_t lw) -> uint2 {
        uint2 o;
        if (kPlanes == 2) {
            const uint32_t pw = __shfl_xor_sync(0xffffffffu, w, 16);
            const uint32_t p2 = h ? pw : w, p3 = h ? w : pw;            // the lower and the upper high byte
            const uint32_t a = h ? p2 >> 16 : p2, b = h ? p3 >> 16 : p3;  // this thread's two elements
            o.x = (lw & 0xFFFFu) | ((a & 0xFFu) << 16) | ((b & 0xFFu) << 24);
            o.y = (lw >> 16) | (((a >> 8) & 0xFFu) << 16) | (((b >> 8) & 0xFFu) << 24);
        } else {
            o.x = __byte_perm(lw, w, 0x5140);
            o.y = __byte_perm(lw, w, 0x7362);
        }
        return o;
    };
    auto store_row = [&](unsigned long long r, uint2 o) {
        uint8_t* dp = g.dst + ((r << 8) + e0) * ES;
        if (dst_ok) {
            *reinterpret_cast<uint2*>(dp) = o;
        } else {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                dp[b] = (uint8_t)(o.x >> (8 * b));
                dp[4 + b] = (uint8_t)(o.y >> (8 * b));
            }
        }
    };

    unsigned long long r = 0;
    // groups of 8 rows; the loop exists twice so that a team without a raw plane carries no test for one
    auto groups_of_8 = [&](auto may_be_raw) {
        uint32_t lw_next[8];
        if (8 <= full_rows) {
#pragma unroll
            for (int u = 0; u < 8; ++u) lw_next[u] = low_word(u);
        }
        while (r + 8 <= full_rows) {
            uint32_t lw[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) lw[u] = lw_next[u];
            if (r + 16 <= full_rows) {  // low bytes of the next group, requested ahead of use
#pragma unroll
                for (int u = 0; u < 8; ++u) lw_next[u] = low_word(r + 8 + u);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) store_row(r + u, assemble(row_word(r + u, may_be_raw), lw[u]));
            if (!(decltype(may_be_raw)::value && it.raw)) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    dec_commit(ch[k], ringw[k]);
                    if (ch[k].rel >= (ch[k].loaded - 1) * 32) dec_request(ch[k], payload);
                }
            }
            r += 8;
        }
    };
    bool any_raw = false;
    for (uint32_t p = 0; p < (uint32_t)kPlanes; ++p) any_raw = any_raw || g.plane[p].raw;
    if (any_raw) groups_of_8(std::true_type{}); else groups_of_8(std::false_type{});
    if (!it.raw) {
#pragma unroll
        for (int k = 0; k < 4; ++k) dec_commit(ch[k], ringw[k]);
    }
    // remaining full rows (at most 7)
    for (; r < full_rows; ++r) store_row(r, assemble(row_word(r, std::true_type{}), low_word(r)));
    // the partial row: elements r*256 .. r*256 + tail, byte by byte
    if (tail) {
        uint32_t acc = 0;
        if (it.raw) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (4 * c + k < tail) acc |= (uint32_t)payload[it.payload_off + (r << 8) + 4 * c + k] << (8 * k);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (4 * c + k < tail) acc = put_byte(acc, dec_step<false>(ch[k], dtab, 0, ringb[k]), k);
        }
        uint32_t p2 = acc, p3 = 0;  // one plane: its bytes 0..3 belong to elements 4c..4c+3
        if (kPlanes == 2) {
            const uint32_t pw = __shfl_xor_sync(0xffffffffu, acc, 16);
            p2 = h ? pw >> 16 : acc;  // bytes 0, 1: the thread's two elements
            p3 = h ? acc >> 16 : pw;
        }
        const uint32_t mine = kPlanes == 2 ? 2u : 4u;
        for (uint32_t q = 0; q < mine; ++q) {
            const uint32_t e = e0 + q;
            if (e >= tail) break;
            const unsigned long long ge = (r << 8) + e;
            uint8_t* dp = g.dst + ge * ES;
            for (uint32_t b = 0; b < ES / 2; ++b) dp[b] = g.low[ge * (ES / 2) + b];
            dp[ES / 2] = (uint8_t)(p2 >> (8 * q));
            if (kPlanes == 2) dp[ES / 2 + 1] = (uint8_t)(p3 >> (8 * q));
        }
    }

    if (!it.raw) {
        uint32_t err = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (ch[k].x != kL) err |= kErrEndState;
            if (ch[k].rel != ch[k].rel_end) err |= kErrEndPointer;
        }
        if (err) atomicOr(&status[it.status_index], err);
    }
    __syncthreads();  // tables and rings are reused by the next tensor
}

template <int kPlanes>
__global__ void __launch_bounds__(kPlanes * kTeam, kPlanes == 2 ? 3 : 6) rans_decode_planes_kernel(const PlaneGroup* __restrict__ groups,
                                                                            const uint32_t* __restrict__ cum_tables,
                                                                            const LaneHeader* __restrict__ hdrs,
                                                                            const uint8_t* __restrict__ payload,
                                                                            const uint32_t* __restrict__ order,
                                                                            uint32_t* __restrict__ ticket, uint32_t n_groups,
                                                                            uint32_t* __restrict__ status) {
    CHK_DYN_SMEM(smem);
    CHK_SHARED uint32_t s_ticket;
    for (;;) {
        const uint32_t tk = next_ticket(ticket, &s_ticket);
        if (tk >= n_groups) break;
        decode_plane_group<kPlanes>(groups[order[tk]], cum_tables, hdrs, payload, status, smem);
    }
}

}  // namespace chk
