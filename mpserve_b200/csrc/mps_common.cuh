// Shared device helpers: the MSB-first bit window, cache-hinted loads/stores, error plumbing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mpserve_b200.h"

namespace mps {

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define MPS_CUDA_TRY(expr)                                       \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) return ::mps::cuda_fail(_e, #expr); \
    } while (0)

// ---------------------------------------------------------------------------------------------
// Streaming global accesses.  Context bytes are read exactly once and BF16 output is written
// exactly once, so neither should displace the bitstream sectors that each sub-stream re-reads
// from L1 (a 32-byte sector serves eight consecutive 32-bit refills of one sub-stream).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_stream_u8(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const uint8_t* p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u64(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_u16(uint16_t* p, uint32_t v) {
    asm volatile("st.global.cs.u16 [%0], %1;" ::"l"(p), "h"((uint16_t)v) : "memory");
}
__device__ __forceinline__ void st_stream_u32(uint16_t* p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_stream_v2(uint16_t* p, uint32_t a, uint32_t b) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_stream_v4(uint16_t* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Bit window over an MSB-first stream of u64 words.
//
// The stream is addressed in 32-bit units in bit order: unit r of a stream that starts at the
// u64-aligned pointer `bs32` lives at bs32[r ^ 1] (the high half of a little-endian u64 comes
// first in bit order).  `hi:lo` hold the next `avail` unread bits left-aligned, everything below
// is zero.  Invariant between symbols of the fast path: avail >= 33 at the start of every run of
// RP = 32/L symbols, which leaves >= L bits for each peek and >= 1 bit before the refill.
// Loads are clamped to `lim` (the last valid unit of the bitstream): a prefix code never looks at
// bits past its own end, so clamped garbage past the end of the last sub-stream is harmless and
// nothing is ever read out of bounds, whatever the start offsets say.
// ---------------------------------------------------------------------------------------------
struct BitWin {
    uint32_t hi, lo;
    int avail;
    uint32_t r;  // next unread 32-bit unit, relative to bs32
};

__device__ __forceinline__ uint32_t ld_unit(const uint32_t* __restrict__ bs32, uint32_t r, uint32_t lim) {
    return __ldg(bs32 + min(r ^ 1u, lim));
}

__device__ __forceinline__ void win_init(BitWin& w, const uint32_t* __restrict__ bs32, uint32_t lim, uint32_t bit) {
    const uint32_t r0 = bit >> 5, off = bit & 31u;
    const uint32_t a = ld_unit(bs32, r0, lim), b = ld_unit(bs32, r0 + 1, lim);
    w.hi = __funnelshift_l(b, a, off);
    w.lo = b << off;
    w.avail = 64 - (int)off;
    w.r = r0 + 2;
}

__device__ __forceinline__ void win_consume(BitWin& w, uint32_t nbits) {
    w.hi = __funnelshift_l(w.lo, w.hi, nbits);
    w.lo <<= nbits;
    w.avail -= (int)nbits;
}

// Append one 32-bit unit below the valid bits; requires avail <= 32 (then lo == 0).
__device__ __forceinline__ void win_refill(BitWin& w, const uint32_t* __restrict__ bs32, uint32_t lim) {
    const uint32_t nx = ld_unit(bs32, w.r, lim);
    w.hi |= __funnelshift_rc(nx, 0u, (uint32_t)w.avail);
    w.lo = __funnelshift_rc(0u, nx, (uint32_t)w.avail);
    w.avail += 32;
    w.r += 1;
}

}  // namespace mps
