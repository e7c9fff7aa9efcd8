// Bucketed sub-stream Huffman decode for the FP8 (L=7, 256 contexts) and AWQ-INT4 (L=11, 16
// contexts) sidecar formats, rectangular or ragged buckets, one tensor or a whole model per launch.
//
// Format recap (what the encoder guarantees, kernel/build_huffman.cu:811-918 in the reference):
// bucket b owns rows x column-window (or a list of groups); its elements, flattened row-major to
// e in [0,total), are dealt round-robin to k_eff = min(k, max(1,total)) sub-streams: sub-stream t
// holds e = t, t+k_eff, ... as one contiguous run of prefix codes starting at bit
// bucket_bit_base[b] + startbit[b][t].  The code of an element is chosen by its context byte (the
// FP8 byte / INT4 code): gid = bucket_table[b][ctx] selects a 2^L-entry lookup table.
//
// Design for B200:
//  * persistent CTAs (one per SM: the fused table takes 128 KB of shared memory) pull work items
//    (tensor, bucket, chunk of sub-streams) from a global counter; a scout warp prepares the next item
//    while the current one is decoded;
//  * per item the bucket's tables are fused once into 32-bit entries sym << 16 | esc | len laid out
//    [ctx][prefix], so a symbol costs ONE shared-memory load; staging is skipped when the next item
//    uses the same tables; tables that are one run of table ids (what the reference encoder writes) are
//    bulk-copied raw into the table's own space and expanded in place;
//  * each thread decodes CH adjacent sub-streams in lock-step: CH independent dependency chains for
//    ILP, one CH-byte context read and one 2*CH-byte BF16 store per step, both fully coalesced across
//    the warp; context bytes arrive through cp.async.bulk issued by a producer warp (a block of eight
//    steps at a time, one copy per row the block touches, everything worked out before the warp waits
//    for the block's stage to come free: the three-stage ring runs close to dry), the bitstream through
//    a ring of 16-byte cp.async chunks per sub-stream, or whole with one bulk copy when the bucket's code
//    bits fit the rings' space;
//  * every sub-stream decodes from a 32-bit left-aligned window that is rebuilt from its bit position
//    every (32 - L) / L + 1 symbols, branch-free, so that the rebuild is warp-uniform;
//  * ESC (raw 16-bit symbol after the code) is rare: buckets whose tables contain no ESC entry run
//    a loop with no ESC test at all; the others test per symbol.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "stream_common.cuh"

namespace mps {

// ------------------------------------------------------------------------------------------------
// error plumbing
// ------------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s failed: %s", what, cudaGetErrorString(e));
    return (int)e;
}

// ------------------------------------------------------------------------------------------------
// kernel
// ------------------------------------------------------------------------------------------------
constexpr int kTableEntries = 32768;  // 256 ctx x 2^7 == 16 ctx x 2^11
constexpr int kRowCap = 1024;         // rows / groups of a bucket cached in shared memory
constexpr int kSteps = 4;             // steps per software-pipeline block (register-prefetch path)
constexpr int kSS = 8;                // steps per stage of the streaming path's context ring
constexpr int kLook = 1;              // bitstream units requested ahead of use, per sub-stream (register-prefetch path)


constexpr int kStages = 3;                     // context-byte ring: stages of kSS steps each for the widest items
constexpr int kMaxStages = 4;                  // narrower items split the same ring into more stages
static_assert(kMaxStages >= kStages, "the widest items use kStages stages");
// Stages of the context ring for items of `span` sub-streams: a narrow item leaves each decoding
// thread waiting on memory latency rather than on issue slots, so it needs more steps in flight.
__host__ __device__ constexpr uint32_t ring_stages(uint32_t span) {
    return (kStages * 1024u / span) < (uint32_t)kMaxStages ? (kStages * 1024u / span) : (uint32_t)kMaxStages;
}
constexpr int kMaxSpan = 1024;        // sub-streams per work item (threads x chains), at most


struct Smem {
    uint32_t tbl[kTableEntries];                 // fused entries: sym << 16 | esc << 15 | code length
    uint4 bitring[4 * kMaxSpan];                 // per sub-stream: four 16-byte chunks of its bitstream
    uint8_t ctxring[kStages * kSS * kMaxSpan];   // context bytes of the next kStages blocks of steps
    uint32_t rowbase[2][kRowCap];                // element offset of each row / group start (0xFFFFFFFF: invalid),
                                                 // one set for the item being decoded, one being prepared
    Prepared prep[2];
    mps_bucket_tensor tensor[2];                 // descriptor of the item's tensor, copied by the scout
    uint32_t stepofs[kMaxStages][kSS];           // element offset (row start + column) of every step of a stage
    uint32_t stepofs_b[kMaxStages][kSS];         // same for the sub-streams of a step that already sit in the next row
    uint32_t stepsplit[kMaxStages][kSS];         // first local sub-stream of a step that sits in the next row
    unsigned long long full_bar[kMaxStages];     // bulk copies of a stage have landed
    unsigned long long empty_bar[kMaxStages];    // every warp is done reading a stage
    int32_t gid[256];                            // context -> table id of the staged tables
    int32_t gid_next[256];                       // same for the prepared item (written by the scout once the
                                                 // decoding warps have taken the previous contents)
    int abort;                                   // a bounded wait gave up
    unsigned long long tab_bar;                  // the raw tables of the item have landed (bulk copy into the table's own space)
    uint32_t armed;                              // blocks of steps the producer has armed so far (abort path)
    uint32_t zero;                               // always 0; read back to tie an instruction to values it must wait for
};

static_assert(sizeof(Smem) <= 227 * 1024, "one CTA per SM: everything must fit the 227 KB a CTA can have");

// Entry layout.  L=7 (FP8): sym << 16 | raw length nibble (bits 0-2 code length, bit 3 = ESC), which a
// byte permute builds straight from the sidecar's packed arrays.  L=11 (AWQ): sym << 16 | esc << 15 |
// code length (lengths there go up to 11, so the ESC flag cannot share the low nibble).
template <int L> struct Entry {
    static constexpr uint32_t kEsc = (L == 7) ? 0x8u : 0x8000u;
    static constexpr uint32_t kLenMask = (L == 7) ? 0x7u : 0xFu;
};



// symbols sit in the HIGH half of an entry
template <int CH>
__device__ __forceinline__ void store_syms(uint16_t* p, const uint32_t (&e)[CH]) {
    if constexpr (CH == 1) st_stream_u16(p, e[0] >> 16);
    else if constexpr (CH == 2) st_stream_u32(p, __byte_perm(e[0], e[1], 0x7632));
    else if constexpr (CH == 4) st_stream_v2(p, __byte_perm(e[0], e[1], 0x7632), __byte_perm(e[2], e[3], 0x7632));
    else st_stream_v4(p, __byte_perm(e[0], e[1], 0x7632), __byte_perm(e[2], e[3], 0x7632),
                      __byte_perm(e[4], e[5], 0x7632), __byte_perm(e[6], e[7], 0x7632));
}

template <int L>
__device__ __forceinline__ uint32_t ctx_of(uint32_t byte) {
    if constexpr (L == 7) return byte;
    else return byte & 0xFu;
}

// ------------------------------------------------------------------------------------------------
// Fast path reader.  Decoding runs in blocks of RP = (32-L)/L + 1 symbols on a 32-bit window that
// is rebuilt at every block start from the sub-stream's bit position and two cached 32-bit units;
// a block consumes fewer than 32 bits, so at most one new unit is needed per block, and that unit
// was requested LOOK blocks earlier (software prefetch: the load has whole blocks of other work to
// complete behind).  Everything is branch-free: the unit load is a predicated instruction, the
// register rotation is selects, so the CH chains of a thread interleave freely.  Within a block a
// symbol costs: one funnel shift that fuses context and prefix into the table index, one shift to a
// byte address, one shared-memory load, one shift of the window by the entry's low bits, one add
// that accumulates the code lengths in the low half of a register.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lds_table(uint32_t addr) {  // the table is constant while decoding
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Unit r of the stream (bit order) is bs32[r ^ 1]; clamped to the last valid unit.  On an L2 miss
// the whole 128-byte line is brought into L2: the seven following sectors of this sub-stream
// then hit L2 (each sub-stream walks its own line, so L1 cannot hold all of them).
__device__ __forceinline__ uint32_t unit_addr_ofs(uint32_t r, uint32_t lim) { return min(r ^ 1u, lim); }

__device__ __forceinline__ uint32_t ld_unit_l2(const uint32_t* __restrict__ bs32, uint32_t r, uint32_t lim) {
    uint32_t v;
    asm volatile("ld.global.nc.L2::128B.u32 %0, [%1];" : "=r"(v) : "l"(bs32 + unit_addr_ofs(r, lim)));
    return v;
}
__device__ __forceinline__ void ld_unit_l2_if(uint32_t& v, const uint32_t* __restrict__ bs32, uint32_t r, uint32_t lim,
                                              uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %2, 0;\n\t@p ld.global.nc.L2::128B.u32 %0, [%1];\n\t}"
        : "+r"(v)
        : "l"(bs32 + unit_addr_ofs(r, lim)), "r"(pred));
}

template <int LOOK>
struct Chain {
    uint32_t pos;           // bit position relative to bs32
    uint32_t w[2 + LOOK];   // units pos>>5, +1, and LOOK prefetched ones
};

template <int LOOK>
__device__ __forceinline__ void chain_init(Chain<LOOK>& ch, const uint32_t* __restrict__ bs32, uint32_t lim, uint32_t pos) {
    ch.pos = pos;
    const uint32_t u = pos >> 5;
#pragma unroll
    for (int i = 0; i < 2 + LOOK; ++i) ch.w[i] = ld_unit_l2(bs32, u + i, lim);
}

// Advance by `used` (< 32) bits and return the fresh 32-bit window.
template <int LOOK>
__device__ __forceinline__ uint32_t chain_window(Chain<LOOK>& ch, const uint32_t* __restrict__ bs32, uint32_t lim,
                                                 uint32_t used) {
    const uint32_t np = ch.pos + used;
    const uint32_t cross = ((np ^ ch.pos) > 31u) ? 1u : 0u;  // moved into the next unit
    ch.pos = np;
#pragma unroll
    for (int i = 0; i < 1 + LOOK; ++i) ch.w[i] = cross ? ch.w[i + 1] : ch.w[i];
    ld_unit_l2_if(ch.w[1 + LOOK], bs32, (np >> 5) + 1 + LOOK, lim, cross);
    return __funnelshift_l(ch.w[1], ch.w[0], np);
}

// Vector path: CH adjacent sub-streams per thread, all CH elements of a step contiguous in memory.
template <int L, int CH, bool ESC>
__device__ __forceinline__ void decode_vec(const Smem& sm, const uint32_t* rowbase, const uint8_t* __restrict__ ctx_bytes,
                                           uint16_t* __restrict__ out, const uint32_t* __restrict__ bs32, uint32_t lim,
                                           const uint32_t* __restrict__ startbit, uint32_t bit_lo, uint32_t t0, uint32_t k_eff,
                                           uint32_t col_len, uint32_t nrows, uint32_t total) {
    constexpr int RP = ESC ? 1 : ((32 - L) / L + 1);  // symbols per 32-bit window
    constexpr int LOOK = kLook;
    static_assert(kSteps % RP == 0, "a block of steps must hold whole windows");
    using CT = typename Ctx<CH>::T;
    const uint32_t tbl = smem_u32(sm.tbl);

    Chain<LOOK> ch[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) chain_init(ch[c], bs32, lim, startbit[t0 + c] + bit_lo);

    const uint32_t nsteps = (total - t0 - 1) / k_eff + 1;  // t0 < k_eff <= total
    // (row, col) walk of the prefetcher; division only here, then incremental
    uint32_t p_rr = t0 / col_len;
    uint32_t p_cc = t0 - p_rr * col_len;
    uint32_t p_base = rowbase[p_rr];
    auto fetch = [&](uint32_t s, uint32_t& o, CT& v) {
        if (s < nsteps) {
            o = p_base + p_cc;
            v = Ctx<CH>::ld(ctx_bytes + o);
            p_cc += k_eff;
            if (p_cc >= col_len) {
                do { p_cc -= col_len; ++p_rr; } while (p_cc >= col_len);
                p_base = (p_rr < nrows) ? rowbase[p_rr] : 0u;
            }
        }
    };
    uint32_t offA[kSteps], offB[kSteps];
    CT valA[kSteps], valB[kSteps];
#pragma unroll
    for (int u = 0; u < kSteps; ++u) fetch((uint32_t)u, offA[u], valA[u]);

    uint32_t hi[CH], acc[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) acc[c] = 0;

    // `count` (<= kSteps) steps from one prefetched block
    auto run = [&](const uint32_t (&off)[kSteps], const CT (&val)[kSteps], uint32_t count) {
#pragma unroll
        for (int u = 0; u < kSteps; ++u) {
            if ((uint32_t)u < count) {
                if (u % RP == 0) {
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        hi[c] = chain_window(ch[c], bs32, lim, acc[c] & 0xFFFFu);
                        acc[c] = 0;
                    }
                }
                uint32_t e[CH];
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    // index = ctx << L | top L bits of the window, in one funnel shift
                    const uint32_t idx = __funnelshift_l(hi[c], ctx_of<L>(Ctx<CH>::byte(val[u], c)), L);
                    e[c] = lds_table(tbl + (idx << 2));
                    if constexpr (!ESC) {
                        hi[c] = __funnelshift_l(0u, hi[c], e[c]);  // shift by the low 5 bits = code length
                        acc[c] += e[c];                            // low half accumulates the lengths
                    } else {
                        uint32_t used = e[c] & Entry<L>::kLenMask;
                        if (e[c] & Entry<L>::kEsc) {                     // 16 raw bits follow the ESC code
                            e[c] = __funnelshift_l(0u, hi[c], used) & 0xFFFF0000u;
                            used += 16;
                        }
                        acc[c] = used;
                    }
                }
                store_syms<CH>(out + off[u], e);
            }
        }
    };

    uint32_t s0 = 0;
    for (;;) {
        if (s0 + kSteps > nsteps) { run(offA, valA, nsteps - s0); break; }
#pragma unroll
        for (int u = 0; u < kSteps; ++u) fetch(s0 + kSteps + u, offB[u], valB[u]);
        run(offA, valA, kSteps);
        s0 += kSteps;
        if (s0 + kSteps > nsteps) { run(offB, valB, nsteps - s0); break; }
#pragma unroll
        for (int u = 0; u < kSteps; ++u) fetch(s0 + kSteps + u, offA[u], valA[u]);
        run(offB, valB, kSteps);
        s0 += kSteps;
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming fast path: everything a work item reads from HBM arrives through asynchronous copies
// into shared memory, deep enough ahead of use to cover HBM latency at full rate (Little's law
// wants tens of KB in flight per SM; register prefetch gave a few KB).
//
//  * Context bytes: a dedicated producer warp issues cp.async.bulk (the TMA bulk-copy engine, no tensor
//    map, no multicast) of the SPAN contiguous bytes every step needs, kSS steps per stage, several
//    stages ahead; stages are handed over with full/empty mbarriers.  Consumers read their CH bytes
//    of a step with one conflict-free shared-memory load.
//  * Bitstream: each sub-stream owns a ring of kRingChunks 16-byte chunks in shared memory and keeps
//    the chunks ahead of its window requested with cp.async: at most one new request every CHK steps,
//    committed as a group by every thread and awaited with cp.async.wait_group LAG, where LAG follows
//    from the most bits CHK steps can consume (see stream_run).  The divergent access (every lane a
//    different 128-byte line) thus happens once per 16 bytes (~21 symbols) per sub-stream instead of
//    once per 4 bytes.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void lds_ordered_if(uint32_t& v, uint32_t addr, uint32_t pred) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %2, 0;\n\t@p ld.shared.u32 %0, [%1];\n\t}"
                 : "+r"(v) : "r"(addr), "r"(pred) : "memory");
}

constexpr int kRingChunks = 4;                        // 16-byte chunks of bitstream kept per sub-stream
constexpr uint32_t kRingBytes = 16u * kRingChunks;    // 64

// 32-bit unit x (bit order) of the stream sits at byte 4*(x^1); the ring keeps byte offsets mod 64.
__device__ __forceinline__ uint32_t ring_unit_addr(uint32_t ring, uint32_t x) {
    return ring + (((x ^ 1u) & (kRingBytes / 4 - 1)) << 2);
}

struct SChain {
    uint32_t pos;     // bit position relative to BitOrigin::base
    uint32_t w0, w1;  // units pos>>5 and (pos>>5)+1
    uint32_t next;    // next 16-byte chunk to request
};

// Move by `used` (< 32) bits and return the fresh 32-bit window.  Branch-free: the register
// rotation and the ring read are predicated on having moved into the next unit.
// MASK: 60 for a sub-stream's own ring of 64 bytes; kFlatMask when the bucket's whole bitstream lies in
// shared memory from `ring` on (every sub-stream then reads the same copy at its own position).
constexpr uint32_t kFlatBytes = sizeof(uint4) * 4 * 1024;   // the space of the rings: 64 KB
constexpr uint32_t kFlatMask = kFlatBytes - 4;
template <uint32_t MASK = 60u>
__device__ __forceinline__ uint32_t schain_window(SChain& ch, uint32_t ring, uint32_t used) {
    const uint32_t np = ch.pos + used;
    const uint32_t moved = np ^ ch.pos;
    // byte address of unit (np >> 5) + 1: units are 4 bytes, swapped in pairs (^4)
    uint32_t addr;
    asm("lop3.b32 %0, %1, 4, %2, 0x28;" : "=r"(addr) : "r"((np >> 3) + 4u), "n"(MASK));  // (x ^ 4) & MASK
    addr += ring;
    ch.pos = np;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.gt.u32 p, %2, 31;\n\t@p mov.u32 %0, %1;\n\t@p ld.shared.u32 %1, [%3];\n\t}"
        : "+r"(ch.w0), "+r"(ch.w1)
        : "r"(moved), "r"(addr)
        : "memory");
    return __funnelshift_l(ch.w1, ch.w0, np);
}

// Keep kRingChunks chunks requested from the one w1 sits in: at most one new request per call,
// which is enough as long as fewer than 128 bits are consumed between calls.  Chunk c lives in ring
// slot c % kRingChunks; slot reuse is safe because chunk c - kRingChunks lies wholly before w0.
__device__ __forceinline__ void schain_request(SChain& ch, uint32_t ring, const BitOrigin& bo) {
    const uint32_t need = (((ch.pos >> 5) + 1) >> 2) + kRingChunks;  // chunks below `need` must be on their way
    const uint32_t ofs = ch.next << 4;
    const uint8_t* src = bo.base + ofs;
    const uint32_t dst = ring + (ofs & (kRingBytes - 1));
    // a chunk past the end of the bitstream is never copied (its ring slot keeps stale bits that no
    // valid sub-stream decodes from); a bitstream that ends mid-chunk gives up its last 8 bytes alone
    asm volatile(
        "{\n\t.reg .pred p, q, r;\n\t"
        "setp.lt.u32 p, %0, %1;\n\t"
        "setp.le.and.u32 q, %4, %5, p;\n\t"
        "setp.eq.and.u32 r, %4, %6, p;\n\t"
        "@q cp.async.cg.shared.global [%2], [%3], 16;\n\t"
        "@r cp.async.ca.shared.global [%2], [%3], 8;\n\t"
        "@p add.u32 %0, %0, 1;\n\t}"
        : "+r"(ch.next)
        : "r"(need), "r"(dst), "l"(src), "r"(ofs), "r"(bo.last_ofs), "r"(bo.tail_ofs)
        : "memory");
}

// First chunks of a sub-stream (same rules as schain_request, plain control flow).
__device__ __forceinline__ void chunk_fetch(uint32_t ring, const BitOrigin& bo, uint32_t ofs) {
    const uint32_t dst = ring + (ofs & (kRingBytes - 1));
    if (ofs <= bo.last_ofs) cp_async_16(dst, bo.base + ofs);
    else if (ofs == bo.tail_ofs) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(bo.base + ofs) : "memory");
}

// Producer warp.  What a block of steps needs (where each step reads and writes, which bytes to copy) is
// worked out BEFORE the warp waits for the stage to come free: the path from "stage freed" to "bytes
// landed" is what the decoding warps end up waiting for, and it then holds only the arming of the "full"
// barrier, the stores of the offsets and the copies.  Lanes 0..kSS-1 issue one bulk copy each (the context
// bytes of one step; two where a step starts in one row and ends in the next).  The producer never
// decodes, so consumers are never held back by a slow sibling: they only ever wait for data.  Returns
// false if a stage never freed.
template <int SPAN, bool SPLIT>
__device__ __forceinline__ bool producer_run(Smem& sm, const StreamItem& it, uint32_t blk, uint32_t nblocks, int stall_block,
                                             uint32_t spin_limit) {
    constexpr uint32_t NST = ring_stages(SPAN);
    const uint32_t lane = threadIdx.x & 31u;
    // row and column of the first element of this lane's step of the block, kept running instead of divided out
    uint32_t run_r, run_c;
    {
        const unsigned long long e0 = (unsigned long long)lane * it.k_eff;
        run_r = (uint32_t)(e0 / it.col_len);
        run_c = (uint32_t)(e0 - (unsigned long long)run_r * it.col_len);
    }
    for (uint32_t jb = 0; jb < nblocks; ++jb) {
        const uint32_t g = blk + jb, stage = g % NST, round = g / NST;
        const uint32_t full = smem_u32(&sm.full_bar[stage]);
        const uint32_t left = it.nsteps - jb * kSS;
        const uint32_t nst = left < (uint32_t)kSS ? left : (uint32_t)kSS;
        uint32_t bytes = nst * SPAN;
        if (SPLIT && it.nsteps > it.nfull && jb * kSS + nst == it.nsteps) bytes -= SPAN - it.last_active;  // ragged last step
        // where this lane's step reads and writes: the consumers take the offset from shared memory instead
        // of tracking rows themselves.  A step may start in one row and end in the next (never further: rows
        // are at least as long as a step), so with SPLIT it is two copies and two offsets.
        uint32_t ofs_a = 0, ofs_b = 0, part_a = 0, part_b = 0, split = 0;
        if (lane < nst) {
            const uint32_t rr = run_r, cc = run_c;
            ofs_a = it.rowbase[rr < kRowCap ? rr : 0] + cc;
            if constexpr (SPLIT) {
                const uint32_t s = jb * kSS + lane;
                const uint32_t act = (s < it.nfull) ? SPAN : it.last_active;       // sub-streams with an element in this step
                const uint32_t room = it.col_len - cc;                               // sub-streams 0..room-1 stay in row rr
                split = room > it.t_begin ? (room - it.t_begin < SPAN ? room - it.t_begin : SPAN) : 0u;
                ofs_b = it.rowbase[rr + 1 < kRowCap ? rr + 1 : 0] + cc - it.col_len;
                part_a = split < act ? split : act;
                part_b = act - part_a;
            } else {
                part_a = SPAN;
            }
        }
        const bool good = mbar_wait(smem_u32(&sm.empty_bar[stage]), (round & 1u) ^ 1u, spin_limit);
        if (!__all_sync(0xFFFFFFFFu, good)) return false;
        if (lane == 0) mbar_expect_tx(full, bytes);   // as early as possible: arming the barrier late costs the consumers dearly
        const bool stall = (int)g == stall_block;   // self-test: the bytes never come, the consumers' wait runs out
        const uint32_t dst = smem_u32(sm.ctxring) + (stage * kSS + lane) * SPAN;
        if (part_a && !stall) bulk_g2s(dst, it.ctx_bytes + ofs_a + it.t_begin, part_a, full);
        if constexpr (SPLIT) {
            if (part_b && !stall) bulk_g2s(dst + part_a, it.ctx_bytes + ofs_b + it.t_begin + part_a, part_b, full);
        }
        if (lane == 0) sm.armed = g + 1;
        if (lane < nst) {
            sm.stepofs[stage][lane] = ofs_a;
            if constexpr (SPLIT) {
                sm.stepofs_b[stage][lane] = ofs_b;
                sm.stepsplit[stage][lane] = split;
            }
        }
        if (lane < (uint32_t)kSS) mbar_arrive(full);   // every lane releases its offsets with its own arrive
        // the same lane's step of the next block lies kSS steps on
        run_c += (uint32_t)kSS * it.k_eff;
        while (run_c >= it.col_len) { run_c -= it.col_len; ++run_r; }
    }
    return true;
}

// Rows that do not hold whole steps, under an item that spans the bucket's sub-streams (SPAN == k_eff: the
// down-projection shards of a tensor-parallel rank, 3584 columns under 1024 sub-streams).  A block of steps is
// then one contiguous run of the bucket's elements, and so are its bytes in the ring: the block is copied as
// one piece per row it touches (lane i: row of the block's first element + i) instead of one or two per step.
// The offsets of every step are published as in producer_run<SPAN, true>, which the same loop reads.
template <int SPAN>
__device__ __forceinline__ bool producer_split_rows(Smem& sm, const StreamItem& it, uint32_t blk, uint32_t nblocks, int stall_block,
                                                    uint32_t spin_limit) {
    constexpr uint32_t NST = ring_stages(SPAN);
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t br = 0, bc = 0;   // row and column of the block's first element
    for (uint32_t jb = 0; jb < nblocks; ++jb) {
        const uint32_t g = blk + jb, stage = g % NST, round = g / NST;
        const uint32_t full = smem_u32(&sm.full_bar[stage]);
        const uint32_t left = it.nsteps - jb * kSS;
        const uint32_t nst = left < (uint32_t)kSS ? left : (uint32_t)kSS;
        uint32_t bytes = nst * SPAN;
        if (it.nsteps > it.nfull && jb * kSS + nst == it.nsteps) bytes -= SPAN - it.last_active;  // ragged last step
        // this lane's step (lanes >= nst: unused): rows are longer than a step, so a few rounds at most
        uint32_t rr = br, cc = bc + (lane < (uint32_t)kSS ? lane : 0u) * SPAN;
        while (cc >= it.col_len) { cc -= it.col_len; ++rr; }
        const uint32_t room = it.col_len - cc;
        const uint32_t split = room < SPAN ? room : SPAN;
        const uint32_t ofs_a = it.rowbase[rr < kRowCap ? rr : 0] + cc;
        const uint32_t ofs_b = it.rowbase[rr + 1 < kRowCap ? rr + 1 : 0] + cc - it.col_len;
        // this lane's piece of the block: what the block holds of row br + lane
        const uint32_t in_first = it.col_len - bc;
        const uint32_t seg_off = lane == 0 ? 0u : in_first + (lane - 1u) * it.col_len;   // within the block
        const uint32_t seg_cap = lane == 0 ? in_first : it.col_len;
        const uint32_t seg_len = seg_off < bytes ? (bytes - seg_off < seg_cap ? bytes - seg_off : seg_cap) : 0u;
        const uint32_t seg_row = br + lane;
        const uint32_t seg_src = it.rowbase[seg_row < kRowCap ? seg_row : 0] + (lane == 0 ? bc : 0u);
        const bool good = mbar_wait(smem_u32(&sm.empty_bar[stage]), (round & 1u) ^ 1u, spin_limit);
        if (!__all_sync(0xFFFFFFFFu, good)) return false;
        if (lane == 0) mbar_expect_tx(full, bytes);
        if (seg_len && (int)g != stall_block)
            bulk_g2s(smem_u32(sm.ctxring) + stage * kSS * SPAN + seg_off, it.ctx_bytes + seg_src, seg_len, full);
        if (lane == 0) sm.armed = g + 1;
        if (lane < nst) {
            sm.stepofs[stage][lane] = ofs_a;
            sm.stepofs_b[stage][lane] = ofs_b;
            sm.stepsplit[stage][lane] = split;
        }
        if (lane < (uint32_t)kSS) mbar_arrive(full);
        bc += nst * SPAN;
        while (bc >= it.col_len) { bc -= it.col_len; ++br; }
    }
    return true;
}

// The common case made cheap: an item that spans the bucket's sub-streams (SPAN == k_eff) over rows that
// hold whole steps.  The producer's time per block lies on the path from "stage freed" to "bytes landed",
// so it keeps a running (row, step in row) instead of dividing, copies a block as one piece per row it
// touches (one or two for rows of at least kSS steps) instead of one per step.  (Bringing the rows into L2
// ahead of the copies with bulk prefetches was measured too: 1.5 % slower on the whole-model workload.)

template <int SPAN>
__device__ __forceinline__ bool producer_rows(Smem& sm, const StreamItem& it, uint32_t blk, uint32_t nblocks, int stall_block,
                                              uint32_t spin_limit) {
    constexpr uint32_t NST = ring_stages(SPAN);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t spr = it.col_len / it.k_eff;       // steps per row
    const uint8_t* const src0 = it.ctx_bytes;         // (t_begin is 0 when the item spans the bucket)
    uint32_t rr = 0, sc = 0;                          // the block's first step: row, step within the row
    for (uint32_t jb = 0; jb < nblocks; ++jb) {
        const uint32_t g = blk + jb, stage = g % NST, round = g / NST;
        const uint32_t full = smem_u32(&sm.full_bar[stage]);
        const uint32_t left = it.nsteps - jb * kSS;
        const uint32_t nst = left < (uint32_t)kSS ? left : (uint32_t)kSS;
        // this lane's step (lanes >= nst: unused) ...
        // (no loop over lanes' worth of rows where a row is one step: this runs once per block, and when the
        // stage is already free it is time the decoding warps wait)
        uint32_t my_r = rr, my_s = sc + (lane < (uint32_t)kSS ? lane : 0u);
        if (spr == 1u) { my_r += my_s; my_s = 0u; }
        while (my_s >= spr) { my_s -= spr; ++my_r; }
        const uint32_t ofs = it.rowbase[my_r < kRowCap ? my_r : 0] + my_s * SPAN;
        // ... and this lane's piece of the block: lane i copies what the block takes of row rr + i
        const uint32_t in_first = spr - sc;           // steps of the block that can stay in row rr
        const uint32_t seg_s0 = lane == 0 ? 0u : in_first + (lane - 1u) * spr;      // first step of the piece, within the block
        const uint32_t seg_cap = lane == 0 ? in_first : spr;
        const uint32_t seg_n = seg_s0 < nst ? (nst - seg_s0 < seg_cap ? nst - seg_s0 : seg_cap) : 0u;
        const uint32_t seg_row = rr + lane;
        const uint32_t seg_src = it.rowbase[seg_row < kRowCap ? seg_row : 0] + (lane == 0 ? sc * SPAN : 0u);
        const bool good = mbar_wait(smem_u32(&sm.empty_bar[stage]), (round & 1u) ^ 1u, spin_limit);
        if (!__all_sync(0xFFFFFFFFu, good)) return false;
        // arm, copy, and only then publish the offsets: the bytes have the longest way to go
        if (lane == 0) mbar_expect_tx(full, nst * SPAN);
        // (self-test: the bytes of one block never come, the consumers' wait runs out)
        if (seg_n && (int)g != stall_block) bulk_g2s(smem_u32(sm.ctxring) + (stage * kSS + seg_s0) * SPAN, src0 + seg_src, seg_n * SPAN, full);
        if (lane == 0) sm.armed = g + 1;
        if (lane < nst) sm.stepofs[stage][lane] = ofs;
        if (lane < (uint32_t)kSS) mbar_arrive(full);  // every lane releases its offset with its own arrive
        sc += nst;
        if (spr == 1u) { rr += sc; sc = 0u; }
        while (sc >= spr) { sc -= spr; ++rr; }
    }
    return true;
}

// Rows shorter than a step (the groups of an AWQ sidecar are 128 elements, a step of 256 sub-streams is
// two of them): a step is a whole number of rows, each copied as one piece; the decoding threads find
// their own row of a step themselves (stream_run, MROW).
template <int SPAN>
__device__ __forceinline__ bool producer_mrow(Smem& sm, const StreamItem& it, uint32_t blk, uint32_t nblocks, int stall_block,
                                              uint32_t spin_limit) {
    constexpr uint32_t NST = ring_stages(SPAN);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t rows_item = SPAN / it.col_len;        // rows of a step that hold this item's sub-streams
    const uint32_t rows_step = it.k_eff / it.col_len;    // rows of a step of the bucket
    const uint32_t row0 = it.t_begin / it.col_len;
    for (uint32_t jb = 0; jb < nblocks; ++jb) {
        const uint32_t g = blk + jb, stage = g % NST, round = g / NST;
        const uint32_t full = smem_u32(&sm.full_bar[stage]);
        const uint32_t left = it.nsteps - jb * kSS;
        const uint32_t nst = left < (uint32_t)kSS ? left : (uint32_t)kSS;
        uint32_t bytes = nst * SPAN;
        if (it.nsteps > it.nfull && jb * kSS + nst == it.nsteps) bytes -= SPAN - it.last_active;  // ragged last step: fewer rows
        // this lane's first piece (its only one unless a block holds more than 32 rows of the item), worked
        // out before the wait like everything else that does not need the stage
        const uint32_t pieces = nst * rows_item;
        const uint32_t u0 = lane / rows_item, j0 = lane - u0 * rows_item;
        const uint32_t r0 = (jb * kSS + u0) * rows_step + row0 + j0;
        const bool have0 = lane < pieces && r0 < it.nrows;
        const uint32_t src0 = it.rowbase[r0 < kRowCap ? r0 : 0];
        const bool good = mbar_wait(smem_u32(&sm.empty_bar[stage]), (round & 1u) ^ 1u, spin_limit);
        if (!__all_sync(0xFFFFFFFFu, good)) return false;
        if (lane == 0) {
            mbar_expect_tx(full, bytes);
            sm.armed = g + 1;
        }
        if (lane < (uint32_t)kSS) mbar_arrive(full);
        if ((int)g == stall_block) continue;   // self-test: the bytes never come, the consumers' wait runs out
        if (have0)
            bulk_g2s(smem_u32(sm.ctxring) + (stage * kSS + u0) * SPAN + j0 * it.col_len, it.ctx_bytes + src0, it.col_len, full);
        for (uint32_t p = lane + 32u; p < pieces; p += 32u) {
            const uint32_t u = p / rows_item, j = p - u * rows_item;
            const uint32_t row = (jb * kSS + u) * rows_step + row0 + j;
            if (row < it.nrows)
                bulk_g2s(smem_u32(sm.ctxring) + (stage * kSS + u) * SPAN + j * it.col_len,
                         it.ctx_bytes + it.rowbase[row < kRowCap ? row : 0], it.col_len, full);
        }
    }
    return true;
}

template <int L, int THREADS, int CH>
struct StreamThread {  // per-thread state that lives from stream_begin to stream_run
    SChain ch[CH];
};

// Start what can overlap with table staging: the first chunks of every sub-stream's bitstream.
// The four chunks of a sub-stream are 64 contiguous bytes, so four neighbouring lanes fetch them
// together: one cp.async instruction of a warp then touches 8 cache lines instead of 32, and the
// load/store unit, which looks lines up one per cycle, gets through an item's first 64 KB four
// times sooner.  A lane therefore writes into its neighbours' rings; stream_run orders that with
// cp.async.wait_group followed by __syncwarp before anyone reads.
template <int L, int THREADS, int CH>
__device__ __forceinline__ void stream_begin(Smem& sm, const StreamItem& it, StreamThread<L, THREADS, CH>& st) {
    static_assert(kRingChunks == 4, "four lanes share a sub-stream's first chunks");
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp0 = tid & ~31u;
    const uint32_t rings = smem_u32(sm.bitring);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const uint32_t pos = it.startbit[it.t_begin + tid * CH + c] + it.bo.bit_delta;
        st.ch[c].pos = pos;
        st.ch[c].next = (pos >> 7) + kRingChunks;
    }
    if (it.flat_bytes) return;   // the whole bitstream comes with one bulk copy
#pragma unroll
    for (int c = 0; c < CH; ++c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t owner = j * 8 + (lane >> 2);  // lane of this warp whose chain c is served
            const uint32_t pos = __shfl_sync(0xFFFFFFFFu, st.ch[c].pos, owner);
            const uint32_t ring = rings + (c * THREADS + warp0 + owner) * kRingBytes;
            chunk_fetch(ring, it.bo, ((pos >> 7) + (lane & 3u)) << 4);
        }
    }
    cp_async_commit();
}

// FLAT: the bucket's bitstream was bulk-copied whole into the space of the rings (a bucket of up to 64 KB of
// code bits: the attention projections, every shard of them): no first chunks to fetch, no requests in the loop.
// MROW: rows shorter than a step; a thread's element of step s lies in row s * (rows per step) + (its own row of
// the step), whose start it reads from the row bases in shared memory (see producer_mrow).
template <int L, int THREADS, int CH, bool ESC, bool SPLIT, bool FLAT = false, bool MROW = false>
__device__ __forceinline__ bool stream_run(Smem& sm, const StreamItem& it, StreamThread<L, THREADS, CH>& st,
                                           uint32_t blk, uint32_t bulk_parity, uint32_t spin_limit) {
    static_assert(!(FLAT && SPLIT) && !(MROW && (SPLIT || FLAT)), "one special shape at a time");
    // (MROW) this thread's row within a step, its column in that row, rows per step of the bucket
    const uint32_t my_row = MROW ? (it.t_begin + threadIdx.x * CH) / it.col_len : 0u;
    const uint32_t my_col = MROW ? (it.t_begin + threadIdx.x * CH) - my_row * it.col_len : 0u;
    const uint32_t rows_step = MROW ? it.k_eff / it.col_len : 0u;
    const uint32_t rowbase_s = MROW ? smem_u32(it.rowbase) : 0u;
    constexpr uint32_t WMASK = FLAT ? kFlatMask : 60u;
    constexpr int RP = ESC ? 1 : ((32 - L) / L + 1);   // symbols per 32-bit window
    // Steps between bitstream requests: rare requests cost fewer instructions, frequent ones let
    // cp.async.wait_group leave more of them in flight, which is what a thread with few chains needs.
    constexpr int CHK_MAX = (2 * kSS * L < 128) ? 2 * kSS : kSS;
    constexpr int CHK = ESC ? 4 : (4 * CH < CHK_MAX ? 4 * CH : CHK_MAX);
    constexpr int MAXBITS = ESC ? (L + 16) : L;          // most bits one step can consume
    static_assert(CHK * MAXBITS < 128, "at most one chunk boundary between two requests");
    // A chunk requested when w1 enters chunk k is first read when w1 enters chunk k + kRingChunks - 1,
    // at least NEED steps later; requests are committed every CHK steps and cp.async.wait_group LAG
    // then guarantees everything committed LAG commits ago, so LAG = NEED / CHK - 2 is always safe.
    constexpr int NEED = ((kRingChunks - 1) * 128 + MAXBITS - 1) / MAXBITS;
    constexpr int LAG = (NEED / CHK - 2) > 0 ? (NEED / CHK - 2) : 0;
    constexpr uint32_t SPAN = THREADS * CH;
    constexpr uint32_t NST = ring_stages(SPAN);
    static_assert(kSS % RP == 0 && (kSS % CHK == 0 || CHK == 2 * kSS), "a stage must hold whole windows and request periods");
    using CT = typename Ctx<CH>::T;
    const uint32_t tid = threadIdx.x;
    const uint32_t tbl = smem_u32(sm.tbl);
    const uint32_t ring0 = smem_u32(sm.bitring) + tid * kRingBytes;
    const uint32_t ctx0 = smem_u32(sm.ctxring) + tid * CH;
    const uint32_t t0 = it.t_begin + tid * CH;
    const uint32_t zero = *reinterpret_cast<volatile uint32_t*>(&sm.zero);

    // first units of every sub-stream (their chunks were requested in stream_begin by this warp's lanes, or the
    // whole bitstream was copied by the producer warp)
    const uint32_t flat0 = smem_u32(sm.bitring);
    auto ring_of = [&](int c) { return FLAT ? flat0 : ring0 + c * THREADS * kRingBytes; };
    if constexpr (FLAT) {
        if (!mbar_wait(smem_u32(&sm.tab_bar), bulk_parity, spin_limit)) return false;
    } else {
        cp_async_wait<0>();
        __syncwarp();
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const uint32_t u = st.ch[c].pos >> 5;
        if constexpr (FLAT) {
            st.ch[c].w0 = lds_ordered(flat0 + (((u ^ 1u) << 2) & kFlatMask));
            st.ch[c].w1 = lds_ordered(flat0 + ((((u + 1u) ^ 1u) << 2) & kFlatMask));
        } else {
            st.ch[c].w0 = lds_ordered(ring_unit_addr(ring_of(c), u));
            st.ch[c].w1 = lds_ordered(ring_unit_addr(ring_of(c), u + 1));
        }
    }

    uint32_t hi[CH], acc[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) acc[c] = 0;
    uint16_t* const out0 = it.out + t0;
    const uint32_t nblocks = (it.nsteps + kSS - 1) / kSS;

    for (uint32_t jb = 0; jb < nblocks; ++jb) {
        const uint32_t g = blk + jb, stage = g % NST, round = g / NST;
        if (!mbar_wait(smem_u32(&sm.full_bar[stage]), round & 1u, spin_limit)) return false;
        const uint32_t left = it.nsteps - jb * kSS;
        const uint32_t count = left < (uint32_t)kSS ? left : (uint32_t)kSS;
        CT val[kSS];
#pragma unroll
        for (int u = 0; u < kSS; ++u) val[u] = lds_ctx<CH>(ctx0 + (stage * kSS + u) * SPAN);
        uint32_t ofs[kSS];   // element offset of every step's row position (written by the producer warp)
        {
            static_assert(kSS == 8, "two 16-byte loads fetch a stage's step offsets");
            const uint32_t so = smem_u32(&sm.stepofs[stage][0]);
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(ofs[0]), "=r"(ofs[1]), "=r"(ofs[2]), "=r"(ofs[3]) : "r"(so) : "memory");
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(ofs[4]), "=r"(ofs[5]), "=r"(ofs[6]), "=r"(ofs[7]) : "r"(so + 16u) : "memory");
        }
        uint32_t ofs_b[kSS], split[kSS];   // rows that do not hold whole steps: see producer_run
        if constexpr (SPLIT) {
            const uint32_t sb = smem_u32(&sm.stepofs_b[stage][0]), sx = smem_u32(&sm.stepsplit[stage][0]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(ofs_b[4 * h]), "=r"(ofs_b[4 * h + 1]), "=r"(ofs_b[4 * h + 2]), "=r"(ofs_b[4 * h + 3])
                             : "r"(sb + 16u * h) : "memory");
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(split[4 * h]), "=r"(split[4 * h + 1]), "=r"(split[4 * h + 2]), "=r"(split[4 * h + 3])
                             : "r"(sx + 16u * h) : "memory");
            }
        }
        // The stage's bytes and offsets are in registers now: hand the stage back at once, so that the
        // producer refills it while this block is decoded.  Nothing but a data dependency keeps the
        // assembler from moving a load below the arrive, or the hardware from arriving before a load has
        // read the stage: the arrive's address is offset by (every loaded register OR-ed together) AND a
        // zero that is itself read from shared memory, which no tool can fold away.
        {
            uint32_t dep = 0;
#pragma unroll
            for (int u = 0; u < kSS; ++u) {
                dep |= ofs[u];
                if constexpr (CH == 8) dep |= val[u].x | val[u].y; else dep |= val[u];
                if constexpr (SPLIT) dep |= ofs_b[u] | split[u];
            }
            dep &= zero;
            __syncwarp();
            if ((tid & 31u) == 0) mbar_arrive(smem_u32(&sm.empty_bar[stage]) + dep);
        }
        // (SPLIT) which of a step's two rows this thread's sub-streams lie in is settled here, so that the
        // block below carries one offset per step like any other and not three
        if constexpr (SPLIT) {
#pragma unroll
            for (int u = 0; u < kSS; ++u) ofs[u] = (tid * CH >= split[u]) ? ofs_b[u] : ofs[u];
        }
        // a whole block runs without per-step checks; only the last block of an item can be shorter
        auto run_block = [&](auto checked) {
            constexpr bool CHECKED = decltype(checked)::value;
#pragma unroll
            for (int u = 0; u < kSS; ++u) {
                if (!CHECKED || (uint32_t)u < count) {
                    if (u % RP == 0) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            hi[c] = schain_window<WMASK>(st.ch[c], ring_of(c), acc[c] & 0xFFFFu);
                            acc[c] = 0;
                        }
                    }
                    uint32_t e[CH];
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        // index = ctx << L | top L bits of the window, in one funnel shift
                        const uint32_t idx = __funnelshift_l(hi[c], ctx_of<L>(Ctx<CH>::byte(val[u], c)), L);
                        e[c] = lds_table(tbl + (idx << 2));
                        if constexpr (!ESC) {
                            hi[c] = __funnelshift_l(0u, hi[c], e[c]);  // shift by the low 5 bits = code length
                            acc[c] += e[c];                            // low half accumulates the lengths
                        } else {
                            uint32_t used = e[c] & Entry<L>::kLenMask;
                            if (e[c] & Entry<L>::kEsc) {                     // 16 raw bits follow the ESC code
                                e[c] = __funnelshift_l(0u, hi[c], used) & 0xFFFF0000u;
                                used += 16;
                            }
                            acc[c] = used;
                        }
                    }
                    uint32_t o = ofs[u];
                    if constexpr (MROW) {
                        const uint32_t row = (jb * kSS + (uint32_t)u) * rows_step + my_row;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(o) : "r"(rowbase_s + 4u * (row < (uint32_t)kRowCap ? row : 0u)) : "memory");
                        o += my_col;   // the element's own offset: added to the tensor's start below, not to out0
                    }
                    uint16_t* dst;   // out0 + o elements, as one multiply-add
                    asm("mad.wide.u32 %0, %1, 2, %2;" : "=l"(dst) : "r"(o), "l"(MROW ? it.out : out0));
                    bool mine = true;   // the ragged last step holds an element for the first sub-streams only
                    if constexpr ((SPLIT || MROW) && CHECKED) mine = (jb * kSS + u < it.nfull) || (tid * CH < it.last_active);
                    if (mine) store_syms<CH>(dst, e);
                    if (!FLAT && ((CHK <= kSS) ? ((u + 1) % CHK == 0) : (u == kSS - 1 && (jb & 1u)))) {
                        // the position used for the request is the one of the last window; the bits consumed
                        // since then (< 32) can only make the request one period late, which NEED allows for
#pragma unroll
                        for (int c = 0; c < CH; ++c) schain_request(st.ch[c], ring0 + c * THREADS * kRingBytes, it.bo);
                        cp_async_commit();
                        cp_async_wait<LAG>();
                    }
                }
            }
        };
        // (the block that holds a ragged last step always takes the checked form)
        if (count == (uint32_t)kSS && !((SPLIT || MROW) && it.last_active != 0u && jb + 1 == nblocks)) run_block(std::false_type{});
        else run_block(std::true_type{});
    }
    if constexpr (!FLAT) cp_async_wait<0>();
    return true;
}

// One symbol with the register bit window (generic path).  Returns the 16-bit symbol.
template <int L>
__device__ __forceinline__ uint32_t decode_one_win(BitWin& w, const uint32_t* __restrict__ tbl, uint32_t ctx) {
    const uint32_t e = tbl[(ctx << L) + (w.hi >> (32 - L))];
    win_consume(w, e & Entry<L>::kLenMask);
    if (e & Entry<L>::kEsc) {
        const uint32_t raw = w.hi >> 16;
        win_consume(w, 16);
        return raw;
    }
    return e >> 16;
}

// Generic path: any shape and alignment, one element at a time, 64-bit indices, per-element checks.
template <int L>
__device__ void decode_generic(const Smem& sm, const uint32_t* rowbase, const mps_bucket_tensor& T, int mode, const uint32_t* __restrict__ bs32,
                               uint32_t lim, const uint32_t* __restrict__ startbit, uint32_t bit_lo, uint32_t t_begin, uint32_t t_end,
                               uint32_t k_eff, long long col_len, long long col_start, long long row_a,
                               long long total) {
    const bool small = T.n * T.m < 0xFFFFFFFFLL;  // cached row bases are 32-bit
    for (uint32_t t = t_begin; t < t_end; ++t) {
        BitWin w;
        win_init(w, bs32, lim, startbit[t] + bit_lo);
        for (long long e = t; e < total; e += k_eff) {
            const long long rr = e / col_len, cc = e - rr * col_len;
            long long base;
            if (rr < kRowCap && small) base = (rowbase[rr] == 0xFFFFFFFFu) ? -1 : (long long)rowbase[rr];
            else {
                const long long row = T.row_indices[row_a + rr];
                const long long c0 = (mode == 2) ? (long long)T.group_col_start[row_a + rr] : col_start;
                const bool ok = row >= 0 && row < T.n && c0 >= 0 && c0 + col_len <= T.m;
                base = ok ? row * T.m + c0 : -1;
            }
            uint32_t ctx = 0;
            if (base >= 0) ctx = T.ctx_bytes[base + cc];
            const uint32_t sym = decode_one_win<L>(w, sm.tbl, ctx_of<L>(ctx));
            if (base >= 0) T.out[base + cc] = (uint16_t)sym;
            if (w.avail <= 32) win_refill(w, bs32, lim);
        }
    }
}

// Eight fused entries from eight raw symbols and their eight packed length nibbles; returns whether any is an ESC.
template <int L>
__device__ __forceinline__ bool fuse_group(const uint4& sv, uint32_t lv, uint32_t (&ent)[8]) {
    const uint32_t s[4] = {sv.x, sv.y, sv.z, sv.w};
    bool esc = false;
    if constexpr (L == 7) {
        // nibbles i and i+4 of the eight, each alone in a 16-bit lane; one byte permute then
        // glues a symbol's two bytes above its nibble
        const uint32_t t = lv;
        esc = (t & 0x88888888u) != 0u;
        const uint32_t z[4] = {t & 0x000F000Fu, (t >> 4) & 0x000F000Fu, (t >> 8) & 0x000F000Fu, (t >> 12) & 0x000F000Fu};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // bytes: [nibble, 0, sym.lo, sym.hi]; operand a = z (bytes 0-3), b = syms (bytes 4-7)
            const uint32_t sel = ((i & 1) ? 0x7600u : 0x5400u) | ((i & 4) ? 0x32u : 0x10u);
            ent[i] = __byte_perm(z[i & 3], s[i >> 1], sel);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t sym = (s[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
            const uint32_t nib = (lv >> (4 * i)) & 0xFu;
            const uint32_t e = (nib == 15u);            // nibble 15 = ESC with an L-bit code
            const uint32_t len = e ? (uint32_t)L : nib;
            esc |= (e != 0);
            ent[i] = (sym << 16) | (e << 15) | len;
        }
    }
    return esc;
}

// The eight entries of a context without a table: the FP8 decoder emits zeros and consumes nothing
// (decode_huffman.cu:252-264); the AWQ decoders treat it as an ESC (:476-485).  Returns whether that is an ESC.
template <int L>
__device__ __forceinline__ bool fill_group(uint32_t (&ent)[8]) {
    const uint32_t fill = (L == 7) ? 0u : ((uint32_t)L | Entry<L>::kEsc);
#pragma unroll
    for (int i = 0; i < 8; ++i) ent[i] = fill;
    return L != 7;
}

// Fuse the bucket's tables into shared memory; returns whether any entry is an ESC.
// The raw tables of a bucket (up to 80 KB) usually come straight from HBM, so every thread first
// issues a whole batch of independent 16-byte + 4-byte loads and only then converts them: the batch,
// not a single load, is what waits for memory.
template <int L, int THREADS, typename F>
__device__ __forceinline__ bool stage_tables(Smem& sm, const mps_bucket_tensor& T, int tid, F&& after_first_loads) {
    constexpr int TS = 1 << L;                 // entries per table
    constexpr int GROUPS_PER_CTX = TS / 8;     // 8 entries per thread-iteration
    constexpr int NGROUPS = kTableEntries / 8;
    constexpr int ITERS = NGROUPS / THREADS;
    constexpr int BATCH = (THREADS >= 512) ? 4 : (ITERS < 8 ? ITERS : 8);  // loads in flight per thread
    static_assert(NGROUPS % THREADS == 0 && ITERS % BATCH == 0, "table groups must split evenly");
    const bool aligned = ((reinterpret_cast<uintptr_t>(T.decode_syms) & 15u) == 0) &&
                         ((reinterpret_cast<uintptr_t>(T.decode_lens) & 3u) == 0);
    bool esc = false;
    for (int it0 = 0; it0 < ITERS; it0 += BATCH) {
        uint4 sv[BATCH];
        uint32_t lv[BATCH];
        int32_t gv[BATCH];
#pragma unroll
        for (int q = 0; q < BATCH; ++q) {
            const int g = tid + (it0 + q) * THREADS;
            const int ctx = g / GROUPS_PER_CTX;
            const int j0 = (g - ctx * GROUPS_PER_CTX) * 8;
            const int32_t gid = sm.gid[ctx];
            gv[q] = gid;
            sv[q] = make_uint4(0u, 0u, 0u, 0u);
            lv[q] = 0u;
            if (gid >= 0) {
                const uint16_t* sp = T.decode_syms + (long long)gid * TS + j0;
                const uint8_t* lp = T.decode_lens + (long long)gid * (TS / 2) + (j0 >> 1);
                if (aligned) {
                    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(sv[q].x), "=r"(sv[q].y), "=r"(sv[q].z), "=r"(sv[q].w) : "l"(sp));
                    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(lv[q]) : "l"(lp));
                } else {
                    sv[q].x = (uint32_t)sp[0] | ((uint32_t)sp[1] << 16);
                    sv[q].y = (uint32_t)sp[2] | ((uint32_t)sp[3] << 16);
                    sv[q].z = (uint32_t)sp[4] | ((uint32_t)sp[5] << 16);
                    sv[q].w = (uint32_t)sp[6] | ((uint32_t)sp[7] << 16);
                    lv[q] = (uint32_t)lp[0] | ((uint32_t)lp[1] << 8) | ((uint32_t)lp[2] << 16) | ((uint32_t)lp[3] << 24);
                }
            }
        }
        if (it0 == 0) after_first_loads();
#pragma unroll
        for (int q = 0; q < BATCH; ++q) {
            const int g = tid + (it0 + q) * THREADS;
            const int ctx = g / GROUPS_PER_CTX;
            const int j0 = (g - ctx * GROUPS_PER_CTX) * 8;
            uint32_t ent[8];
            if (gv[q] >= 0) esc |= fuse_group<L>(sv[q], lv[q], ent);
            else esc |= fill_group<L>(ent);
            uint4* dst = reinterpret_cast<uint4*>(&sm.tbl[ctx * TS + j0]);
            dst[0] = make_uint4(ent[0], ent[1], ent[2], ent[3]);
            dst[1] = make_uint4(ent[4], ent[5], ent[6], ent[7]);
        }
    }
    return group_or(esc ? 1 : 0, THREADS) != 0;
}

// The same fusion when the bucket's tables are one run of consecutive table ids (what the reference encoder
// writes: tables are numbered by (scale, context), so the tables of one scale follow each other).  The
// producer warp has then copied the raw run with two bulk copies into the upper end of the table's own
// space -- symbols of the U tables at [end - 2.5 TS U, end - 0.5 TS U), packed lengths above them -- and
// the decoding warps expand it in place: no load instruction, no address arithmetic per load, no trip
// through the L1 for 80 KB per bucket.  Two waves of half the contexts each, lower half first; in a wave
// every thread reads the raw groups of its share, all threads meet, then every thread writes its fused
// groups.  The lower wave writes bytes [0, end/2), which hold raw symbols only of ranks below
// 1.25 U - NCTX; those belong to contexts below U/4, which that same wave has read before it writes.  The
// upper wave has read everything that is left before it writes anywhere.
// Returns 1 if any entry is an ESC, 0 if none, -1 if the copy never landed (bounded wait).
template <int L, int THREADS, typename F>
__device__ __forceinline__ int stage_tables_inplace(Smem& sm, int tid, int32_t first, uint32_t count, uint32_t parity,
                                                    uint32_t spin_limit, F&& after_issue) {
    constexpr int TS = 1 << L;
    constexpr int GROUPS_PER_CTX = TS / 8;
    constexpr int NGROUPS = kTableEntries / 8;
    constexpr int PER_WAVE = NGROUPS / 2 / THREADS;   // groups of 8 entries per thread and wave
    static_assert(NGROUPS % (2 * THREADS) == 0 && PER_WAVE <= 8, "a wave's raw groups must fit a thread's registers");
    after_issue();
    if (!mbar_wait(smem_u32(&sm.tab_bar), parity, spin_limit)) return -1;
    const uint32_t tbl = smem_u32(sm.tbl);
    const uint32_t raw_syms = tbl + (uint32_t)kTableEntries * 4u - (uint32_t)(TS * 2 + TS / 2) * count;
    const uint32_t raw_lens = tbl + (uint32_t)kTableEntries * 4u - (uint32_t)(TS / 2) * count;
    bool esc = false;
#pragma unroll
    for (int wave = 0; wave < 2; ++wave) {
        uint4 sv[PER_WAVE];
        uint32_t lv[PER_WAVE];
#pragma unroll
        for (int q = 0; q < PER_WAVE; ++q) {
            const int g = wave * (NGROUPS / 2) + tid + q * THREADS;
            const int ctx = g / GROUPS_PER_CTX;
            const int j0 = (g - ctx * GROUPS_PER_CTX) * 8;
            const int32_t gid = sm.gid[ctx];
            sv[q] = make_uint4(0u, 0u, 0u, 0u);
            lv[q] = 0u;
            if (gid >= 0) {
                const uint32_t e0 = (uint32_t)(gid - first) * (uint32_t)TS + (uint32_t)j0;   // first entry of the group in the raw run
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(sv[q].x), "=r"(sv[q].y), "=r"(sv[q].z), "=r"(sv[q].w) : "r"(raw_syms + e0 * 2u) : "memory");
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lv[q]) : "r"(raw_lens + (e0 >> 1)) : "memory");
            }
        }
        group_sync(THREADS);   // every raw byte this wave may overwrite has been read
#pragma unroll
        for (int q = 0; q < PER_WAVE; ++q) {
            const int g = wave * (NGROUPS / 2) + tid + q * THREADS;
            const int ctx = g / GROUPS_PER_CTX;
            const int j0 = (g - ctx * GROUPS_PER_CTX) * 8;
            uint32_t ent[8];
            if (sm.gid[ctx] >= 0) esc |= fuse_group<L>(sv[q], lv[q], ent);
            else esc |= fill_group<L>(ent);
            uint4* dst = reinterpret_cast<uint4*>(&sm.tbl[ctx * TS + j0]);
            dst[0] = make_uint4(ent[0], ent[1], ent[2], ent[3]);
            dst[1] = make_uint4(ent[4], ent[5], ent[6], ent[7]);
        }
    }
    return group_or(esc ? 1 : 0, THREADS) != 0 ? 1 : 0;
}

// What the scout warp remembers between items: the context -> table map that is staged once the item
// it prepared last has been decoded (lane i holds contexts i, i + 32, ...).
template <int L>
struct ScoutMemo {
    int valid = 0, ti = -1;
    int32_t gids[((L == 7 ? 256 : 16) + 31) / 32];
};

template <int L, int THREADS, int CH>
__device__ void scout_prepare(const BatchArgs& args, Smem& sm, unsigned int* ws, int slot,
                              int wait_iter, int& q_cur, int& q_end, ScoutMemo<L>& memo) {
    constexpr int NCTX = (L == 7) ? 256 : 16;
    constexpr int TS = 1 << L;
    constexpr uint32_t SPAN = THREADS * CH;
    const int lane = threadIdx.x & 31;
    Prepared& P = sm.prep[slot];
    // Work queue with guided grabs: consecutive items belong to the same tensor more often than not, so
    // a CTA that takes several in a row stages that tensor's tables once for all of them.  The grab
    // shrinks to single items towards the end of the launch, where balance matters more than reuse.
    if (wait_iter < 0) {
        // A CTA's first item is the one of its own number: a launch starts without a round trip to the queue
        // counter, which therefore counts from the grid size on.
        q_cur = (int)blockIdx.x < args.total_items ? (int)blockIdx.x : args.total_items;
        q_end = q_cur < args.total_items ? q_cur + 1 : q_cur;
    } else if (q_cur >= q_end) {
        const int remaining = args.total_items - q_cur;  // q_cur: end of this CTA's last grab, a lower bound of the queue head
        int want = remaining / (int)(kGrabSlack * gridDim.x);
        want = want < 1 ? 1 : (want > kMaxGrab ? kMaxGrab : want);
        unsigned int start = 0;
        if (lane == 0) start = atomicAdd(&ws[0], (unsigned int)want) + gridDim.x;
        start = __shfl_sync(0xFFFFFFFFu, start, 0);
        if (start >= (unsigned int)args.total_items) {
            q_cur = q_end = args.total_items;  // queue exhausted
        } else {
            q_cur = (int)start;
            q_end = (args.total_items - q_cur < want) ? args.total_items : q_cur + want;
        }
    }
    const int item = q_cur;
    if (item < args.total_items) ++q_cur;
    if (item >= args.total_items) {
        if (lane == 0) P.valid = 0;
        __syncwarp();
        return;
    }
    int ti = 0;
    long long local = item;
    if (args.tensors != nullptr) {
        int lo = 0, hi = args.count;  // largest ti with prefix[ti] <= item
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            const long long p = args.item_prefix[mid];
            if (p <= item) lo = mid; else hi = mid;
        }
        ti = lo;
        local = item - args.item_prefix[ti];
    }
    // the decoding warps read the descriptor from shared memory: a dependent chain of global loads at
    // the start of every item would be time nobody decodes in
    {
        static_assert(sizeof(mps_bucket_tensor) % 4 == 0, "descriptor is copied word by word");
        const uint32_t* src = reinterpret_cast<const uint32_t*>((args.tensors != nullptr) ? &args.tensors[ti] : &args.single);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.tensor[slot]);
        for (int i = lane; i < (int)(sizeof(mps_bucket_tensor) / 4); i += 32) dst[i] = src[i];
        __syncwarp();
    }
    const mps_bucket_tensor& T = sm.tensor[slot];
    const int mode = T.mode;
    const uint32_t k = (uint32_t)T.k;
    const uint32_t chunks = (k + SPAN - 1) / SPAN;
    const long long b = local / chunks;
    const uint32_t chunk = (uint32_t)(local - b * chunks);
    // Everything that depends on the bucket's number alone is requested before any of it is used: the scout's
    // time for an item is a chain of round trips to memory, and a launch's first item has nothing to hide it behind.
    const long long row_a = T.bucket_row_offsets[b];
    const long long row_e = T.bucket_row_offsets[b + 1];
    long long col_start = 0, col_len = T.group_size;
    if (mode != 2) { col_start = T.bucket_col_start[b]; col_len = T.bucket_col_len[b]; }
    const long long bit_base = T.bucket_bit_base[b];
    const uint32_t* const startbit = T.thread_startbit + b * ((long long)k + 1);
    const uint32_t ebits_k = startbit[k];    // the bucket's bits, unless it has fewer elements than sub-streams
    int32_t gids[(NCTX + 31) / 32];
#pragma unroll
    for (int j = 0; j < (NCTX + 31) / 32; ++j) {
        const int c = lane + 32 * j;
        gids[j] = (c < NCTX) ? T.bucket_table[b * NCTX + c] : -1;
    }
    const long long nrows = row_e - row_a;
    const long long total = nrows * col_len;
    bool ok = nrows > 0 && col_len > 0 && row_a >= 0 && row_a + nrows <= T.num_rows &&
              (mode == 2 || (col_start >= 0 && col_start + col_len <= T.m));
    const long long wb = bit_base >> 6;
    ok = ok && bit_base >= 0 && wb < T.bitstream_words;
    uint32_t k_eff = k;
    if (total < (long long)k_eff) k_eff = (uint32_t)(total > 0 ? total : 1);
    const uint32_t t_begin = chunk * SPAN;
    ok = ok && t_begin < k_eff;

    int rows_ok = 1, rows_vec = 1, rows_al16 = 1;
    uint32_t ebits = 0;
#pragma unroll
    for (int j = 0; j < (NCTX + 31) / 32; ++j)
        if (!ok || gids[j] >= T.num_tables) gids[j] = -1;
    if (ok) {
        ebits = (k_eff == k) ? ebits_k : startbit[k_eff];
        // row bases of the bucket (element offset of each row / group start)
        const long long ncache = nrows < kRowCap ? nrows : kRowCap;
        for (long long i = lane; i < ncache; i += 32) {
            const long long row = T.row_indices[row_a + i];
            const long long c0 = (mode == 2) ? (long long)T.group_col_start[row_a + i] : col_start;
            const bool good = row >= 0 && row < T.n && c0 >= 0 && c0 + col_len <= T.m;
            const long long base = row * T.m + c0;
            sm.rowbase[slot][i] = (good && base < 0xFFFFFFFFLL) ? (uint32_t)base : 0xFFFFFFFFu;
            rows_ok &= good;
            rows_vec &= ((base & (CH - 1)) == 0);
            rows_al16 &= ((base & 15) == 0);
        }
        rows_ok = __all_sync(0xFFFFFFFFu, rows_ok);
        rows_vec = __all_sync(0xFFFFFFFFu, rows_vec);
        rows_al16 = __all_sync(0xFFFFFFFFu, rows_al16);
        // pull what the item will read first into L2: its tables, its sub-stream offsets
#pragma unroll
        for (int j = 0; j < (NCTX + 31) / 32; ++j) {
            const int32_t gid = gids[j];
            if (gid >= 0) {
                const uint8_t* sp = reinterpret_cast<const uint8_t*>(T.decode_syms + (long long)gid * TS);
                const uint8_t* lp = T.decode_lens + (long long)gid * (TS / 2);
                for (int o = 0; o < TS * 2; o += 128) prefetch_l2(sp + o);
                for (int o = 0; o < TS / 2; o += 128) prefetch_l2(lp + o);
            }
        }
        const uint8_t* sb = reinterpret_cast<const uint8_t*>(startbit + t_begin);
        for (uint32_t o = lane * 128u; o < SPAN * 4u; o += 32u * 128u) prefetch_l2(sb + o);
        // hand the context -> table map over once the decoding warps have taken the previous one
    }
    // Hand the context -> table map over once the decoding warps have taken the previous one: their first
    // warp arrives on barrier 2 once per item, this warp joins it once per item it prepares during another
    // item (a hardware barrier: the waiting warp issues nothing while it waits).
    if (wait_iter >= 0) asm volatile("bar.sync 2, 64;" ::: "memory");
    int restage = 0, dense = 0, first = 0;
    uint32_t count = 0;
    if (ok) {
#pragma unroll
        for (int j = 0; j < (NCTX + 31) / 32; ++j) {
            const int c = lane + 32 * j;
            if (c < NCTX) sm.gid_next[c] = gids[j];
        }
        // does the item need other tables than the one before it, and are its tables one run of ids?
        int differs = !memo.valid || memo.ti != ti;
        int lowest = 0x7FFFFFFF;
#pragma unroll
        for (int j = 0; j < (NCTX + 31) / 32; ++j) {
            differs |= (gids[j] != memo.gids[j]);
            if (gids[j] >= 0 && gids[j] < lowest) lowest = gids[j];
        }
        restage = __any_sync(0xFFFFFFFFu, differs);
        lowest = __reduce_min_sync(0xFFFFFFFFu, lowest);
        int run = 1;
#pragma unroll
        for (int j = 0; j < (NCTX + 31) / 32; ++j) {   // contexts 32 j + lane: consecutive contexts are consecutive lanes
            const uint32_t has = __ballot_sync(0xFFFFFFFFu, gids[j] >= 0);
            const uint32_t rank = count + __popc(has & ((1u << lane) - 1u));
            if (gids[j] >= 0 && gids[j] != lowest + (int)rank) run = 0;
            count += __popc(has);
        }
        dense = __all_sync(0xFFFFFFFFu, run) && count > 0;
        first = lowest;
        memo.valid = 1; memo.ti = ti;
#pragma unroll
        for (int j = 0; j < (NCTX + 31) / 32; ++j) memo.gids[j] = gids[j];
    }
    if (lane == 0) {
        P.restage = (int16_t)restage; P.tab_dense = (int16_t)dense; P.tab_first = first; P.tab_count = count;
        P.valid = 1; P.ok = ok ? 1 : 0; P.ti = ti; P.mode = mode;
        P.k = k; P.k_eff = k_eff; P.t_begin = t_begin; P.ebits = ebits;
        P.b = b; P.row_a = (int32_t)row_a; P.nrows = (int32_t)nrows; P.col_start = (int32_t)col_start; P.col_len = (int32_t)col_len;
        P.total = total; P.wb = wb;
        P.rows_ok = rows_ok; P.rows_vec = rows_vec; P.rows_al16 = rows_al16;
        P.bit_lo = (uint32_t)(bit_base & 63);
    }
    __syncwarp();
}

template <int L, int THREADS, int CH>
// (registers are handed out to a CTA four warps at a time, so 320 threads get what 384 would: 168 each)
__global__ void __launch_bounds__(THREADS + 64, 1)
bucket_decode_kernel(const __grid_constant__ BatchArgs args, unsigned int* __restrict__ ws) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    constexpr int NCTX = (L == 7) ? 256 : 16;
    constexpr uint32_t SPAN = THREADS * CH;  // sub-streams per work item
    const int tid = threadIdx.x;
    const bool is_consumer = tid < THREADS;
    const bool is_producer = tid >= THREADS && tid < THREADS + 32;  // the whole producer warp
    const bool is_scout = tid >= THREADS + 32;       // the whole scout warp

    if (tid == 0) {
        sm.abort = 0;
        sm.armed = 0;
        sm.zero = 0;
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(smem_u32(&sm.full_bar[i]), 1u + kSS);  // lane 0's expect_tx + one arrive per step offset
            mbar_init(smem_u32(&sm.empty_bar[i]), THREADS / 32);
        }
        mbar_init(smem_u32(&sm.tab_bar), 1u);                // the producer's expect_tx
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    int q_cur = 0, q_end = 0;  // the scout's current grab from the work queue
    const uint32_t spin_limit = args.spin_limit ? args.spin_limit : kSpinLimit;
    const int stall_block = args.stall_block_plus1 - 1;
    ScoutMemo<L> memo;
    if (is_scout) scout_prepare<L, THREADS, CH>(args, sm, ws, 0, -1, q_cur, q_end, memo);
    __syncthreads();

    bool staged_esc = false;
    uint32_t blk = 0;  // blocks of steps streamed so far by this CTA (same value in every thread)
    uint32_t tab_copies = 0;   // bulk copies of raw tables so far: the phase of tab_bar (same value in every thread)
    bool tab_inflight = false; // the item just handled armed tab_bar (abort path)
    for (int iter = 0;; ++iter) {
        const int slot = iter & 1;
        const Prepared& P = sm.prep[slot];
        if (!P.valid) break;
        if (is_scout) {
            // next item's geometry, row bases and L2 prefetches, while the others decode this one
            scout_prepare<L, THREADS, CH>(args, sm, ws, slot ^ 1, iter + 1, q_cur, q_end, memo);
        } else if (P.ok) {
            const int ti = P.ti, mode = P.mode;
            const mps_bucket_tensor& T = sm.tensor[slot];
            const uint32_t k = P.k, k_eff = P.k_eff, t_begin = P.t_begin;
            const long long b = P.b, row_a = P.row_a, nrows = P.nrows, col_start = P.col_start, col_len = P.col_len;
            const long long total = P.total, wb = P.wb;
            const uint32_t* rowbase = sm.rowbase[slot];
            const uint32_t* bs32 = reinterpret_cast<const uint32_t*>(T.bitstream) + 2 * wb;
            const long long units = 2 * (T.bitstream_words - wb);
            const uint32_t lim = (uint32_t)((units > 0x7FFFFFFELL ? 0x7FFFFFFELL : units) - 1);  // odd: r <= lim <=> r^1 <= lim
            const uint32_t* startbit = T.thread_startbit + b * ((long long)k + 1);
            const bool vec = P.rows_ok && P.rows_vec && nrows <= kRowCap && (k_eff % CH) == 0 && (col_len % CH) == 0 &&
                             T.n * T.m < 0xFFFFFFFFLL && ((reinterpret_cast<uintptr_t>(T.ctx_bytes) & (CH - 1)) == 0) &&
                             ((reinterpret_cast<uintptr_t>(T.out) & (2 * CH - 1)) == 0);

            // ---- streaming path: start the asynchronous copies before the tables are staged ------------
            StreamItem it;
            it.flat_bytes = 0;
            StreamThread<L, THREADS, CH> st;
            bool stream = false;
            // rows that hold whole steps, or rows at least one step long whose length keeps 16-byte alignment
            const bool split = (col_len % k_eff) != 0;
            // rows shorter than a step: a step is whole rows, and so is this item's share of it
            // (instantiated for one or two chains per thread only: such buckets have few sub-streams, and the widest
            // kernel, which decodes whole models, is at its register limit)
            constexpr bool kMrowBuilt = CH <= 2;
            const bool mrow = kMrowBuilt && col_len < k_eff && (k_eff % col_len) == 0 && (SPAN % col_len) == 0 &&
                              (t_begin % col_len) == 0 && (col_len % 16) == 0 && total < 0xFFFFFFFFLL;
            if (vec && P.rows_al16 && t_begin + SPAN <= k_eff && (k_eff % 16u) == 0 &&
                (!split || mrow || (col_len > k_eff && (col_len % 16) == 0 && total < 0xFFFFFFFFLL)) &&
                ((reinterpret_cast<uintptr_t>(T.ctx_bytes) & 15u) == 0)) {
                const uint8_t* bucket_bytes = reinterpret_cast<const uint8_t*>(T.bitstream) + 8 * wb;
                const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(bucket_bytes) & 15u);  // 0 or 8
                const long long valid = 8 * (T.bitstream_words - wb) + mis;
                const long long bits = (long long)P.ebits + 8 * mis + P.bit_lo;  // end of the bucket's bits from the origin
                // the bucket's own bits must lie inside the bitstream; look-ahead past its end is never copied
                if ((mis == 0u || wb > 0) && valid >= 16 && valid <= 0x7FFFFFF0LL && ((bits + 7) >> 3) <= valid) {
                    stream = true;
                    it.ctx_bytes = T.ctx_bytes; it.out = T.out; it.startbit = startbit; it.rowbase = rowbase;
                    it.bo.base = bucket_bytes - mis; it.bo.last_ofs = (uint32_t)((valid - 16) & ~15LL); it.bo.bit_delta = 8 * mis + P.bit_lo;
                    it.bo.tail_ofs = (valid & 8) ? it.bo.last_ofs + 16u : 0xFFFFFFFFu;
                    it.t_begin = t_begin; it.k_eff = k_eff; it.col_len = (uint32_t)col_len; it.nrows = (uint32_t)nrows;
                    it.nfull = (uint32_t)(total / k_eff);
                    const uint32_t rem = (uint32_t)(total - (long long)it.nfull * k_eff);  // sub-streams with one more element
                    it.last_active = rem > t_begin ? (rem - t_begin < SPAN ? rem - t_begin : SPAN) : 0u;
                    it.nsteps = it.nfull + (it.last_active ? 1u : 0u);
                    // a bucket whose code bits fit the space of the rings comes in with one bulk copy
                    const long long need = (((bits + 7) >> 3) + 15) & ~15LL;   // bytes from the origin, whole 16-byte chunks
                    if (!split && k_eff == SPAN && need <= (long long)kFlatBytes && need <= (long long)it.bo.last_ofs + 16)
                        it.flat_bytes = (uint32_t)need;
                }
            }
            bool run_ok = true;
            uint32_t nblocks = 0;
            if (stream) nblocks = (it.nsteps + kSS - 1) / kSS;
            // tables that are one run of table ids are copied raw by the bulk-copy engine and expanded in place
            constexpr bool kInplaceFits = (kTableEntries / 8) % (2 * THREADS) == 0 && (kTableEntries / 8) / (2 * THREADS) <= 8;
            const bool tab_bulk = kInplaceFits && P.restage && P.tab_dense &&
                                  ((reinterpret_cast<uintptr_t>(T.decode_syms) | reinterpret_cast<uintptr_t>(T.decode_lens)) & 15u) == 0;
            const bool flat = stream && it.flat_bytes != 0u;
            const bool bulk_any = tab_bulk || flat;   // one barrier phase covers the raw tables and the resident bitstream
            const uint32_t tab_parity = tab_copies & 1u;
            tab_inflight = bulk_any;
            if (is_producer) {
                if (bulk_any && tid == THREADS) {
                    constexpr uint32_t TS = 1u << L;
                    const uint32_t count = tab_bulk ? P.tab_count : 0u;
                    const uint32_t end = smem_u32(sm.tbl) + (uint32_t)kTableEntries * 4u;
                    const uint32_t bar = smem_u32(&sm.tab_bar);
                    // the spaces copied into were written by ordinary stores and cp.async while the previous bucket was handled
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_expect_tx(bar, (TS * 2u + TS / 2u) * count + (flat ? it.flat_bytes : 0u));
                    if (tab_bulk) {
                        bulk_g2s(end - (TS * 2u + TS / 2u) * count, T.decode_syms + (long long)P.tab_first * TS, TS * 2u * count, bar);
                        bulk_g2s(end - (TS / 2u) * count, T.decode_lens + (long long)P.tab_first * (TS / 2), (TS / 2u) * count, bar);
                    }
                    if (flat) bulk_g2s(smem_u32(sm.bitring), it.bo.base, it.flat_bytes, bar);
                }
                if (stream) {
                    bool fed = false;
                    if constexpr (kMrowBuilt) {
                        if (mrow) { run_ok = producer_mrow<SPAN>(sm, it, blk, nblocks, stall_block, spin_limit); fed = true; }
                    }
                    if (fed) {
                    } else if (!split && it.k_eff == SPAN && (it.col_len & 15u) == 0u) run_ok = producer_rows<SPAN>(sm, it, blk, nblocks, stall_block, spin_limit);
                    else if (split && it.k_eff == SPAN) run_ok = producer_split_rows<SPAN>(sm, it, blk, nblocks, stall_block, spin_limit);
                    else run_ok = split ? producer_run<SPAN, true>(sm, it, blk, nblocks, stall_block, spin_limit)
                                        : producer_run<SPAN, false>(sm, it, blk, nblocks, stall_block, spin_limit);
                }
            } else if (is_consumer) {
                // ---- tables: restage only when the context->table map changed ------------------------
                // The first chunks of the bitstream are requested right after the first batch of table
                // loads: both wait on memory, and the table loads are the ones the threads need first.
                constexpr int CPT = (NCTX + THREADS - 1) / THREADS;  // contexts per thread
                auto begin = [&] { if (stream) stream_begin<L, THREADS, CH>(sm, it, st); };
                if (P.restage) {   // (the scout compared this item's map with the one staged now)
#pragma unroll
                    for (int i = 0; i < CPT; ++i) {
                        const int c = tid + i * THREADS;
                        if (c < NCTX) sm.gid[c] = sm.gid_next[c];
                    }
                    group_sync(THREADS);
                }
                if (tid < 32) asm volatile("bar.arrive 2, 64;" ::: "memory");  // the scout may now overwrite gid_next
                if (P.restage) {
                    bool expanded = false;
                    if constexpr (kInplaceFits) {
                        if (tab_bulk) {
                            const int r = stage_tables_inplace<L, THREADS>(sm, tid, P.tab_first, P.tab_count, tab_parity, spin_limit, begin);
                            if (r < 0) run_ok = false;
                            staged_esc = r > 0;
                            expanded = true;
                        }
                    }
                    if (!expanded) staged_esc = stage_tables<L, THREADS>(sm, T, tid, begin);
                } else {
                    begin();
                }

                // ---- decode --------------------------------------------------------------------------
                const uint32_t t0 = t_begin + (uint32_t)tid * CH;
                if (!run_ok) {
                    // the raw tables never landed: the wait gave up, the CTA reports and stops below
                } else if (stream) {
                    bool ran = false;
                    if constexpr (kMrowBuilt) {
                        if (mrow) {
                            run_ok = staged_esc ? stream_run<L, THREADS, CH, true, false, false, true>(sm, it, st, blk, tab_parity, spin_limit)
                                                : stream_run<L, THREADS, CH, false, false, false, true>(sm, it, st, blk, tab_parity, spin_limit);
                            ran = true;
                        }
                    }
                    if (ran) {
                    } else if (split)
                        run_ok = staged_esc ? stream_run<L, THREADS, CH, true, true>(sm, it, st, blk, tab_parity, spin_limit)
                                            : stream_run<L, THREADS, CH, false, true>(sm, it, st, blk, tab_parity, spin_limit);
                    else if (flat)
                        run_ok = staged_esc ? stream_run<L, THREADS, CH, true, false, true>(sm, it, st, blk, tab_parity, spin_limit)
                                            : stream_run<L, THREADS, CH, false, false, true>(sm, it, st, blk, tab_parity, spin_limit);
                    else
                        run_ok = staged_esc ? stream_run<L, THREADS, CH, true, false>(sm, it, st, blk, tab_parity, spin_limit)
                                            : stream_run<L, THREADS, CH, false, false>(sm, it, st, blk, tab_parity, spin_limit);
                } else if (vec) {
                    if (t0 < k_eff) {
                        if (staged_esc)
                            decode_vec<L, CH, true>(sm, rowbase, T.ctx_bytes, T.out, bs32, lim, startbit, P.bit_lo, t0, k_eff,
                                                    (uint32_t)col_len, (uint32_t)nrows, (uint32_t)total);
                        else
                            decode_vec<L, CH, false>(sm, rowbase, T.ctx_bytes, T.out, bs32, lim, startbit, P.bit_lo, t0, k_eff,
                                                     (uint32_t)col_len, (uint32_t)nrows, (uint32_t)total);
                    }
                } else if (t0 < k_eff) {
                    const uint32_t t1 = (t0 + CH < k_eff) ? t0 + CH : k_eff;
                    decode_generic<L>(sm, rowbase, T, mode, bs32, lim, startbit, P.bit_lo, t0, t1, k_eff, col_len, col_start, row_a,
                                      total);
                }
            }
            if (!run_ok) sm.abort = 1;
            blk += nblocks;
            tab_copies += bulk_any ? 1u : 0u;
        }
        if (!P.ok && tid < 32) asm volatile("bar.arrive 2, 64;" ::: "memory");
        __syncthreads();  // item done: tables, rings and the other prepared slot may now be overwritten
        if (sm.abort) {   // a bounded wait ran out: report and stop taking work (uniform: read after the barrier)
            if (tid == 0) atomicOr(&ws[2], 1u);
            break;
        }
    }

    // A CTA that gave up may still have copies on their way into its shared memory: before it leaves
    // (and the memory goes to the next CTA) it waits, again with a limit, for every armed stage.
    if (sm.abort) {
        if (is_consumer) cp_async_wait<0>();
        if (tid == THREADS) {
            if (tab_inflight) mbar_wait(smem_u32(&sm.tab_bar), (tab_copies - 1u) & 1u, spin_limit);
            constexpr uint32_t NST = ring_stages(SPAN);
            const uint32_t armed = sm.armed;
            for (uint32_t g = (armed > NST ? armed - NST : 0u); g < armed; ++g)
                mbar_wait(smem_u32(&sm.full_bar[g % NST]), (g / NST) & 1u, spin_limit);
        }
    }

    // last CTA out re-zeroes the queue so the next launch on this stream can reuse the workspace
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&ws[1], 1u);
        if (done == gridDim.x - 1) {
            ws[0] = 0u;
            ws[1] = 0u;
            __threadfence();
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Direct path for tensors made of tiny buckets (AWQ with one bucket per 128-element group, small
// per-channel weights): staging 128 KB of fused tables per bucket would cost far more than decoding
// it, so here every sub-stream is one thread that looks its codes up in the sidecar's own tables in
// global memory (they stay in L2), exactly as the sidecar stores them.  Parallelism comes from the
// number of sub-streams, which is what such tensors have plenty of.
// ------------------------------------------------------------------------------------------------
template <int L>
__global__ void __launch_bounds__(256) direct_decode_kernel(const __grid_constant__ mps_bucket_tensor T, long long total_sub) {
    constexpr int NCTX = (L == 7) ? 256 : 16;
    constexpr int TS = 1 << L;
    const int mode = T.mode;
    const long long k = T.k;
    for (long long w = blockIdx.x * 256LL + threadIdx.x; w < total_sub; w += (long long)gridDim.x * 256LL) {
        const long long b = w / k;
        const uint32_t t = (uint32_t)(w - b * k);
        const long long row_a = T.bucket_row_offsets[b];
        const long long nrows = (long long)T.bucket_row_offsets[b + 1] - row_a;
        long long col_start = 0, col_len = T.group_size;
        if (mode != 2) { col_start = T.bucket_col_start[b]; col_len = T.bucket_col_len[b]; }
        const long long bit_base = T.bucket_bit_base[b];
        const long long wb = bit_base >> 6;
        const bool ok = nrows > 0 && col_len > 0 && row_a >= 0 && row_a + nrows <= T.num_rows &&
                        (mode == 2 || (col_start >= 0 && col_start + col_len <= T.m)) && bit_base >= 0 && wb < T.bitstream_words;
        if (!ok) continue;
        const long long total = nrows * col_len;
        const uint32_t k_eff = (total < k) ? (uint32_t)total : (uint32_t)k;
        if (t >= k_eff) continue;
        const uint32_t* bs32 = reinterpret_cast<const uint32_t*>(T.bitstream) + 2 * wb;
        const long long units = 2 * (T.bitstream_words - wb);
        const uint32_t lim = (uint32_t)((units > 0x7FFFFFFELL ? 0x7FFFFFFELL : units) - 1);
        const int32_t* btab = T.bucket_table + b * NCTX;
        BitWin win;
        win_init(win, bs32, lim, T.thread_startbit[b * (k + 1) + t] + (uint32_t)(bit_base & 63));
        for (long long e = t; e < total; e += k_eff) {
            const long long rr = e / col_len, cc = e - rr * col_len;
            const long long row = T.row_indices[row_a + rr];
            const long long c0 = (mode == 2) ? (long long)T.group_col_start[row_a + rr] : col_start;
            const bool good = row >= 0 && row < T.n && c0 >= 0 && c0 + col_len <= T.m;
            const long long idx = row * T.m + c0 + cc;
            const uint32_t ctx = good ? ctx_of<L>(T.ctx_bytes[idx]) : 0u;
            int32_t gid = btab[ctx];
            if (gid >= T.num_tables) gid = -1;
            const uint32_t peek = win.hi >> (32 - L);
            uint32_t sym = 0, len = 0, esc = 0;
            if (gid >= 0) {
                const uint32_t nib = (__ldg(T.decode_lens + (long long)gid * (TS / 2) + (peek >> 1)) >> ((peek & 1u) * 4u)) & 0xFu;
                sym = __ldg(T.decode_syms + (long long)gid * TS + peek);
                if constexpr (L == 7) { len = nib & 7u; esc = nib & 8u; }
                else { esc = (nib == 15u); len = esc ? (uint32_t)L : nib; }
            } else if constexpr (L != 7) {
                esc = 1u; len = (uint32_t)L;  // AWQ: a context without a table reads as an ESC
            }
            win_consume(win, len);
            if (esc) {
                sym = win.hi >> 16;
                win_consume(win, 16);
            }
            if (good) T.out[idx] = (uint16_t)sym;
            if (win.avail <= 32) win_refill(win, bs32, lim);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <int L, int THREADS, int CH>
static int launch_cfg(const BatchArgs& a, unsigned int* ws, cudaStream_t st) {
    static bool attr_set[64] = {false};  // per instantiation and device
    const size_t smem = sizeof(Smem);
    int dev = 0;
    MPS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        MPS_CUDA_TRY(cudaFuncSetAttribute(bucket_decode_kernel<L, THREADS, CH>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    int grid = sm_count();
    if (a.total_items < grid) grid = a.total_items;
    if (grid <= 0) return MPS_OK;
    bucket_decode_kernel<L, THREADS, CH><<<grid, THREADS + 64, smem, st>>>(a, ws);
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

template <int L>
static int launch_L(const BatchArgs& a, int threads, int chains, unsigned int* ws, cudaStream_t st) {
#define MPS_CASE(T_, C_) if (threads == T_ && chains == C_) return launch_cfg<L, T_, C_>(a, ws, st)
    MPS_CASE(512, 2);
    MPS_CASE(512, 1);
    MPS_CASE(256, 4);
    MPS_CASE(256, 2);
    MPS_CASE(256, 1);
    MPS_CASE(128, 8);
    MPS_CASE(128, 4);
#undef MPS_CASE
    set_error("unsupported decode configuration threads=%d chains=%d", threads, chains);
    return MPS_ERR_UNSUPPORTED;
}

static int env_int(const char* name, int dflt) {
    const char* s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}

// threads x chains = sub-streams per work item.  Wide items (more chains per thread) cost fewer
// instructions per symbol and keep an SM 2.6 times busier than one chain per thread does; narrow
// items give more SMs something to do when a launch has few sub-streams in total, and cut the largest
// bucket, which bounds a lone tensor's time, in two.  Halving the width pays while the wider shape has
// no more items than the GPU has SMs (measured on single tensors of 82 to 322 buckets: 129 buckets
// decode 9 % faster halved, 188 buckets 36 % slower).  Buckets of more sub-streams than an item holds are
// cut into equal parts already: there halving only pays while every item still gets an SM of its own
// (a 4096 x 4096 weight of 32 buckets x 4096 sub-streams: 33.7 us as 128 items of (256,4), 39.8 us as 256 of (256,2)).
static void pick_config(long long total_substreams, int k_min, int* threads, int* chains) {
    const int sms = sm_count();
    int t = 256, c = 4;
    while (c > 1) {
        const long long items = total_substreams / ((long long)t * c);
        const bool parts = k_min > t * c;
        if (t * c > k_min || (parts ? 2 * items <= sms : items <= sms)) c >>= 1; else break;
    }
    while (t > 256 && t * c > k_min) t >>= 1;
    const int et = env_int("MPS_DECODE_THREADS", 0), ec = env_int("MPS_DECODE_CHAINS", 0);
    if (et > 0) t = et;
    if (ec > 0) c = ec;
    *threads = t;
    *chains = c;
}

static int validate_tensor(const mps_bucket_tensor& T, int L) {
    if (!T.ctx_bytes || !T.bitstream || !T.decode_syms || !T.decode_lens || !T.bucket_table || !T.bucket_row_offsets ||
        !T.row_indices || !T.thread_startbit || !T.bucket_bit_base || !T.out) {
        set_error("null device pointer in tensor descriptor");
        return MPS_ERR_INVALID;
    }
    if (T.mode != 2 && (!T.bucket_col_start || !T.bucket_col_len)) { set_error("bucket_col_start/len missing"); return MPS_ERR_INVALID; }
    if (T.mode == 2 && (!T.group_col_start || T.group_size <= 0 || T.group_size > T.m)) {
        set_error("group_size must be in (0,m]");
        return MPS_ERR_INVALID;
    }
    if (T.n <= 0 || T.m <= 0) { set_error("n,m must be > 0"); return MPS_ERR_INVALID; }
    if (T.k <= 0 || T.k > MPS_MAX_SUBSTREAMS) { set_error("bucket_thread_startbit_u32 has invalid k (must be 1..%d)", MPS_MAX_SUBSTREAMS); return MPS_ERR_INVALID; }
    if (T.num_buckets < 0 || T.num_tables < 0 || T.bitstream_words < 0 || T.num_rows < 0) { set_error("negative size"); return MPS_ERR_INVALID; }
    if ((L == 7) != (T.mode == 0)) { set_error("tensor mode does not match the table width"); return MPS_ERR_INVALID; }
    if ((reinterpret_cast<uintptr_t>(T.bitstream) & 7u) != 0) { set_error("bitstream must be 8-byte aligned"); return MPS_ERR_INVALID; }
    return MPS_OK;
}

// Tensors whose sub-streams hold this few symbols (on average) are decoded by the direct kernel.  It
// pays about ten times more per symbol of a sub-stream than the persistent kernel, whose cost before a
// bucket's first symbol is worth some twenty such symbols.  Measured on single per-channel tensors of
// 67 to 291 buckets: 0.4-0.9 K elements per bucket 11-13 us direct against 16-20 us persistent, 1.8-2.6 K
// a tie, 6.6 K 30 against 21 us, 8.7 K 42 against 23 us.
constexpr long long kDirectMaxSteps = 2;

static bool use_direct(const mps_bucket_tensor& T) {
    const int forced = env_int("MPS_DECODE_DIRECT", -1);
    if (forced >= 0) return forced != 0;
    if (T.num_buckets <= 0) return false;
    const long long per_bucket = (T.n * T.m) / T.num_buckets;
    const long long k_eff = per_bucket < T.k ? (per_bucket > 0 ? per_bucket : 1) : T.k;
    return per_bucket / k_eff <= kDirectMaxSteps;
}

static int decode_direct(const mps_bucket_tensor& T, int L, void* stream) {
    const long long total_sub = T.num_buckets * (long long)T.k;
    long long blocks = (total_sub + 255) / 256;
    const long long cap = 16LL * sm_count();
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (L == 7) direct_decode_kernel<7><<<(unsigned)blocks, 256, 0, st>>>(T, total_sub);
    else direct_decode_kernel<11><<<(unsigned)blocks, 256, 0, st>>>(T, total_sub);
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

static int decode_single(const mps_bucket_tensor& T, int L, void* workspace, size_t workspace_bytes, void* stream,
                         int stall_block = -1, uint32_t spin_limit = 0) {
    int rc = validate_tensor(T, L);
    if (rc) return rc;
    if (!workspace || workspace_bytes < mps_workspace_bytes()) { set_error("workspace missing or too small"); return MPS_ERR_WORKSPACE; }
    if (T.num_buckets == 0) return MPS_OK;
    if (use_direct(T) && stall_block < 0) return decode_direct(T, L, stream);
    int threads, chains;
    pick_config(T.num_buckets * (long long)T.k, T.k, &threads, &chains);
    const long long chunks = ((long long)T.k + (long long)threads * chains - 1) / ((long long)threads * chains);
    const long long items = T.num_buckets * chunks;
    if (items > 0x7FFFFFF0LL) { set_error("too many work items"); return MPS_ERR_INVALID; }
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.single = T;
    a.tensors = nullptr;
    a.item_prefix = nullptr;
    a.count = 1;
    a.total_items = (int)items;
    a.stall_block_plus1 = stall_block + 1;
    a.spin_limit = spin_limit;
    unsigned int* ws = static_cast<unsigned int*>(workspace);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return (L == 7) ? launch_L<7>(a, threads, chains, ws, st) : launch_L<11>(a, threads, chains, ws, st);
}

// ------------------------------------------------------------------------------------------------
// checksum
// ------------------------------------------------------------------------------------------------
__global__ void checksum_u16_kernel(const uint16_t* __restrict__ d, long long count, unsigned long long* __restrict__ res) {
    unsigned long long sum = 0, x = 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long v = d[i];
        sum += v;
        x ^= v * (unsigned long long)(i + 1);
    }
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        x ^= __shfl_xor_sync(0xFFFFFFFFu, x, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&res[0], sum);
        atomicXor(&res[1], x);
    }
}

// ------------------------------------------------------------------------------------------------
// Scratch for callers that cannot allocate: the work-queue counters of ONE decode launch at a time,
// resident in every GPU that loads this library until the process exits.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 256;
static __device__ __align__(256) unsigned int g_static_scratch[kStaticScratchBytes / sizeof(unsigned int)];

// Device address of g_static_scratch on the current device.  In host code the array's name is only a
// handle for the runtime, never a pointer a kernel may be given; the address is asked for once per
// device (with that device current) and remembered.
static int static_scratch(unsigned int** out) {
    static unsigned int* cached[64] = {nullptr};
    int dev = 0;
    MPS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { set_error("device ordinal %d out of range for the static scratch", dev); return MPS_ERR_UNSUPPORTED; }
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        MPS_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        cached[dev] = static_cast<unsigned int*>(p);
    }
    *out = cached[dev];
    return MPS_OK;
}

}  // namespace mps

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
using namespace mps;

extern "C" {

int mps_abi_version(void) { return 1; }

const char* mps_last_error(void) { return g_err; }

int64_t mps_cuda_clock_rate_khz(void) {
    int dev = 0, khz = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(clockRate)");
    return khz;
}

size_t mps_workspace_bytes(void) { return 256; }

int mps_decode_status(void* workspace, size_t workspace_bytes, void* stream, int32_t* timed_out) {
    if (!timed_out || (workspace && workspace_bytes < mps_workspace_bytes())) { set_error("mps_decode_status: bad argument"); return MPS_ERR_INVALID; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int* ws = static_cast<unsigned int*>(workspace);
    if (!ws) {   // the library's own scratch: what mps_decode_fp8_noalloc decodes with
        int rc = static_scratch(&ws);
        if (rc) return rc;
    }
    unsigned int flag = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&flag, ws + 2, sizeof(flag), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    if (flag) MPS_CUDA_TRY(cudaMemsetAsync(ws + 2, 0, sizeof(flag), st));
    *timed_out = flag ? 1 : 0;
    return MPS_OK;
}

int mps_decode_fp8(const uint8_t* fp8_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                   const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                   const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                   const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                   const int32_t* row_indices_i32, int64_t num_row_indices,
                   const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                   int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                   uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream) {
    if (max_len <= 0 || max_len > 15) { set_error("max_len must be in [1,15]"); return MPS_ERR_INVALID; }
    if (max_len != 7) { set_error("decode kernel is specialized: max_len must be 7"); return MPS_ERR_INVALID; }
    mps_bucket_tensor T;
    memset(&T, 0, sizeof(T));
    T.ctx_bytes = fp8_u8; T.bitstream = bitstream_u64; T.bitstream_words = bitstream_words;
    T.decode_syms = decode_syms_u16; T.decode_lens = decode_lens_u8; T.num_tables = num_tables;
    T.bucket_table = bucket_table_i32; T.bucket_col_start = bucket_col_start_i32; T.bucket_col_len = bucket_col_len_i32;
    T.bucket_row_offsets = bucket_row_offsets_i32; T.row_indices = row_indices_i32; T.num_rows = num_row_indices;
    T.thread_startbit = bucket_thread_startbit_u32; T.bucket_bit_base = bucket_bit_base_i64;
    T.num_buckets = num_buckets; T.k = k; T.mode = 0; T.n = n; T.m = m; T.out = out_bf16;
    return decode_single(T, 7, workspace, workspace_bytes, stream);
}

int mps_decode_awq_int4_bucket(const uint8_t* int4_values_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                               const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                               const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                               const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                               const int32_t* row_indices_i32, int64_t num_row_indices,
                               const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                               int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                               uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream) {
    if (max_len <= 0 || max_len > 15) { set_error("max_len must be in [1,15]"); return MPS_ERR_INVALID; }
    if (max_len != 11) { set_error("AWQ bucket decode kernel is specialized: max_len must be 11"); return MPS_ERR_INVALID; }
    mps_bucket_tensor T;
    memset(&T, 0, sizeof(T));
    T.ctx_bytes = int4_values_u8; T.bitstream = bitstream_u64; T.bitstream_words = bitstream_words;
    T.decode_syms = decode_syms_u16; T.decode_lens = decode_lens_u8; T.num_tables = num_tables;
    T.bucket_table = bucket_table_i32; T.bucket_col_start = bucket_col_start_i32; T.bucket_col_len = bucket_col_len_i32;
    T.bucket_row_offsets = bucket_row_offsets_i32; T.row_indices = row_indices_i32; T.num_rows = num_row_indices;
    T.thread_startbit = bucket_thread_startbit_u32; T.bucket_bit_base = bucket_bit_base_i64;
    T.num_buckets = num_buckets; T.k = k; T.mode = 1; T.n = n; T.m = m; T.out = out_bf16;
    return decode_single(T, 11, workspace, workspace_bytes, stream);
}

int mps_decode_awq_int4_bucket_by_scale(const uint8_t* int4_values_u8, const uint64_t* bitstream_u64,
                                        int64_t bitstream_words, const uint16_t* decode_syms_u16,
                                        const uint8_t* decode_lens_u8, int64_t num_tables,
                                        const int32_t* bucket_table_i32, const int32_t* bucket_group_offsets_i32,
                                        const int32_t* group_rows_i32, const int32_t* group_col_start_i32,
                                        int64_t num_groups, const uint32_t* bucket_thread_startbit_u32,
                                        const int64_t* bucket_bit_base_i64, int64_t num_buckets, int32_t k,
                                        int64_t n, int64_t m, int64_t max_len, int64_t group_size,
                                        uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream) {
    if (max_len <= 0 || max_len > 15) { set_error("max_len must be in [1,15]"); return MPS_ERR_INVALID; }
    if (max_len != 11) { set_error("AWQ ragged bucket decode kernel is specialized: max_len must be 11"); return MPS_ERR_INVALID; }
    if (group_size <= 0 || group_size > m) { set_error("group_size must be in (0,m]"); return MPS_ERR_INVALID; }
    mps_bucket_tensor T;
    memset(&T, 0, sizeof(T));
    T.ctx_bytes = int4_values_u8; T.bitstream = bitstream_u64; T.bitstream_words = bitstream_words;
    T.decode_syms = decode_syms_u16; T.decode_lens = decode_lens_u8; T.num_tables = num_tables;
    T.bucket_table = bucket_table_i32; T.bucket_row_offsets = bucket_group_offsets_i32;
    T.row_indices = group_rows_i32; T.group_col_start = group_col_start_i32; T.num_rows = num_groups;
    T.thread_startbit = bucket_thread_startbit_u32; T.bucket_bit_base = bucket_bit_base_i64;
    T.num_buckets = num_buckets; T.k = k; T.group_size = (int32_t)group_size; T.mode = 2; T.n = n; T.m = m;
    T.out = out_bf16;
    return decode_single(T, 11, workspace, workspace_bytes, stream);
}

int mps_decode_fp8_noalloc(const uint8_t* fp8_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                           const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                           const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                           const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                           const int32_t* row_indices_i32, int64_t num_row_indices,
                           const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                           int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                           uint16_t* out_bf16, void* stream) {
    if (num_buckets > MPS_NOALLOC_MAX_BUCKETS) {
        set_error("mps_decode_fp8_noalloc: %lld buckets exceed the supported maximum of %d", (long long)num_buckets,
                  MPS_NOALLOC_MAX_BUCKETS);
        return MPS_ERR_INVALID;
    }
    unsigned int* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc) return rc;
    // every call shares the array and finds what the last one left: start from zeroed queue counters
    // (words 0 and 1); word 2, the record of a wait that ran out, stays until mps_decode_status reads it
    MPS_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * sizeof(unsigned int), static_cast<cudaStream_t>(stream)));
    return mps_decode_fp8(fp8_u8, bitstream_u64, bitstream_words, decode_syms_u16, decode_lens_u8, num_tables,
                          bucket_table_i32, bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32,
                          row_indices_i32, num_row_indices, bucket_thread_startbit_u32, bucket_bit_base_i64, num_buckets, k,
                          n, m, max_len, out_bf16, scratch, kStaticScratchBytes, stream);
}

int mps_bucket_batch_plan(const mps_bucket_tensor* tensors_host, int count, int64_t* item_prefix_host,
                          int32_t* threads_out, int32_t* chains_out) {
    if (!tensors_host || count <= 0 || !item_prefix_host || !threads_out || !chains_out) {
        set_error("mps_bucket_batch_plan: bad arguments");
        return MPS_ERR_INVALID;
    }
    const int L = (tensors_host[0].mode == 0) ? 7 : 11;
    long long subs = 0;
    int k_min = MPS_MAX_SUBSTREAMS;
    for (int i = 0; i < count; ++i) {
        int rc = validate_tensor(tensors_host[i], L);
        if (rc) return rc;
        if (use_direct(tensors_host[i])) continue;  // decoded on its own (mps_decode_bucket_tensor)
        subs += tensors_host[i].num_buckets * (long long)tensors_host[i].k;
        if (tensors_host[i].k < k_min) k_min = tensors_host[i].k;
    }
    int threads, chains;
    pick_config(subs, k_min, &threads, &chains);
    long long acc = 0;
    for (int i = 0; i < count; ++i) {
        item_prefix_host[i] = acc;
        const long long span = (long long)threads * chains;
        if (!use_direct(tensors_host[i])) acc += tensors_host[i].num_buckets * ((tensors_host[i].k + span - 1) / span);
    }
    item_prefix_host[count] = acc;
    if (acc > 0x7FFFFFF0LL) { set_error("too many work items"); return MPS_ERR_INVALID; }
    *threads_out = threads;
    *chains_out = chains;
    return MPS_OK;
}

int mps_decode_bucket_tensor(const mps_bucket_tensor* tensor_host, void* workspace, size_t workspace_bytes, void* stream) {
    if (!tensor_host) { set_error("mps_decode_bucket_tensor: null descriptor"); return MPS_ERR_INVALID; }
    return decode_single(*tensor_host, tensor_host->mode == 0 ? 7 : 11, workspace, workspace_bytes, stream);
}

int mps_selftest_stalled_decode(const mps_bucket_tensor* tensor_host, int32_t stall_block, uint32_t polls, void* workspace,
                                size_t workspace_bytes, void* stream) {
    if (!tensor_host || stall_block < 0 || polls == 0) { set_error("mps_selftest_stalled_decode: bad arguments"); return MPS_ERR_INVALID; }
    return decode_single(*tensor_host, tensor_host->mode == 0 ? 7 : 11, workspace, workspace_bytes, stream, stall_block, polls);
}

int mps_decode_bucket_batch(const mps_bucket_tensor* tensors_dev, const int64_t* item_prefix_dev, int count,
                            int64_t total_items, int32_t threads, int32_t chains, int32_t mode,
                            void* workspace, size_t workspace_bytes, void* stream) {
    if (!tensors_dev || !item_prefix_dev || count <= 0 || total_items < 0 || total_items > 0x7FFFFFF0LL) {
        set_error("mps_decode_bucket_batch: bad arguments");
        return MPS_ERR_INVALID;
    }
    if (!workspace || workspace_bytes < mps_workspace_bytes()) { set_error("workspace missing or too small"); return MPS_ERR_WORKSPACE; }
    if (total_items == 0) return MPS_OK;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.tensors = tensors_dev;
    a.item_prefix = item_prefix_dev;
    a.count = count;
    a.total_items = (int)total_items;
    unsigned int* ws = static_cast<unsigned int*>(workspace);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return (mode == 0) ? launch_L<7>(a, threads, chains, ws, st) : launch_L<11>(a, threads, chains, ws, st);
}

int mps_checksum_u16(const uint16_t* data_dev, int64_t count, uint64_t* result_dev, void* stream) {
    if (!data_dev || !result_dev || count < 0) { set_error("mps_checksum_u16: bad arguments"); return MPS_ERR_INVALID; }
    if (count == 0) return MPS_OK;
    const int threads = 256;
    long long blocks = (count + threads * 8 - 1) / (threads * 8);
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    checksum_u16_kernel<<<(int)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        data_dev, count, reinterpret_cast<unsigned long long*>(result_dev));
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

}  // extern "C"
