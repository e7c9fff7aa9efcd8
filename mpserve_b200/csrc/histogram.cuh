// Histogram of every (scale, context) pair's symbols, the first pass of the sidecar builder
// (kernel/build_huffman.cu:392-412 does it with one std::map per context on one CPU thread).
//
// Two levels, no sort over the elements:
//
//   1. Scales.  The tensor is cut into units that have one scale each (a piece of a row, or a block of
//      a block-scaled tensor).  A 65536-bin count of the units' 16-bit scale values gives every
//      distinct scale its rank (ascending value) and a list of the units that carry it.
//   2. Contexts.  Segment (rank, context) is the multiset of symbols seen under that pair.  One pass
//      counts the segments' sizes, a second one moves every symbol into its segment: each warp walks
//      units of one scale, counts their contexts in its own shared-memory counters, reserves room in
//      every segment with one global atomic per context, and scatters.  A segment is then counted by
//      value in shared memory in windows of kWindow symbol values starting at its smallest symbol (a
//      context of a quantised weight sees a few dozen neighbouring BF16 patterns, so one window is
//      the rule); segments longer than kChunk elements are split over several CTAs that add their
//      windows into a dense 65536-counter array of that segment, of which the range between the
//      segment's smallest and largest symbol is then read back.
//
// The result is what the sort-based formulation produced: items (scale << 32 | context << 16 | symbol)
// in ascending order with their counts, and for every non-empty segment, in the same order, its first
// item and its key.  Scans are CUB device scans; everything else is written here.
#pragma once

#include <cub/device/device_scan.cuh>

#include "mps_common.cuh"

namespace mps {
namespace hist {

constexpr int kScaleValues = 65536;
constexpr int kChunk = 65536;       // elements of a segment counted by one CTA
constexpr int kWindow = 8192;       // symbol values counted at once
constexpr int kWarpElems = 8192;    // elements a warp walks in the counting and scattering passes
constexpr int kWalkWarps = 8;

// Units: blocks of ub0 x ub1 elements, nbu1 per block row.  Scalar and per-row scales cut rows into
// pieces (ub0 = 1); block scales use the scale blocks themselves.
struct Geom {
    long long n, m;
    long long ub0, ub1, nbu0, nbu1;
    int scale_mode;   // 0 scalar, 1 per row, 2 per block (the unit grid is the block grid)
    uint32_t ctx_mask;
    int nctx;
};

__device__ __forceinline__ uint32_t unit_scale(const Geom& g, const uint16_t* __restrict__ scales, long long u) {
    if (g.scale_mode == 0) return scales[0];
    if (g.scale_mode == 1) return scales[u / g.nbu1];
    return scales[u];
}

__global__ void unit_scale_count_kernel(Geom g, const uint16_t* __restrict__ scales, long long units, uint32_t* __restrict__ per_scale) {
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x)
        atomicAdd(&per_scale[unit_scale(g, scales, u)], 1u);
}

__global__ void scale_flags_kernel(const uint32_t* __restrict__ per_scale, uint32_t* __restrict__ flag) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v < kScaleValues) flag[v] = per_scale[v] ? 1u : 0u;
    if (v == 0) flag[kScaleValues] = 0u;
}

// rank -> scale value, and the cursors of the unit lists
__global__ void scale_ranks_kernel(const uint32_t* __restrict__ per_scale, const uint32_t* __restrict__ rank,
                                   const uint32_t* __restrict__ unit_ofs, uint16_t* __restrict__ scale_of_rank,
                                   uint32_t* __restrict__ unit_cur) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= kScaleValues) return;
    unit_cur[v] = unit_ofs[v];
    if (per_scale[v]) scale_of_rank[rank[v]] = (uint16_t)v;
}

__global__ void unit_scatter_kernel(Geom g, const uint16_t* __restrict__ scales, long long units, uint32_t* __restrict__ unit_cur,
                                    uint32_t* __restrict__ unit_sorted) {
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (long long)gridDim.x * blockDim.x)
        unit_sorted[atomicAdd(&unit_cur[unit_scale(g, scales, u)], 1u)] = (uint32_t)u;
}

// Calls f(context, symbol) for every element of unit u, lanes striding along rows, four (eight when the
// symbols are read too) elements of a lane loaded before any is handed on, so that as many loads are in
// flight per lane, not one.
template <bool WITH_SYM, class F>
__device__ __forceinline__ void for_unit_elements(const Geom& g, long long u, int lane, const uint8_t* __restrict__ ctx,
                                                  const uint16_t* __restrict__ sym, F&& f) {
    const long long bi = u / g.nbu1, bj = u - bi * g.nbu1;
    const long long r0 = bi * g.ub0, c0 = bj * g.ub1;
    const long long r1 = (r0 + g.ub0 < g.n) ? r0 + g.ub0 : g.n;
    const long long c1 = (c0 + g.ub1 < g.m) ? c0 + g.ub1 : g.m;
    constexpr int UN = WITH_SYM ? 8 : 4;
    for (long long r = r0; r < r1; ++r) {
        const uint8_t* crow = ctx + r * g.m;
        const uint16_t* srow = sym + r * g.m;
        for (long long c = c0 + lane; c < c1; c += 32 * UN) {
            uint32_t cv[UN], sv[UN];
#pragma unroll
            for (int k = 0; k < UN; ++k) {
                const long long cc = c + 32 * k;
                cv[k] = (cc < c1) ? crow[cc] : 0u;
                if (WITH_SYM) sv[k] = (cc < c1) ? srow[cc] : 0u; else sv[k] = 0u;
            }
#pragma unroll
            for (int k = 0; k < UN; ++k)
                if (c + 32 * k < c1) f(cv[k] & g.ctx_mask, sv[k]);
        }
    }
}

// Pass 1 (SCATTER = false): sizes of the segments.  Pass 2 (SCATTER = true): symbols into segments;
// `seg` then holds the segments' write cursors, which start at the segments' offsets.
// A warp takes units_per_warp consecutive entries of the unit list; the list is ordered by scale, so
// the warp sees each of its scales as one run of units.
template <bool SCATTER>
__global__ void __launch_bounds__(kWalkWarps * 32)
segment_walk_kernel(Geom g, const uint16_t* __restrict__ sym, const uint8_t* __restrict__ ctx, const uint16_t* __restrict__ scales,
                    const uint32_t* __restrict__ rank, const uint32_t* __restrict__ unit_sorted, long long units,
                    long long units_per_warp, uint32_t* __restrict__ seg, uint16_t* __restrict__ seg_syms) {
    __shared__ uint32_t s_cnt[kWalkWarps][256];
    __shared__ uint32_t s_base[kWalkWarps][256];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t* cnt = s_cnt[w];
    uint32_t* base = s_base[w];
    const long long warp = (long long)blockIdx.x * kWalkWarps + w;
    long long j = warp * units_per_warp;
    const long long end = (j + units_per_warp < units) ? j + units_per_warp : units;
    while (j < end) {
        const uint32_t v = unit_scale(g, scales, unit_sorted[j]);
        long long j2 = j + 1;
        while (j2 < end && unit_scale(g, scales, unit_sorted[j2]) == v) ++j2;
        const long long seg0 = (long long)rank[v] * g.nctx;
        for (int c = lane; c < g.nctx; c += 32) cnt[c] = 0;
        __syncwarp();
        for (long long uu = j; uu < j2; ++uu)
            for_unit_elements<false>(g, unit_sorted[uu], lane, ctx, sym, [&](uint32_t c, uint32_t) { atomicAdd(&cnt[c], 1u); });
        __syncwarp();
        if constexpr (!SCATTER) {
            for (int c = lane; c < g.nctx; c += 32)
                if (cnt[c]) atomicAdd(&seg[seg0 + c], cnt[c]);
        } else {
            for (int c = lane; c < g.nctx; c += 32) {
                base[c] = cnt[c] ? atomicAdd(&seg[seg0 + c], cnt[c]) : 0u;
                cnt[c] = 0;
            }
            __syncwarp();
            for (long long uu = j; uu < j2; ++uu)
                for_unit_elements<true>(g, unit_sorted[uu], lane, ctx, sym, [&](uint32_t c, uint32_t v) {
                    seg_syms[base[c] + atomicAdd(&cnt[c], 1u)] = (uint16_t)v;
                });
        }
        __syncwarp();
        j = j2;
    }
}

// chunks per segment, and which segments are split over several chunks
__global__ void chunk_plan_kernel(const uint32_t* __restrict__ seg_cnt, long long nseg, uint32_t* __restrict__ nchunks,
                                  uint32_t* __restrict__ split, uint32_t* __restrict__ present) {
    for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s <= nseg; s += (long long)gridDim.x * blockDim.x) {
        const uint32_t c = (s < nseg) ? seg_cnt[s] : 0u;
        nchunks[s] = (c + kChunk - 1) / kChunk;
        split[s] = c > (uint32_t)kChunk ? 1u : 0u;
        present[s] = c ? 1u : 0u;
    }
}

// after the scans: chunk -> segment, split segment -> segment
__global__ void chunk_fill_kernel(const uint32_t* __restrict__ seg_cnt, long long nseg, const uint32_t* __restrict__ chunk_ofs,
                                  const uint32_t* __restrict__ split_id, uint32_t* __restrict__ chunk_seg,
                                  uint32_t* __restrict__ split_seg) {
    for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s < nseg; s += (long long)gridDim.x * blockDim.x) {
        const uint32_t c = seg_cnt[s];
        const uint32_t nch = (c + kChunk - 1) / kChunk;
        for (uint32_t q = 0; q < nch; ++q) chunk_seg[chunk_ofs[s] + q] = (uint32_t)s;
        if (c > (uint32_t)kChunk) split_seg[split_id[s]] = (uint32_t)s;
    }
}

__global__ void split_range_init_kernel(uint32_t* __restrict__ split_range, long long num_split) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < num_split; i += (long long)gridDim.x * blockDim.x) {
        split_range[2 * i] = 0xFFFFu;
        split_range[2 * i + 1] = 0u;
    }
}

// Exclusive prefix of `flag` over the CTA (256 threads) and the CTA's total.
__device__ __forceinline__ uint32_t block_prefix(bool flag, uint32_t* s_warp, uint32_t& total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const uint32_t mask = __ballot_sync(0xFFFFFFFFu, flag);
    if (lane == 0) s_warp[w] = __popc(mask);
    __syncthreads();
    uint32_t before = 0, all = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t t = s_warp[i];
        if (i < w) before += t;
        all += t;
    }
    __syncthreads();
    total = all;
    return before + __popc(mask & ((1u << lane) - 1u));
}

// Writes the non-zero counters `count(d)`, d in [0, range), as (first + d, count) pairs from position
// `out` on, in ascending d; returns how many there were.  Called by all 256 threads of a CTA.
template <class F>
__device__ __forceinline__ uint32_t emit_nonzero(uint32_t range, uint32_t first, F&& count, uint32_t out, uint16_t* __restrict__ st_sym,
                                                 uint32_t* __restrict__ st_cnt, uint32_t* s_warp) {
    uint32_t written = 0;
    for (uint32_t d0 = 0; d0 < range; d0 += 256) {
        const uint32_t d = d0 + threadIdx.x;
        const uint32_t c = (d < range) ? count(d) : 0u;
        uint32_t total;
        const uint32_t p = block_prefix(c != 0, s_warp, total);
        if (c) {
            st_sym[out + written + p] = (uint16_t)(first + d);
            st_cnt[out + written + p] = c;
        }
        written += total;
    }
    return written;
}

// One chunk of one segment: count its symbols by value.  A segment that is a single chunk is finished
// here (its distinct symbols, ascending, with counts, go to the staging arrays at the segment's
// offset); a chunk of a split segment adds its counters to the segment's dense array.
__global__ void __launch_bounds__(256)
chunk_count_kernel(const uint16_t* __restrict__ seg_syms, const uint32_t* __restrict__ seg_cnt, const uint32_t* __restrict__ seg_ofs,
                   const uint32_t* __restrict__ chunk_seg, const uint32_t* __restrict__ chunk_ofs,
                   const uint32_t* __restrict__ split_id, uint32_t* __restrict__ dense, uint32_t* __restrict__ split_range,
                   uint16_t* __restrict__ st_sym, uint32_t* __restrict__ st_cnt, uint32_t* __restrict__ distinct) {
    __shared__ uint32_t s_count[kWindow];
    __shared__ uint32_t s_warp[8];
    __shared__ uint32_t s_lo, s_hi;
    const uint32_t s = chunk_seg[blockIdx.x];
    const uint32_t q = blockIdx.x - chunk_ofs[s];
    const uint32_t n = seg_cnt[s];
    const uint32_t e0 = seg_ofs[s] + q * (uint32_t)kChunk;
    const uint32_t e1 = (q * (uint32_t)kChunk + (uint32_t)kChunk < n) ? e0 + (uint32_t)kChunk : seg_ofs[s] + n;
    const bool split = n > (uint32_t)kChunk;
    if (threadIdx.x == 0) { s_lo = 0xFFFFu; s_hi = 0u; }
    __syncthreads();
    uint32_t lo = 0xFFFFu, hi = 0u;
    for (uint32_t e = e0 + threadIdx.x; e < e1; e += 256) {
        const uint32_t v = seg_syms[e];
        lo = v < lo ? v : lo;
        hi = v > hi ? v : hi;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint32_t a = __shfl_xor_sync(0xFFFFFFFFu, lo, o), b = __shfl_xor_sync(0xFFFFFFFFu, hi, o);
        lo = a < lo ? a : lo;
        hi = b > hi ? b : hi;
    }
    if ((threadIdx.x & 31) == 0) { atomicMin(&s_lo, lo); atomicMax(&s_hi, hi); }
    __syncthreads();
    lo = s_lo; hi = s_hi;
    uint32_t written = 0;
    for (uint32_t first = lo; first <= hi; first += (uint32_t)kWindow) {
        const uint32_t range = (hi - first + 1u < (uint32_t)kWindow) ? hi - first + 1u : (uint32_t)kWindow;
        for (uint32_t d = threadIdx.x; d < range; d += 256) s_count[d] = 0;
        __syncthreads();
        for (uint32_t e = e0 + threadIdx.x; e < e1; e += 256) {
            const uint32_t d = (uint32_t)seg_syms[e] - first;
            if (d < range) atomicAdd(&s_count[d], 1u);
        }
        __syncthreads();
        if (split) {
            uint32_t* mine = dense + (size_t)split_id[s] * 65536u + first;
            for (uint32_t d = threadIdx.x; d < range; d += 256)
                if (s_count[d]) atomicAdd(&mine[d], s_count[d]);
            if (threadIdx.x == 0 && first == lo) {   // the segment's symbol range, for split_finish_kernel
                atomicMin(&split_range[2 * split_id[s]], lo);
                atomicMax(&split_range[2 * split_id[s] + 1], hi);
            }
        } else {
            written += emit_nonzero(range, first, [&](uint32_t d) { return s_count[d]; }, seg_ofs[s] + written, st_sym, st_cnt, s_warp);
        }
        __syncthreads();
    }
    if (!split && threadIdx.x == 0) distinct[s] = written;
}

// A split segment's dense counters -> its distinct symbols, ascending, with counts.
__global__ void __launch_bounds__(256)
split_finish_kernel(const uint32_t* __restrict__ split_seg, const uint32_t* __restrict__ seg_ofs, const uint32_t* __restrict__ dense,
                    const uint32_t* __restrict__ split_range, uint16_t* __restrict__ st_sym, uint32_t* __restrict__ st_cnt,
                    uint32_t* __restrict__ distinct) {
    __shared__ uint32_t s_warp[8];
    const uint32_t s = split_seg[blockIdx.x];
    const uint32_t lo = split_range[2 * blockIdx.x], hi = split_range[2 * blockIdx.x + 1];   // the chunks' smallest and largest symbol
    const uint32_t* mine = dense + (size_t)blockIdx.x * 65536u + lo;
    const uint32_t written = emit_nonzero(hi - lo + 1u, lo, [&](uint32_t d) { return mine[d]; }, seg_ofs[s], st_sym, st_cnt, s_warp);
    if (threadIdx.x == 0) distinct[s] = written;
}

// Staging arrays -> items and counts, in segment order; a warp per segment.
__global__ void gather_items_kernel(const uint32_t* __restrict__ seg_cnt, const uint32_t* __restrict__ seg_ofs,
                                    const uint32_t* __restrict__ item_ofs, const uint32_t* __restrict__ ctx_id, long long nseg,
                                    int nctx, const uint16_t* __restrict__ scale_of_rank, const uint16_t* __restrict__ st_sym,
                                    const uint32_t* __restrict__ st_cnt, unsigned long long* __restrict__ items,
                                    int* __restrict__ counts, int* __restrict__ ctx_ofs, uint32_t* __restrict__ ctx_key) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long s = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < nseg; s += warps) {
        if (seg_cnt[s] == 0) continue;
        const uint32_t g = ctx_id[s], a = item_ofs[s], nd = item_ofs[s + 1] - a, from = seg_ofs[s];
        const uint32_t key = ((uint32_t)scale_of_rank[s / nctx] << 16) | (uint32_t)(s % nctx);
        if (lane == 0) { ctx_ofs[g] = (int)a; ctx_key[g] = key; }
        for (uint32_t i = lane; i < nd; i += 32) {
            items[a + i] = ((unsigned long long)key << 16) | st_sym[from + i];
            counts[a + i] = (int)st_cnt[from + i];
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) ctx_ofs[ctx_id[nseg]] = (int)item_ofs[nseg];
}

}  // namespace hist
}  // namespace mps
