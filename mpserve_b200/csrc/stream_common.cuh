// Pieces shared by the persistent decode kernels: launch arguments, the work item a scout warp
// prepares, and thin wrappers over the sm_100a instructions they are built from (mbarrier,
// cp.async, cp.async.bulk without tensor map or multicast, named barriers, cache-hinted prefetch).
#pragma once

#include "mps_common.cuh"

namespace mps {

struct BatchArgs {
    mps_bucket_tensor single;            // used when tensors == nullptr
    const mps_bucket_tensor* tensors;    // device array, or nullptr
    const int64_t* item_prefix;          // device [count+1], or nullptr (single tensor)
    int count;
    int total_items;
    int stall_block_plus1;               // self-test only: the producer leaves block (this - 1) of steps out; 0: never
    uint32_t spin_limit;                 // polls before a wait gives up; 0: kSpinLimit
};

// ------------------------------------------------------------------------------------------------
// Work item prepared one item ahead by the scout warp, so that the decoding warps start every item
// with its geometry and row bases already in shared memory and its tables already on their way
// into L2 instead of walking a chain of dependent global loads.
// ------------------------------------------------------------------------------------------------
struct Prepared {
    int valid;  // 0: the queue is empty
    int ok;     // geometry usable, else the item is skipped
    int ti, mode;
    uint32_t k, k_eff, t_begin, ebits;
    long long b, total, wb;
    int32_t row_a, nrows, col_start, col_len;   // (int32 in the sidecar)
    int rows_ok, rows_vec, rows_al16;
    uint32_t bit_lo;  // low six bits of the bucket's bit base (0 in every sidecar the reference encoder writes)
    // tables: must they be staged (another context -> table map than the item decoded before), and are they
    // one run of consecutive table ids in context order (the reference encoder numbers tables by (scale, context))
    int16_t restage, tab_dense;
    int32_t tab_first;   // table id of the first context that has one
    uint32_t tab_count;  // contexts that have one
};

struct BitOrigin {        // bitstream of the item seen from a 16-byte aligned origin
    const uint8_t* base;  // 16-byte aligned
    uint32_t last_ofs;    // largest 16-byte aligned offset whose chunk lies wholly inside the bitstream
    uint32_t tail_ofs;    // offset of a final 8-byte half chunk (bitstream ends mid-chunk), else 0xFFFFFFFF
    uint32_t bit_delta;   // bits between the origin and the bucket's first bit
};

// Geometry of one work item on the streaming path (uniform across the CTA).
struct StreamItem {
    const uint8_t* ctx_bytes;
    uint16_t* out;
    const uint32_t* startbit;
    const uint32_t* rowbase;
    BitOrigin bo;
    uint32_t t_begin, k_eff, col_len;
    uint32_t nsteps;       // steps of this item, a ragged last one included
    uint32_t nfull;        // steps in which every sub-stream of the bucket has an element
    uint32_t last_active;  // local sub-streams that have an element in the ragged last step (0: there is none)
    uint32_t flat_bytes;   // != 0: the bucket's whole bitstream, this many bytes from bo.base, is copied into shared memory
    uint32_t nrows;        // rows (groups) of the bucket
};

constexpr uint32_t kSpinLimit = 1u << 22;  // bounded waits: give up, flag, return
constexpr int kMaxGrab = 8;          // most work items one CTA takes from the queue at once
constexpr int kGrabSlack = 4;        // a grab is at most 1/(kGrabSlack * CTAs) of what is left

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(p)); }

// barrier 1 (decoding threads only) with an OR reduction
__device__ __forceinline__ int group_or(int pred, int nthreads) {
    int r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.s32 p, %1, 0;\n\tbar.red.or.pred q, 1, %2, p;\n\tselp.s32 %0, 1, 0, q;\n\t}"
        : "=r"(r) : "r"(pred), "r"(nthreads) : "memory");
    return r;
}
__device__ __forceinline__ void group_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false when the barrier did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit) {
#pragma unroll 1
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds_ordered(uint32_t addr) {  // ordered with the async copies
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// CH context bytes of one step, as the decoding thread loads them from the ring
template <int CH> struct Ctx;
template <> struct Ctx<1> {
    using T = uint32_t;
    static __device__ __forceinline__ T ld(const uint8_t* p) { return ld_stream_u8(p); }
    static __device__ __forceinline__ uint32_t byte(T v, int) { return v; }
};
template <> struct Ctx<2> {
    using T = uint32_t;
    static __device__ __forceinline__ T ld(const uint8_t* p) { return ld_stream_u16(p); }
    static __device__ __forceinline__ uint32_t byte(T v, int c) { return __byte_perm(v, 0u, 0x4440u | (uint32_t)c); }
};
template <> struct Ctx<4> {
    using T = uint32_t;
    static __device__ __forceinline__ T ld(const uint8_t* p) { return ld_stream_u32(p); }
    static __device__ __forceinline__ uint32_t byte(T v, int c) { return __byte_perm(v, 0u, 0x4440u | (uint32_t)c); }
};
template <> struct Ctx<8> {
    using T = uint2;
    static __device__ __forceinline__ T ld(const uint8_t* p) { return ld_stream_u64(p); }
    static __device__ __forceinline__ uint32_t byte(T v, int c) { return __byte_perm((c < 4) ? v.x : v.y, 0u, 0x4440u | (uint32_t)(c & 3)); }
};

template <int CH>
__device__ __forceinline__ typename Ctx<CH>::T lds_ctx(uint32_t addr) {
    if constexpr (CH == 8) {
        uint2 v;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
        return v;
    } else {
        uint32_t v;
        if constexpr (CH == 4) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        else if constexpr (CH == 2) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        else asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        return v;
    }
}

// SM count of the current device (148 on B200), remembered per device.
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace mps
