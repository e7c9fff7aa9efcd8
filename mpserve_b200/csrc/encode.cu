// GPU builder of the Huffman sidecar: replaces the single-threaded CPU encoder of the reference
// (kernel/build_huffman.cu) with device passes that produce byte-identical artifacts.
//
//   analyze    the histogram of every context (build_huffman.cu:392-412), contexts in ascending key
//              order: a two-level count, by scale and then by context, with no sort over the elements
//              (histogram.cuh); then each context's items ordered by (count, symbol)
//   codebooks  per context: order by (count, symbol), ESC reduction when there are more symbols than
//              table slots (:479-535), length-limited code lengths (package-merge, :46-118), canonical
//              codes in item order (:171-203), lookup-table fill and 4-bit length packing (:205-239)
//   layout     bits of every sub-stream (one thread per sub-stream, elements t, t+k_eff, ...), prefix
//              sums per bucket, 64-bit aligned bucket bases (:811-879)
//   emit       the same walk again, writing codes MSB-first with one 64-bit atomic OR per word (:881-911)
//
// Scans, and the sorts of the distinct (context, symbol) items -- a hundredth of the elements for a
// quantised weight -- use CUB (device-wide scan / radix sort from the CUDA toolkit); everything that
// touches every element is written here.  Bucket row lists are small host-side
// metadata and are built by the caller from the scale tensor (mpserve_b200/encoder.py).
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <string.h>

#include "histogram.cuh"
#include "mps_common.cuh"

namespace mps {

// ------------------------------------------------------------------------------------------------
// build state: where things live inside the caller's workspace (host-side POD, opaque to callers)
// ------------------------------------------------------------------------------------------------
struct BuildState {
    int64_t numel, n, m;
    int64_t N;                 // distinct (context, symbol) pairs
    int64_t G;                 // contexts
    int32_t L, variant;
    int32_t group_size, pad_;  // elements per group of the ragged layout
    uint8_t* ws;               // device workspace base
    size_t ws_bytes;
    // offsets (bytes) into ws
    size_t o_items;            // uint64 [N]  scale<<32 | ctx<<16 | sym, ascending
    size_t o_counts;           // int32  [N]
    size_t o_ctx_ofs;          // int32  [G+1] first item of each context
    size_t o_ctx_key;          // uint32 [G]   scale<<16 | ctx
    size_t o_perm;             // int32  [N]   items of each context ordered by (count, sym)
    size_t o_enc;              // uint32 [N]   len<<16 | code of each item, 0 = not coded (ESC'd)
    size_t o_esc;              // uint32 [G]   len<<16 | code of the context's ESC code (0: none)
    size_t o_escsym;           // uint16 [G]
    size_t o_scratch;          // start of the reusable scratch area
    size_t scratch_bytes;
    int32_t* d_flag;           // device error flag (first word of ws)
    // shared-table layout only (carved from the scratch area by the shared-table calls)
    int64_t num_scales, num_chunks;
    size_t o_sh_keep;          // start of what the layout call leaves for the emit call
    size_t o_sh_end;           // end of it
    // rectangular buckets: what the layout call leaves in the scratch area for the emit call
    size_t o_rect_codes;       // uint32 [numel] code of every element, in bucket order (see rect_codes_kernel)
    size_t o_rect_ebase;       // uint64 [B+1]   first element of every bucket in that order
    int64_t rect_buckets;      // B of the layout call (0: no layout yet)
};
static_assert(sizeof(BuildState) <= 256, "mps_build_state is 256 bytes");

static inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

enum { V_FP8 = 0, V_AWQ_BUCKET = 1, V_AWQ_BYSCALE = 2, V_AWQ_SHARED = 3 };

// ------------------------------------------------------------------------------------------------
// analyze
// ------------------------------------------------------------------------------------------------
// keys that order the items of every context by (count, symbol), and the context of every item
__global__ void item_sort_keys_kernel(const unsigned long long* __restrict__ items, const int* __restrict__ counts,
                                      const int* __restrict__ ctx_ofs, int G, long long N, unsigned long long* __restrict__ k1,
                                      int* __restrict__ v, uint32_t* __restrict__ ctx_of_item) {
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < N; j += (long long)gridDim.x * blockDim.x) {
        k1[j] = ((unsigned long long)(uint32_t)counts[j] << 16) | (items[j] & 0xFFFFull);
        v[j] = (int)j;
        int lo = 0, hi = G;  // last context that starts at or before item j
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((long long)ctx_ofs[mid] <= j) lo = mid; else hi = mid;
        }
        ctx_of_item[j] = (uint32_t)lo;
    }
}

__global__ void gather_u32_kernel(const uint32_t* __restrict__ src, const int* __restrict__ idx, long long N,
                                  uint32_t* __restrict__ dst) {
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < N; j += (long long)gridDim.x * blockDim.x)
        dst[j] = src[idx[j]];
}

// SM count of the current device (148 on B200)
static int sm_count_host() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
}

static int grid_for(long long n, int threads = 256) {
    long long b = (n + threads - 1) / threads;
    if (b > 148LL * 32) b = 148LL * 32;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace mps

namespace mps {

// ------------------------------------------------------------------------------------------------
// codebooks: one thread per context, thread-private arrays interleaved in global scratch
// ------------------------------------------------------------------------------------------------
struct CbScratch {      // arrays of a chunk of `chunk` contexts; element i of slot s at [i * chunk + s]
    unsigned long long* w;    // [TS]   weights of the final item list (ascending)
    uint16_t* sym;            // [TS]
    int* src;                 // [TS]   index into the histogram items, -1 for the ESC item
    unsigned long long* cur;  // [KEEP] package-merge list of the current level
    unsigned long long* nxt;  // [KEEP]
    uint8_t* flag;            // [L * KEEP] 1 where the level's list holds a leaf
    uint8_t* len;             // [TS]
    int chunk;
};

__device__ __forceinline__ void set_nibble(uint8_t* packed, long long idx, uint32_t v) {
    uint8_t b = packed[idx >> 1];
    b = (idx & 1) ? (uint8_t)((b & 0x0F) | (v << 4)) : (uint8_t)((b & 0xF0) | (v & 0x0F));
    packed[idx >> 1] = b;
}

// Length-limited code lengths of n >= 2 ascending weights (build_huffman.cu:46-118), by counting
// leaves in list prefixes instead of walking package trees: the items chosen at every level are a
// prefix of that level's list, because packages pair consecutive items from the front and a leaf
// wins a tie when lists are merged.
__device__ bool package_merge_device(const CbScratch& S, int s, int n, int L) {
#define AT(arr, i) arr[(long long)(i) * S.chunk + s]
    const int K = 2 * (n - 1), keep = 2 * K;
    const int KEEP = 4 * ((1 << L) - 1);
    int cur_n = n;
    for (int i = 0; i < n; ++i) { AT(S.cur, i) = AT(S.w, i); AT(S.flag, i) = 1; }
    unsigned long long* cur = S.cur;
    unsigned long long* nxt = S.nxt;
    for (int p = 0; p < L - 1; ++p) {
        const int trunc = cur_n < keep ? cur_n : keep;
        const int npk = trunc / 2;
        uint8_t* fl = S.flag + (long long)(p + 1) * KEEP * S.chunk;
        int i = 0, j = 0, o = 0;
        while (o < keep && (i < n || j < npk)) {
            bool leaf;
            unsigned long long pw = 0;
            if (j < npk) pw = AT(cur, 2 * j) + AT(cur, 2 * j + 1);
            if (i < n && j < npk) leaf = AT(S.w, i) <= pw;
            else leaf = (i < n);
            if (leaf) { AT(nxt, o) = AT(S.w, i); ++i; } else { AT(nxt, o) = pw; ++j; }
            AT(fl, o) = leaf ? 1 : 0;
            ++o;
        }
        cur_n = o;
        unsigned long long* t = cur; cur = nxt; nxt = t;
    }
    if (cur_n < K) return false;
    for (int i = 0; i < n; ++i) AT(S.len, i) = 0;
    int take = K;
    for (int lvl = L - 1; lvl >= 0 && take > 0; --lvl) {
        const uint8_t* fl = S.flag + (long long)lvl * KEEP * S.chunk;
        int c = 0;
        for (int i = 0; i < take; ++i) c += AT(fl, i);
        for (int i = 0; i < c; ++i) AT(S.len, i) = (uint8_t)(AT(S.len, i) + 1);
        take = 2 * (take - c);
    }
    return true;
}

// variant: V_FP8, V_AWQ_BUCKET or V_AWQ_BYSCALE.  Tables are written at index g (contexts in ascending key order).
__global__ void codebook_kernel(const unsigned long long* __restrict__ items, const int* __restrict__ counts,
                                const int* __restrict__ ctx_ofs, const int* __restrict__ perm, long long g0, long long g1,
                                int L, int variant, CbScratch S, uint16_t* __restrict__ out_syms,
                                uint8_t* __restrict__ out_lens, uint32_t* __restrict__ enc, uint32_t* __restrict__ esc,
                                uint16_t* __restrict__ escsym, int* __restrict__ err, const int* __restrict__ row_of) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    const long long g = g0 + s;
    if (g >= g1 || s >= S.chunk) return;
    const int TS = 1 << L;
    const int a = ctx_ofs[g], b = ctx_ofs[g + 1], cnt = b - a;
    // shared-table sidecars keep one table per (scale id, context) stream, present or not, and whole-byte
    // lengths; the bucket formats keep one table per context that occurs, lengths packed two per byte
    const bool bytes = (variant == V_AWQ_SHARED);
    const long long row = row_of ? row_of[g] : g;
    uint16_t* tsym = out_syms + row * TS;
    uint8_t* tlen = out_lens + (bytes ? row * TS : row * (TS / 2));
    esc[g] = 0;
    escsym[g] = 0;
    if (cnt <= 0) return;
    if (cnt == 1) {  // single symbol: length 1, code 0, every slot (build_huffman.cu:464-472)
        const uint16_t sy = (uint16_t)(items[a] & 0xFFFF);
        for (int i = 0; i < TS; ++i) tsym[i] = sy;
        if (bytes) for (int i = 0; i < TS; ++i) tlen[i] = 1;
        else for (int i = 0; i < TS / 2; ++i) tlen[i] = 0x11;
        enc[a] = (1u << 16);
        return;
    }
    int n = cnt;
    bool use_esc = false;
    uint16_t esc_sym = 0;
    int esc_pos = -1;
    if (cnt > TS) {
        // keep the TS-1 most frequent (ties: smaller symbol first), fold the rest into one ESC item
        use_esc = true;
        const int keepk = TS - 1;
        const int p = b - keepk;                       // lowest kept position if there were no ties
        const int fb = counts[perm[p]];                // count of the boundary class
        int lo = p, hi = p;
        while (lo > a && counts[perm[lo - 1]] == fb) --lo;
        while (hi < b && counts[perm[hi]] == fb) ++hi;  // class fb is perm[lo, hi)
        const int r = keepk - (b - hi);                // how many of the class are kept: its first r
        long long esc_w = 0;
        int seen = 0;
        uint32_t cand = 0;
        bool cand_done = false;
        for (int j = a; j < b; ++j) {                  // histogram order = ascending symbol
            const int c = counts[j];
            const bool kept = c > fb || (c == fb && seen < r);
            if (c == fb) ++seen;
            const uint32_t sy = (uint32_t)(items[j] & 0xFFFF);
            if (!kept) { esc_w += c; enc[j] = 0; }
            if (!cand_done) {  // smallest symbol not among the kept ones (by-scale: not in the context at all)
                if ((kept || variant == V_AWQ_BYSCALE) && sy == cand) ++cand;
                else if (sy > cand) cand_done = true;
            }
        }
        esc_sym = (uint16_t)(cand <= 0xFFFFu ? cand : 0xFFFFu);
        int esc_i = (int)esc_w;                        // the reference accumulates in int
        if (variant == V_AWQ_SHARED) esc_i = esc_w > 2147483647LL ? 2147483647 : (int)esc_w;  // (:2345-2352)
        if ((variant == V_AWQ_BUCKET || variant == V_AWQ_SHARED) && esc_i <= 0) esc_i = 1;
        n = 0;
        bool placed = false;
        if (variant == V_AWQ_BYSCALE) {
            // The by-scale builder keeps the kept items in DESCENDING order with the ESC item last and
            // does not re-sort them (build_huffman.cu:1283-1301), while the lengths it pairs them with
            // positionally are those of the ASCENDING weights: weights go in ascending, symbols in
            // descending order (classes from the most frequent down, ascending symbol inside a class).
            int wq = 0;  // ascending weights with the ESC weight merged in
            for (int q = 0; q < keepk; ++q) {
                const int j = perm[q < r ? lo + q : hi + (q - r)];
                const unsigned long long w = (unsigned long long)(uint32_t)counts[j];
                if (!placed && (unsigned long long)(uint32_t)esc_i <= w) { AT(S.w, wq) = (unsigned long long)(uint32_t)esc_i; ++wq; placed = true; }
                AT(S.w, wq) = w; ++wq;
            }
            if (!placed) { AT(S.w, wq) = (unsigned long long)(uint32_t)esc_i; ++wq; }
            int top = b;  // classes are runs of equal count in perm[a, b)
            while (n < keepk) {
                int cs = top - 1;
                const int f = counts[perm[cs]];
                while (cs > a && counts[perm[cs - 1]] == f) --cs;
                for (int q = cs; q < top && n < keepk; ++q) {
                    const int j = perm[q];
                    AT(S.sym, n) = (uint16_t)(items[j] & 0xFFFF); AT(S.src, n) = j; ++n;
                }
                top = cs;
            }
            AT(S.sym, n) = esc_sym; AT(S.src, n) = -1; esc_pos = n; ++n;
            placed = true;
        }
        // final list, ascending by (weight, symbol): perm[lo, lo+r), perm[hi, b), ESC inserted in order
        for (int q = 0; q < keepk && variant != V_AWQ_BYSCALE; ++q) {
            const int j = perm[q < r ? lo + q : hi + (q - r)];
            const unsigned long long w = (unsigned long long)(uint32_t)counts[j];
            const uint16_t sy = (uint16_t)(items[j] & 0xFFFF);
            if (!placed && ((unsigned long long)(uint32_t)esc_i < w || ((unsigned long long)(uint32_t)esc_i == w && esc_sym < sy))) {
                AT(S.w, n) = (unsigned long long)(uint32_t)esc_i; AT(S.sym, n) = esc_sym; AT(S.src, n) = -1; esc_pos = n; ++n;
                placed = true;
            }
            AT(S.w, n) = w; AT(S.sym, n) = sy; AT(S.src, n) = j; ++n;
        }
        if (!placed) { AT(S.w, n) = (unsigned long long)(uint32_t)esc_i; AT(S.sym, n) = esc_sym; AT(S.src, n) = -1; esc_pos = n; ++n; }
    } else {
        for (int q = 0; q < cnt; ++q) {
            const int j = perm[a + q];
            AT(S.w, q) = (unsigned long long)(uint32_t)counts[j];
            AT(S.sym, q) = (uint16_t)(items[j] & 0xFFFF);
            AT(S.src, q) = j;
        }
    }
    if (!package_merge_device(S, s, n, L)) { atomicExch(err, 2); return; }
    if (use_esc && (variant == V_AWQ_BUCKET || variant == V_AWQ_BYSCALE)) AT(S.len, esc_pos) = (uint8_t)L;  // ESC code forced to L bits (:1812-1816)

    // canonical codes handed out in item order within each length (build_huffman.cu:171-203)
    uint32_t next_code[17];
    {
        int bl[17];
        for (int i = 0; i < 17; ++i) bl[i] = 0;
        for (int i = 0; i < n; ++i) bl[AT(S.len, i)]++;
        uint32_t code = 0;
        next_code[0] = 0;
        for (int bits = 1; bits < 17; ++bits) { code = (code + (uint32_t)bl[bits - 1]) << 1; next_code[bits] = code; }
    }
    for (int i = 0; i < n; ++i) {
        const int len = AT(S.len, i);
        const uint32_t code = next_code[len]++;
        const uint16_t sy = AT(S.sym, i);
        const int src = AT(S.src, i);
        const uint32_t packed = ((uint32_t)len << 16) | code;
        if (src >= 0) enc[src] = packed; else { esc[g] = packed; escsym[g] = sy; }
        const uint32_t nib = (variant == V_FP8 && src < 0) ? (uint32_t)(len | 8) : (uint32_t)len;
        const uint32_t base = code << (L - len), fill = 1u << (L - len);
        for (uint32_t t = 0; t < fill; ++t) {
            const uint32_t idx = base + t;
            if (idx < (uint32_t)TS) {
                tsym[idx] = sy;
                if (bytes) tlen[idx] = (uint8_t)len; else set_nibble(tlen, idx, nib);
            }
        }
    }
    if (use_esc && (variant == V_AWQ_BUCKET || variant == V_AWQ_BYSCALE)) {  // every slot that shows the ESC symbol is marked 15 (:1822-1829)
        for (int i = 0; i < TS; ++i)
            if (tsym[i] == esc_sym) set_nibble(tlen, i, 15u);
    }
    if (use_esc && bytes) {             // shared tables mark them with bit 7 (:2410-2415)
        for (int i = 0; i < TS; ++i)
            if (tsym[i] == esc_sym) tlen[i] = (uint8_t)(tlen[i] | 0x80u);
    }
#undef AT
}

}  // namespace mps

namespace mps {

// ------------------------------------------------------------------------------------------------
// bucket tables, layout, emit (rectangular buckets: FP8 and AWQ bucket builders)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ int find_u32(const uint32_t* __restrict__ a, int n, uint32_t key) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1;
        const uint32_t v = a[mid];
        if (v == key) return mid;
        if (v < key) lo = mid + 1; else hi = mid - 1;
    }
    return -1;
}

// context -> table id of every bucket (build_huffman.cu:737-746)
__global__ void bucket_table_kernel(const uint32_t* __restrict__ ctx_key, int G, const uint16_t* __restrict__ bucket_scale,
                                    long long B, int nctx, int32_t* __restrict__ out) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < B * nctx; i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / nctx;
        const uint32_t c = (uint32_t)(i - b * nctx);
        out[i] = find_u32(ctx_key, G, ((uint32_t)bucket_scale[b] << 16) | c);
    }
}

// first-appearance list of a bucket's tables and context -> position in it (build_huffman.cu:748-783).
// One warp per bucket walks the 256 contexts 32 at a time: every lane first looks its table id up in
// the list built so far (kept in shared memory), the lanes that bring a new id are grouped by value
// with a warp match, and the lowest lane of each group appends the id at the position its rank
// among those leaders gives, which is the order a sequential scan would have appended them in.
constexpr int kUniqueWarps = 4;
__global__ void __launch_bounds__(kUniqueWarps * 32)
bucket_unique_kernel(const int32_t* __restrict__ bt, long long B, int32_t* __restrict__ U, int32_t* __restrict__ uniq,
                     int16_t* __restrict__ uidx) {
    __shared__ int32_t s_list[kUniqueWarps][256];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int32_t* list = s_list[w];
    for (long long b = (long long)blockIdx.x * kUniqueWarps + w; b < B; b += (long long)gridDim.x * kUniqueWarps) {
        int32_t u = 0;
        for (int c0 = 0; c0 < 256; c0 += 32) {
            const int32_t gid = bt[b * 256 + c0 + lane];
            const bool valid = gid >= 0;
            int32_t pos = -1;
            if (valid)
                for (int32_t j = 0; j < u; ++j)
                    if (list[j] == gid) { pos = j; break; }
            const bool fresh = valid && pos < 0;
            // lanes without a new id get a key no other lane has (-1 - lane is below every table id)
            const uint32_t same = __match_any_sync(0xFFFFFFFFu, fresh ? gid : -1 - lane);
            const int first = __ffs(same) - 1;
            const bool leader = fresh && first == lane;
            const uint32_t leaders = __ballot_sync(0xFFFFFFFFu, leader);
            int32_t mine = u + __popc(leaders & ((1u << lane) - 1u));
            if (leader) list[mine] = gid;
            mine = __shfl_sync(0xFFFFFFFFu, mine, first);
            if (fresh) pos = mine;
            uidx[b * 256 + c0 + lane] = (int16_t)pos;
            u += __popc(leaders);
            __syncwarp();
        }
        for (int j = lane; j < 256; j += 32) uniq[b * 256 + j] = (j < u) ? list[j] : -1;
        if (lane == 0) U[b] = u;
        __syncwarp();
    }
}

struct RectGeom {
    const uint16_t* sym;              // [n*m] BF16 bit patterns
    const uint8_t* ctx;               // [n*m]
    const int32_t* bucket_table;      // [B, nctx]
    const int32_t* col_start;         // [B]
    const int32_t* col_len;           // [B]
    const int32_t* row_ofs;           // [B+1]
    const int32_t* rows;              // row lists
    const int32_t* group_col;         // ragged buckets: column start of every listed group, else nullptr
    long long B, m;
    int k, nctx, group_size;          // group_size: elements per group (ragged buckets)
    uint32_t ctx_mask;
};

struct CodeBook {
    const unsigned long long* items;
    const int* ctx_ofs;
    const uint32_t* enc;
    const uint32_t* esc;
    const uint16_t* escsym;
};

// (code, length) of one element, ESC expansion included: returns total bits, code(s) via out params
__device__ __forceinline__ int element_code(const CodeBook& cb, int gid, uint32_t sym, uint32_t& code, int& len,
                                            bool& raw) {
    const int a = cb.ctx_ofs[gid], b = cb.ctx_ofs[gid + 1];
    int lo = a, hi = b - 1, j = -1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1;
        const uint32_t v = (uint32_t)(cb.items[mid] & 0xFFFF);
        if (v == sym) { j = mid; break; }
        if (v < sym) lo = mid + 1; else hi = mid - 1;
    }
    raw = false;
    if (j < 0) return -1;
    uint32_t lc = cb.enc[j];
    if (lc == 0) {                       // not in the codebook: ESC code, then the raw 16 bits ...
        lc = cb.esc[gid];
        if (lc == 0) return -1;
        raw = (sym != cb.escsym[gid]);   // ... unless the symbol equals the synthetic ESC symbol, which the
    }                                    // reference's encoder map resolves to the bare ESC code
    code = lc & 0xFFFF;
    len = (int)(lc >> 16);
    return len + (raw ? 16 : 0);
}

// elements of every bucket (rows x columns), [B] = 0 for the scan that follows
__global__ void bucket_totals_kernel(RectGeom g, unsigned long long* __restrict__ totals) {
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b <= g.B; b += (long long)gridDim.x * blockDim.x) {
        unsigned long long t = 0;
        if (b < g.B) t = (unsigned long long)(g.row_ofs[b + 1] - g.row_ofs[b]) * (unsigned long long)(g.group_col ? g.group_size : g.col_len[b]);
        totals[b] = t;
    }
}

// The code of every element, looked up once, in parallel, and stored in bucket order (element e of
// bucket b at ebase[b] + e), so that the two walks over the sub-streams (sizes, then bits) read their
// elements t, t + k, ... as coalesced words instead of searching a codebook per element.
// An entry is len << 16 | code, bit 31 set when 16 raw bits follow (ESC); 0xFFFFFFFF: no code.
// A CTA serves slabs of one bucket and first copies that bucket's codebooks (the symbols and codes of
// its contexts, a few thousand items) into shared memory; a bucket with more items than fit is
// searched in global memory instead.
constexpr int kCodeCap = 6144;     // items of a bucket's codebooks that fit shared memory as (symbol, code) lists
constexpr int kDirectCap = 9216;   // ... or, in the same space, entries of its direct maps (see below)
constexpr int kCodeSlab = 8192;
constexpr uint32_t kNoCode = 0xFFFFFFFFu;
// How a CTA finds an element's code, in order of preference:
//   direct  the symbols a context of a quantised weight sees are a few dozen neighbouring BF16 patterns, so
//           every context gets a map indexed by (symbol - its smallest symbol); used when the maps of the
//           bucket's contexts fit kDirectCap entries together: one shared-memory load per element;
//   lists   the contexts' sorted symbol lists in shared memory, binary search (some hundred instructions
//           per element, half of the lanes idle);
//   global  the same search in global memory, for buckets whose lists do not fit either.
__global__ void __launch_bounds__(256)
rect_codes_kernel(RectGeom g, CodeBook cb, long long G, const unsigned long long* __restrict__ ebase, uint32_t* __restrict__ lc) {
    __shared__ uint32_t s_ofs[257];    // first item of every context in the lists
    __shared__ uint32_t s_dofs[257];   // first entry of every context's direct map
    __shared__ uint16_t s_lo[256];     // smallest symbol of every context
    __shared__ int32_t s_gid[256];
    __shared__ int s_first[256];       // first item of every context in the global arrays
    __shared__ uint32_t s_esc[256];
    __shared__ uint16_t s_escsym[256];
    __shared__ uint32_t s_pool[kDirectCap];   // direct maps, or lists: codes [kCodeCap] then symbols [kCodeCap]
    __shared__ uint32_t s_warp[2][8];
    static_assert(kDirectCap * 4 >= kCodeCap * 6, "the lists share the direct maps' space");
    uint32_t* const s_enc = s_pool;
    uint16_t* const s_sym = reinterpret_cast<uint16_t*>(s_pool + kCodeCap);
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const long long b = blockIdx.x;
    const int row_a = g.row_ofs[b];
    const unsigned long long nrows = (unsigned long long)(g.row_ofs[b + 1] - row_a);
    const unsigned long long col_len = (unsigned long long)(g.group_col ? g.group_size : g.col_len[b]);
    const long long col_start = g.group_col ? 0 : g.col_start[b];
    const unsigned long long total = nrows * col_len;
    const unsigned long long nslab = (total + kCodeSlab - 1) / kCodeSlab;
    if (blockIdx.y >= nslab) return;

    // this bucket's contexts: table id, items, range of symbols, ESC code
    int32_t gid = -1;
    uint32_t nd = 0, span = 0, lo_sym = 0;
    int first = 0;
    if (tid < g.nctx) {
        gid = g.bucket_table[b * g.nctx + tid];
        if (gid >= G) gid = -1;
        if (gid >= 0) {
            first = cb.ctx_ofs[gid];
            nd = (uint32_t)(cb.ctx_ofs[gid + 1] - first);
            if (nd) {   // items are in ascending symbol order
                lo_sym = (uint32_t)(cb.items[first] & 0xFFFF);
                span = (uint32_t)(cb.items[first + (int)nd - 1] & 0xFFFF) - lo_sym + 1u;
            }
        }
    }
    s_gid[tid] = gid;
    s_first[tid] = first;
    s_lo[tid] = (uint16_t)lo_sym;
    s_esc[tid] = gid >= 0 ? cb.esc[gid] : 0u;
    s_escsym[tid] = gid >= 0 ? cb.escsym[gid] : (uint16_t)0;
    uint32_t incl = nd, incl_span = span;   // inclusive prefixes over the CTA
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o), vs = __shfl_up_sync(0xFFFFFFFFu, incl_span, o);
        if (lane >= o) { incl += v; incl_span += vs; }
    }
    if (lane == 31) { s_warp[0][w] = incl; s_warp[1][w] = incl_span; }
    __syncthreads();
    uint32_t before = 0, items_total = 0, before_span = 0, span_total = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i < w) { before += s_warp[0][i]; before_span += s_warp[1][i]; }
        items_total += s_warp[0][i];
        span_total += s_warp[1][i];
    }
    s_ofs[tid] = before + incl - nd;
    s_dofs[tid] = before_span + incl_span - span;
    if (tid == 255) { s_ofs[256] = items_total; s_dofs[256] = span_total; }
    const bool direct = span_total <= (uint32_t)kDirectCap;
    const bool staged = !direct && items_total <= (uint32_t)kCodeCap;
    if (direct)
        for (uint32_t i = tid; i < span_total; i += 256) s_pool[i] = kNoCode;
    __syncthreads();
    if (direct || staged) {
        // every item of the bucket's contexts, four copies in flight per thread
        constexpr int SUN = 4;
        for (uint32_t j0 = tid; j0 < items_total; j0 += 256 * SUN) {
            long long src[SUN];
            int cx[SUN];
#pragma unroll
            for (int u = 0; u < SUN; ++u) {
                const uint32_t j = j0 + 256u * u;
                int lo = 0, hi = 256;   // last context whose items start at or before j
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (s_ofs[mid] <= j) lo = mid; else hi = mid;
                }
                cx[u] = lo;
                src[u] = (j < items_total) ? (long long)s_first[lo] + (j - s_ofs[lo]) : -1;
            }
            unsigned long long it[SUN];
            uint32_t en[SUN];
#pragma unroll
            for (int u = 0; u < SUN; ++u) {
                it[u] = src[u] >= 0 ? cb.items[src[u]] : 0ull;
                en[u] = src[u] >= 0 ? cb.enc[src[u]] : 0u;
            }
#pragma unroll
            for (int u = 0; u < SUN; ++u) {
                if (src[u] < 0) continue;
                const uint32_t sy = (uint32_t)(it[u] & 0xFFFF);
                if (direct) s_pool[s_dofs[cx[u]] + sy - s_lo[cx[u]]] = en[u];
                else { s_sym[j0 + 256u * u] = (uint16_t)sy; s_enc[j0 + 256u * u] = en[u]; }
            }
        }
    }
    __syncthreads();

    // the code of one element
    auto finish = [&](uint32_t lcv, uint32_t c, uint32_t sym) -> uint32_t {
        bool raw = false;
        if (lcv == 0) {                   // not in the codebook: the ESC code, then the raw 16 bits ...
            lcv = s_esc[c];
            raw = (sym != s_escsym[c]);   // ... unless the symbol is the synthetic ESC symbol itself
        }
        return lcv != 0 ? (lcv | (raw ? 0x80000000u : 0u)) : kNoCode;
    };
    auto lookup = [&](uint32_t c, uint32_t sym) -> uint32_t {
        const int32_t gd = s_gid[c];
        if (gd < 0) return kNoCode;
        if (direct) {
            const uint32_t d = sym - s_lo[c], at = s_dofs[c];
            if (d >= s_dofs[c + 1] - at) return kNoCode;
            const uint32_t lcv = s_pool[at + d];
            return lcv == kNoCode ? kNoCode : finish(lcv, c, sym);
        }
        if (staged) {
            int lo = (int)s_ofs[c], hi = (int)s_ofs[c + 1] - 1;
            while (lo <= hi) {
                const int mid = (lo + hi) >> 1;
                const uint32_t x = s_sym[mid];
                if (x == sym) return finish(s_enc[mid], c, sym);
                if (x < sym) lo = mid + 1; else hi = mid - 1;
            }
            return kNoCode;
        }
        uint32_t code = 0; int len = 0; bool raw = false;
        if (element_code(cb, gd, sym, code, len, raw) < 0) return kNoCode;
        return ((uint32_t)len << 16) | code | (raw ? 0x80000000u : 0u);
    };
    uint32_t* out = lc + ebase[b];
    constexpr int UN = 4;   // elements in flight per thread: their loads are issued before any is looked up
    for (unsigned long long slab = blockIdx.y; slab < nslab; slab += gridDim.y) {
        const unsigned long long e_end = (slab + 1) * kCodeSlab < total ? (slab + 1) * kCodeSlab : total;
        unsigned long long e = slab * kCodeSlab + tid;
        unsigned long long rr = e / col_len, cc = e - rr * col_len;   // one division per slab, then a running (row, column)
        for (; e < e_end; e += 256 * UN) {
            uint32_t c[UN], sy[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                while (cc >= col_len) { cc -= col_len; ++rr; }
                if (e + 256ull * u < e_end) {
                    const long long i = (long long)g.rows[row_a + rr] * g.m + (g.group_col ? g.group_col[row_a + rr] : col_start) + (long long)cc;
                    c[u] = g.ctx[i] & g.ctx_mask;
                    sy[u] = g.sym[i];
                }
                cc += 256;
            }
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (e + 256ull * u < e_end) out[e + 256ull * u] = lookup(c[u], sy[u]);
        }
    }
}

// One thread per sub-stream walks its elements t, t + k_eff, ...: the size of the sub-stream in bits,
// or (EMIT) its bits written MSB-first, whole words with one 64-bit atomic OR each.
template <bool EMIT>
__global__ void rect_walk_kernel(RectGeom g, const unsigned long long* __restrict__ ebase, const uint32_t* __restrict__ lc,
                                 const uint32_t* __restrict__ startbit, const long long* __restrict__ bit_base,
                                 uint32_t* __restrict__ bits_out, unsigned long long* __restrict__ bitstream, int* __restrict__ err) {
    const long long total_threads = g.B * g.k;
    for (long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x; id < total_threads; id += (long long)gridDim.x * blockDim.x) {
        const long long b = id / g.k;
        const int t = (int)(id - b * g.k);
        const int row_a = g.row_ofs[b];
        const long long nrows = g.row_ofs[b + 1] - row_a;
        const long long col_len = g.group_col ? g.group_size : g.col_len[b];
        const long long col_start = g.group_col ? 0 : g.col_start[b];
        const long long total = nrows * col_len;
        long long k_eff = total < 1 ? 1 : total;
        if (k_eff > g.k) k_eff = g.k;
        if (t >= k_eff) { if (!EMIT) bits_out[id] = 0; continue; }
        const uint32_t* codes = lc + ebase[b];
        long long w = 0; int fill = 0; unsigned long long acc = 0;   // output cursor (emit)
        if (EMIT) {
            const long long bitpos = bit_base[b] + (long long)startbit[b * ((long long)g.k + 1) + t];
            w = bitpos >> 6; fill = (int)(bitpos & 63);
        }
        unsigned long long bits = 0;
        constexpr int UN = 4;   // codes loaded ahead of their use
        bool bad = false;
        for (long long e0 = t; e0 < total && !bad; e0 += UN * k_eff) {
          uint32_t ahead[UN];
#pragma unroll
          for (int u = 0; u < UN; ++u) ahead[u] = (e0 + u * k_eff < total) ? codes[e0 + u * k_eff] : 0u;
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const long long e = e0 + u * k_eff;
            if (e >= total) break;
            const uint32_t v = ahead[u];
            if (v == kNoCode) { atomicExch(err, 3); bad = true; break; }
            const bool raw = (v >> 31) != 0;
            const int nb = (int)((v >> 16) & 0x7FFFu) + (raw ? 16 : 0);
            bits += (unsigned long long)nb;
            if (EMIT) {
                // the code, then (after an ESC) the 16 raw bits, MSB first
                unsigned long long val = v & 0xFFFFu;
                if (raw) {
                    const long long rr = e / col_len, cc = e - rr * col_len;
                    const long long i = (long long)g.rows[row_a + rr] * g.m + (g.group_col ? g.group_col[row_a + rr] : col_start) + cc;
                    val = (val << 16) | g.sym[i];
                }
                int left = nb;
                while (left > 0) {
                    const int room = 64 - fill;
                    const int take = left < room ? left : room;
                    const unsigned long long part = (val >> (left - take)) & ((take >= 64) ? ~0ull : ((1ull << take) - 1ull));
                    acc |= part << (room - take);
                    fill += take; left -= take;
                    if (fill == 64) { atomicOr(&bitstream[w], acc); ++w; acc = 0; fill = 0; }
                }
            }
          }
        }
        if (EMIT) { if (acc) atomicOr(&bitstream[w], acc); }
        else bits_out[id] = (uint32_t)bits;
    }
}

// per bucket: start bit of every sub-stream relative to the bucket (build_huffman.cu:869-879)
__global__ void rect_starts_kernel(const uint32_t* __restrict__ bits, const int32_t* __restrict__ row_ofs,
                                   const int32_t* __restrict__ col_len, int group_size, long long B, int k,
                                   uint32_t* __restrict__ startbit, unsigned long long* __restrict__ bucket_bits) {
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < B; b += (long long)gridDim.x * blockDim.x) {
        const long long total = (long long)(row_ofs[b + 1] - row_ofs[b]) * (col_len ? col_len[b] : group_size);
        long long k_eff = total < 1 ? 1 : total;
        if (k_eff > k) k_eff = k;
        uint32_t* st = startbit + b * ((long long)k + 1);
        unsigned long long rel = 0;
        st[0] = 0;
        for (long long t = 0; t < k_eff; ++t) { rel += bits[b * k + t]; st[t + 1] = (uint32_t)rel; }
        for (long long t = k_eff + 1; t <= k; ++t) st[t] = st[k_eff];
        bucket_bits[b] = rel;
    }
}

// 64-bit aligned start of every bucket, [B] = end of the stream (build_huffman.cu:811-817, 918)
__global__ void bucket_bases_kernel(const unsigned long long* __restrict__ bucket_bits, long long B,
                                    long long* __restrict__ bit_base) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    long long pos = 0;
    for (long long b = 0; b < B; ++b) {
        if (pos & 63) pos = (pos + 63) & ~63LL;
        bit_base[b] = pos;
        pos += (long long)bucket_bits[b];
    }
    bit_base[B] = pos;
}

__global__ void table_keys_kernel(const uint32_t* __restrict__ ctx_key, long long G, uint16_t* __restrict__ tscale,
                                  uint16_t* __restrict__ tctx) {
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < G; g += (long long)gridDim.x * blockDim.x) {
        tscale[g] = (uint16_t)(ctx_key[g] >> 16);
        tctx[g] = (uint16_t)(ctx_key[g] & 0xFFFF);
    }
}

// ------------------------------------------------------------------------------------------------
// shared-table layout (build_huffman.cu:2157-2633): one stream per (scale id, context), present or
// not; one bitstream per scale holding its elements in flat order; chunks of at most 255 consecutive
// elements of one stream
// ------------------------------------------------------------------------------------------------
__global__ void shared_rows_kernel(const uint32_t* __restrict__ ctx_key, long long G, const int32_t* __restrict__ sid_lut,
                                   int* __restrict__ row_of, int* __restrict__ stream_ctx) {
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < G; g += (long long)gridDim.x * blockDim.x) {
        const uint32_t key = ctx_key[g];
        const int sid = sid_lut[key >> 16];
        const int row = sid * 16 + (int)(key & 0xFu);
        row_of[g] = row;
        stream_ctx[row] = (int)g;
    }
}

// per element: its stream, its code (len << 16 | code, bit 31: 16 raw bits follow) and its bit count
__global__ void shared_elem_kernel(const uint16_t* __restrict__ sym, const uint8_t* __restrict__ q,
                                   const uint16_t* __restrict__ scales, int scale_mode, long long m, long long nb1,
                                   long long sb0, long long sb1, const int32_t* __restrict__ sid_lut,
                                   const int* __restrict__ stream_ctx, CodeBook cb, long long numel,
                                   int* __restrict__ stream, uint32_t* __restrict__ lc, int* __restrict__ nbits,
                                   int* __restrict__ run_head, int* __restrict__ err) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x) {
        auto stream_at = [&](long long e) -> int {
            uint16_t sc;
            if (scale_mode == 0) sc = scales[0];
            else {
                const long long r = e / m, c = e - r * m;
                sc = (scale_mode == 1) ? scales[r] : scales[(r / sb0) * nb1 + (c / sb1)];
            }
            return sid_lut[sc] * 16 + (int)(q[e] & 0xFu);
        };
        const int st = stream_at(i);
        stream[i] = st;
        run_head[i] = (i == 0 || stream_at(i - 1) != st) ? (int)i : 0;
        const int gid = stream_ctx[st];
        uint32_t code = 0; int len = 0; bool raw = false;
        const int nb = (gid >= 0) ? element_code(cb, gid, sym[i], code, len, raw) : -1;
        if (nb < 0) { atomicExch(err, 3); lc[i] = 0; nbits[i] = 0; continue; }
        lc[i] = ((uint32_t)len << 16) | code | (raw ? 0x80000000u : 0u);
        nbits[i] = nb;
    }
}

__global__ void shared_chunk_heads_kernel(const int* __restrict__ run_start, long long numel, int* __restrict__ chead) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x)
        chead[i] = ((i - run_start[i]) % 255 == 0) ? 1 : 0;
}

__global__ void shared_sid_keys_kernel(const int* __restrict__ stream, long long numel, int* __restrict__ key, int* __restrict__ val) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x)
        { key[i] = stream[i] >> 4; val[i] = (int)i; }
}

__global__ void gather_bits_kernel(const int* __restrict__ src, const int* __restrict__ idx, long long N,
                                   unsigned long long* __restrict__ dst) {   // 64-bit: the running sum passes 2^31 bits
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (long long)gridDim.x * blockDim.x)
        dst[i] = (unsigned long long)src[idx[i]];
}

// in scale-sorted order: where every scale's run starts and how many bits it holds
__global__ void shared_segments_kernel(const int* __restrict__ sid_sorted, const unsigned long long* __restrict__ nb_sorted,
                                       const unsigned long long* __restrict__ cum, long long numel,
                                       unsigned long long* __restrict__ seg_base, unsigned long long* __restrict__ seg_bits_end) {
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < numel; j += (long long)gridDim.x * blockDim.x) {
        const int sid = sid_sorted[j];
        if (j == 0 || sid_sorted[j - 1] != sid) seg_base[sid] = cum[j] - nb_sorted[j];
        if (j == numel - 1 || sid_sorted[j + 1] != sid) seg_bits_end[sid] = cum[j];
    }
}

__global__ void shared_relpos_kernel(const int* __restrict__ sid_sorted, const int* __restrict__ idx_sorted,
                                     const unsigned long long* __restrict__ nb_sorted, const unsigned long long* __restrict__ cum,
                                     const unsigned long long* __restrict__ seg_base, long long numel,
                                     uint32_t* __restrict__ rel) {
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < numel; j += (long long)gridDim.x * blockDim.x) {
        rel[idx_sorted[j]] = (uint32_t)(cum[j] - nb_sorted[j] - seg_base[sid_sorted[j]]);
    }
}

// scale_bit_base: every scale's bitstream starts on a 64-bit boundary (:2543-2560); res[0] = total bits
__global__ void shared_bases_kernel(const unsigned long long* __restrict__ seg_base, const unsigned long long* __restrict__ seg_end,
                                    long long S, long long* __restrict__ scale_bit_base, long long* __restrict__ res) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    long long total = 0;
    for (long long s = 0; s < S; ++s) {
        total = (total + 63) & ~63LL;
        scale_bit_base[s] = total;
        total += (long long)(seg_end[s] - seg_base[s]);
    }
    total = (total + 63) & ~63LL;
    scale_bit_base[S] = total;
    res[0] = total;
}

__global__ void shared_chunk_pos_kernel(const int* __restrict__ chead, const int* __restrict__ cidx, long long numel,
                                        long long C, int* __restrict__ cpos) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x) {
        if (chead[i]) cpos[cidx[i]] = (int)i;
        if (i == 0) cpos[C] = (int)numel;
    }
}

__global__ void shared_chunk_fill_kernel(const int* __restrict__ cpos, long long C, const int* __restrict__ stream,
                                         const uint32_t* __restrict__ rel, uint32_t* __restrict__ c_start,
                                         uint32_t* __restrict__ c_base, uint32_t* __restrict__ c_meta,
                                         int32_t* __restrict__ c_sid, int* __restrict__ c_stream) {
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < C; c += (long long)gridDim.x * blockDim.x) {
        const int i = cpos[c];
        const int st = stream[i];
        c_base[c] = (uint32_t)i;
        c_start[c] = rel[i];
        c_sid[c] = st >> 4;
        c_meta[c] = ((uint32_t)(cpos[c + 1] - i) << 8) | (uint32_t)(st & 15);
        c_stream[c] = st;
    }
}

__global__ void shared_emit_kernel(const uint16_t* __restrict__ sym, const int* __restrict__ stream,
                                   const uint32_t* __restrict__ lc, const uint32_t* __restrict__ rel,
                                   const long long* __restrict__ scale_bit_base, long long numel,
                                   unsigned long long* __restrict__ bitstream) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += (long long)gridDim.x * blockDim.x) {
        const uint32_t v = lc[i];
        const int len = (int)((v >> 16) & 0x7FFFu);
        const bool raw = (v >> 31) != 0;
        unsigned long long bits = v & 0xFFFFu;
        int nb = len;
        if (raw) { bits = (bits << 16) | sym[i]; nb += 16; }
        if (nb <= 0) continue;
        const long long pos = scale_bit_base[stream[i] >> 4] + (long long)rel[i];
        const long long w = pos >> 6;
        const int o = (int)(pos & 63);
        if (o + nb <= 64) atomicOr(&bitstream[w], bits << (64 - o - nb));
        else {
            const int second = o + nb - 64;
            atomicOr(&bitstream[w], bits >> second);
            atomicOr(&bitstream[w + 1], bits << (64 - second));
        }
    }
}

__global__ void shared_stream_ofs_kernel(const int* __restrict__ keys_sorted, long long C, long long num_streams,
                                         long long* __restrict__ ofs) {
    for (long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x; s <= num_streams; s += (long long)gridDim.x * blockDim.x) {
        long long lo = 0, hi = C;  // first chunk whose stream is >= s
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if (keys_sorted[mid] < s) lo = mid + 1; else hi = mid;
        }
        ofs[s] = lo;
    }
}

__global__ void iota_i32_kernel(int32_t* __restrict__ p, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        p[i] = (int32_t)i;
}

}  // namespace mps

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
using namespace mps;

namespace {

// device-wide primitives' temporary storage: the radix sort may want a full extra key buffer
static size_t cub_temp_bytes(int64_t numel) { return (64ull << 20) + (size_t)numel * 9; }
constexpr size_t kCodebookScratch = 160ull << 20;  // interleaved per-context arrays of the codebook pass

struct Carver {
    uint8_t* base; size_t off, cap;
    template <typename T> T* take(size_t count) {
        off = align_up(off);
        T* p = reinterpret_cast<T*>(base + off);
        off += count * sizeof(T);
        return p;
    }
    bool ok() const { return off <= cap; }
};

inline BuildState* state_of(mps_build_state* s) { return reinterpret_cast<BuildState*>(s); }

size_t codebook_slot_bytes(int L) {
    const size_t TS = 1ull << L, KEEP = 4 * (TS - 1);
    return TS * (8 + 2 + 4 + 1) + KEEP * 16 + (size_t)L * KEEP;
}

}  // namespace

extern "C" {

size_t mps_build_workspace_bytes(int64_t numel, int64_t substreams) {
    if (numel < 0) numel = 0;
    if (substreams < numel) substreams = numel;
    // (the last term: six 32-bit arrays over the (scale, context) segments, of which a tensor has at most
    // 256 per distinct scale and no more distinct scales than elements or 16-bit values)
    const size_t max_scales = (size_t)(numel < 65536 ? numel : 65536);
    return 256 + (size_t)numel * 34 + (size_t)numel * 40 + (size_t)substreams * 4 + cub_temp_bytes(numel) + kCodebookScratch +
           (4ull << 20) + (max_scales * 256 + 1) * 24;
}

int mps_build_analyze(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                      const uint16_t* scales_u16, int32_t scale_mode, int64_t nb1, int64_t sb0, int64_t sb1, int64_t n,
                      int64_t m, int32_t variant, int64_t max_len, void* workspace, size_t workspace_bytes, void* stream,
                      int64_t* num_tables_out, int64_t* num_items_out) {
    if (!state || !bf16_bits || !ctx_bytes || !scales_u16 || !workspace || !num_tables_out || !num_items_out) {
        set_error("mps_build_analyze: null argument");
        return MPS_ERR_INVALID;
    }
    if (n <= 0 || m <= 0) { set_error("bf16_params shape must be non-empty"); return MPS_ERR_INVALID; }
    if (variant < V_FP8 || variant > V_AWQ_SHARED) { set_error("unknown builder variant %d", variant); return MPS_ERR_INVALID; }
    if (max_len <= 0 || max_len > 15) { set_error("max_len must be in [1, 15]"); return MPS_ERR_INVALID; }
    if (scale_mode < 0 || scale_mode > 2 || (scale_mode == 2 && (nb1 <= 0 || sb0 <= 0 || sb1 <= 0))) {
        set_error("unsupported scales layout");
        return MPS_ERR_INVALID;
    }
    const int64_t numel = n * m;
    if (numel >= (1LL << 31)) { set_error("tensors of 2^31 elements or more are not supported by the builder"); return MPS_ERR_UNSUPPORTED; }
    if (workspace_bytes < mps_build_workspace_bytes(numel, numel)) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BuildState& S = *state_of(state);
    memset(&S, 0, sizeof(S));
    S.numel = numel; S.n = n; S.m = m; S.L = (int32_t)max_len; S.variant = variant;
    S.group_size = (int32_t)((scale_mode == 2) ? sb1 : m);
    S.ws = static_cast<uint8_t*>(workspace); S.ws_bytes = workspace_bytes;
    Carver C{S.ws, 256, workspace_bytes};
    S.d_flag = reinterpret_cast<int32_t*>(S.ws);
    auto* items = C.take<unsigned long long>(numel);  S.o_items = (uint8_t*)items - S.ws;
    auto* counts = C.take<int>(numel);                S.o_counts = (uint8_t*)counts - S.ws;
    auto* ctx_ofs = C.take<int>(numel + 1);           S.o_ctx_ofs = (uint8_t*)ctx_ofs - S.ws;
    auto* ctx_key = C.take<uint32_t>(numel);          S.o_ctx_key = (uint8_t*)ctx_key - S.ws;
    auto* perm = C.take<int>(numel);                  S.o_perm = (uint8_t*)perm - S.ws;
    auto* enc = C.take<uint32_t>(numel);              S.o_enc = (uint8_t*)enc - S.ws;
    auto* esc = C.take<uint32_t>(numel);              S.o_esc = (uint8_t*)esc - S.ws;
    auto* escsym = C.take<uint16_t>(numel);           S.o_escsym = (uint8_t*)escsym - S.ws;
    C.off = align_up(C.off);
    S.o_scratch = C.off; S.scratch_bytes = workspace_bytes - C.off;
    // ---- scratch of the histogram ------------------------------------------------------------------
    MPS_CUDA_TRY(cudaMemsetAsync(S.d_flag, 0, 256, st));
    hist::Geom g;
    g.n = n; g.m = m; g.scale_mode = scale_mode;
    g.ctx_mask = (variant == V_FP8) ? 0xFFu : 0x0Fu;
    g.nctx = (variant == V_FP8) ? 256 : 16;
    if (scale_mode == 2) {
        if (nb1 * sb1 < m) { set_error("unsupported scales layout"); return MPS_ERR_INVALID; }
        g.ub0 = sb0; g.ub1 = sb1; g.nbu1 = nb1; g.nbu0 = (n + sb0 - 1) / sb0;
    } else {  // pieces of rows
        g.ub0 = 1; g.ub1 = (m <= 8192) ? m : 4096; g.nbu1 = (m + g.ub1 - 1) / g.ub1; g.nbu0 = n;
    }
    const long long units = g.nbu0 * g.nbu1;
    const size_t kCubTempBytes = cub_temp_bytes(numel);
    void* cub_tmp = C.take<uint8_t>(kCubTempBytes);
    auto* per_scale = C.take<uint32_t>(hist::kScaleValues + 1);   // units of every scale value
    auto* unit_ofs = C.take<uint32_t>(hist::kScaleValues + 1);
    auto* rank = C.take<uint32_t>(hist::kScaleValues + 1);        // flags, then ranks; [65536] = number of distinct scales
    auto* unit_cur = C.take<uint32_t>(hist::kScaleValues);
    auto* scale_of_rank = C.take<uint16_t>(hist::kScaleValues);
    auto* unit_sorted = C.take<uint32_t>(units);
    auto* seg_syms = C.take<uint16_t>(numel);
    auto* st_sym = C.take<uint16_t>(numel);
    auto* st_cnt = C.take<uint32_t>(numel);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    size_t need = 0;

    // scales: rank of every distinct value, units listed by scale
    MPS_CUDA_TRY(cudaMemsetAsync(per_scale, 0, (hist::kScaleValues + 1) * sizeof(uint32_t), st));
    hist::unit_scale_count_kernel<<<grid_for(units), 256, 0, st>>>(g, scales_u16, units, per_scale);
    hist::scale_flags_kernel<<<hist::kScaleValues / 256, 256, 0, st>>>(per_scale, rank);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, per_scale, unit_ofs, hist::kScaleValues + 1, st));
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, rank, rank, hist::kScaleValues + 1, st));
    hist::scale_ranks_kernel<<<hist::kScaleValues / 256, 256, 0, st>>>(per_scale, rank, unit_ofs, scale_of_rank, unit_cur);
    hist::unit_scatter_kernel<<<grid_for(units), 256, 0, st>>>(g, scales_u16, units, unit_cur, unit_sorted);
    uint32_t num_scales = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&num_scales, rank + hist::kScaleValues, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    const long long nseg = (long long)num_scales * g.nctx;

    // segments (scale rank, context): sizes, offsets, symbols
    auto* seg_cnt = C.take<uint32_t>(nseg + 1);
    auto* seg_ofs = C.take<uint32_t>(nseg + 1);
    auto* seg_cur = C.take<uint32_t>(nseg + 1);      // write cursors, later distinct symbols per segment, then item offsets
    auto* chunk_ofs = C.take<uint32_t>(nseg + 1);    // chunks per segment, then their prefix
    auto* split_id = C.take<uint32_t>(nseg + 1);     // split flags, then their prefix
    auto* ctx_id = C.take<uint32_t>(nseg + 1);       // non-empty flags, then their prefix: the context index
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    long long upw = hist::kWarpElems / (g.ub0 * g.ub1);
    if (upw < 1) upw = 1;
    const long long walk_warps = (units + upw - 1) / upw;
    const unsigned walk_grid = (unsigned)((walk_warps + hist::kWalkWarps - 1) / hist::kWalkWarps);
    MPS_CUDA_TRY(cudaMemsetAsync(seg_cnt, 0, (nseg + 1) * sizeof(uint32_t), st));
    hist::segment_walk_kernel<false><<<walk_grid, hist::kWalkWarps * 32, 0, st>>>(g, bf16_bits, ctx_bytes, scales_u16, rank, unit_sorted,
                                                                                  units, upw, seg_cnt, nullptr);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, seg_cnt, seg_ofs, (int)(nseg + 1), st));
    MPS_CUDA_TRY(cudaMemcpyAsync(seg_cur, seg_ofs, (nseg + 1) * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
    hist::segment_walk_kernel<true><<<walk_grid, hist::kWalkWarps * 32, 0, st>>>(g, bf16_bits, ctx_bytes, scales_u16, rank, unit_sorted,
                                                                                 units, upw, seg_cur, seg_syms);
    hist::chunk_plan_kernel<<<grid_for(nseg + 1), 256, 0, st>>>(seg_cnt, nseg, chunk_ofs, split_id, ctx_id);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, chunk_ofs, chunk_ofs, (int)(nseg + 1), st));
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, split_id, split_id, (int)(nseg + 1), st));
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, ctx_id, ctx_id, (int)(nseg + 1), st));
    uint32_t totals[3] = {0, 0, 0};  // chunks, split segments, contexts
    MPS_CUDA_TRY(cudaMemcpyAsync(&totals[0], chunk_ofs + nseg, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&totals[1], split_id + nseg, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&totals[2], ctx_id + nseg, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    const long long num_chunks = totals[0], num_split = totals[1];
    const int G = (int)totals[2];

    // symbols of every segment counted by value
    auto* chunk_seg = C.take<uint32_t>(num_chunks);
    auto* split_seg = C.take<uint32_t>(num_split);
    auto* dense = C.take<uint32_t>((size_t)num_split * 65536u);
    auto* split_range = C.take<uint32_t>((size_t)num_split * 2);     // smallest, largest symbol of every split segment
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    hist::chunk_fill_kernel<<<grid_for(nseg), 256, 0, st>>>(seg_cnt, nseg, chunk_ofs, split_id, chunk_seg, split_seg);
    if (num_split) {
        MPS_CUDA_TRY(cudaMemsetAsync(dense, 0, (size_t)num_split * 65536u * sizeof(uint32_t), st));
        hist::split_range_init_kernel<<<grid_for(num_split), 256, 0, st>>>(split_range, num_split);
    }
    MPS_CUDA_TRY(cudaMemsetAsync(seg_cur, 0, (nseg + 1) * sizeof(uint32_t), st));
    if (num_chunks)
        hist::chunk_count_kernel<<<(unsigned)num_chunks, 256, 0, st>>>(seg_syms, seg_cnt, seg_ofs, chunk_seg, chunk_ofs, split_id, dense,
                                                                       split_range, st_sym, st_cnt, seg_cur);
    if (num_split) hist::split_finish_kernel<<<(unsigned)num_split, 256, 0, st>>>(split_seg, seg_ofs, dense, split_range, st_sym, st_cnt, seg_cur);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, seg_cur, seg_cur, (int)(nseg + 1), st));
    hist::gather_items_kernel<<<grid_for(nseg * 32), 256, 0, st>>>(seg_cnt, seg_ofs, seg_cur, ctx_id, nseg, g.nctx, scale_of_rank, st_sym,
                                                                   st_cnt, items, counts, ctx_ofs, ctx_key);
    uint32_t n_items = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&n_items, seg_cur + nseg, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaGetLastError());
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    const long long N = n_items;
    S.N = N;

    // ---- scratch of the per-context ordering (the histogram's is no longer needed) ---------------------
    C.off = S.o_scratch;
    auto* k1 = C.take<unsigned long long>(N);
    auto* k1o = C.take<unsigned long long>(N);
    auto* v = C.take<int>(N);
    auto* vo = C.take<int>(N);
    auto* ci = C.take<uint32_t>(N);
    auto* cio = C.take<uint32_t>(N);
    cub_tmp = C.take<uint8_t>(kCubTempBytes);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    // items of every context ordered by (count, symbol): sort by that key, then stably by context
    item_sort_keys_kernel<<<grid_for(N), 256, 0, st>>>(items, counts, ctx_ofs, G, N, k1, v, ci);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceRadixSort::SortPairs(cub_tmp, need, k1, k1o, v, vo, (int)N, 0, 48, st));
    gather_u32_kernel<<<grid_for(N), 256, 0, st>>>(ci, vo, N, cio);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceRadixSort::SortPairs(cub_tmp, need, cio, ci, vo, perm, (int)N, 0, 32, st));
    MPS_CUDA_TRY(cudaGetLastError());
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    S.G = G;
    *num_tables_out = G;
    *num_items_out = N;
    return MPS_OK;
}

int mps_build_codebooks(mps_build_state* state, uint16_t* decode_syms_u16, uint8_t* decode_lens_u8,
                        uint16_t* table_scale_u16, uint16_t* table_ctx_u16, void* stream) {
    if (!state || !decode_syms_u16 || !decode_lens_u8 || !table_scale_u16 || !table_ctx_u16) {
        set_error("mps_build_codebooks: null argument");
        return MPS_ERR_INVALID;
    }
    BuildState& S = *state_of(state);
    if (S.variant == V_AWQ_SHARED) { set_error("shared-table sidecars use mps_build_shared_codebooks"); return MPS_ERR_INVALID; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int L = S.L;
    const size_t TS = 1ull << L, KEEP = 4 * (TS - 1);
    const size_t slot = codebook_slot_bytes(L);
    long long chunk = (long long)((kCodebookScratch - (1 << 16)) / slot);
    if (chunk > S.G) chunk = S.G;
    if (chunk < 1) { set_error("codebook scratch too small for max_len=%d", L); return MPS_ERR_WORKSPACE; }
    chunk = (chunk / 32) * 32 > 0 ? (chunk / 32) * 32 : chunk;
    Carver C{S.ws, S.o_scratch, S.ws_bytes};
    CbScratch cs;
    cs.chunk = (int)chunk;
    cs.w = C.take<unsigned long long>(TS * chunk);
    cs.cur = C.take<unsigned long long>(KEEP * chunk);
    cs.nxt = C.take<unsigned long long>(KEEP * chunk);
    cs.src = C.take<int>(TS * chunk);
    cs.sym = C.take<uint16_t>(TS * chunk);
    cs.flag = C.take<uint8_t>((size_t)L * KEEP * chunk);
    cs.len = C.take<uint8_t>(TS * chunk);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    auto* items = reinterpret_cast<unsigned long long*>(S.ws + S.o_items);
    auto* counts = reinterpret_cast<int*>(S.ws + S.o_counts);
    auto* ctx_ofs = reinterpret_cast<int*>(S.ws + S.o_ctx_ofs);
    auto* ctx_key = reinterpret_cast<uint32_t*>(S.ws + S.o_ctx_key);
    auto* perm = reinterpret_cast<int*>(S.ws + S.o_perm);
    auto* enc = reinterpret_cast<uint32_t*>(S.ws + S.o_enc);
    auto* esc = reinterpret_cast<uint32_t*>(S.ws + S.o_esc);
    auto* escsym = reinterpret_cast<uint16_t*>(S.ws + S.o_escsym);
    MPS_CUDA_TRY(cudaMemsetAsync(decode_syms_u16, 0, (size_t)S.G * TS * 2, st));
    MPS_CUDA_TRY(cudaMemsetAsync(decode_lens_u8, 0, (size_t)S.G * TS / 2, st));
    for (long long g0 = 0; g0 < S.G; g0 += chunk) {
        const long long g1 = (g0 + chunk < S.G) ? g0 + chunk : S.G;
        codebook_kernel<<<(int)((g1 - g0 + 63) / 64), 64, 0, st>>>(items, counts, ctx_ofs, perm, g0, g1, L, S.variant, cs,
                                                                    decode_syms_u16, decode_lens_u8, enc, esc, escsym,
                                                                    S.d_flag, nullptr);
    }
    table_keys_kernel<<<grid_for(S.G), 256, 0, st>>>(ctx_key, S.G, table_scale_u16, table_ctx_u16);
    MPS_CUDA_TRY(cudaGetLastError());
    int flag = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&flag, S.d_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    if (flag == 2) { set_error("Internal error: not enough packages"); return (int)cudaErrorUnknown; }
    return MPS_OK;
}

int mps_build_bucket_table(mps_build_state* state, const uint16_t* bucket_scale_u16, int64_t num_buckets,
                           int32_t* bucket_table_i32, void* stream) {
    if (!state || !bucket_scale_u16 || !bucket_table_i32 || num_buckets < 0) { set_error("mps_build_bucket_table: bad argument"); return MPS_ERR_INVALID; }
    BuildState& S = *state_of(state);
    const int nctx = (S.variant == V_FP8) ? 256 : 16;
    auto* ctx_key = reinterpret_cast<uint32_t*>(S.ws + S.o_ctx_key);
    if (num_buckets == 0) return MPS_OK;
    bucket_table_kernel<<<grid_for(num_buckets * nctx), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ctx_key, (int)S.G, bucket_scale_u16, num_buckets, nctx, bucket_table_i32);
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

int mps_build_bucket_unique(const int32_t* bucket_table_i32, int64_t num_buckets, int32_t* bucket_U_i32,
                            int32_t* bucket_unique_gid_i32, int16_t* bucket_fp8_uidx_i16, void* stream) {
    if (!bucket_table_i32 || !bucket_U_i32 || !bucket_unique_gid_i32 || !bucket_fp8_uidx_i16 || num_buckets < 0) {
        set_error("mps_build_bucket_unique: bad argument");
        return MPS_ERR_INVALID;
    }
    if (num_buckets == 0) return MPS_OK;
    bucket_unique_kernel<<<grid_for((num_buckets + kUniqueWarps - 1) / kUniqueWarps, 1), kUniqueWarps * 32, 0,
                           static_cast<cudaStream_t>(stream)>>>(
        bucket_table_i32, num_buckets, bucket_U_i32, bucket_unique_gid_i32, bucket_fp8_uidx_i16);
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

static int rect_common(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                       const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                       const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                       const int32_t* row_indices_i32, int64_t num_buckets, int32_t k, RectGeom* g, CodeBook* cb) {
    if (!state || !bf16_bits || !ctx_bytes || !bucket_table_i32 || !bucket_col_start_i32 ||
        !bucket_row_offsets_i32 || !row_indices_i32 || num_buckets < 0 || k <= 0 || k > MPS_MAX_SUBSTREAMS) {
        set_error("sidecar layout: bad argument");
        return MPS_ERR_INVALID;
    }
    BuildState& S = *state_of(state);
    // ragged (by-scale) layout: bucket_col_len is null, bucket_col_start lists the column start of every
    // group, the row list holds the groups' rows and every group has S.group_size elements
    const bool ragged = (bucket_col_len_i32 == nullptr);
    if (ragged && S.group_size <= 0) { set_error("sidecar layout: group size not set"); return MPS_ERR_INVALID; }
    g->sym = bf16_bits; g->ctx = ctx_bytes; g->bucket_table = bucket_table_i32;
    g->col_start = ragged ? nullptr : bucket_col_start_i32; g->group_col = ragged ? bucket_col_start_i32 : nullptr;
    g->group_size = S.group_size;
    g->col_len = bucket_col_len_i32; g->row_ofs = bucket_row_offsets_i32; g->rows = row_indices_i32;
    g->B = num_buckets; g->m = S.m; g->k = k; g->nctx = (S.variant == V_FP8) ? 256 : 16;
    g->ctx_mask = (S.variant == V_FP8) ? 0xFFu : 0x0Fu;
    cb->items = reinterpret_cast<unsigned long long*>(S.ws + S.o_items);
    cb->ctx_ofs = reinterpret_cast<int*>(S.ws + S.o_ctx_ofs);
    cb->enc = reinterpret_cast<uint32_t*>(S.ws + S.o_enc);
    cb->esc = reinterpret_cast<uint32_t*>(S.ws + S.o_esc);
    cb->escsym = reinterpret_cast<uint16_t*>(S.ws + S.o_escsym);
    return MPS_OK;
}

int mps_build_rect_layout(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                          const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                          const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                          const int32_t* row_indices_i32, int64_t num_buckets, int32_t k,
                          uint32_t* bucket_thread_startbit_u32, int64_t* bucket_bit_base_i64, void* stream,
                          int64_t* total_bits_out) {
    RectGeom g; CodeBook cb;
    int rc = rect_common(state, bf16_bits, ctx_bytes, bucket_table_i32, bucket_col_start_i32, bucket_col_len_i32,
                         bucket_row_offsets_i32, row_indices_i32, num_buckets, k, &g, &cb);
    if (rc) return rc;
    if (!bucket_thread_startbit_u32 || !bucket_bit_base_i64 || !total_bits_out) { set_error("sidecar layout: null output"); return MPS_ERR_INVALID; }
    BuildState& S = *state_of(state);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Carver C{S.ws, S.o_scratch, S.ws_bytes};
    auto* codes = C.take<uint32_t>((size_t)S.numel);                      // kept for the emit call, with ...
    auto* ebase = C.take<unsigned long long>(num_buckets + 1);            // ... the buckets' offsets into it
    auto* bits = C.take<uint32_t>((size_t)num_buckets * k);
    auto* bucket_bits = C.take<unsigned long long>(num_buckets + 1);
    auto* totals = C.take<unsigned long long>(num_buckets + 1);
    const size_t kScanTemp = 1 << 20;
    void* scan_tmp = C.take<uint8_t>(kScanTemp);
    if (!C.ok()) { set_error("workspace too small for %lld buckets of %d sub-streams", (long long)num_buckets, k); return MPS_ERR_WORKSPACE; }
    S.o_rect_codes = (uint8_t*)codes - S.ws; S.o_rect_ebase = (uint8_t*)ebase - S.ws; S.rect_buckets = 0;
    if (num_buckets > 0) {
        bucket_totals_kernel<<<grid_for(num_buckets + 1), 256, 0, st>>>(g, totals);
        size_t need = 0;
        MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(nullptr, need, totals, ebase, (int)(num_buckets + 1), st));
        if (need > kScanTemp) { set_error("scan temporary storage exceeds the reserved %zu bytes", kScanTemp); return MPS_ERR_WORKSPACE; }
        need = kScanTemp;
        MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(scan_tmp, need, totals, ebase, (int)(num_buckets + 1), st));
        unsigned long long covered = 0;
        MPS_CUDA_TRY(cudaMemcpyAsync(&covered, ebase + num_buckets, sizeof(covered), cudaMemcpyDeviceToHost, st));
        MPS_CUDA_TRY(cudaStreamSynchronize(st));
        if (covered > (unsigned long long)S.numel) { set_error("the buckets hold more elements than the tensor has"); return MPS_ERR_INVALID; }
        // buckets of a weight are few and large, buckets of a grouped tensor many and small: as many CTAs
        // share a bucket's slabs as it takes to fill the GPU once (every one of them stages the bucket's
        // codebooks), the spare ones of a small bucket leave at once
        long long share = (5LL * sm_count_host()) / num_buckets;   // about five CTAs of this kernel fit an SM
        const unsigned split = (unsigned)(share < 1 ? 1 : (share > 32 ? 32 : share));
        if (num_buckets > 0x7FFFFFFFLL) { set_error("too many buckets"); return MPS_ERR_INVALID; }
        rect_codes_kernel<<<dim3((unsigned)num_buckets, split), 256, 0, st>>>(g, cb, S.G, ebase, codes);
        S.rect_buckets = num_buckets;
        rect_walk_kernel<false><<<grid_for(num_buckets * k), 256, 0, st>>>(g, ebase, codes, nullptr, nullptr, bits, nullptr, S.d_flag);
        rect_starts_kernel<<<grid_for(num_buckets, 64), 64, 0, st>>>(bits, bucket_row_offsets_i32, g.group_col ? nullptr : bucket_col_len_i32,
                                                                     g.group_size, num_buckets, k, bucket_thread_startbit_u32, bucket_bits);
    }
    bucket_bases_kernel<<<1, 32, 0, st>>>(bucket_bits, num_buckets, reinterpret_cast<long long*>(bucket_bit_base_i64));
    MPS_CUDA_TRY(cudaGetLastError());
    long long total = 0; int flag = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&total, bucket_bit_base_i64 + num_buckets, sizeof(total), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&flag, S.d_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    if (flag == 3) { set_error("symbol not found and no ESC for (scale,ctx) key"); return (int)cudaErrorUnknown; }
    *total_bits_out = total;
    return MPS_OK;
}

int mps_build_rect_emit(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                        const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                        const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                        const int32_t* row_indices_i32, int64_t num_buckets, int32_t k,
                        const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                        uint64_t* bitstream_u64, int64_t bitstream_words, void* stream) {
    RectGeom g; CodeBook cb;
    int rc = rect_common(state, bf16_bits, ctx_bytes, bucket_table_i32, bucket_col_start_i32, bucket_col_len_i32,
                         bucket_row_offsets_i32, row_indices_i32, num_buckets, k, &g, &cb);
    if (rc) return rc;
    if (!bucket_thread_startbit_u32 || !bucket_bit_base_i64 || (bitstream_words > 0 && !bitstream_u64)) { set_error("sidecar emit: null argument"); return MPS_ERR_INVALID; }
    BuildState& S = *state_of(state);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (bitstream_words > 0) MPS_CUDA_TRY(cudaMemsetAsync(bitstream_u64, 0, (size_t)bitstream_words * 8, st));
    if (num_buckets > 0) {
        if (S.rect_buckets != num_buckets) { set_error("sidecar emit: call mps_build_rect_layout for the same buckets first"); return MPS_ERR_INVALID; }
        rect_walk_kernel<true><<<grid_for(num_buckets * k), 256, 0, st>>>(
            g, reinterpret_cast<const unsigned long long*>(S.ws + S.o_rect_ebase), reinterpret_cast<const uint32_t*>(S.ws + S.o_rect_codes),
            bucket_thread_startbit_u32, reinterpret_cast<const long long*>(bucket_bit_base_i64), nullptr,
            reinterpret_cast<unsigned long long*>(bitstream_u64), S.d_flag);
    }
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}

// ---- shared-table layout -----------------------------------------------------------------------

int mps_build_shared_codebooks(mps_build_state* state, const int32_t* sid_lut_i32, int64_t num_scales,
                               int16_t* decode_syms_i16, uint8_t* decode_nbits_u8, void* stream) {
    if (!state || !sid_lut_i32 || !decode_syms_i16 || !decode_nbits_u8 || num_scales <= 0) {
        set_error("mps_build_shared_codebooks: bad argument");
        return MPS_ERR_INVALID;
    }
    BuildState& S = *state_of(state);
    if (S.variant != V_AWQ_SHARED) { set_error("state was not analyzed for the shared-table layout"); return MPS_ERR_INVALID; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int L = S.L;
    const size_t TS = 1ull << L, KEEP = 4 * (TS - 1);
    const long long num_streams = num_scales * 16;
    S.num_scales = num_scales;
    Carver C{S.ws, S.o_scratch, S.ws_bytes};
    auto* row_of = C.take<int>(S.G);
    auto* stream_ctx = C.take<int>(num_streams);
    S.o_sh_keep = (uint8_t*)row_of - S.ws;
    S.o_sh_end = align_up(C.off);
    const size_t slot = codebook_slot_bytes(L);
    long long chunk = (long long)((kCodebookScratch - (1 << 16)) / slot);
    if (chunk > S.G) chunk = S.G;
    if (chunk < 1) { set_error("codebook scratch too small for max_len=%d", L); return MPS_ERR_WORKSPACE; }
    chunk = (chunk / 32) * 32 > 0 ? (chunk / 32) * 32 : chunk;
    CbScratch cs;
    cs.chunk = (int)chunk;
    cs.w = C.take<unsigned long long>(TS * chunk);
    cs.cur = C.take<unsigned long long>(KEEP * chunk);
    cs.nxt = C.take<unsigned long long>(KEEP * chunk);
    cs.src = C.take<int>(TS * chunk);
    cs.sym = C.take<uint16_t>(TS * chunk);
    cs.flag = C.take<uint8_t>((size_t)L * KEEP * chunk);
    cs.len = C.take<uint8_t>(TS * chunk);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    auto* items = reinterpret_cast<unsigned long long*>(S.ws + S.o_items);
    auto* counts = reinterpret_cast<int*>(S.ws + S.o_counts);
    auto* ctx_ofs = reinterpret_cast<int*>(S.ws + S.o_ctx_ofs);
    auto* ctx_key = reinterpret_cast<uint32_t*>(S.ws + S.o_ctx_key);
    auto* perm = reinterpret_cast<int*>(S.ws + S.o_perm);
    auto* enc = reinterpret_cast<uint32_t*>(S.ws + S.o_enc);
    auto* esc = reinterpret_cast<uint32_t*>(S.ws + S.o_esc);
    auto* escsym = reinterpret_cast<uint16_t*>(S.ws + S.o_escsym);
    MPS_CUDA_TRY(cudaMemsetAsync(decode_syms_i16, 0, (size_t)num_streams * TS * 2, st));
    MPS_CUDA_TRY(cudaMemsetAsync(decode_nbits_u8, 0, (size_t)num_streams * TS, st));
    MPS_CUDA_TRY(cudaMemsetAsync(stream_ctx, 0xFF, (size_t)num_streams * sizeof(int), st));
    shared_rows_kernel<<<grid_for(S.G), 256, 0, st>>>(ctx_key, S.G, sid_lut_i32, row_of, stream_ctx);
    for (long long g0 = 0; g0 < S.G; g0 += chunk) {
        const long long g1 = (g0 + chunk < S.G) ? g0 + chunk : S.G;
        codebook_kernel<<<(int)((g1 - g0 + 63) / 64), 64, 0, st>>>(items, counts, ctx_ofs, perm, g0, g1, L, S.variant, cs,
                                                                    reinterpret_cast<uint16_t*>(decode_syms_i16),
                                                                    decode_nbits_u8, enc, esc, escsym, S.d_flag, row_of);
    }
    MPS_CUDA_TRY(cudaGetLastError());
    int flag = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&flag, S.d_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    if (flag == 2) { set_error("Internal error: not enough packages"); return (int)cudaErrorUnknown; }
    return MPS_OK;
}

namespace {
struct SharedArrays {   // what the layout call leaves in the workspace for the emit call
    int* stream; uint32_t* lc; uint32_t* rel; int* chead; int* cidx;
};
SharedArrays shared_arrays(BuildState& S, Carver& C) {
    SharedArrays a;
    C.off = S.o_sh_end;
    a.stream = C.take<int>(S.numel);
    a.lc = C.take<uint32_t>(S.numel);
    a.rel = C.take<uint32_t>(S.numel);
    a.chead = C.take<int>(S.numel);
    a.cidx = C.take<int>(S.numel);
    return a;
}
}  // namespace

int mps_build_shared_layout(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* int4_u8,
                            const uint16_t* scales_u16, int32_t scale_mode, int64_t nb1, int64_t sb0, int64_t sb1,
                            const int32_t* sid_lut_i32, int64_t* scale_bit_base_i64, void* stream,
                            int64_t* num_chunks_out, int64_t* total_bits_out) {
    if (!state || !bf16_bits || !int4_u8 || !scales_u16 || !sid_lut_i32 || !scale_bit_base_i64 || !num_chunks_out ||
        !total_bits_out) {
        set_error("mps_build_shared_layout: null argument");
        return MPS_ERR_INVALID;
    }
    BuildState& S = *state_of(state);
    if (S.variant != V_AWQ_SHARED || S.num_scales <= 0) { set_error("call mps_build_shared_codebooks first"); return MPS_ERR_INVALID; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long numel = S.numel, NS = S.num_scales;
    Carver C{S.ws, 0, S.ws_bytes};
    SharedArrays A = shared_arrays(S, C);
    // scratch of this call
    auto* nbits = C.take<int>(numel);
    auto* tmp_a = C.take<int>(numel);      // run heads, then sorted scale ids
    auto* tmp_b = C.take<int>(numel);      // run starts, then sorted element ids
    auto* key = C.take<int>(numel);
    auto* val = C.take<int>(numel);
    auto* nb_sorted = C.take<unsigned long long>(numel);
    auto* cum = C.take<unsigned long long>(numel);
    auto* seg_base = C.take<unsigned long long>(NS);
    auto* seg_end = C.take<unsigned long long>(NS);
    auto* d_res = C.take<long long>(4);
    const size_t kCubTempBytes = cub_temp_bytes(numel);
    void* cub_tmp = C.take<uint8_t>(kCubTempBytes);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    // kept by mps_build_shared_codebooks: row_of [G], then stream_ctx [num_streams]
    auto* stream_ctx = reinterpret_cast<int*>(S.ws + align_up(S.o_sh_keep + (size_t)S.G * sizeof(int)));
    CodeBook cb{reinterpret_cast<unsigned long long*>(S.ws + S.o_items), reinterpret_cast<int*>(S.ws + S.o_ctx_ofs),
                reinterpret_cast<uint32_t*>(S.ws + S.o_enc), reinterpret_cast<uint32_t*>(S.ws + S.o_esc),
                reinterpret_cast<uint16_t*>(S.ws + S.o_escsym)};
    shared_elem_kernel<<<grid_for(numel), 256, 0, st>>>(bf16_bits, int4_u8, scales_u16, scale_mode, S.m, nb1, sb0, sb1,
                                                        sid_lut_i32, stream_ctx, cb, numel, A.stream, A.lc, nbits, tmp_a,
                                                        S.d_flag);
    MPS_CUDA_TRY(cudaGetLastError());
    size_t need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::InclusiveScan(cub_tmp, need, tmp_a, tmp_b, cub::Max(), (int)numel, st));
    shared_chunk_heads_kernel<<<grid_for(numel), 256, 0, st>>>(tmp_b, numel, A.chead);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(cub_tmp, need, A.chead, A.cidx, (int)numel, st));
    // every scale's elements in flat order: stable sort by scale id
    shared_sid_keys_kernel<<<grid_for(numel), 256, 0, st>>>(A.stream, numel, key, val);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceRadixSort::SortPairs(cub_tmp, need, key, tmp_a, val, tmp_b, (int)numel, 0, 16, st));
    gather_bits_kernel<<<grid_for(numel), 256, 0, st>>>(nbits, tmp_b, numel, nb_sorted);
    need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceScan::InclusiveSum(cub_tmp, need, nb_sorted, cum, (int)numel, st));
    MPS_CUDA_TRY(cudaMemsetAsync(seg_base, 0, (size_t)NS * 8, st));
    MPS_CUDA_TRY(cudaMemsetAsync(seg_end, 0, (size_t)NS * 8, st));
    shared_segments_kernel<<<grid_for(numel), 256, 0, st>>>(tmp_a, nb_sorted, cum, numel, seg_base, seg_end);
    shared_relpos_kernel<<<grid_for(numel), 256, 0, st>>>(tmp_a, tmp_b, nb_sorted, cum, seg_base, numel, A.rel);
    shared_bases_kernel<<<1, 32, 0, st>>>(seg_base, seg_end, NS, reinterpret_cast<long long*>(scale_bit_base_i64), d_res);
    MPS_CUDA_TRY(cudaGetLastError());
    long long total_bits = 0;
    int last_head = 0, last_idx = 0, flag = 0;
    MPS_CUDA_TRY(cudaMemcpyAsync(&total_bits, d_res, sizeof(long long), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&last_head, A.chead + (numel - 1), sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&last_idx, A.cidx + (numel - 1), sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaMemcpyAsync(&flag, S.d_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    if (flag == 3) { set_error("symbol not found in enc table for AWQ stream"); return (int)cudaErrorUnknown; }
    S.num_chunks = (long long)last_idx + last_head;
    *num_chunks_out = S.num_chunks;
    *total_bits_out = total_bits;
    return MPS_OK;
}

int mps_build_shared_emit(mps_build_state* state, const uint16_t* bf16_bits, const int64_t* scale_bit_base_i64,
                          uint64_t* bitstream_u64, int64_t bitstream_words, uint32_t* chunk_startbit_rel_u32,
                          uint32_t* chunk_out_base_u32, uint32_t* chunk_meta_u32, int32_t* chunk_scale_id_i32,
                          int32_t* out_idx_i32, int64_t* stream_chunk_ofs_i64, int32_t* stream_chunk_ids_i32, void* stream) {
    if (!state || !bf16_bits || !scale_bit_base_i64 || !bitstream_u64 || !chunk_startbit_rel_u32 || !chunk_out_base_u32 ||
        !chunk_meta_u32 || !chunk_scale_id_i32 || !out_idx_i32 || !stream_chunk_ofs_i64 || !stream_chunk_ids_i32) {
        set_error("mps_build_shared_emit: null argument (state %d, inputs %d%d, bitstream %d, chunks %d%d%d%d, out_idx %d, csr %d%d)",
                  state != nullptr, bf16_bits != nullptr, scale_bit_base_i64 != nullptr, bitstream_u64 != nullptr,
                  chunk_startbit_rel_u32 != nullptr, chunk_out_base_u32 != nullptr, chunk_meta_u32 != nullptr,
                  chunk_scale_id_i32 != nullptr, out_idx_i32 != nullptr, stream_chunk_ofs_i64 != nullptr,
                  stream_chunk_ids_i32 != nullptr);
        return MPS_ERR_INVALID;
    }
    BuildState& S = *state_of(state);
    if (S.variant != V_AWQ_SHARED || S.num_chunks <= 0) { set_error("call mps_build_shared_layout first"); return MPS_ERR_INVALID; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long numel = S.numel, NC = S.num_chunks, num_streams = S.num_scales * 16;
    Carver C{S.ws, 0, S.ws_bytes};
    SharedArrays A = shared_arrays(S, C);
    auto* cpos = C.take<int>(NC + 1);
    auto* c_stream = C.take<int>(NC);
    auto* c_stream_sorted = C.take<int>(NC);
    auto* c_ids = C.take<int>(NC);
    const size_t kCubTempBytes = cub_temp_bytes(numel);
    void* cub_tmp = C.take<uint8_t>(kCubTempBytes);
    if (!C.ok()) { set_error("workspace too small"); return MPS_ERR_WORKSPACE; }
    shared_chunk_pos_kernel<<<grid_for(numel), 256, 0, st>>>(A.chead, A.cidx, numel, NC, cpos);
    shared_chunk_fill_kernel<<<grid_for(NC), 256, 0, st>>>(cpos, NC, A.stream, A.rel, chunk_startbit_rel_u32, chunk_out_base_u32,
                                                           chunk_meta_u32, chunk_scale_id_i32, c_stream);
    MPS_CUDA_TRY(cudaMemsetAsync(bitstream_u64, 0, (size_t)bitstream_words * 8, st));
    shared_emit_kernel<<<grid_for(numel), 256, 0, st>>>(bf16_bits, A.stream, A.lc, A.rel,
                                                        reinterpret_cast<const long long*>(scale_bit_base_i64), numel,
                                                        reinterpret_cast<unsigned long long*>(bitstream_u64));
    // chunk ids of every stream, ascending (stable sort by stream id) and the CSR offsets
    iota_i32_kernel<<<grid_for(NC), 256, 0, st>>>(c_ids, NC);
    size_t need = kCubTempBytes;
    MPS_CUDA_TRY(cub::DeviceRadixSort::SortPairs(cub_tmp, need, c_stream, c_stream_sorted, c_ids, stream_chunk_ids_i32, (int)NC,
                                                 0, 21, st));
    shared_stream_ofs_kernel<<<grid_for(num_streams + 1), 256, 0, st>>>(c_stream_sorted, NC, num_streams,
                                                                        reinterpret_cast<long long*>(stream_chunk_ofs_i64));
    iota_i32_kernel<<<grid_for(numel), 256, 0, st>>>(out_idx_i32, numel);
    MPS_CUDA_TRY(cudaGetLastError());
    MPS_CUDA_TRY(cudaStreamSynchronize(st));
    return MPS_OK;
}


}  // extern "C"
