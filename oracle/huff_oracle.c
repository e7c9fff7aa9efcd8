/*
 * huff_oracle.c -- CPU restatement of the MPServe context-conditioned Huffman codec.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the tests, the
 * smoke entry and the CPU-baseline leg of the benchmark may call it; no product code path does.
 *
 * It restates, in plain C and with different data structures (sort-based histograms, prefix
 * counting instead of package trees, sorted arrays instead of hash maps), the algorithms of the
 * reference so that, on the same inputs, every produced artifact is byte-identical:
 *
 *   encoders   kernel/build_huffman.cu:292-969    (FP8, per (scale,fp8) context, L=7 decode)
 *              kernel/build_huffman.cu:1582-2126  (AWQ int4 rectangular buckets)
 *              kernel/build_huffman.cu:1074-1580  (AWQ int4 ragged buckets, by exact scale)
 *              kernel/build_huffman.cu:2157-2633  (AWQ shared-table / chunked)
 *   helpers    kernel/build_huffman.cu:46-118     (length-limited code lengths, package-merge)
 *              kernel/build_huffman.cu:171-239    (canonical codes, LUT fill, 4-bit packing)
 *   decoders   kernel/decode_huffman.cu:188-372   (FP8 bucket kernel; ESC honoured as the encoder
 *                                                  writes it, build_huffman.cu:220-225, 893-903;
 *                                                  element mapping by div/mod as :838-839)
 *              kernel/decode_huffman.cu:378-495   (AWQ bucket kernel)
 *              kernel/decode_huffman.cu:503-589   (AWQ by-scale kernel)
 *              kernel/decode_huffman_encode_only.cu:197-277 (shared-table kernel)
 *
 * Parity pin: the encoders are checked byte-for-byte against the reference encoder compiled from
 * its own sources (oracle/build_ref.sh) and against the golden fixtures made with it; the decoders
 * are pinned by decode(encode(x)) == x on those same artifacts (the reference ships no CPU decoder
 * and no golden vectors).
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------ */
/* Result container handed to Python through ctypes                                            */
/* ------------------------------------------------------------------------------------------ */

enum { ORC_U8 = 0, ORC_U16 = 1, ORC_I16 = 2, ORC_I32 = 3, ORC_U32 = 4, ORC_I64 = 5, ORC_U64 = 6 };
static const int k_dtype_size[] = {1, 2, 2, 4, 4, 8, 8};

typedef struct {
    char name[48];
    int dtype;
    int ndim;
    int64_t shape[2];
    void* data;
} orc_tensor;

typedef struct {
    int ntensors;
    int err_kind; /* 0 ok, 1 invalid argument (ValueError), 2 runtime error (RuntimeError) */
    char err[256];
    orc_tensor t[24];
} orc_result;

static orc_result* res_new(void) { return (orc_result*)calloc(1, sizeof(orc_result)); }

static void* res_add(orc_result* r, const char* name, int dtype, int ndim, int64_t d0, int64_t d1) {
    orc_tensor* t = &r->t[r->ntensors++];
    snprintf(t->name, sizeof(t->name), "%s", name);
    t->dtype = dtype;
    t->ndim = ndim;
    t->shape[0] = d0;
    t->shape[1] = (ndim > 1) ? d1 : 1;
    int64_t numel = d0 * ((ndim > 1) ? d1 : 1);
    t->data = calloc((size_t)(numel > 0 ? numel : 1), (size_t)k_dtype_size[dtype]);
    return t->data;
}

static orc_result* res_fail(orc_result* r, int kind, const char* msg) {
    for (int i = 0; i < r->ntensors; ++i) free(r->t[i].data);
    r->ntensors = 0;
    r->err_kind = kind;
    snprintf(r->err, sizeof(r->err), "%s", msg);
    return r;
}

void orc_free(orc_result* r) {
    if (!r) return;
    for (int i = 0; i < r->ntensors; ++i) free(r->t[i].data);
    free(r);
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads of the decode loops from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Most sub-streams per bucket orc_build_fp8 accepts.  1024 is the reference's limit (build_huffman.cu:313)
 * and the default; a test of the library's finer sub-streams raises it: the layout code below follows
 * build_huffman.cu:811-918, where nothing but that argument check depends on the number. */
static int64_t g_substream_limit = 1024;
void orc_set_substream_limit(int64_t n) { g_substream_limit = n > 0 ? n : 1024; }

/* ------------------------------------------------------------------------------------------ */
/* Length-limited code lengths (package-merge), build_huffman.cu:46-118                        */
/*                                                                                             */
/* The reference keeps explicit package trees and walks them.  Because every round's packages  */
/* are pairs of *consecutive* items from the front of the previous list, and merging is stable */
/* (a leaf wins a tie), the items selected at each level are always a prefix of that level's   */
/* list.  So it is enough to remember, per level, which positions of the list are leaves:      */
/* taking the first T items of a level bumps the first c leaves (c = leaves among them) and    */
/* selects the first 2*(T-c) items of the level below.                                         */
/* ------------------------------------------------------------------------------------------ */

static int cmp_i64(const void* a, const void* b) {
    int64_t x = *(const int64_t*)a, y = *(const int64_t*)b;
    return (x > y) - (x < y);
}

/* weights: any order (sorted ascending internally, as the reference does).  lens[i] is the
 * length of the i-th smallest weight.  Returns 0 ok, 1 invalid argument, 2 runtime error. */
static int package_merge_lengths(const int64_t* weights, int n, int L, int* lens, const char** why) {
    if (L <= 0 || L > 30) { *why = "max_len must be in (0, 30]"; return 1; }
    if (n == 0) return 0;
    if (n == 1) { lens[0] = 1; return 0; }
    if ((int64_t)n > ((int64_t)1 << L)) { *why = "Too many symbols for max_len"; return 1; }

    int64_t* w = (int64_t*)malloc(sizeof(int64_t) * (size_t)n);
    memcpy(w, weights, sizeof(int64_t) * (size_t)n);
    qsort(w, (size_t)n, sizeof(int64_t), cmp_i64);

    const int K = 2 * (n - 1);
    const int keep = 2 * K;
    uint8_t* leaf_flag = (uint8_t*)malloc((size_t)L * (size_t)keep);
    int* level_size = (int*)malloc(sizeof(int) * (size_t)L);
    int64_t* cur = (int64_t*)malloc(sizeof(int64_t) * (size_t)keep);
    int64_t* nxt = (int64_t*)malloc(sizeof(int64_t) * (size_t)keep);
    int64_t* pk = (int64_t*)malloc(sizeof(int64_t) * (size_t)keep);

    int cur_n = n < keep ? n : keep;
    memcpy(cur, w, sizeof(int64_t) * (size_t)cur_n);
    memset(leaf_flag, 1, (size_t)cur_n);
    level_size[0] = cur_n;

    for (int p = 0; p < L - 1; ++p) {
        const int trunc = cur_n < keep ? cur_n : keep;
        int npk = 0;
        for (int i = 0; i + 1 < trunc; i += 2) pk[npk++] = cur[i] + cur[i + 1];
        uint8_t* fl = leaf_flag + (size_t)(p + 1) * (size_t)keep;
        int i = 0, j = 0, o = 0;
        while (o < keep && i < n && j < npk) {
            if (w[i] <= pk[j]) { nxt[o] = w[i++]; fl[o++] = 1; }
            else { nxt[o] = pk[j++]; fl[o++] = 0; }
        }
        while (o < keep && i < n) { nxt[o] = w[i++]; fl[o++] = 1; }
        while (o < keep && j < npk) { nxt[o] = pk[j++]; fl[o++] = 0; }
        cur_n = o;
        level_size[p + 1] = o;
        int64_t* tmp = cur; cur = nxt; nxt = tmp;
    }

    int rc = 0;
    if (cur_n < K) { *why = "Internal error: not enough packages"; rc = 2; }
    else {
        for (int i = 0; i < n; ++i) lens[i] = 0;
        int take = K;
        for (int lvl = L - 1; lvl >= 0 && take > 0; --lvl) {
            const uint8_t* fl = leaf_flag + (size_t)lvl * (size_t)keep;
            int c = 0;
            for (int i = 0; i < take; ++i) c += fl[i];
            for (int i = 0; i < c; ++i) lens[i] += 1;
            take = 2 * (take - c);
        }
    }
    free(w); free(leaf_flag); free(level_size); free(cur); free(nxt); free(pk);
    return rc;
}

/* Exposed for unit tests. */
int orc_package_merge(const int64_t* weights, int n, int L, int* lens) {
    const char* why = "";
    return package_merge_lengths(weights, n, L, lens, &why);
}

/* ------------------------------------------------------------------------------------------ */
/* Per-context codebook                                                                        */
/* ------------------------------------------------------------------------------------------ */

enum { V_FP8 = 0, V_AWQ_BUCKET = 1, V_AWQ_BYSCALE = 2, V_AWQ_SHARED = 3 };

typedef struct { int64_t w; uint16_t sym; } item_t;

static int cmp_item_asc(const void* a, const void* b) {
    const item_t* x = (const item_t*)a; const item_t* y = (const item_t*)b;
    if (x->w != y->w) return (x->w > y->w) - (x->w < y->w);
    return (x->sym > y->sym) - (x->sym < y->sym);
}
static int cmp_item_desc(const void* a, const void* b) {
    const item_t* x = (const item_t*)a; const item_t* y = (const item_t*)b;
    if (x->w != y->w) return (x->w < y->w) - (x->w > y->w);
    return (x->sym > y->sym) - (x->sym < y->sym);
}

typedef struct { uint16_t sym; uint8_t len; uint32_t code; } enc_t;
static int cmp_enc_sym(const void* a, const void* b) {
    const enc_t* x = (const enc_t*)a; const enc_t* y = (const enc_t*)b;
    return (x->sym > y->sym) - (x->sym < y->sym);
}

/* Scratch shared by all contexts of one build (single-threaded build, like the reference). */
typedef struct {
    uint8_t* in_set;   /* 65536 flags */
    item_t* items;     /* capacity max_items + 1 */
    int64_t* weights;
    int* lens;
} cb_scratch;

/*
 * Build one context's decode table and encoder list.
 *   syms/freq: the context's distinct symbols (ascending) with counts.
 *   dec_sym[2^L], dec_len[2^L]: unpacked decode table (dec_len carries the variant's ESC marking).
 *   enc[]: (sym,len,code) sorted by sym, *n_enc entries.
 * Follows build_huffman.cu:452-571 (FP8), :1730-1840 (AWQ bucket), :1225-1335 (AWQ by-scale),
 * :2311-2428 (AWQ shared).
 */
static int build_codebook(int variant, const uint16_t* syms, const uint32_t* freq, int nitems, int L,
                          uint16_t* dec_sym, uint8_t* dec_len, enc_t* enc, int* n_enc,
                          int* has_esc, uint16_t* esc_sym_out, cb_scratch* sc, const char** why) {
    const int64_t table_size = (int64_t)1 << L;
    *n_enc = 0; *has_esc = 0; *esc_sym_out = 0;
    if (nitems == 0) {
        memset(dec_sym, 0, sizeof(uint16_t) * (size_t)table_size);
        memset(dec_len, 0, (size_t)table_size);
        return 0;
    }
    if (nitems == 1) {
        for (int64_t i = 0; i < table_size; ++i) { dec_sym[i] = syms[0]; dec_len[i] = 1; }
        enc[0].sym = syms[0]; enc[0].len = 1; enc[0].code = 0; *n_enc = 1;
        return 0;
    }
    item_t* items = sc->items;
    for (int i = 0; i < nitems; ++i) { items[i].w = (int64_t)(int32_t)freq[i]; items[i].sym = syms[i]; }
    int n = nitems;
    int use_esc = 0;
    uint16_t esc_sym = 0;

    if ((int64_t)nitems > table_size) {
        use_esc = 1;
        qsort(items, (size_t)n, sizeof(item_t), cmp_item_desc);
        const int keep_k = (int)(table_size - 1);
        int64_t esc_freq = 0;
        for (int i = keep_k; i < n; ++i) esc_freq += items[i].w;
        /* candidate set the ESC symbol must avoid: the kept symbols, or (by-scale) every symbol */
        const int avoid_n = (variant == V_AWQ_BYSCALE) ? n : keep_k;
        for (int i = 0; i < avoid_n; ++i) sc->in_set[items[i].sym] = 1;
        uint32_t cand = 0;
        while (cand <= 0xFFFFu && sc->in_set[cand]) ++cand;
        esc_sym = (cand <= 0xFFFFu) ? (uint16_t)cand : (uint16_t)0xFFFFu;
        for (int i = 0; i < avoid_n; ++i) sc->in_set[items[i].sym] = 0;
        if (variant == V_AWQ_BUCKET || variant == V_AWQ_SHARED) { if (esc_freq <= 0) esc_freq = 1; }
        if (variant == V_AWQ_SHARED && esc_freq > 2147483647LL) esc_freq = 2147483647LL;
        n = keep_k + 1;
        items[keep_k].w = esc_freq;
        items[keep_k].sym = esc_sym;
        if (variant != V_AWQ_BYSCALE) qsort(items, (size_t)n, sizeof(item_t), cmp_item_asc);
    } else {
        qsort(items, (size_t)n, sizeof(item_t), cmp_item_asc);
    }

    for (int i = 0; i < n; ++i) sc->weights[i] = items[i].w;
    int rc = package_merge_lengths(sc->weights, n, L, sc->lens, why);
    if (rc) return rc;

    /* canonical first-code per length, codes handed out in item order (build_huffman.cu:171-203) */
    int bl_count[32]; uint32_t next_code[32];
    memset(bl_count, 0, sizeof(bl_count));
    for (int i = 0; i < n; ++i) {
        int li = sc->lens[i];
        if (li <= 0 || li > L) { *why = "invalid code length"; return 2; }
        if (use_esc && items[i].sym == esc_sym && (variant == V_AWQ_BUCKET || variant == V_AWQ_BYSCALE)) li = L;
        sc->lens[i] = li;
        bl_count[li]++;
    }
    uint32_t code = 0; next_code[0] = 0;
    for (int bits = 1; bits < 32; ++bits) { code = (code + (uint32_t)bl_count[bits - 1]) << 1; next_code[bits] = code; }

    memset(dec_sym, 0, sizeof(uint16_t) * (size_t)table_size);
    memset(dec_len, 0, (size_t)table_size);
    for (int i = 0; i < n; ++i) {
        const int len = sc->lens[i];
        const uint32_t c = next_code[len]++;
        enc[i].sym = items[i].sym; enc[i].len = (uint8_t)len; enc[i].code = c;
        const uint32_t fill = 1u << (L - len);
        const uint32_t base = c << (L - len);
        uint8_t mark = (uint8_t)len;
        if (variant == V_FP8 && use_esc && items[i].sym == esc_sym) mark = (uint8_t)(len | 0x8);
        for (uint32_t s = 0; s < fill; ++s) {
            const uint32_t idx = base + s;
            if ((int64_t)idx < table_size) { dec_sym[idx] = items[i].sym; dec_len[idx] = mark; }
        }
    }
    if (use_esc && (variant == V_AWQ_BUCKET || variant == V_AWQ_BYSCALE)) {
        for (int64_t i = 0; i < table_size; ++i) if (dec_sym[i] == esc_sym) dec_len[i] = 15;
    }
    if (use_esc && variant == V_AWQ_SHARED) {
        for (int64_t i = 0; i < table_size; ++i) if (dec_sym[i] == esc_sym) dec_len[i] = (uint8_t)(dec_len[i] | 0x80u);
    }
    qsort(enc, (size_t)n, sizeof(enc_t), cmp_enc_sym);
    *n_enc = n; *has_esc = use_esc; *esc_sym_out = esc_sym;
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* Histogram by (context key, symbol): radix sort of 48-bit composites, then run lengths       */
/* ------------------------------------------------------------------------------------------ */

static void radix_sort48(uint64_t* a, uint64_t* tmp, int64_t n) {
    size_t* cnt = (size_t*)malloc(sizeof(size_t) * 65537);
    for (int pass = 0; pass < 3; ++pass) {
        const int sh = pass * 16;
        memset(cnt, 0, sizeof(size_t) * 65537);
        for (int64_t i = 0; i < n; ++i) cnt[((a[i] >> sh) & 0xFFFF) + 1]++;
        for (int i = 0; i < 65536; ++i) cnt[i + 1] += cnt[i];
        for (int64_t i = 0; i < n; ++i) tmp[cnt[(a[i] >> sh) & 0xFFFF]++] = a[i];
        uint64_t* t = a; a = tmp; tmp = t;
    }
    /* three passes: result ended up in the buffer that was 'tmp' at entry; copy back */
    memcpy(tmp, a, sizeof(uint64_t) * (size_t)n);
}

typedef struct {
    int64_t G;            /* contexts */
    uint32_t* key;        /* [G] (scale<<16)|ctx, ascending */
    int64_t* item_ofs;    /* [G+1] */
    uint16_t* sym;        /* distinct symbols per context, ascending */
    uint32_t* freq;
    int max_items;        /* largest context */
} hist_t;

static void hist_free(hist_t* h) { free(h->key); free(h->item_ofs); free(h->sym); free(h->freq); }

/* comp[i] = key32<<16 | sym  (destroyed) */
static void hist_build(uint64_t* comp, int64_t numel, hist_t* h) {
    uint64_t* tmp = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(numel > 0 ? numel : 1));
    radix_sort48(comp, tmp, numel);
    free(tmp);
    int64_t nitems = 0, G = 0;
    for (int64_t i = 0; i < numel; ++i) {
        if (i == 0 || comp[i] != comp[i - 1]) ++nitems;
        if (i == 0 || (comp[i] >> 16) != (comp[i - 1] >> 16)) ++G;
    }
    h->G = G;
    h->key = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(G + 1));
    h->item_ofs = (int64_t*)malloc(sizeof(int64_t) * (size_t)(G + 2));
    h->sym = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(nitems + 1));
    h->freq = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(nitems + 1));
    int64_t g = -1, it = -1;
    for (int64_t i = 0; i < numel; ++i) {
        if (i == 0 || (comp[i] >> 16) != (comp[i - 1] >> 16)) { ++g; h->key[g] = (uint32_t)(comp[i] >> 16); h->item_ofs[g] = it + 1; }
        if (i == 0 || comp[i] != comp[i - 1]) { ++it; h->sym[it] = (uint16_t)(comp[i] & 0xFFFF); h->freq[it] = 0; }
        h->freq[it]++;
    }
    h->item_ofs[G] = nitems;
    h->max_items = 0;
    for (int64_t i = 0; i < G; ++i) {
        int c = (int)(h->item_ofs[i + 1] - h->item_ofs[i]);
        if (c > h->max_items) h->max_items = c;
    }
}

static int64_t find_key(const hist_t* h, uint32_t key) {
    int64_t lo = 0, hi = h->G - 1;
    while (lo <= hi) {
        int64_t mid = (lo + hi) >> 1;
        if (h->key[mid] == key) return mid;
        if (h->key[mid] < key) lo = mid + 1; else hi = mid - 1;
    }
    return -1;
}

/* ------------------------------------------------------------------------------------------ */
/* Scale broadcasting (build_huffman.cu:331-390 for FP8, :1124-1159 for AWQ)                    */
/* ------------------------------------------------------------------------------------------ */

typedef struct {
    int scalar, per_elem, per_row, block2d;
    int64_t n, m, nb0, nb1, sb0, sb1;
    const uint16_t* s;
} scale_map;

static inline uint16_t scale_at(const scale_map* sm, int64_t r, int64_t c) {
    if (sm->scalar) return sm->s[0];
    if (sm->per_elem) return sm->s[r * sm->m + c];
    if (sm->block2d) return sm->s[(r / sm->sb0) * sm->nb1 + (c / sm->sb1)];
    return sm->s[r];
}

static int scale_map_init(scale_map* sm, int fp8_rules, const uint16_t* scales, int scale_ndim,
                          int64_t sd0, int64_t sd1, int64_t n, int64_t m, const char** why) {
    memset(sm, 0, sizeof(*sm));
    sm->s = scales; sm->n = n; sm->m = m;
    int64_t numel = 1;
    if (scale_ndim >= 1) numel *= sd0;
    if (scale_ndim >= 2) numel *= sd1;
    sm->scalar = (numel == 1);
    if (fp8_rules) {
        sm->per_elem = (!sm->scalar && numel == n * m);
        if (!sm->scalar && !sm->per_elem) {
            sm->per_row = (numel == n);
            if (!sm->per_row && scale_ndim == 2) {
                if (sd0 > 0 && sd1 > 0 && (n % sd0 == 0) && (m % sd1 == 0)) {
                    sm->nb0 = sd0; sm->nb1 = sd1; sm->sb0 = n / sd0; sm->sb1 = m / sd1; sm->block2d = 1;
                }
            }
        }
        if (!sm->scalar && !sm->per_elem && !sm->per_row && !sm->block2d) {
            *why = "unsupported scales shape: use scalar, per-row (n,), per-element (numel), or 2D block-wise [n/bs0,m/bs1]";
            return 1;
        }
    } else {
        sm->per_row = (!sm->scalar && scale_ndim == 1 && numel == n);
        if (!sm->scalar && !sm->per_row && scale_ndim == 2) {
            if (sd0 > 0 && sd1 > 0 && (n % sd0 == 0) && (m % sd1 == 0)) {
                sm->nb0 = sd0; sm->nb1 = sd1; sm->sb0 = n / sd0; sm->sb1 = m / sd1; sm->block2d = 1;
            }
        }
        if (!sm->scalar && !sm->per_row && !sm->block2d) {
            *why = "unsupported scales_u16 shape: use scalar, per-row (n,), or 2D block-wise [n/bs0,m/bs1]";
            return 1;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* Codebooks for all contexts of a tensor                                                      */
/* ------------------------------------------------------------------------------------------ */

typedef struct {
    int64_t G;
    int L;
    uint16_t* dec_sym;  /* [G, 2^L] */
    uint8_t* dec_len;   /* [G, 2^L] unpacked */
    int64_t* enc_ofs;   /* [G+1] */
    enc_t* enc;
    uint8_t* has_esc;   /* [G] */
    uint16_t* esc_sym;  /* [G] */
} books_t;

static void books_free(books_t* b) {
    free(b->dec_sym); free(b->dec_len); free(b->enc_ofs); free(b->enc); free(b->has_esc); free(b->esc_sym);
}

/* ctx_of_table[g] gives, for table g, the histogram context index or -1 (empty table). */
static int books_build(int variant, const hist_t* h, const int64_t* ctx_of_table, int64_t T, int L,
                       books_t* b, const char** why) {
    const int64_t table_size = (int64_t)1 << L;
    memset(b, 0, sizeof(*b));
    b->G = T; b->L = L;
    b->dec_sym = (uint16_t*)calloc((size_t)(T * table_size + 1), sizeof(uint16_t));
    b->dec_len = (uint8_t*)calloc((size_t)(T * table_size + 1), 1);
    b->enc_ofs = (int64_t*)calloc((size_t)(T + 2), sizeof(int64_t));
    b->has_esc = (uint8_t*)calloc((size_t)(T + 1), 1);
    b->esc_sym = (uint16_t*)calloc((size_t)(T + 1), sizeof(uint16_t));
    int64_t enc_cap = 0;
    for (int64_t g = 0; g < T; ++g) {
        int64_t c = ctx_of_table[g];
        int64_t cnt = (c >= 0) ? (h->item_ofs[c + 1] - h->item_ofs[c]) : 0;
        enc_cap += (cnt > table_size) ? table_size : cnt;
    }
    b->enc = (enc_t*)calloc((size_t)(enc_cap + 1), sizeof(enc_t));
    cb_scratch sc;
    sc.in_set = (uint8_t*)calloc(65536, 1);
    sc.items = (item_t*)malloc(sizeof(item_t) * (size_t)(h->max_items + 2));
    sc.weights = (int64_t*)malloc(sizeof(int64_t) * (size_t)(h->max_items + 2));
    sc.lens = (int*)malloc(sizeof(int) * (size_t)(h->max_items + 2));
    int rc = 0;
    int64_t pos = 0;
    for (int64_t g = 0; g < T && !rc; ++g) {
        int64_t c = ctx_of_table[g];
        int nitems = (c >= 0) ? (int)(h->item_ofs[c + 1] - h->item_ofs[c]) : 0;
        int n_enc = 0, has_esc = 0; uint16_t esc = 0;
        b->enc_ofs[g] = pos;
        rc = build_codebook(variant, (c >= 0) ? h->sym + h->item_ofs[c] : NULL, (c >= 0) ? h->freq + h->item_ofs[c] : NULL,
                            nitems, L, b->dec_sym + g * table_size, b->dec_len + g * table_size,
                            b->enc + pos, &n_enc, &has_esc, &esc, &sc, why);
        pos += n_enc;
        b->has_esc[g] = (uint8_t)has_esc;
        b->esc_sym[g] = esc;
    }
    b->enc_ofs[T] = pos;
    free(sc.in_set); free(sc.items); free(sc.weights); free(sc.lens);
    return rc;
}

static inline const enc_t* books_find(const books_t* b, int64_t g, uint16_t sym) {
    int64_t lo = b->enc_ofs[g], hi = b->enc_ofs[g + 1] - 1;
    while (lo <= hi) {
        int64_t mid = (lo + hi) >> 1;
        uint16_t s = b->enc[mid].sym;
        if (s == sym) return &b->enc[mid];
        if (s < sym) lo = mid + 1; else hi = mid - 1;
    }
    return NULL;
}

/* ------------------------------------------------------------------------------------------ */
/* MSB-first bit writer into u64 words (build_huffman.cu:793-806)                               */
/* ------------------------------------------------------------------------------------------ */

typedef struct { uint64_t* w; int64_t cap; int64_t bitpos; } bitw_t;

static void bitw_reserve(bitw_t* bw, int64_t words) {
    if (words <= bw->cap) return;
    int64_t nc = bw->cap ? bw->cap : 1024;
    while (nc < words) nc *= 2;
    bw->w = (uint64_t*)realloc(bw->w, sizeof(uint64_t) * (size_t)nc);
    memset(bw->w + bw->cap, 0, sizeof(uint64_t) * (size_t)(nc - bw->cap));
    bw->cap = nc;
}

static inline void bitw_put(bitw_t* bw, uint32_t code, int len) {
    if (len == 0) return;
    const int64_t wi = bw->bitpos >> 6;
    const int o = (int)(bw->bitpos & 63);
    bitw_reserve(bw, wi + 2);
    const uint64_t v = (uint64_t)code & ((len >= 32) ? 0xFFFFFFFFull : ((1ull << len) - 1ull));
    const int room = 64 - o;
    if (len <= room) bw->w[wi] |= v << (room - len);
    else { bw->w[wi] |= v >> (len - room); bw->w[wi + 1] |= v << (64 - (len - room)); }
    bw->bitpos += len;
}

/* Emit one element; returns bits written, or -1 when the symbol is missing and there is no ESC. */
static inline int emit_symbol(const books_t* b, int64_t g, uint16_t sym, bitw_t* bw) {
    const enc_t* e = books_find(b, g, sym);
    if (e) { if (bw) bitw_put(bw, e->code, e->len); return e->len; }
    if (!b->has_esc[g]) return -1;
    const enc_t* x = books_find(b, g, b->esc_sym[g]);
    if (!x) return -1;
    if (bw) { bitw_put(bw, x->code, x->len); bitw_put(bw, sym, 16); }
    return x->len + 16;
}

static void pack_lens_4bit(const uint8_t* unpacked, int64_t count, uint8_t* packed) {
    for (int64_t i = 0; i < count / 2; ++i)
        packed[i] = (uint8_t)((unpacked[2 * i] & 0x0F) | ((unpacked[2 * i + 1] & 0x0F) << 4));
}

/* ------------------------------------------------------------------------------------------ */
/* Bucket lists                                                                                */
/* ------------------------------------------------------------------------------------------ */

typedef struct {
    int64_t B;
    uint16_t* scale;
    int32_t* row_ofs;    /* [B+1] */
    int32_t* rows;       /* concatenated row lists */
    int64_t nrows;
    int32_t* col_start;
    int32_t* col_len;
} buckets_t;

static void buckets_free(buckets_t* bk) { free(bk->scale); free(bk->row_ofs); free(bk->rows); free(bk->col_start); free(bk->col_len); }

typedef struct { uint16_t sc; int32_t row; } sr_t;
static int cmp_sr(const void* a, const void* b) {
    const sr_t* x = (const sr_t*)a; const sr_t* y = (const sr_t*)b;
    if (x->sc != y->sc) return (x->sc > y->sc) - (x->sc < y->sc);
    return (x->row > y->row) - (x->row < y->row);
}

/* Rectangular buckets of <=128 rows: build_huffman.cu:611-696 (FP8) and :1868-1938 (AWQ). */
static void buckets_build(const scale_map* sm, buckets_t* bk) {
    const int64_t n = sm->n, m = sm->m;
    memset(bk, 0, sizeof(*bk));
    int64_t capB, capR;
    if (!sm->block2d) { capB = n / 1 + 1; capR = n; }
    else { int64_t chunks = (sm->sb0 + 127) / 128; capB = sm->nb0 * sm->nb1 * chunks + 1; capR = n * sm->nb1; }
    bk->scale = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)capB);
    bk->row_ofs = (int32_t*)malloc(sizeof(int32_t) * (size_t)(capB + 1));
    bk->col_start = (int32_t*)malloc(sizeof(int32_t) * (size_t)capB);
    bk->col_len = (int32_t*)malloc(sizeof(int32_t) * (size_t)capB);
    bk->rows = (int32_t*)malloc(sizeof(int32_t) * (size_t)(capR + 1));
    bk->row_ofs[0] = 0;
    int64_t B = 0, R = 0;
    if (!sm->block2d) {
        sr_t* sr = (sr_t*)malloc(sizeof(sr_t) * (size_t)n);
        for (int64_t r = 0; r < n; ++r) { sr[r].sc = sm->scalar ? sm->s[0] : sm->s[r]; sr[r].row = (int32_t)r; }
        qsort(sr, (size_t)n, sizeof(sr_t), cmp_sr);
        int64_t i = 0;
        while (i < n) {
            int64_t j = i;
            while (j < n && sr[j].sc == sr[i].sc) ++j;
            for (int64_t off = i; off < j; off += 128) {
                int64_t take = (j - off < 128) ? (j - off) : 128;
                for (int64_t q = 0; q < take; ++q) bk->rows[R++] = sr[off + q].row;
                bk->scale[B] = sr[i].sc; bk->col_start[B] = 0; bk->col_len[B] = (int32_t)m;
                ++B; bk->row_ofs[B] = (int32_t)R;
            }
            i = j;
        }
        free(sr);
    } else {
        for (int64_t br = 0; br < sm->nb0; ++br) {
            const int64_t r0 = br * sm->sb0;
            for (int64_t bc = 0; bc < sm->nb1; ++bc) {
                const uint16_t sc = sm->s[br * sm->nb1 + bc];
                for (int64_t off = 0; off < sm->sb0; off += 128) {
                    int64_t take = (sm->sb0 - off < 128) ? (sm->sb0 - off) : 128;
                    for (int64_t q = 0; q < take; ++q) bk->rows[R++] = (int32_t)(r0 + off + q);
                    bk->scale[B] = sc; bk->col_start[B] = (int32_t)(bc * sm->sb1); bk->col_len[B] = (int32_t)sm->sb1;
                    ++B; bk->row_ofs[B] = (int32_t)R;
                }
            }
        }
    }
    bk->B = B; bk->nrows = R;
}

/* ------------------------------------------------------------------------------------------ */
/* Sub-stream layout + bitstream for rectangular buckets (FP8 :811-918, AWQ bucket :2004-2102)  */
/* ------------------------------------------------------------------------------------------ */

static int encode_rect_buckets(const buckets_t* bk, const books_t* books, const int32_t* bucket_table, int nctx,
                               const uint16_t* bf16, const uint8_t* ctxv, int ctx_mask, int64_t m, int k_threads,
                               uint32_t* startbit /*[B,k+1]*/, int64_t* bit_base /*[B+1]*/, bitw_t* bw, const char** why) {
    for (int64_t bi = 0; bi < bk->B; ++bi) {
        if (bw->bitpos & 63) bw->bitpos = (bw->bitpos + 63) & ~63LL;
        const int64_t base = bw->bitpos;
        bit_base[bi] = base;
        const int32_t row_a = bk->row_ofs[bi];
        const int64_t rows = bk->row_ofs[bi + 1] - row_a;
        const int64_t col_len = bk->col_len[bi], col_start = bk->col_start[bi];
        const int64_t total = rows * col_len;
        int64_t k_eff = total < 1 ? 1 : total;
        if (k_eff > k_threads) k_eff = k_threads;
        uint32_t* st = startbit + bi * ((int64_t)k_threads + 1);
        const int32_t* bt = bucket_table + bi * nctx;
        int64_t rel = 0;
        st[0] = 0;
        for (int64_t t = 0; t < k_eff; ++t) {
            for (int64_t e = t; e < total; e += k_eff) {
                const int64_t rr = e / col_len, cc = e - rr * col_len;
                const int64_t idx = (int64_t)bk->rows[row_a + rr] * m + col_start + cc;
                const int32_t g = bt[ctxv[idx] & ctx_mask];
                if (g < 0) { *why = "missing enc table for (scale,ctx) key"; return 2; }
                const int bits = emit_symbol(books, g, bf16[idx], bw);
                if (bits < 0) { *why = "symbol not found and no ESC for (scale,ctx) key"; return 2; }
                rel += bits;
            }
            st[t + 1] = (uint32_t)rel;
        }
        for (int64_t t = k_eff + 1; t <= k_threads; ++t) st[t] = st[k_eff];
        if ((uint32_t)(bw->bitpos - base) != st[k_eff]) { *why = "internal error: bucket bit length mismatch"; return 2; }
    }
    bit_base[bk->B] = bw->bitpos;
    return 0;
}

static void fill_bucket_table(const hist_t* h, const buckets_t* bk, int nctx, int32_t* bt) {
    for (int64_t bi = 0; bi < bk->B; ++bi)
        for (int c = 0; c < nctx; ++c)
            bt[bi * nctx + c] = (int32_t)find_key(h, ((uint32_t)bk->scale[bi] << 16) | (uint32_t)c);
}

static void copy_bitstream(orc_result* r, bitw_t* bw) {
    const int64_t nwords = (bw->bitpos + 63) >> 6;
    uint64_t* out = (uint64_t*)res_add(r, "bitstream_u64", ORC_U64, 1, nwords, 1);
    for (int64_t i = 0; i < nwords; ++i) out[i] = (i < bw->cap) ? bw->w[i] : 0ull;
}

/* ------------------------------------------------------------------------------------------ */
/* FP8 encoder entry (build_huffman.cu:292-969)                                                 */
/* ------------------------------------------------------------------------------------------ */

orc_result* orc_build_fp8(const uint16_t* bf16, const uint8_t* fp8, const uint16_t* scales, int scale_ndim,
                          int64_t sd0, int64_t sd1, int64_t n, int64_t m, int64_t max_len, int64_t threads_per_block) {
    orc_result* r = res_new();
    const char* why = "";
    if (max_len <= 0 || max_len > 15) return res_fail(r, 1, "max_len must be in [1, 15]");
    if (threads_per_block <= 0 || threads_per_block > g_substream_limit) return res_fail(r, 1, "threads_per_block must be in [1, 1024]");
    if (n <= 0 || m <= 0) return res_fail(r, 1, "bf16_params shape must be non-empty");
    scale_map sm;
    if (scale_map_init(&sm, 1, scales, scale_ndim, sd0, sd1, n, m, &why)) return res_fail(r, 1, why);
    const int L = (int)max_len, k = (int)threads_per_block;
    const int64_t numel = n * m, table_size = (int64_t)1 << L;

    uint64_t* comp = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)numel);
    for (int64_t rr = 0; rr < n; ++rr)
        for (int64_t c = 0; c < m; ++c) {
            const int64_t i = rr * m + c;
            comp[i] = ((uint64_t)scale_at(&sm, rr, c) << 32) | ((uint64_t)fp8[i] << 16) | bf16[i];
        }
    hist_t h; hist_build(comp, numel, &h); free(comp);

    int64_t* ident = (int64_t*)malloc(sizeof(int64_t) * (size_t)(h.G + 1));
    for (int64_t g = 0; g < h.G; ++g) ident[g] = g;
    books_t books;
    int rc = books_build(V_FP8, &h, ident, h.G, L, &books, &why);
    free(ident);
    if (rc) { hist_free(&h); books_free(&books); return res_fail(r, rc, why); }

    if (sm.per_elem) { hist_free(&h); books_free(&books);
        return res_fail(r, 1, "bucket packing requires scales to be scalar, per-row (n,), or 2D block-wise"); }

    const int64_t G = h.G;
    uint16_t* o_syms = (uint16_t*)res_add(r, "decode_syms_u16", ORC_U16, 2, G, table_size);
    uint8_t* o_lens = (uint8_t*)res_add(r, "decode_lens_u8", ORC_U8, 2, G, table_size / 2);
    uint16_t* o_tscale = (uint16_t*)res_add(r, "table_scale_u16", ORC_U16, 1, G, 1);
    uint16_t* o_tfp8 = (uint16_t*)res_add(r, "table_fp8_u16", ORC_U16, 1, G, 1);
    memcpy(o_syms, books.dec_sym, sizeof(uint16_t) * (size_t)(G * table_size));
    for (int64_t g = 0; g < G; ++g) {
        pack_lens_4bit(books.dec_len + g * table_size, table_size, o_lens + g * (table_size / 2));
        o_tscale[g] = (uint16_t)(h.key[g] >> 16);
        o_tfp8[g] = (uint16_t)(h.key[g] & 0xFFFF);
    }

    buckets_t bk; buckets_build(&sm, &bk);
    const int64_t B = bk.B;
    uint16_t* o_bscale = (uint16_t*)res_add(r, "bucket_scale_u16", ORC_U16, 1, B, 1);
    int32_t* o_rofs = (int32_t*)res_add(r, "bucket_row_offsets_i32", ORC_I32, 1, B + 1, 1);
    int32_t* o_rows = (int32_t*)res_add(r, "row_indices_i32", ORC_I32, 1, bk.nrows, 1);
    int32_t* o_bt = (int32_t*)res_add(r, "bucket_table_i32", ORC_I32, 2, B, 256);
    int32_t* o_cs = (int32_t*)res_add(r, "bucket_col_start_i32", ORC_I32, 1, B, 1);
    int32_t* o_cl = (int32_t*)res_add(r, "bucket_col_len_i32", ORC_I32, 1, B, 1);
    uint32_t* o_tsb = (uint32_t*)res_add(r, "bucket_thread_startbit_u32", ORC_U32, 2, B, (int64_t)k + 1);
    int64_t* o_base = (int64_t*)res_add(r, "bucket_bit_base_i64", ORC_I64, 1, B + 1, 1);
    memcpy(o_bscale, bk.scale, sizeof(uint16_t) * (size_t)B);
    memcpy(o_rofs, bk.row_ofs, sizeof(int32_t) * (size_t)(B + 1));
    memcpy(o_rows, bk.rows, sizeof(int32_t) * (size_t)bk.nrows);
    memcpy(o_cs, bk.col_start, sizeof(int32_t) * (size_t)B);
    memcpy(o_cl, bk.col_len, sizeof(int32_t) * (size_t)B);
    fill_bucket_table(&h, &bk, 256, o_bt);

    bitw_t bw; memset(&bw, 0, sizeof(bw));
    rc = encode_rect_buckets(&bk, &books, o_bt, 256, bf16, fp8, 0xFF, m, k, o_tsb, o_base, &bw, &why);
    if (rc) { free(bw.w); buckets_free(&bk); hist_free(&h); books_free(&books); return res_fail(r, rc, why); }
    copy_bitstream(r, &bw);
    free(bw.w);

    int64_t* o_shape = (int64_t*)res_add(r, "shape_nmk_i64", ORC_I64, 1, 3, 1);
    o_shape[0] = n; o_shape[1] = m; o_shape[2] = k;
    int32_t* o_U = (int32_t*)res_add(r, "bucket_U_i32", ORC_I32, 1, B, 1);
    int32_t* o_uniq = (int32_t*)res_add(r, "bucket_unique_gid_i32", ORC_I32, 2, B, 256);
    int16_t* o_uidx = (int16_t*)res_add(r, "bucket_fp8_uidx_i16", ORC_I16, 2, B, 256);
    /* first-appearance list of the bucket's tables and fp8 -> position (build_huffman.cu:748-783) */
    for (int64_t bi = 0; bi < B; ++bi) {
        int32_t U = 0;
        for (int i = 0; i < 256; ++i) { o_uniq[bi * 256 + i] = -1; o_uidx[bi * 256 + i] = -1; }
        for (int i = 0; i < 256; ++i) {
            const int32_t gid = o_bt[bi * 256 + i];
            if (gid < 0) continue;
            int32_t found = -1;
            for (int32_t j = 0; j < U; ++j) if (o_uniq[bi * 256 + j] == gid) { found = j; break; }
            if (found < 0) { o_uniq[bi * 256 + U] = gid; found = U++; }
            o_uidx[bi * 256 + i] = (int16_t)found;
        }
        o_U[bi] = U;
    }
    buckets_free(&bk); hist_free(&h); books_free(&books);
    return r;
}

/* ------------------------------------------------------------------------------------------ */
/* AWQ rectangular-bucket encoder entry (build_huffman.cu:1582-2126)                            */
/* ------------------------------------------------------------------------------------------ */

static uint64_t* awq_composites(const scale_map* sm, const uint16_t* bf16, const uint8_t* q, int64_t n, int64_t m) {
    uint64_t* comp = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n * m));
    for (int64_t rr = 0; rr < n; ++rr)
        for (int64_t c = 0; c < m; ++c) {
            const int64_t i = rr * m + c;
            comp[i] = ((uint64_t)scale_at(sm, rr, c) << 32) | ((uint64_t)(q[i] & 0x0F) << 16) | bf16[i];
        }
    return comp;
}

static void emit_awq_tables(orc_result* r, const hist_t* h, const books_t* books, int L) {
    const int64_t G = h->G, table_size = (int64_t)1 << L;
    uint16_t* o_syms = (uint16_t*)res_add(r, "decode_syms_u16", ORC_U16, 2, G, table_size);
    uint8_t* o_lens = (uint8_t*)res_add(r, "decode_lens_u8", ORC_U8, 2, G, table_size / 2);
    uint16_t* o_tscale = (uint16_t*)res_add(r, "table_scale_u16", ORC_U16, 1, G, 1);
    uint16_t* o_tqv = (uint16_t*)res_add(r, "table_qv_u16", ORC_U16, 1, G, 1);
    memcpy(o_syms, books->dec_sym, sizeof(uint16_t) * (size_t)(G * table_size));
    for (int64_t g = 0; g < G; ++g) {
        pack_lens_4bit(books->dec_len + g * table_size, table_size, o_lens + g * (table_size / 2));
        o_tscale[g] = (uint16_t)(h->key[g] >> 16);
        o_tqv[g] = (uint16_t)(h->key[g] & 0xFFFF);
    }
}

orc_result* orc_build_awq_bucket(const uint16_t* bf16, const uint8_t* q, const uint16_t* scales, int scale_ndim,
                                 int64_t sd0, int64_t sd1, int64_t n, int64_t m, int64_t max_len, int64_t threads_per_block) {
    orc_result* r = res_new();
    const char* why = "";
    if (max_len <= 0 || max_len > 15) return res_fail(r, 1, "max_len must be in (0,15]");
    if (threads_per_block <= 0 || threads_per_block > 1024) return res_fail(r, 1, "threads_per_block must be in [1,1024]");
    if (n <= 0 || m <= 0) return res_fail(r, 1, "bf16_params shape must be non-empty");
    scale_map sm;
    if (scale_map_init(&sm, 0, scales, scale_ndim, sd0, sd1, n, m, &why)) return res_fail(r, 1, why);
    const int L = (int)max_len, k = (int)threads_per_block;

    uint64_t* comp = awq_composites(&sm, bf16, q, n, m);
    hist_t h; hist_build(comp, n * m, &h); free(comp);
    int64_t* ident = (int64_t*)malloc(sizeof(int64_t) * (size_t)(h.G + 1));
    for (int64_t g = 0; g < h.G; ++g) ident[g] = g;
    books_t books;
    int rc = books_build(V_AWQ_BUCKET, &h, ident, h.G, L, &books, &why);
    free(ident);
    if (rc) { hist_free(&h); books_free(&books); return res_fail(r, rc, why); }
    emit_awq_tables(r, &h, &books, L);

    buckets_t bk; buckets_build(&sm, &bk);
    const int64_t B = bk.B;
    uint16_t* o_bscale = (uint16_t*)res_add(r, "bucket_scale_u16", ORC_U16, 1, B, 1);
    int32_t* o_rofs = (int32_t*)res_add(r, "bucket_row_offsets_i32", ORC_I32, 1, B + 1, 1);
    int32_t* o_rows = (int32_t*)res_add(r, "row_indices_i32", ORC_I32, 1, bk.nrows, 1);
    int32_t* o_bt = (int32_t*)res_add(r, "bucket_table_i32", ORC_I32, 2, B, 16);
    int32_t* o_cs = (int32_t*)res_add(r, "bucket_col_start_i32", ORC_I32, 1, B, 1);
    int32_t* o_cl = (int32_t*)res_add(r, "bucket_col_len_i32", ORC_I32, 1, B, 1);
    uint32_t* o_tsb = (uint32_t*)res_add(r, "bucket_thread_startbit_u32", ORC_U32, 2, B, (int64_t)k + 1);
    int64_t* o_base = (int64_t*)res_add(r, "bucket_bit_base_i64", ORC_I64, 1, B + 1, 1);
    memcpy(o_bscale, bk.scale, sizeof(uint16_t) * (size_t)B);
    memcpy(o_rofs, bk.row_ofs, sizeof(int32_t) * (size_t)(B + 1));
    memcpy(o_rows, bk.rows, sizeof(int32_t) * (size_t)bk.nrows);
    memcpy(o_cs, bk.col_start, sizeof(int32_t) * (size_t)B);
    memcpy(o_cl, bk.col_len, sizeof(int32_t) * (size_t)B);
    fill_bucket_table(&h, &bk, 16, o_bt);

    bitw_t bw; memset(&bw, 0, sizeof(bw));
    rc = encode_rect_buckets(&bk, &books, o_bt, 16, bf16, q, 0x0F, m, k, o_tsb, o_base, &bw, &why);
    if (rc) { free(bw.w); buckets_free(&bk); hist_free(&h); books_free(&books); return res_fail(r, rc, why); }
    copy_bitstream(r, &bw);
    free(bw.w);
    int64_t* o_shape = (int64_t*)res_add(r, "shape_nmk_i64", ORC_I64, 1, 3, 1);
    o_shape[0] = n; o_shape[1] = m; o_shape[2] = k;
    buckets_free(&bk); hist_free(&h); books_free(&books);
    return r;
}

/* ------------------------------------------------------------------------------------------ */
/* AWQ ragged (by exact scale) encoder entry (build_huffman.cu:1074-1580)                       */
/* ------------------------------------------------------------------------------------------ */

typedef struct { uint16_t sc; int32_t row; int32_t c0; } grp_t;
static int cmp_grp(const void* a, const void* b) {
    const grp_t* x = (const grp_t*)a; const grp_t* y = (const grp_t*)b;
    if (x->sc != y->sc) return (x->sc > y->sc) - (x->sc < y->sc);
    if (x->row != y->row) return (x->row > y->row) - (x->row < y->row);
    return (x->c0 > y->c0) - (x->c0 < y->c0);
}

orc_result* orc_build_awq_by_scale(const uint16_t* bf16, const uint8_t* q, const uint16_t* scales, int scale_ndim,
                                   int64_t sd0, int64_t sd1, int64_t n, int64_t m, int64_t max_len,
                                   int64_t threads_per_block, int64_t group_cap) {
    orc_result* r = res_new();
    const char* why = "";
    if (max_len <= 0 || max_len > 15) return res_fail(r, 1, "max_len must be in (0,15]");
    if (threads_per_block <= 0 || threads_per_block > 1024) return res_fail(r, 1, "threads_per_block must be in [1,1024]");
    if (group_cap <= 0) return res_fail(r, 1, "group_cap must be > 0");
    if (n <= 0 || m <= 0) return res_fail(r, 1, "bf16_params shape must be non-empty");
    scale_map sm;
    if (scale_map_init(&sm, 0, scales, scale_ndim, sd0, sd1, n, m, &why)) return res_fail(r, 1, why);
    const int L = (int)max_len, k = (int)threads_per_block;
    const int64_t group_size = sm.block2d ? sm.sb1 : m;
    const int64_t groups_per_row = sm.block2d ? sm.nb1 : 1;

    uint64_t* comp = awq_composites(&sm, bf16, q, n, m);
    hist_t h; hist_build(comp, n * m, &h); free(comp);
    int64_t* ident = (int64_t*)malloc(sizeof(int64_t) * (size_t)(h.G + 1));
    for (int64_t g = 0; g < h.G; ++g) ident[g] = g;
    books_t books;
    int rc = books_build(V_AWQ_BYSCALE, &h, ident, h.G, L, &books, &why);
    free(ident);
    if (rc) { hist_free(&h); books_free(&books); return res_fail(r, rc, why); }
    emit_awq_tables(r, &h, &books, L);

    /* groups sorted by (scale, row, col) and cut into buckets of <= group_cap (:1353-1392) */
    const int64_t NG = n * groups_per_row;
    grp_t* grp = (grp_t*)malloc(sizeof(grp_t) * (size_t)NG);
    for (int64_t rr = 0; rr < n; ++rr)
        for (int64_t bc = 0; bc < groups_per_row; ++bc) {
            grp_t* g = &grp[rr * groups_per_row + bc];
            g->row = (int32_t)rr; g->c0 = (int32_t)(bc * group_size); g->sc = scale_at(&sm, rr, g->c0);
        }
    qsort(grp, (size_t)NG, sizeof(grp_t), cmp_grp);
    int64_t B = 0;
    for (int64_t i = 0; i < NG;) {
        int64_t j = i;
        while (j < NG && grp[j].sc == grp[i].sc) ++j;
        B += (j - i + group_cap - 1) / group_cap;
        i = j;
    }
    uint16_t* o_bscale = (uint16_t*)res_add(r, "bucket_scale_u16", ORC_U16, 1, B, 1);
    int32_t* o_gofs = (int32_t*)res_add(r, "bucket_group_offsets_i32", ORC_I32, 1, B + 1, 1);
    int32_t* o_grow = (int32_t*)res_add(r, "group_rows_i32", ORC_I32, 1, NG, 1);
    int32_t* o_gcol = (int32_t*)res_add(r, "group_col_start_i32", ORC_I32, 1, NG, 1);
    int32_t* o_bt = (int32_t*)res_add(r, "bucket_table_i32", ORC_I32, 2, B, 16);
    uint32_t* o_tsb = (uint32_t*)res_add(r, "bucket_thread_startbit_u32", ORC_U32, 2, B, (int64_t)k + 1);
    int64_t* o_base = (int64_t*)res_add(r, "bucket_bit_base_i64", ORC_I64, 1, B + 1, 1);
    {
        int64_t b = 0; o_gofs[0] = 0;
        for (int64_t i = 0; i < NG;) {
            int64_t j = i;
            while (j < NG && grp[j].sc == grp[i].sc) ++j;
            for (int64_t off = i; off < j; off += group_cap) {
                int64_t take = (j - off < group_cap) ? (j - off) : group_cap;
                o_bscale[b] = grp[i].sc;
                ++b; o_gofs[b] = (int32_t)(off + take);
            }
            i = j;
        }
        for (int64_t i = 0; i < NG; ++i) { o_grow[i] = grp[i].row; o_gcol[i] = grp[i].c0; }
    }
    free(grp);
    for (int64_t bi = 0; bi < B; ++bi)
        for (int c = 0; c < 16; ++c)
            o_bt[bi * 16 + c] = (int32_t)find_key(&h, ((uint32_t)o_bscale[bi] << 16) | (uint32_t)c);

    bitw_t bw; memset(&bw, 0, sizeof(bw));
    for (int64_t bi = 0; bi < B && !rc; ++bi) {
        if (bw.bitpos & 63) bw.bitpos = (bw.bitpos + 63) & ~63LL;
        const int64_t base = bw.bitpos;
        o_base[bi] = base;
        const int32_t ga = o_gofs[bi];
        const int64_t total = (int64_t)(o_gofs[bi + 1] - ga) * group_size;
        int64_t k_eff = total < 1 ? 1 : total;
        if (k_eff > k) k_eff = k;
        uint32_t* st = o_tsb + bi * ((int64_t)k + 1);
        int64_t rel = 0;
        for (int64_t t = 0; t < k_eff && !rc; ++t) {
            for (int64_t e = t; e < total; e += k_eff) {
                const int64_t gi = e / group_size, j = e - gi * group_size;
                const int64_t idx = (int64_t)o_grow[ga + gi] * m + o_gcol[ga + gi] + j;
                const int32_t g = o_bt[bi * 16 + (q[idx] & 0x0F)];
                if (g < 0) { why = "missing enc table for (scale,qv) key"; rc = 2; break; }
                const int bits = emit_symbol(&books, g, bf16[idx], &bw);
                if (bits < 0) { why = "symbol not found and no ESC for (scale,qv) key"; rc = 2; break; }
                rel += bits;
            }
            st[t + 1] = (uint32_t)rel;
        }
        for (int64_t t = k_eff + 1; t <= k; ++t) st[t] = st[k_eff];
        if (!rc && (uint32_t)(bw.bitpos - base) != st[k_eff]) { why = "internal error: bucket bit length mismatch"; rc = 2; }
    }
    if (rc) { free(bw.w); hist_free(&h); books_free(&books); return res_fail(r, rc, why); }
    o_base[B] = bw.bitpos;
    copy_bitstream(r, &bw);
    free(bw.w);
    int64_t* o_shape = (int64_t*)res_add(r, "shape_nmkg_i64", ORC_I64, 1, 4, 1);
    o_shape[0] = n; o_shape[1] = m; o_shape[2] = k; o_shape[3] = group_size;
    hist_free(&h); books_free(&books);
    return r;
}

/* ------------------------------------------------------------------------------------------ */
/* AWQ shared-table (chunked) encoder entry (build_huffman.cu:2157-2633)                        */
/* ------------------------------------------------------------------------------------------ */

static int cmp_u16(const void* a, const void* b) {
    uint16_t x = *(const uint16_t*)a, y = *(const uint16_t*)b;
    return (x > y) - (x < y);
}

orc_result* orc_build_awq_shared(const uint16_t* bf16, const uint8_t* q, const uint16_t* scales, int scale_ndim,
                                 int64_t sd0, int64_t sd1, int64_t n, int64_t m, int64_t max_len) {
    orc_result* r = res_new();
    const char* why = "";
    if (max_len <= 0 || max_len > 20) return res_fail(r, 1, "max_len must be in (0,20]");
    if (n <= 0 || m <= 0) return res_fail(r, 1, "bf16_params shape must be non-empty");
    scale_map sm;
    if (scale_map_init(&sm, 0, scales, scale_ndim, sd0, sd1, n, m, &why)) return res_fail(r, 1, why);
    const int L = (int)max_len;
    const int64_t table_size = (int64_t)1 << L, numel = n * m;

    /* dense scale ids over the sorted distinct scale values (:2221-2256) */
    int64_t ns = 1;
    if (scale_ndim >= 1) ns *= sd0;
    if (scale_ndim >= 2) ns *= sd1;
    uint16_t* sv = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)ns);
    memcpy(sv, scales, sizeof(uint16_t) * (size_t)ns);
    qsort(sv, (size_t)ns, sizeof(uint16_t), cmp_u16);
    int64_t S = 0;
    for (int64_t i = 0; i < ns; ++i) if (i == 0 || sv[i] != sv[i - 1]) sv[S++] = sv[i];
    int32_t* sid_of = (int32_t*)malloc(sizeof(int32_t) * 65536);
    for (int i = 0; i < 65536; ++i) sid_of[i] = -1;
    for (int64_t i = 0; i < S; ++i) sid_of[sv[i]] = (int32_t)i;
    const int64_t num_streams = S * 16;

    uint64_t* comp = awq_composites(&sm, bf16, q, n, m);
    hist_t h; hist_build(comp, numel, &h); free(comp);
    int64_t* ctx_of = (int64_t*)malloc(sizeof(int64_t) * (size_t)(num_streams + 1));
    for (int64_t s = 0; s < num_streams; ++s) ctx_of[s] = find_key(&h, ((uint32_t)sv[s / 16] << 16) | (uint32_t)(s % 16));
    books_t books;
    int rc = books_build(V_AWQ_SHARED, &h, ctx_of, num_streams, L, &books, &why);
    free(ctx_of);
    if (rc) { hist_free(&h); books_free(&books); free(sv); free(sid_of); return res_fail(r, rc, why); }

    int16_t* o_syms = (int16_t*)res_add(r, "decode_syms_i16", ORC_I16, 2, num_streams, table_size);
    uint8_t* o_nbits = (uint8_t*)res_add(r, "decode_nbits_u8", ORC_U8, 2, num_streams, table_size);
    memcpy(o_syms, books.dec_sym, sizeof(uint16_t) * (size_t)(num_streams * table_size));
    memcpy(o_nbits, books.dec_len, (size_t)(num_streams * table_size));
    uint16_t* o_sv = (uint16_t*)res_add(r, "scale_values_u16", ORC_U16, 1, S, 1);
    memcpy(o_sv, sv, sizeof(uint16_t) * (size_t)S);
    int64_t* o_sbase = (int64_t*)res_add(r, "scale_bit_base_i64", ORC_I64, 1, S + 1, 1);

    /* per-scale bit writers; chunks of <=255 consecutive elements of one (scale,qv) (:2434-2537) */
    bitw_t* bws = (bitw_t*)calloc((size_t)S, sizeof(bitw_t));
    int64_t cap = 1024, C = 0;
    uint32_t* c_start = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)cap);
    uint32_t* c_base = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)cap);
    uint32_t* c_meta = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)cap);
    int32_t* c_sid = (int32_t*)malloc(sizeof(int32_t) * (size_t)cap);
    int64_t flat = 0;
    while (flat < numel && !rc) {
        const int64_t r0 = flat / m, c0 = flat - r0 * m;
        const uint8_t qv0 = q[flat] & 0x0F;
        const int32_t sid0 = sid_of[scale_at(&sm, r0, c0)];
        const int64_t stream0 = (int64_t)sid0 * 16 + qv0;
        const uint32_t startbit = (uint32_t)bws[sid0].bitpos;
        uint32_t take = 0;
        for (; take < 255 && flat + take < numel; ++take) {
            const int64_t idx = flat + take;
            const int64_t rr = idx / m, cc = idx - rr * m;
            if (sid_of[scale_at(&sm, rr, cc)] != sid0 || (q[idx] & 0x0F) != qv0) break;
            if (emit_symbol(&books, stream0, bf16[idx], &bws[sid0]) < 0) {
                why = "symbol not found in enc table for AWQ stream"; rc = 2; break;
            }
        }
        if (!rc && take == 0) { why = "internal error: zero-length chunk"; rc = 2; }
        if (C == cap) {
            cap *= 2;
            c_start = (uint32_t*)realloc(c_start, sizeof(uint32_t) * (size_t)cap);
            c_base = (uint32_t*)realloc(c_base, sizeof(uint32_t) * (size_t)cap);
            c_meta = (uint32_t*)realloc(c_meta, sizeof(uint32_t) * (size_t)cap);
            c_sid = (int32_t*)realloc(c_sid, sizeof(int32_t) * (size_t)cap);
        }
        c_base[C] = (uint32_t)flat; c_start[C] = startbit; c_sid[C] = sid0; c_meta[C] = (take << 8) | qv0;
        ++C;
        flat += take;
    }
    if (rc) {
        for (int64_t s = 0; s < S; ++s) free(bws[s].w);
        free(bws); free(c_start); free(c_base); free(c_meta); free(c_sid); free(sv); free(sid_of);
        hist_free(&h); books_free(&books);
        return res_fail(r, rc, why);
    }
    int64_t total_bits = 0;
    for (int64_t s = 0; s < S; ++s) {
        if (total_bits & 63) total_bits = (total_bits + 63) & ~63LL;
        o_sbase[s] = total_bits;
        total_bits += bws[s].bitpos;
    }
    if (total_bits & 63) total_bits = (total_bits + 63) & ~63LL;
    o_sbase[S] = total_bits;

    uint32_t* o_cstart = (uint32_t*)res_add(r, "chunk_startbit_rel_u32", ORC_U32, 1, C, 1);
    uint32_t* o_cbase = (uint32_t*)res_add(r, "chunk_out_base_u32", ORC_U32, 1, C, 1);
    uint32_t* o_cmeta = (uint32_t*)res_add(r, "chunk_meta_u32", ORC_U32, 1, C, 1);
    int32_t* o_csid = (int32_t*)res_add(r, "chunk_scale_id_i32", ORC_I32, 1, C, 1);
    memcpy(o_cstart, c_start, sizeof(uint32_t) * (size_t)C);
    memcpy(o_cbase, c_base, sizeof(uint32_t) * (size_t)C);
    memcpy(o_cmeta, c_meta, sizeof(uint32_t) * (size_t)C);
    memcpy(o_csid, c_sid, sizeof(int32_t) * (size_t)C);
    int32_t* o_idx = (int32_t*)res_add(r, "out_idx_i32", ORC_I32, 1, numel, 1);
    for (int64_t i = 0; i < numel; ++i) o_idx[i] = (int32_t)i;
    int64_t* o_sofs = (int64_t*)res_add(r, "stream_chunk_ofs_i64", ORC_I64, 1, num_streams + 1, 1);
    int32_t* o_sids = (int32_t*)res_add(r, "stream_chunk_ids_i32", ORC_I32, 1, C, 1);
    for (int64_t c = 0; c < C; ++c) o_sofs[(int64_t)c_sid[c] * 16 + (c_meta[c] & 0xFF) + 1]++;
    for (int64_t s = 0; s < num_streams; ++s) o_sofs[s + 1] += o_sofs[s];
    {
        int64_t* cursor = (int64_t*)malloc(sizeof(int64_t) * (size_t)(num_streams + 1));
        memcpy(cursor, o_sofs, sizeof(int64_t) * (size_t)num_streams);
        for (int64_t c = 0; c < C; ++c) o_sids[cursor[(int64_t)c_sid[c] * 16 + (c_meta[c] & 0xFF)]++] = (int32_t)c;
        free(cursor);
    }
    const int64_t total_words = total_bits >> 6;
    uint64_t* o_bs = (uint64_t*)res_add(r, "bitstream_u64", ORC_U64, 1, total_words, 1);
    for (int64_t s = 0; s < S; ++s) {
        const int64_t wbase = o_sbase[s] >> 6, words = (bws[s].bitpos + 63) >> 6;
        if (words > 0) memcpy(o_bs + wbase, bws[s].w, sizeof(uint64_t) * (size_t)words);
        free(bws[s].w);
    }
    free(bws); free(c_start); free(c_base); free(c_meta); free(c_sid); free(sv); free(sid_of);
    hist_free(&h); books_free(&books);
    return r;
}

/* ------------------------------------------------------------------------------------------ */
/* Decoders                                                                                    */
/* ------------------------------------------------------------------------------------------ */

/* Top `L` bits at absolute bit position; words past the end read as zero
 * (decode_huffman.cu:39-57, 82-88, 154-169). */
static inline uint32_t peek_bits(const uint64_t* bs, int64_t nwords, int64_t bitpos, int L) {
    const int64_t w = bitpos >> 6;
    const int o = (int)(bitpos & 63);
    const uint64_t a = (w >= 0 && w < nwords) ? bs[w] : 0ull;
    const uint64_t b = (w + 1 >= 0 && w + 1 < nwords) ? bs[w + 1] : 0ull;
    const uint64_t hi = o ? ((a << o) | (b >> (64 - o))) : a;
    return (uint32_t)(hi >> (64 - L));
}

/* FP8 buckets, L=7 (decode_huffman.cu:268-371).  Differences from the shipped kernel, both stated
 * by the encoder: the ESC flag (bit 3 of the length nibble) is honoured by reading 16 raw bits
 * after the code (build_huffman.cu:220-225, 893-903), and elements map to (row, col) by true
 * div/mod (build_huffman.cu:838-839) so buckets narrower than k decode correctly. */
int orc_decode_fp8(const uint8_t* fp8, const uint64_t* bs, int64_t nwords, const uint16_t* syms, const uint8_t* lens,
                   const int32_t* bucket_table, const int32_t* col_start, const int32_t* col_len,
                   const int32_t* row_ofs, const int32_t* rows, const uint32_t* startbit, const int64_t* bit_base,
                   int64_t B, int64_t k, int64_t n, int64_t m, uint16_t* out) {
    (void)n;
#pragma omp parallel for collapse(2) schedule(dynamic, 64)
    for (int64_t bi = 0; bi < B; ++bi) {
        for (int64_t t = 0; t < k; ++t) {
            const int32_t row_a = row_ofs[bi];
            const int64_t row_count = (int64_t)row_ofs[bi + 1] - row_a;
            if (row_count <= 0) continue;
            const int64_t cs = col_start[bi], cl = col_len[bi];
            if (cl <= 0 || cs < 0 || cs + cl > m) continue;
            const int64_t total = row_count * cl;
            int64_t k_eff = k; if (total < k_eff) k_eff = total; if (k_eff < 1) k_eff = 1;
            if (t >= k_eff) continue;
            const int32_t* bt = bucket_table + bi * 256;
            int64_t bitpos = bit_base[bi] + (int64_t)startbit[bi * (k + 1) + t];
            for (int64_t e = t; e < total; e += k_eff) {
                const int64_t rr = e / cl, cc = e - rr * cl;
                const int64_t idx = (int64_t)rows[row_a + rr] * m + cs + cc;
                const int32_t gid = bt[fp8[idx]];
                if (gid < 0) { out[idx] = 0; continue; }
                const uint32_t p = peek_bits(bs, nwords, bitpos, 7);
                const uint8_t v = lens[(int64_t)gid * 64 + (p >> 1)];
                const uint8_t nib = (uint8_t)((v >> ((p & 1u) << 2)) & 0x0F);
                uint16_t sym = syms[(int64_t)gid * 128 + p];
                bitpos += nib & 7;
                if (nib & 8) { sym = (uint16_t)peek_bits(bs, nwords, bitpos, 16); bitpos += 16; }
                out[idx] = sym;
            }
        }
    }
    return 0;
}

/* AWQ int4 rectangular buckets, L=11 (decode_huffman.cu:415-494, element mapping by div/mod). */
int orc_decode_awq_bucket(const uint8_t* q, const uint64_t* bs, int64_t nwords, const uint16_t* syms, const uint8_t* lens,
                          const int32_t* bucket_table, const int32_t* col_start, const int32_t* col_len,
                          const int32_t* row_ofs, const int32_t* rows, const uint32_t* startbit, const int64_t* bit_base,
                          int64_t B, int64_t k, int64_t n, int64_t m, uint16_t* out) {
    (void)n;
#pragma omp parallel for collapse(2) schedule(dynamic, 256)
    for (int64_t bi = 0; bi < B; ++bi) {
        for (int64_t t = 0; t < k; ++t) {
            const int32_t row_a = row_ofs[bi];
            const int64_t row_count = (int64_t)row_ofs[bi + 1] - row_a;
            if (row_count <= 0) continue;
            const int64_t cs = col_start[bi], cl = col_len[bi];
            if (cl <= 0 || cs < 0 || cs + cl > m) continue;
            const int64_t total = row_count * cl;
            int64_t k_eff = k; if (total < k_eff) k_eff = total; if (k_eff < 1) k_eff = 1;
            if (t >= k_eff) continue;
            const int32_t* bt = bucket_table + bi * 16;
            int64_t bitpos = bit_base[bi] + (int64_t)startbit[bi * (k + 1) + t];
            for (int64_t e = t; e < total; e += k_eff) {
                const int64_t rr = e / cl, cc = e - rr * cl;
                const int64_t idx = (int64_t)rows[row_a + rr] * m + cs + cc;
                const int32_t gid = bt[q[idx] & 0x0F];
                const uint32_t p = peek_bits(bs, nwords, bitpos, 11);
                uint8_t nib = 0;
                if (gid >= 0) { const uint8_t v = lens[(int64_t)gid * 1024 + (p >> 1)]; nib = (uint8_t)((v >> ((p & 1u) << 2)) & 0x0F); }
                if (gid >= 0 && nib != 15) { out[idx] = syms[(int64_t)gid * 2048 + p]; bitpos += nib; }
                else { bitpos += 11; out[idx] = (uint16_t)peek_bits(bs, nwords, bitpos, 16); bitpos += 16; }
            }
        }
    }
    return 0;
}

/* AWQ int4 ragged buckets, L=11 (decode_huffman.cu:534-588). */
int orc_decode_awq_by_scale(const uint8_t* q, const uint64_t* bs, int64_t nwords, const uint16_t* syms, const uint8_t* lens,
                            const int32_t* bucket_table, const int32_t* group_ofs, const int32_t* group_rows,
                            const int32_t* group_col, const uint32_t* startbit, const int64_t* bit_base,
                            int64_t B, int64_t k, int64_t n, int64_t m, int64_t group_size, uint16_t* out) {
    (void)n;
#pragma omp parallel for collapse(2) schedule(dynamic, 64)
    for (int64_t bi = 0; bi < B; ++bi) {
        for (int64_t t = 0; t < k; ++t) {
            const int32_t ga = group_ofs[bi];
            const int64_t gcount = (int64_t)group_ofs[bi + 1] - ga;
            if (gcount <= 0 || group_size <= 0) continue;
            const int64_t total = gcount * group_size;
            int64_t k_eff = k; if (total < k_eff) k_eff = total; if (k_eff < 1) k_eff = 1;
            if (t >= k_eff) continue;
            const int32_t* bt = bucket_table + bi * 16;
            int64_t bitpos = bit_base[bi] + (int64_t)startbit[bi * (k + 1) + t];
            for (int64_t e = t; e < total; e += k_eff) {
                const int64_t gi = e / group_size, j = e - gi * group_size;
                const int64_t idx = (int64_t)group_rows[ga + gi] * m + group_col[ga + gi] + j;
                const int32_t gid = bt[q[idx] & 0x0F];
                const uint32_t p = peek_bits(bs, nwords, bitpos, 11);
                uint8_t nib = 0;
                if (gid >= 0) { const uint8_t v = lens[(int64_t)gid * 1024 + (p >> 1)]; nib = (uint8_t)((v >> ((p & 1u) << 2)) & 0x0F); }
                if (gid >= 0 && nib != 15) { out[idx] = syms[(int64_t)gid * 2048 + p]; bitpos += nib; }
                else { bitpos += 11; out[idx] = (uint16_t)peek_bits(bs, nwords, bitpos, 16); bitpos += 16; }
            }
        }
    }
    return 0;
}

/* AWQ shared-table chunks (decode_huffman_encode_only.cu:228-275).  Every stream is visited
 * (the shipped launch stops at 65535 streams); unvisited outputs stay as the caller left them. */
int orc_decode_awq_shared(const uint64_t* bs, int64_t nwords, const int16_t* syms, const uint8_t* nbits, int64_t table_size,
                          const int64_t* scale_bit_base, const uint32_t* chunk_startbit, const uint32_t* chunk_out_base,
                          const uint32_t* chunk_meta, const int32_t* chunk_scale_id, const int32_t* out_idx,
                          const int64_t* stream_ofs, const int32_t* stream_ids, int64_t num_streams,
                          int64_t out_len, int L, int16_t* out) {
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t s = 0; s < num_streams; ++s) {
        const int16_t* ts = syms + s * table_size;
        const uint8_t* tn = nbits + s * table_size;
        for (int64_t i = stream_ofs[s]; i < stream_ofs[s + 1]; ++i) {
            const int64_t chunk = stream_ids[i];
            const uint32_t take = chunk_meta[chunk] >> 8;
            int64_t bitpos = scale_bit_base[chunk_scale_id[chunk]] + (int64_t)chunk_startbit[chunk];
            const int64_t flat = chunk_out_base[chunk];
            for (uint32_t j = 0; j < take; ++j) {
                const uint32_t p = peek_bits(bs, nwords, bitpos, L);
                const uint8_t nb = tn[p];
                int16_t sym = ts[p];
                bitpos += nb & 0x7F;
                if (nb & 0x80) { sym = (int16_t)peek_bits(bs, nwords, bitpos, 16); bitpos += 16; }
                const int64_t pp = flat + j;
                if (pp >= 0 && pp < out_len) out[out_idx[pp]] = sym;
            }
        }
    }
    return 0;
}
