/*
 * mpserve_b200.h -- C ABI of libmpserve_b200.so
 *
 * B200 (sm_100a) implementation of one path of MPServe: reconstructing BF16 weights from an FP8
 * (or AWQ-INT4) checkpoint plus its context-conditioned Huffman sidecar, and building that sidecar.
 * Plain pointers and sizes only; every pointer marked "device" must be a CUDA device pointer on the
 * current device.  All launches are asynchronous on `stream` (a cudaStream_t passed as void*).
 *
 * Return value of every int function: 0 on success, a negative MPS_ERR_* for bad arguments, or a
 * positive cudaError_t value when a CUDA call failed (text via mps_last_error()).
 *
 * Each entry point names the reference interface it replaces (file:line in the reference tree).
 */
#ifndef MPSERVE_B200_H
#define MPSERVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MPS_API __attribute__((visibility("default")))
#else
#define MPS_API
#endif

#define MPS_OK 0
#define MPS_ERR_INVALID (-1)      /* bad argument (reference: std::invalid_argument -> ValueError) */
#define MPS_ERR_UNSUPPORTED (-2)  /* valid but not implemented by this build                      */
#define MPS_ERR_WORKSPACE (-3)    /* workspace missing or too small                                */

/* Most sub-streams per bucket (k) this library builds and decodes.  The reference stops at 1024, the
 * size of the one thread block that decodes a bucket there (kernel/decode_huffman.cu:695,
 * kernel/build_huffman.cu:313); a sidecar written with more is the same format with a longer
 * bucket_thread_startbit row, and only this library reads it.  Finer sub-streams are what gives a lone
 * weight of few buckets enough independent chains to fill the GPU. */
#define MPS_MAX_SUBSTREAMS_REFERENCE 1024
#define MPS_MAX_SUBSTREAMS 8192

/* Library / device ---------------------------------------------------------------------------- */

/* Version of this ABI (bumped on incompatible change). */
MPS_API int mps_abi_version(void);

/* Text of the last error raised on the calling thread. */
MPS_API const char* mps_last_error(void);

/* Replaces MPServe_cuda.cuda_clock_rate_khz (kernel/wrapper.cpp:133-141): SM clock of the current
 * device in kHz, or a negative/positive error code as above. */
MPS_API int64_t mps_cuda_clock_rate_khz(void);

/* Bytes of zero-initialised device scratch every decode call needs (work-queue counters).  The
 * caller allocates it once per (device, stream), zero-fills it once, and passes it to every call;
 * the kernels leave it zeroed again.  Two calls that may overlap on the GPU need two workspaces. */
MPS_API size_t mps_workspace_bytes(void);

/* Every wait inside the decode kernels is bounded; a kernel whose wait ran out stops taking work and
 * records it in the workspace.  This call waits for the stream, reports whether any launch since the
 * last query gave up (*timed_out = 1; its outputs are then incomplete) and clears the record.
 * workspace == NULL asks about the library's own scratch, i.e. about mps_decode_fp8_noalloc calls (that
 * entry keeps the record across calls until it is read here).  The reference has no counterpart: its
 * kernels have no waits. */
MPS_API int mps_decode_status(void* workspace, size_t workspace_bytes, void* stream, int32_t* timed_out);

/* One compressed tensor (all pointers device) ---------------------------------------------------
 * mode 0: FP8 rectangular buckets, L=7, 256 contexts   (huffman_decode_fp8_entry)
 * mode 1: AWQ-INT4 rectangular buckets, L=11, 16 ctx   (huffman_decode_awq_int4_bucket_entry)
 * mode 2: AWQ-INT4 ragged buckets by exact scale       (huffman_decode_awq_int4_bucket_by_scale_entry)
 */
typedef struct mps_bucket_tensor {
    const uint8_t* ctx_bytes;          /* [n*m] fp8 byte or unpacked int4 code per element        */
    const uint64_t* bitstream;         /* [bitstream_words] MSB-first                             */
    int64_t bitstream_words;
    const uint16_t* decode_syms;       /* [num_tables, 2^L]                                       */
    const uint8_t* decode_lens;        /* [num_tables, 2^(L-1)] two 4-bit entries per byte        */
    int64_t num_tables;
    const int32_t* bucket_table;       /* [num_buckets, 256 or 16] context -> table id or -1      */
    const int32_t* bucket_col_start;   /* [num_buckets]            (modes 0,1)                    */
    const int32_t* bucket_col_len;     /* [num_buckets]            (modes 0,1)                    */
    const int32_t* bucket_row_offsets; /* [num_buckets+1] CSR      (modes 0,1; group offsets in 2) */
    const int32_t* row_indices;        /* [num_rows]               (modes 0,1; group rows in 2)    */
    const int32_t* group_col_start;    /* [num_rows]               (mode 2 only)                   */
    int64_t num_rows;                  /* length of row_indices / group arrays                    */
    const uint32_t* thread_startbit;   /* [num_buckets, k+1]                                      */
    const int64_t* bucket_bit_base;    /* [num_buckets+1]                                         */
    int64_t num_buckets;
    int32_t k;                         /* sub-streams per bucket                                  */
    int32_t group_size;                /* mode 2 only                                             */
    int32_t mode;
    int32_t reserved;
    int64_t n, m;
    uint16_t* out;                     /* [n*m] BF16 bit patterns                                 */
} mps_bucket_tensor;

/* Decode ---------------------------------------------------------------------------------------- */

/* Replaces huffman_cpp::huffman_decode_fp8_entry (kernel/decode_huffman.cu:591-758; Python name
 * huffman_decode_fp8, kernel/wrapper.cpp:457-503).  max_len must be 7.  Output is written to
 * `out_bf16` (caller-allocated [n,m] BF16).  Unlike the shipped kernel, the ESC flag of a length
 * nibble is honoured (16 raw bits follow the code, as the encoder writes them) and elements map to
 * rows/columns by true division, so buckets narrower than k decode correctly. */
MPS_API int mps_decode_fp8(const uint8_t* fp8_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                   const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                   const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                   const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                   const int32_t* row_indices_i32, int64_t num_row_indices,
                   const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                   int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                   uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces huffman_cpp::huffman_decode_awq_int4_bucket_entry (kernel/decode_huffman.cu:877-1017;
 * Python name huffman_decode_awq_int4_bucket, kernel/wrapper.cpp:324-369).  max_len must be 11. */
MPS_API int mps_decode_awq_int4_bucket(const uint8_t* int4_values_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                               const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                               const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                               const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                               const int32_t* row_indices_i32, int64_t num_row_indices,
                               const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                               int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                               uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces huffman_cpp::huffman_decode_awq_int4_bucket_by_scale_entry
 * (kernel/decode_huffman.cu:760-875; Python name huffman_decode_awq_int4_bucket_by_scale,
 * kernel/wrapper.cpp:371-416).  max_len must be 11. */
MPS_API int mps_decode_awq_int4_bucket_by_scale(const uint8_t* int4_values_u8, const uint64_t* bitstream_u64,
                                        int64_t bitstream_words, const uint16_t* decode_syms_u16,
                                        const uint8_t* decode_lens_u8, int64_t num_tables,
                                        const int32_t* bucket_table_i32, const int32_t* bucket_group_offsets_i32,
                                        const int32_t* group_rows_i32, const int32_t* group_col_start_i32,
                                        int64_t num_groups, const uint32_t* bucket_thread_startbit_u32,
                                        const int64_t* bucket_bit_base_i64, int64_t num_buckets, int32_t k,
                                        int64_t n, int64_t m, int64_t max_len, int64_t group_size,
                                        uint16_t* out_bf16, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces huffman_decode_cpp::huffman_decode_awq_shared_table_entry
 * (kernel/decode_huffman_encode_only.cu:279-383, 416-444; Python name
 * huffman_decode_awq_shared_table, kernel/wrapper.cpp:212-255).  Output int16 [out_len].  Every
 * stream is decoded (the shipped launch silently stops after 65535 streams). */
MPS_API int mps_decode_awq_shared_table(const uint64_t* bitstream_u64, int64_t bitstream_words,
                                const int16_t* decode_syms_i16, const uint8_t* decode_nbits_u8,
                                int64_t num_streams, const int64_t* scale_bit_base_i64, int64_t num_scales_plus1,
                                const uint32_t* chunk_startbit_rel_u32, const uint32_t* chunk_out_base_u32,
                                const uint32_t* chunk_meta_u32, const int32_t* chunk_scale_id_i32, int64_t num_chunks,
                                const int32_t* out_idx_i32, const int64_t* stream_chunk_ofs_i64,
                                const int32_t* stream_chunk_ids_i32, int64_t out_len, int64_t max_len,
                                int16_t* out_i16, void* stream);

/* No counterpart in the reference.  Same decode as mps_decode_fp8 for callers that must not allocate
 * device memory and therefore cannot supply a workspace: code running inside another framework's
 * memory pool or under a fixed memory budget, a plugin loaded into a process that forbids cudaMalloc
 * after start-up, a real-time loop.  The work-queue counters live in a 256-byte array that is part of
 * this library's device image (every GPU that loads the library holds it until the process exits);
 * the call itself allocates and frees nothing.
 *  - Limit: at most MPS_NOALLOC_MAX_BUCKETS buckets per call; more is rejected with MPS_ERR_INVALID.
 *  - The first call on a device looks the array's device address up (once per device); make that first
 *    call outside any stream capture.
 *  - All calls share the one array: calls whose kernels may overlap on the GPU (different streams,
 *    no ordering between them) race on it.  Calls on one stream, or otherwise ordered, are fine. */
#define MPS_NOALLOC_MAX_BUCKETS (1 << 20)
MPS_API int mps_decode_fp8_noalloc(const uint8_t* fp8_u8, const uint64_t* bitstream_u64, int64_t bitstream_words,
                                   const uint16_t* decode_syms_u16, const uint8_t* decode_lens_u8, int64_t num_tables,
                                   const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                                   const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                                   const int32_t* row_indices_i32, int64_t num_row_indices,
                                   const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                                   int64_t num_buckets, int32_t k, int64_t n, int64_t m, int64_t max_len,
                                   uint16_t* out_bf16, void* stream);

/* Many tensors in one launch (whole-model decompression).  `tensors_dev` is a DEVICE array of
 * `count` descriptors; `item_prefix_dev` a DEVICE array of count+1 int64 work-item prefix sums as
 * returned by mps_bucket_batch_plan for the same descriptors.  No reference counterpart: the
 * reference launches one kernel per weight (scripts/mpserve_vllm_fp8_huffman.py:526-543). */
MPS_API int mps_bucket_batch_plan(const mps_bucket_tensor* tensors_host, int count, int64_t* item_prefix_host,
                          int32_t* threads_out, int32_t* chains_out);
/* One tensor from a HOST descriptor (device pointers inside), any mode: what the per-format entries
 * above do after packing their arguments.  A plan gives zero work items to tensors made of tiny
 * buckets (item_prefix[i+1] == item_prefix[i]); those are decoded with this call instead, by a
 * kernel that reads the sidecar's tables in place.  No reference counterpart. */
MPS_API int mps_decode_bucket_tensor(const mps_bucket_tensor* tensor_host, void* workspace, size_t workspace_bytes,
                                     void* stream);
MPS_API int mps_decode_bucket_batch(const mps_bucket_tensor* tensors_dev, const int64_t* item_prefix_dev, int count,
                            int64_t total_items, int32_t threads, int32_t chains, int32_t mode,
                            void* workspace, size_t workspace_bytes, void* stream);

/* Self-test of the bounded waits, for bring-up on a new machine and for the test-suite; no counterpart in
 * the reference.  Decodes one tensor (through the persistent kernel, whatever its size) with the context
 * bytes of ONE block of steps deliberately never copied: block `stall_block` (0-based, counted per CTA) is
 * announced to the decoding warps but its bytes do not come.  Their wait gives up after `polls` polls,
 * the CTA stops taking work, waits (bounded again) for the copies it still has in flight and returns;
 * mps_decode_status then reports 1.  Nothing hangs or faults; the output is incomplete by design. */
MPS_API int mps_selftest_stalled_decode(const mps_bucket_tensor* tensor_host, int32_t stall_block, uint32_t polls,
                                        void* workspace, size_t workspace_bytes, void* stream);


/* Sidecar builder -------------------------------------------------------------------------------
 * Together these replace huffman_cpp::huffman_build_fp8_decode_tables_entry
 * (kernel/build_huffman.cu:292-969; Python name huffman_build_fp8_decode_tables,
 * kernel/wrapper.cpp:419-454) and huffman_build_awq_int4_bucket_decode_tables_entry
 * (kernel/build_huffman.cu:1582-2126; wrapper.cpp:258-288).  All tensors are DEVICE pointers; the
 * produced artifacts are byte-identical to the reference's.  The caller allocates outputs between
 * the steps, whose sizes each step returns:
 *   analyze      -> number of tables G          then allocate decode_syms [G,2^L], decode_lens [G,2^(L-1)]
 *   codebooks    fills the tables and table_scale / table_ctx [G]
 *   bucket_table fills bucket_table [B, 256|16] from the buckets' scales (bucket lists are built by
 *                the caller from the scale tensor: build_huffman.cu:611-696)
 *   rect_layout  fills bucket_thread_startbit [B,k+1] and bucket_bit_base [B+1], returns total bits; leaves the code
 *                of every element in the workspace for the next step
 *   rect_emit    fills bitstream_u64 [(total_bits+63)/64]; must follow rect_layout for the same buckets, with
 *                nothing else using the workspace in between
 * variant: 0 FP8 (context = fp8 byte), 1 AWQ-INT4 rectangular buckets (context = int4 code),
 *          3 AWQ-INT4 shared tables (analysis only; continue with the mps_build_shared_* calls below),
 *          2 AWQ-INT4 ragged buckets by exact scale (huffman_build_awq_int4_bucket_decode_tables_by_scale_entry,
 *            kernel/build_huffman.cu:1074-1580; wrapper.cpp:290-321): pass bucket_col_len = NULL, the groups'
 *            rows as row_indices, their column starts as bucket_col_start and the group offsets as
 *            bucket_row_offsets to rect_layout / rect_emit; the group size is m for scalar / per-row scales,
 *            sb1 for block scales.
 * scale_mode: 0 scalar, 1 per row [n], 2 two-dimensional blocks [n/sb0, nb1] of sb0 x sb1 elements. */
typedef struct mps_build_state { unsigned char opaque[256]; } mps_build_state;

MPS_API size_t mps_build_workspace_bytes(int64_t numel, int64_t substreams);
MPS_API int mps_build_analyze(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                              const uint16_t* scales_u16, int32_t scale_mode, int64_t nb1, int64_t sb0, int64_t sb1,
                              int64_t n, int64_t m, int32_t variant, int64_t max_len, void* workspace,
                              size_t workspace_bytes, void* stream, int64_t* num_tables_out, int64_t* num_items_out);
MPS_API int mps_build_codebooks(mps_build_state* state, uint16_t* decode_syms_u16, uint8_t* decode_lens_u8,
                                uint16_t* table_scale_u16, uint16_t* table_ctx_u16, void* stream);
MPS_API int mps_build_bucket_table(mps_build_state* state, const uint16_t* bucket_scale_u16, int64_t num_buckets,
                                   int32_t* bucket_table_i32, void* stream);
/* bucket_U / bucket_unique_gid / bucket_fp8_uidx of the FP8 builder (build_huffman.cu:748-783) */
MPS_API int mps_build_bucket_unique(const int32_t* bucket_table_i32, int64_t num_buckets, int32_t* bucket_U_i32,
                                    int32_t* bucket_unique_gid_i32, int16_t* bucket_fp8_uidx_i16, void* stream);
MPS_API int mps_build_rect_layout(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                                  const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                                  const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                                  const int32_t* row_indices_i32, int64_t num_buckets, int32_t k,
                                  uint32_t* bucket_thread_startbit_u32, int64_t* bucket_bit_base_i64, void* stream,
                                  int64_t* total_bits_out);
MPS_API int mps_build_rect_emit(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* ctx_bytes,
                                const int32_t* bucket_table_i32, const int32_t* bucket_col_start_i32,
                                const int32_t* bucket_col_len_i32, const int32_t* bucket_row_offsets_i32,
                                const int32_t* row_indices_i32, int64_t num_buckets, int32_t k,
                                const uint32_t* bucket_thread_startbit_u32, const int64_t* bucket_bit_base_i64,
                                uint64_t* bitstream_u64, int64_t bitstream_words, void* stream);

/* Shared-table sidecar (huffman_build_awq_decode_tables_entry, build_huffman.cu:2157-2633):
 * mps_build_analyze with variant 3, then these three.  sid_lut_i32: DEVICE int32[65536], the dense id
 * of every scale value that occurs (ascending by value), -1 elsewhere; num_scales = S.
 *   codebooks: decode_syms_i16 / decode_nbits_u8 [S*16, 2^max_len], one table per (scale id, int4 code)
 *              stream whether it occurs or not; whole-byte lengths, bit 7 marks an ESC slot (:2311-2428)
 *   layout:    scale_bit_base_i64 [S+1] (device) and, returned to the host, the chunk count and the total
 *              bits; chunks are runs of <= 255 consecutive elements of one stream (:2434-2537)
 *   emit:      bitstream (every scale's bits in flat element order, 64-bit aligned), the four chunk
 *              arrays [C], out_idx_i32 [numel] (identity, :2586-2588), the stream -> chunk CSR (:2590-2610) */
MPS_API int mps_build_shared_codebooks(mps_build_state* state, const int32_t* sid_lut_i32, int64_t num_scales,
                                       int16_t* decode_syms_i16, uint8_t* decode_nbits_u8, void* stream);
MPS_API int mps_build_shared_layout(mps_build_state* state, const uint16_t* bf16_bits, const uint8_t* int4_u8,
                                    const uint16_t* scales_u16, int32_t scale_mode, int64_t nb1, int64_t sb0, int64_t sb1,
                                    const int32_t* sid_lut_i32, int64_t* scale_bit_base_i64, void* stream,
                                    int64_t* num_chunks_out, int64_t* total_bits_out);
MPS_API int mps_build_shared_emit(mps_build_state* state, const uint16_t* bf16_bits, const int64_t* scale_bit_base_i64,
                                  uint64_t* bitstream_u64, int64_t bitstream_words, uint32_t* chunk_startbit_rel_u32,
                                  uint32_t* chunk_out_base_u32, uint32_t* chunk_meta_u32, int32_t* chunk_scale_id_i32,
                                  int32_t* out_idx_i32, int64_t* stream_chunk_ofs_i64, int32_t* stream_chunk_ids_i32,
                                  void* stream);

/* Checksum of a decoded tensor: sum of the 16-bit patterns (mod 2^64) and an XOR fold of
 * (pattern * (index+1)) -- what ranks all-reduce after a sharded decode.  result_dev: device
 * uint64[2], accumulated into (zero it first). */
MPS_API int mps_checksum_u16(const uint16_t* data_dev, int64_t count, uint64_t* result_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MPSERVE_B200_H */
