// AWQ "shared-table" sidecar: chunks of <=255 consecutive elements that share one (scale, qv)
// stream; every stream has a dense 2^L lookup table (int16 symbol + uint8 length, bit 7 = ESC).
//
// On random weights a chunk holds 1.1 elements on average, so the work is a gather: one thread per
// chunk position in the stream->chunk index, table entries read straight from global memory (L2),
// no shared-memory staging (a 6 KB table per ~200 symbols would cost more than it saves).  The
// stream of a position is found by binary search in stream_chunk_ofs, which keeps the semantics of
// the reference kernel (the table is chosen by the stream that lists the chunk) while covering
// every stream -- the reference launch stops at 65535 blocks.
#include "mps_common.cuh"

namespace mps {

__device__ __forceinline__ uint32_t peek_bits_global(const uint64_t* __restrict__ bs, long long nwords, long long bitpos,
                                                     int nbits) {
    const long long w = bitpos >> 6;
    const int o = (int)(bitpos & 63);
    const uint64_t a = (w >= 0 && w < nwords) ? __ldg(bs + w) : 0ull;
    const uint64_t b = (w + 1 >= 0 && w + 1 < nwords) ? __ldg(bs + w + 1) : 0ull;
    const uint64_t hi = o ? ((a << o) | (b >> (64 - o))) : a;
    return (uint32_t)(hi >> (64 - nbits));
}

__global__ void __launch_bounds__(256)
shared_table_decode_kernel(const uint64_t* __restrict__ bs, long long nwords, const int16_t* __restrict__ syms,
                           const uint8_t* __restrict__ nbits, long long table_size, long long num_streams,
                           const long long* __restrict__ scale_bit_base, long long num_scales,
                           const uint32_t* __restrict__ chunk_startbit, const uint32_t* __restrict__ chunk_out_base,
                           const uint32_t* __restrict__ chunk_meta, const int32_t* __restrict__ chunk_scale_id,
                           long long num_chunks, const int32_t* __restrict__ out_idx,
                           const long long* __restrict__ stream_ofs, const int32_t* __restrict__ stream_ids,
                           long long out_len, int L, int16_t* __restrict__ out) {
    const long long npos = stream_ofs[num_streams] < num_chunks ? stream_ofs[num_streams] : num_chunks;
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < npos; p += (long long)gridDim.x * blockDim.x) {
        // stream s with stream_ofs[s] <= p < stream_ofs[s+1]
        long long lo = 0, hi = num_streams;
        while (hi - lo > 1) {
            const long long mid = (lo + hi) >> 1;
            if (__ldg(stream_ofs + mid) <= p) lo = mid; else hi = mid;
        }
        const long long s = lo;
        const long long chunk = stream_ids[p];
        if (chunk < 0 || chunk >= num_chunks) continue;
        const int sid = chunk_scale_id[chunk];
        if (sid < 0 || sid >= num_scales) continue;
        const uint32_t take = chunk_meta[chunk] >> 8;
        long long bitpos = scale_bit_base[sid] + (long long)chunk_startbit[chunk];
        const long long flat = chunk_out_base[chunk];
        const int16_t* ts = syms + s * table_size;
        const uint8_t* tn = nbits + s * table_size;
        for (uint32_t j = 0; j < take; ++j) {
            const uint32_t t = peek_bits_global(bs, nwords, bitpos, L);
            const uint32_t nb = __ldg(tn + t);
            int16_t sym = __ldg(ts + t);
            bitpos += nb & 0x7Fu;
            if (nb & 0x80u) {
                sym = (int16_t)peek_bits_global(bs, nwords, bitpos, 16);
                bitpos += 16;
            }
            const long long q = flat + j;
            if (q < out_len) {
                const long long dst = out_idx[q];
                if (dst >= 0 && dst < out_len) out[dst] = sym;
            }
        }
    }
}

}  // namespace mps

using namespace mps;

extern "C" int mps_decode_awq_shared_table(const uint64_t* bitstream_u64, int64_t bitstream_words,
                                           const int16_t* decode_syms_i16, const uint8_t* decode_nbits_u8,
                                           int64_t num_streams, const int64_t* scale_bit_base_i64, int64_t num_scales_plus1,
                                           const uint32_t* chunk_startbit_rel_u32, const uint32_t* chunk_out_base_u32,
                                           const uint32_t* chunk_meta_u32, const int32_t* chunk_scale_id_i32,
                                           int64_t num_chunks, const int32_t* out_idx_i32,
                                           const int64_t* stream_chunk_ofs_i64, const int32_t* stream_chunk_ids_i32,
                                           int64_t out_len, int64_t max_len, int16_t* out_i16, void* stream) {
    if (max_len <= 0 || max_len > 20) { set_error("max_len must be in (0,20]"); return MPS_ERR_INVALID; }
    if (num_streams < 0 || num_chunks < 0 || out_len < 0 || num_scales_plus1 < 1 || bitstream_words < 0) {
        set_error("mps_decode_awq_shared_table: negative size");
        return MPS_ERR_INVALID;
    }
    if (num_chunks == 0 || num_streams == 0 || out_len == 0) return MPS_OK;
    if (!bitstream_u64 || !decode_syms_i16 || !decode_nbits_u8 || !scale_bit_base_i64 || !chunk_startbit_rel_u32 ||
        !chunk_out_base_u32 || !chunk_meta_u32 || !chunk_scale_id_i32 || !out_idx_i32 || !stream_chunk_ofs_i64 ||
        !stream_chunk_ids_i32 || !out_i16) {
        set_error("mps_decode_awq_shared_table: null device pointer");
        return MPS_ERR_INVALID;
    }
    const int threads = 256;
    long long blocks = (num_chunks + threads - 1) / threads;
    if (blocks > 148LL * 64) blocks = 148LL * 64;
    shared_table_decode_kernel<<<(int)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        bitstream_u64, bitstream_words, decode_syms_i16, decode_nbits_u8, 1LL << max_len, num_streams,
        reinterpret_cast<const long long*>(scale_bit_base_i64), num_scales_plus1 - 1, chunk_startbit_rel_u32,
        chunk_out_base_u32, chunk_meta_u32, chunk_scale_id_i32, num_chunks, out_idx_i32,
        reinterpret_cast<const long long*>(stream_chunk_ofs_i64), stream_chunk_ids_i32, out_len, (int)max_len, out_i16);
    MPS_CUDA_TRY(cudaGetLastError());
    return MPS_OK;
}
