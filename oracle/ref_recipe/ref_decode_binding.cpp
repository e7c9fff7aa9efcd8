// Minimal Python binding of the reference's CUDA FP8 decode entry, used only as a second checker of this
// library's decoder on a B200 (on inputs the reference kernel handles correctly) and to time the
// reference kernel once for context.  The reference's own binding file cannot be compiled (it names
// symbols that exist nowhere), so this file declares just the one entry, whose definition is compiled
// unmodified from the reference source where it lies.  Nothing here is product code.
#include <torch/extension.h>

namespace huffman_cpp {
torch::Tensor huffman_decode_fp8_entry(torch::Tensor fp8_params_u8, torch::Tensor bitstream_u64, torch::Tensor decode_syms_u16,
                                       torch::Tensor decode_lens_u8, torch::Tensor bucket_table_i32,
                                       torch::Tensor bucket_col_start_i32, torch::Tensor bucket_col_len_i32,
                                       torch::Tensor bucket_row_offsets_i32, torch::Tensor row_indices_i32,
                                       torch::Tensor bucket_thread_startbit_u32, torch::Tensor bucket_bit_base_i64, int64_t n,
                                       int64_t m, int64_t max_len);
}  // namespace huffman_cpp

PYBIND11_MODULE(mpserve_ref_decode, m) {
    m.def("huffman_decode_fp8", &huffman_cpp::huffman_decode_fp8_entry);
}
