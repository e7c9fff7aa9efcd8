// Minimal Python binding of the reference's four CPU encoder entry points, used only to pin the
// oracle (byte-for-byte artifact comparison) and as the timed "reference" CPU encode baseline.
// The reference's own binding file cannot be compiled (it names symbols that exist nowhere), so
// this file declares just the encoder entries, whose definitions are compiled from the reference
// sources where they lie.  Nothing here is product code.
#include <torch/extension.h>
#include <tuple>

namespace huffman_cpp {
using T = torch::Tensor;
std::tuple<T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T, T>
huffman_build_fp8_decode_tables_entry(T bf16_params, T fp8_params, T scales, int64_t max_len, int64_t threads_per_block);
std::tuple<T, T, T, T, T, T, T, T, T, T, T, T, T, T>
huffman_build_awq_int4_bucket_decode_tables_entry(T bf16_params, T int4_values_u8, T scales_u16, int64_t max_len,
                                                  int64_t threads_per_block);
std::tuple<T, T, T, T, T, T, T, T, T, T, T, T, T>
huffman_build_awq_int4_bucket_decode_tables_by_scale_entry(T bf16_values, T int4_values, T scales_u16, int64_t max_len,
                                                           int64_t threads, int64_t group_cap);
std::tuple<T, T, T, T, T, T, T, T, T, T, T, T>
huffman_build_awq_decode_tables_entry(T bf16_params, T int4_values_u8, T scales_u16, int64_t max_len);
}  // namespace huffman_cpp

template <typename Tup, size_t... I>
static pybind11::list to_list(const Tup& t, std::index_sequence<I...>) {
    pybind11::list l;
    (l.append(std::get<I>(t)), ...);
    return l;
}
template <typename Tup>
static pybind11::list to_list(const Tup& t) {
    return to_list(t, std::make_index_sequence<std::tuple_size<Tup>::value>{});
}

PYBIND11_MODULE(mpserve_ref_build, m) {
    m.def("build_fp8", [](torch::Tensor a, torch::Tensor b, torch::Tensor c, int64_t L, int64_t k) {
        return to_list(huffman_cpp::huffman_build_fp8_decode_tables_entry(a, b, c, L, k));
    });
    m.def("build_awq_bucket", [](torch::Tensor a, torch::Tensor b, torch::Tensor c, int64_t L, int64_t k) {
        return to_list(huffman_cpp::huffman_build_awq_int4_bucket_decode_tables_entry(a, b, c, L, k));
    });
    m.def("build_awq_by_scale", [](torch::Tensor a, torch::Tensor b, torch::Tensor c, int64_t L, int64_t k, int64_t cap) {
        return to_list(huffman_cpp::huffman_build_awq_int4_bucket_decode_tables_by_scale_entry(a, b, c, L, k, cap));
    });
    m.def("build_awq_shared", [](torch::Tensor a, torch::Tensor b, torch::Tensor c, int64_t L) {
        return to_list(huffman_cpp::huffman_build_awq_decode_tables_entry(a, b, c, L));
    });
}
