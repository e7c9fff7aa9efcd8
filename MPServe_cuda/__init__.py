"""Drop-in stand-in for the reference's ``MPServe_cuda`` extension module.

``import MPServe_cuda`` (scripts/mpserve_vllm_fp8_huffman.py:72-77,
scripts/compress_llm_fp8_huffman.py:236) resolves to this package when the repository root is on
``sys.path``; every Huffman entry point of kernel/wrapper.cpp:182-503 is here under the same name.
The seventeen legacy "trie" names that the reference binds at kernel/wrapper.cpp:142-179 have no
implementation anywhere in the reference tree; they exist here only to raise.
"""
from mpserve_b200.api import (  # noqa: F401
    cuda_clock_rate_khz,
    huffman_build_awq_decode_tables,
    huffman_build_awq_int4_bucket_decode_tables,
    huffman_build_awq_int4_bucket_decode_tables_by_scale,
    huffman_build_fp8_decode_tables,
    huffman_decode_awq_int4_bucket,
    huffman_decode_awq_int4_bucket_by_scale,
    huffman_decode_awq_shared_table,
    huffman_decode_fp8,
)

_LEGACY = (
    "init_cuda", "cleanup_cuda", "build_trie_AWQ", "build_trie", "query_trie", "free_trie", "get_trie_count",
    "get_tot_path_length", "save_trie_collection", "load_trie_collection", "save_trie_collection_awq",
    "load_trie_collection_awq", "load_bf16_from_int8", "dequantize_awq", "build_trie_AWQ_to_FP8",
    "save_trie_collection_awq_to_fp8", "load_trie_collection_awq_to_fp8",
)


def _legacy(name):
    def _raise(*args, **kwargs):
        raise NotImplementedError(f"MPServe_cuda.{name}: the legacy trie codec has no implementation in the reference")

    _raise.__name__ = name
    return _raise


for _n in _LEGACY:
    globals()[_n] = _legacy(_n)
del _n
