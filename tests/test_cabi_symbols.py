"""The C-ABI library loads here (no GPU) and exports every symbol its header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def built_lib():
    from mpserve_b200 import build

    return build.build()


def _declared():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"MPS_API\s+[\w\s\*]+?\b(mps_\w+)\s*\(", h.read_text()))
    return sorted(names)


def test_header_declares_entry_points():
    names = _declared()
    for must in ("mps_decode_fp8", "mps_decode_awq_int4_bucket", "mps_decode_awq_int4_bucket_by_scale",
                 "mps_decode_awq_shared_table", "mps_decode_bucket_batch", "mps_decode_bucket_tensor", "mps_decode_status", "mps_checksum_u16"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(str(built_lib))
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_binding_prototypes_cover_the_header(built_lib):
    from mpserve_b200 import _lib

    assert set(_lib.exported_names()) == set(_declared())
    lib = _lib.load()
    assert lib.mps_abi_version() >= 1
    assert lib.mps_workspace_bytes() >= 8


def test_struct_layout_matches_header():
    from mpserve_b200 import _lib

    # 16 pointers/int64 fields + 4 int32 + n,m + out
    assert ctypes.sizeof(_lib.BucketTensor) == 8 * 16 + 4 * 4 + 8 * 3


def test_drop_in_module_surface():
    import MPServe_cuda

    for name in ("cuda_clock_rate_khz", "huffman_build_fp8_decode_tables", "huffman_decode_fp8",
                 "huffman_build_awq_int4_bucket_decode_tables", "huffman_decode_awq_int4_bucket",
                 "huffman_build_awq_int4_bucket_decode_tables_by_scale", "huffman_decode_awq_int4_bucket_by_scale",
                 "huffman_build_awq_decode_tables", "huffman_decode_awq_shared_table"):
        assert callable(getattr(MPServe_cuda, name))
    with pytest.raises(NotImplementedError):
        MPServe_cuda.build_trie()


def test_decode_rejects_cpu_tensors():
    import torch

    import MPServe_cuda

    z = torch.zeros(4, dtype=torch.uint8)
    with pytest.raises(ValueError, match="must be a CUDA tensor"):
        MPServe_cuda.huffman_decode_fp8(z, z, z, z, z, z, z, z, z, z, z, 2, 2, 7)
