"""The CPU oracle against the golden fixtures produced by the reference's own encoder."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests._util import golden_names, has_esc_awq, has_esc_fp8


def _encode(g):
    p = g.params
    if g.kind == "fp8":
        return orc.build_fp8(g.bf16, g.ctx, g.scales, p["max_len"], p["threads_per_block"])
    if g.kind == "awq_bucket":
        return orc.build_awq_bucket(g.bf16, g.ctx, g.scales, p["max_len"], p["threads_per_block"])
    if g.kind == "awq_by_scale":
        return orc.build_awq_by_scale(g.bf16, g.ctx, g.scales, p["max_len"], p["threads"], p["group_cap"])
    if g.kind == "awq_shared":
        return orc.build_awq_shared(g.bf16, g.ctx, g.scales, p["max_len"])
    raise AssertionError(g.kind)


def _decode(g, art):
    n, m = g.bf16.shape
    if g.kind == "fp8":
        return orc.decode_fp8(g.ctx, art, n, m)
    if g.kind == "awq_bucket":
        return orc.decode_awq_bucket(g.ctx, art, n, m)
    if g.kind == "awq_by_scale":
        return orc.decode_awq_by_scale(g.ctx, art, n, m, int(art["shape_nmkg_i64"][3]))
    return orc.decode_awq_shared(art, n * m, g.params["max_len"]).view(np.uint16).reshape(n, m)


@pytest.mark.parametrize("name", golden_names())
def test_oracle_encoder_matches_reference_artifacts(golden_cases, name):
    g = golden_cases[name]
    g.check_artifacts(_encode(g))


@pytest.mark.parametrize("name", golden_names())
def test_oracle_decode_restores_bf16(golden_cases, name):
    g = golden_cases[name]
    art = _encode(g)
    np.testing.assert_array_equal(_decode(g, art), g.bf16)


def test_golden_esc_cases_really_escape(golden_cases):
    assert has_esc_fp8(_encode(golden_cases["fp8_esc_96x256_k128"]))
    assert has_esc_awq(_encode(golden_cases["awq_esc_96x256_k256_bucket"]))
    assert has_esc_awq(_encode(golden_cases["awq_esc_96x256_k256_byscale"]))
    sh = _encode(golden_cases["awq_esc_96x256_k256_shared"])
    assert bool((sh["decode_nbits_u8"] & 0x80).any())
    assert not has_esc_fp8(_encode(golden_cases["fp8_tensor_64x256_k256"]))
