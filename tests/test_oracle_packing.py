"""The CPU oracle against the vectors made by the reference's own Python packer
(tests/golden/make_packer_vectors.py -> packer_vectors.npz)."""
import numpy as np
import pytest

import oracle

CASES = ["gauss_k512", "gauss_k256", "edges_k256"]


@pytest.fixture(scope="module")
def vec(golden_dir):
    return np.load(golden_dir / "packer_vectors.npz")


@pytest.mark.parametrize("name", CASES)
def test_quantize_weights_matches_reference_packer(vec, name):
    packed, scales = oracle.quantize_weights(vec[f"{name}_w"])
    assert np.array_equal(scales.view(np.uint16), vec[f"{name}_scales"].view(np.uint16))
    assert np.array_equal(packed, vec[f"{name}_packed"])


@pytest.mark.parametrize("name", CASES)
def test_pack_unpack_round_trip_and_nibble_order(vec, name):
    packed = vec[f"{name}_packed"]
    q = oracle.unpack_nibbles(packed)
    assert q.min() >= 0 and q.max() <= 15
    assert np.array_equal(oracle.pack_nibbles(q), packed)
    # include/quant_primitives.cuh:28-31: low nibbles of the four bytes are elements 0..3,
    # high nibbles are elements 4..7 of the octet.
    lo = packed & 0x0F0F0F0F
    hi = (packed >> 4) & 0x0F0F0F0F
    q8 = q.reshape(q.shape[0], -1, 8)
    for j in range(4):
        assert np.array_equal((lo >> (8 * j)) & 0xFF, q8[..., j])
        assert np.array_equal((hi >> (8 * j)) & 0xFF, q8[..., 4 + j])


def test_edge_groups_have_expected_nibbles(vec):
    q = oracle.unpack_nibbles(vec["edges_k256_packed"])
    assert np.all(q[0, :128] == 8)    # zero group -> zero-point
    assert np.all(q[5, :128] == 15)
    assert np.all(q[6, :128] == 1)
    assert vec["edges_k256_scales"][0, 0] == 0
