"""Pins the CPU oracle to the reference engine itself: tests/golden/refkernel_vectors.npz holds
outputs of the reference's own CUDA kernels (compiled from the reference sources for sm_100a and
run on a B200 by tests/golden/make_refkernel_vectors.py) on small seeded inputs.

"ieee" is the reference source as written; "fastmath" adds the reference's --use_fast_math build
flag, which replaces the two IEEE divisions of the Q8_1 quantiser by approximate ones.  The
oracle's canonical behaviour is the source as written, so it must agree with "ieee" bit for bit
on all integer outputs; against "fastmath" the quantised bytes still agree on these inputs and
only group scales may differ in the last bit (counted and bounded below).
"""
import numpy as np
import pytest

import oracle
from tests import util


@pytest.fixture(scope="module")
def v(golden_dir):
    return np.load(golden_dir / "refkernel_vectors.npz")


def test_q8_1_bit_exact_against_reference_source_build(v):
    q8, sc, s8 = oracle.quantize_q8_1(v["quant_x"])
    assert np.array_equal(q8, v["ieee_quant_q8"])
    assert np.array_equal(sc.view(np.uint32), v["ieee_quant_scale"].view(np.uint32))
    assert np.array_equal(s8, v["ieee_quant_sum8"])


def test_q8_1_against_reference_fastmath_build(v):
    q8, sc, s8 = oracle.quantize_q8_1(v["quant_x"])
    assert np.mean(q8 != v["fastmath_quant_q8"]) <= 0.01
    rel = np.abs(sc - v["fastmath_quant_scale"]) / sc
    assert rel.max() <= 2.0 ** -21          # approximate division: a few ulp at most
    assert np.mean(sc.view(np.uint32) != v["fastmath_quant_scale"].view(np.uint32)) <= 0.25


@pytest.mark.parametrize("flavour", ["ieee", "fastmath"])
def test_gemv_outputs_of_reference_kernels(v, flavour):
    f = flavour
    # W4A8 uint4 kernel with residual, evaluated on the Q8_1 arrays the reference itself produced
    y64, y16 = oracle.gemv_q8(v["gemv_w"], v["gemv_s"], v[f"{f}_gemv_q8"], v[f"{f}_gemv_xscale"],
                              residual=v["gemv_res"])
    rep = util.assert_fp16_close(v[f"{f}_gemv_y"], y64, what="ref gemv")
    assert rep["max_ulp"] <= 0.75
    assert np.mean(y16.view(np.uint16) == v[f"{f}_gemv_y"].view(np.uint16)) >= 0.98
    # SwiGLU, W4A8 and fp16-input entry points
    q8h, sch, _ = oracle.quantize_q8_1(v["gemv_x"][:512])
    s64, _ = oracle.gemv_q8(v["swiglu_w"], v["swiglu_s"], q8h, sch, swiglu=True)
    for key in ("swiglu_y_w4a8", "swiglu_y_w4a16"):
        rep = util.assert_fp16_close(v[f"{f}_{key}"], s64, what=key)
        assert rep["max_ulp"] <= 1.0
    # fused QKV
    q8q, scq, _ = oracle.quantize_q8_1(v["qkv_x"])
    for i in range(3):
        q64, _ = oracle.gemv_q8(v[f"qkv_w{i}"], v[f"qkv_s{i}"], q8q, scq)
        rep = util.assert_fp16_close(v[f"{f}_qkv_y{i}"], q64, what=f"qkv{i}")
        assert rep["max_ulp"] <= 0.75


def test_fp16_input_gemv_of_reference_source_build(v):
    q8, sc, _ = oracle.quantize_q8_1(v["gemv2_x"])
    y64, _ = oracle.gemv_q8(v["gemv2_w"], v["gemv2_s"], q8, sc)
    rep = util.assert_fp16_close(v["ieee_gemv2_y"], y64, what="ref gemv fp16-in")
    assert rep["max_ulp"] <= 0.75


@pytest.mark.parametrize("flavour", ["ieee", "fastmath"])
def test_prefill_outputs_of_reference_kernels(v, flavour):
    f = flavour
    M, N = v["prefill_x"].shape[0], v["gemv_w"].shape[0]
    m_idx = np.arange(M, dtype=np.int32)
    o64, o16 = oracle.gemm_prefill(v["gemv_w"], v["gemv_s"], v["prefill_x"], m_idx, np.arange(N, dtype=np.int32),
                                   residual=v["prefill_res"])
    # fp16(acc) + residual in fp16: the oracle restates that double rounding -> identical bits
    assert np.mean(o16.view(np.uint16) == v[f"{f}_prefill_y"].view(np.uint16)) >= 0.99
    for i in range(3):
        n = v[f"qkv_w{i}"].shape[0]
        q64, _ = oracle.gemm_prefill(v[f"qkv_w{i}"], v[f"qkv_s{i}"], v["prefill_qkv_x"], m_idx,
                                     np.arange(n, dtype=np.int32))
        rep = util.assert_fp16_close(v[f"{f}_prefill_qkv_y{i}"], q64, what=f"prefill qkv{i}")
        assert rep["max_ulp"] <= 1.0
    I = v["swiglu_w"].shape[0] // 2
    s64, _ = oracle.gemm_prefill(v["swiglu_w"], v["swiglu_s"], np.ascontiguousarray(v["prefill_x"][:, :512]), m_idx,
                                 np.arange(I, dtype=np.int32), swiglu=True)
    rep = util.assert_fp16_close(v[f"{f}_prefill_swiglu_y"], s64, what="prefill swiglu")
    assert rep["max_ulp"] <= 1.0


@pytest.mark.parametrize("flavour", ["ieee", "fastmath"])
def test_rmsnorm_q8_1_of_reference_kernels(v, flavour):
    f = flavour
    y, _ = oracle.rmsnorm(v["norm_x"], v["norm_gamma"])
    assert np.mean(y.view(np.uint16) == v[f"{f}_norm_y"].view(np.uint16)) >= 0.999
    q8, sc, _ = oracle.quantize_q8_1(v[f"{f}_norm_y"])
    assert np.mean(q8 != v[f"{f}_norm_q8"]) <= 0.01
    if flavour == "ieee":
        assert np.array_equal(q8, v["ieee_norm_q8"])
        assert np.array_equal(sc.view(np.uint32), v["ieee_norm_scale"].view(np.uint32))
