"""CPU checks of the oracle's arithmetic against independent numpy restatements and against
the reference's packed-weight vectors (tests/golden/packer_vectors.npz)."""
import numpy as np
import pytest

import oracle


def _np_q8_1(x16, half_away=False):
    x = x16.astype(np.float32).reshape(-1, 128)
    d = np.maximum(np.abs(x).max(axis=1) / np.float32(127.0), np.float32(1e-8)).astype(np.float32)
    inv = (np.float32(1.0) / d).astype(np.float32)
    t = (x * inv[:, None]).astype(np.float32)
    q = np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5))) if half_away else np.rint(t)
    q = np.clip(q, -127, 127).astype(np.int8)
    s8 = -8 * q.reshape(-1, 8).astype(np.int32).sum(axis=1)
    return q.reshape(-1), d, s8


@pytest.mark.parametrize("n", [128, 1536, 8960])
def test_q8_1_against_numpy(n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float16)
    x[:5] = [0.0, 65504.0, -65504.0, 6e-8, -6e-8]
    for mode, ha in ((oracle.ROUND_HALF_EVEN, False), (oracle.ROUND_HALF_AWAY, True)):
        q8, sc, s8 = oracle.quantize_q8_1(x, mode)
        rq, rd, rs = _np_q8_1(x, ha)
        assert np.array_equal(q8, rq) and np.array_equal(sc, rd) and np.array_equal(s8, rs)


def test_q8_1_zero_group_and_tie_rounding():
    x = np.zeros(256, dtype=np.float16)
    x[128] = 127.0
    x[129] = 0.5     # x/d = 0.5 exactly: half-even -> 0, half-away -> 1
    x[130] = 1.5     # -> 2 both ways
    x[131] = 2.5     # half-even -> 2, half-away -> 3
    q8, sc, s8 = oracle.quantize_q8_1(x)
    assert sc[0] == np.float32(1e-8) and not q8[:128].any() and not s8[:16].any()
    assert sc[1] == 1.0 and list(q8[128:132]) == [127, 0, 2, 2]
    q8a, _, _ = oracle.quantize_q8_1(x, oracle.ROUND_HALF_AWAY)
    assert list(q8a[128:132]) == [127, 1, 2, 3]
    assert s8[16] == -8 * (127 + 0 + 2 + 2)


def test_group_dots_and_gemv_against_numpy(golden_dir):
    vec = np.load(golden_dir / "packer_vectors.npz")
    packed, scales = vec["gauss_k512_packed"], vec["gauss_k512_scales"]
    N, K = packed.shape[0], packed.shape[1] * 8
    rng = np.random.default_rng(3)
    x = rng.standard_normal(K).astype(np.float16)
    q8, xs, _ = oracle.quantize_q8_1(x)
    q = oracle.unpack_nibbles(packed).astype(np.int32) - 8
    D = (q.reshape(N, -1, 128) * q8.astype(np.int32).reshape(1, -1, 128)).sum(axis=2)
    assert np.array_equal(oracle.group_dots(packed, q8, threads=3), D)
    factor = scales.astype(np.float32) * xs[None, :]
    y = (D.astype(np.float64) * factor.astype(np.float64)).sum(axis=1)
    res = rng.standard_normal(N).astype(np.float16)
    y64, y16 = oracle.gemv_q8(packed, scales, q8, xs, residual=res, threads=2)
    assert np.allclose(y64, y + res.astype(np.float64), rtol=1e-13, atol=1e-13)
    assert np.array_equal(y16, (y + res.astype(np.float64)).astype(np.float32).astype(np.float16))
    # SwiGLU pairing: rows 2i / 2i+1
    g64, _ = oracle.gemv_q8(packed, scales, q8, xs, swiglu=True)
    assert np.allclose(g64, y[0::2] / (1 + np.exp(-y[0::2])) * y[1::2], rtol=1e-12)
    # dequantise-then-matmul on the dequantised activation is the same number
    xq = q8.astype(np.float32) * np.repeat(xs, 128)
    d64, _ = oracle.gemv_dequant(packed, scales, xq)
    assert np.allclose(d64, y, rtol=1e-6, atol=1e-6)


def test_gemm_prefill_against_numpy(golden_dir):
    vec = np.load(golden_dir / "packer_vectors.npz")
    packed, scales = vec["gauss_k256_packed"], vec["gauss_k256_scales"]
    N, K = packed.shape[0], packed.shape[1] * 8
    rng = np.random.default_rng(5)
    M = 6
    x = rng.standard_normal((M, K)).astype(np.float16)
    q = oracle.unpack_nibbles(packed).astype(np.float16) - np.float16(8)
    w16 = (q.reshape(N, -1, 128) * scales[:, :, None]).astype(np.float16).reshape(N, K)   # one fp16 rounding
    ref = x.astype(np.float64) @ w16.astype(np.float64).T
    m_idx, n_idx = np.arange(M, dtype=np.int32), np.arange(N, dtype=np.int32)
    res = rng.standard_normal((M, N)).astype(np.float16)
    o64, o16 = oracle.gemm_prefill(packed, scales, x, m_idx, n_idx, residual=res)
    assert np.allclose(o64, ref + res.astype(np.float64), rtol=1e-12, atol=1e-12)
    expect16 = (ref.astype(np.float32).astype(np.float16).astype(np.float32) + res.astype(np.float32)).astype(np.float16)
    assert np.array_equal(o16, expect16)
    s64, _ = oracle.gemm_prefill(packed, scales, x, m_idx, np.arange(N // 2, dtype=np.int32), swiglu=True)
    assert np.allclose(s64, ref[:, 0::2] / (1 + np.exp(-ref[:, 0::2])) * ref[:, 1::2], rtol=1e-12)


def test_rmsnorm_against_numpy():
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(1536) * 2).astype(np.float16)
    g = (1 + 0.1 * rng.standard_normal(1536)).astype(np.float16)
    y, inv = oracle.rmsnorm(x, g)
    mean = np.float32(np.sum(x.astype(np.float64) ** 2)) / np.float32(1536)
    inv_ref = np.float32(1) / np.sqrt(mean + np.float32(1e-6), dtype=np.float32)
    assert np.float32(inv) == inv_ref      # IEEE fp32 after the double-precision sum
    ih = np.float16(inv_ref)
    expect = ((x * ih).astype(np.float16) * g).astype(np.float16)
    assert np.array_equal(y.view(np.uint16), expect.view(np.uint16))


def test_philox_known_answer_and_sampler_rules():
    """Philox-4x32-10: the published known-answer vector for an all-zero counter and key (Random123), then the
    selection rules of the reference's sampler (src/kernels/sampling.cu:86-100): greedy at temperature <= 1e-5,
    lowest index among equal scores, index offset only moves the counter and the reported index."""
    assert oracle.philox_first(0, 0, 0) == 0x6627E8D5
    logits = np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float16)
    tok, best, scores = oracle.sample(logits)
    assert (tok, best) == (1, 2.0) and np.array_equal(scores, logits.astype(np.float32))
    assert oracle.sample(logits, 1e-5)[0] == 1
    t1, _, s1 = oracle.sample(logits, 0.8, seed=99, seq_pos=4)
    t2, _, s2 = oracle.sample(logits[2:], 0.8, seed=99, seq_pos=4, index_offset=2)
    assert np.array_equal(s1[2:], s2)                      # same counters -> same noise
    assert t2 == 2 + int(np.argmax(s2))
    assert not np.array_equal(s1, oracle.sample(logits, 0.8, seed=99, seq_pos=5)[2])
    u = np.exp(-np.exp(-(s1 - logits.astype(np.float32) / np.float32(0.8))))   # invert the Gumbel transform
    assert np.all((u > 0) & (u < 1))


def test_attention_head_quantiser_follows_the_division_rule():
    """orc_quantize_heads_f32 (reference src/kernels/attention_gqa.cu:263-310) against the same rule written
    with numpy float32 operations: d = max(max|acc| / 127, 1e-8), q = clip(rint(acc / d)), sum8 = -8 * octet sums."""
    rng = np.random.default_rng(3)
    acc = (rng.standard_normal((6, 128)) * rng.uniform(0.01, 50, size=(6, 1))).astype(np.float32)
    acc[4] = 0.0
    out16, q8, scale, sum8 = oracle.quantize_heads_f32(acc)
    d = np.maximum(np.abs(acc).max(axis=1) / np.float32(127.0), np.float32(1e-8)).astype(np.float32)
    want = np.clip(np.rint(acc / d[:, None]), -127, 127).astype(np.int8)
    assert np.array_equal(scale, d)
    assert np.array_equal(q8.reshape(6, 128), want)
    assert np.array_equal(sum8.reshape(6, 16), -8 * want.reshape(6, 16, 8).astype(np.int32).sum(axis=2))
    assert np.array_equal(out16, acc.astype(np.float16))
    assert np.all(q8.reshape(6, 128)[4] == 0) and scale[4] == np.float32(1e-8)
