"""Parity of the CUDA decode path with the CPU oracle, through the C ABI.

Integer work (Q8_1 bytes, scales, sum8, per-group int32 dots) must be bit-exact.
fp16 outputs must meet the path's stated tolerance against the golden computed on the
same Q8_1 activations: max relative error <= 1e-2 and median error <= 2 fp16 ulp
(util.assert_fp16_close); in practice they land within one ulp, which is asserted too.
"""
import numpy as np
import pytest

import oracle
from tests import util

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    import qwen_engine_b200 as pkg
    pkg.init()
    return pkg


def _x(seed, n, kind="normal"):
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = rng.standard_normal(n).astype(np.float32)
    if kind == "edges":
        x[:128] = 0.0                       # all-zero group -> scale 1e-8
        x[128:256] = 65504.0                # fp16 max
        x[256:384] = -x[256:384] * 1e-4     # tiny values
        x[384] = 127.5 * (np.abs(x[384:512]).max() / 127.0)  # near a rounding tie
    return x.astype(np.float16)


def _weights(seed, N, K):
    from qwen_engine_b200 import synth
    return synth.packed_weights(seed, "t", N, K), synth.scales(seed, "t", N, K)


def _quantize_gpu(ops, x):
    n = x.size
    d_x = util.to_dev(x)
    q8 = torch.empty(n, dtype=torch.int8, device="cuda")
    sc = torch.empty(n // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(n // 8, dtype=torch.int32, device="cuda")
    ops.launch_quantize_fp16_to_q8_1(d_x, q8, sc, s8, n)
    torch.cuda.synchronize()
    return q8, sc, s8


@pytest.mark.parametrize("n,kind", [(128, "normal"), (256, "normal"), (1536, "normal"), (8960, "normal"),
                                    (1536, "edges"), (27648, "normal")])
def test_quantize_q8_1_bit_exact(ops, n, kind):
    x = _x(n + 7, n, kind)
    q8, sc, s8 = _quantize_gpu(ops, x)
    r_q8, r_sc, r_s8 = oracle.quantize_q8_1(x)
    assert np.array_equal(util.to_np(q8), r_q8)
    assert np.array_equal(util.to_np(sc).view(np.uint32), r_sc.view(np.uint32))
    assert np.array_equal(util.to_np(s8), r_s8)


@pytest.mark.parametrize("N,K", [(16, 256), (40, 512), (1536, 1536), (1536, 8960), (2048, 1536), (1000, 2560)])
def test_group_dots_bit_exact(ops, N, K):
    qw, _ = _weights(N * 31 + K, N, K)
    x = _x(K, K)
    q8, sc, s8 = _quantize_gpu(ops, x)
    out = torch.empty((N, K // 128), dtype=torch.int32, device="cuda")
    ops.gemv_group_dots(util.to_dev(qw), q8, s8, out, N, K)
    torch.cuda.synchronize()
    ref = oracle.group_dots(qw, util.to_np(q8))
    assert np.array_equal(util.to_np(out), ref)
    # extremes: all nibbles 0 or 15 against saturated activations stay exact in int32
    qw_hi = np.full_like(qw, 0xFFFFFFFF)
    q8_sat = torch.full((K,), 127, dtype=torch.int8, device="cuda")
    s8_sat = torch.full((K // 8,), -8 * 8 * 127, dtype=torch.int32, device="cuda")
    ops.gemv_group_dots(util.to_dev(qw_hi), q8_sat, s8_sat, out, N, K)
    torch.cuda.synchronize()
    assert np.all(util.to_np(out) == 128 * 7 * 127)


SHAPES = [
    # (N, K, residual)
    (1536, 1536, True),    # O
    (1536, 8960, True),    # down (benchmark configuration 0)
    (2048, 1536, False),
    (16, 256, False),      # smallest legal
    (17, 256, True),       # ragged N
    (1000, 2560, True),
    (5000, 1536, False),
    (151936, 1536, False),  # lm_head: tall enough for the persistent streaming kernel
    (80000, 1536, True),    # streaming kernel with an in-place residual and a ragged last row block
    (76001, 1024, False),   # streaming kernel, 4 steps per lane, odd row count
    (28672, 8192, True),    # tall and K > 2048: the streaming kernel that takes K in slices of 2048 (benchmark shape)
    (20001, 4352, False),   # the same with a ragged last slice (17 steps) and an odd row count
]


@pytest.mark.parametrize("pdl", [True, False])
@pytest.mark.parametrize("N,K,use_res", SHAPES)
def test_gemv_w4a8_matches_oracle(ops, N, K, use_res, pdl):
    ops.set_pdl(pdl)
    try:
        qw, sc = _weights(N + K, N, K)
        x = _x(N * 3 + K, K)
        res = _x(N, (N + 127) // 128 * 128)[:N] if use_res else None
        q8, xs, s8 = _quantize_gpu(ops, x)
        d_qw, d_sc = util.to_dev(qw), util.to_dev(sc)
        y = torch.full((N + 64,), float("nan"), dtype=torch.float16, device="cuda")  # guard band behind the output
        d_res = None
        if use_res:
            y[:N] = util.to_dev(res)   # in place, as the engine calls it: residual == output
            d_res = y
        ops.launch_gemv_w4a8(d_qw, d_sc, q8, xs, s8, d_res, y, N, K)
        torch.cuda.synchronize()
        out = util.to_np(y)
        assert np.isnan(out[N:]).all(), "wrote past the output"
        y64, y16 = oracle.gemv_q8(qw, sc, util.to_np(q8), util.to_np(xs), residual=res)
        rep = util.assert_fp16_close(out[:N], y64, what=f"gemv {N}x{K}")
        assert rep["max_ulp"] <= 1.0, rep
        assert np.mean(out[:N].view(np.uint16) == y16.view(np.uint16)) > 0.98
    finally:
        ops.set_pdl(True)


def test_gemv_w4a8_unaligned_weights_and_activations(ops):
    """Pointers that are only 4-byte aligned take the narrow-load variants; same results."""
    N, K = 200, 1536
    qw, sc = _weights(5, N, K)
    x = _x(9, K)
    q8, xs, s8 = _quantize_gpu(ops, x)
    buf = torch.zeros(qw.size + 1, dtype=torch.int32, device="cuda")
    buf[1:] = util.to_dev(qw).reshape(-1)
    q8_buf = torch.zeros(K + 4, dtype=torch.int8, device="cuda")
    q8_buf[4:] = q8
    s8_buf = torch.zeros(K // 8 + 1, dtype=torch.int32, device="cuda")
    s8_buf[1:] = s8
    y_a = torch.empty(N, dtype=torch.float16, device="cuda")
    y_u = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(util.to_dev(qw), util.to_dev(sc), q8, xs, s8, None, y_a, N, K)
    ops.launch_gemv_w4a8(buf[1:], util.to_dev(sc), q8_buf[4:], xs, s8_buf[1:], None, y_u, N, K)
    torch.cuda.synchronize()
    assert torch.equal(y_a, y_u)


@pytest.mark.parametrize("N,K", [(1536, 8960), (1536, 1536), (48, 512)])
def test_gemv_w4a16_fp16_input_equals_prequantised(ops, N, K):
    """The fp16-input entry quantises inside the kernel: identical bits to quantise + W4A8."""
    qw, sc = _weights(N ^ K, N, K)
    x = _x(K + 1, K)
    res = _x(N + 2, (N + 127) // 128 * 128)[:N]
    q8, xs, s8 = _quantize_gpu(ops, x)
    d_qw, d_sc, d_res = util.to_dev(qw), util.to_dev(sc), util.to_dev(res)
    y1 = torch.empty(N, dtype=torch.float16, device="cuda")
    y2 = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(d_qw, d_sc, q8, xs, s8, d_res, y1, N, K)
    ops.launch_gemv_w4a16(d_qw, d_sc, util.to_dev(x), d_res, y2, N, K)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    # and against the fp32 dequantise-then-matmul golden on the dequantised Q8_1 activation
    xq = util.to_np(q8).astype(np.float32) * np.repeat(util.to_np(xs), 128)
    y64, _ = oracle.gemv_dequant(qw, sc, xq, residual=res)
    util.assert_fp16_close(util.to_np(y2), y64, what="gemv_w4a16 vs dequant golden")


@pytest.mark.parametrize("nq,nkv,hd,K", [(12, 2, 128, 1536), (4, 1, 64, 512), (3, 1, 16, 256)])
def test_gemv_qkv_matches_oracle(ops, nq, nkv, hd, K):
    x = _x(K * 5, K)
    q8, xs, s8 = _quantize_gpu(ops, x)
    dims = [nq * hd, nkv * hd, nkv * hd]
    ws = [_weights(100 + i, n, K) for i, n in enumerate(dims)]
    outs = [torch.full((n + 8,), float("nan"), dtype=torch.float16, device="cuda") for n in dims]
    dev = [(util.to_dev(w), util.to_dev(s)) for w, s in ws]
    view = ops.QKVProjectionView(dev[0][0], dev[0][1], outs[0], dev[1][0], dev[1][1], outs[1],
                                 dev[2][0], dev[2][1], outs[2])
    ops.launch_gemv_qkv_w4a8(view, q8, xs, s8, None, K, nq, nkv, hd)
    torch.cuda.synchronize()
    for (w, s), o, n in zip(ws, outs, dims):
        got = util.to_np(o)
        assert np.isnan(got[n:]).all()
        y64, _ = oracle.gemv_q8(w, s, util.to_np(q8), util.to_np(xs))
        rep = util.assert_fp16_close(got[:n], y64, what="qkv")
        assert rep["max_ulp"] <= 1.0, rep


@pytest.mark.parametrize("H,I", [(1536, 8960), (256, 512), (512, 100), (2560, 10240)])
def test_gemv_swiglu_matches_oracle(ops, H, I):
    qw, sc = _weights(H + I, 2 * I, H)
    x = _x(H + 3, H)
    q8, xs, s8 = _quantize_gpu(ops, x)
    d_qw, d_sc = util.to_dev(qw), util.to_dev(sc)
    y8 = torch.full((I + 8,), float("nan"), dtype=torch.float16, device="cuda")
    y16 = torch.empty(I, dtype=torch.float16, device="cuda")
    ops.launch_gemv_dual_gate_up_swiglu_w4a8(d_qw, d_sc, q8, xs, s8, y8, H, I)
    ops.launch_gemv_dual_gate_up_swiglu_w4a16(d_qw, d_sc, util.to_dev(x), y16, H, I)
    torch.cuda.synchronize()
    got = util.to_np(y8)
    assert np.isnan(got[I:]).all()
    assert torch.equal(y8[:I], y16)
    y64, _ = oracle.gemv_q8(qw, sc, util.to_np(q8), util.to_np(xs), swiglu=True)
    rep = util.assert_fp16_close(got[:I], y64, what="swiglu")
    assert rep["max_ulp"] <= 1.5, rep


def test_reference_synthetic_suite3_restated(ops):
    """The reference's own synthetic GEMV+SwiGLU test (tests/test_kernels.cu:242-403), restated:
    same dimension list, x ~ U(+-1/sqrt(H)), nibbles uniform in 2..14, every scale 0.05/sqrt(H),
    CPU golden with std::round semantics and double accumulation, pass = max abs error <= 5e-3.
    (numpy's generator stands in for std::mt19937; the distributions are the reference's.)"""
    for H, I in [(1536, 8960), (2560, 10240), (5120, 27648), (256, 512)]:
        rng = np.random.Generator(np.random.Philox(key=42 + H))
        sf = 1.0 / np.sqrt(np.float32(H))
        x = rng.uniform(-sf, sf, H).astype(np.float32).astype(np.float16)
        nib = rng.integers(2, 15, size=(2 * I, H), dtype=np.uint8)
        qw = oracle.pack_nibbles(nib)
        sc = np.full((2 * I, H // 128), np.float16(np.float32(0.05) * sf), dtype=np.float16)
        out = torch.empty(I, dtype=torch.float16, device="cuda")
        ops.launch_gemv_dual_gate_up_swiglu_w4a16(util.to_dev(qw), util.to_dev(sc), util.to_dev(x), out, H, I)
        torch.cuda.synchronize()
        q8, xs, _ = oracle.quantize_q8_1(x, oracle.ROUND_HALF_AWAY)
        _, ref16 = oracle.gemv_q8(qw, sc, q8, xs, swiglu=True)
        got = util.to_np(out).astype(np.float32)
        assert np.isfinite(got).all()
        assert np.abs(got - ref16.astype(np.float32)).max() <= 5e-3


def test_rmsnorm_q8_1_matches_oracle(ops):
    for H in (1536, 256, 5120):
        x = (_x(H, H).astype(np.float32) * 3.0).astype(np.float16)
        gamma = (1.0 + 0.1 * _x(H + 1, H).astype(np.float32)).astype(np.float16)
        q8 = torch.empty(H, dtype=torch.int8, device="cuda")
        sc = torch.empty(H // 128, dtype=torch.float32, device="cuda")
        s8 = torch.empty(H // 8, dtype=torch.int32, device="cuda")
        yo = torch.empty(H, dtype=torch.float16, device="cuda")
        ops.launch_rmsnorm_q8_1(util.to_dev(x), util.to_dev(gamma), yo, q8, sc, s8, None, H)
        ops.launch_rmsnorm_q8_1(util.to_dev(x), util.to_dev(gamma), None, q8, sc, s8, None, H)
        torch.cuda.synchronize()
        y_ref, _ = oracle.rmsnorm(x, gamma)
        assert np.array_equal(util.to_np(yo).view(np.uint16), y_ref.view(np.uint16))
        r_q8, r_sc, r_s8 = oracle.quantize_q8_1(y_ref)
        assert np.array_equal(util.to_np(q8), r_q8)
        assert np.array_equal(util.to_np(sc).view(np.uint32), r_sc.view(np.uint32))
        assert np.array_equal(util.to_np(s8), r_s8)


def test_layer_chain_in_cuda_graph_equals_eager(ops):
    """The engine captures its decode pass into a CUDA graph after one eager call
    (reference src/engine.cu:453-470); a captured chain must replay to the same bits."""
    from qwen_engine_b200 import synth
    H, I = 1536, 8960
    w = {n: (util.to_dev(synth.packed_weights(1, n, *synth.SHAPES[n])), util.to_dev(synth.scales(1, n, *synth.SHAPES[n])))
         for n in ("o", "gate_up", "down")}
    h0 = util.to_dev(_x(77, H))
    q8 = torch.empty(I, dtype=torch.int8, device="cuda")
    xs = torch.empty(I // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(I // 8, dtype=torch.int32, device="cuda")
    mlp = torch.empty(I, dtype=torch.float16, device="cuda")
    h = torch.empty(H, dtype=torch.float16, device="cuda")

    def chain():
        ops.launch_quantize_fp16_to_q8_1(h, q8, xs, s8, H)
        ops.launch_gemv_w4a8(w["o"][0], w["o"][1], q8, xs, s8, h, h, H, H)
        ops.launch_quantize_fp16_to_q8_1(h, q8, xs, s8, H)
        ops.launch_gemv_dual_gate_up_swiglu_w4a8(w["gate_up"][0], w["gate_up"][1], q8, xs, s8, mlp, H, I)
        ops.launch_quantize_fp16_to_q8_1(mlp, q8, xs, s8, I)
        ops.launch_gemv_w4a8(w["down"][0], w["down"][1], q8, xs, s8, h, h, H, I)

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        h.copy_(h0)
        chain()
        s.synchronize()
        eager = h.clone()
        g = torch.cuda.CUDAGraph()
        h.copy_(h0)
        with torch.cuda.graph(g, stream=s):
            chain()
        for _ in range(3):
            h.copy_(h0)
            g.replay()
            s.synchronize()
            assert torch.equal(h, eager)


def test_argument_errors_return_status(ops):
    y = torch.empty(16, dtype=torch.float16, device="cuda")
    q8 = torch.empty(512, dtype=torch.int8, device="cuda")
    xs = torch.empty(4, dtype=torch.float32, device="cuda")
    s8 = torch.empty(64, dtype=torch.int32, device="cuda")
    w = torch.empty(16 * 64, dtype=torch.int32, device="cuda")
    sc = torch.empty(16 * 4, dtype=torch.float16, device="cuda")
    with pytest.raises(ops.W4A16Error) as e:
        ops.launch_gemv_w4a8(w, sc, q8, xs, s8, None, y, 16, 384)   # K not a multiple of 256
    assert e.value.status == -2
    with pytest.raises(ops.W4A16Error) as e:
        ops.launch_gemv_w4a8(None, sc, q8, xs, s8, None, y, 16, 512)
    assert e.value.status == -1


# ---- the two ways the GEMV brings its weights on chip -----------------------------------------------------
FORM_SHAPES = [
    # (N, K): the model's projections, small and ragged cases, a K whose slices are uneven (2560 = 10 steps),
    # a long K (the cluster split with 8 slices), rows that do not fill the last CTA
    (1536, 1536), (2048, 1536), (1536, 8960), (16, 256), (17, 256), (1000, 2560), (5000, 1536), (1536, 4096),
    (100, 8960), (28672, 8192), (333, 17920),
]


def _both_forms(ops, fn):
    """Runs fn() with register-held weight loads and with bulk copies into shared memory (where the K slices of a
    long vector go to the CTAs of a cluster); returns (register form, bulk form) after checking that the default
    choice gives those bits too."""
    outs = []
    try:
        for form in (ops.GEMV_FORM_REGISTERS, ops.GEMV_FORM_BULK, ops.GEMV_FORM_AUTO):
            ops.set_option(ops.OPT_GEMV_FORM, form)
            outs.append(fn())
            torch.cuda.synchronize()
    finally:
        ops.set_option(ops.OPT_GEMV_FORM, ops.GEMV_FORM_AUTO)
    for o in outs[2:]:
        assert torch.equal(o.view(torch.int16), outs[1].view(torch.int16))
    return outs[0], outs[1]


@pytest.mark.parametrize("N,K", FORM_SHAPES)
def test_bulk_copy_form_gives_the_bits_of_the_register_form(ops, N, K):
    """Same plan, same integer dots, same fp32 order: the shared-memory form (cp.async.bulk + mbarrier, and the
    cluster K split for long vectors) must not change a bit, for every input form and epilogue."""
    qw, sc = _weights(N * 7 + K, N, K)
    d_qw, d_sc = util.to_dev(qw), util.to_dev(sc)
    x = _x(N + K, K)
    d_x = util.to_dev(x)
    q8, xs, s8 = _quantize_gpu(ops, x)
    res = util.to_dev(_x(N, (N + 127) // 128 * 128)[:N])
    gamma = util.to_dev((0.5 + 0.1 * np.random.default_rng(K).standard_normal(K)).astype(np.float16))

    def plain_q8():
        y = torch.full((N + 32,), float("nan"), dtype=torch.float16, device="cuda")
        y[:N] = res
        ops.launch_gemv_w4a8(d_qw, d_sc, q8, xs, s8, y, y, N, K)
        return y

    def plain_fp16():
        y = torch.full((N + 32,), float("nan"), dtype=torch.float16, device="cuda")
        ops.launch_gemv_w4a16(d_qw, d_sc, d_x, None, y, N, K)
        return y

    def plain_norm():
        y = torch.full((N + 32,), float("nan"), dtype=torch.float16, device="cuda")
        ops.launch_gemv_rmsnorm_w4a16(d_qw, d_sc, d_x, gamma, None, y, N, K)
        return y

    for fn in (plain_q8, plain_fp16, plain_norm):
        a, b = _both_forms(ops, fn)
        assert torch.equal(a[:N].view(torch.int16), b[:N].view(torch.int16)), fn.__name__
        assert torch.isnan(b[N:]).all(), fn.__name__
    # against the oracle too (the register form is checked elsewhere; this pins the new form directly)
    y64, _ = oracle.gemv_q8(qw, sc, util.to_np(q8), util.to_np(xs), residual=util.to_np(res))
    _, b = _both_forms(ops, plain_q8)
    rep = util.assert_fp16_close(util.to_np(b)[:N], y64, what=f"bulk-copy gemv {N}x{K}")
    assert rep["max_ulp"] <= 1.0, rep
    if N % 2 == 0:
        I = N // 2

        def swiglu_q8():
            y = torch.full((I + 32,), float("nan"), dtype=torch.float16, device="cuda")
            ops.launch_gemv_dual_gate_up_swiglu_w4a8(d_qw, d_sc, q8, xs, s8, y, K, I)
            return y

        def swiglu_norm():
            y = torch.full((I + 32,), float("nan"), dtype=torch.float16, device="cuda")
            ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(d_qw, d_sc, d_x, gamma, y, K, I)
            return y

        for fn in (swiglu_q8, swiglu_norm):
            a, b = _both_forms(ops, fn)
            assert torch.equal(a[:I].view(torch.int16), b[:I].view(torch.int16)), fn.__name__
            assert torch.isnan(b[I:]).all(), fn.__name__
    assert ops.debug_counter(1) == 0, "a bulk copy did not land within its bounded wait"


@pytest.mark.parametrize("nq,nkv,hd,K", [(12, 2, 128, 1536), (4, 1, 64, 512), (16, 8, 128, 2560)])
def test_bulk_copy_form_qkv(ops, nq, nkv, hd, K):
    from qwen_engine_b200 import synth
    dims = [nq * hd, nkv * hd, nkv * hd]
    ws = [(util.to_dev(synth.packed_weights(K, f"f{i}", n, K)), util.to_dev(synth.scales(K, f"f{i}", n, K)))
          for i, n in enumerate(dims)]
    x = _x(K + nq, K)
    q8, xs, s8 = _quantize_gpu(ops, x)
    gamma = util.to_dev(np.full(K, 0.7, dtype=np.float16))

    def run(norm):
        outs = [torch.full((n + 8,), float("nan"), dtype=torch.float16, device="cuda") for n in dims]
        view = ops.QKVProjectionView(ws[0][0], ws[0][1], outs[0], ws[1][0], ws[1][1], outs[1], ws[2][0], ws[2][1], outs[2])
        if norm:
            ops.launch_gemv_qkv_rmsnorm_w4a16(view, util.to_dev(x), gamma, None, K, nq, nkv, hd)
        else:
            ops.launch_gemv_qkv_w4a8(view, q8, xs, s8, None, K, nq, nkv, hd)
        return torch.cat(outs)

    for norm in (False, True):
        a, b = _both_forms(ops, lambda: run(norm))
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert ops.debug_counter(1) == 0
