"""Parity of the M-token contraction (small-M decode batches, prefill) with the CPU oracle.

Arithmetic under test: fp16 weights dequantised as (q-8)*scale with one fp16 rounding, exact
fp16 x fp16 products, fp32 accumulation, fp16 output (+ fp16 residual add / SwiGLU).
Tolerance against the golden that sums the same products in double: max relative error
<= 1e-2, median <= 2 fp16 ulp (util.assert_fp16_close).
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


def _inputs(seed, M, N, K):
    from qwen_engine_b200 import synth
    return (synth.packed_weights(seed, "g", N, K), synth.scales(seed, "g", N, K),
            synth.activations(seed, "g", M, K))


def _sample(rng, n, k):
    k = min(n, k)
    idx = np.unique(np.concatenate([[0, n - 1], rng.choice(n, size=k, replace=False)]))
    return idx.astype(np.int32)


CASES = [
    # (M, N, K, residual)
    (1, 1536, 1536, True), (2, 2048, 1536, False), (3, 100, 256, True), (5, 1536, 8960, True),
    (8, 1536, 1536, True), (16, 1536, 1536, False), (33, 520, 512, True), (64, 1536, 8960, True),
    (128, 1536, 1536, True), (200, 2048, 1536, False), (512, 1536, 8960, True),
]


@pytest.mark.parametrize("M,N,K,use_res", CASES)
def test_gemm_prefill_matches_oracle(ops, M, N, K, use_res):
    qw, sc, x = _inputs(M * 7 + N + K, M, N, K)
    rng = np.random.default_rng(M + N)
    res = rng.standard_normal((M, N)).astype(np.float16) if use_res else None
    y = torch.full((M * N + 64,), float("nan"), dtype=torch.float16, device="cuda")
    d_res = None
    if use_res:
        y[:M * N] = util.to_dev(res).reshape(-1)   # in place: residual == output
        d_res = y
    ops.launch_gemm_prefill_w4a16(util.to_dev(qw), util.to_dev(sc), util.to_dev(x), d_res, y, M, N, K)
    torch.cuda.synchronize()
    out = util.to_np(y)
    assert np.isnan(out[M * N:]).all(), "wrote past the output"
    out = out[:M * N].reshape(M, N)
    m_idx, n_idx = _sample(rng, M, 24), _sample(rng, N, 96)
    ref64, ref16 = oracle.gemm_prefill(qw, sc, x, m_idx, n_idx, residual=res)
    got = out[np.ix_(m_idx, n_idx)]
    acc = ref64 - res[np.ix_(m_idx, n_idx)].astype(np.float64) if use_res else None
    rep = util.assert_fp16_close(got, ref64, what=f"gemm M={M} N={N} K={K}", magnitude=acc)
    # fp32 accumulation inside the tensor core is not IEEE-rounded per addition: allow a little over
    # one fp16 step at the size of the accumulator
    assert rep["max_ulp"] <= 2.5, rep
    # the oracle rounds like the kernel (fp16(acc), then the fp16 residual add): nearly all bits agree
    assert np.mean(got.view(np.uint16) == ref16.view(np.uint16)) > 0.95
    assert np.isfinite(out).all()


@pytest.mark.parametrize("M,K,nq,nkv,hd", [(1, 1536, 12, 2, 128), (4, 1536, 12, 2, 128), (16, 1536, 12, 2, 128),
                                           (70, 1536, 12, 2, 128), (256, 1536, 12, 2, 128),
                                           # k/v widths below the tensor-core tile: the CUDA-core form at any
                                           # token count (several token passes, ragged last one, deep K slices)
                                           (19, 1536, 4, 1, 64), (7, 8960, 4, 1, 64), (2, 256, 2, 1, 32)])
def test_gemm_prefill_qkv_matches_oracle(ops, M, K, nq, nkv, hd):
    from qwen_engine_b200 import synth
    dims = [nq * hd, nkv * hd, nkv * hd]
    x = synth.activations(M, "qkv", M, K)
    ws = [(synth.packed_weights(M, f"t{i}", n, K), synth.scales(M, f"t{i}", n, K)) for i, n in enumerate(dims)]
    outs = [torch.full((M * n + 8,), float("nan"), dtype=torch.float16, device="cuda") for n in dims]
    dev = [(util.to_dev(w), util.to_dev(s)) for w, s in ws]
    view = ops.QKVProjectionView(dev[0][0], dev[0][1], outs[0], dev[1][0], dev[1][1], outs[1],
                                 dev[2][0], dev[2][1], outs[2])
    ops.launch_gemm_prefill_qkv_w4a16(view, util.to_dev(x), M, None, K, nq, nkv, hd)
    torch.cuda.synchronize()
    rng = np.random.default_rng(M)
    for (w, s), o, n in zip(ws, outs, dims):
        got = util.to_np(o)
        assert np.isnan(got[M * n:]).all()
        got = got[:M * n].reshape(M, n)
        m_idx, n_idx = _sample(rng, M, 16), _sample(rng, n, 64)
        ref64, _ = oracle.gemm_prefill(w, s, x, m_idx, n_idx)
        util.assert_fp16_close(got[np.ix_(m_idx, n_idx)], ref64, what=f"qkv M={M}")


@pytest.mark.parametrize("M,H,I", [(1, 1536, 8960), (6, 256, 512), (16, 1536, 8960), (130, 1536, 8960), (40, 512, 100)])
def test_gemm_prefill_swiglu_matches_oracle(ops, M, H, I):
    qw, sc, x = _inputs(M + H + I, M, 2 * I, H)
    y = torch.full((M * I + 8,), float("nan"), dtype=torch.float16, device="cuda")
    ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(util.to_dev(qw), util.to_dev(sc), util.to_dev(x), y, M, None,
                                                      H, I)
    torch.cuda.synchronize()
    out = util.to_np(y)
    assert np.isnan(out[M * I:]).all()
    out = out[:M * I].reshape(M, I)
    rng = np.random.default_rng(M + I)
    m_idx, n_idx = _sample(rng, M, 16), _sample(rng, I, 96)
    ref64, _ = oracle.gemm_prefill(qw, sc, x, m_idx, n_idx, swiglu=True)
    util.assert_fp16_close(out[np.ix_(m_idx, n_idx)], ref64, what=f"swiglu M={M}")


def test_tensor_core_kernel_never_gave_up_waiting(ops):
    """Every wait in the tcgen05 kernel is bounded; a wait that ran out is counted on the device.
    Collected after the GEMM cases above: the count must still be zero."""
    assert ops.debug_counter(0) == 0


@pytest.mark.parametrize("M,N,K,ldc,col", [(40, 256, 512, 1024, 384), (200, 384, 1536, 384, 0), (3, 128, 256, 512, 128)])
def test_gemm_into_a_column_block_with_peer_copies(ops, M, N, K, ldc, col):
    """The contraction written as a column block of a wider [M][ldc] matrix (one rank's share of an output split
    by weight rows), and the same block stored into two more matrices standing in for peer GPUs' memory."""
    qw, sc, x = _inputs(M + N + K, M, N, K)
    d_qw, d_sc, d_x = util.to_dev(qw), util.to_dev(sc), util.to_dev(x)
    ref = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ops.launch_gemm_prefill_w4a16(d_qw, d_sc, d_x, None, ref, M, N, K)
    full = torch.full((M, ldc), 7.0, dtype=torch.float16, device="cuda")
    peers = [torch.full((M, ldc), 7.0, dtype=torch.float16, device="cuda") for _ in range(2)]
    ops.gemm_prefill_w4a16_block(d_qw, d_sc, d_x, None, full.data_ptr() + 2 * col, ldc,
                                 [p.data_ptr() + 2 * col for p in peers], M, N, K)
    torch.cuda.synchronize()
    for t in [full] + peers:
        if M >= 5:      # same kernel as the reference launch: same bits
            assert torch.equal(t[:, col:col + N], ref)
        else:           # peer stores force the tensor-core form where the plain launch takes the few-token form
            util.assert_fp16_close(util.to_np(t[:, col:col + N].contiguous()), util.to_np(ref).astype(np.float64), what="block")
        untouched = torch.ones(ldc, dtype=torch.bool, device="cuda")
        untouched[col:col + N] = False
        assert bool((t[:, untouched] == 7.0).all())
    # without peers a few tokens go through the CUDA-core form, which honours the row stride as well
    alone = torch.full((M, ldc), 7.0, dtype=torch.float16, device="cuda")
    ops.gemm_prefill_w4a16_block(d_qw, d_sc, d_x, None, alone.data_ptr() + 2 * col, ldc, [], M, N, K)
    torch.cuda.synchronize()
    assert torch.equal(alone[:, col:col + N], ref)


def test_full_size_prefill_row_split_agrees_with_the_unsplit_launch(ops):
    """The scaled-up shape of the benchmark (8192 -> 28672) at 256 tokens: eight column blocks written through the
    block entry point into one [M][N] matrix against the unsplit launch.  The narrow pieces split K over a cluster
    and use two issuing warps, so their fp32 sums are added in another order: nearly all entries are identical
    bits, the rest one fp16 step apart; sampled entries of both agree with the oracle."""
    N, K, M, parts = 28672, 8192, 256, 8
    rng = np.random.default_rng(99)
    qw = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint32)
    sc = rng.uniform(0.002, 0.02, size=(N, K // 128)).astype(np.float16)
    x = rng.standard_normal((M, K)).astype(np.float16)
    d_qw, d_sc, d_x = util.to_dev(qw), util.to_dev(sc), util.to_dev(x)
    whole = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ops.launch_gemm_prefill_w4a16(d_qw, d_sc, d_x, None, whole, M, N, K)
    pieces = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    rows = N // parts
    for p in range(parts):
        w = d_qw[p * rows:(p + 1) * rows].contiguous()
        s = d_sc[p * rows:(p + 1) * rows].contiguous()
        ops.gemm_prefill_w4a16_block(w, s, d_x, None, pieces.data_ptr() + 2 * p * rows, N, [], M, rows, K)
    torch.cuda.synchronize()
    a, b = util.to_np(whole), util.to_np(pieces)
    assert np.mean(a.view(np.uint16) == b.view(np.uint16)) >= 0.97
    util.assert_fp16_close(b, a.astype(np.float64), what="row-split pieces vs unsplit")
    m_idx, n_idx = _sample(rng, M, 6), _sample(rng, N, 40)
    ref64, _ = oracle.gemm_prefill(qw, sc, x, m_idx, n_idx)
    util.assert_fp16_close(a[np.ix_(m_idx, n_idx)], ref64, what="full-size prefill")
    util.assert_fp16_close(b[np.ix_(m_idx, n_idx)], ref64, what="full-size prefill, row-split")
    assert ops.debug_counter(0) == 0


# ---- the benchmark's own sizes ----------------------------------------------------------------------------
# Configuration 3: M in {1, 2, 4, 8, 16, 32, 64} over the four projection shapes (both sides of every dispatch
# threshold between the few-token CUDA-core forms and the tensor-core kernel).  Configuration 4:
# M in {128, 512, 1024, 4096} over the same shapes plus 8192 -> 28672.  Outputs are compared on sampled rows and
# columns (the oracle dequantises only the sampled weight rows), which keeps the CPU side to seconds.

_QWEN = {"qkv": (2048, 1536), "o": (1536, 1536), "gate_up": (17920, 1536), "down": (1536, 8960)}
_cache = {}


def _shape_weights(name):
    """(packed, scales) on host and device, made once per shape."""
    if name not in _cache:
        from qwen_engine_b200 import synth
        if name == "qkv":
            parts = [(synth.packed_weights(31, f"q{i}", n, 1536), synth.scales(31, f"q{i}", n, 1536))
                     for i, n in enumerate((1536, 256, 256))]
            _cache[name] = (parts, [(util.to_dev(w), util.to_dev(s)) for w, s in parts])
        elif name == "big":
            rng = np.random.default_rng(99)
            w = rng.integers(0, 2 ** 32, size=(28672, 8192 // 8), dtype=np.uint32)
            s = rng.uniform(0.002, 0.02, size=(28672, 8192 // 128)).astype(np.float16)
            _cache[name] = ((w, s), (util.to_dev(w), util.to_dev(s)))
        else:
            N, K = _QWEN[name]
            w, s = synth.packed_weights(31, name, N, K), synth.scales(31, name, N, K)
            _cache[name] = ((w, s), (util.to_dev(w), util.to_dev(s)))
    return _cache[name]


def _check_shape_at(ops, name, M, n_rows=6, n_cols=40):
    rng = np.random.default_rng(M * 13 + len(name))
    host, dev = _shape_weights(name)
    K = 8192 if name == "big" else _QWEN[name][1]
    x = rng.standard_normal((M, K)).astype(np.float16)
    d_x = util.to_dev(x)
    m_idx = _sample(rng, M, n_rows)
    if name == "qkv":
        dims = (1536, 256, 256)
        outs = [torch.full((M * n + 8,), float("nan"), dtype=torch.float16, device="cuda") for n in dims]
        view = ops.QKVProjectionView(dev[0][0], dev[0][1], outs[0], dev[1][0], dev[1][1], outs[1], dev[2][0], dev[2][1], outs[2])
        ops.launch_gemm_prefill_qkv_w4a16(view, d_x, M, None, K, 12, 2, 128)
        torch.cuda.synchronize()
        for (w, s), o, n in zip(host, outs, dims):
            got = util.to_np(o)
            assert np.isnan(got[M * n:]).all()
            n_idx = _sample(rng, n, n_cols)
            ref64, _ = oracle.gemm_prefill(w, s, x, m_idx, n_idx)
            util.assert_fp16_close(got[:M * n].reshape(M, n)[np.ix_(m_idx, n_idx)], ref64, what=f"qkv M={M}")
    elif name == "gate_up":
        I = 8960
        y = torch.full((M * I + 8,), float("nan"), dtype=torch.float16, device="cuda")
        ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(dev[0], dev[1], d_x, y, M, None, K, I)
        torch.cuda.synchronize()
        got = util.to_np(y)
        assert np.isnan(got[M * I:]).all()
        n_idx = _sample(rng, I, n_cols)
        ref64, _ = oracle.gemm_prefill(host[0], host[1], x, m_idx, n_idx, swiglu=True)
        util.assert_fp16_close(got[:M * I].reshape(M, I)[np.ix_(m_idx, n_idx)], ref64, what=f"gate_up M={M}")
    else:
        N = 28672 if name == "big" else _QWEN[name][0]
        use_res = name != "big"
        res = rng.standard_normal((M, N)).astype(np.float16) if use_res else None
        y = torch.full((M * N + 8,), float("nan"), dtype=torch.float16, device="cuda")
        if use_res:
            y[:M * N] = util.to_dev(res).reshape(-1)      # in place, as the engine calls O and down
        ops.launch_gemm_prefill_w4a16(dev[0], dev[1], d_x, y if use_res else None, y, M, N, K)
        torch.cuda.synchronize()
        got = util.to_np(y)
        assert np.isnan(got[M * N:]).all()
        n_idx = _sample(rng, N, n_cols)
        ref64, _ = oracle.gemm_prefill(host[0], host[1], x, m_idx, n_idx, residual=res)
        acc = ref64 - res[np.ix_(m_idx, n_idx)].astype(np.float64) if use_res else None
        rep = util.assert_fp16_close(got[:M * N].reshape(M, N)[np.ix_(m_idx, n_idx)], ref64,
                                     what=f"{name} M={M}", magnitude=acc)
        assert rep["max_ulp"] <= 2.5, rep


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
@pytest.mark.parametrize("M", [1, 2, 4, 5, 8, 16, 32, 64])
def test_decode_batch_grid_matches_oracle(ops, name, M):
    _check_shape_at(ops, name, M, n_rows=8, n_cols=48)


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
@pytest.mark.parametrize("M", [2, 3, 7, 9, 13, 16, 24, 40])
def test_mma_sync_few_token_form_matches_oracle(ops, name, M):
    """The weight-streaming kernel with warp-level MMAs, forced up to 64 tokens (several token passes for the long K,
    token tiles that are not full, a last pass with fewer tokens than a tile): against the oracle on sampled
    entries, including the last token row."""
    ops.set_option(ops.OPT_GEMM_MMA_MAX_TOKENS, 64)
    try:
        _check_shape_at(ops, name, M, n_rows=8, n_cols=48)
    finally:
        ops.set_option(ops.OPT_GEMM_MMA_MAX_TOKENS, 0)


@pytest.mark.parametrize("name,M", [(n, m) for n in ("qkv", "o", "gate_up", "down") for m in (128, 512, 1024, 4096)]
                         + [("big", 128), ("big", 1024), ("big", 4096)])
def test_prefill_sizes_of_the_benchmark_match_oracle(ops, name, M):
    _check_shape_at(ops, name, M)
    assert ops.debug_counter(0) == 0


def test_release_cached_benchmark_weights():
    _cache.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("M,N,K,mode", [(300, 1536, 1536, "res"), (257, 256, 512, "plain"), (700, 512, 256, "swiglu"),
                                        (1000, 1536, 8960, "res"), (260, 2048, 1536, "qkv")])
def test_cta_pair_kernel_on_small_and_ragged_shapes(ops, M, N, K, mode):
    """The cta_group::2 kernel forced (W4A16_OPT_GEMM_FORM = 2) onto shapes the dispatcher would give to the
    single-CTA kernel: a ragged last token tile, a single pair tile, SwiGLU, the in-place residual, three tensors.
    Checked against the oracle on sampled entries and against the single-CTA kernel on all of them."""
    from qwen_engine_b200 import synth
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    d_x = util.to_dev(x)

    def run(form):
        ops.set_option(ops.OPT_GEMM_FORM, form)
        try:
            if mode == "qkv":
                dims = (1536, 256, 256)
                ws = [(synth.packed_weights(M, f"p{i}", n, K), synth.scales(M, f"p{i}", n, K)) for i, n in enumerate(dims)]
                dev = [(util.to_dev(w), util.to_dev(s)) for w, s in ws]
                outs = [torch.full((M * n + 8,), float("nan"), dtype=torch.float16, device="cuda") for n in dims]
                view = ops.QKVProjectionView(dev[0][0], dev[0][1], outs[0], dev[1][0], dev[1][1], outs[1], dev[2][0], dev[2][1], outs[2])
                ops.launch_gemm_prefill_qkv_w4a16(view, d_x, M, None, K, 12, 2, 128)
                torch.cuda.synchronize()
                return ws, [util.to_np(o) for o in outs]
            qw, sc = synth.packed_weights(M, "p", N, K), synth.scales(M, "p", N, K)
            if mode == "swiglu":
                y = torch.full((M * (N // 2) + 8,), float("nan"), dtype=torch.float16, device="cuda")
                ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(util.to_dev(qw), util.to_dev(sc), d_x, y, M, None, K, N // 2)
                torch.cuda.synchronize()
                return (qw, sc), util.to_np(y)
            res = np.random.default_rng(7).standard_normal((M, N)).astype(np.float16) if mode == "res" else None
            y = torch.full((M * N + 8,), float("nan"), dtype=torch.float16, device="cuda")
            if res is not None:
                y[:M * N] = util.to_dev(res).reshape(-1)
            ops.launch_gemm_prefill_w4a16(util.to_dev(qw), util.to_dev(sc), d_x, y if res is not None else None, y, M, N, K)
            torch.cuda.synchronize()
            return (qw, sc, res), util.to_np(y)
        finally:
            ops.set_option(ops.OPT_GEMM_FORM, 0)

    w, pair = run(2)
    _, single = run(1)
    m_idx = _sample(rng, M, 8)
    if mode == "qkv":
        for (qw, sc), a, b, n in zip(w, pair, single, (1536, 256, 256)):
            assert np.isnan(a[M * n:]).all()
            a, b = a[:M * n].reshape(M, n), b[:M * n].reshape(M, n)
            util.assert_fp16_close(a, b.astype(np.float64), what="pair vs single")
            n_idx = _sample(rng, n, 32)
            util.assert_fp16_close(a[np.ix_(m_idx, n_idx)], oracle.gemm_prefill(qw, sc, x, m_idx, n_idx)[0], what="pair qkv")
    elif mode == "swiglu":
        I = N // 2
        assert np.isnan(pair[M * I:]).all()
        a, b = pair[:M * I].reshape(M, I), single[:M * I].reshape(M, I)
        util.assert_fp16_close(a, b.astype(np.float64), what="pair vs single")
        n_idx = _sample(rng, I, 32)
        util.assert_fp16_close(a[np.ix_(m_idx, n_idx)], oracle.gemm_prefill(w[0], w[1], x, m_idx, n_idx, swiglu=True)[0], what="pair swiglu")
    else:
        assert np.isnan(pair[M * N:]).all()
        a, b = pair[:M * N].reshape(M, N), single[:M * N].reshape(M, N)
        res = w[2]
        acc_all = b.astype(np.float64) - res.astype(np.float64) if res is not None else None
        util.assert_fp16_close(a, b.astype(np.float64), what="pair vs single", magnitude=acc_all)
        n_idx = _sample(rng, N, 32)
        ref64, _ = oracle.gemm_prefill(w[0], w[1], x, m_idx, n_idx, residual=res)
        acc = ref64 - res[np.ix_(m_idx, n_idx)].astype(np.float64) if res is not None else None
        util.assert_fp16_close(a[np.ix_(m_idx, n_idx)], ref64, what="pair plain", magnitude=acc)
    assert ops.debug_counter(0) == 0
