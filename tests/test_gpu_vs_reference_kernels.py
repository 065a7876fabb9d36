"""This library's kernels against the reference engine's own CUDA kernels, both run live on the
same inputs.  The reference kernels are compiled from the reference sources for sm_100a by
`make -C oracle ref` (oracle/_ref/); the tests skip when that checker library is absent."""
import numpy as np
import pytest

from tests import util
from tests.util import RefKernels

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    import qwen_engine_b200 as pkg
    pkg.init()
    return pkg


@pytest.fixture(scope="module", params=["ieee", "fastmath"])
def ref(request):
    if not RefKernels.available(request.param):
        pytest.skip("oracle/_ref not built")
    return RefKernels(request.param)


def _q8_buffers(n):
    return (torch.empty(n, dtype=torch.int8, device="cuda"), torch.empty(n // 128, dtype=torch.float32, device="cuda"),
            torch.empty(n // 8, dtype=torch.int32, device="cuda"))


def test_q8_1_equals_reference_kernel(ops, ref):
    from qwen_engine_b200 import synth
    sp = util.stream_ptr()
    for n in (1536, 8960):
        x = util.to_dev(synth.activations(n, "cmp", n))
        a, b = _q8_buffers(n), _q8_buffers(n)
        ops.launch_quantize_fp16_to_q8_1(x, *a, n)
        ref.call("ref_quantize_fp16_to_q8_1", x, *b, n, sp)
        torch.cuda.synchronize()
        if ref.flavour == "ieee":      # the source as written: identical bits
            for t, r in zip(a, b):
                assert torch.equal(t, r)
        else:                          # approximate division in the reference's fast-math build
            assert (a[0] != b[0]).float().mean().item() <= 0.01
            assert torch.allclose(a[1], b[1], rtol=2.0 ** -21, atol=0)


@pytest.mark.parametrize("N,K,res", [(1536, 1536, True), (1536, 8960, True), (151936, 1536, False)])
def test_gemv_w4a8_equals_reference_kernel(ops, ref, N, K, res):
    from qwen_engine_b200 import synth
    sp = util.stream_ptr()
    qw, sc = util.to_dev(synth.packed_weights(3, "cmp", N, K)), util.to_dev(synth.scales(3, "cmp", N, K))
    x = util.to_dev(synth.activations(3, "cmpx", K))
    r = util.to_dev(synth.activations(4, "cmpr", N)) if res else None
    q8, xs, s8 = _q8_buffers(K)
    ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, K)
    y_a = torch.empty(N, dtype=torch.float16, device="cuda")
    y_b = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(qw, sc, q8, xs, s8, r, y_a, N, K)
    ref.call("ref_gemv_w4a8", qw, sc, q8, xs, s8, r, y_b, N, K, sp)
    torch.cuda.synchronize()
    a, b = util.to_np(y_a), util.to_np(y_b)
    # same integers, fp32 sums in a different order: at most one fp16 step apart, nearly all equal
    assert np.mean(a.view(np.uint16) == b.view(np.uint16)) >= 0.97
    step = util.fp16_ulp(np.maximum(np.abs(b.astype(np.float64)), 1e-3))
    assert (np.abs(a.astype(np.float64) - b.astype(np.float64)) <= step * 1.01).all()


def test_swiglu_and_qkv_equal_reference_kernels(ops, ref):
    from qwen_engine_b200 import synth
    sp = util.stream_ptr()
    H, I = 1536, 8960
    qw, sc = util.to_dev(synth.packed_weights(5, "gu", 2 * I, H)), util.to_dev(synth.scales(5, "gu", 2 * I, H))
    x = util.to_dev(synth.activations(5, "gux", H))
    q8, xs, s8 = _q8_buffers(H)
    ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, H)
    y_a = torch.empty(I, dtype=torch.float16, device="cuda")
    y_b = torch.empty(I, dtype=torch.float16, device="cuda")
    ops.launch_gemv_dual_gate_up_swiglu_w4a8(qw, sc, q8, xs, s8, y_a, H, I)
    ref.call("ref_gemv_dual_gate_up_swiglu_w4a8", qw, sc, q8, xs, s8, y_b, H, I, sp)
    torch.cuda.synchronize()
    a, b = util.to_np(y_a).astype(np.float64), util.to_np(y_b).astype(np.float64)
    step = util.fp16_ulp(np.maximum(np.abs(b), 1e-3))
    assert (np.abs(a - b) <= 2.01 * step).all()     # expf vs the fast-math __expf, then one rounding each
    assert np.mean(a == b) >= 0.9
    dims = [1536, 256, 256]
    ws = [(util.to_dev(synth.packed_weights(6, f"t{i}", n, H)), util.to_dev(synth.scales(6, f"t{i}", n, H)))
          for i, n in enumerate(dims)]
    oa = [torch.empty(n, dtype=torch.float16, device="cuda") for n in dims]
    ob = [torch.empty(n, dtype=torch.float16, device="cuda") for n in dims]
    ops.launch_gemv_qkv_w4a8(ops.QKVProjectionView(ws[0][0], ws[0][1], oa[0], ws[1][0], ws[1][1], oa[1], ws[2][0],
                                                   ws[2][1], oa[2]), q8, xs, s8)
    pod = RefKernels.QKVPod(ws[0][0].data_ptr(), ws[0][1].data_ptr(), ob[0].data_ptr(), ws[1][0].data_ptr(),
                            ws[1][1].data_ptr(), ob[1].data_ptr(), ws[2][0].data_ptr(), ws[2][1].data_ptr(),
                            ob[2].data_ptr())
    ref.call("ref_gemv_qkv_w4a8", pod, q8, xs, s8, sp, H, 12, 2, 128)
    torch.cuda.synchronize()
    for ta, tb in zip(oa, ob):
        a, b = util.to_np(ta).astype(np.float64), util.to_np(tb).astype(np.float64)
        assert (np.abs(a - b) <= 1.01 * util.fp16_ulp(np.maximum(np.abs(b), 1e-3))).all()


@pytest.mark.parametrize("M", [8, 64, 256])
def test_gemm_prefill_equals_reference_kernel(ops, ref, M):
    from qwen_engine_b200 import synth
    sp = util.stream_ptr()
    N, K = 1536, 1536
    qw, sc = util.to_dev(synth.packed_weights(8, "pf", N, K)), util.to_dev(synth.scales(8, "pf", N, K))
    x = util.to_dev(synth.activations(8, "pfx", M, K))
    r = util.to_dev(synth.activations(9, "pfr", M, N))
    y_a = torch.empty((M, N), dtype=torch.float16, device="cuda")
    y_b = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ops.launch_gemm_prefill_w4a16(qw, sc, x, r, y_a, M, N, K)
    ref.call("ref_gemm_prefill_w4a16", qw, sc, x, r, y_b, M, N, K, sp, 148)
    torch.cuda.synchronize()
    a, b = util.to_np(y_a), util.to_np(y_b)
    assert np.mean(a.view(np.uint16) == b.view(np.uint16)) >= 0.97
    acc_size = np.abs(b.astype(np.float64) - util.to_np(r).astype(np.float64))
    step = util.fp16_ulp(np.maximum(np.maximum(np.abs(b.astype(np.float64)), acc_size), 1e-3))
    assert (np.abs(a.astype(np.float64) - b.astype(np.float64)) <= 2.01 * step).all()  # one step in fp16(acc), one in the add


@pytest.mark.parametrize("name", ["o", "down", "qkv", "gate_up"])
def test_prefill_at_1024_tokens_equals_reference_kernels(ops, ref, name):
    """Configuration 4 at a benchmarked token count: this library's tensor-core kernel (256-token tiles) against
    the reference's 64x64 wmma kernels (src/kernels/gemm_prefill.cu:319-610) on the same inputs."""
    from qwen_engine_b200 import synth
    sp = util.stream_ptr()
    M, H, I = 1024, 1536, 8960
    x = util.to_dev(synth.activations(41, "pf1k", M, 8960 if name == "down" else H))

    def close(a, b, extra=None, steps=2.01, same=0.95):
        a, b = util.to_np(a), util.to_np(b)
        assert np.mean(a.view(np.uint16) == b.view(np.uint16)) >= same
        size = np.abs(b.astype(np.float64))
        if extra is not None:
            size = np.maximum(size, np.abs(b.astype(np.float64) - util.to_np(extra).astype(np.float64)))
        # two fp32 accumulation orders differ by absolute amounts that scale with the terms, not with an output
        # that happens to cancel to nearly zero: such outputs are judged at 1 % of the matrix's rms
        rms = float(np.sqrt(np.mean(b.astype(np.float64) ** 2)))
        step = util.fp16_ulp(np.maximum(size, 1e-2 * rms))
        assert (np.abs(a.astype(np.float64) - b.astype(np.float64)) <= steps * step).all()

    if name in ("o", "down"):
        N, K = (H, H) if name == "o" else (H, I)
        qw, sc = util.to_dev(synth.packed_weights(42, name, N, K)), util.to_dev(synth.scales(42, name, N, K))
        r = util.to_dev(synth.activations(43, "pfr", M, N))
        y_a = torch.empty((M, N), dtype=torch.float16, device="cuda")
        y_b = torch.empty((M, N), dtype=torch.float16, device="cuda")
        ops.launch_gemm_prefill_w4a16(qw, sc, x, r, y_a, M, N, K)
        ref.call("ref_gemm_prefill_w4a16", qw, sc, x, r, y_b, M, N, K, sp, 148)
        torch.cuda.synchronize()
        # fp16(acc) one step apart at most (two when the accumulators straddle a power of two and the step is
        # measured at the smaller), then one rounding in the fp16 residual add
        close(y_a, y_b, extra=r, steps=3.01)
    elif name == "qkv":
        dims = [1536, 256, 256]
        ws = [(util.to_dev(synth.packed_weights(44, f"t{i}", n, H)), util.to_dev(synth.scales(44, f"t{i}", n, H)))
              for i, n in enumerate(dims)]
        oa = [torch.empty((M, n), dtype=torch.float16, device="cuda") for n in dims]
        ob = [torch.empty((M, n), dtype=torch.float16, device="cuda") for n in dims]
        ops.launch_gemm_prefill_qkv_w4a16(ops.QKVProjectionView(ws[0][0], ws[0][1], oa[0], ws[1][0], ws[1][1], oa[1],
                                                                ws[2][0], ws[2][1], oa[2]), x, M)
        pod = RefKernels.QKVPod(ws[0][0].data_ptr(), ws[0][1].data_ptr(), ob[0].data_ptr(), ws[1][0].data_ptr(),
                                ws[1][1].data_ptr(), ob[1].data_ptr(), ws[2][0].data_ptr(), ws[2][1].data_ptr(),
                                ob[2].data_ptr())
        ref.call("ref_gemm_prefill_qkv_w4a16", pod, x, M, sp, H, 12, 2, 128, 148)
        torch.cuda.synchronize()
        for ta, tb in zip(oa, ob):
            close(ta, tb, steps=2.01)
    else:
        qw, sc = util.to_dev(synth.packed_weights(45, "gu", 2 * I, H)), util.to_dev(synth.scales(45, "gu", 2 * I, H))
        y_a = torch.empty((M, I), dtype=torch.float16, device="cuda")
        y_b = torch.empty((M, I), dtype=torch.float16, device="cuda")
        ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(qw, sc, x, y_a, M, None, H, I)
        ref.call("ref_gemm_prefill_dual_gate_up_swiglu_w4a16", qw, sc, x, y_b, M, sp, H, I)
        torch.cuda.synchronize()
        # SwiGLU on fp32 accumulators whose sums were taken in different orders, expf against the fast-math
        # __expf in one flavour: a couple of fp16 steps at most
        close(y_a, y_b, steps=3.01, same=0.85)
