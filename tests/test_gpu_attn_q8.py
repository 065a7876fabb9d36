"""Q8_1 of the attention output with the rule of the reference's flash-decode combine step
(src/kernels/attention_gqa.cu:258-310): one group per head, quantised from the fp32 accumulator with a
division per element.  Integer work: bytes, per-octet sums and the fp32 scale must be bit-exact against the
oracle (orc_quantize_heads_f32) and against the reference's own kernel built for sm_100a as written; the
fused O projection must give the bits of quantiser + w4a16_gemv_w4a8."""
import ctypes

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


def _heads(seed, heads):
    rng = np.random.default_rng(seed)
    acc = rng.standard_normal((heads, 128)).astype(np.float32) * rng.uniform(1e-3, 30.0, size=(heads, 1)).astype(np.float32)
    if heads >= 4:
        acc[1] = 0.0                                   # an all-zero head: the scale floor 1e-8
        acc[2, ::2] = np.float32(65504.0) * 3.0        # beyond fp16: only the Q8_1 form stays finite
        acc[3] = np.round(acc[3] * 4.0) / 4.0 + 0.5    # many values on rounding ties of the quotient
    return acc


def _run_lib(ops, acc, want_fp16=True):
    heads = acc.shape[0]
    d_acc = util.to_dev(acc)
    q8 = torch.zeros(heads * 128, dtype=torch.int8, device="cuda")
    sc = torch.zeros(heads, dtype=torch.float32, device="cuda")
    s8 = torch.zeros(heads * 16, dtype=torch.int32, device="cuda")
    o16 = torch.zeros(heads * 128, dtype=torch.float16, device="cuda") if want_fp16 else None
    ops.quantize_attn_heads_f32_to_q8_1(d_acc, o16, q8, sc, s8, heads)
    torch.cuda.synchronize()
    return q8, sc, s8, o16


@pytest.mark.parametrize("heads", [1, 12, 37])
def test_attn_head_quantiser_bit_exact_against_oracle(ops, heads):
    acc = _heads(heads, heads)
    q8, sc, s8, o16 = _run_lib(ops, acc)
    r16, r8, rs, rsum = oracle.quantize_heads_f32(acc)
    assert np.array_equal(util.to_np(q8), r8)
    assert np.array_equal(util.to_np(sc).view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(util.to_np(s8), rsum)
    assert np.array_equal(util.to_np(o16).view(np.uint16), r16.reshape(-1).view(np.uint16))


def test_division_rule_differs_from_the_fp16_quantiser(ops):
    """Why the variant exists: on the same accumulators, quantising fp16(acc) with the stand-alone quantiser
    (multiply by 1 / d) does not give the same bytes."""
    acc = _heads(5, 12)
    acc[2] = np.clip(acc[2], -60000, 60000)
    _, r8, _, _ = oracle.quantize_heads_f32(acc)
    q8b, _, _ = oracle.quantize_q8_1(acc.astype(np.float16).reshape(-1))
    assert np.mean(r8 != q8b) > 0


def test_o_projection_from_attention_accumulators_equals_quantiser_plus_gemv(ops):
    from qwen_engine_b200 import synth
    N, K = 1536, 1536
    acc = _heads(77, K // 128)
    acc[2] = np.clip(acc[2], -40.0, 40.0)     # keep the projection's fp16 output finite
    qw, sc = util.to_dev(synth.packed_weights(7, "attn.o", N, K)), util.to_dev(synth.scales(7, "attn.o", N, K))
    res = util.to_dev(synth.activations(7, "attn.res", N))
    q8, xs, s8, _ = _run_lib(ops, acc, want_fp16=False)
    want = res.clone()
    ops.launch_gemv_w4a8(qw, sc, q8, xs, s8, want, want, N, K)
    got = torch.full((N + 16,), float("nan"), dtype=torch.float16, device="cuda")
    got[:N] = res
    ops.gemv_attn_heads_f32_w4a16(qw, sc, util.to_dev(acc.reshape(-1)), got, got, N, K)
    torch.cuda.synchronize()
    assert torch.equal(got[:N], want)
    assert np.isnan(util.to_np(got)[N:]).all()
    # and against the oracle's GEMV on the oracle's bytes
    _, r8, rs, _ = oracle.quantize_heads_f32(acc)
    y64, _ = oracle.gemv_q8(synth.packed_weights(7, "attn.o", N, K), synth.scales(7, "attn.o", N, K), r8, rs,
                            residual=synth.activations(7, "attn.res", N))
    util.assert_fp16_close(util.to_np(want), y64, what="O projection from attention accumulators")


@pytest.mark.parametrize("flavour", ["ieee", "fastmath"])
def test_attn_head_quantiser_against_the_reference_combine_kernel(ops, flavour):
    """The reference's stage-2 kernel fed with partials that make its accumulator equal a chosen fp32 value:
    split 0 carries (maximum 0, denominator 1, partial = value), all other splits are empty, so the combine
    weight is expf(0) * (1 / 1) = 1 and acc = 0 + 1 * value."""
    if not util.RefKernels.available(flavour):
        pytest.skip("reference kernels not built (oracle/Makefile ref)")
    ref = util.RefKernels(flavour)
    if not hasattr(ref.lib, "ref_flash_decode_combine"):
        pytest.skip("checker library built without the combine-kernel wrapper")
    splits = ref.lib.ref_flash_decode_splits()
    heads = 12
    acc = _heads(21, heads)
    part = np.zeros((heads, splits, 128), dtype=np.float32)
    part[:, 0, :] = acc
    lse = np.zeros((heads, splits, 2), dtype=np.float32)
    lse[:, :, 0] = -np.inf
    lse[:, 0, 0] = 0.0
    lse[:, 0, 1] = 1.0
    q8 = torch.zeros(heads * 128, dtype=torch.int8, device="cuda")
    sc = torch.zeros(heads, dtype=torch.float32, device="cuda")
    s8 = torch.zeros(heads * 16, dtype=torch.int32, device="cuda")
    o16 = torch.zeros(heads * 128, dtype=torch.float16, device="cuda")
    ref.call("ref_flash_decode_combine", util.to_dev(part), util.to_dev(lse), o16, q8, sc, s8, heads, 128,
             util.stream_ptr())
    torch.cuda.synchronize()
    mine = _run_lib(ops, acc)
    if flavour == "ieee":
        assert torch.equal(mine[0], q8) and torch.equal(mine[2], s8)
        assert np.array_equal(util.to_np(mine[1]).view(np.uint32), util.to_np(sc).view(np.uint32))
        assert torch.equal(mine[3].view(torch.int16), o16.view(torch.int16))
    else:
        # approximate division under --use_fast_math: a quotient next to a rounding tie may land on the other side
        diff = (mine[0].to(torch.int32) - q8.to(torch.int32)).abs()
        assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 0.02
        a, b = util.to_np(mine[1]), util.to_np(sc)
        assert np.all(np.abs(a - b) <= np.spacing(np.maximum(np.abs(a), np.abs(b))))
