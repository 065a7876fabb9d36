"""The decode projection sweep (C ABI w4a16_sweep_*) at the benchmark's full size against the CPU
oracle, and its size-independent properties."""
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


@pytest.fixture(scope="module")
def model():
    import bench
    layers_np = bench.make_layers_np(28)
    return layers_np, bench.upload_layers(layers_np)


def test_full_size_sweep_matches_oracle_layer_by_layer(ops, model):
    """28 layers, benchmark shapes.  Each layer is run alone on the device from the oracle's hidden
    state entering it (so a 1-ulp difference cannot snowball through later quantisers) and compared
    with the oracle's hidden state leaving it."""
    from qwen_engine_b200 import synth
    layers_np, layers_dev = model
    h0 = synth.activations(7, "h0", synth.HIDDEN)
    _, trace = oracle.decode_sweep(layers_np, h0, collect=True)
    h_in = torch.empty(synth.HIDDEN, dtype=torch.float16, device="cuda")
    h_out = torch.empty_like(h_in)
    worst = 0.0
    for l, t in enumerate(trace):
        one = ops.DecodeSweep(layers_dev[l:l + 1])
        h_in.copy_(util.to_dev(t["h_in"]))
        one.run_device(h_in, h_out)
        torch.cuda.synchronize()
        got = util.to_np(h_out)
        # intermediate buffers of the layer: q projection and MLP activation
        rep = util.error_report(got, t["h_out"].astype(np.float64))
        assert rep["finite"]
        # the oracle value is itself fp16-rounded: agreement within 2 fp16 steps of the final add,
        # and the path's stated tolerance
        assert rep["max_rel"] <= 1e-2, (l, rep)
        assert rep["median_ulp"] <= 2.0, (l, rep)
        worst = max(worst, rep["max_ulp"])
        one.close()
    assert worst <= 8.0


def test_sweep_is_deterministic_and_host_path_equals_device_path(ops, model):
    from qwen_engine_b200 import synth
    _, layers_dev = model
    sweep = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_SEPARATE)
    assert sweep.launches == 28 * 8
    h0 = synth.activations(7, "h0", synth.HIDDEN)
    h_in = util.to_dev(h0)
    a, b = torch.empty_like(h_in), torch.empty_like(h_in)
    sweep.run_device(h_in, a)
    sweep.run_device(h_in, b)
    pin_in, pin_out = torch.from_numpy(h0).pin_memory(), torch.empty(synth.HIDDEN, dtype=torch.float16).pin_memory()
    sweep.run_host(pin_in, pin_out)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert np.array_equal(util.to_np(a).view(np.uint16), pin_out.numpy().view(np.uint16))
    assert np.isfinite(pin_out.numpy().astype(np.float32)).all()
    sweep.close()


def test_row_split_consistency_at_full_size(ops):
    """Rows are independent: the lm_head GEMV computed as 8 row slabs equals the one-launch result
    bit for bit (the property the multi-GPU split relies on)."""
    from qwen_engine_b200 import synth
    N, K = synth.SHAPES["lm_head"]
    qw, sc = synth.packed_weights(2, "lm", N, K), synth.scales(2, "lm", N, K)
    x = util.to_dev(synth.activations(2, "lmx", K))
    q8 = torch.empty(K, dtype=torch.int8, device="cuda")
    xs = torch.empty(K // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(K // 8, dtype=torch.int32, device="cuda")
    ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, K)
    d_qw, d_sc = util.to_dev(qw), util.to_dev(sc)
    full = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(d_qw, d_sc, q8, xs, s8, None, full, N, K)
    parts = torch.empty(N, dtype=torch.float16, device="cuda")
    rows = N // 8
    for r in range(8):
        w_slab = d_qw[r * rows:(r + 1) * rows].contiguous()
        s_slab = d_sc[r * rows:(r + 1) * rows].contiguous()
        ops.launch_gemv_w4a8(w_slab, s_slab, q8, xs, s8, None, parts[r * rows:(r + 1) * rows], rows, K)
    torch.cuda.synchronize()
    assert torch.equal(full, parts)


@pytest.mark.parametrize("flags", [1, 2, 4, 7])
def test_fused_sweeps_give_the_bits_of_the_separate_launch_sequence(ops, model, flags):
    """Folding the RMSNorm / Q8_1 launches into the GEMV prologues must not change a single bit."""
    from qwen_engine_b200 import synth
    _, layers_dev = model
    h_in = util.to_dev(synth.activations(7, "h0", synth.HIDDEN))
    ref_sweep = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_SEPARATE)
    fused = ops.DecodeSweep(layers_dev, flags=flags)
    assert fused.launches == 28 * (8 - bin(flags).count("1") - (1 if flags & 1 else 0))
    a, b = torch.empty_like(h_in), torch.empty_like(h_in)
    ref_sweep.run_device(h_in, a)
    fused.run_device(h_in, b)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    ref_sweep.close()
    fused.close()


@pytest.mark.parametrize("seed,flags", [(7, 32), (8, 64), (9, 96)])
def test_sweep_with_published_reductions_gives_the_same_bits(ops, model, seed, flags):
    """Producers publishing what their consumers would reduce again (sum of squares for the next RMSNorm by the O
    and down launches, |max| per group of 128 by the gate_up launch) removes the quantiser launch and the
    reductions from the prologues without changing a bit; replays of the graph (which clear and refill the
    published words every layer) agree with each other."""
    from qwen_engine_b200 import synth
    _, layers_dev = model
    h_in = util.to_dev(synth.activations(seed, "h0", synth.HIDDEN))
    ref_sweep = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_SEPARATE)
    fused = ops.DecodeSweep(layers_dev, flags=flags)
    assert fused.launches == 28 * (4 if flags & ops.SWEEP_PUBLISH_AMAX else 5)
    a, b = torch.empty_like(h_in), torch.empty_like(h_in)
    ref_sweep.run_device(h_in, a)
    for _ in range(4):
        fused.run_device(h_in, b)
        torch.cuda.synchronize()
        assert torch.equal(a, b)
    ref_sweep.close()
    fused.close()


@pytest.mark.parametrize("flags", [16, 19, 23])
def test_sweep_with_q8_1_written_by_gate_up_gives_the_same_bits(ops, model, flags):
    """The gate_up launch quantising its own output (clusters of four CTAs per group of 128) replaces the
    quantiser launch in front of down without changing a bit of the hidden state."""
    from qwen_engine_b200 import synth
    _, layers_dev = model
    h_in = util.to_dev(synth.activations(7, "h0", synth.HIDDEN))
    ref_sweep = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_SEPARATE)
    fused = ops.DecodeSweep(layers_dev, flags=flags)
    assert fused.launches == 28 * (8 - (2 if flags & 1 else 0) - (1 if flags & 2 else 0) - 1)
    a, b = torch.empty_like(h_in), torch.empty_like(h_in)
    ref_sweep.run_device(h_in, a)
    for _ in range(3):      # replays must agree with each other too
        fused.run_device(h_in, b)
        torch.cuda.synchronize()
        assert torch.equal(a, b)
    ref_sweep.close()
    fused.close()


@pytest.mark.parametrize("H,I,norm", [(1536, 8960, True), (1024, 1280, True), (512, 128, False), (2048, 4864, True)])
def test_gate_up_q8_1_epilogue_equals_the_standalone_quantiser(ops, H, I, norm):
    from qwen_engine_b200 import synth
    x = util.to_dev((synth.activations(41, "fx", H).astype(np.float32) * 3).astype(np.float16))
    gamma = util.to_dev((1 + 0.1 * synth.activations(42, "fg", H).astype(np.float32)).astype(np.float16)) if norm else None
    gw, gs = util.to_dev(synth.packed_weights(43, "gu", 2 * I, H)), util.to_dev(synth.scales(43, "gu", 2 * I, H))
    y = torch.empty(I, dtype=torch.float16, device="cuda")
    q8 = torch.full((I,), 99, dtype=torch.int8, device="cuda")
    xs = torch.full((I // 128,), -1.0, dtype=torch.float32, device="cuda")
    s8 = torch.full((I // 8,), 12345, dtype=torch.int32, device="cuda")
    ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(gw, gs, x, gamma, y, q8, xs, s8, H, I)
    # the two-launch form: fused gate_up (same output to within the summation order), then the quantiser on y
    y_ref = torch.empty_like(y)
    ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(gw, gs, x, gamma, y_ref, H, I)
    q8r, xsr, s8r = torch.empty_like(q8), torch.empty_like(xs), torch.empty_like(s8)
    ops.launch_quantize_fp16_to_q8_1(y, q8r, xsr, s8r, I)
    torch.cuda.synchronize()
    assert torch.equal(q8, q8r) and torch.equal(xs, xsr) and torch.equal(s8, s8r)
    util.assert_fp16_close(util.to_np(y), util.to_np(y_ref).astype(np.float64), what="gate_up with Q8_1 epilogue")
    if I // 32 >= 193:   # same CTA shape as the plain launch: same bits
        assert torch.equal(y, y_ref)
    # a width that is not a whole number of groups is refused
    with pytest.raises(ops.W4A16Error):
        ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(gw, gs, x, gamma, y, q8, xs, s8, H, I - 64)


def test_fused_entry_points_equal_two_call_sequences(ops):
    from qwen_engine_b200 import synth
    H, I = 1536, 8960
    x = util.to_dev((synth.activations(31, "fx", H).astype(np.float32) * 3).astype(np.float16))
    gamma = util.to_dev((1 + 0.1 * synth.activations(32, "fg", H).astype(np.float32)).astype(np.float16))
    q8 = torch.empty(H, dtype=torch.int8, device="cuda")
    xs = torch.empty(H // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(H // 8, dtype=torch.int32, device="cuda")
    ops.launch_rmsnorm_q8_1(x, gamma, None, q8, xs, s8, None, H)
    # gate_up + SwiGLU
    gw, gs = util.to_dev(synth.packed_weights(33, "gu", 2 * I, H)), util.to_dev(synth.scales(33, "gu", 2 * I, H))
    y1, y2 = torch.empty(I, dtype=torch.float16, device="cuda"), torch.empty(I, dtype=torch.float16, device="cuda")
    ops.launch_gemv_dual_gate_up_swiglu_w4a8(gw, gs, q8, xs, s8, y1, H, I)
    ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(gw, gs, x, gamma, y2, H, I)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    # plain GEMV with residual (lm_head / O style)
    N = 3000
    w, s = util.to_dev(synth.packed_weights(34, "p", N, H)), util.to_dev(synth.scales(34, "p", N, H))
    r = util.to_dev(synth.activations(35, "r", N))
    z1, z2 = torch.empty(N, dtype=torch.float16, device="cuda"), torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(w, s, q8, xs, s8, r, z1, N, H)
    ops.launch_gemv_rmsnorm_w4a16(w, s, x, gamma, r, z2, N, H)
    torch.cuda.synchronize()
    assert torch.equal(z1, z2)
    # fused QKV
    dims = [1536, 256, 256]
    ws = [(util.to_dev(synth.packed_weights(36, f"t{i}", n, H)), util.to_dev(synth.scales(36, f"t{i}", n, H)))
          for i, n in enumerate(dims)]
    oa = [torch.empty(n, dtype=torch.float16, device="cuda") for n in dims]
    ob = [torch.empty(n, dtype=torch.float16, device="cuda") for n in dims]
    mk = lambda o: ops.QKVProjectionView(ws[0][0], ws[0][1], o[0], ws[1][0], ws[1][1], o[1], ws[2][0], ws[2][1], o[2])
    ops.launch_gemv_qkv_w4a8(mk(oa), q8, xs, s8)
    ops.launch_gemv_qkv_rmsnorm_w4a16(mk(ob), x, gamma)
    torch.cuda.synchronize()
    for ta, tb in zip(oa, ob):
        assert torch.equal(ta, tb)


def test_persistent_sweep_matches_oracle_layer_by_layer(ops, model):
    """The one-kernel form of the sweep (all CTAs resident, weights streamed through a shared-memory
    ring, activations exchanged as tagged words): each layer from the oracle's input, as above."""
    from qwen_engine_b200 import synth
    layers_np, layers_dev = model
    h0 = synth.activations(7, "h0", synth.HIDDEN)
    _, trace = oracle.decode_sweep(layers_np, h0, collect=True)
    h_in = torch.empty(synth.HIDDEN, dtype=torch.float16, device="cuda")
    h_out = torch.empty_like(h_in)
    for l, t in enumerate(trace[:6] + trace[-2:]):
        idx = l if l < 6 else len(trace) - 8 + l
        one = ops.DecodeSweep(layers_dev[idx:idx + 1], flags=ops.SWEEP_PERSISTENT)
        assert one.launches == 1
        h_in.copy_(util.to_dev(t["h_in"]))
        one.run_device(h_in, h_out)
        torch.cuda.synchronize()
        assert one.status() == 0
        rep = util.error_report(util.to_np(h_out), t["h_out"].astype(np.float64))
        assert rep["finite"]
        assert rep["max_rel"] <= 1e-2, (idx, rep)
        assert rep["median_ulp"] <= 2.0, (idx, rep)
        one.close()


def test_persistent_sweep_full_depth_is_deterministic_and_close_to_the_launch_sequence(ops, model):
    from qwen_engine_b200 import synth
    _, layers_dev = model
    h_in = util.to_dev(synth.activations(7, "h0", synth.HIDDEN))
    graph = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_FUSE_ALL)
    pers = ops.DecodeSweep(layers_dev, flags=ops.SWEEP_PERSISTENT)
    a, b, c = torch.empty_like(h_in), torch.empty_like(h_in), torch.empty_like(h_in)
    graph.run_device(h_in, a)
    pers.run_device(h_in, b)
    pers.run_device(h_in, c)     # second launch: new tags over the same exchange buffers
    torch.cuda.synchronize()
    assert pers.status() == 0
    assert torch.equal(b, c)
    x, y = util.to_np(a).astype(np.float64), util.to_np(b).astype(np.float64)
    assert np.isfinite(y).all()
    # 28 layers of re-quantisation amplify one-ulp differences in the fp32 summation order; the two
    # forms must still describe the same vector
    rms = np.sqrt(np.mean(x * x))
    assert np.sqrt(np.mean((x - y) ** 2)) <= 0.05 * rms
    graph.close()
    pers.close()


def test_persistent_sweep_recovers_after_a_wait_that_ran_out(ops, model):
    """A bounded wait of the persistent kernel is made to run out on the host side of the protocol only: with a
    limit of one poll a CTA gives up on the first counter or tagged word that is not there yet.  The kernel must
    return, report it, and -- because the status call re-bases tags and counters -- the next pass with the usual
    limit must be clean and give the bits of an undisturbed sweep."""
    from qwen_engine_b200 import synth
    _, layers_dev = model
    h_in = util.to_dev(synth.activations(11, "h0", synth.HIDDEN))
    ref = ops.DecodeSweep(layers_dev[:4], flags=ops.SWEEP_PERSISTENT)
    want = torch.empty_like(h_in)
    ref.run_device(h_in, want)
    torch.cuda.synchronize()
    assert ref.status() == 0
    ref.close()
    pers = ops.DecodeSweep(layers_dev[:4], flags=ops.SWEEP_PERSISTENT)
    out = torch.empty_like(h_in)
    usual = ops.get_option(ops.OPT_SIGNAL_WAIT_SPINS)
    try:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, 1)
        pers.run_device(h_in, out)
        torch.cuda.synchronize()
        assert pers.status() != 0          # reported, and re-based by the same call
    finally:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, usual)
    for _ in range(2):
        pers.run_device(h_in, out)
        torch.cuda.synchronize()
        assert pers.status() == 0
        assert torch.equal(out, want)
    pers.close()
