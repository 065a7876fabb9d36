"""Token selection after lm_head: the stand-alone sampler and the lm_head GEMV that samples in its epilogue,
against the CPU oracle (oracle.sample) and against each other."""
import numpy as np
import pytest
import torch

import oracle
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import qwen_engine_b200 as pkg
    pkg.init()
    return pkg


def _scratch(n):
    return (torch.full((n,), float("nan"), dtype=torch.float32, device="cuda"),
            torch.full((n,), -7, dtype=torch.int32, device="cuda"))


def _check_token(tok, logits, temperature, seed, seq_pos):
    """Greedy: the oracle's token exactly.  With noise the device's logf may differ from libm's in the last
    bit, so the chosen entry must score within a few ulp of the oracle's best."""
    ref_tok, ref_best, scores = oracle.sample(logits, temperature, seed, seq_pos)
    if temperature <= 1e-5:
        assert tok == ref_tok
    else:
        assert tok == ref_tok or abs(scores[tok] - ref_best) <= 4e-6 * max(1.0, abs(ref_best))


@pytest.mark.parametrize("vocab", [151936, 1000, 77, 1])
@pytest.mark.parametrize("temperature,seed,seq_pos", [(0.0, 0, 0), (0.7, 0x1234567890ABCDEF, 17), (1.3, 42, 100000)])
def test_sample_and_advance_matches_oracle(ops, vocab, temperature, seed, seq_pos):
    rng = np.random.default_rng(vocab)
    logits = (rng.standard_normal(vocab) * 4).astype(np.float16)
    if vocab > 50:   # ties at the top: the lowest index must win
        top = np.float16(logits.max() + 1)
        logits[[vocab // 3, vocab // 2, vocab - 1]] = top
    d_logits = util.to_dev(logits)
    val, idx = _scratch(256)
    control = ops.make_sample_control(temperature, seed, seq_pos)
    token = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    ops.launch_sample_and_advance(d_logits, val, idx, control, token, None, vocab)
    torch.cuda.synchronize()
    tok = int(token.item())
    _check_token(tok, logits, temperature, seed, seq_pos)
    if temperature == 0.0 and vocab > 50:
        assert tok == vocab // 3
    after = ops.read_sample_control(control)
    assert after["token_id"] == tok and after["seq_pos"] == seq_pos + 1
    assert after["rng_seed"] == (seed + 0x9E3779B97F4A7C15) % 2**64
    # without a control block: greedy, token only through the pointer
    ops.launch_sample_and_advance(d_logits, val, idx, None, token, None, vocab)
    torch.cuda.synchronize()
    assert int(token.item()) == oracle.sample(logits)[0]


@pytest.mark.parametrize("N,K", [(151936, 1536), (5000, 1024), (97, 512), (32, 256)])
@pytest.mark.parametrize("temperature,seed,seq_pos", [(0.0, 0, 0), (0.9, 987654321, 3)])
def test_lm_head_with_sampling_epilogue(ops, N, K, temperature, seed, seq_pos):
    from qwen_engine_b200 import synth
    qw, sc = synth.packed_weights(N + K, "lm", N, K), synth.scales(N + K, "lm", N, K)
    if N >= 97:   # two identical rows: identical logits, the lower index must win if they are the best
        qw[N - 1] = qw[5]
        sc[N - 1] = sc[5]
    x = synth.activations(N, "x", K)
    q8, xs, s8 = oracle.quantize_q8_1(x)
    d = [util.to_dev(t) for t in (qw, sc, q8, xs, s8)]
    # the plain launch, for the logits themselves
    logits = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(d[0], d[1], d[2], d[3], d[4], None, logits, N, K)
    # the fused launch, with and without storing the logits
    slots = ops.sample_slots(N)
    assert 1 <= slots <= 2 * torch.cuda.get_device_properties(0).multi_processor_count
    tokens, controls, fused_logits = [], [], None
    for keep_logits in (True, False):
        fval, fidx = _scratch(slots)
        c2 = ops.make_sample_control(temperature, seed, seq_pos)
        t2 = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        logits2 = torch.full((N,), float("nan"), dtype=torch.float16, device="cuda") if keep_logits else None
        ops.launch_gemv_w4a8_sample_and_advance(d[0], d[1], d[2], d[3], d[4], logits2, fval, fidx, c2, t2, N, K)
        torch.cuda.synchronize()
        tokens.append(int(t2.item()))
        controls.append(ops.read_sample_control(c2))
        if keep_logits:
            fused_logits = logits2
    assert tokens[0] == tokens[1] and controls[0] == controls[1]
    # one launch: the GEMV's last CTA reduces the candidates and advances the control block itself
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    c3 = ops.make_sample_control(temperature, seed, seq_pos)
    for rep in range(2):        # twice: the counter wraps back to zero, the control block moves on
        fval, fidx = _scratch(slots)
        t3 = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        ops.launch_gemv_w4a8_sample_one_launch(d[0], d[1], d[2], d[3], d[4], None, fval, fidx, counter, c3, t3, N, K)
        torch.cuda.synchronize()
        assert int(counter.item()) == 0
        if rep == 0:
            assert int(t3.item()) == tokens[0] and ops.read_sample_control(c3) == controls[0]
        else:
            ref_tok, _, scores = oracle.sample(util.to_np(fused_logits), temperature, controls[0]["rng_seed"], seq_pos + 1)
            assert ops.read_sample_control(c3)["seq_pos"] == seq_pos + 2
            if temperature <= 1e-5:
                assert int(t3.item()) == ref_tok
    # the logits it stores are the plain launch's: bit for bit where both use one K slice per row (lm_head),
    # within the path's tolerance where the plain launch splits K inside the CTA
    if K == 1536 and N >= 100000:
        assert torch.equal(fused_logits, logits)
    else:
        util.assert_fp16_close(util.to_np(fused_logits), util.to_np(logits).astype(np.float64), what="fused logits")
    # the stand-alone sampler on those logits: same arithmetic on the device, so the same token and control block
    val, idx = _scratch(256)
    c1 = ops.make_sample_control(temperature, seed, seq_pos)
    t1 = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    ops.launch_sample_and_advance(fused_logits, val, idx, c1, t1, None, N)
    torch.cuda.synchronize()
    assert int(t1.item()) == tokens[0]
    assert ops.read_sample_control(c1) == controls[0]
    _check_token(tokens[0], util.to_np(fused_logits), temperature, seed, seq_pos)


def test_row_split_lm_head_candidates_give_the_same_token(ops):
    """Two slabs of the vocabulary, each scored with its own index offset; the candidates of both go through
    one finishing reduction -- the exchange a row-split lm_head needs is 8 bytes per candidate."""
    from qwen_engine_b200 import synth
    N, K = 20000, 1536
    qw, sc = synth.packed_weights(3, "lm2", N, K), synth.scales(3, "lm2", N, K)
    x = synth.activations(4, "x2", K)
    q8, xs, s8 = oracle.quantize_q8_1(x)
    dq8, dxs, ds8 = util.to_dev(q8), util.to_dev(xs), util.to_dev(s8)
    for temperature, seed in ((0.0, 0), (1.1, 5555)):
        ref_val, ref_idx = _scratch(ops.sample_slots(N))
        c0 = ops.make_sample_control(temperature, seed, 9)
        t0 = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        ops.launch_gemv_w4a8_sample_and_advance(util.to_dev(qw), util.to_dev(sc), dq8, dxs, ds8, None, ref_val, ref_idx,
                                                c0, t0, N, K)
        bounds = [0, 12000, N]
        vals, idxs = [], []
        c = ops.make_sample_control(temperature, seed, 9)
        for lo, hi in zip(bounds[:-1], bounds[1:]):
            n = hi - lo
            v, i = _scratch(ops.sample_slots(n))
            ops.launch_gemv_w4a8_sample_candidates(util.to_dev(qw[lo:hi]), util.to_dev(sc[lo:hi]), dq8, dxs, ds8, None,
                                                   v, i, c, lo, n, K)
            vals.append(v)
            idxs.append(i)
        allv, alli = torch.cat(vals), torch.cat(idxs)
        t = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        ops.launch_sample_finish(allv, alli, allv.numel(), c, t)
        torch.cuda.synchronize()
        assert int(t.item()) == int(t0.item())
        assert ops.read_sample_control(c) == ops.read_sample_control(c0)


def test_sampling_epilogue_refuses_what_it_cannot_run(ops):
    from qwen_engine_b200 import synth
    N, K = 64, 4096   # deeper than the streaming form's eight steps
    qw, sc = util.to_dev(synth.packed_weights(1, "r", N, K)), util.to_dev(synth.scales(1, "r", N, K))
    q8, xs, s8 = oracle.quantize_q8_1(synth.activations(2, "r", K))
    v, i = _scratch(64)
    with pytest.raises(ops.W4A16Error):
        ops.launch_gemv_w4a8_sample_candidates(qw, sc, util.to_dev(q8), util.to_dev(xs), util.to_dev(s8), None, v, i,
                                               None, 0, N, K)


@pytest.mark.parametrize("H,vocab,M", [(1536, 3000, 1), (1536, 3000, 9), (256, 40, 3)])
def test_embed_lookup_matches_the_dequantised_rows(ops, H, vocab, M):
    """Row gather from the W4 table: (q - 8) * scale with one fp16 rounding -- exact, so bit for bit."""
    from qwen_engine_b200 import synth
    qw, sc = synth.packed_weights(H + vocab, "emb", vocab, H), synth.scales(H + vocab, "emb", vocab, H)
    nib = oracle.unpack_nibbles(qw).astype(np.float32) - 8.0                          # [vocab][H], exact in fp16
    table = (nib.astype(np.float16) * np.repeat(sc, 128, axis=1)).astype(np.float16)   # fp16 * fp16, rounded once
    ids = np.array([(7 * i + 3) % vocab for i in range(M)], dtype=np.int32)
    ids[-1] = vocab + 5 if M > 1 else ids[-1]            # out of range -> row 0, as the reference
    out = torch.full((M * H + 8,), float("nan"), dtype=torch.float16, device="cuda")
    ops.launch_embed_lookup_w4a16(util.to_dev(qw), util.to_dev(sc), util.to_dev(ids), out, None, M, None, H, vocab)
    torch.cuda.synchronize()
    got = util.to_np(out)
    assert np.isnan(got[M * H:]).all()
    rows = np.where((ids >= 0) & (ids < vocab), ids, 0)
    assert np.array_equal(got[:M * H].reshape(M, H).view(np.uint16), table[rows].view(np.uint16))
    # token taken from the control block when no id array is given
    control = ops.make_sample_control(0.0, 0, 0, token_id=int(ids[0]))
    ops.launch_embed_lookup_w4a16(util.to_dev(qw), util.to_dev(sc), None, out, control, 1, None, H, vocab)
    torch.cuda.synchronize()
    assert np.array_equal(util.to_np(out)[:H].view(np.uint16), table[ids[0]].view(np.uint16))


def test_peer_store_epilogues_write_the_same_values_everywhere(ops):
    """The two epilogues that also store into peer GPUs' buffers (logit slice; sampling candidates), with
    ordinary local allocations standing in for the peers' mapped memory."""
    from qwen_engine_b200 import synth
    N, K = 6000, 1536
    qw, sc = util.to_dev(synth.packed_weights(8, "p", N, K)), util.to_dev(synth.scales(8, "p", N, K))
    q8, xs, s8 = (util.to_dev(t) for t in oracle.quantize_q8_1(synth.activations(9, "p", K)))
    ref = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a8(qw, sc, q8, xs, s8, None, ref, N, K)
    # logit slices: the local output and three "peers", each at an offset inside a larger gathered buffer
    local = torch.zeros(N, dtype=torch.float16, device="cuda")
    peers = [torch.zeros(3 * N, dtype=torch.float16, device="cuda") for _ in range(3)]
    ops.gemv_w4a8_peers(qw, sc, q8, xs, s8, local, [p.data_ptr() + 2 * N for p in peers], N, K)
    torch.cuda.synchronize()
    assert torch.equal(local, ref)
    for p in peers:
        assert torch.equal(p[N:2 * N], ref) and not p[:N].any() and not p[2 * N:].any()
    # candidates
    slots = ops.sample_slots(N)
    control = ops.make_sample_control(0.6, 31337, 2)
    v0, i0 = _scratch(slots)
    ops.launch_gemv_w4a8_sample_candidates(qw, sc, q8, xs, s8, None, v0, i0, control, 100, N, K)
    v1, i1 = _scratch(slots)
    pv = [torch.zeros(2 * slots, dtype=torch.float32, device="cuda") for _ in range(2)]
    pi = [torch.zeros(2 * slots, dtype=torch.int32, device="cuda") for _ in range(2)]
    ops.gemv_w4a8_sample_candidates_peers(qw, sc, q8, xs, s8, v1, i1, [t.data_ptr() + 4 * slots for t in pv],
                                          [t.data_ptr() + 4 * slots for t in pi], control, 100, N, K)
    torch.cuda.synchronize()
    assert torch.equal(v1, v0) and torch.equal(i1, i0)
    for tv, ti in zip(pv, pi):
        assert torch.equal(tv[slots:], v0) and torch.equal(ti[slots:], i0)
        assert not tv[:slots].any() and not ti[:slots].any()


def test_completion_signal_protocol_on_one_gpu(ops):
    """The signalled form with this GPU standing in for its own peers: candidates and the step number go to the
    local arrays and to two more "peer" arrays; the reduction that waits for the flags finds them set (the
    producing launch is earlier on the stream, so nothing waits across launches here) and gives the token of
    the plain fused form, step after step, alternating halves."""
    from qwen_engine_b200 import synth
    N, K = 9000, 1536
    qw, sc = util.to_dev(synth.packed_weights(21, "sig", N, K)), util.to_dev(synth.scales(21, "sig", N, K))
    slots = ops.sample_slots(N)
    half = slots
    mk = lambda: (torch.full((2 * half,), float("nan"), dtype=torch.float32, device="cuda"),
                  torch.full((2 * half,), -3, dtype=torch.int32, device="cuda"), torch.zeros(3, dtype=torch.int32, device="cuda"))
    lv, li, lf = mk()
    peers = [mk() for _ in range(2)]
    step_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    c_sig = ops.make_sample_control(0.7, 2024, 0)
    c_ref = ops.make_sample_control(0.7, 2024, 0)
    t_sig = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    t_ref = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rv, ri = _scratch(slots)
    for step in range(1, 5):
        q8, xs, s8 = (util.to_dev(t) for t in oracle.quantize_q8_1(synth.activations(30 + step, "sig", K)))
        ops.gemv_w4a8_sample_candidates_signal(qw, sc, q8, xs, s8, lv.data_ptr(), li.data_ptr(),
                                               [p[0].data_ptr() for p in peers], [p[1].data_ptr() for p in peers],
                                               [p[2].data_ptr() + 4 for p in peers], lf.data_ptr() + 4, counter, step_word,
                                               half, c_sig, 0, N, K)
        # flags [0] and [2] play ranks whose launches are done as well
        lf[0] = step; lf[2] = step
        ops.sample_finish_after_signals(lv.data_ptr(), li.data_ptr(), slots, half, lf.data_ptr(), 3, step_word, status,
                                        c_sig, t_sig)
        ops.launch_gemv_w4a8_sample_and_advance(qw, sc, q8, xs, s8, None, rv, ri, c_ref, t_ref, N, K)
        torch.cuda.synchronize()
        assert int(step_word.item()) == step and int(counter.item()) == 0 and int(status.item()) == 0
        assert int(t_sig.item()) == int(t_ref.item())
        assert ops.read_sample_control(c_sig) == ops.read_sample_control(c_ref)
        lo = (step & 1) * half
        assert torch.equal(lv[lo:lo + slots], rv) and torch.equal(li[lo:lo + slots], ri)
        for pv, pi, pf in peers:
            assert torch.equal(pv[lo:lo + slots], rv) and torch.equal(pi[lo:lo + slots], ri) and int(pf[1].item()) == step
        assert int(lf[1].item()) == step


def test_a_flag_that_nothing_sets_makes_the_bounded_wait_run_out(ops):
    """Failure detection without a fault: the reduction waits for three ranks' flags, one of which is never set
    (a rank that did not take part in the step).  With the poll budget cut to about a millisecond
    (W4A16_OPT_SIGNAL_WAIT_SPINS) the kernel must give up, report 1 + the rank it missed in *d_status, still
    reduce the candidates that are there and return -- the context stays usable and the next, complete step
    is served normally."""
    from qwen_engine_b200 import synth
    N, K = 6000, 1536
    qw, sc = util.to_dev(synth.packed_weights(23, "exp", N, K)), util.to_dev(synth.scales(23, "exp", N, K))
    slots = ops.sample_slots(N)
    half = slots
    lv = torch.full((2 * half,), float("nan"), dtype=torch.float32, device="cuda")
    li = torch.full((2 * half,), -3, dtype=torch.int32, device="cuda")
    lf = torch.zeros(3, dtype=torch.int32, device="cuda")
    step_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    c_sig, c_ref = ops.make_sample_control(0.0, 7, 0), ops.make_sample_control(0.0, 7, 0)
    t_sig = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    t_ref = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rv, ri = _scratch(slots)
    old = ops.get_option(ops.OPT_SIGNAL_WAIT_SPINS)
    assert old == 1 << 22
    try:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, 4000)     # 4000 polls of about 0.2 us
        for step, missing in ((1, 2), (2, None)):
            q8, xs, s8 = (util.to_dev(t) for t in oracle.quantize_q8_1(synth.activations(40 + step, "exp", K)))
            ops.gemv_w4a8_sample_candidates_signal(qw, sc, q8, xs, s8, lv.data_ptr(), li.data_ptr(), [], [], [],
                                                   lf.data_ptr() + 4, counter, step_word, half, c_sig, 0, N, K)
            lf[0] = step
            if missing is None:
                lf[2] = step            # the late rank has caught up
            status.zero_()
            t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            ops.sample_finish_after_signals(lv.data_ptr(), li.data_ptr(), slots, half, lf.data_ptr(), 3, step_word,
                                            status, c_sig, t_sig)
            t1.record()
            ops.launch_gemv_w4a8_sample_and_advance(qw, sc, q8, xs, s8, None, rv, ri, c_ref, t_ref, N, K)
            torch.cuda.synchronize()
            if missing is None:
                assert int(status.item()) == 0
            else:
                assert int(status.item()) == 1 + missing          # which rank never signalled
                assert t0.elapsed_time(t1) < 100.0                # gave up after milliseconds, not the default second
            # this rank's own candidates were all there, so the token is still the right one
            assert int(t_sig.item()) == int(t_ref.item())
            assert ops.read_sample_control(c_sig) == ops.read_sample_control(c_ref)
    finally:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, old)
    with pytest.raises(ops.W4A16Error):
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, 0)


def test_signalled_logits_gather_on_one_gpu(ops):
    """The barrier-free row split of a whole output vector, with this GPU standing in for its own peers: rank 1 of
    3 stores its slice into its own gathered vector and into two more "peer" vectors (16-byte stores, two halves
    used in turn) and signals; the gathering kernel waits for the three flags (the other two set by the test) and
    copies the vector out.  Checked against the plain GEMV, step after step; then with one flag left unset and a
    short poll budget the gather must report the missing rank and return."""
    from qwen_engine_b200 import synth
    # tall enough that the plain launch takes the streaming kernel too (same summation order, so the same bits);
    # 76008 rows end in a ragged block of 8
    rows, K, world, rank = 76008, 1536, 3, 1
    stride = rows
    half = world * stride
    qw, sc = util.to_dev(synth.packed_weights(25, "sg", rows, K)), util.to_dev(synth.scales(25, "sg", rows, K))
    mk = lambda: torch.full((2 * half,), float("nan"), dtype=torch.float16, device="cuda")
    local, peers = mk(), [mk(), mk()]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(3)]
    step_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(half, dtype=torch.float16, device="cuda")
    want = torch.empty(rows, dtype=torch.float16, device="cuda")
    off = rank * stride * 2
    for step in range(1, 5):
        q8, xs, s8 = (util.to_dev(t) for t in oracle.quantize_q8_1(synth.activations(50 + step, "sg", K)))
        ops.gemv_w4a8_peers_signal(qw, sc, q8, xs, s8, local.data_ptr() + off, [p.data_ptr() + off for p in peers],
                                   [f.data_ptr() + 4 * rank for f in flags[1:]], flags[0].data_ptr() + 4 * rank, counter,
                                   step_word, half, rows, K)
        # the other two ranks' slices and flags, as their launches would have left them
        lo = (step & 1) * half
        local[lo:lo + stride] = 1.0
        local[lo + 2 * stride:lo + 3 * stride] = 2.0
        flags[0][0] = step
        flags[0][2] = step
        ops.gather_after_signals(local.data_ptr(), half, flags[0].data_ptr(), world, step_word, status, out, half)
        ops.launch_gemv_w4a8(qw, sc, q8, xs, s8, None, want, rows, K)
        torch.cuda.synchronize()
        assert int(step_word.item()) == step and int(counter.item()) == 0 and int(status.item()) == 0
        assert torch.equal(out[stride:2 * stride], want)
        assert bool((out[:stride] == 1.0).all()) and bool((out[2 * stride:] == 2.0).all())
        for p, f in zip(peers, flags[1:]):
            assert torch.equal(p[lo + stride:lo + 2 * stride], want) and int(f[rank].item()) == step
        assert int(flags[0][rank].item()) == step
    # a rank that never signals: bounded wait, status = 1 + rank, the call returns
    old = ops.get_option(ops.OPT_SIGNAL_WAIT_SPINS)
    try:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, 3000)
        flags[0][2] = 0
        ops.gather_after_signals(local.data_ptr(), half, flags[0].data_ptr(), world, step_word, status, out, half)
        torch.cuda.synchronize()
        assert int(status.item()) == 1 + 2
    finally:
        ops.set_option(ops.OPT_SIGNAL_WAIT_SPINS, old)
