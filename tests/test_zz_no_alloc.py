"""The GEMV entry point that brings its own scratch (w4a16_gemv_w4a16_static_scratch).

Some hosts of this library cannot give it a scratch buffer and may not allocate one: an engine
that spent its device-memory budget on one arena at start-up, a plugin interface that rules out
allocation calls while serving.  For them the Q8_1 form of the activation is kept in a fixed
array inside the library.  This file checks, through the C ABI, that the result is the one the
ordinary fp16-input entry point gives -- twice in a row with different shapes, so that whatever
the first call left in the shared array cannot leak into the second -- and that a vector longer
than the array is refused.

It is named to be collected last: a run that stops at the first failure has then already
executed every other test.
"""
import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _case(ops, seed, N, K, with_residual):
    from qwen_engine_b200 import synth
    qw = util.to_dev(synth.packed_weights(seed, "na", N, K))
    sc = util.to_dev(synth.scales(seed, "na", N, K))
    x = util.to_dev(synth.activations(seed, "na.x", K))
    res = util.to_dev(synth.activations(seed, "na.r", N)) if with_residual else None
    want = torch.empty(N, dtype=torch.float16, device="cuda")
    got = torch.full((N + 16,), float("nan"), dtype=torch.float16, device="cuda")
    ops.launch_gemv_w4a16(qw, sc, x, res, want, N, K)
    ops.gemv_w4a16_static_scratch(qw, sc, x, res, got, N, K)
    torch.cuda.synchronize()
    assert np.isnan(util.to_np(got)[N:]).all(), "wrote past the output"
    # same integers, same fp32 order as the existing entry point: identical fp16 bits
    assert torch.equal(got[:N], want)


def test_static_scratch_gemv_matches_existing_entry_point_twice_in_a_row():
    import qwen_engine_b200 as ops
    ops.init()
    _case(ops, 101, 1536, 8960, True)    # long vector first: fills most of what later calls could see
    _case(ops, 102, 2000, 1536, False)   # shorter vector next: stale tail of the array must not matter
    _case(ops, 103, 1536, 8960, True)


def test_static_scratch_gemv_refuses_vectors_beyond_the_array():
    import qwen_engine_b200 as ops
    ops.init()
    K = 32768 + 256
    w = torch.zeros(8 * K // 8, dtype=torch.int32, device="cuda")
    s = torch.zeros(8 * K // 128, dtype=torch.float16, device="cuda")
    x = torch.zeros(K, dtype=torch.float16, device="cuda")
    y = torch.full((8,), 7.0, dtype=torch.float16, device="cuda")
    with pytest.raises(ops.W4A16Error) as e:
        ops.gemv_w4a16_static_scratch(w, s, x, None, y, 8, K)
    assert e.value.status == -5
    torch.cuda.synchronize()
    assert (y == 7.0).all(), "a refused call must not launch anything"
    # the largest accepted size still works
    K = 32768
    ops.gemv_w4a16_static_scratch(w[:8 * K // 8], s[:8 * K // 128], x[:K], None, y, 8, K)
    torch.cuda.synchronize()
    assert (y == 0.0).all()


def test_static_scratch_gemv_allocates_no_device_memory():
    """The claim in the entry point's name: once the first call on the device has looked up the array's address,
    further calls leave the device's free memory and torch's allocator untouched -- measured around the calls
    themselves, with every tensor made beforehand -- and the in-place form (residual == output) that the
    ordinary GEMV allows works here too."""
    import ctypes
    import qwen_engine_b200 as ops
    from qwen_engine_b200 import synth
    ops.init()
    N, K = 1536, 8960
    qw = util.to_dev(synth.packed_weights(104, "na", N, K))
    sc = util.to_dev(synth.scales(104, "na", N, K))
    x = util.to_dev(synth.activations(104, "na.x", K))
    res = util.to_dev(synth.activations(104, "na.r", N))
    want, got = res.clone(), res.clone()
    ops.launch_gemv_w4a16(qw, sc, x, want, want, N, K)
    ops.gemv_w4a16_static_scratch(qw, sc, x, None, torch.empty_like(got), N, K)     # warm-up: first call set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(5):
        got.copy_(res)
        ops.gemv_w4a16_static_scratch(qw, sc, x, got, got, N, K)                    # in place
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    assert torch.equal(got, want)
