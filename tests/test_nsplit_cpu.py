"""Host logic of the output-row split (qwen_engine_b200/nsplit.py) with two gloo ranks on CPU:
slab bounds, one slab per rank in its own allocation, equal-sized all-gather, padded tail.
The local GEMV is played by the CPU oracle here; on GPUs it is the CUDA launcher."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from qwen_engine_b200 import nsplit, synth


def test_slab_bounds_cover_all_rows_once():
    for n, world, align in [(151936, 8, 1), (151936, 4, 1), (1000, 3, 1), (17920, 8, 2), (2048, 3, 128), (5, 8, 1)]:
        seen = []
        stride = None
        for r in range(world):
            s = nsplit.slab_bounds(n, world, r, align)
            stride = stride or s.stride
            assert s.stride == stride and s.rows >= 0 and s.first % align == 0
            seen += list(range(s.first, s.first + s.rows))
        assert seen == list(range(n))
    with pytest.raises(ValueError):
        nsplit.slab_bounds(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_launch(qw, sc, q8, xs, s8, out, rows, K):
    _, y16 = oracle.gemv_q8(qw.numpy().view(np.uint32), sc.numpy(), q8.numpy(), xs.numpy(), threads=1)
    out[:rows] = torch.from_numpy(y16)


def _worker(rank, world, port, n_rows, K, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qw = synth.packed_weights(5, "ns", n_rows, K)
        sc = synth.scales(5, "ns", n_rows, K)
        x = synth.activations(5, "ns.x", K)
        q8, xs, s8 = oracle.quantize_q8_1(x)
        slab = nsplit.slab_bounds(n_rows, world, rank)
        w_slab = torch.from_numpy(qw[slab.first:slab.first + slab.rows].view(np.int32).copy())
        s_slab = torch.from_numpy(sc[slab.first:slab.first + slab.rows].copy())
        op = nsplit.NSplitGemv(w_slab, s_slab, n_rows, K, _oracle_launch)
        y = op.forward(torch.from_numpy(q8), torch.from_numpy(xs), torch.from_numpy(s8))
        _, full = oracle.gemv_q8(qw, sc, q8, xs, threads=1)
        ret[rank] = bool(np.array_equal(y.numpy().view(np.uint16), full.view(np.uint16)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [512, 515])     # divisible and padded-tail cases
def test_two_rank_gloo_split_equals_unsplit(n_rows):
    world, K = 2, 256
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, n_rows, K, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert dict(ret) == {0: True, 1: True}


# ---- token selection over a row-split lm_head: candidates per rank, 8 bytes each, instead of the logits ----

def _oracle_candidates(qw, sc, q8, xs, s8, val, idx, control, offset, rows, K):
    """Plays the GEMV with the sampling epilogue: `slots` contiguous row chunks, one candidate each."""
    _, y16 = oracle.gemv_q8(qw.numpy().view(np.uint32), sc.numpy(), q8.numpy(), xs.numpy(), threads=1)
    slots = val.numel()
    chunk = -(-rows // slots)
    for j in range(slots):
        lo, hi = j * chunk, min((j + 1) * chunk, rows)
        if lo >= hi:
            val[j], idx[j] = float("-inf"), 0
            continue
        tok, best, _ = oracle.sample(y16[lo:hi], control["temperature"], control["rng_seed"], control["seq_pos"],
                                     index_offset=offset + lo)
        val[j], idx[j] = best, tok


def _oracle_finish(allv, alli, count, control, token):
    v, i = allv.numpy()[:count], alli.numpy()[:count]
    order = np.lexsort((i, -v.astype(np.float64)))     # larger score first, then smaller index
    token[0] = int(i[order[0]])
    control["seq_pos"] += 1


def _sampler_worker(rank, world, port, n_rows, K, temperature, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qw = synth.packed_weights(6, "nss", n_rows, K)
        sc = synth.scales(6, "nss", n_rows, K)
        qw[n_rows - 2] = qw[1]          # equal logits in different slabs: the lower index has to win
        sc[n_rows - 2] = sc[1]
        q8, xs, s8 = oracle.quantize_q8_1(synth.activations(6, "nss.x", K))
        slab = nsplit.slab_bounds(n_rows, world, rank)
        w_slab = torch.from_numpy(qw[slab.first:slab.first + slab.rows].view(np.int32).copy())
        s_slab = torch.from_numpy(sc[slab.first:slab.first + slab.rows].copy())
        control = {"temperature": temperature, "rng_seed": 77, "seq_pos": 3}
        op = nsplit.NSplitSampler(w_slab, s_slab, n_rows, K, 5, _oracle_candidates, _oracle_finish)
        tok = int(op.forward(torch.from_numpy(q8), torch.from_numpy(xs), torch.from_numpy(s8), control)[0])
        _, full = oracle.gemv_q8(qw, sc, q8, xs, threads=1)
        expect, _, _ = oracle.sample(full, temperature, 77, 3)
        ret[rank] = (tok, expect, control["seq_pos"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows,temperature", [(512, 0.0), (515, 0.9), (3, 0.0)])
def test_two_rank_gloo_split_sampler_picks_the_unsplit_token(n_rows, temperature):
    world, K = 2, 256
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_sampler_worker, args=(r, world, port, n_rows, K, temperature, ret))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        got = dict(ret)
        assert got[0] == got[1]                      # every rank ends with the same token
        assert got[0][0] == got[0][1] and got[0][2] == 4


# ---- M-token contraction split by weight rows: column blocks gathered side by side ----

def _oracle_gemm_launch(qw, sc, x, out, M, rows, K):
    _, y16 = oracle.gemm_prefill(qw.numpy().view(np.uint32), sc.numpy(), x.numpy(), np.arange(M, dtype=np.int32),
                                 np.arange(rows, dtype=np.int32))
    out.copy_(torch.from_numpy(y16))


def _gemm_worker(rank, world, port, n_rows, K, M, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        qw = synth.packed_weights(7, "nsg", n_rows, K)
        sc = synth.scales(7, "nsg", n_rows, K)
        x = synth.activations(7, "nsg.x", M, K)
        slab = nsplit.slab_bounds(n_rows, world, rank, 128)
        w_slab = torch.from_numpy(qw[slab.first:slab.first + slab.rows].view(np.int32).copy())
        s_slab = torch.from_numpy(sc[slab.first:slab.first + slab.rows].copy())
        op = nsplit.NSplitGemm(w_slab, s_slab, n_rows, K, 8, _oracle_gemm_launch)
        y = op.forward(torch.from_numpy(x), M)
        _, full = oracle.gemm_prefill(qw, sc, x, np.arange(M, dtype=np.int32), np.arange(n_rows, dtype=np.int32))
        ret[rank] = bool(y.shape == (M, n_rows) and np.array_equal(y.contiguous().numpy().view(np.uint16), full.view(np.uint16)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [512, 300])     # two full slabs; a ragged second slab (256 + 44)
def test_two_rank_gloo_split_gemm_equals_unsplit(n_rows):
    world, K, M = 2, 256, 5
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_gemm_worker, args=(r, world, port, n_rows, K, M, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert dict(ret) == {0: True, 1: True}
