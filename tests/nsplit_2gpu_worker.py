"""Worker of tests/test_gpu_nsplit_multi.py: one process per GPU (launched with RANK / WORLD_SIZE / MASTER_* set).

Runs the row-split GEMV in its barrier-free form, in its barrier form, and the row-split prefill GEMM for several
steps back to back with a different activation per step, while rank 1 is made SLOW: a long sleep kernel sits
between its GEMV and whatever reads the gathered result.  A fast rank that ran ahead and overwrote data a slow
rank had not read yet would show up as a step whose result is not the reference's (an NCCL all-gather of plain
launches).  Prints "OK <rank>" on success.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    import qwen_engine_b200 as ops
    from qwen_engine_b200 import nsplit, synth
    ops.init()
    slow = rank == 1
    sleep_cycles = 4_000_000      # about 2 ms

    # ---- GEMV: 80000 x 1536, rows split over the ranks ----
    N, K = 80000, 1536
    slab = nsplit.slab_bounds(N, world, rank, 8)
    qw = torch.from_numpy(synth.packed_weights(3, f"mg.r{slab.first}", slab.rows, K).view(np.int32)).cuda()
    sc = torch.from_numpy(synth.scales(3, f"mg.r{slab.first}", slab.rows, K)).cuda()
    steps = 6
    xs_all = [torch.from_numpy(synth.activations(100 + s, "mgx", K)).cuda() for s in range(steps)]
    q8 = torch.empty(K, dtype=torch.int8, device="cuda")
    xs = torch.empty(K // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(K // 8, dtype=torch.int32, device="cuda")

    def reference(step):
        ops.launch_quantize_fp16_to_q8_1(xs_all[step], q8, xs, s8, K)
        mine = torch.zeros(slab.stride, dtype=torch.float16, device="cuda")
        ops.launch_gemv_w4a8(qw, sc, q8, xs, s8, None, mine, slab.rows, K)
        full = torch.empty(world * slab.stride, dtype=torch.float16, device="cuda")
        dist.all_gather_into_tensor(full, mine)
        return full[:N].clone()

    refs = [reference(s) for s in range(steps)]
    torch.cuda.synchronize()

    def slow_gather(*args):
        if slow:
            torch.cuda._sleep(sleep_cycles)
        ops.gather_after_signals(*args)

    sig = nsplit.NSplitSignalGemv(qw, sc, N, K, ops.gemv_w4a8_peers_signal, slow_gather, align=8)
    got = []
    for s in range(steps):      # no host synchronisation between the steps: the ranks drift apart
        ops.launch_quantize_fp16_to_q8_1(xs_all[s], q8, xs, s8, K)
        got.append(sig.forward(q8, xs, s8).clone())
    torch.cuda.synchronize()
    assert int(sig.status.item()) == 0, "a signal wait ran out"
    for s in range(steps):
        assert torch.equal(got[s], refs[s]), f"signal form, step {s}, rank {rank}"

    launch = lambda w, s_, a, b, c, out, r, k: ops.launch_gemv_w4a8(w, s_, a, b, c, None, out, r, k)
    peer_launch = lambda w, s_, a, b, c, out, peers, r, k: ops.gemv_w4a8_peers(w, s_, a, b, c, out, peers, r, k)
    bar = nsplit.NSplitGemv(qw, sc, N, K, launch, align=8, peer_launch=peer_launch)
    got = []
    for s in range(steps):
        ops.launch_quantize_fp16_to_q8_1(xs_all[s], q8, xs, s8, K)
        y = bar.forward(q8, xs, s8)
        if slow:
            torch.cuda._sleep(sleep_cycles)     # a slow reader of the gathered vector
        got.append(y[:N].clone())
    torch.cuda.synchronize()
    for s in range(steps):
        assert torch.equal(got[s], refs[s]), f"barrier form, step {s}, rank {rank}"

    # ---- prefill GEMM: 2048 -> 4096 at 512 tokens, weight rows split, peer stores from the pair kernel ----
    Ng, Kg, M = 8192, 2048, 512
    gslab = nsplit.slab_bounds(Ng, world, rank, 256)
    gw = torch.from_numpy(synth.packed_weights(5, f"mm.r{gslab.first}", gslab.rows, Kg).view(np.int32)).cuda()
    gs = torch.from_numpy(synth.scales(5, f"mm.r{gslab.first}", gslab.rows, Kg)).cuda()
    xg = [torch.from_numpy(synth.activations(200 + s, "mmx", M, Kg)).cuda() for s in range(3)]
    launch_g = lambda w, s_, xx, out, m, rows, k: ops.launch_gemm_prefill_w4a16(w, s_, xx, None, out, m, rows, k)
    block_g = lambda w, s_, xx, ptr, ldc, peers, m, rows, k: ops.gemm_prefill_w4a16_block(w, s_, xx, None, ptr, ldc, peers, m, rows, k)
    plain = nsplit.NSplitGemm(gw, gs, Ng, Kg, M, launch_g)
    fused = nsplit.NSplitGemm(gw, gs, Ng, Kg, M, launch_g, block_launch=block_g)
    want = [plain.forward(x, M).clone() for x in xg]
    got = []
    for x in xg:
        y = fused.forward(x, M)
        if slow:
            torch.cuda._sleep(sleep_cycles)
        got.append(y.clone())
    torch.cuda.synchronize()
    for s in range(3):
        a, b = got[s].float(), want[s].float()
        step_size = torch.maximum(b.abs(), torch.tensor(1.0, device="cuda")) * 2.0 ** -10
        assert bool(((a - b).abs() <= step_size).all()), f"prefill, step {s}, rank {rank}"
    assert ops.debug_counter(0) == 0
    print(f"OK {rank}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
