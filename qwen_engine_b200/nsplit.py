"""Output-row split of a W4 GEMV over the GPUs of one node (one process per GPU).

The projection path shards along output rows only: rows are independent, a split along K would
need a reduction and would break the fused residual / SwiGLU epilogues.  Each rank owns one
contiguous slab of rows of `qweight` and `scales` in its OWN allocation (slab offsets of the
scale tensor are not 16-byte multiples inside a global tensor), activations are replicated, and
the fp16 output slices are all-gathered (NCCL over NVLink on GPUs; any torch.distributed backend
works, which is how the host logic is tested with gloo on CPU).

The reference engine is single-GPU; this has no counterpart there.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Slab:
    first: int      # first global row of this rank
    rows: int       # rows this rank owns (may be 0 on trailing ranks)
    stride: int     # rows reserved per rank in the gathered buffer (same on all ranks)


def slab_bounds(n_rows: int, world: int, rank: int, align: int = 1) -> Slab:
    """Contiguous, `align`-row-aligned slabs (align=2 keeps gate/up row pairs on one rank, align=head_dim
    keeps attention heads whole).  All ranks reserve `stride` rows so that one equal-sized all-gather works
    for any n_rows."""
    if n_rows <= 0 or world <= 0 or not 0 <= rank < world or align <= 0:
        raise ValueError("bad split arguments")
    stride = math.ceil(n_rows / world / align) * align
    first = min(rank * stride, n_rows)
    return Slab(first, min(first + stride, n_rows) - first, stride)


class NSplitGemv:
    """y[N] = W[N][K] . x, rows split over the ranks of `group`, logits gathered on every rank.

    launch(qweight_slab, scales_slab, q8, xscale, sum8, out_slice, rows, K) runs the local GEMV; on GPUs
    it is `launch_gemv_w4a8` of this package.
    """

    def __init__(self, qweight_slab: torch.Tensor, scales_slab: torch.Tensor, n_rows: int, in_features: int,
                 launch, group=None, align: int = 1, peer_launch=None):
        """peer_launch (optional, GPUs with peer access only): launch(qw, sc, q8, xs, s8, out_slice, peer_ptrs,
        rows, K) whose epilogue also writes the slice into every peer's gathered buffer; the gathered buffer
        then lives in symmetric memory and the all-gather becomes a barrier."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_rows, self.K = n_rows, in_features
        self.slab = slab_bounds(n_rows, self.world, self.rank, align)
        if qweight_slab.shape[0] != self.slab.rows or scales_slab.shape[0] != self.slab.rows:
            raise ValueError(f"rank {self.rank} expects a slab of {self.slab.rows} rows")
        self.qweight, self.scales, self.launch = qweight_slab, scales_slab, launch
        # gathered buffer: world x stride halves; rank r's slice starts at r * stride
        self.peer_launch = peer_launch if self.world > 1 else None
        self.symm = None
        if self.peer_launch is not None:
            import torch.distributed._symmetric_memory as symm_mem
            self.gathered = symm_mem.empty(self.world * self.slab.stride, dtype=torch.float16,
                                           device=qweight_slab.device)
            self.symm = symm_mem.rendezvous(self.gathered, group=group if group is not None else dist.group.WORLD)
            off = self.rank * self.slab.stride * 2          # this rank's slice, in bytes, inside every buffer
            self.peer_ptrs = [int(self.symm.buffer_ptrs[r]) + off for r in range(self.world) if r != self.rank]
        else:
            self.gathered = torch.empty(self.world * self.slab.stride, dtype=torch.float16,
                                        device=qweight_slab.device)

    def local_slice(self) -> torch.Tensor:
        s = self.slab
        return self.gathered[self.rank * s.stride: self.rank * s.stride + s.stride]

    def forward(self, q8, xscale, sum8) -> torch.Tensor:
        """Returns the full fp16 output [n_rows] (a view of the gathered buffer when no padding exists)."""
        mine = self.local_slice()
        if self.peer_launch is not None:
            # One gathered buffer is reused step after step: a rank that is already past the barrier below must
            # not store its next slice into the buffer of a rank whose consumers of this step are still reading.
            # The leading barrier holds every rank's stores until all ranks have launched their next step, which
            # on each of them is stream-ordered after the consumers of the previous one.  (NSplitSignalGemv keeps
            # two halves and needs neither barrier.)
            self.symm.barrier()
            if self.slab.rows > 0:
                self.peer_launch(self.qweight, self.scales, q8, xscale, sum8, mine, self.peer_ptrs, self.slab.rows,
                                 self.K)
            self.symm.barrier()      # every rank's stores have landed before anyone reads the gathered vector
        else:
            if self.slab.rows > 0:
                self.launch(self.qweight, self.scales, q8, xscale, sum8, mine, self.slab.rows, self.K)
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered, mine, group=self.group)
        if self.world * self.slab.stride == self.n_rows:
            return self.gathered
        # padded layout -> compact
        parts = []
        for r in range(self.world):
            rows = min(max(self.n_rows - r * self.slab.stride, 0), self.slab.stride)
            parts.append(self.gathered[r * self.slab.stride: r * self.slab.stride + rows])
        return torch.cat(parts)


class NSplitSignalGemv:
    """NSplitGemv without any barrier kernel: the GEMV epilogue stores the slice into every GPU's gathered vector
    (two halves used in turn) and its last CTA writes a step number into every GPU's flag array; a small gathering
    kernel waits for all flags and copies the vector out.  Step numbers and the choice of half live in device
    memory, so the pair of launches replays as a CUDA graph, and a fast rank can never overwrite the half a slow
    rank's readers still use.  GPUs with peer access only; every rank needs rows.

    signal_launch / gather_launch: ops.gemv_w4a8_peers_signal / ops.gather_after_signals.
    """

    def __init__(self, qweight_slab: torch.Tensor, scales_slab: torch.Tensor, n_rows: int, in_features: int,
                 signal_launch, gather_launch, group=None, align: int = 8):
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_rows, self.K = n_rows, in_features
        self.slab = slab_bounds(n_rows, self.world, self.rank, align)      # 8-row alignment keeps 16-byte stores
        if self.slab.rows <= 0 or qweight_slab.shape[0] != self.slab.rows or scales_slab.shape[0] != self.slab.rows:
            raise ValueError(f"rank {self.rank} expects a slab of {self.slab.rows} > 0 rows")
        self.qweight, self.scales = qweight_slab, scales_slab
        self.signal_launch, self.gather_launch = signal_launch, gather_launch
        dev = qweight_slab.device
        self.half = (self.world * self.slab.stride + 7) // 8 * 8          # elements per half of the gathered vector
        words = self.half + self.world                                    # 2 halves of fp16 = `half` 32-bit words, then flags
        self.buf = symm_mem.empty(words, dtype=torch.int32, device=dev)
        self.buf.zero_()
        self.symm = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
        base = lambda r: int(self.symm.buffer_ptrs[r])
        flag_off = self.half * 4
        mine = self.rank * self.slab.stride * 2                           # this rank's slice inside a half, in bytes
        peers = [r for r in range(self.world) if r != self.rank]
        self.gathered_ptr = base(self.rank)
        self.flags_ptr = base(self.rank) + flag_off
        self.my_slice = base(self.rank) + mine
        self.my_flag = self.flags_ptr + 4 * self.rank
        self.peer_slices = [base(r) + mine for r in peers]
        self.peer_flags = [base(r) + flag_off + 4 * self.rank for r in peers]
        self.step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.empty(n_rows, dtype=torch.float16, device=dev)
        torch.cuda.synchronize()
        self.symm.barrier()      # everyone's buffers are zeroed before the first remote store
        torch.cuda.synchronize()

    def forward(self, q8, xscale, sum8) -> torch.Tensor:
        """Returns the full fp16 output [n_rows] (this object's own buffer, rewritten by the next call)."""
        self.signal_launch(self.qweight, self.scales, q8, xscale, sum8, self.my_slice, self.peer_slices, self.peer_flags,
                           self.my_flag, self.done_counter, self.step_word, self.half, self.slab.rows, self.K)
        self.gather_launch(self.gathered_ptr, self.half, self.flags_ptr, self.world, self.step_word, self.status, self.out,
                           self.n_rows)
        return self.out


class NSplitSampler:
    """Token selection for a row-split lm_head without gathering the logits: every rank scores its own slab
    in the GEMV's epilogue (vocabulary indices offset by the slab's first row), the ranks all-gather their
    (score, index) candidates -- 8 bytes each, `slots` per rank -- and every rank reduces all of them to the
    same token.

    candidates(qweight_slab, scales_slab, q8, xscale, sum8, cand_val, cand_idx, control, index_offset, rows, K)
    runs the local GEMV with the sampling epilogue; finish(cand_val, cand_idx, count, control, token_out)
    reduces.  On GPUs they are launch_gemv_w4a8_sample_candidates / launch_sample_finish with logits=None.
    A rank without rows contributes candidates that can never win (-inf score).
    """

    def __init__(self, qweight_slab: torch.Tensor, scales_slab: torch.Tensor, n_rows: int, in_features: int,
                 slots: int, candidates, finish, group=None, peer_candidates=None):
        """peer_candidates (optional, GPUs with peer access only): launch(qw, sc, q8, xs, s8, val, idx,
        peer_val_ptrs, peer_idx_ptrs, control, index_offset, rows, K) whose epilogue also stores the candidates
        into every peer's gathered array; the arrays then live in symmetric memory and the all-gather becomes a
        barrier."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_rows, self.K, self.slots = n_rows, in_features, slots
        self.slab = slab_bounds(n_rows, self.world, self.rank)
        if qweight_slab.shape[0] != self.slab.rows or scales_slab.shape[0] != self.slab.rows:
            raise ValueError(f"rank {self.rank} expects a slab of {self.slab.rows} rows")
        self.qweight, self.scales = qweight_slab, scales_slab
        self.candidates, self.finish = candidates, finish
        self.peer_candidates = peer_candidates if self.world > 1 else None
        dev = qweight_slab.device
        # [world][2][slots] 32-bit words: scores (as bits) then indices, so that one all-gather moves both
        self.symm = None
        if self.peer_candidates is not None:
            # Two gathered arrays used in turn: a fast rank's stores of step i+1 must not land in the array a
            # slow rank is still reducing for step i.  With two, step i+2 reuses step i's array only after the
            # barrier of step i+1, which no rank passes before every rank has finished reducing step i.
            import torch.distributed._symmetric_memory as symm_mem
            flat = symm_mem.empty(2 * self.world * 2 * slots, dtype=torch.int32, device=dev)
            flat.zero_()
            self.symm = symm_mem.rendezvous(flat, group=group if group is not None else dist.group.WORLD)
            self._both = flat.view(2, self.world, 2, slots)
            self._parity = 0
            self.gathered = self._both[0]
            peers = [r for r in range(self.world) if r != self.rank]
            self._peer_ptrs = []
            for half in range(2):
                off = (half * self.world + self.rank) * 2 * slots * 4     # this rank's rows, in bytes, in every buffer
                self._peer_ptrs.append(([int(self.symm.buffer_ptrs[r]) + off for r in peers],
                                        [int(self.symm.buffer_ptrs[r]) + off + slots * 4 for r in peers]))
        else:
            self.gathered = torch.zeros((self.world, 2, slots), dtype=torch.int32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward(self, q8, xscale, sum8, control) -> torch.Tensor:
        """Returns the int32 token tensor [1] (the same value on every rank); advances `control`."""
        if self.peer_candidates is not None:
            self.gathered = self._both[self._parity]
            peer_val_ptrs, peer_idx_ptrs = self._peer_ptrs[self._parity]
            self._parity ^= 1        # (a captured graph keeps the half it was captured with)
        mine = self.gathered[self.rank]
        val, idx = mine[0].view(torch.float32), mine[1]
        if self.peer_candidates is not None:
            if self.slab.rows == 0:
                raise ValueError("the peer-store form needs rows on every rank")
            self.peer_candidates(self.qweight, self.scales, q8, xscale, sum8, val, idx, peer_val_ptrs,
                                 peer_idx_ptrs, control, self.slab.first, self.slab.rows, self.K)
            self.symm.barrier()      # every rank's candidates have landed everywhere
        else:
            if self.slab.rows > 0:
                self.candidates(self.qweight, self.scales, q8, xscale, sum8, val, idx, control, self.slab.first,
                                self.slab.rows, self.K)
            else:
                val.fill_(float("-inf"))
                idx.zero_()
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered.view(-1), mine.reshape(-1), group=self.group)
        if self.world > 1:
            allv = self.gathered[:, 0, :].contiguous().view(torch.float32).view(-1)
            alli = self.gathered[:, 1, :].contiguous().view(-1)
        else:
            allv, alli = val, idx
        self.finish(allv, alli, allv.numel(), control, self.token)
        return self.token


class NSplitSignalSampler:
    """NSplitSampler without a barrier kernel: the lm_head epilogue stores the candidates into every GPU's
    gathered arrays AND, when its last CTA is through, a step number into every GPU's flag array; the reduction
    kernel waits for all flags itself.  Step numbers live in device memory, so the pair of launches can be
    replayed as a CUDA graph.  GPUs with peer access only; every rank needs rows.

    signal_launch / finish_launch: ops.gemv_w4a8_sample_candidates_signal / ops.sample_finish_after_signals.
    """

    def __init__(self, qweight_slab: torch.Tensor, scales_slab: torch.Tensor, n_rows: int, in_features: int,
                 slots: int, signal_launch, finish_launch, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_rows, self.K, self.slots = n_rows, in_features, slots
        self.slab = slab_bounds(n_rows, self.world, self.rank)
        if self.slab.rows <= 0 or qweight_slab.shape[0] != self.slab.rows or scales_slab.shape[0] != self.slab.rows:
            raise ValueError(f"rank {self.rank} expects a slab of {self.slab.rows} > 0 rows")
        self.qweight, self.scales = qweight_slab, scales_slab
        self.signal_launch, self.finish_launch = signal_launch, finish_launch
        dev = qweight_slab.device
        self.half = self.world * slots                       # entries per half of a gathered array
        words = 4 * self.half + self.world                   # values [2][half], indices [2][half], flags [world]
        self.buf = symm_mem.empty(words, dtype=torch.int32, device=dev)
        self.buf.zero_()
        self.symm = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
        base = lambda r: int(self.symm.buffer_ptrs[r])
        val_off, idx_off, flag_off = 0, 2 * self.half * 4, 4 * self.half * 4
        mine = self.rank * slots * 4                         # this rank's slots inside a half, in bytes
        peers = [r for r in range(self.world) if r != self.rank]
        self.val_ptr, self.idx_ptr = base(self.rank) + val_off, base(self.rank) + idx_off
        self.flags_ptr = base(self.rank) + flag_off
        self.my_val, self.my_idx = self.val_ptr + mine, self.idx_ptr + mine
        self.my_flag = self.flags_ptr + 4 * self.rank
        self.peer_val = [base(r) + val_off + mine for r in peers]
        self.peer_idx = [base(r) + idx_off + mine for r in peers]
        self.peer_flag = [base(r) + flag_off + 4 * self.rank for r in peers]
        self.step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        self.symm.barrier()      # everyone's arrays are zeroed before the first remote store
        torch.cuda.synchronize()

    def forward(self, q8, xscale, sum8, control) -> torch.Tensor:
        self.signal_launch(self.qweight, self.scales, q8, xscale, sum8, self.my_val, self.my_idx, self.peer_val,
                           self.peer_idx, self.peer_flag, self.my_flag, self.done_counter, self.step_word, self.half,
                           control, self.slab.first, self.slab.rows, self.K)
        self.finish_launch(self.val_ptr, self.idx_ptr, self.half, self.half, self.flags_ptr, self.world, self.step_word,
                           self.status, control, self.token)
        return self.token


class NSplitGemm:
    """Y[M][N] = X[M][K] . W^T for M tokens, the weight rows (output columns) split over the ranks; every rank
    ends with the whole Y.  Slabs are aligned to the tensor-core tile (128 rows).

    launch(qweight_slab, scales_slab, x, out, M, rows, K): the local contraction into a contiguous [M][rows]
    block (launch_gemm_prefill_w4a16 of this package); the blocks are all-gathered (NCCL) and put side by side.
    block_launch (optional, GPUs with peer access): launch(qw, sc, x, out_ptr, ldc, peer_ptrs, M, rows, K) writing the
    block into its columns of an [M][ldc] matrix here AND in every peer's copy of it (symmetric memory); the
    gather is then done by the epilogue's stores while other tiles are still being computed, and a barrier
    follows.
    """

    def __init__(self, qweight_slab: torch.Tensor, scales_slab: torch.Tensor, n_rows: int, in_features: int,
                 max_tokens: int, launch, group=None, block_launch=None, align: int = 128):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_rows, self.K, self.max_tokens = n_rows, in_features, max_tokens
        self.slab = slab_bounds(n_rows, self.world, self.rank, align)
        if qweight_slab.shape[0] != self.slab.rows or scales_slab.shape[0] != self.slab.rows:
            raise ValueError(f"rank {self.rank} expects a slab of {self.slab.rows} rows")
        self.qweight, self.scales, self.launch = qweight_slab, scales_slab, launch
        self.block_launch = block_launch if self.world > 1 else None
        dev = qweight_slab.device
        self.ld = self.world * self.slab.stride              # columns of the gathered matrix (padded)
        self.symm = None
        if self.block_launch is not None:
            import torch.distributed._symmetric_memory as symm_mem
            self.full = symm_mem.empty(max_tokens * self.ld, dtype=torch.float16, device=dev)
            self.symm = symm_mem.rendezvous(self.full, group=group if group is not None else dist.group.WORLD)
            off = self.slab.first * 2
            self.my_ptr = int(self.symm.buffer_ptrs[self.rank]) + off
            self.peer_ptrs = [int(self.symm.buffer_ptrs[r]) + off for r in range(self.world) if r != self.rank]
        else:
            self.local = torch.empty(max_tokens * self.slab.stride, dtype=torch.float16, device=dev)
            self.gathered = torch.empty(self.world * max_tokens * self.slab.stride, dtype=torch.float16, device=dev)

    def forward(self, x: torch.Tensor, M: int) -> torch.Tensor:
        """x: fp16 [M][K]; returns fp16 [M][n_rows]."""
        if M > self.max_tokens:
            raise ValueError("more tokens than the buffers were sized for")
        s = self.slab
        if self.block_launch is not None:
            if s.rows == 0:
                raise ValueError("the peer-store form needs rows on every rank")
            # the matrix is reused call after call: no rank may store into a peer's copy before that peer has
            # launched this call too, i.e. is past the readers of the previous result on its stream
            self.symm.barrier()
            self.block_launch(self.qweight, self.scales, x, self.my_ptr, self.ld, self.peer_ptrs, M, s.rows, self.K)
            self.symm.barrier()
            return self.full[:M * self.ld].view(M, self.ld)[:, :self.n_rows]
        mine = self.local[:M * s.stride].view(M, s.stride)
        if s.rows > 0:
            block = mine if s.rows == s.stride else self.local[:M * s.rows].view(M, s.rows)
            self.launch(self.qweight, self.scales, x, block, M, s.rows, self.K)
            if s.rows != s.stride:        # ragged last slab: widen to the common stride
                widened = torch.zeros((M, s.stride), dtype=torch.float16, device=x.device)
                widened[:, :s.rows] = block
                mine = widened
        else:
            mine = torch.zeros((M, s.stride), dtype=torch.float16, device=x.device)
        if self.world == 1:
            return mine[:, :self.n_rows]
        gathered = self.gathered[:self.world * M * s.stride]
        dist.all_gather_into_tensor(gathered, mine.contiguous().view(-1), group=self.group)
        # [rank][M][stride] -> [M][rank * stride]
        return gathered.view(self.world, M, s.stride).permute(1, 0, 2).reshape(M, self.ld)[:, :self.n_rows]
