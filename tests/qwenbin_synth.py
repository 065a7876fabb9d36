"""Writes a random `.qwenbin` version-2 container of any dimensions (test infrastructure).

The layout is the published one (reference include/config.cuh:103-170, docs/SPECIFICATION.md): a 192-byte
header (152 bytes of fields, 64-byte aligned), the table of 216-byte layer descriptors, then the tensors, each 256-byte aligned; gate and up are one
row-interleaved matrix that both descriptor slots point at; embeddings are tied.  Weights are uniform nibbles,
scales uniform in [0.002, 0.02], norm gains small so that a random stack stays finite in fp16 -- the
distributions of the benchmark.  It exists so that the reference's own engine can be started on the GPU box,
where the real model file is not available; the files the reference's exporter wrote are under tests/golden/.
"""
from __future__ import annotations

import struct

import numpy as np


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def write_random_v2(path: str, hidden=1536, inter=8960, layers=28, nq=12, nkv=2, hd=128, vocab=151936,
                    max_seq_len=4096, seed=20250, gain=0.05) -> dict:
    """Returns {"bytes": file size, "offsets": {name: offset}}."""
    rng = np.random.default_rng(seed)
    qdim, kvdim = nq * hd, nkv * hd
    header_bytes = 192
    table_off = header_bytes
    weights_off = max(4096, _align(table_off + layers * 216))
    cur = weights_off
    blobs = []   # (offset, bytes-like)
    offsets = {}

    def put(name: str, data: np.ndarray) -> int:
        nonlocal cur
        cur = _align(cur)
        off = cur
        blobs.append((off, data))
        offsets[name] = off
        cur += data.nbytes
        return off

    def packed(rows: int, k: int) -> np.ndarray:
        return rng.integers(0, 256, size=rows * k // 2, dtype=np.uint8)

    def scales(rows: int, k: int) -> np.ndarray:
        return rng.uniform(0.002, 0.02, size=rows * (k // 128)).astype(np.float16)

    def gains(n: int) -> np.ndarray:
        return (gain * (1.0 + 0.1 * rng.standard_normal(n))).astype(np.float16)

    embed_w = put("embed.weight", packed(vocab, hidden))
    embed_s = put("embed.scale", scales(vocab, hidden))
    final_norm = put("final_norm", gains(hidden))
    table = bytearray()
    for l in range(layers):
        slot = [0] * 26
        slot[0] = put(f"l{l}.norm1", gains(hidden))
        slot[1] = put(f"l{l}.norm2", gains(hidden))
        slot[2] = put(f"l{l}.q.weight", packed(qdim, hidden))
        slot[3] = put(f"l{l}.q.bias", (0.01 * rng.standard_normal(qdim)).astype(np.float16))
        slot[4] = put(f"l{l}.k.bias", (0.01 * rng.standard_normal(kvdim)).astype(np.float16))
        slot[5] = put(f"l{l}.v.bias", (0.01 * rng.standard_normal(kvdim)).astype(np.float16))
        slot[6] = put(f"l{l}.o.weight", packed(hidden, qdim))
        slot[12] = slot[13] = put(f"l{l}.gate_up.weight", packed(2 * inter, hidden))
        slot[14] = put(f"l{l}.down.weight", packed(hidden, inter))
        slot[17] = put(f"l{l}.k.weight", packed(kvdim, hidden))
        slot[18] = put(f"l{l}.v.weight", packed(kvdim, hidden))
        slot[19] = put(f"l{l}.q.scale", scales(qdim, hidden))
        slot[20] = put(f"l{l}.k.scale", scales(kvdim, hidden))
        slot[21] = put(f"l{l}.v.scale", scales(kvdim, hidden))
        slot[22] = put(f"l{l}.o.scale", scales(hidden, qdim))
        slot[23] = slot[24] = put(f"l{l}.gate_up.scale", scales(2 * inter, hidden))
        slot[25] = put(f"l{l}.down.scale", scales(hidden, inter))
        slot[15] = slot[19]   # quant_scales_offset: first scale tensor of the layer
        table += struct.pack("<II26Q", 0, 0, *slot)
    total = _align(cur)
    head = struct.pack("<12I2f2I", 0x5157454E, 2, hidden, inter, layers, nq, nkv, hd, vocab, max_seq_len, 1, 1,
                       1e-6, 1000000.0, 0, 0)
    head += struct.pack("<5Q6Q", table_off, embed_w, final_norm, embed_w, weights_off, embed_s, 0, 0, 0, 0, 0)
    assert len(head) == 152, len(head)
    head += bytes(header_bytes - len(head))
    with open(path, "wb") as f:
        f.write(head)
        f.write(bytes(table))
        for off, data in blobs:
            f.seek(off)
            f.write(data.tobytes())
        f.truncate(total)
    return {"bytes": total, "offsets": offsets}
