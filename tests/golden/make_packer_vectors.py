"""Generates tests/golden/packer_vectors.npz from the reference's own Python packer.

Run where the reference checkout is readable (it is not needed afterwards):
    python tests/golden/make_packer_vectors.py [/path/to/reference]
It imports `quantize_and_pack_w4a16` from the reference's tools/convert_gguf_to_qwenbin.py
(numpy only; the same function body as tools/export_qwen25.py:42-78) and records its
output on seeded matrices that include the edge cases the packer has: an all-zero group
(scale 0 -> divisor fp16(1e-5)), exact .5 rounding ties, a negative maximum, values that
clip at both ends, and tiny magnitudes whose fp16 scale is subnormal.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np

if len(sys.argv) < 2:
    sys.exit("usage: make_packer_vectors.py <reference checkout>")
ref_root = Path(sys.argv[1])
spec = importlib.util.spec_from_file_location("ref_gguf_conv", ref_root / "tools" / "convert_gguf_to_qwenbin.py")
mod = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mod)

rng = np.random.Generator(np.random.Philox(key=0x5EED0001))
cases = {}


def add(name, w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    packed, scales = mod.quantize_and_pack_w4a16(w)
    cases[f"{name}_w"] = w
    cases[f"{name}_packed"] = packed.astype(np.uint32)
    cases[f"{name}_scales"] = scales.astype(np.float16)


# plain gaussian rows, two K sizes
add("gauss_k512", rng.standard_normal((24, 512)) * 0.05)
add("gauss_k256", rng.standard_normal((8, 256)) * 2.0)

# edge cases
w = rng.standard_normal((8, 256)).astype(np.float32) * 0.02
w[0, :128] = 0.0                          # all-zero group
w[1, :128] = np.linspace(-7, 7, 128) * 0.5  # with scale 0.5 -> exact .5 ties
w[1, 0] = 3.5
w[2, 128:] = -np.abs(w[2, 128:])          # negative-only group (max at a negative)
w[3, :] *= 1e-6                            # subnormal fp16 scales
w[4, 5] = 1e4                              # one huge outlier: everything else rounds to 8
w[5, :128] = 7.0                           # constant group -> every nibble 15
w[6, :128] = -7.0                          # constant group -> every nibble 1
add("edges_k256", w)

out = Path(__file__).resolve().parent / "packer_vectors.npz"
np.savez_compressed(out, **cases)
print("wrote", out, {k: v.shape for k, v in cases.items()})
