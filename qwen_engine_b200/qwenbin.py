"""The reference's `.qwenbin` weight container, through the library's reader (w4a16_qwenbin_*).

`QwenBin(path)` keeps the file's bytes in host memory; `tensors(base)` gives the addresses of every tensor the
projection path uses, relative to a copy of the file at `base` (host or device).  `to_device()` uploads the
file as it is -- what the reference engine does (src/engine.cu:85-348) -- and returns the layer table as the
list of dicts `ops.DecodeSweep` takes is not needed: `sweep()` builds the native sweep straight from the table.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ._lib import LayerWeights, QwenBinBiases, QwenBinGlobals, QwenBinHeader, check, load

_FIELDS = [n for n, _ in LayerWeights._fields_]


class QwenBin:
    def __init__(self, path_or_bytes):
        raw = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
        # a 256-byte aligned host copy, so that the same object can also serve as `base`
        buf = np.zeros(len(raw) + 256, dtype=np.uint8)
        shift = (-buf.ctypes.data) % 256
        self.bytes = buf[shift:shift + len(raw)]
        self.bytes[:] = np.frombuffer(raw, dtype=np.uint8)
        self._keep = buf
        self.header = QwenBinHeader()
        check("w4a16_qwenbin_parse", load().w4a16_qwenbin_parse(self.bytes.ctypes.data, self.bytes.size,
                                                                 ctypes.byref(self.header)))

    def dims(self) -> dict:
        return {n: getattr(self.header, n) for n, _ in QwenBinHeader._fields_}

    def tensors(self, base: int):
        """(layers: list of {field: address}, globals: {field: address}, biases: list of {field: address})."""
        n = self.header.num_layers
        layers = (LayerWeights * n)()
        glob = QwenBinGlobals()
        bias = (QwenBinBiases * n)()
        check("w4a16_qwenbin_tensors", load().w4a16_qwenbin_tensors(
            self.bytes.ctypes.data, self.bytes.size, base, layers, n, ctypes.byref(glob), bias))
        as_dict = lambda st: {name: getattr(st, name) for name, _ in st._fields_}
        return [as_dict(layers[i]) for i in range(n)], as_dict(glob), [as_dict(bias[i]) for i in range(n)]

    def host_base(self) -> int:
        return int(self.bytes.ctypes.data)

    def layer_table(self, base: int):
        """The ctypes array w4a16_sweep_create takes."""
        n = self.header.num_layers
        layers = (LayerWeights * n)()
        check("w4a16_qwenbin_tensors", load().w4a16_qwenbin_tensors(
            self.bytes.ctypes.data, self.bytes.size, base, layers, n, None, None))
        return layers
