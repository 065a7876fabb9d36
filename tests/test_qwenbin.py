"""The reader of the reference's `.qwenbin` container (w4a16_qwenbin_*), against two files written by the
reference's own exporter (tests/golden/make_qwenbin_fixture.py: format versions 1 and 2, a tiny random Qwen2
model) and against a few of the original fp16 tensors.  The CPU tests need no GPU: addresses are formed
relative to a host copy of the file.  The GPU test runs the decode sweep on the uploaded file."""
import ctypes
import pathlib
import struct

import numpy as np
import pytest

import oracle

GOLDEN = pathlib.Path(__file__).parent / "golden"
DIMS = dict(hidden_size=256, intermediate_size=512, num_layers=2, num_q_heads=2, num_kv_heads=1, head_dim=128,
            vocab_size=384, quant_type=1)


def _independent_offsets(raw: bytes):
    """Offsets read straight from the published layouts (docs/SPECIFICATION.md; include/config.cuh:75-97)."""
    version = struct.unpack_from("<I", raw, 4)[0]
    names = ["input_norm_gamma", "q_weight", "q_scale", "k_weight", "k_scale", "v_weight", "v_scale", "o_weight",
             "o_scale", "post_norm_gamma", "gate_up_weight", "gate_up_scale", "down_weight", "down_scale"]
    layers, biases = [], []
    if version == 1:
        h = struct.unpack_from("<12I3Q", raw, 0)
        glob = dict(embed_weight=h[12], embed_scale=h[13], final_norm_gamma=h[14], lm_head_weight=h[12], lm_head_scale=h[13])
        for l in range(h[6]):
            t = struct.unpack_from("<17Q", raw, struct.calcsize("<12I3Q") + l * 17 * 8)
            order = dict(input_norm_gamma=0, q_weight=1, q_scale=2, k_weight=4, k_scale=5, v_weight=7, v_scale=8, o_weight=10,
                         o_scale=11, post_norm_gamma=12, gate_up_weight=13, gate_up_scale=14, down_weight=15, down_scale=16)
            layers.append({n: t[order[n]] for n in names})
            biases.append(dict(q_bias=t[3], k_bias=t[6], v_bias=t[9]))
    else:
        h = struct.unpack_from("<12I2f2I11Q", raw, 0)
        glob = dict(embed_weight=h[17], embed_scale=h[21], final_norm_gamma=h[18], lm_head_weight=h[19], lm_head_scale=h[21])
        for l in range(h[4]):
            d = struct.unpack_from("<2I26Q", raw, h[16] + l * 216)[2:]
            layers.append(dict(input_norm_gamma=d[0], post_norm_gamma=d[1], q_weight=d[2], o_weight=d[6], gate_up_weight=d[12],
                               down_weight=d[14], k_weight=d[17], v_weight=d[18], q_scale=d[19], k_scale=d[20], v_scale=d[21],
                               o_scale=d[22], gate_up_scale=d[23], down_scale=d[25]))
            biases.append(dict(q_bias=d[3], k_bias=d[4], v_bias=d[5]))
    return layers, glob, biases


def _read(qb, addr, dtype, count):
    off = addr - qb.host_base()
    return np.frombuffer(qb.bytes.tobytes(), dtype=dtype, count=count, offset=off)


def _w4(qb, w_addr, s_addr, rows, K):
    packed = _read(qb, w_addr, np.uint32, rows * K // 8).reshape(rows, K // 8)
    scales = _read(qb, s_addr, np.float16, rows * (K // 128)).reshape(rows, K // 128)
    return packed, scales


def _dequant(packed, scales):
    q = oracle.unpack_nibbles(packed).astype(np.float32) - 8.0
    return q * np.repeat(scales.astype(np.float32), 128, axis=1)


@pytest.mark.parametrize("version", [1, 2])
def test_reader_agrees_with_the_published_layout_and_the_original_tensors(version):
    from qwen_engine_b200.qwenbin import QwenBin
    path = GOLDEN / f"tiny_w4a16_v{version}.qwenbin"
    raw = path.read_bytes()
    qb = QwenBin(path)
    d = qb.dims()
    assert d["version"] == version and all(d[k] == v for k, v in DIMS.items())
    assert d["tie_word_embeddings"] == 1 and d["file_bytes"] == len(raw)
    layers, glob, biases = qb.tensors(qb.host_base())
    ref_layers, ref_glob, ref_biases = _independent_offsets(raw)
    base = qb.host_base()
    for got, ref in zip(layers + [glob] + biases, ref_layers + [ref_glob] + ref_biases):
        assert {k: v - base for k, v in got.items()} == ref
    # the tensors behind the addresses are the model's: dequantised weights within half a quantisation step of
    # the original fp16 weights (first 16 rows kept by the generator), norms and biases bit for bit
    probe = np.load(GOLDEN / "tiny_w4a16_probe.npz")
    H, I, qdim, kvdim, V = 256, 512, 256, 128, 384

    def check_w4(w_addr, s_addr, rows, K, original, row_map=lambda r: r):
        packed, scales = _w4(qb, w_addr, s_addr, rows, K)
        deq = _dequant(packed, scales)
        for r in range(original.shape[0]):
            rr = row_map(r)
            step = np.repeat(scales[rr].astype(np.float32), 128)
            err = np.abs(deq[rr] - original[r].astype(np.float32))
            assert np.all(err <= 0.5 * step + 1e-3 * np.abs(original[r].astype(np.float32)) + 1e-6)

    check_w4(glob["embed_weight"], glob["embed_scale"], V, H, probe["model__embed_tokens__weight"])
    check_w4(layers[0]["q_weight"], layers[0]["q_scale"], qdim, H, probe["model__layers__0__self_attn__q_proj__weight"])
    check_w4(layers[1]["k_weight"], layers[1]["k_scale"], kvdim, H, probe["model__layers__1__self_attn__k_proj__weight"])
    check_w4(layers[1]["v_weight"], layers[1]["v_scale"], kvdim, H, probe["model__layers__1__self_attn__v_proj__weight"])
    check_w4(layers[0]["o_weight"], layers[0]["o_scale"], H, qdim, probe["model__layers__0__self_attn__o_proj__weight"])
    check_w4(layers[0]["down_weight"], layers[0]["down_scale"], H, I, probe["model__layers__0__mlp__down_proj__weight"])
    # gate and up rows are interleaved: gate row i -> 2i, up row i -> 2i + 1 (tools/export_qwen25.py:336-339)
    check_w4(layers[1]["gate_up_weight"], layers[1]["gate_up_scale"], 2 * I, H, probe["model__layers__1__mlp__gate_proj__weight"],
             row_map=lambda r: 2 * r)
    check_w4(layers[1]["gate_up_weight"], layers[1]["gate_up_scale"], 2 * I, H, probe["model__layers__1__mlp__up_proj__weight"],
             row_map=lambda r: 2 * r + 1)
    eq = lambda addr, name: np.array_equal(_read(qb, addr, np.float16, 16).view(np.uint16), probe[name][:16].view(np.uint16))
    assert eq(glob["final_norm_gamma"], "model__norm__weight")
    assert eq(layers[0]["input_norm_gamma"], "model__layers__0__input_layernorm__weight")
    assert eq(layers[1]["post_norm_gamma"], "model__layers__1__post_attention_layernorm__weight")
    assert eq(biases[0]["q_bias"], "model__layers__0__self_attn__q_proj__bias")
    assert eq(biases[1]["k_bias"], "model__layers__1__self_attn__k_proj__bias")
    assert eq(biases[1]["v_bias"], "model__layers__1__self_attn__v_proj__bias")


def test_reader_refuses_damaged_files():
    from qwen_engine_b200 import W4A16Error
    from qwen_engine_b200.qwenbin import QwenBin
    raw = bytearray((GOLDEN / "tiny_w4a16_v2.qwenbin").read_bytes())
    with pytest.raises(W4A16Error):
        QwenBin(bytes(raw[:1000]))                          # shorter than a header
    bad = bytearray(raw); bad[0] ^= 0xFF
    with pytest.raises(W4A16Error):
        QwenBin(bytes(bad))                                 # magic
    bad = bytearray(raw); struct.pack_into("<I", bad, 4, 3)
    with pytest.raises(W4A16Error):
        QwenBin(bytes(bad))                                 # version
    bad = bytearray(raw); struct.pack_into("<I", bad, 40, 0)
    with pytest.raises(W4A16Error):
        QwenBin(bytes(bad))                                 # fp16 container: not this path
    qb = QwenBin(bytes(raw[:300000]))                       # header fine, tensors cut off
    with pytest.raises(W4A16Error):
        qb.tensors(qb.host_base())
    bad = bytearray(raw); struct.pack_into("<Q", bad, 4096 + 8 + 8 * 2, 56320 + 16)   # q weight off its 256-byte boundary
    qb = QwenBin(bytes(bad))
    with pytest.raises(W4A16Error):
        qb.tensors(qb.host_base())
    qb = QwenBin(bytes(raw))
    with pytest.raises(W4A16Error):
        qb.tensors(qb.host_base() + 8)                      # base must keep the alignment


@pytest.mark.gpu
@pytest.mark.parametrize("version", [1, 2])
def test_decode_sweep_runs_on_an_uploaded_container(version):
    """The file goes to the GPU as it is; the sweep's layer table is the reader's; the result equals the oracle's
    sweep over tensors cut out of the file by this test."""
    import torch
    import qwen_engine_b200 as ops
    from qwen_engine_b200.qwenbin import QwenBin
    from tests import util
    ops.init()
    qb = QwenBin(GOLDEN / f"tiny_w4a16_v{version}.qwenbin")
    d = qb.dims()
    H, I, nq, nkv, hd = d["hidden_size"], d["intermediate_size"], d["num_q_heads"], d["num_kv_heads"], d["head_dim"]
    dev = torch.zeros(qb.bytes.size + 256, dtype=torch.uint8, device="cuda")
    shift = (-dev.data_ptr()) % 256
    dev[shift:shift + qb.bytes.size] = torch.from_numpy(qb.bytes.copy()).cuda()
    base = dev.data_ptr() + shift
    sweep = ops.DecodeSweep(qb.layer_table(base), hidden=H, inter=I, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    assert sweep.launches == 5 * d["num_layers"]
    layers, _, _ = qb.tensors(qb.host_base())
    layers_np = []
    for L in layers:
        g16 = lambda a: _read(qb, a, np.float16, H).copy()
        layers_np.append({"input_norm": g16(L["input_norm_gamma"]), "post_norm": g16(L["post_norm_gamma"]),
                          "q": _w4(qb, L["q_weight"], L["q_scale"], nq * hd, H), "k": _w4(qb, L["k_weight"], L["k_scale"], nkv * hd, H),
                          "v": _w4(qb, L["v_weight"], L["v_scale"], nkv * hd, H), "o": _w4(qb, L["o_weight"], L["o_scale"], H, nq * hd),
                          "gate_up": _w4(qb, L["gate_up_weight"], L["gate_up_scale"], 2 * I, H),
                          "down": _w4(qb, L["down_weight"], L["down_scale"], H, I)})
    rng = np.random.default_rng(version)
    h0 = rng.standard_normal(H).astype(np.float16)
    h_in, h_out = util.to_dev(h0), torch.empty(H, dtype=torch.float16, device="cuda")
    sweep.run_device(h_in, h_out)
    torch.cuda.synchronize()
    ref = oracle.decode_sweep(layers_np, h0)
    util.assert_fp16_close(util.to_np(h_out), ref.astype(np.float64), what=f"sweep over .qwenbin v{version}")
    sweep.close()


def test_random_container_writer_is_read_back_by_the_library(tmp_path):
    """tests/qwenbin_synth.py writes the random model file the drop-in test starts the reference's engine on;
    its descriptor slots must be the ones the library's reader maps to the same tensors."""
    from qwen_engine_b200.qwenbin import QwenBin
    from tests import qwenbin_synth
    path = tmp_path / "tiny_random.qwenbin"
    info = qwenbin_synth.write_random_v2(str(path), hidden=256, inter=512, layers=2, nq=2, nkv=1, hd=128, vocab=384)
    qb = QwenBin(str(path))
    assert qb.dims()["version"] == 2 and qb.dims()["file_bytes"] == info["bytes"]
    base = qb.host_base()
    layers, glob, biases = qb.tensors(base)
    off = info["offsets"]
    short = {"q_weight": "q.weight", "q_scale": "q.scale", "k_weight": "k.weight", "k_scale": "k.scale",
             "v_weight": "v.weight", "v_scale": "v.scale", "o_weight": "o.weight", "o_scale": "o.scale",
             "gate_up_weight": "gate_up.weight", "gate_up_scale": "gate_up.scale", "down_weight": "down.weight",
             "down_scale": "down.scale", "input_norm_gamma": "norm1", "post_norm_gamma": "norm2"}
    for l, L in enumerate(layers):
        for field, name in short.items():
            assert L[field] - base == off[f"l{l}.{name}"], (l, field)
        for field in ("q_bias", "k_bias", "v_bias"):
            assert biases[l][field] - base == off[f"l{l}.{field[0]}.bias"]
    assert glob["embed_weight"] - base == off["embed.weight"] and glob["lm_head_scale"] - base == off["embed.scale"]
    assert glob["final_norm_gamma"] - base == off["final_norm"]
