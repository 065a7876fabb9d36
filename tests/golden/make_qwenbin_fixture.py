"""Generates tests/golden/tiny_w4a16_v1.qwenbin, tiny_w4a16_v2.qwenbin (+ tiny_w4a16_probe.npz) with the
REFERENCE's own exporter.

Run in a container that has the reference checkout (not on the GPU box):

    python tests/golden/make_qwenbin_fixture.py /path/to/reference

A tiny random Qwen2 model (hidden 256, intermediate 512, 2 layers, 2 query heads / 1 kv head of 128,
vocabulary 384, tied embeddings, QKV biases) is built with transformers, saved to a temporary directory and
exported by tools/export_qwen25.py::export_model in its ordinary (non-dummy) path, W4A16, once per container
format version.  The version-2 branch of the exporter as checked in stops with a NameError
(tools/export_qwen25.py:369 packs `norm1_off`, which line 268 defined as `norm1_offset`); for that file the
generator loads the exporter's source with this one identifier corrected, nothing else.
Only the loading calls are stubbed: the tiny model has no tokenizer (the tokenizer file is not part of the
weight container), and AutoModelForCausalLM.from_pretrained is replaced by a function that hands back the
in-memory model (the exporter passes device_map="cpu", which needs the `accelerate` package).  The probe file keeps the first 16 rows (entries) of a few of the ORIGINAL fp16 tensors so that a reader can check it maps
every descriptor slot to the right tensor.
"""
import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch


def main(ref_root: str) -> None:
    from transformers import Qwen2Config, Qwen2ForCausalLM
    here = os.path.dirname(os.path.abspath(__file__))
    src_path = os.path.join(ref_root, "tools", "export_qwen25.py")

    def load_exporter(fix_v2: bool):
        import types
        src = open(src_path).read()
        if fix_v2:
            assert src.count("norm1_off, norm2_off,") == 1
            src = src.replace("norm1_off, norm2_off,", "norm1_offset, norm2_off,")
        mod = types.ModuleType("ref_export_qwen25")
        mod.__file__ = src_path
        exec(compile(src, src_path, "exec"), mod.__dict__)
        return mod

    torch.manual_seed(1234)
    cfg = Qwen2Config(vocab_size=384, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=128,
                      rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
    model = Qwen2ForCausalLM(cfg).half()
    with torch.no_grad():   # norm gains away from exactly 1.0 and non-zero biases, so that mix-ups show
        for name, p in model.named_parameters():
            if name.endswith("layernorm.weight") or name.endswith("norm.weight"):
                p.copy_((1.0 + 0.25 * torch.randn_like(p.float())).half())
            if name.endswith("bias"):
                p.copy_((0.1 * torch.randn_like(p.float())).half())

    class _NoTokenizer:
        @staticmethod
        def from_pretrained(*a, **k):
            return None
    class _InMemoryModel:
        @staticmethod
        def from_pretrained(*a, **k):
            return model

    for version in (1, 2):
        exp = load_exporter(fix_v2=(version == 2))
        exp.AutoTokenizer = _NoTokenizer
        exp.export_tokenizer = lambda tokenizer, path: None
        exp.AutoModelForCausalLM = _InMemoryModel
        with tempfile.TemporaryDirectory() as tmp:
            out = os.path.join(here, f"tiny_w4a16_v{version}.qwenbin")
            exp.export_model(tmp, "w4a16", out, os.path.join(tmp, "tokenizer.bin"), dummy=False, version=version)
        print("wrote", out, os.path.getsize(out), "bytes")

    sd = model.state_dict()
    keep = ["model.embed_tokens.weight", "model.norm.weight",
            "model.layers.0.input_layernorm.weight", "model.layers.1.post_attention_layernorm.weight",
            "model.layers.0.self_attn.q_proj.weight", "model.layers.1.self_attn.k_proj.weight",
            "model.layers.1.self_attn.v_proj.weight", "model.layers.0.self_attn.o_proj.weight",
            "model.layers.1.mlp.gate_proj.weight", "model.layers.1.mlp.up_proj.weight",
            "model.layers.0.mlp.down_proj.weight", "model.layers.1.self_attn.k_proj.bias",
            "model.layers.0.self_attn.q_proj.bias", "model.layers.1.self_attn.v_proj.bias"]
    np.savez_compressed(os.path.join(here, "tiny_w4a16_probe.npz"),
                        **{k.replace(".", "__"): sd[k].numpy().astype(np.float16)[:16] for k in keep})   # first 16 rows / entries


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_qwenbin_fixture.py <reference checkout>")
    main(sys.argv[1])
