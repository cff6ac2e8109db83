"""Checkpoint reading and sharding (CPU)."""
import json
import os

import pytest
import torch

from xixi_vllm_b200.config import load_model_config
from xixi_vllm_b200.models.loader import SafetensorsSource, write_safetensors
from xixi_vllm_b200.models.synth import hf_tensor_shapes, make_model_dir


def test_reader_matches_safetensors_wheel(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    g = torch.Generator().manual_seed(0)
    tensors = {"w": torch.randn(37, 24, generator=g).bfloat16(), "b": torch.randn(24, generator=g),
               "i": torch.arange(10, dtype=torch.int64), "h": torch.randn(5, 3, 4, generator=g).half()}
    path = tmp_path / "x.safetensors"
    write_safetensors(str(path), tensors)
    loaded = st.load_file(str(path))                         # our writer is readable by the wheel
    for k, v in tensors.items():
        assert torch.equal(loaded[k], v)
    st.save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "y.safetensors"))
    for native in (True, False):
        if not native:
            os.environ["XV_NO_HOSTLIB"] = "1"
        try:
            src = SafetensorsSource(str(tmp_path))
            if not native:
                src._lib = None
            assert set(src.names()) == set(tensors)
            assert torch.equal(src.read("w"), tensors["w"])
            assert torch.equal(src.read("w", 5, 7), tensors["w"][5:12])
            assert torch.equal(src.read("w", 0, None, 8, 8), tensors["w"][:, 8:16])
            assert torch.equal(src.read("w", 30, 7, 20, 4), tensors["w"][30:37, 20:24])
            assert torch.equal(src.read("b", 4, 10), tensors["b"][4:14])
            assert torch.equal(src.read("i"), tensors["i"])
            with pytest.raises(IndexError):
                src.read("w", 30, 10)
            src.close()
        finally:
            os.environ.pop("XV_NO_HOSTLIB", None)


def test_synth_dir_and_model_load_roundtrip(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "tiny")
    cfg = load_model_config(d)
    assert cfg.head_dim == 64 and cfg.tie_word_embeddings
    src = SafetensorsSource(d)
    shapes = hf_tensor_shapes(json.load(open(os.path.join(d, "config.json"))))
    assert {n: src.shape(n) for n in src.names()} == shapes
    from xixi_vllm_b200.models.qwen3 import Qwen3ForCausalLM
    from xixi_vllm_b200.parallel import groups
    groups.single_process_groups()
    model = Qwen3ForCausalLM(cfg, dtype=torch.float32, device="cpu")
    rep = model.load_weights(src)
    assert not rep["skipped"] and rep["loaded"] == len(shapes)
    q = src.read("model.layers.1.self_attn.q_proj.weight")
    k = src.read("model.layers.1.self_attn.k_proj.weight")
    fused = model.model.layers[1].self_attn.qkv_proj.weight
    assert torch.equal(fused[: q.shape[0]], q) and torch.equal(fused[q.shape[0]: q.shape[0] + k.shape[0]], k)
    assert model.lm_head.weight.data_ptr() == model.model.embed_tokens.weight.data_ptr()      # tied
    assert {n for n, _ in model.named_parameters()} >= {"model.norm.weight", "lm_head.weight"}


def test_head_dim_and_rope_defaults(tmp_path):
    d = tmp_path / "c"
    d.mkdir()
    json.dump({"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "num_hidden_layers": 1,
               "intermediate_size": 128, "vocab_size": 100, "rope_parameters": {"rope_theta": 5000.0},
               "dtype": "float16"}, open(d / "config.json", "w"))
    c = load_model_config(str(d))
    assert c.head_dim == 16 and c.rope_theta == 5000.0 and c.torch_dtype == "float16"
