"""from_quantized(..., use_tvm=True): checkpoint round trip on CPU (module replacement, tensor loading,
file naming); the forward itself needs a GPU and is covered in tests/test_gpu_modeling.py."""
import json
import os

import pytest
import torch

from autogptq.tvm_b200 import QuantLinear, modeling


def _tiny_llama_dir(tmp_path, bits=4, group_size=32, safetensors=True):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=320, max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).half()
    qc = modeling.BaseQuantizeConfig(bits=bits, group_size=group_size, desc_act=False)
    names = [n for n in modeling.find_layers(model) if n.startswith("model.layers")]
    dense = {}
    for n in names:
        lin = model.get_submodule(n)
        W = lin.weight.data.float()
        G = W.shape[1] // group_size
        Wg = W.reshape(W.shape[0], G, group_size)
        wmin, wmax = Wg.min(-1).values.clamp(max=0), Wg.max(-1).values.clamp(min=0)
        scale = ((wmax - wmin) / (2 ** bits - 1)).clamp(min=1e-5)
        zero = torch.round(-wmin / scale)
        q = QuantLinear(bits, group_size, W.shape[1], W.shape[0], False)
        fake = torch.nn.Linear(W.shape[1], W.shape[0], bias=False)
        fake.weight.data = W
        q.pack(fake, scale, zero, None)
        parent, _, leaf = n.rpartition(".")
        setattr(model.get_submodule(parent), leaf, q)
        dense[n] = (scale, zero)
    wrapped = modeling.GPTQModel(model, qc)
    wrapped.save_quantized(str(tmp_path), use_safetensors=safetensors)
    return cfg, names, model


@pytest.mark.parametrize("safetensors", [True, False])
def test_from_quantized_round_trip(tmp_path, safetensors):
    cfg, names, saved = _tiny_llama_dir(tmp_path, safetensors=safetensors)
    files = set(os.listdir(tmp_path))
    assert {"config.json", "quantize_config.json"} <= files
    assert ("gptq_model-4bit-32g.safetensors" if safetensors else "gptq_model-4bit-32g.bin") in files
    assert json.load(open(tmp_path / "quantize_config.json"))["bits"] == 4
    loaded = modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cpu", use_safetensors=safetensors,
                                                         use_tvm=True)
    assert loaded.model.seqlen == 64
    for n in names:
        a, b = loaded.model.get_submodule(n), saved.get_submodule(n)
        assert isinstance(a, QuantLinear)
        for buf in ("qweight", "qzeros", "scales", "g_idx"):
            assert torch.equal(getattr(a, buf), getattr(b, buf)), (n, buf)
    assert not isinstance(loaded.model.lm_head, QuantLinear)
    assert torch.equal(loaded.model.model.embed_tokens.weight, saved.model.embed_tokens.weight)
    assert torch.equal(loaded.model.lm_head.weight, saved.lm_head.weight)
    # buffers that no checkpoint holds must carry the values a normally constructed model computes
    from transformers import LlamaForCausalLM
    fresh = LlamaForCausalLM(cfg)
    bufs, fresh_bufs = dict(loaded.model.named_buffers()), dict(fresh.named_buffers())
    checked = 0
    for name, ref in fresh_bufs.items():
        if "inv_freq" in name:
            assert torch.allclose(bufs[name].float(), ref.float()), name
            checked += 1
    assert checked >= 1
    assert not any(p.device.type == "meta" for p in loaded.model.parameters())


def test_missing_lm_head_is_reported(tmp_path):
    """With untied embeddings a checkpoint without lm_head.weight must not load silently."""
    _tiny_llama_dir(tmp_path, safetensors=False)
    path = os.path.join(tmp_path, "gptq_model-4bit-32g.bin")
    state = torch.load(path)
    del state["lm_head.weight"]
    torch.save(state, path)
    with pytest.raises(RuntimeError, match="lacks tensors"):
        modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cpu", use_tvm=True)


def test_other_backends_are_refused(tmp_path):
    _tiny_llama_dir(tmp_path)
    with pytest.raises(NotImplementedError):
        modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), use_triton=True, use_tvm=True)
    with pytest.raises(NotImplementedError):
        modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), use_tvm=False)
    with pytest.raises(FileNotFoundError):
        modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), use_tvm=True, model_basename="nope")


def test_load_time_fusion_of_projections(tmp_path):
    """fuse_projections=True: q/k/v and gate/up of every layer become one QuantLinear each whose dequantised weights
    are the parts' weights side by side (N = 3 * hidden for q|k|v)."""
    import numpy as np
    from oracle import gptq_oracle as O
    cfg, names, saved = _tiny_llama_dir(tmp_path)
    loaded = modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cpu", use_safetensors=True, use_tvm=True,
                                                         fuse_projections=True)

    def dense(m):
        return O.dequantize(m.qweight.numpy(), m.qzeros.numpy(), m.scales.numpy(), m.g_idx.numpy(), m.bits)[2]

    layer0, saved0 = loaded.model.model.layers[0], saved.model.layers[0]
    fused = layer0.self_attn.q_proj.owner.fused
    assert isinstance(fused, QuantLinear) and fused.outfeatures == 3 * cfg.hidden_size
    want = np.concatenate([dense(saved0.self_attn.q_proj), dense(saved0.self_attn.k_proj),
                           dense(saved0.self_attn.v_proj)], axis=1)
    assert np.array_equal(dense(fused).view(np.uint16), want.view(np.uint16))
    mlp = layer0.mlp.gate_proj.owner.fused
    assert mlp.outfeatures == 2 * cfg.intermediate_size
    want = np.concatenate([dense(saved0.mlp.gate_proj), dense(saved0.mlp.up_proj)], axis=1)
    assert np.array_equal(dense(mlp).view(np.uint16), want.view(np.uint16))
    # the fused layers are part of the module tree exactly once
    n_q = sum(isinstance(m, QuantLinear) for m in loaded.model.modules())
    assert n_q == cfg.num_hidden_layers * (1 + 1 + 1 + 1)      # qkv, o, gate|up, down
