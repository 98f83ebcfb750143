"""from_quantized(..., use_tvm=True) end to end on a GPU: a tiny Llama checkpoint in the standard AutoGPTQ
file layout is loaded, run through transformers' forward with the B200 QuantLinear modules, and compared
with the same model on dense dequantised weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import QuantLinear, modeling, ops
    from test_modeling_cpu import _tiny_llama_dir
    DEV = torch.device("cuda:0")


def test_loaded_model_matches_dense_weights(tmp_path):
    _, _, saved = _tiny_llama_dir(tmp_path, bits=4, group_size=32, safetensors=True)
    m = modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cuda:0", use_safetensors=True, use_tvm=True)
    ids = torch.randint(0, 320, (1, 24), generator=torch.Generator().manual_seed(3)).to(DEV)
    with torch.no_grad():
        logits_q = m.model(input_ids=ids).logits.float()          # 24 rows: the tcgen05 GEMM path
        step_q = m.model(input_ids=ids[:, :1]).logits.float()     # 1 row: the GEMV path
    # The yardstick is the model that was SAVED (constructed normally, never reloaded), with every QuantLinear
    # swapped for a dense layer of the oracle's dequantised weights: a loader that damaged anything outside the
    # linears (rotary tables, norms, embeddings) shows up as a difference.
    from oracle import gptq_oracle as O
    for name, mod in list(saved.named_modules()):
        if isinstance(mod, QuantLinear):
            _, _, W = O.dequantize(mod.qweight.numpy(), mod.qzeros.numpy(), mod.scales.numpy(), mod.g_idx.numpy(), mod.bits)
            lin = torch.nn.Linear(mod.infeatures, mod.outfeatures, bias=False, dtype=torch.float16)
            lin.weight.data = torch.from_numpy(W).t().contiguous()
            parent, _, leaf = name.rpartition(".")
            setattr(saved.get_submodule(parent), leaf, lin)
    saved = saved.to(DEV).eval()
    with torch.no_grad():
        logits_d = saved(input_ids=ids).logits.float()
        step_d = saved(input_ids=ids[:, :1]).logits.float()
    assert (logits_q - logits_d).abs().max() <= 2e-2 * max(1.0, logits_d.abs().max().item())
    assert (step_q - step_d).abs().max() <= 2e-2 * max(1.0, step_d.abs().max().item())
    out = m.generate(input_ids=ids[:, :4], max_new_tokens=4, do_sample=False)
    assert out.shape == (1, 8)


def test_fused_projections_give_the_same_logits(tmp_path):
    """Load-time q|k|v and gate|up fusion: same logits as the unfused model (bit for bit on the GEMV path, where a
    column's sum does not depend on its neighbours; within fp16 rounding on the GEMM path)."""
    _tiny_llama_dir(tmp_path, bits=4, group_size=32, safetensors=True)
    plain = modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cuda:0", use_safetensors=True, use_tvm=True)
    fused = modeling.AutoGPTQForCausalLM.from_quantized(str(tmp_path), device="cuda:0", use_safetensors=True, use_tvm=True,
                                                        fuse_projections=True)
    assert fused.model.model.layers[0].self_attn.q_proj.owner.fused.outfeatures == 3 * 64
    ids = torch.randint(0, 320, (1, 24), generator=torch.Generator().manual_seed(4)).to(DEV)
    with torch.no_grad():
        a, b = plain.model(input_ids=ids).logits.float(), fused.model(input_ids=ids).logits.float()
        a1, b1 = plain.model(input_ids=ids[:, :1]).logits.float(), fused.model(input_ids=ids[:, :1]).logits.float()
    assert (a - b).abs().max() <= 2e-2 * max(1.0, a.abs().max().item())
    assert (a1 - b1).abs().max() <= 2e-2 * max(1.0, a1.abs().max().item())
