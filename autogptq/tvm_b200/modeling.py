"""``AutoGPTQForCausalLM.from_quantized(..., use_tvm=True)`` for the B200 backend.

Mirrors the loading path of the reference (``auto_gptq/modeling/auto.py:50-77``,
``auto_gptq/modeling/_base.py:479-569``, ``_utils.py:38-89``) for standard AutoGPTQ checkpoints:
``config.json`` + ``quantize_config.json`` + ``gptq_model-{bits}bit-{group_size}g.{safetensors|bin}``.
The transformers model is built without weights, every linear inside the decoder layers is
replaced by :class:`QuantLinear`, and the checkpoint tensors are loaded directly; ``accelerate``
is not needed.  ``use_tvm=True`` selects this backend (the only one implemented here), the other
selectors of the reference raise.

Llama and OPT layer tables follow ``modeling/llama.py:4-12`` and ``modeling/opt.py:4-16``.
"""
from __future__ import annotations

import contextlib
import json
import os
from dataclasses import dataclass, asdict
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from .qlinear import QuantLinear


@dataclass
class BaseQuantizeConfig:
    """Same keys as the reference's ``quantize_config.json`` (``_base.py:26-62``)."""
    bits: int = 4
    group_size: int = -1
    damp_percent: float = 0.01
    desc_act: bool = True
    sym: bool = True
    true_sequential: bool = True

    def __post_init__(self):
        if self.bits not in (2, 3, 4, 8):
            raise ValueError("only support quantize to [2, 3, 4, 8] bits.")
        if self.group_size != -1 and self.group_size <= 0:
            raise ValueError("unless equal to -1, group_size must greater then 0.")

    @classmethod
    def from_pretrained(cls, save_dir: str):
        with open(os.path.join(save_dir, "quantize_config.json"), "r", encoding="utf-8") as f:
            d = json.load(f)
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def save_pretrained(self, save_dir: str):
        with open(os.path.join(save_dir, "quantize_config.json"), "w", encoding="utf-8") as f:
            json.dump(asdict(self), f, indent=2)


# model_type -> (layers block, modules that stay unquantised, lm head)
MODEL_TABLES: Dict[str, dict] = {
    "llama": dict(layers_block="model.layers", outside=["model.embed_tokens", "model.norm"], lm_head="lm_head"),
    "opt": dict(layers_block="model.decoder.layers",
                outside=["model.decoder.embed_tokens", "model.decoder.embed_positions", "model.decoder.project_out",
                         "model.decoder.project_in", "model.decoder.final_layer_norm"], lm_head="lm_head"),
}
SUPPORTED_MODELS = sorted(MODEL_TABLES)


def find_layers(module: nn.Module, layer_types=(nn.Linear,), name: str = "") -> Dict[str, nn.Module]:
    found = {}
    for child_name, child in module.named_children():
        full = f"{name}.{child_name}" if name else child_name
        if isinstance(child, tuple(layer_types)):
            found[full] = child
        found.update(find_layers(child, layer_types, full))
    return found


def make_quant(model: nn.Module, names: List[str], bits: int, group_size: int) -> None:
    """Replace the named ``nn.Linear`` modules by empty QuantLinear modules (reference ``_utils.py:59-89``)."""
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, leaf)
        setattr(parent, leaf, QuantLinear(bits, group_size, old.in_features, old.out_features, old.bias is not None))


@contextlib.contextmanager
def _parameters_on_meta():
    """Build a model whose *parameters* take no memory while its buffers are created for real.

    Buffers that are not part of a checkpoint (rotary ``inv_freq``, causal masks, QuantLinear's default
    ``g_idx``) keep the values their modules compute at construction; a model built wholly on the meta device
    and materialised with ``to_empty`` would leave them uninitialised."""
    register = nn.Module.register_parameter

    def register_on_meta(module, name, param):
        register(module, name, param)
        if param is not None and param.device.type != "meta":
            module._parameters[name] = nn.Parameter(param.detach().to("meta"), requires_grad=param.requires_grad)

    nn.Module.register_parameter = register_on_meta
    try:
        yield
    finally:
        nn.Module.register_parameter = register


def fuse_quant_linears(parts: List[QuantLinear]) -> QuantLinear:
    """One QuantLinear whose output is the concatenation of the parts' outputs (same input features, bit width,
    group size and ``g_idx``): ``qweight`` / ``scales`` / ``bias`` are joined along the columns and so are the packed
    words of ``qzeros`` (every part's width is a multiple of 32 columns = whole words)."""
    first = parts[0]
    for p_ in parts[1:]:
        if (p_.bits, p_.groupsize, p_.infeatures) != (first.bits, first.groupsize, first.infeatures):
            raise ValueError("layers to fuse must agree in bits, group size and input features")
        if not torch.equal(p_.g_idx, first.g_idx):
            raise ValueError("layers to fuse must share g_idx (act-order layers quantised apart cannot be fused)")
        if (p_.bias is None) != (first.bias is None):
            raise ValueError("layers to fuse must all have a bias or none")
    fused = QuantLinear(first.bits, first.groupsize, first.infeatures, sum(p_.outfeatures for p_ in parts),
                        first.bias is not None)
    fused.qweight = torch.cat([p_.qweight for p_ in parts], dim=1).contiguous()
    fused.qzeros = torch.cat([p_.qzeros for p_ in parts], dim=1).contiguous()
    fused.scales = torch.cat([p_.scales for p_ in parts], dim=1).contiguous()
    fused.g_idx = first.g_idx.clone()
    if first.bias is not None:
        fused.bias = torch.cat([p_.bias for p_ in parts]).contiguous()
    return fused


class _FusedProjection(nn.Module):
    """Runs the fused layer once per input tensor and hands its column blocks to the stand-ins of the original
    projections (transformers calls q_proj / k_proj / v_proj -- or gate_proj / up_proj -- with the same tensor)."""

    def __init__(self, fused: QuantLinear, widths: List[int]):
        super().__init__()
        self.fused = fused
        self.bounds = [0]
        for w in widths:
            self.bounds.append(self.bounds[-1] + w)
        self._x = None
        self._y = None
        self._served = 0

    def part(self, x, i: int):
        if self._x is not x:
            self._y = self.fused(x)
            self._x, self._served = x, 0
        y = self._y[..., self.bounds[i]:self.bounds[i + 1]]
        self._served += 1
        if self._served == len(self.bounds) - 1:      # every block handed out: drop the references
            self._x = self._y = None
        return y


class _FusedPart(nn.Module):
    def __init__(self, owner: _FusedProjection, index: int, holds_owner: bool):
        super().__init__()
        if holds_owner:
            self.owner = owner                      # registered once, so that state_dict / .to() see the fused layer
        else:
            object.__setattr__(self, "_owner_ref", owner)
        self.index = index

    def forward(self, x):
        owner = self.owner if "owner" in self._modules else self._owner_ref
        return owner.part(x, self.index)


# projections that read the same input and can therefore run as one layer (the reference's own TODO,
# quantization/opt.py:228)
FUSABLE = {
    "llama": [("self_attn", ["q_proj", "k_proj", "v_proj"]), ("mlp", ["gate_proj", "up_proj"])],
    "opt": [("self_attn", ["q_proj", "k_proj", "v_proj"])],
}


def fuse_projections(model: nn.Module, model_type: str) -> int:
    """Replace q/k/v (and gate/up) of every decoder layer by one fused QuantLinear each; returns how many were
    fused.  Layers whose parts cannot be fused (different ``g_idx``) are left as they are."""
    table = MODEL_TABLES[model_type]
    done = 0
    for layer in model.get_submodule(table["layers_block"]):
        for holder_name, names in FUSABLE.get(model_type, []):
            holder = getattr(layer, holder_name, None)
            parts = [getattr(holder, n, None) for n in names] if holder is not None else []
            if not parts or not all(isinstance(p_, QuantLinear) for p_ in parts):
                continue
            try:
                fused = fuse_quant_linears(parts)
            except ValueError:
                continue
            owner = _FusedProjection(fused, [p_.outfeatures for p_ in parts])
            for i, n in enumerate(names):
                setattr(holder, n, _FusedPart(owner, i, holds_owner=(i == 0)))
            done += 1
    return done


class GPTQModel(nn.Module):
    """Thin wrapper like the reference's ``BaseGPTQForCausalLM``: holds the model and its quantize config."""

    def __init__(self, model: nn.Module, quantize_config: BaseQuantizeConfig):
        super().__init__()
        self.model = model
        self.quantize_config = quantize_config
        self.config = model.config

    def forward(self, **kwargs):
        return self.model(**kwargs)

    def generate(self, **kwargs):
        with torch.inference_mode():
            return self.model.generate(**kwargs)

    def save_quantized(self, save_dir: str, use_safetensors: bool = False):
        os.makedirs(save_dir, exist_ok=True)
        qc = self.quantize_config
        base = f"gptq_model-{qc.bits}bit-{qc.group_size}g"
        state = {k: v.detach().cpu().contiguous() for k, v in self.model.state_dict().items()}
        if use_safetensors:
            from safetensors.torch import save_file
            save_file(state, os.path.join(save_dir, base + ".safetensors"))
        else:
            torch.save(state, os.path.join(save_dir, base + ".bin"))
        self.model.config.save_pretrained(save_dir)
        qc.save_pretrained(save_dir)


class AutoGPTQForCausalLM:
    @classmethod
    def from_quantized(cls, save_dir: str, device: str = "cpu", use_safetensors: bool = False,
                       use_triton: bool = False, use_tvm: bool = False, export_nnfusion: bool = False,
                       max_memory: Optional[dict] = None, device_map: Optional[str] = None,
                       quantize_config: Optional[BaseQuantizeConfig] = None, model_basename: Optional[str] = None,
                       trust_remote_code: bool = False, fuse_projections: bool = False) -> GPTQModel:
        """Same arguments as the reference (``_base.py:479-493``) plus ``fuse_projections``: join q/k/v and gate/up
        of every decoder layer into one QuantLinear each after loading (one N = 3 * hidden launch instead of three)."""
        if use_triton or export_nnfusion or not use_tvm:
            raise NotImplementedError("this package implements the use_tvm=True backend only")
        if max_memory or device_map:
            raise NotImplementedError("multi-device placement is done by the tensor-parallel harness, not device maps")
        from transformers import AutoConfig, AutoModelForCausalLM
        config = AutoConfig.from_pretrained(save_dir, trust_remote_code=trust_remote_code)
        if config.model_type not in MODEL_TABLES:
            raise TypeError(f"{config.model_type} isn't supported yet.")
        table = MODEL_TABLES[config.model_type]
        if quantize_config is None:
            quantize_config = BaseQuantizeConfig.from_pretrained(save_dir)
        if model_basename is None:
            model_basename = f"gptq_model-{quantize_config.bits}bit-{quantize_config.group_size}g"
        path = os.path.join(save_dir, model_basename + (".safetensors" if use_safetensors else ".bin"))
        if not os.path.isfile(path):
            raise FileNotFoundError(f"Could not find model at {path}")

        with _parameters_on_meta():
            model = AutoModelForCausalLM.from_config(config, trust_remote_code=trust_remote_code, torch_dtype=torch.float16)
        ignore = [table["lm_head"]] + table["outside"]
        names = [n for n in find_layers(model) if not any(n.startswith(i) for i in ignore)]
        make_quant(model, names, quantize_config.bits, quantize_config.group_size)

        if use_safetensors:
            from safetensors.torch import load_file
            state = load_file(path)
        else:
            state = torch.load(path, map_location="cpu")
        model.load_state_dict(state, strict=False, assign=True)
        if getattr(config, "tie_word_embeddings", False):
            model.tie_weights()                             # lm_head shares the embedding loaded above
        # every parameter must have come from the checkpoint (buffers it does not hold keep their constructed values)
        missing = [n for n, p_ in model.named_parameters() if p_.device.type == "meta"]
        if missing:
            raise RuntimeError(f"checkpoint lacks tensors: {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        if fuse_projections:
            globals()["fuse_projections"](model, config.model_type)
        model = model.to(device)
        for key in ("max_position_embeddings", "seq_length", "n_positions"):
            if hasattr(model.config, key):
                model.seqlen = getattr(model.config, key)
                break
        else:
            model.seqlen = 4096
        model.eval()
        if torch.device(device).type == "cuda":
            for m in model.modules():
                if isinstance(m, QuantLinear):
                    m.post_init()
        return GPTQModel(model, quantize_config)


__all__ = ["AutoGPTQForCausalLM", "BaseQuantizeConfig", "GPTQModel", "make_quant", "find_layers", "SUPPORTED_MODELS",
           "fuse_quant_linears", "fuse_projections"]
