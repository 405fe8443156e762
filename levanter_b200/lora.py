"""LoRA (src/levanter/lora.py): low-rank adapters on Linear layers, trainable-parameter filter, merging, PEFT export.

``loraize`` replaces every ``Linear`` whose path matches ``LoraConfig.target_modules`` (regex, list of name suffixes, or None =
all) by ``LoraLinear(wrapped, LowRankLinear(lora_A, lora_B, scale = alpha / r))`` (:249-294); ``lora_A`` is initialised like a
Linear, ``lora_B`` with zeros, so the model is unchanged at step 0.  ``y = W x + (B (A dropout(x))) * alpha / r`` (:131-168).
``merge_lora_modules`` folds ``B A * scale`` into the wrapped weight (:298).  ``save_peft_pretrained`` writes
``adapter_model.safetensors`` + ``adapter_config.json`` in PEFT's naming (:318-360, 479-526)."""
from __future__ import annotations

import dataclasses
import json
import os
import re
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from .nn import Dropout, Linear

LORA_R = "LORA_R"
DEFAULT_DICT_PREFIX = "base_model.model"


@dataclass(frozen=True)
class LoraConfig:
    target_modules: Union[None, List[str], str] = None
    r: int = 8
    alpha: float = 8.0
    dropout: float = 0.0

    def matches_target(self, key_path: str) -> bool:
        if isinstance(self.target_modules, str):
            return re.compile(self.target_modules).match(key_path) is not None
        if self.target_modules is None:
            return True
        return any(key_path.endswith(t) for t in self.target_modules)


class LowRankLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, r: int, alpha: float, dropout_prob: float, device=None, dtype=None):
        super().__init__()
        self.lora_A = Linear(in_features, r, bias=False, device=device, dtype=dtype)
        self.lora_B = Linear(r, out_features, bias=False, device=device, dtype=dtype)
        with torch.no_grad():
            self.lora_B.weight.zero_()
        self.dropout = Dropout(dropout_prob)
        self.scale = alpha / r

    def forward(self, x):
        return self.lora_B(self.lora_A(self.dropout(x))) * self.scale

    def merge(self) -> torch.Tensor:
        """``B A * scale`` as an ``[out, in]`` matrix."""
        return (self.lora_B.weight.float() @ self.lora_A.weight.float()) * self.scale


class LoraLinear(nn.Module):
    def __init__(self, wrapped: Linear, lora: LowRankLinear):
        super().__init__()
        self.wrapped = wrapped
        self.lora = lora

    @property
    def weight(self):
        return self.wrapped.weight

    @property
    def bias(self):
        return self.wrapped.bias

    @property
    def in_features(self):
        return self.wrapped.in_features

    @property
    def out_features(self):
        return self.wrapped.out_features

    def forward(self, x, *, skip_bias: bool = False):
        base = self.wrapped(x, skip_bias=skip_bias)
        lo = self.lora
        if x.is_cuda and x.dtype == torch.bfloat16 and lo.lora_B.weight.dtype == torch.bfloat16 and lo.lora_B.weight.shape[1] % 8 == 0:
            # y = base + scale * B (A x): the up-projection GEMM adds the base output in its epilogue, so the low-rank branch costs
            # two skinny GEMMs and no separate scale or add pass over the [tokens, out] activations
            from .ops.gemm import linear_residual

            t = lo.lora_A(lo.dropout(x))
            return linear_residual(t * lo.scale, lo.lora_B.weight, None, base)
        return base + lo(x)

    def merge(self) -> Linear:
        with torch.no_grad():
            self.wrapped.weight.add_(self.lora.merge().to(self.wrapped.weight.dtype))
        return self.wrapped

    @staticmethod
    def init(wrapped: Linear, r: int, alpha: float, dropout_prob: float) -> "LoraLinear":
        lora = LowRankLinear(wrapped.in_features, wrapped.out_features, r, alpha, dropout_prob, device=wrapped.weight.device,
                             dtype=wrapped.weight.dtype)
        return LoraLinear(wrapped, lora)


def loraize(model: nn.Module, config: LoraConfig, seed: Optional[int] = None) -> nn.Module:
    """Replace matching Linear layers by LoRA-wrapped ones (in place; returns the model)."""
    gen_ctx = torch.random.fork_rng() if seed is not None else None
    if gen_ctx is not None:
        gen_ctx.__enter__()
        torch.manual_seed(seed)
    try:
        for name, mod in list(model.named_modules()):
            for child_name, child in list(mod.named_children()):
                path = f"{name}.{child_name}" if name else child_name
                if type(child) is Linear and config.matches_target(path):
                    setattr(mod, child_name, LoraLinear.init(child, config.r, config.alpha, config.dropout))
    finally:
        if gen_ctx is not None:
            gen_ctx.__exit__(None, None, None)
    return model


def is_lora_param(name: str) -> bool:
    return ".lora." in name or name.startswith("lora.") or "lora_A" in name or "lora_B" in name


def lora_trainable_params_filter(model: nn.Module) -> Callable[[str], bool]:
    """Filter for ``Trainer.initial_state(is_trainable=...)``: only adapter weights train."""
    return is_lora_param


def filter_lora_params(params: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v for k, v in params.items() if is_lora_param(k)}


def partition_lora_params(params: Dict[str, torch.Tensor]) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    lora = {k: v for k, v in params.items() if is_lora_param(k)}
    base = {k: v for k, v in params.items() if not is_lora_param(k)}
    return lora, base


def combine_lora_params(params: Dict[str, torch.Tensor], lora_params: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = dict(params)
    out.update(lora_params)
    return out


def merge_lora_modules(model: nn.Module) -> nn.Module:
    """Fold every adapter into its wrapped Linear and restore plain Linear modules (in place)."""
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, LoraLinear):
                setattr(mod, child_name, child.merge())
    return model


def lora_state_dict(model: nn.Module, prefix: Optional[str] = DEFAULT_DICT_PREFIX) -> Dict[str, torch.Tensor]:
    """Adapter weights with PEFT's names: ``base_model.model.<hf path>.lora_A.weight`` / ``lora_B.weight``."""
    from .compat.hf_checkpoints import _hf_name

    key_map = model.hf_key_map() if hasattr(model, "hf_key_map") else {}
    out = {}
    for name, p in model.named_parameters():
        if not is_lora_param(name):
            continue
        # "<path>.lora.lora_A.weight" -> "<hf path>.lora_A.weight"
        clean = name.replace(".lora.lora_A.", ".lora_A.").replace(".lora.lora_B.", ".lora_B.")
        hf = _hf_name(clean, key_map)
        out[f"{prefix}.{hf}" if prefix else hf] = p.detach().cpu().contiguous()
    return out


def to_hf_config(config: LoraConfig, base_model_name_or_path: Optional[str] = None, **kwargs) -> dict:
    target = config.target_modules
    return {
        "base_model_name_or_path": base_model_name_or_path, "bias": "none", "enable_lora": None, "fan_in_fan_out": False,
        "inference_mode": True, "lora_alpha": config.alpha, "lora_dropout": config.dropout, "merge_weights": False,
        "modules_to_save": None, "peft_type": "LORA", "r": config.r, "target_modules": target, "task_type": "CAUSAL_LM", **kwargs,
    }


def save_peft_pretrained(lora_model: nn.Module, config: LoraConfig, base_model_name_or_path, path: str, prefix: Optional[str] = DEFAULT_DICT_PREFIX,
                         upload_to: Optional[str] = None, **upload_kwargs) -> None:
    """Write ``adapter_config.json`` and ``adapter_model.safetensors`` that ``peft.PeftModel.from_pretrained`` loads."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump(to_hf_config(config, str(base_model_name_or_path) if base_model_name_or_path is not None else None), f)
    save_file(lora_state_dict(lora_model, prefix), os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
    if upload_to:
        try:
            from huggingface_hub import upload_folder

            upload_folder(repo_id=upload_to, folder_path=path, **upload_kwargs)
        except Exception:  # noqa: BLE001
            pass


def save_peft_checkpoint_callback(base_path: str, config: LoraConfig, base_model_name_or_path, upload_to_hf: Optional[str] = None,
                                  **hf_upload_kwargs):
    def cb(step):
        if step.step == 0:
            return
        save_peft_pretrained(step.eval_model, config, base_model_name_or_path, os.path.join(base_path, f"step-{step.step}"),
                             upload_to=upload_to_hf, **hf_upload_kwargs)

    return cb


def save_merged_hf_model(lora_model: nn.Module, converter, destination: str, *, upload_to_hf=False, **upload_kwargs) -> None:
    import copy

    merged = merge_lora_modules(copy.deepcopy(lora_model))
    converter.save_pretrained(merged, destination, upload_to_hf=upload_to_hf, **upload_kwargs)


def save_merged_hf_checkpoint_callback(base_path: str, converter, upload_to_hf=False, **hf_upload_kwargs):
    def cb(step):
        if step.step == 0:
            return
        save_merged_hf_model(step.eval_model, converter, os.path.join(base_path, f"step-{step.step}"), upload_to_hf=upload_to_hf,
                             **hf_upload_kwargs)

    return cb
