"""Hugging Face checkpoint import / export (src/levanter/compat/hf_checkpoints.py).

* ``HFCompatConfig``: model configs that convert to and from HF ``config.json``.
* ``HFCheckpointConverter``: ``load_pretrained`` reads ``model.safetensors[.index.json]`` or ``pytorch_model.bin[.index.json]``
  from a local directory / fsspec URL / the hub cache (:490-607), sizes the vocabulary to the checkpoint and then to the
  tokenizer (:633-677), and copies tensors into the model; ``save_pretrained`` writes sharded safetensors
  (``model-0000i-of-0000N.safetensors`` + index, :1157-1229), ``config.json`` and the tokenizer (:754-954).
* key naming: every model class supplies ``hf_key_map()`` (path segment -> HF segment, ``None`` drops the segment), the
  counterpart of the reference's ``_state_dict_key_map`` hooks.  Linear weights are already 2-D ``[out, in]`` here; modules
  whose reference layout is inputs-first (GPT-2's Conv1D) are transposed, and Mixtral's stacked experts are split per expert.
* ``save_hf_checkpoint_callback``: periodic export hook (:1029-1064).
"""
from __future__ import annotations

import dataclasses
import json
import logging
import os
import re
import shutil
import tempfile
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generic, List, Optional, Tuple, Type, TypeVar, Union

import torch
import torch.nn as nn

from ..models.lm_model import LmConfig, LmHeadModel
from ..utils import fsspec_utils

logger = logging.getLogger(__name__)
SAFE_TENSORS_MODEL = "model.safetensors"
SAFE_TENSORS_INDEX_NAME = "model.safetensors.index.json"
PYTORCH_MODEL = "pytorch_model.bin"
PYTORCH_WEIGHTS_INDEX_NAME = "pytorch_model.bin.index.json"
DEFAULT_MAX_SHARD_SIZE = int(10e9)


@dataclass(frozen=True)
class HFCompatConfig(LmConfig):
    hf_model_type = None
    hf_architecture = None

    def hf_checkpoint_converter(self, ref_checkpoint: Optional[str] = None) -> "HFCheckpointConverter":
        raise NotImplementedError

    @classmethod
    def from_hf_config(cls, hf_config):
        raise NotImplementedError

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[dict] = None) -> dict:
        raise NotImplementedError


@dataclass(frozen=True)
class RepoRef:
    """``model_name_or_path[@revision]``."""

    model_name_or_path: str
    revision: Optional[str] = None

    @staticmethod
    def from_string(s: str) -> "RepoRef":
        if "://" not in s and "@" in s and not os.path.exists(s):
            name, rev = s.rsplit("@", 1)
            return RepoRef(name, rev)
        return RepoRef(s, None)

    def __str__(self):
        return self.model_name_or_path if self.revision is None else f"{self.model_name_or_path}@{self.revision}"

    @classmethod
    def from_config_value(cls, value) -> "RepoRef":
        """Config files give a repo reference as a plain ``name[@revision]`` string."""
        return cls.from_string(str(value))


def _coerce_ref(ref) -> Optional[RepoRef]:
    if ref is None or isinstance(ref, RepoRef):
        return ref
    return RepoRef.from_string(str(ref))


# ------------------------------------------------------------------------------------------------ key mapping
def _hf_name(torch_name: str, key_map: Dict[str, Optional[str]]) -> str:
    parts = torch_name.split(".")
    out: List[str] = []
    for p in parts:
        if p in key_map:
            rep = key_map[p]
            if rep is None:
                continue
            out.append(rep)
        else:
            out.append(p)
    name = ".".join(out)
    # a replacement may carry its own absolute prefix (e.g. token_embeddings -> model.embed_tokens)
    for rep in key_map.values():
        if rep and "." in rep and rep in name and not name.startswith(rep):
            name = name[name.index(rep):]
    return name


def to_hf_state_dict(model: nn.Module, dtype: Optional[torch.dtype] = None, params: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """HF-named, HF-shaped tensors of ``model`` (CPU).  ``params`` overrides the values (e.g. fp32 master weights)."""
    key_map = model.hf_key_map() if hasattr(model, "hf_key_map") else {}
    out: Dict[str, torch.Tensor] = {}
    for name, p in model.named_parameters():
        t = params[name] if params is not None and name in params else p
        t = t.detach()
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        t = t.cpu()
        leaf = name.rsplit(".", 1)[-1]
        if ".experts." in name and leaf in ("w1", "w2", "w3") and t.dim() == 3:
            base = _hf_name(name.rsplit(".", 1)[0], key_map)
            for e in range(t.shape[0]):
                out[f"{base}.{e}.{leaf}.weight"] = t[e].contiguous()
            continue
        if getattr(p, "lev_transposed", False) and t.dim() == 2:
            t = t.t()
        out[_hf_name(name, key_map)] = t.contiguous()
    return out


def load_hf_state_dict(model: nn.Module, state_dict: Dict[str, torch.Tensor], *, strict: bool = True,
                       ignore_prefix: Optional[str] = None) -> List[str]:
    """Copy HF tensors into ``model``.  Returns the names of model parameters that had no counterpart."""
    key_map = model.hf_key_map() if hasattr(model, "hf_key_map") else {}

    def lookup(name: str) -> Optional[torch.Tensor]:
        for cand in (name, f"{ignore_prefix}.{name}" if ignore_prefix else None,
                     name[len(ignore_prefix) + 1:] if ignore_prefix and name.startswith(ignore_prefix + ".") else None):
            if cand is not None and cand in state_dict:
                return state_dict[cand]
        return None

    missing: List[str] = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if ".experts." in name and leaf in ("w1", "w2", "w3") and p.dim() == 3:
                base = _hf_name(name.rsplit(".", 1)[0], key_map)
                ok = True
                for e in range(p.shape[0]):
                    t = lookup(f"{base}.{e}.{leaf}.weight")
                    if t is None:
                        ok = False
                        break
                    p.data[e].copy_(t.to(p.dtype))
                if not ok:
                    missing.append(name)
                continue
            t = lookup(_hf_name(name, key_map))
            if t is None:
                missing.append(name)
                continue
            if getattr(p, "lev_transposed", False) and t.dim() == 2:
                t = t.t()
            if t.shape != p.shape:
                if t.dim() == p.dim() and t.shape[1:] == p.shape[1:] and name.endswith(("token_embeddings.weight", "lm_head.weight", "wte.weight")):
                    n = min(t.shape[0], p.shape[0])
                    p.data[:n].copy_(t[:n].to(p.dtype))
                    continue
                raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(t.shape)} vs model {tuple(p.shape)}")
            p.data.copy_(t.to(p.dtype))
    if missing and strict:
        raise KeyError(f"HF checkpoint is missing tensors for: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    return missing


# ------------------------------------------------------------------------------------------------ tokenizer
def load_tokenizer(model_name_or_path, revision=None, local_cache_dir=None, trust_remote_code=True):
    """Tokenizer from a local directory, an fsspec URL (copied to a temp dir) or the hub (:1067)."""
    from transformers import AutoTokenizer

    path = str(model_name_or_path)
    if "://" in path:
        import fsspec

        fs, plain = fsspec.core.url_to_fs(path)
        tmp = local_cache_dir or tempfile.mkdtemp(prefix="lvb_tok_")
        for f in fs.ls(plain, detail=False):
            base = os.path.basename(f)
            if base.startswith("tokenizer") or base in ("vocab.json", "merges.txt", "special_tokens_map.json", "added_tokens.json"):
                fs.get(f, os.path.join(tmp, base))
        return AutoTokenizer.from_pretrained(tmp, trust_remote_code=trust_remote_code)
    return AutoTokenizer.from_pretrained(path, revision=revision, trust_remote_code=trust_remote_code)


def load_processor(model_name_or_path, revision=None, local_cache_dir=None, trust_remote_code=True):
    """``AutoProcessor`` (feature extractor + tokenizer of an audio model) from a local directory, an fsspec URL (copied to a
    temp dir) or the hub (:1075)."""
    from transformers import AutoProcessor

    path = str(model_name_or_path)
    if "://" in path:
        import fsspec

        fs, plain = fsspec.core.url_to_fs(path)
        tmp = local_cache_dir or tempfile.mkdtemp(prefix="lvb_proc_")
        for f in fs.ls(plain, detail=False):
            base = os.path.basename(f)
            if not base.endswith((".safetensors", ".bin", ".pt")):  # everything but the weights
                fs.get(f, os.path.join(tmp, base))
        return AutoProcessor.from_pretrained(tmp, trust_remote_code=trust_remote_code)
    return AutoProcessor.from_pretrained(path, revision=revision, cache_dir=local_cache_dir, trust_remote_code=trust_remote_code)


def upload_to_hub(local_path: str, repo_ref, **hf_upload_kwargs) -> None:
    """Upload a saved directory to the hub from process 0; the other processes wait for it (:1086)."""
    import torch.distributed as dist

    ref = _coerce_ref(repo_ref)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0:
        from huggingface_hub import upload_folder

        logger.info(f"Uploading HF-compatible checkpoint to {ref.model_name_or_path}")
        upload_folder(folder_path=local_path, repo_id=ref.model_name_or_path, revision=ref.revision, **hf_upload_kwargs)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


# ------------------------------------------------------------------------------------------------ converter
class HFCheckpointConverter:
    def __init__(self, config_class, reference_checkpoint: Optional[Union[str, RepoRef]] = None, tokenizer=None,
                 ignore_prefix: Optional[str] = None, trust_remote_code: bool = False, config_overrides: Optional[dict] = None,
                 HfConfigClass=None, **_):
        self.LevConfigClass = config_class if isinstance(config_class, type) else type(config_class)
        self.reference_checkpoint = _coerce_ref(reference_checkpoint)
        self._tokenizer_ref = tokenizer if tokenizer is not None else (str(self.reference_checkpoint.model_name_or_path) if self.reference_checkpoint else None)
        self.ignore_prefix = ignore_prefix
        self.trust_remote_code = trust_remote_code
        self.config_overrides = config_overrides
        self._tokenizer = tokenizer if (tokenizer is not None and not isinstance(tokenizer, str)) else None

    def replaced(self, **kw) -> "HFCheckpointConverter":
        ref = kw.get("reference_checkpoint", self.reference_checkpoint)
        tok = kw.get("tokenizer", self._tokenizer if self._tokenizer is not None else
                     (str(_coerce_ref(ref).model_name_or_path) if "reference_checkpoint" in kw and ref is not None else self._tokenizer_ref))
        return HFCheckpointConverter(self.LevConfigClass, ref, tok, self.ignore_prefix, self.trust_remote_code,
                                     kw.get("config_overrides", self.config_overrides))

    def with_config_overrides(self, config_overrides: dict, merge: bool = True) -> "HFCheckpointConverter":
        merged = {**(self.config_overrides or {}), **config_overrides} if merge else config_overrides
        return self.replaced(config_overrides=merged)

    @staticmethod
    def from_hf(model_name_or_path, trust_remote_code: bool = False) -> "HFCheckpointConverter":
        """Infer the config class from the checkpoint's ``model_type``."""
        ref = _coerce_ref(model_name_or_path)
        cfg = _read_hf_config(ref)
        mt = cfg.get("model_type")
        for name, cls in LmConfig.get_known_choices().items():
            if getattr(cls, "hf_model_type", None) == mt:
                try:
                    conv = cls().hf_checkpoint_converter(str(ref))  # picks up per-family settings (ignore_prefix, ...)
                    return conv.replaced(reference_checkpoint=ref)
                except Exception:  # noqa: BLE001
                    return HFCheckpointConverter(cls, ref, trust_remote_code=trust_remote_code)
        raise ValueError(f"no model config class handles HF model_type {mt!r}")

    # -- tokenizer / vocab ---------------------------------------------------------------------------------------
    @property
    def tokenizer(self):
        if self._tokenizer is None:
            if self._tokenizer_ref is None:
                raise ValueError("no tokenizer was configured")
            self._tokenizer = load_tokenizer(self._tokenizer_ref)
        return self._tokenizer

    @property
    def Vocab(self) -> int:
        return len(self.tokenizer)

    # -- configs -------------------------------------------------------------------------------------------------
    def hf_config_from_hf_checkpoint(self, ref=None) -> dict:
        return _read_hf_config(self._get_ref(ref))

    def config_from_hf_checkpoint(self, ref=None):
        return self.config_from_hf_config(self.hf_config_from_hf_checkpoint(ref))

    def config_from_hf_config(self, hf_config, overrides: Optional[dict] = None):
        cfg = self.LevConfigClass.from_hf_config(hf_config)
        if overrides:
            cfg = dataclasses.replace(cfg, **overrides)
        return cfg

    @property
    def default_hf_config(self) -> dict:
        return self.hf_config_from_hf_checkpoint(None)

    @property
    def default_config(self):
        return self.config_from_hf_config(self.default_hf_config)

    def _get_ref(self, ref) -> RepoRef:
        ref = _coerce_ref(ref) or self.reference_checkpoint
        if ref is None:
            raise ValueError("Must provide a reference checkpoint to load HF checkpoints")
        return ref

    # -- loading -------------------------------------------------------------------------------------------------
    def load_state_dict(self, ref=None, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        """Tensors of an HF checkpoint, trying safetensors index, torch index, single safetensors, single torch file."""
        ref = self._get_ref(ref)
        path = _resolve_local(ref)
        fs, plain = fsspec_utils.url_to_fs(path)

        def exists(name):
            return fs.exists(os.path.join(plain, name))

        def open_local(name) -> str:
            full = os.path.join(plain, name)
            if "://" not in path:
                return full
            tmp = os.path.join(tempfile.mkdtemp(prefix="lvb_hf_"), name)
            fs.get(full, tmp)
            return tmp

        sd: Dict[str, torch.Tensor] = {}
        if exists(SAFE_TENSORS_INDEX_NAME) or exists(PYTORCH_WEIGHTS_INDEX_NAME):
            idx_name = SAFE_TENSORS_INDEX_NAME if exists(SAFE_TENSORS_INDEX_NAME) else PYTORCH_WEIGHTS_INDEX_NAME
            with open(open_local(idx_name)) as f:
                index = json.load(f)
            for shard in sorted(set(index["weight_map"].values())):
                sd.update(_load_file(open_local(shard)))
        elif exists(SAFE_TENSORS_MODEL):
            sd = _load_file(open_local(SAFE_TENSORS_MODEL))
        elif exists(PYTORCH_MODEL):
            sd = _load_file(open_local(PYTORCH_MODEL))
        else:
            raise FileNotFoundError(f"no model weights found under {path}")
        if dtype is not None:
            sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
        return sd

    def load_pretrained(self, lm_model_cls=None, ref=None, config=None, axis_mapping=None,
                        resize_vocab_to_match_tokenizer: bool = True, dtype: Optional[torch.dtype] = None, device=None,
                        tp=None) -> LmHeadModel:
        """Build the model for the checkpoint's config (or ``config``) and load the HF weights into it."""
        ref = self._get_ref(ref)
        hf_config = self.hf_config_from_hf_checkpoint(ref)
        if config is None:
            config = self.config_from_hf_config(hf_config)
        elif isinstance(config, dict):
            config = self.config_from_hf_config(hf_config, config)
        ckpt_vocab = hf_config.get("vocab_size")
        sd = self.load_state_dict(ref, dtype=dtype)
        if ckpt_vocab is None:
            for k, v in sd.items():
                if k.endswith(("embed_tokens.weight", "wte.weight")):
                    ckpt_vocab = v.shape[0]
        model = config.build(ckpt_vocab, device=device, tp=tp)
        if dtype is not None:
            model = model.to(dtype)
        missing = load_hf_state_dict(model, sd, strict=False, ignore_prefix=self.ignore_prefix)
        tied = getattr(config, "tie_word_embeddings", False)
        real_missing = [m for m in missing if not (m.startswith("lm_head") and tied)]
        if "lm_head.weight" in real_missing:
            # untied head absent from the checkpoint: HF ties it implicitly
            with torch.no_grad():
                model.lm_head.weight.copy_(model.embeddings.token_embeddings.weight)
            real_missing.remove("lm_head.weight")
        if real_missing:
            raise KeyError(f"checkpoint {ref} is missing {real_missing[:8]}")
        if resize_vocab_to_match_tokenizer and self._tokenizer_ref is not None:
            try:
                tv = self.Vocab
                if tv != model.vocab_size:
                    logger.info(f"Resizing model from {model.vocab_size} to {tv} to match the tokenizer vocab size")
                    model = model.resize_vocab(tv)
            except Exception as e:  # noqa: BLE001
                logger.warning(f"could not load the tokenizer to match vocab sizes: {e}")
        return model

    # -- saving --------------------------------------------------------------------------------------------------
    def save_pretrained(self, model: LmHeadModel, path: str, upload_to_hf: Union[bool, str, RepoRef] = False,
                        save_reference_code: Optional[bool] = None, save_tokenizer: bool = True,
                        max_shard_size: int = DEFAULT_MAX_SHARD_SIZE, save_feature_extractor: bool = False,
                        dtype: Optional[torch.dtype] = None, params: Optional[Dict[str, torch.Tensor]] = None, **hf_upload_kwargs):
        """Write an HF-loadable directory: sharded safetensors + index, ``config.json``, tokenizer files."""
        import torch.distributed as dist

        rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
        remote = "://" in str(path)
        local = tempfile.mkdtemp(prefix="lvb_hf_save_") if remote else str(path)
        if rank == 0:
            os.makedirs(local, exist_ok=True)
            sd = to_hf_state_dict(model, dtype=dtype, params=params)
            _save_sharded(sd, local, max_shard_size)
            cfg = model.config.to_hf_config(model.vocab_size, self.config_overrides)
            if self.reference_checkpoint is not None:
                try:
                    ref_cfg = self.hf_config_from_hf_checkpoint(None)
                    for k in ("architectures", "auto_map"):
                        if k in ref_cfg and k not in (self.config_overrides or {}):
                            cfg.setdefault(k, ref_cfg[k])
                except Exception:
                    pass
            if save_tokenizer and self._tokenizer_ref is not None:
                try:
                    tok = self.tokenizer
                    tok.save_pretrained(local)
                    for k in ("pad_token_id", "eos_token_id", "bos_token_id"):
                        v = getattr(tok, k, None)
                        if v is not None:
                            cfg[k] = v
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"could not save the tokenizer: {e}")
            if dtype is not None:
                cfg["torch_dtype"] = str(dtype).replace("torch.", "")
            with open(os.path.join(local, "config.json"), "w") as f:
                json.dump(cfg, f, indent=2, default=str)
            if remote:
                import fsspec

                fs, plain = fsspec.core.url_to_fs(str(path))
                fs.makedirs(plain, exist_ok=True)
                # file by file: a recursive put of a directory into an existing one nests it under its own name
                for root, _, files in os.walk(local):
                    rel = os.path.relpath(root, local)
                    dest = plain.rstrip("/") if rel == "." else f"{plain.rstrip('/')}/{rel}"
                    if rel != ".":
                        fs.makedirs(dest, exist_ok=True)
                    for name in files:
                        fs.put_file(os.path.join(root, name), f"{dest}/{name}")
                shutil.rmtree(local, ignore_errors=True)
            if upload_to_hf:
                try:
                    from huggingface_hub import upload_folder

                    ref = _coerce_ref(upload_to_hf)
                    upload_folder(repo_id=ref.model_name_or_path, revision=ref.revision, folder_path=local, **hf_upload_kwargs)
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"upload to the hub failed: {e}")
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()


def _read_hf_config(ref: RepoRef) -> dict:
    path = _resolve_local(ref)
    fs, plain = fsspec_utils.url_to_fs(path)
    with fs.open(os.path.join(plain, "config.json"), "r") as f:
        return json.load(f)


def _resolve_local(ref: RepoRef) -> str:
    p = str(ref.model_name_or_path)
    if "://" in p or os.path.isdir(p):
        return p
    try:
        from huggingface_hub import snapshot_download

        return snapshot_download(p, revision=ref.revision, allow_patterns=["*.json", "*.safetensors", "*.bin", "*.model", "*.txt"])
    except Exception as e:  # noqa: BLE001
        raise FileNotFoundError(f"{p} is not a local directory and could not be fetched from the hub: {e}")


def _load_file(path: str) -> Dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        return load_file(path)
    return torch.load(path, map_location="cpu", weights_only=True)


def _save_sharded(sd: Dict[str, torch.Tensor], out_dir: str, max_shard_size: int) -> None:
    from safetensors.torch import save_file

    # tied tensors share storage in torch; safetensors refuses aliases, so clone lazily
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    total = 0
    for k, v in sd.items():
        n = v.numel() * v.element_size()
        if size + n > max_shard_size and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = v.contiguous().clone()
        size += n
        total += n
    if len(shards) == 1:
        save_file(shards[0], os.path.join(out_dir, SAFE_TENSORS_MODEL), metadata={"format": "pt"})
        return
    weight_map = {}
    for i, shard in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(out_dir, name), metadata={"format": "pt"})
        for k in shard:
            weight_map[k] = name
    with open(os.path.join(out_dir, SAFE_TENSORS_INDEX_NAME), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)


def save_hf_checkpoint_callback(base_path: str, converter: HFCheckpointConverter, upload_to_hf: Union[bool, str, RepoRef] = False,
                                save_dtype: Optional[torch.dtype] = None, **hf_upload_kwargs):
    """Hook that exports ``step.eval_model`` (the averaged model when averaging is on) to ``<base_path>/step-<n>``,
    skipping step 0 (src/levanter/compat/hf_checkpoints.py:1029-1064)."""

    def cb(step):
        nonlocal hf_upload_kwargs
        if step.step == 0:
            return
        my_kwargs = dict(hf_upload_kwargs)
        if upload_to_hf:
            my_kwargs.setdefault("commit_message", f"Upload for step {step.step} from Levanter")
        params = None
        state = step.state
        if hasattr(state, "engine") and state.model_averaging is None:
            params = state.engine.full_master()
        converter.save_pretrained(step.eval_model, os.path.join(base_path, f"step-{step.step}"), upload_to_hf=upload_to_hf,
                                  dtype=save_dtype, params=params, **my_kwargs)

    return cb
