"""Mixtral sparse mixture-of-experts (src/levanter/models/mixtral.py).

Routing math is the reference's (:343-347, 374-379, 408-415, 451-466): router logits ``gate(x)``, softmax over experts,
``top_k`` with renormalised weights, tokens repeated per selected expert and sorted by expert id, three grouped GEMMs
(``w1`` gate, ``w3`` up, ``w2`` down; SwiGLU), inverse permutation and the weighted sum over the selected experts.
Auxiliary losses: ``load_balancing_loss = lbl_coef * sum_e f_e p_e`` with ``f = load * E / k`` and
``router_z_loss = rzl_coef * mean(logsumexp(logits)^2)``; they are summed over layers and returned next to the activations
so that ``compute_next_token_loss`` adds them (:556-561, 644-649).  Optional dense shared experts (``n_shared_experts``).

Expert weights are kept ``[experts, out, in]`` (row-major GEMM operands) and written to checkpoints in the reference's
``[experts, in, out]`` orientation.  With an expert-parallel group (``parallel.expert``) each rank holds a slice of the
experts and tokens travel by all-to-all; without one the computation is local, as in the reference."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Type

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import tracker as trk
from ..layers.attention import Attention, AttentionBackend
from ..nn import Linear, trunc_normal_
from ..ops.moe import grouped_mlp
from ..utils.activation import ActivationFunctionEnum
from ..utils.flop_utils import lm_flops_per_token
from ..utils.remat import should_recompute
from .llama import LlamaEmbedding, LlamaMlp, _getter
from .lm_model import LmConfig, LmHeadModel
from .mistral import MistralConfig
from ..layers.rotary import rope_config_from_hf, rope_to_hf_dict, RotaryEmbeddingsConfig


@LmConfig.register_subclass("mixtral")
@dataclass(frozen=True)
class MixtralConfig(MistralConfig):
    num_experts_per_tok: int = 2
    n_routed_experts: int = 8
    n_shared_experts: int = 0
    lbl_coef: Optional[float] = 0.01
    rzl_coef: Optional[float] = 0.001
    flash_attention_block_size: Optional[int] = 2048
    reference_checkpoint: str = "mistralai/Mixtral-8x7B-v0.1"
    expert_parallel: bool = False  # shard experts over the data axis and route tokens by all-to-all
    expert_capacity_factor: float = 2.0  # rows an expert-parallel rank can receive, relative to a balanced load of T * k

    hf_model_type = "mixtral"
    hf_architecture = "MixtralForCausalLM"

    @property
    def model_type(self) -> Type["MixtralLMHeadModel"]:
        return MixtralLMHeadModel

    @classmethod
    def from_hf_config(cls, hf_config) -> "MixtralConfig":
        g = _getter(hf_config)
        return cls(seq_len=g("max_position_embeddings"), hidden_dim=g("hidden_size"), intermediate_dim=g("intermediate_size"),
                   num_layers=g("num_hidden_layers"), num_heads=g("num_attention_heads"), num_kv_heads=g("num_key_value_heads"),
                   activation_function=ActivationFunctionEnum(g("hidden_act", "silu")),
                   initializer_range=g("initializer_range", 0.02), layer_norm_epsilon=g("rms_norm_eps", 1e-5),
                   sliding_window=g("sliding_window", 4096) or 4096,
                   num_experts_per_tok=g("num_experts_per_tok", 2), n_routed_experts=g("num_local_experts", 8),
                   lbl_coef=g("router_aux_loss_coef", 0.01),
                   rope=rope_config_from_hf(g, 1e6))

    def to_hf_config(self, vocab_size: int, config_overrides: Optional[Dict] = None) -> dict:
        theta, _ = self.rope.to_hf_config()
        cfg = dict(model_type="mixtral", architectures=["MixtralForCausalLM"], max_position_embeddings=self.seq_len,
                   hidden_size=self.hidden_dim, intermediate_size=self.intermediate_dim, num_hidden_layers=self.num_layers,
                   num_attention_heads=self.num_heads, num_key_value_heads=self.num_kv_heads,
                   hidden_act=self.activation_function.name, initializer_range=self.initializer_range,
                   rms_norm_eps=self.layer_norm_epsilon, sliding_window=self.sliding_window,
                   num_experts_per_tok=self.num_experts_per_tok, num_local_experts=self.n_routed_experts,
                   router_aux_loss_coef=self.lbl_coef, vocab_size=vocab_size, rope_theta=theta, tie_word_embeddings=False)
        cfg.update({k: v for k, v in rope_to_hf_dict(self.rope).items() if k == "rope_parameters"})
        cfg.update(config_overrides or {})
        return cfg

    def flops_per_token(self, vocab_size: int):
        return lm_flops_per_token(hidden_dim=self.hidden_dim, intermediate_dim=self.intermediate_dim, num_layers=self.num_layers,
                                  num_kv_heads=self.num_kv_heads, num_heads=self.num_heads, seq_len=self.seq_len,
                                  vocab_size=vocab_size, glu=True, num_experts=self.n_routed_experts,
                                  num_shared_experts=self.n_shared_experts, num_experts_per_tok=self.num_experts_per_tok)

    def total_trainable_params(self, vocab_size: int) -> int:
        e, hs = self.hidden_dim, self.actual_head_size
        attn = e * hs * self.num_heads + 2 * e * hs * self.num_kv_heads + hs * self.num_heads * e
        moe = 3 * e * self.intermediate_dim * self.n_routed_experts + e * self.n_routed_experts
        shared = 3 * e * self.intermediate_dim * self.n_shared_experts
        layer = attn + moe + shared + 2 * e
        return self.num_layers * layer + e + 2 * vocab_size * e


class MixtralMoEMlp(nn.Module):
    """Expert weights ``w1`` (gate), ``w3`` (up): ``[E, mlp, embed]``; ``w2`` (down): ``[E, embed, mlp]``."""

    def __init__(self, num_experts: int, hidden: int, intermediate: int, activation: ActivationFunctionEnum, init_std: float,
                 num_local: Optional[int] = None):
        super().__init__()
        n = num_local or num_experts
        self.num_experts = num_experts
        self.num_local = n
        self.act = activation
        self.w1 = nn.Parameter(torch.empty(n, intermediate, hidden))
        self.w2 = nn.Parameter(torch.empty(n, hidden, intermediate))
        self.w3 = nn.Parameter(torch.empty(n, intermediate, hidden))
        for w, fan_in in ((self.w1, hidden), (self.w2, intermediate), (self.w3, hidden)):
            if w.device.type != "meta":
                trunc_normal_(w, init_std)
            w.lev_permute = (0, 2, 1)
            w.lev_shape = (num_experts, w.shape[2], w.shape[1])  # checkpoints hold every expert, whatever the slicing
            w.ep_dim = 0 if n != num_experts else None

    def forward(self, x_sorted: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
        return grouped_mlp(x_sorted, group_sizes, self.w1, self.w3, self.w2, self.act)


class MixtralSparseMoeBlock(nn.Module):
    def __init__(self, config: MixtralConfig, *, ep=None):
        super().__init__()
        self.config = config
        self.ep = ep
        E = config.n_routed_experts
        self.gate = Linear(config.hidden_dim, E, bias=config.use_bias, init_std=config.initializer_range)
        local = E // ep.size if ep is not None else E
        self.experts = MixtralMoEMlp(E, config.hidden_dim, config.intermediate_dim, config.activation_function,
                                     config.initializer_range, num_local=local)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        c = self.config
        E, k = c.n_routed_experts, c.num_experts_per_tok
        shape = x.shape
        x_flat = x.reshape(-1, shape[-1])
        T = x_flat.shape[0]
        from ..ops.moe import moe_route

        router_logits = self.gate(x_flat).float()
        # softmax, top-k, renormalised weights, tokens per expert, probability sums and log-sum-exp in one kernel per direction
        topk_w, topk_idx, group_sizes, p_sum, lse = moe_route(router_logits, k)
        flat_idx = topk_idx.reshape(-1)
        if self.ep is not None and self.ep.size > 1:
            from ..parallel.expert import dispatch_combine, dispatch_combine_peer

            sort_idx = torch.argsort(flat_idx, stable=True)
            # own kernels over peer memory where the ranks share a node (permutation and exchange in one launch per direction,
            # no host read-back); otherwise all-to-all through the collective library
            ex = self.ep.peer_exchange(E, shape[-1], T * k, x_flat.dtype, c.expert_capacity_factor) if x_flat.is_cuda else None
            if ex is not None:
                out_repeat = dispatch_combine_peer(ex, x_flat, sort_idx, group_sizes, k, self.experts)
            else:
                out_repeat = dispatch_combine(self.ep, x_flat, sort_idx, group_sizes, k, self.experts)
        elif x_flat.is_cuda:
            # one grouped launch per projection over a padded expert-sorted layout; nothing is read back by the host
            from ..ops.moe import grouped_mlp_padded

            e = self.experts
            out_repeat = grouped_mlp_padded(x_flat, topk_idx, e.w1, e.w3, e.w2, e.act)
        else:
            sort_idx = torch.argsort(flat_idx, stable=True)
            x_sorted = x_flat.index_select(0, sort_idx // k)
            out_sorted = self.experts(x_sorted, group_sizes)
            inv = torch.empty_like(sort_idx)
            inv[sort_idx] = torch.arange(sort_idx.numel(), device=sort_idx.device)
            out_repeat = out_sorted.index_select(0, inv)
        out = (out_repeat.view(T, k, -1) * topk_w.to(out_repeat.dtype).unsqueeze(-1)).sum(1)
        loads = group_sizes.float() / group_sizes.sum().clamp_min(1)
        extras: Dict[str, torch.Tensor] = {"expert_loads": loads}
        if c.lbl_coef is not None:
            f = loads * E / k
            p = p_sum / T
            extras["load_balancing_loss"] = c.lbl_coef * (f * p).sum()
        if c.rzl_coef is not None:
            extras["router_z_loss"] = c.rzl_coef * (lse ** 2).mean()
        return out.view(shape), extras


class MixtralDecoderLayer(nn.Module):
    def __init__(self, config: MixtralConfig, *, tp=None, ep=None):
        super().__init__()
        self.config = config
        self.tp = tp
        self.self_attn = Attention(config.attention_config(), init_std=config.initializer_range, tp=tp)
        self.block_sparse_moe = MixtralSparseMoeBlock(config, ep=ep)
        self.input_layernorm = config.mk_LayerNorm(config.hidden_dim)
        self.post_attention_layernorm = config.mk_LayerNorm(config.hidden_dim)
        if config.n_shared_experts > 0:
            self.shared_mlp = LlamaMlp(config.hidden_dim, config.intermediate_dim * config.n_shared_experts,
                                       config.activation_function, use_bias=config.use_bias, init_std=config.initializer_range)
        else:
            self.shared_mlp = None

    def forward(self, x, mask=None, pos_ids=None):
        if self.tp is not None and self.tp.size > 1:
            # heads split over the model axis: the block's input enters the tensor-parallel region (its gradient is summed over the
            # axis on the way back) and the output projection's partial products are summed before the bias and the residual.
            # The expert block below runs replicated on the model axis (experts are sliced over the data axis only).
            a = self.self_attn
            out = a.forward(self.tp.copy_to_region(self.input_layernorm(x)), mask, pos_ids, skip_out_bias=True, row_parallel=self.tp)
            if a.o_proj.bias is not None:
                out = out + a.o_proj.bias
            x = x + out
        else:
            x = self.self_attn(self.input_layernorm(x), mask, pos_ids, residual=x)
        h = self.post_attention_layernorm(x)
        moe_out, extras = self.block_sparse_moe(h)
        if self.shared_mlp is not None:
            moe_out = moe_out + self.shared_mlp(h)
        aux = torch.zeros((), dtype=torch.float32, device=x.device)
        for key in ("load_balancing_loss", "router_z_loss"):
            if key in extras:
                aux = aux + extras[key]
        stats = torch.stack([extras.get("load_balancing_loss", aux.new_zeros(())), extras.get("router_z_loss", aux.new_zeros(()))])
        return x + moe_out, aux, extras["expert_loads"].detach(), stats.detach()


class MixtralTransformer(nn.Module):
    def __init__(self, config: MixtralConfig, *, tp=None, ep=None):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([MixtralDecoderLayer(config, tp=tp, ep=ep) for _ in range(config.num_layers)])
        self.norm = config.mk_LayerNorm(config.hidden_dim)

    def forward(self, x, mask=None, pos_ids=None):
        remat = should_recompute(self.config.gradient_checkpointing) and torch.is_grad_enabled() and self.training
        aux_total = torch.zeros((), dtype=torch.float32, device=x.device)
        stats_total = torch.zeros(2, dtype=torch.float32, device=x.device)
        metrics = {}
        for i, layer in enumerate(self.layers):
            if remat:
                x, aux, loads, stats = checkpoint(layer, x, mask, pos_ids, use_reentrant=False)
            else:
                x, aux, loads, stats = layer(x, mask, pos_ids)
            aux_total = aux_total + aux
            stats_total = stats_total + stats
            for j in range(loads.shape[0]):
                metrics[f"moe/layer{i}/expert{j}_load"] = loads[j]
            metrics[f"moe/layer{i}/routing_entropy"] = -(loads * torch.log(loads + 1e-6)).sum()
        if self.config.lbl_coef is not None:
            metrics["train/load_balancing_loss"] = stats_total[0]
        if self.config.rzl_coef is not None:
            metrics["train/router_z_loss"] = stats_total[1]
        trk.jit_log(metrics)
        return self.norm(x), aux_total


class MixtralLMHeadModel(LmHeadModel):
    def __init__(self, vocab_size: int, config: MixtralConfig, *, tp=None, ep=None):
        super().__init__()
        self.config = config
        self._vocab_size = vocab_size
        self.transformer = MixtralTransformer(config, tp=tp, ep=ep)
        self.embeddings = LlamaEmbedding(vocab_size, config)
        self.lm_head = Linear(config.hidden_dim, vocab_size, bias=False, init_std=config.initializer_range)

    @classmethod
    def init(cls, vocab_size: int, config, *, tp=None, ep=None):
        if ep is None and getattr(config, "expert_parallel", False):
            import torch.distributed as dist

            from ..parallel.expert import ExpertParallel

            mesh = getattr(tp, "mesh", None)
            if mesh is not None:
                ep = ExpertParallel.from_mesh(mesh)  # with a model axis the experts are sliced over the data axis only
            elif dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                ep = ExpertParallel(None)
        return cls(vocab_size, config, tp=tp, ep=ep)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def activations(self, input_ids, attn_mask=None, *, pos_ids=None):
        x = self.embeddings.embed(input_ids)
        x, aux = self.transformer(x, attn_mask, pos_ids)
        return x, aux

    def get_lm_head(self) -> torch.Tensor:
        return self.lm_head.weight

    def resize_vocab(self, new_size: int):
        self.embeddings.token_embeddings = self.embeddings.token_embeddings.resize_embeddings(new_size, self.config.initializer_range)
        old = self.lm_head
        new = Linear(self.config.hidden_dim, new_size, bias=False, init_std=self.config.initializer_range,
                     device=old.weight.device, dtype=old.weight.dtype)
        n = min(new_size, old.out_features)
        with torch.no_grad():
            new.weight[:n].copy_(old.weight[:n])
        self.lm_head = new
        self._vocab_size = new_size
        return self

    @staticmethod
    def hf_key_map() -> Dict[str, Optional[str]]:
        return {"transformer": "model", "embeddings": None, "token_embeddings": "model.embed_tokens"}
