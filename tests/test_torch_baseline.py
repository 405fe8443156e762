"""The stock-PyTorch comparison model of the benchmark computes the same loss as the framework's Llama for the same weights
(so the two arms of ``bench.py`` time the same mathematics)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from baseline.torch_baseline import Llama, LlamaShape, next_token_loss  # noqa: E402
from levanter_b200.models.llama import LlamaConfig  # noqa: E402
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss  # noqa: E402

MAP = {"self_attn.q_proj": "q", "self_attn.k_proj": "k", "self_attn.v_proj": "v", "self_attn.o_proj": "o", "mlp.gate_proj": "gate",
       "mlp.up_proj": "up", "mlp.down_proj": "down", "input_layernorm": "ln1", "post_attention_layernorm": "ln2"}


def test_same_loss_for_same_weights():
    shape = LlamaShape(vocab=50, hidden=32, intermediate=64, layers=2, heads=2, kv_heads=2, seq_len=16)
    cfg = LlamaConfig(seq_len=16, hidden_dim=32, intermediate_dim=64, num_layers=2, num_heads=2, num_kv_heads=2, gradient_checkpointing=False)
    ours = cfg.build(50, seed=0)
    base = Llama(shape)
    sd = {}
    for n, p in ours.named_parameters():
        if n.startswith("transformer.layers."):
            _, _, i, rest = n.split(".", 3)
            mod, leaf = rest.rsplit(".", 1)
            sd[f"blocks.{i}.{MAP[mod]}.{leaf}"] = p.detach()
        elif n == "transformer.norm.weight":
            sd["norm.weight"] = p.detach()
        elif n == "embeddings.token_embeddings.weight":
            sd["embed.weight"] = p.detach()
        elif n == "lm_head.weight":
            sd["lm_head.weight"] = p.detach()
    base.load_state_dict(sd)
    tokens = torch.randint(0, 50, (3, 16), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    ex = LmExample.stack([LmExample.causal(t) for t in tokens])
    a = compute_next_token_loss(ours, ex)
    b = next_token_loss(base, tokens.long(), ex.loss_mask)
    assert abs(float(a.detach()) - float(b.detach())) < 1e-4, (float(a), float(b))
