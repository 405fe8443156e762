"""Which parameters of a real GPT-2 get weight decay: by path fragments, by a regular expression, by owner class names and by
default (levanter_b200/optim/config.py:build_weight_decay_mask; scenarios after the reference's tests/test_weight_decay_mask.py)."""
from levanter_b200.models.gpt2 import Gpt2Config
from levanter_b200.optim import AdamConfig
from levanter_b200.optim.config import ParamInfo, levanter_path


def _model():
    return Gpt2Config(seq_len=32, hidden_dim=32, num_layers=2, num_heads=2).build(100, seed=0)


def _expected(model, decay_embeddings=True):
    """The hand-written answer: matrices of the attention and MLP projections (and the two embedding tables when asked);
    never a bias or a layer norm."""
    out = {}
    for name, _ in model.named_parameters():
        p = levanter_path(name)
        matrix = p.endswith("weight") and any(s in p for s in ("attn.c_attn", "attn.c_proj", "mlp.c_fc", "mlp.c_proj"))
        emb = decay_embeddings and p.endswith("weight") and ("token_embeddings" in p or "position_embeddings" in p)
        out[name] = bool(matrix or emb)
    return out


def _mask(cfg, model):
    params = dict(model.named_parameters())
    return cfg.build_weight_decay_mask(ParamInfo(model))(params)


def test_mask_by_path_fragments_and_by_regex():
    m = _model()
    want = _expected(m)
    assert sum(want.values()) == 2 * 4 + 2 and len(want) > sum(want.values())
    by_list = AdamConfig(weight_decay_modules=["attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight",
                                               "token_embeddings.weight", "position_embeddings.weight"])
    by_regex = AdamConfig(weight_decay_modules=r".*attn.*weight|.*mlp.*weight|.*token_embeddings|.*position_embeddings")
    assert _mask(by_list, m) == want
    assert _mask(by_regex, m) == want


def test_mask_by_owner_class_names():
    m = _model()
    assert _mask(AdamConfig(weight_decay_modules=["Linear.weight", "Embedding.weight"]), m) == _expected(m)


def test_default_mask_skips_biases_norms_and_embeddings():
    m = _model()
    assert AdamConfig(default_weight_decay_mask=False).build_weight_decay_mask() is None
    default = _mask(AdamConfig(default_weight_decay_mask=True), m)
    implied = _mask(AdamConfig(weight_decay_modules=None, default_weight_decay_mask=None), m)
    assert default == implied == _expected(m, decay_embeddings=False)
