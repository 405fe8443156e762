"""Tagged evaluation: bits per byte from the byte lengths of the target tokens, tag hierarchies, example limits, the names under
which results are logged, and the hook that also scores the averaged weights (levanter_b200/eval.py)."""
import math
from types import SimpleNamespace

import pytest
import torch

import levanter_b200.tracker as T
from levanter_b200.data.dataset import ListAsyncDataset
from levanter_b200.eval import TaggedEvaluator, cb_tagged_lm_evaluate, eval_model
from levanter_b200.models.llama import LlamaConfig
from levanter_b200.models.lm_model import LmExample, compute_next_token_loss
from levanter_b200.utils.hf_utils import byte_length_of_token


@pytest.fixture(scope="module")
def tokenizer():
    pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog, naïve café"] * 4,
                            trainers.BpeTrainer(vocab_size=320, special_tokens=["<s>", "</s>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    return transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>")


def _examples(tokenizer, texts, S=24):
    out = []
    for t in texts:
        ids = tokenizer(t)["input_ids"][:S]
        ids = ids + [tokenizer.eos_token_id] * (S - len(ids))
        lm = torch.zeros(S)
        lm[:len(tokenizer(t)["input_ids"][:S]) - 1] = 1
        out.append(LmExample.causal(torch.tensor(ids, dtype=torch.int32), loss_mask=lm))
    return out


def test_bits_per_byte_use_the_utf8_length_of_the_scored_tokens(tokenizer):
    model = LlamaConfig(seq_len=24, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2).build(len(tokenizer), seed=0).eval()
    web = _examples(tokenizer, ["the quick brown fox", "naïve café over the lazy dog", "the dog"])
    code = _examples(tokenizer, ["jumps over", "fox fox fox fox"])
    ev = TaggedEvaluator(2, [(ListAsyncDataset(web, is_complete=True), ["text/web"]), (ListAsyncDataset(code, is_complete=True), ["text/code"])],
                         tokenizer=tokenizer)
    r = ev.evaluate(model)

    def totals(examples):
        loss = nbytes = tokens = 0.0
        with torch.no_grad():
            for e in examples:
                per = compute_next_token_loss(model, LmExample.stack([e]), reduction=None)[0]
                loss += float((per * e.loss_mask).sum())
                tokens += float(e.loss_mask.sum())
                targets = torch.roll(e.tokens, -1).tolist()
                nbytes += sum(byte_length_of_token(tokenizer, t) for t, m in zip(targets, e.loss_mask.tolist()) if m)
        return loss, tokens, nbytes

    lw, tw, bw = totals(web)
    lc, tc, bc = totals(code)
    # the scored targets of "naïve café ..." are every character but its first token: multi-byte characters count their bytes
    assert bw >= len("naïve café over the lazy dog".encode()) - 4 + len("the quick brown fox") - 4
    log2e = math.log2(math.e)
    assert r.tag_micro_bpb["text/web"] == pytest.approx(lw * log2e / bw, rel=1e-4)
    assert r.tag_micro_bpb["text/code"] == pytest.approx(lc * log2e / bc, rel=1e-4)
    assert r.micro_bpb == pytest.approx((lw + lc) * log2e / (bw + bc), rel=1e-4)
    assert r.macro_bpb == pytest.approx(0.5 * (lw * log2e / bw + lc * log2e / bc), rel=1e-4)
    assert r.tag_micro_bpb["text"] == pytest.approx(r.micro_bpb, rel=1e-6) and r.tag_macro_bpb["text"] == pytest.approx(r.macro_bpb, rel=1e-6)
    assert r.micro_avg_loss == pytest.approx((lw + lc) / (tw + tc), rel=1e-4)

    logged = eval_model(ev, model, prefix="eval")
    assert {"eval/loss", "eval/macro_loss", "eval/bpb", "eval/macro_bpb", "eval/text/web/loss", "eval/text/code/bpb", "eval/text/micro_loss",
            "eval/text/macro_loss", "eval/text/macro_bpb", "eval/text/bpb", "eval/loading_time", "eval/total_time"} <= set(logged)
    assert logged["eval/text/web/bpb"] == pytest.approx(r.tag_micro_bpb["text/web"])

    limited = TaggedEvaluator(2, [(ListAsyncDataset(web, is_complete=True), ["text/web"])], tokenizer=tokenizer, max_examples_per_dataset=1)
    l1, t1, _ = totals(web[:1])
    assert limited.evaluate(model).micro_avg_loss == pytest.approx(l1 / t1, rel=1e-4)
    one = eval_model(limited, model, prefix="")
    assert "loss" in one and "macro_loss" not in one  # a single untagged-like set logs no macro average


def test_the_hook_scores_the_current_and_the_averaged_weights():
    cfg = LlamaConfig(seq_len=8, hidden_dim=16, intermediate_dim=32, num_layers=1, num_heads=2, num_kv_heads=2)
    current, averaged = cfg.build(30, seed=0).eval(), cfg.build(30, seed=1).eval()
    data = ListAsyncDataset([LmExample.causal(torch.randint(0, 30, (8,), generator=torch.Generator().manual_seed(i), dtype=torch.int32))
                             for i in range(5)], is_complete=True)

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.logged = {}

        def log(self, metrics, *, step, commit=None):
            self.logged.setdefault(step, {}).update(metrics)

    rec = Recorder()
    hook = cb_tagged_lm_evaluate(2, [(data, ["val"])])
    with T.current_tracker(rec):
        hook(SimpleNamespace(step=3, model=current, eval_model=averaged, state=SimpleNamespace(model_averaging=object())))
        hook(SimpleNamespace(step=4, model=current, eval_model=current, state=SimpleNamespace(model_averaging=None)))
    assert rec.logged[3]["eval/loss"] != pytest.approx(rec.logged[3]["eval/ema/loss"], rel=1e-6)
    assert "eval/ema/loss" not in rec.logged[4] and rec.logged[4]["eval/loss"] == pytest.approx(rec.logged[3]["eval/loss"])
    assert "eval/bpb" not in rec.logged[3]  # no tokenizer, no byte lengths
    with pytest.raises(ValueError):
        cb_tagged_lm_evaluate(2, [(data, ["val"])], eval_current=False, eval_ema=False)
    only_ema = cb_tagged_lm_evaluate(2, [(data, ["val"])], eval_current=False)
    with T.current_tracker(rec), pytest.raises(ValueError, match="model averaging"):
        only_ema(SimpleNamespace(step=5, model=current, eval_model=current, state=SimpleNamespace(model_averaging=None)))
