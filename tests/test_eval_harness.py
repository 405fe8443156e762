"""The evaluation-harness adapter without the harness installed: request encoding (plain and through a chat template), truncation
that keeps the continuation, scoring through the adapter, task configuration and the averages of a report
(levanter_b200/eval_harness.py; scenarios after the reference's tests/test_eval_harness.py)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from levanter_b200.data.packing import PromptCompletion
from levanter_b200.eval_harness import (LmEvalHarnessConfig, TaskConfig, _compute_averages, _iterate_tokenized_requests,
                                        _LmEvalHarnessWorker)
from levanter_b200.layers.attention import AttentionMask
from levanter_b200.models.llama import LlamaConfig

TEMPLATE = ("{{ bos_token }}{% for m in messages %}<|{{ m['role'] }}|>{{ '\\n' }}{{ m['content'] }}<|end|>{{ '\\n' }}{% endfor %}"
            "{% if add_generation_prompt %}<|assistant|>{{ '\\n' }}{% endif %}")

PAIRS = [("What is the capital of France?", " Paris"), ("The quick brown fox", " jumps over the lazy dog"),
         ("To be or not to be,", " that is the question")]


@pytest.fixture(scope="module")
def tokenizer():
    pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator([a + b for a, b in PAIRS] + ["user assistant"],
                            trainers.BpeTrainer(vocab_size=330, special_tokens=["<s>", "</s>", "<pad>", "<|user|>", "<|assistant|>", "<|end|>"],
                                                initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>")
    fast.chat_template = TEMPLATE
    return fast


def _lm(tokenizer, eval_pos=64, chat=False, batch=2):
    model = LlamaConfig(seq_len=eval_pos, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2).build(len(tokenizer), seed=1).eval()
    worker = _LmEvalHarnessWorker(batch, eval_pos, model, None, tokenizer, None, max_packed_segments=4, apply_chat_template=chat)
    return worker.make_harness_lm(), model


def _requests(pairs):
    return [SimpleNamespace(args=p) for p in pairs]


def test_requests_are_encoded_as_context_then_continuation(tokenizer):
    lm, _ = _lm(tokenizer)
    for context, continuation in PAIRS:
        ctx, cont = lm._encode_pair(context, continuation)
        assert ctx + cont == tokenizer(context + continuation)["input_ids"]
        assert tokenizer.decode(ctx) == context and tokenizer.decode(cont) == continuation
    # a trailing space of the context goes with the continuation, where free-running text has it
    ctx, cont = lm._encode_pair("The quick brown fox ", "jumps")
    assert tokenizer.decode(ctx) == "The quick brown fox" and tokenizer.decode(cont) == " jumps"


@pytest.mark.parametrize("chat", [False, True])
def test_requests_become_prompt_completions_in_order(tokenizer, chat):
    out = list(_iterate_tokenized_requests(_requests(PAIRS), tokenizer, 50, batch_size=2, apply_chat_template=chat))
    assert len(out) == 3
    for i, (pc, (context, continuation)) in enumerate(zip(out, PAIRS)):
        assert isinstance(pc, PromptCompletion) and pc.segment_id == i and pc.prompt_length < len(pc.ids) <= 50
        decoded = tokenizer.decode(pc.ids)
        assert context in decoded and decoded.endswith(continuation)
        prompt = tokenizer.decode(pc.ids[:pc.prompt_length])
        assert context in prompt and continuation.strip() not in prompt
        plain_len = len(tokenizer(context)["input_ids"])
        if chat:
            assert "<|user|>" in prompt and prompt.endswith("<|assistant|>\n") and pc.prompt_length > plain_len
        else:
            assert pc.prompt_length == plain_len
    short = list(_iterate_tokenized_requests(_requests(PAIRS), tokenizer, 6, apply_chat_template=chat))
    assert all(len(pc.ids) == 6 and pc.prompt_length >= 1 for pc in short)
    assert all(pc.ids == full.ids[-6:] for pc, full in zip(short, out))  # cut from the left


def test_scores_through_the_adapter_equal_direct_log_likelihoods(tokenizer):
    lm, model = _lm(tokenizer)
    got = lm.loglikelihood(_requests(PAIRS) + [("", " Paris")])  # plain tuples too; an empty context starts from BOS
    assert len(got) == 4
    for (context, continuation), (ll, greedy) in zip(PAIRS, got):
        ctx, cont = lm._encode_pair(context, continuation)
        ids = torch.tensor([ctx + cont], dtype=torch.int32)
        with torch.no_grad():
            logits = (model.activations(ids, AttentionMask.causal()) @ model.get_lm_head().t()).float()[0]
        lp = torch.log_softmax(logits, -1)
        want = sum(lp[len(ctx) - 1 + j, t].item() for j, t in enumerate(cont))
        assert ll == pytest.approx(want, abs=1e-3) and ll < 0
        assert greedy == all(int(logits[len(ctx) - 1 + j].argmax()) == t for j, t in enumerate(cont))
    bos = tokenizer.bos_token_id
    with torch.no_grad():
        cont = tokenizer(" Paris")["input_ids"]
        ids = torch.tensor([[bos] + cont], dtype=torch.int32)
        lp = torch.log_softmax((model.activations(ids, AttentionMask.causal()) @ model.get_lm_head().t()).float()[0], -1)
    assert got[3][0] == pytest.approx(sum(lp[j, t].item() for j, t in enumerate(cont)), abs=1e-3)


def test_the_chat_template_wraps_the_context_only(tokenizer):
    plain, _ = _lm(tokenizer, chat=False)
    chat, model = _lm(tokenizer, chat=True)
    a, b = plain.loglikelihood(_requests(PAIRS[:1])), chat.loglikelihood(_requests(PAIRS[:1]))
    assert a[0][0] != pytest.approx(b[0][0], abs=1e-6)
    context, continuation = PAIRS[0]
    wrapped = tokenizer.apply_chat_template([{"role": "user", "content": context}], tokenize=False, add_generation_prompt=True)
    assert wrapped.startswith("<s><|user|>\n" + context) and wrapped.endswith("<|assistant|>\n")
    ctx, cont = chat._encode_pair(wrapped, continuation, move_trailing_space=False)  # the template's text is kept as written
    assert len(ctx) > len(tokenizer(context)["input_ids"]) and tokenizer.decode(cont) == continuation
    ids = torch.tensor([ctx + cont], dtype=torch.int32)
    with torch.no_grad():
        lp = torch.log_softmax((model.activations(ids, AttentionMask.causal()) @ model.get_lm_head().t()).float()[0], -1)
    assert b[0][0] == pytest.approx(sum(lp[len(ctx) - 1 + j, t].item() for j, t in enumerate(cont)), abs=1e-3)


def test_a_request_longer_than_the_evaluation_length_keeps_its_continuation(tokenizer):
    lm, model = _lm(tokenizer, eval_pos=16)
    long_context = " ".join(["The quick brown fox"] * 12)
    ctx, cont = lm._encode_pair(long_context, " jumps over the lazy dog")
    assert len(ctx) + len(cont) > 16
    (row,) = lm.leader.scorer.pack([(ctx, cont)])
    assert row.tokens.shape == (16,) and row.tokens.tolist() == (ctx + cont)[-16:]
    assert int(row.loss_mask.sum()) == len(cont)  # every continuation token is still scored
    (ll, _), = lm.loglikelihood(_requests([(long_context, " jumps over the lazy dog")]))
    ids = torch.tensor([(ctx + cont)[-16:]], dtype=torch.int32)
    with torch.no_grad():
        lp = torch.log_softmax((model.activations(ids, AttentionMask.causal()) @ model.get_lm_head().t()).float()[0], -1)
    n = 16 - len(cont)
    assert ll == pytest.approx(sum(lp[n - 1 + j, t].item() for j, t in enumerate(cont)), abs=1e-3)


def test_unsupported_request_types_say_so(tokenizer):
    lm, _ = _lm(tokenizer)
    with pytest.raises(NotImplementedError):
        lm.loglikelihood_rolling([])
    with pytest.raises(NotImplementedError):
        lm.generate_until([])


def test_task_configuration():
    spec = [TaskConfig(task="hellaswag", task_alias="hellaswag_10shot", num_fewshot=10),
            TaskConfig(task="hellaswag", task_alias="hellaswag_5shot", num_fewshot=5), "lambada_openai"]
    cfg = LmEvalHarnessConfig(task_spec=spec)
    assert cfg.to_task_spec() == [{"task": "hellaswag", "task_alias": "hellaswag_10shot", "num_fewshot": 10},
                                  {"task": "hellaswag", "task_alias": "hellaswag_5shot", "num_fewshot": 5}, "lambada_openai"]
    try:
        import lm_eval  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="lm_eval"):
            cfg.to_task_dict()
    else:
        assert len(cfg.to_task_dict()) == 3
    # loaded tasks are renamed to their alias, so one task can run with several few-shot settings
    task = SimpleNamespace(config=SimpleNamespace(task="hellaswag"))
    renamed = LmEvalHarnessConfig._rename({"hellaswag": task, "group": {"hellaswag_sub": SimpleNamespace(config=SimpleNamespace(task="hellaswag_sub"))}},
                                          "hellaswag", "hellaswag_5shot")
    assert set(renamed) == {"hellaswag_5shot", "group"} and task.config.task == "hellaswag_5shot"
    assert set(renamed["group"]) == {"hellaswag_5shot_sub"}


def test_report_averages_are_macro_and_sample_weighted():
    outputs = {"results": {"a": {"acc,none": 0.5, "acc_stderr,none": 0.1, "alias": "a"}, "b": {"acc,none": 1.0, "f1,none": 0.25}},
               "n-samples": {"a": {"effective": 30, "original": 100}, "b": {"effective": 10, "original": 10}}}
    avg = _compute_averages(outputs)
    assert avg["macro_avg_acc,none"] == pytest.approx(0.75) and avg["micro_avg_acc,none"] == pytest.approx((0.5 * 30 + 1.0 * 10) / 40)
    assert avg["macro_avg_f1,none"] == pytest.approx(0.25) and avg["micro_avg_f1,none"] == pytest.approx(0.25)
    assert not any("stderr" in k or "alias" in k for k in avg)
    assert np.isfinite(list(avg.values())).all()


class _FakeEvaluator:
    """Stands in for ``lm_eval.evaluator``: asks the adapter for the log-likelihoods of every task's requests and reports the
    share of requests whose continuation is the greedy one, in the harness's result layout."""

    def __init__(self):
        self.calls = []

    def evaluate(self, lm, task_dict, limit=None, log_samples=False, bootstrap_iters=0):
        self.calls.append({"limit": limit, "log_samples": log_samples, "bootstrap_iters": bootstrap_iters})
        results, n = {}, {}
        for name, requests in task_dict.items():
            reqs = requests[:limit] if limit else requests
            out = lm.loglikelihood(_requests(reqs))
            results[name] = {"acc,none": float(np.mean([g for _, g in out])), "acc_stderr,none": 0.0, "ll,none": float(np.mean([l for l, _ in out])),
                             "alias": name}
            n[name] = {"original": len(requests), "effective": len(reqs)}
        return {"results": results, "n-samples": n}


def test_harness_run_reports_results_averages_and_an_artifact(tokenizer, monkeypatch):
    import levanter_b200.eval_harness as H
    import levanter_b200.tracker as T

    fake = _FakeEvaluator()
    monkeypatch.setattr(H, "_evaluator", fake)
    monkeypatch.setattr(LmEvalHarnessConfig, "to_task_dict", lambda self: {"capitals": PAIRS[:1] * 3, "sayings": PAIRS[1:]})
    _, model = _lm(tokenizer)
    cfg = LmEvalHarnessConfig(task_spec=["capitals", "sayings"], max_examples=2, max_eval_length=64)
    out = H.run_lm_eval_harness(cfg, model, tokenizer, 2)
    assert fake.calls == [{"limit": 2, "log_samples": False, "bootstrap_iters": 0}]
    assert set(out["results"]) == {"capitals", "sayings"} and out["n-samples"]["capitals"] == {"original": 3, "effective": 2}
    assert out["averages"]["macro_avg_ll,none"] == pytest.approx(np.mean([out["results"][t]["ll,none"] for t in out["results"]]))
    assert out["results"]["capitals"]["ll,none"] < 0

    class Recorder(T.NoopTracker):
        def __init__(self):
            self.logged, self.artifacts = {}, []

        def log(self, metrics, *, step, commit=None):
            self.logged.update(metrics)

        def log_artifact(self, artifact_path, *, name=None, type=None):
            self.artifacts.append((name, type, open(artifact_path).read()))

    rec = Recorder()
    with T.current_tracker(rec):
        hook = H.lm_eval_harness(cfg, tokenizer, 2, None, None)
        hook(SimpleNamespace(step=0, eval_model=model))  # nothing at step 0
        assert rec.logged == {}
        hook(SimpleNamespace(step=10, eval_model=model))
    assert rec.logged["lm_eval/capitals/ll"] == pytest.approx(out["results"]["capitals"]["ll,none"])
    assert "lm_eval/sayings/acc" in rec.logged and "lm_eval/averages/macro_avg_acc" in rec.logged
    assert not any("stderr" in k and "averages" in k for k in rec.logged)
    (name, kind, text), = rec.artifacts
    assert name == "lm_eval_harness_results.10.json" and kind == "lm_eval_output" and "n-samples" in text

    monkeypatch.setattr(H, "_evaluator", None)
    with pytest.raises(ImportError, match="lm_eval"):
        H.run_lm_eval_harness(cfg, model, tokenizer, 2)


def test_harness_entry_point_on_a_hugging_face_directory(tokenizer, tmp_path, monkeypatch, capsys):
    import levanter_b200.eval_harness as H
    from levanter_b200 import config as C

    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    tokenizer.save_pretrained(str(tmp_path / "tok"))
    cfg_model = LlamaConfig(seq_len=64, hidden_dim=32, intermediate_dim=64, num_layers=1, num_heads=2, num_kv_heads=2)
    model = cfg_model.build(len(tokenizer), seed=1)
    cfg_model.hf_checkpoint_converter().save_pretrained(model, str(tmp_path / "hf"), save_tokenizer=False)
    monkeypatch.setattr(H, "_evaluator", _FakeEvaluator())
    monkeypatch.setattr(LmEvalHarnessConfig, "to_task_dict", lambda self: {"sayings": PAIRS})
    cfg = C.decode(H.EvalHarnessMainConfig, {
        "eval_harness": {"task_spec": ["sayings"], "max_eval_length": 64}, "tokenizer": str(tmp_path / "tok"), "checkpoint_path": str(tmp_path / "hf"),
        "checkpoint_is_hf": True, "model": {"type": "llama", "seq_len": 64, "hidden_dim": 32, "intermediate_dim": 64, "num_layers": 1, "num_heads": 2, "num_kv_heads": 2},
        "trainer": {"require_accelerator": False, "tracker": {"type": "noop"}, "log_dir": str(tmp_path / "logs"), "per_device_eval_parallelism": 2}})
    assert cfg.EvalBatch == 2
    out = H.run_eval_harness_main(cfg)
    lm, _ = _lm(tokenizer)
    lm.leader.scorer.model = model.eval()
    want = np.mean([l for l, _ in lm.loglikelihood(_requests(PAIRS))])
    assert out["results"]["sayings"]["ll,none"] == pytest.approx(want, abs=1e-3)  # the weights that were saved are the ones scored
    assert "macro_avg_ll,none" in capsys.readouterr().out
