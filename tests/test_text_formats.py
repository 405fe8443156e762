"""Text, chat and prompt/response dataset formats on a tokenizer trained in the test (levanter_b200/data/text.py; scenarios after
the reference's tests/test_text.py)."""
import json

import numpy as np
import pytest
import torch

from levanter_b200.data.text import (BatchTokenizer, ChatLmDatasetFormat, ChatProcessor, MultiturnChatDataset, SupervisedDataset,
                                     SupervisedLmDatasetFormat, UrlSingleDatasetLMConfig, build_lm_dataset_cache, preprocessor_for_format)
from levanter_b200.models.lm_model import LmExample
from levanter_b200.models.loss import next_token_loss

TEMPLATE = ("{{ bos_token }}{% for m in messages %}<|{{ m['role'] }}|>\n{% if m['role'] == 'assistant' %}"
            "{% generation %}{{ m['content'] }}<|end|>{% endgeneration %}{% else %}{{ m['content'] }}<|end|>{% endif %}{{ '\n' }}{% endfor %}")

LOREM = ("Lorem ipsum dolor sit amet, consectetur adipiscing elit. Sed do eiusmod tempor incididunt ut labore et dolore magna aliqua. "
         "Ut enim ad minim veniam, quis nostrud exercitation ullamco laboris nisi ut aliquip ex ea commodo consequat. Duis aute irure "
         "dolor in reprehenderit in voluptate velit esse cillum dolore eu fugiat nulla pariatur.")


@pytest.fixture(scope="module")
def tokenizer():
    pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = [LOREM, "Hello! Hi there, how can I help? Tell me a joke. Why did the chicken cross the road? To get to the other side.",
              "Translate to French: Hello Bonjour Yes Oui user assistant"]
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<s>", "</s>", "<pad>", "<|user|>", "<|assistant|>", "<|end|>"],
                                                        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", pad_token="<pad>")
    fast.chat_template = TEMPLATE
    return fast


def test_a_config_without_validation_urls_has_no_validation_set(tmp_path):
    c = UrlSingleDatasetLMConfig(train_urls=["kaa"], validation_urls=[], cache_dir=str(tmp_path), tokenizer="passthrough", vocab_size=64)
    assert c.validation_set(10) is None and c.validation_sets(10) == {}


def test_lm_example_drops_the_loss_where_the_next_token_is_ignored():
    S = 10
    tokens = torch.arange(S, dtype=torch.int32)
    ignore_id = 6
    ex_ignore = LmExample.causal(tokens, ignore_id=ignore_id, eos_id=S)
    ex_plain = LmExample.causal(tokens, eos_id=S)
    assert ex_ignore.loss_mask[ignore_id - 1] == 0 and ex_plain.loss_mask[ignore_id - 1] == 1
    assert ex_ignore.loss_mask.sum() == ex_plain.loss_mask.sum() - 1 and ex_plain.loss_mask[-1] == 0
    # a head that makes the ignored token very unlikely: only the example that still scores it pays for that
    hidden = torch.ones(1, S, 4)
    head = torch.zeros(4, S + 1)
    head[:, ignore_id] = -25.0
    losses = [float(next_token_loss(hidden @ head, tokens[None], loss_mask=ex.loss_mask[None])) for ex in (ex_ignore, ex_plain)]
    assert losses[1] >= losses[0] + 100 / S


def test_long_strings_tokenised_in_pieces_give_the_same_ids(tokenizer):
    short = BatchTokenizer(tokenizer, _workaround_len=len(LOREM) // 3)
    short.__dict__["_needs_long_sequence_workaround"] = True  # force the path that splits at whitespace
    whole = BatchTokenizer(tokenizer, _workaround_len=50000)
    batch = [{"text": LOREM}, {"text": "Hello!"}]
    a, b = short(batch), whole(batch)
    assert len(a) == len(b) == 2
    for x, y in zip(a, b):
        assert x.keys() == y.keys() and all(np.array_equal(x[k], y[k]) for k in x)
    pieces, merge = short._break_for_long_sequences([LOREM])
    assert len(pieces) >= 3 and merge == [True] * (len(pieces) - 1) + [False] and "".join(pieces) == LOREM


def test_bos_and_eos_are_added_once(tokenizer):
    out = BatchTokenizer(tokenizer)([{"text": "Hello!"}])[0]["input_ids"]
    assert out[0] == tokenizer.bos_token_id and out[-1] == tokenizer.eos_token_id
    assert (out == tokenizer.bos_token_id).sum() == 1 and (out == tokenizer.eos_token_id).sum() == 1
    bare = BatchTokenizer(tokenizer, enforce_bos=False, enforce_eos=False)([{"text": "Hello!"}])[0]["input_ids"]
    assert bare.tolist() == tokenizer("Hello!")["input_ids"]
    meta = BatchTokenizer(tokenizer).metadata
    assert meta["append_bos"] and meta["append_eos"] and meta["vocab_size"] == len(tokenizer)


@pytest.mark.parametrize("segment_ids,source_len,expected", [
    ([0, 0, 1, 1, 1], [1, 2], [0, 1, 0, 0, 1]),
    ([0, 0, 1, 1], [2, 2], [0, 0, 0, 0]),
    ([0, 0, 1, 1], [0, 0], [1, 1, 1, 1]),
    ([0, 0, 0, 1, 1, 1], [2, 1], [0, 0, 1, 0, 1, 1]),
    ([0, 0, 0, 0], [2], [0, 0, 1, 1]),
    ([7, 7, 7, 9, 9, -1, -1], [1, 1], [0, 1, 1, 0, 1, 0, 0]),
    ([], [], []),
])
def test_response_mask_from_segment_ids_and_prompt_lengths(segment_ids, source_len, expected):
    got = SupervisedDataset._make_sequence_mask(np.array(segment_ids, dtype=np.int64), np.array(source_len, dtype=np.int64))
    assert got.tolist() == expected


CHATS = [
    {"messages": [{"role": "user", "content": "Hello!"}, {"role": "assistant", "content": "Hi there, how can I help?"}]},
    {"messages": [{"role": "user", "content": "Tell me a joke."}, {"role": "assistant", "content": "Why did the chicken cross the road?"},
                  {"role": "user", "content": "To get to the other side."}, {"role": "assistant", "content": "No, the other side."}]},
]


def _assert_loss_only_predicts_assistant_text(ex, tokenizer):
    """``loss_mask[t] == 1`` exactly where token ``t + 1`` lies inside an assistant turn: after ``<|assistant|>`` + newline, up to
    and including the ``<|end|>`` that closes the turn."""
    toks = ex.tokens.numpy()
    a_id, end_id = tokenizer.convert_tokens_to_ids("<|assistant|>"), tokenizer.convert_tokens_to_ids("<|end|>")
    nl = tokenizer.encode("\n", add_special_tokens=False)[0]
    inside = np.zeros(len(toks), dtype=np.int32)
    for i in np.where(toks == a_id)[0]:
        assert toks[i + 1] == nl
        j = i + 2
        while toks[j] != end_id:
            j += 1
        inside[i + 2:j + 1] = 1
    expected = np.roll(inside, -1)
    expected[-1] = 0
    assert np.array_equal(ex.loss_mask.numpy(), expected)
    assert expected.sum() > 0


def test_chat_format_build_cache_and_pack(tmp_path, tokenizer):
    path = tmp_path / "chat.jsonl"
    path.write_text("".join(json.dumps(c) + "\n" for c in CHATS))
    config = UrlSingleDatasetLMConfig(train_urls=[str(path)], format=ChatLmDatasetFormat(messages_field="messages"))
    processor = preprocessor_for_format(config.format, tokenizer)
    assert isinstance(processor, ChatProcessor)
    source = config.get_shard_source("train")
    processed = [r for doc in source.open_shard(source.shard_names[0]) for r in processor([doc])]
    assert len(processed) == 2

    cache = build_lm_dataset_cache(str(tmp_path / "cache"), source, config.format, tokenizer)
    cache.await_finished()
    assert len(cache) == 2
    sample = cache[0]
    assert sample["assistant_masks"].shape == sample["input_ids"].shape
    marked = tokenizer.decode(sample["input_ids"][sample["assistant_masks"] == 1], skip_special_tokens=False)
    assert marked == "Hi there, how can I help?<|end|>"
    assert tokenizer.decode(sample["input_ids"], skip_special_tokens=False) == "<s><|user|>\nHello!<|end|>\n<|assistant|>\nHi there, how can I help?<|end|>\n"

    packed = MultiturnChatDataset(cache, 128, max_segments_per_example=2).as_sync_dataset()
    assert len(packed) == 1
    ex = packed[0]
    assert ex.tokens.shape == (128,) and ex.loss_mask.shape == (128,) and ex.attn_mask.segment_ids[0].shape == (128,)
    assert sorted(set(ex.attn_mask.segment_ids[0].tolist())) == [-1, 0, 1]
    _assert_loss_only_predicts_assistant_text(ex, tokenizer)

    single = MultiturnChatDataset(cache, 128, max_segments_per_example=1).as_sync_dataset()
    assert len(single) == 2
    for i in range(2):
        assert set(single[i].attn_mask.segment_ids[0].tolist()) == {i, -1}
        _assert_loss_only_predicts_assistant_text(single[i], tokenizer)

    everything = MultiturnChatDataset(cache, 128, max_segments_per_example=1, mask_user_turns=False).as_sync_dataset()[0]
    assert everything.loss_mask.sum() > single[0].loss_mask.sum()


def test_chat_format_needs_a_template_with_a_generation_block(tokenizer):
    with pytest.raises(ValueError, match="generation"):
        ChatProcessor(tokenizer, chat_template="{% for m in messages %}{{ m['content'] }}{% endfor %}")
    ChatProcessor(tokenizer, chat_template="{% for m in messages %}{{ m['content'] }}{% endfor %}", mask_user_turns=False)
    with pytest.raises(ValueError, match="assistant"):
        ChatProcessor(tokenizer)([{"messages": [{"role": "user", "content": "Hello!"}]}])


def test_supervised_format_build_cache_and_pack(tmp_path, tokenizer):
    path = tmp_path / "sup.jsonl"
    rows = [{"prompt": "Translate to French: Hello", "answer": "Bonjour"}, {"prompt": "Translate to French: Yes", "answer": "Oui"}]
    path.write_text("".join(json.dumps(r) + "\n" for r in rows))
    fmt = SupervisedLmDatasetFormat(input_field="prompt", output_field="answer", separate_with="\n")
    cfg = UrlSingleDatasetLMConfig(train_urls=[str(path)], format=fmt)
    cache = build_lm_dataset_cache(str(tmp_path / "cache"), cfg.get_shard_source("train"), fmt, tokenizer)
    cache.await_finished()
    assert len(cache) == 2
    for row, ex in zip(rows, cache):
        assert ex["input_ids"].ndim == 1 and ex["sources_len"].size == 1
        n = int(ex["sources_len"][0])
        prompt = tokenizer.decode(ex["input_ids"][:n], skip_special_tokens=True)
        assert prompt == row["prompt"] + "\n" and tokenizer.decode(ex["input_ids"][n:], skip_special_tokens=True) == row["answer"]

    packed = SupervisedDataset(cache, 128, max_segments_per_example=2, mask_inputs=True).as_sync_dataset()
    assert len(packed) == 1
    ex = packed[0]
    seg, mask, toks = ex.attn_mask.segment_ids[0].numpy(), ex.loss_mask.numpy(), ex.tokens.numpy()
    assert ex.tokens.shape == (128,) and sorted(set(seg.tolist())) == [-1, 0, 1]
    for s, raw in zip((0, 1), cache):
        idx = np.where(seg == s)[0]
        n = int(raw["sources_len"][0])
        # the positions that predict the response: from the last prompt token to the token before the segment's last
        want = np.zeros(len(idx), dtype=np.int32)
        want[n - 1:len(idx) - 1] = 1
        assert mask[idx].tolist() == want.tolist()
        assert toks[idx].tolist() == raw["input_ids"].tolist()
    assert mask[seg == -1].sum() == 0

    single = SupervisedDataset(cache, 128, max_segments_per_example=1, mask_inputs=True).as_sync_dataset()
    assert len(single) == 2
    for i, raw in enumerate(cache):
        s = single[i].attn_mask.segment_ids[0].numpy()
        assert set(s.tolist()) == {i, -1}
        assert int(single[i].loss_mask.sum()) == int((s == i).sum()) - int(raw["sources_len"][0])
    unmasked = SupervisedDataset(cache, 128, max_segments_per_example=1, mask_inputs=False).as_sync_dataset()[0]
    assert int(unmasked.loss_mask.sum()) > int(single[0].loss_mask.sum())
