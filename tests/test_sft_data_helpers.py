"""The older supervised fine-tuning data helpers (single-turn chat jsonl, prompt / response sources, padding and masking of
examples) and the corpus-size summary (levanter_b200/data/text.py)."""
import json

import numpy as np
import pytest
import torch

from levanter_b200.data.passthrough_tokenizer import PassthroughTokenizer
from levanter_b200.data.text import (ChatUrlDataSourceConfig, LMMixtureDatasetConfig, SupervisedUrlSourceConfig, UrlDatasetSourceConfig,
                                     UrlSingleDatasetLMConfig, _prepare_supervised_examples, count_corpus_sizes, datasource_from_chat_jsonl_single_turn,
                                     mk_chat_sft_dataset, mk_single_turn_cached_sft_dataset, mk_supervised_dataset)


def _chat_file(path, n=6):
    with open(path, "w") as f:
        for i in range(n):
            f.write(json.dumps({"messages": [{"role": "system", "content": "0"}, {"role": "user", "content": f"{10 + i} {11 + i} "},
                                             {"role": "assistant", "content": f"{20 + i} {21 + i} {22 + i} "}]}) + "\n")


def test_single_turn_chat_rows_take_the_first_message_of_each_role(tmp_path):
    _chat_file(tmp_path / "c.jsonl")
    src = datasource_from_chat_jsonl_single_turn([str(tmp_path / "c.jsonl")])
    rows = list(src)
    assert rows[0] == {"input": "10 11 ", "output": "20 21 22 "} and len(rows) == 6
    assert list(src.open_shard_at_row(src.shard_names[0], 4))[0] == {"input": "14 15 ", "output": "24 25 26 "}
    (tmp_path / "bad.jsonl").write_text(json.dumps({"messages": [{"role": "user", "content": "1"}]}) + "\n")
    with pytest.raises(ValueError, match="missing"):
        list(datasource_from_chat_jsonl_single_turn([str(tmp_path / "bad.jsonl")]))
    cfg = ChatUrlDataSourceConfig(cache_dir=str(tmp_path / "cache"), train_urls=[str(tmp_path / "c.jsonl")])
    assert cfg.get_shard_source("validation") is None and cfg.get_shard_source("train") is not None


def test_cached_chat_examples_are_padded_and_masked_to_the_response(tmp_path):
    _chat_file(tmp_path / "c.jsonl")
    tok = PassthroughTokenizer(100)
    cfg = ChatUrlDataSourceConfig(cache_dir=str(tmp_path / "cache"), train_urls=[str(tmp_path / "c.jsonl")])
    raw = mk_single_turn_cached_sft_dataset(cfg, tok, 12).as_sync_dataset()
    assert len(raw) == 6
    first = raw[0]
    assert first["input_ids"].tolist()[:2] == [10, 11] and int(first["sources_len"][0]) == 2
    eos = tok.eos_token_id
    assert first["input_ids"].tolist()[-1] == eos  # the end-of-sequence token was appended once

    ds = mk_chat_sft_dataset(cfg, tok, 12).as_sync_dataset()
    ex = ds[0]
    n = len(first["input_ids"])
    assert ex.tokens.shape == (12,) and ex.tokens.tolist()[:n] == first["input_ids"].tolist()
    pad = tok.pad_token_id if tok.pad_token_id is not None else eos
    assert ex.tokens.tolist()[n:] == [pad] * (12 - n)
    # loss where the next token is a response token and not the padding token: positions src_len - 1 .. n - 3 here, because this
    # tokenizer pads with its end-of-sequence token, so the final token is not told apart from padding (as in the reference)
    want = np.zeros(12, dtype=np.int32)
    want[1:n - 2] = 1
    assert ex.loss_mask.tolist() == want.tolist()


def test_examples_longer_than_the_sequence_keep_their_end():
    tok = PassthroughTokenizer(100)
    (ex,) = _prepare_supervised_examples([{"input_ids": np.arange(1, 21, dtype=np.int32), "sources_len": np.array([15])}], tok, 8)
    assert ex.tokens.tolist() == list(range(13, 21))
    assert int(ex.loss_mask.sum()) == 0 or ex.loss_mask.tolist()[-1] == 0  # never on the last position


def test_prompt_response_sources_by_field_names(tmp_path):
    with open(tmp_path / "s.jsonl", "w") as f:
        for i in range(5):
            f.write(json.dumps({"q": f"{10 + i} ", "a": f"{30 + i} {31 + i}", "other": "x"}) + "\n")
    cfg = SupervisedUrlSourceConfig(cache_dir=str(tmp_path / "cache"), train_urls=[str(tmp_path / "s.jsonl")], input_field="q", output_field="a")
    rows = list(cfg.get_shard_source("train"))
    assert rows[0] == {"q": "10 ", "a": "30 31"} and cfg.get_shard_source("validation") is None
    tok = PassthroughTokenizer(100)
    ds = mk_supervised_dataset(cfg, "train", tok, 8).as_sync_dataset()
    assert len(ds) == 5
    ex = ds[2]
    assert ex.tokens.tolist()[:3] == [12, 32, 33] and int(ex.loss_mask.sum()) >= 2 and ex.loss_mask[0] == 1  # the prompt's last token predicts the response
    with pytest.raises(ValueError, match="No data source"):
        mk_supervised_dataset(cfg, "validation", tok, 8)


def _docs(path, n, offset):
    with open(path, "w") as f:
        for i in range(n):
            f.write(json.dumps({"text": " ".join(str(offset + j) for j in range(i % 5 + 3))}) + "\n")


def test_corpus_sizes_of_a_single_source_and_of_a_mixture(tmp_path):
    d = str(tmp_path)
    _docs(f"{d}/a.jsonl", 20, 10)
    _docs(f"{d}/b.jsonl", 10, 50)
    single = UrlSingleDatasetLMConfig(tokenizer="passthrough", vocab_size=100, cache_dir=f"{d}/single", train_urls=[f"{d}/a.jsonl"])
    stats = count_corpus_sizes(single, seq_len=16)
    tokens = sum(i % 5 + 3 + 1 for i in range(20))  # + the end-of-sequence token of every document
    assert stats == {"data/stats/train/total_tokens": tokens, "data/stats/train/total_docs": 20, "data/stats/train/total_seqs": tokens // 16}
    mix = LMMixtureDatasetConfig(tokenizer="passthrough", vocab_size=100, cache_dir=f"{d}/mix",
                                 configs={"a": UrlDatasetSourceConfig(train_urls=[f"{d}/a.jsonl"]), "b": UrlDatasetSourceConfig(train_urls=[f"{d}/b.jsonl"])},
                                 train_weights={"a": 0.75, "b": 0.25})
    stats = count_corpus_sizes(mix, prefix="corpus/", seq_len=8)
    assert stats["corpus/train/a/total_docs"] == 20 and stats["corpus/train/b/total_docs"] == 10
    assert stats["corpus/train/a/weight"] == 0.75 and stats["corpus/train/b/weight"] == 0.25
    assert stats["corpus/train/b/total_seqs"] == stats["corpus/train/b/total_tokens"] // 8
