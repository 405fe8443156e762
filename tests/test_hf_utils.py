"""Token byte lengths (the denominator of bits-per-byte) on a tokenizer trained in memory: no download needed."""
import pytest

from levanter_b200.utils.hf_utils import byte_length_of_token, num_cpus_used_by_tokenizer


@pytest.fixture(scope="module")
def tokenizer():
    tokenizers = pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<s>", "</s>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog " * 20, "héllo wörld ünïcode " * 20], trainer)
    return transformers.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>")


def test_byte_lengths_sum_to_the_utf8_length(tokenizer):
    for text in ("the quick brown fox", " leading space", "héllo wörld", "a"):
        ids = tokenizer(text)["input_ids"]
        assert sum(byte_length_of_token(tokenizer, i) for i in ids) == len(text.encode("utf-8")), text


def test_special_tokens_count_zero_bytes(tokenizer):
    assert byte_length_of_token(tokenizer, tokenizer.bos_token_id) == 0
    assert byte_length_of_token(tokenizer, tokenizer.eos_token_id) == 0


def test_tokenizer_cpu_budget(monkeypatch, tokenizer):
    monkeypatch.setenv("TOKENIZERS_PARALLELISM", "false")
    assert num_cpus_used_by_tokenizer(tokenizer) == 1
    monkeypatch.setenv("TOKENIZERS_PARALLELISM", "true")
    assert 1 <= num_cpus_used_by_tokenizer(tokenizer) <= 12
