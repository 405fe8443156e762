"""A tokenizer whose "text" is already whitespace-separated token ids (src/levanter/data/passthrough_tokenizer.py:10-38);
used for pre-tokenized corpora and tests.  Implements the slice of the Hugging Face tokenizer API the pipeline calls."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union


class PassthroughTokenizer:
    model_input_names = ["input_ids"]
    is_fast = False
    name_or_path = "passthrough"
    chat_template = None

    def __init__(self, vocab_size: int, **kwargs):
        self._vocab_size = vocab_size
        self._eos = kwargs.get("eos_token_id", vocab_size - 1)
        self._bos = kwargs.get("bos_token_id", None)
        self.pad_token_id = kwargs.get("pad_token_id", self._eos)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def __len__(self) -> int:
        return self._vocab_size

    @property
    def eos_token_id(self):
        return self._eos

    @property
    def bos_token_id(self):
        return self._bos

    @property
    def eos_token(self):
        return str(self._eos)

    @property
    def bos_token(self):
        return None if self._bos is None else str(self._bos)

    def get_vocab(self):
        return {str(i): i for i in range(self._vocab_size)}

    def save_vocabulary(self, save_directory: str, filename_prefix: Optional[str] = None):
        return ()

    def _tokenize(self, text: str) -> List[int]:
        out = []
        for t in text.split():
            try:
                out.append(int(t))
            except ValueError:
                raise ValueError(f"the passthrough tokenizer only accepts whitespace-separated integers, got {t!r}") from None
        return out

    def encode(self, text: str, add_special_tokens: bool = False, **kw) -> List[int]:
        return self._tokenize(text)

    def decode(self, ids: Sequence[int], **kw) -> str:
        return " ".join(str(int(i)) for i in ids)

    def convert_ids_to_tokens(self, ids):
        return [str(int(i)) for i in ids] if not isinstance(ids, int) else str(ids)

    def convert_tokens_to_ids(self, toks):
        return [int(t) for t in toks] if not isinstance(toks, str) else int(toks)

    def __call__(self, text: Union[str, Sequence[str]], return_attention_mask: bool = False, truncation=False, max_length=None,
                 add_special_tokens: bool = False, padding=False, **kw):
        single = isinstance(text, str)
        texts = [text] if single else list(text)
        ids = [self._tokenize(t) for t in texts]
        if truncation and max_length:
            ids = [x[:max_length] for x in ids]
        masks = [[1] * len(x) for x in ids]
        if padding:  # "max_length" pads to max_length, True / "longest" to the longest row of the batch
            width = max_length if (padding == "max_length" and max_length) else max((len(x) for x in ids), default=0)
            masks = [m + [0] * (width - len(m)) for m in masks]
            ids = [x + [self.pad_token_id] * (width - len(x)) for x in ids]
        out = {"input_ids": ids[0] if single else ids}
        if return_attention_mask:
            out["attention_mask"] = masks[0] if single else masks
        return out
