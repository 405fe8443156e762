"""Temperature sampling (src/levanter/layers/sampler.py:15-81): per-row temperature, ``T == 0`` means arg-max, otherwise a
categorical draw from ``softmax(logits / T)``; returns ``(tokens, log-probabilities)``.

The draw uses the Gumbel-max trick with noise from a counter-based hash of ``(row seed, vocabulary index)``, so the CUDA
kernel (``csrc/sampler.cu``) and this module's PyTorch/numpy statement pick the same token for the same seeds."""
from __future__ import annotations

from typing import Optional, Tuple, Union

import numpy as np
import torch

from ..ops import lib

__all__ = ["Sampler", "gumbel_noise"]

_f = {}


def gumbel_noise(seeds: np.ndarray, vocab: int) -> np.ndarray:
    """``[rows, vocab]`` fp32 Gumbel noise, bit-identical in construction to the kernel's."""
    seeds = np.asarray(seeds, dtype=np.int64).astype(np.uint64)[:, None]
    idx = np.arange(vocab, dtype=np.uint64)[None, :]
    with np.errstate(over="ignore"):
        z = seeds ^ (idx * np.uint64(0x9E3779B97F4A7C15))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = ((z >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -np.log(-np.log(u))


class Sampler:
    def __init__(self, Vocab=None):
        self.Vocab = Vocab

    def __call__(self, logits: torch.Tensor, temperatures: Union[torch.Tensor, float], *, key) -> Tuple[torch.Tensor, torch.Tensor]:
        """``logits[..., vocab]``; ``temperatures`` broadcastable to ``logits.shape[:-1]``; ``key``: an int seed or an int64
        tensor of per-row seeds.  Returns int32 tokens and fp32 log-probs of shape ``logits.shape[:-1]``."""
        lead = logits.shape[:-1]
        V = logits.shape[-1]
        z = logits.reshape(-1, V)
        R = z.shape[0]
        t = torch.as_tensor(temperatures, dtype=torch.float32, device=z.device).expand(lead).reshape(-1).contiguous()
        if isinstance(key, torch.Tensor):
            seeds = key.to(device=z.device, dtype=torch.int64).expand(lead).reshape(-1).contiguous()
        else:
            base = int(key)
            seeds = torch.tensor([(base * 1000003 + i) & 0x7FFFFFFFFFFFFFFF for i in range(R)], dtype=torch.int64, device=z.device)
        if z.is_cuda and lib.available() and z.dtype in (torch.float32, torch.bfloat16):
            tokens, lp = self._cuda(z, t, seeds)
        else:
            tokens, lp = self._reference(z, t, seeds)
        return tokens.reshape(lead), lp.reshape(lead)

    @staticmethod
    def _cuda(z, t, seeds):
        c = lib
        if "s" not in _f:
            _f["s"] = lib.fn("lvb_sample", [c.c_void_p, c.c_int, c.c_longlong, c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p,
                                            c.c_void_p, c.c_void_p])
        if z.stride(-1) != 1:
            z = z.contiguous()
        R, V = z.shape
        tokens = torch.empty(R, dtype=torch.int32, device=z.device)
        lp = torch.empty(R, dtype=torch.float32, device=z.device)
        rc = _f["s"](z.data_ptr(), int(z.dtype == torch.bfloat16), z.stride(0), R, V, t.data_ptr(), seeds.data_ptr(), tokens.data_ptr(),
                     lp.data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_sample")
        return tokens, lp

    @staticmethod
    def _reference(z, t, seeds):
        zf = z.float()
        greedy = t == 0
        safe_t = torch.where(greedy, torch.ones_like(t), t)
        scaled = zf / safe_t[:, None]
        g = torch.from_numpy(gumbel_noise(seeds.cpu().numpy(), z.shape[-1])).to(z.device)
        score = torch.where(greedy[:, None], scaled, scaled + g)
        tokens = score.argmax(dim=-1)
        lp = scaled.gather(-1, tokens[:, None]).squeeze(-1) - torch.logsumexp(scaled, dim=-1)
        return tokens.to(torch.int32), lp
