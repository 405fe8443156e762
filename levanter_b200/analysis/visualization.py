"""HTML views of per-token log-probabilities (src/levanter/analysis/visualization.py:21-345): one ``<span>`` per token whose
background encodes the log-probability; a diff view colours tokens by the difference between two models."""
from __future__ import annotations

import html as _html
import os
import re
from typing import Any, List, Optional, Sequence

import numpy as np
import torch

from ..callbacks import StepInfo

_PAGE_HEAD = ("<html><head><meta charset='utf-8'><style>.lp span{font-family:monospace;padding:.2em;border-radius:2px}"
              "</style></head><body><div class='lp'>")


def _escape(s: str) -> str:
    out = _html.escape(str(s), quote=False)
    return re.sub(r"\n", "&#x23CE;<br>", out).replace(" ", "&nbsp;")


def _write(path: str, text: str) -> None:
    import fsspec

    with fsspec.open(path, "w") as f:
        f.write(text)


def visualize_log_probs(tokens: List[List[str]], log_probs: np.ndarray, output_path: str, argmaxes: Optional[List[List[Any]]] = None):
    """Yellow = likely, red = unlikely; opacity grows as the probability falls.  ``argmaxes`` (the model's own best guess
    per position) goes into the tooltip."""
    parts = [_PAGE_HEAD]
    for d, (doc, lps) in enumerate(zip(tokens, log_probs)):
        for i, (tok, lp) in enumerate(zip(doc, lps)):
            extra = ""
            if argmaxes is not None:
                extra = " data-argmax='%s'" % _escape(argmaxes[d][i]).replace("'", "&apos;")
            parts.append(f"<span data-lp='{float(lp):.3f}'{extra}>{_escape(tok)}</span>")
        parts.append("<br><br>")
    parts.append("</div><script>const SCALE=5;document.querySelectorAll('.lp span').forEach(el=>{"
                 "const lp=parseFloat(el.getAttribute('data-lp'));const c=Math.max(lp,-10);const hue=60*((c+10)/10);"
                 "const alpha=(1-Math.exp(lp/SCALE)).toFixed(2);el.style.background=`hsla(${hue},100%,50%,${alpha})`;"
                 "const am=el.getAttribute('data-argmax');el.title=am!==null?`${lp.toFixed(3)} (argmax: ${am})`:lp.toFixed(3);});"
                 "</script></body></html>")
    _write(output_path, "".join(parts))


def visualize_log_prob_diff(tokens: List[List[str]], log_probs_a: np.ndarray, log_probs_b: np.ndarray, output_path: str,
                            diff_threshold: float = 5.0):
    """Blue where model A is more confident than B, red where B is; saturation ~ ``|diff| / diff_threshold``."""
    parts = [_PAGE_HEAD]
    for doc, la, lb in zip(tokens, log_probs_a, log_probs_b):
        for tok, a, b in zip(doc, la, lb):
            d = float(a) - float(b)
            alpha = min(abs(d) / diff_threshold, 1.0)
            hue = 240 if d > 0 else 0
            parts.append(f"<span style='background:hsla({hue},100%,50%,{alpha:.2f})' title='A {float(a):.3f} B {float(b):.3f} "
                         f"diff {d:.3f}'>{_escape(tok)}</span>")
        parts.append("<br><br>")
    parts.append("</div></body></html>")
    _write(output_path, "".join(parts))


def _decode_tokens_pretty(tok, ids: Sequence[int]) -> List[str]:
    if hasattr(tok, "convert_ids_to_tokens") and getattr(tok, "is_fast", False):
        return [str(tok.convert_tokens_to_string([t])) if t is not None else "" for t in tok.convert_ids_to_tokens(list(ids))]
    return [tok.decode([int(i)]) for i in ids]


@torch.no_grad()
def _collect(model, tokenizer, log_prob_fn, test_data, max_docs: int):
    docs, lps, ams = [], [], []
    device = next(model.parameters()).device
    for batch in test_data:
        batch = batch.to(device) if hasattr(batch, "to") else batch
        out = log_prob_fn(model, batch)
        lp, am = out if isinstance(out, tuple) else (out, None)
        for b in range(lp.shape[0]):
            ids = batch.tokens[b].tolist()
            docs.append(_decode_tokens_pretty(tokenizer, ids))
            # log p of token t is produced at position t - 1
            lps.append(np.concatenate([[0.0], lp[b, :-1].float().cpu().numpy()]))
            if am is not None:
                ams.append([""] + _decode_tokens_pretty(tokenizer, am[b, :-1].tolist()))
            if len(docs) >= max_docs:
                return docs, lps, (ams or None)
    return docs, lps, (ams or None)


def compute_and_visualize_log_probs(path: str, model, tokenizer, log_prob_fn, test_data, max_docs: int = 128):
    docs, lps, ams = _collect(model, tokenizer, log_prob_fn, test_data, max_docs)
    visualize_log_probs(docs, np.array(lps, dtype=object), path, argmaxes=ams)


def compute_and_diff_log_probs(path: str, model, comparison_model, tokenizer, log_prob_fn, test_data, max_docs: int = 128):
    batches = list(test_data)
    docs, la, _ = _collect(model, tokenizer, log_prob_fn, batches, max_docs)
    _, lb, _ = _collect(comparison_model, tokenizer, log_prob_fn, batches, max_docs)
    visualize_log_prob_diff(docs, np.array(la, dtype=object), np.array(lb, dtype=object), path)


def cb_compute_and_visualize_log_probs(test_data, tokenizer, log_prob_fn, html_dir: str, max_docs: int = 128):
    def hook(step: StepInfo):
        from .. import tracker as trk

        os.makedirs(html_dir, exist_ok=True)
        path = os.path.join(html_dir, f"step_{step.step}.html")
        compute_and_visualize_log_probs(path, step.eval_model, tokenizer, log_prob_fn, test_data, max_docs=max_docs)
        trk.current_tracker().log_artifact(path, name=f"log_probs_step_{step.step}.html", type="html")

    return hook
