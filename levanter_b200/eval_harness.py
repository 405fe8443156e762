"""LM Evaluation Harness integration (src/levanter/eval_harness.py).

The harness asks for ``loglikelihood(context, continuation)`` of many short requests.  They are tokenised, packed several
to a row with segment ids (``greedy_pack_prompt_completions``), scored by one forward pass per batch, and reduced per segment
on the device (summed log-likelihood and "every continuation token was the arg-max").  Process 0 drives the harness; when
the model is tensor-parallel the other processes sit in :meth:`_LmEvalHarnessWorker.worker_message_loop` and receive each
batch by broadcast, like the reference's worker protocol (:96-225).

The ``lm_eval`` package is optional: configs parse and the scoring core (:class:`LoglikelihoodScorer`) works without it; only
task loading and ``evaluator.evaluate`` need it."""
from __future__ import annotations

import dataclasses
import json
import logging
import tempfile
from dataclasses import dataclass
from functools import cached_property
from typing import Dict, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import tracker as trk
from .callbacks import StepInfo
from .data.packing import PromptCompletion, greedy_pack_prompt_completions
from .models.gpt2 import Gpt2Config
from .models.lm_model import LmConfig, LmExample, LmHeadModel
from .trainer import TrainerConfig

logger = logging.getLogger(__name__)

try:  # pragma: no cover - optional dependency
    from lm_eval import evaluator as _evaluator
    from lm_eval.api.instance import Instance
    from lm_eval.api.model import LM
except ImportError:
    _evaluator = None
    Instance = object  # type: ignore

    class LM:  # type: ignore
        pass


@dataclass(frozen=True)
class TaskConfig:
    """One task of the harness; ``None`` fields are left to the harness defaults (they are dropped by :meth:`to_dict`)."""
    task: str
    task_alias: Optional[str] = None
    num_fewshot: Optional[int] = None
    use_prompt: Optional[str] = None
    description: Optional[str] = None
    target_delimiter: Optional[str] = None
    fewshot_delimiter: Optional[str] = None
    doc_to_text: Optional[str] = None
    doct_to_target: Optional[str] = None
    doc_to_choice: Optional[str] = None

    def to_dict(self) -> dict:
        return {k: v for k, v in dataclasses.asdict(self).items() if v is not None}


@dataclass(frozen=True)
class LmEvalHarnessConfig:
    task_spec: List[Union[TaskConfig, str]]
    max_examples: Optional[int] = None
    max_eval_length: Optional[int] = None
    log_samples: bool = False
    bootstrap_iters: int = 0
    apply_chat_template: bool = False

    def to_task_spec(self) -> List[Union[str, dict]]:
        return [t.to_dict() if isinstance(t, TaskConfig) else t for t in self.task_spec]

    def to_task_dict(self) -> dict:
        """{name: harness task}.  A task given with an alias is loaded under that alias, so the same task can appear with
        several few-shot settings in one run."""
        try:
            import lm_eval.tasks as tasks
        except ImportError as e:
            raise ImportError("the `lm_eval` package is required to load evaluation-harness tasks") from e
        manager = tasks.TaskManager()
        out: dict = {}
        for task in self.to_task_spec():
            if isinstance(task, str):
                out.update(tasks.get_task_dict(task, manager))
                continue
            our_name = task.get("task_alias", task["task"]).replace(" ", "_")
            loaded = tasks.get_task_dict([task], manager)
            for name, obj in self._rename(loaded, task["task"], our_name).items():
                if name in out:
                    raise ValueError(f"Task {name} already exists")
                out[name] = obj
        return out

    @staticmethod
    def _rename(loaded: dict, lm_eval_name: str, our_name: str) -> dict:
        def fix(name):
            name = getattr(name, "group", name)
            return name.replace(lm_eval_name, our_name, 1) if isinstance(name, str) and name.startswith(lm_eval_name) else name

        out = {}
        for k, v in loaded.items():
            if isinstance(v, dict):
                out[fix(k)] = LmEvalHarnessConfig._rename(v, lm_eval_name, our_name)
            else:
                cfg = getattr(v, "config", None)
                if cfg is not None and hasattr(cfg, "task"):
                    cfg.task = fix(cfg.task)
                out[fix(k)] = v
        return out


@dataclass(frozen=True)
class EvalHarnessMainConfig:
    eval_harness: LmEvalHarnessConfig
    tokenizer: str
    checkpoint_path: str
    checkpoint_is_hf: bool = False
    apply_chat_template: bool = False
    trainer: TrainerConfig = dataclasses.field(default_factory=TrainerConfig)
    model: LmConfig = dataclasses.field(default_factory=Gpt2Config)

    @property
    def EvalBatch(self) -> int:
        return self.trainer.eval_batch_size

    @cached_property
    def the_tokenizer(self):
        from .compat.hf_checkpoints import load_tokenizer

        return load_tokenizer(self.tokenizer)


# ------------------------------------------------------------------------------------------------------- requests
def _encode_pair(tokenizer, context: str, continuation: str, move_trailing_space: bool = True) -> Tuple[List[int], List[int]]:
    """Token ids of the context and of the continuation, split where the context's own encoding ends.  Trailing spaces of a
    plain context go with the continuation, so that the token boundary is where free-running text has it."""
    if move_trailing_space:
        n_spaces = len(context) - len(context.rstrip())
        if n_spaces > 0:
            continuation = context[-n_spaces:] + continuation
            context = context[:-n_spaces]
    whole = tokenizer(context + continuation)["input_ids"]
    ctx = tokenizer(context)["input_ids"] if context else []
    return list(whole[:len(ctx)]), list(whole[len(ctx):])


def _iterate_tokenized_requests(requests, tokenizer, max_len: int, batch_size: int = 128,
                                apply_chat_template: bool = False) -> Iterator[PromptCompletion]:
    """``(context, continuation)`` requests as :class:`PromptCompletion` s for packing; ``segment_id`` is the request's position
    (src/levanter/eval_harness.py:821-866).  With ``apply_chat_template`` the context becomes a user turn followed by the
    generation prompt, kept exactly as the template writes it.  A request longer than ``max_len`` loses tokens from the left:
    the continuation is what is scored.  An empty context is replaced by the beginning-of-text token."""
    chat = apply_chat_template and getattr(tokenizer, "chat_template", None)
    for i, r in enumerate(requests):
        context, continuation = r.args if hasattr(r, "args") else r
        if chat:
            context = tokenizer.apply_chat_template([{"role": "user", "content": context}], tokenize=False, add_generation_prompt=True)
        ctx, cont = _encode_pair(tokenizer, context, continuation, move_trailing_space=not chat)
        if not ctx:
            ctx = [tokenizer.bos_token_id if tokenizer.bos_token_id is not None else tokenizer.eos_token_id]
        ids, prompt_len = ctx + cont, len(ctx)
        if len(ids) > max_len:
            logger.warning(f"Request {i} is too long. Truncating.")
            prompt_len -= len(ids) - max_len
            ids = ids[-max_len:]
        yield PromptCompletion(ids=ids, prompt_length=max(prompt_len, 1), segment_id=i)


# ------------------------------------------------------------------------------------------------------- scoring
class LoglikelihoodScorer:
    """Scores ``(context ids, continuation ids)`` pairs: returns ``(sum log p(continuation | context), greedy?)`` each."""

    def __init__(self, model: LmHeadModel, eval_pos: int, eval_batch: int, pad_token_id: int, max_packed_segments: int = 64,
                 device=None):
        self.model, self.eval_pos, self.eval_batch = model, eval_pos, eval_batch
        self.pad_token_id = pad_token_id
        self.max_packed_segments = max_packed_segments
        self.device = device or next(model.parameters()).device

    def pack(self, pairs: Sequence[Tuple[Sequence[int], Sequence[int]]]) -> List[LmExample]:
        seqs = []
        for i, (ctx, cont) in enumerate(pairs):
            ids = list(ctx) + list(cont)
            prompt_len = len(ctx)
            if len(ids) > self.eval_pos:  # keep the end: the continuation must survive
                cut = len(ids) - self.eval_pos
                ids = ids[cut:]
                prompt_len = max(prompt_len - cut, 1)
            seqs.append(PromptCompletion(ids=ids, prompt_length=max(prompt_len, 1), segment_id=i))
        return greedy_pack_prompt_completions(self.eval_pos, seqs, self.pad_token_id, self.max_packed_segments)

    @torch.no_grad()
    def score_batch(self, batch: LmExample) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``batch``: stacked packed rows.  Returns (segment ids, log-likelihoods, all-greedy flags) flattened over rows,
        with -1 ids for unused slots."""
        batch = batch.to(self.device)
        m = self.model
        acts = m.activations(batch.tokens, batch.attn_mask)
        acts = acts[0] if isinstance(acts, tuple) else acts
        logits = (acts @ m.get_lm_head().to(acts.dtype).t()).float()
        targets = torch.roll(batch.tokens, -1, dims=-1).long()
        logp = torch.log_softmax(logits, dim=-1)
        tok_lp = logp.gather(-1, targets.unsqueeze(-1)).squeeze(-1)
        correct = logits.argmax(-1) == targets
        mask = batch.loss_mask.bool()
        seg = batch.attn_mask.segment_ids[0]
        B = seg.shape[0]
        K = self.max_packed_segments
        ids = torch.full((B, K), -1, dtype=torch.long, device=seg.device)
        lls = torch.zeros((B, K), dtype=torch.float32, device=seg.device)
        oks = torch.ones((B, K), dtype=torch.bool, device=seg.device)
        for b in range(B):
            uniq = torch.unique(seg[b][seg[b] >= 0])[:K]
            n = uniq.numel()
            member = (uniq[:, None] == seg[b][None, :]) & mask[b][None, :]
            ids[b, :n] = uniq
            lls[b, :n] = (member.float() * tok_lp[b][None, :]).sum(-1)
            oks[b, :n] = (~member | correct[b][None, :]).all(-1)
        return ids.reshape(-1), lls.reshape(-1), oks.reshape(-1)

    def score(self, pairs: Sequence[Tuple[Sequence[int], Sequence[int]]]) -> List[Tuple[float, bool]]:
        packed = self.pack(pairs)
        ll = np.zeros(len(pairs))
        ok = np.zeros(len(pairs), dtype=bool)
        seen = np.zeros(len(pairs), dtype=bool)
        was_training = self.model.training
        self.model.eval()
        try:
            for i in range(0, len(packed), self.eval_batch):
                rows = packed[i:i + self.eval_batch]
                ids, lls, oks = self.score_batch(LmExample.stack(rows))
                ids, lls, oks = ids.cpu().numpy(), lls.cpu().numpy(), oks.cpu().numpy()
                valid = ids >= 0
                ll[ids[valid]] = lls[valid]
                ok[ids[valid]] = oks[valid]
                seen[ids[valid]] = True
        finally:
            self.model.train(was_training)
        missing = np.nonzero(~seen)[0]
        assert len(missing) == 0, f"Missing points: {missing[:10]}"
        return [(float(a), bool(b)) for a, b in zip(ll, ok)]


class _Message:
    STOP = 0
    LOGLIKELIHOOD = 1


class _LmEvalHarnessWorker:
    """Runs scoring on every process of the job.  Process 0 calls :meth:`dispatch_loglikelihood`; the others loop in
    :meth:`worker_message_loop` until :meth:`stop`."""

    def __init__(self, EvalBatch: int, EvalPos: int, model: LmHeadModel, axis_resources, tokenizer, mp, max_packed_segments: int = 64,
                 apply_chat_template: bool = False):
        self.tokenizer = tokenizer
        self.EvalBatch, self.EvalPos = int(getattr(EvalBatch, "size", EvalBatch)), int(getattr(EvalPos, "size", EvalPos))
        self.model = model
        self.max_packed_segments = max_packed_segments
        self.apply_chat_template = apply_chat_template
        pad = tokenizer.pad_token_id if getattr(tokenizer, "pad_token_id", None) is not None else tokenizer.eos_token_id
        self.scorer = LoglikelihoodScorer(model, self.EvalPos, self.EvalBatch, pad, max_packed_segments)

    @staticmethod
    def _multi() -> bool:
        import torch.distributed as dist

        return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1

    def _bcast(self, obj):
        if not self._multi():
            return obj
        import torch.distributed as dist

        box = [obj]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def make_harness_lm(self) -> "LevanterHarnessLM":
        return LevanterHarnessLM(self)

    def worker_message_loop(self) -> None:
        while True:
            msg = self._bcast(None)
            if msg is None or msg[0] == _Message.STOP:
                return
            self.scorer.score_batch(msg[1])

    def dispatch_loglikelihood(self, batch: LmExample):
        self._bcast((_Message.LOGLIKELIHOOD, batch))
        return self.scorer.score_batch(batch)

    def stop(self) -> None:
        self._bcast((_Message.STOP, None))


class LevanterHarnessLM(LM):
    def __init__(self, leader: _LmEvalHarnessWorker):
        try:
            super().__init__()
        except TypeError:
            pass
        self.leader = leader
        self.tokenizer = leader.tokenizer

    def _encode_pair(self, context: str, continuation: str, move_trailing_space: bool = True) -> Tuple[List[int], List[int]]:
        return _encode_pair(self.tokenizer, context, continuation, move_trailing_space)

    def loglikelihood(self, requests) -> List[Tuple[float, bool]]:
        scorer = self.leader.scorer
        seqs = list(_iterate_tokenized_requests(requests, self.tokenizer, scorer.eval_pos, 128, self.leader.apply_chat_template))
        packed = greedy_pack_prompt_completions(scorer.eval_pos, seqs, scorer.pad_token_id, scorer.max_packed_segments)
        ll = np.zeros(len(seqs))
        ok = np.zeros(len(seqs), dtype=bool)
        for i in range(0, len(packed), scorer.eval_batch):
            ids, lls, oks = self.leader.dispatch_loglikelihood(LmExample.stack(packed[i:i + scorer.eval_batch]))
            ids, lls, oks = ids.cpu().numpy(), lls.cpu().numpy(), oks.cpu().numpy()
            valid = ids >= 0
            ll[ids[valid]] = lls[valid]
            ok[ids[valid]] = oks[valid]
        return [(float(a), bool(b)) for a, b in zip(ll, ok)]

    def loglikelihood_rolling(self, requests):
        raise NotImplementedError()

    def generate_until(self, requests):
        raise NotImplementedError()


def _compute_averages(outputs: dict) -> Dict[str, float]:
    """Macro (plain mean over tasks) and micro (weighted by effective sample count) averages of every metric."""
    averages: Dict[str, float] = {}
    metric_keys = set()
    for res in outputs["results"].values():
        metric_keys.update(k for k in res.keys() if "stderr" not in k and k != "alias")
    for metric in metric_keys:
        vals = [(outputs["results"][t].get(metric), outputs["n-samples"][t]["effective"]) for t in outputs["n-samples"]
                if outputs["results"][t].get(metric) is not None]
        if not vals:
            continue
        v, n = zip(*vals)
        averages["macro_avg_" + metric] = float(np.mean(v))
        if sum(n) > 0:
            averages["micro_avg_" + metric] = float(np.average(v, weights=n))
    return averages


def _actually_run_eval_harness(config: LmEvalHarnessConfig, model: LmHeadModel, tasks_to_run: dict, tokenizer, EvalBatch,
                               axis_resources, mp) -> Optional[dict]:
    from .distributed import process_index

    eval_pos = model.config.seq_len if config.max_eval_length is None else config.max_eval_length
    worker = _LmEvalHarnessWorker(EvalBatch, eval_pos, model, axis_resources, tokenizer, mp, max_packed_segments=64,
                                  apply_chat_template=config.apply_chat_template)
    if process_index() != 0:
        worker.worker_message_loop()
        return None
    if _evaluator is None:
        raise ImportError("the `lm_eval` package is required to run the evaluation harness")
    harness = worker.make_harness_lm()
    try:
        outputs = _evaluator.evaluate(harness, tasks_to_run, limit=config.max_examples, log_samples=config.log_samples,
                                      bootstrap_iters=config.bootstrap_iters)
    finally:
        worker.stop()
    outputs["averages"] = _compute_averages(outputs)
    return outputs


def log_report_to_tracker(prefix: str, report: dict, tracker=None) -> None:
    tracker = tracker or trk.current_tracker()
    to_log = {}
    for task, res in report["results"].items():
        for name, value in res.items():
            name = name[:-5] if name.endswith(",none") else name
            if isinstance(value, (float, int)):
                to_log[f"{prefix}/{task}/{name}"] = value
    for name, value in report.get("averages", {}).items():
        name = name[:-5] if name.endswith(",none") else name
        if isinstance(value, (float, int)):
            to_log[f"{prefix}/averages/{name}"] = value
    tracker.log(to_log, step=None)


def lm_eval_harness(config: LmEvalHarnessConfig, tokenizer, EvalBatch, axis_resources, mp):
    """Training hook: runs the harness on the evaluation weights and logs ``lm_eval/<task>/<metric>``."""
    tasks_to_run = config.to_task_dict()

    def hook(step: StepInfo, force: bool = False):
        if step.step == 0 and not force:
            return
        outputs = _actually_run_eval_harness(config, step.eval_model, tasks_to_run, tokenizer, EvalBatch, axis_resources, mp)
        if outputs is not None:
            log_report_to_tracker("lm_eval", outputs, trk.current_tracker())
            with tempfile.NamedTemporaryFile("w", delete=False, suffix=".json") as f:
                json.dump(outputs, f, default=str)
                f.flush()
                trk.current_tracker().log_artifact(f.name, name=f"lm_eval_harness_results.{step.step}.json", type="lm_eval_output")

    return hook


def run_lm_eval_harness(config: LmEvalHarnessConfig, model, tokenizer, EvalBatch, axis_resources=None, mp=None) -> Optional[dict]:
    return _actually_run_eval_harness(config, model, config.to_task_dict(), tokenizer, EvalBatch, axis_resources, mp)


def run_eval_harness_main(config: EvalHarnessMainConfig):
    """``python -m levanter_b200.eval_harness``: evaluate a framework or Hugging Face checkpoint on harness tasks."""
    from .checkpoint import load_checkpoint
    from .distributed import process_index
    from .trainer import local_device

    config.trainer.initialize()
    tokenizer = config.the_tokenizer
    device = local_device()
    dtype = config.trainer.mp.compute_dtype
    if config.checkpoint_is_hf:
        converter = config.model.hf_checkpoint_converter().replaced(reference_checkpoint=config.checkpoint_path, tokenizer=tokenizer)
        model = converter.load_pretrained(ref=config.checkpoint_path, dtype=dtype, device=device)
    else:
        model = config.model.build(len(tokenizer), seed=0, device=device)
        model = load_checkpoint(model, config.checkpoint_path, subpath="model").to(dtype)
    outputs = run_lm_eval_harness(config.eval_harness, model, tokenizer, config.EvalBatch, None, config.trainer.mp)
    if process_index() == 0 and outputs is not None:
        log_report_to_tracker("lm_eval", outputs, trk.current_tracker())
        print(json.dumps(outputs.get("averages", {}), indent=2))
    return outputs


if __name__ == "__main__":
    from . import config as _cfg

    _cfg.main(run_eval_harness_main)()
