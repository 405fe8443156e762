"""OpenAI-compatible HTTP server over the generation engine (src/levanter/inference/openai.py:57-810).

``/health``, ``/v1/completions`` and ``/v1/chat/completions`` (no streaming).  HTTP handlers tokenise and hand an
``InferenceRequest`` with a future to a queue; one scheduler thread groups what arrived within ``batch_timeout`` into batches
that fit the engine (sequence slots, tokens per sequence, pages) and one worker thread runs them through
``engine.generate`` under the model lock.  ``reload`` swaps weights between batches: it waits for the lock, so running
requests finish on the old weights; ``unload`` drops model and engine."""
from __future__ import annotations

import asyncio
import dataclasses
import logging
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Literal, Optional, Union

import numpy as np
import torch

from ..compat.hf_checkpoints import RepoRef
from ..models.lm_model import LmConfig, LmHeadModel
from ..trainer import TrainerConfig
from .engine import InferenceEngine, InferenceEngineConfig, Request
from .jit_scheduler import SeqDecodingParams

logger = logging.getLogger(__name__)

try:
    from fastapi import FastAPI, HTTPException
    from pydantic import BaseModel, Field
except ImportError as _e:  # pragma: no cover
    raise ImportError("the OpenAI-compatible server needs `fastapi` and `pydantic`") from _e


class ChatMessage(BaseModel):
    role: Literal["system", "user", "assistant", "tool", "function", "developer"]
    content: Optional[str] = None
    name: Optional[str] = None
    tool_calls: Optional[List[Dict]] = None
    tool_call_id: Optional[str] = None
    function_call: Optional[Dict] = None


class ChatCompletionRequest(BaseModel):
    model: str
    messages: List[ChatMessage]
    frequency_penalty: Optional[float] = None
    logit_bias: Optional[Dict[str, int]] = None
    logprobs: bool = False
    top_logprobs: Optional[int] = None
    max_tokens: int = 1024
    n: Optional[int] = None
    presence_penalty: Optional[float] = None
    response_format: Optional[Dict] = None
    seed: Optional[int] = None
    service_tier: Optional[str] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: Optional[bool] = None
    stream_options: Optional[Dict] = None
    temperature: float = 1.0
    top_p: Optional[float] = None
    tools: Optional[List[Dict]] = None
    tool_choice: Optional[Union[str, Dict]] = None
    parallel_tool_calls: Optional[bool] = None
    user: Optional[str] = None


class CompletionRequest(BaseModel):
    model: str
    prompt: Union[str, List[str]]
    best_of: Optional[int] = None
    echo: Optional[bool] = None
    frequency_penalty: Optional[float] = None
    logit_bias: Optional[Dict[str, int]] = None
    logprobs: Optional[int] = None
    max_tokens: int = 1024
    n: Optional[int] = None
    presence_penalty: Optional[float] = None
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: Optional[bool] = None
    stream_options: Optional[Dict] = None
    suffix: Optional[str] = None
    temperature: float = 1.0
    top_p: Optional[float] = None
    user: Optional[str] = None


@dataclass
class InferenceServerConfig:
    checkpoint_path: Optional[str] = None
    hf_checkpoint: Optional[RepoRef] = None
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    model: LmConfig = field(default_factory=LmConfig)
    tokenizer: Optional[str] = None
    service: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    temperature: float = 0.7
    seed: int = 42
    batch_timeout: float = 0.1  # seconds to wait for more requests before a batch is closed
    host: str = "localhost"
    port: int = 10243


@dataclass
class InferenceRequest:
    request_id: str
    prompt_tokens: List[int]
    max_tokens: int
    temperature: float
    stop_tokens: Optional[List[List[int]]]
    seed: Optional[int]
    future: "asyncio.Future"
    n_generations: int = 1
    enable_logprobs: bool = False


@dataclass
class InferenceResponse:
    request_id: str
    text: str
    tokens: List[int]
    prompt_tokens: int
    completion_tokens: int
    logprobs: Optional[List[float]] = None


class InferenceBatch(list):
    def num_seqs(self) -> int:
        return sum(r.n_generations for r in self)

    def total_tokens(self) -> int:
        return sum(len(r.prompt_tokens) + r.max_tokens for r in self)


WeightSource = Callable[[LmHeadModel], LmHeadModel]


def _fetch_all_from_queue(q: "queue.Queue", timeout: float) -> list:
    """Block up to ``timeout`` for the first item, then take whatever else is already there."""
    out = []
    try:
        out.append(q.get(timeout=timeout))
        while True:
            out.append(q.get_nowait())
    except queue.Empty:
        pass
    return out


class InferenceContext:
    def __init__(self, model: Optional[LmHeadModel], tokenizer, engine: Optional[InferenceEngine], config: InferenceServerConfig):
        self.model, self.tokenizer, self.engine, self.config = model, tokenizer, engine, config
        self.model_lock = threading.Lock()
        self.request_queue: "queue.Queue[InferenceRequest]" = queue.Queue()
        self.batch_queue: "queue.Queue[InferenceBatch]" = queue.Queue()
        self.shutdown_event = threading.Event()
        self._next_request_id = 0
        self._threads: List[threading.Thread] = []

    def start(self) -> None:
        for target, name in ((self._inference_loop, "inference-scheduler"), (self._batch_processing_loop, "inference-worker")):
            t = threading.Thread(target=target, name=name, daemon=True)
            t.start()
            self._threads.append(t)

    def shutdown(self) -> None:
        self.shutdown_event.set()
        for t in self._threads:
            t.join(timeout=5)

    def unload(self) -> None:
        with self.model_lock:
            self.model = None
            self.engine = None

    def reload(self, weight_callback: WeightSource) -> None:
        t0 = time.time()
        with self.model_lock:
            waited = time.time() - t0
            self.model = weight_callback(self.model)
            self.engine = InferenceEngine.from_model_with_config(model=self.model, tokenizer=self.tokenizer, config=self.config.service)
        logger.info(f"Model reloaded (waited {waited:.2f}s for running requests, {time.time() - t0 - waited:.2f}s to load)")

    def submit_request(self, prompt_tokens: List[int], max_tokens: int, temperature: float, stop_tokens, seed: Optional[int],
                       future, n_generations: int = 1, enable_logprobs: bool = False) -> str:
        assert not self.shutdown_event.is_set(), "InferenceContext is shut down"
        rid = f"req_{self._next_request_id}"
        self._next_request_id += 1
        self.request_queue.put(InferenceRequest(rid, prompt_tokens, max_tokens, temperature, stop_tokens, seed, future, n_generations,
                                                enable_logprobs))
        return rid

    # -- threads ------------------------------------------------------------------------------------------------
    def _fail(self, req: InferenceRequest, exc: Exception) -> None:
        loop = req.future.get_loop()
        loop.call_soon_threadsafe(lambda: (not req.future.done()) and req.future.set_exception(exc))

    def _inference_loop(self) -> None:
        while not self.shutdown_event.is_set():
            requests = _fetch_all_from_queue(self.request_queue, self.config.batch_timeout)
            if not requests:
                continue
            cfg = self.config.service
            max_per_seq = cfg.max_pages_per_seq * cfg.page_size
            max_per_batch = cfg.imputed_max_pages * cfg.page_size
            batch = InferenceBatch()
            for r in requests:
                if len(r.prompt_tokens) + r.max_tokens > max_per_seq or r.n_generations > cfg.max_seqs:
                    self._fail(r, ValueError(f"request needs {len(r.prompt_tokens) + r.max_tokens} tokens / {r.n_generations} sequences; "
                                             f"the server allows {max_per_seq} tokens per sequence and {cfg.max_seqs} sequences"))
                    continue
                if batch and (batch.num_seqs() + r.n_generations > cfg.max_seqs
                              or batch.total_tokens() + len(r.prompt_tokens) + r.max_tokens > max_per_batch):
                    self.batch_queue.put(batch)
                    batch = InferenceBatch()
                batch.append(r)
            if batch:
                self.batch_queue.put(batch)

    def _batch_processing_loop(self) -> None:
        while not self.shutdown_event.is_set():
            try:
                batch = self.batch_queue.get(timeout=0.2)
            except queue.Empty:
                continue
            try:
                with self.model_lock:
                    self._execute_batch(batch)
            except Exception as e:  # noqa: BLE001 - forwarded to the waiting HTTP handlers
                logger.exception("batch failed")
                for r in batch:
                    self._fail(r, e)

    def _execute_batch(self, batch: InferenceBatch) -> None:
        if self.engine is None:
            raise RuntimeError("no model is loaded")
        reqs = []
        for i, r in enumerate(batch):
            stops = None
            if r.stop_tokens:
                L = max(len(s) for s in r.stop_tokens)
                from .utils import INVALID

                stops = np.full((len(r.stop_tokens), L), INVALID, np.int32)
                for j, s in enumerate(r.stop_tokens):
                    stops[j, L - len(s):] = s
            seed = r.seed if r.seed is not None else self.config.seed + hash(r.request_id) % 100003
            params = SeqDecodingParams(max_num_tokens=len(r.prompt_tokens) + r.max_tokens, stop_tokens=stops,
                                       temperature=float(r.temperature), key=int(seed))
            reqs.append(Request(prompt_tokens=r.prompt_tokens, request_id=i, decode_params=params, n_generations=r.n_generations,
                                enable_logprobs=r.enable_logprobs))
        result = self.engine.generate(reqs)
        k = 0
        for r in batch:
            responses = []
            for _ in range(r.n_generations):
                toks = result.tokens[k]
                lps = result.logprobs[k] if (result.logprobs is not None and r.enable_logprobs) else None
                k += 1
                text = self.tokenizer.decode(toks, skip_special_tokens=True)
                responses.append(InferenceResponse(r.request_id, text, toks, len(r.prompt_tokens), len(toks), lps))
            r.future.get_loop().call_soon_threadsafe(lambda f=r.future, v=responses: (not f.done()) and f.set_result(v))


# --------------------------------------------------------------------------------------------------------- handlers
def _health_check() -> dict:
    return {"status": "healthy", "service": "levanter_b200-inference"}


def _stop_token_lists(tokenizer, stop) -> Optional[List[List[int]]]:
    if stop is None:
        return None
    stops = [stop] if isinstance(stop, str) else list(stop)
    out = []
    for s in stops:
        ids = tokenizer(s, add_special_tokens=False)["input_ids"] if callable(tokenizer) else tokenizer.encode(s)
        if ids:
            out.append(list(ids))
    return out or None


def _logprob_payload(tokenizer, resp: InferenceResponse):
    toks = [tokenizer.decode([t]) for t in resp.tokens]
    return {"tokens": toks, "token_logprobs": resp.logprobs, "top_logprobs": None, "text_offset": [int(x) for x in np.cumsum([0] + [len(t) for t in toks[:-1]])]}


async def _await_responses(ctx: InferenceContext, prompt_tokens, request, n: int, want_lp: bool) -> List[InferenceResponse]:
    fut = asyncio.get_event_loop().create_future()
    ctx.submit_request(prompt_tokens, request.max_tokens, request.temperature, _stop_token_lists(ctx.tokenizer, request.stop), request.seed,
                       fut, n_generations=n, enable_logprobs=want_lp)
    try:
        return await fut
    except ValueError as e:
        raise HTTPException(status_code=400, detail=str(e))
    except Exception as e:  # noqa: BLE001
        raise HTTPException(status_code=500, detail=str(e))


async def _create_completion(ctx: InferenceContext, request: CompletionRequest) -> dict:
    if request.stream:
        raise HTTPException(status_code=400, detail="streaming is not supported")
    prompts = [request.prompt] if isinstance(request.prompt, str) else list(request.prompt)
    n = request.n or 1
    want_lp = request.logprobs is not None and request.logprobs > 0
    choices, p_tok, c_tok = [], 0, 0
    pending = [_await_responses(ctx, ctx.tokenizer(p)["input_ids"], request, n, want_lp) for p in prompts]
    for responses in await asyncio.gather(*pending):
        for r in responses:
            choices.append({"index": len(choices), "text": r.text, "finish_reason": "stop" if r.completion_tokens < request.max_tokens else "length",
                            "logprobs": _logprob_payload(ctx.tokenizer, r) if want_lp else None})
            c_tok += r.completion_tokens
        p_tok += responses[0].prompt_tokens
    return {"id": f"cmpl-{uuid.uuid4().hex}", "object": "text_completion", "created": int(time.time()), "model": request.model,
            "choices": choices, "usage": {"prompt_tokens": p_tok, "completion_tokens": c_tok, "total_tokens": p_tok + c_tok}}


async def _create_chat_completion(ctx: InferenceContext, request: ChatCompletionRequest) -> dict:
    if request.stream:
        raise HTTPException(status_code=400, detail="streaming is not supported")
    messages = [{k: v for k, v in m.model_dump().items() if v is not None} for m in request.messages]
    try:
        prompt_tokens = ctx.tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
    except Exception as e:  # noqa: BLE001 - no template: fall back to a plain transcript
        logger.warning(f"chat template failed ({e}); using a plain transcript")
        text = "".join(f"{m['role']}: {m.get('content', '')}\n" for m in messages) + "assistant: "
        prompt_tokens = ctx.tokenizer(text)["input_ids"]
    if hasattr(prompt_tokens, "keys"):  # a dict, or the tokenizer's mapping class (not a dict subclass) in newer releases
        prompt_tokens = prompt_tokens["input_ids"]
    prompt_tokens = [int(t) for t in prompt_tokens]
    n = request.n or 1
    responses = await _await_responses(ctx, list(prompt_tokens), request, n, request.logprobs)
    choices = []
    for i, r in enumerate(responses):
        lp = None
        if request.logprobs and r.logprobs is not None:
            lp = {"content": [{"token": ctx.tokenizer.decode([t]), "logprob": float(l), "bytes": list(ctx.tokenizer.decode([t]).encode()),
                               "top_logprobs": []} for t, l in zip(r.tokens, r.logprobs)]}
        choices.append({"index": i, "message": {"role": "assistant", "content": r.text},
                        "finish_reason": "stop" if r.completion_tokens < request.max_tokens else "length", "logprobs": lp})
    c_tok = sum(r.completion_tokens for r in responses)
    return {"id": f"chatcmpl-{uuid.uuid4().hex}", "object": "chat.completion", "created": int(time.time()), "model": request.model,
            "choices": choices, "usage": {"prompt_tokens": responses[0].prompt_tokens, "completion_tokens": c_tok,
                                          "total_tokens": responses[0].prompt_tokens + c_tok}}


class InferenceServer:
    def __init__(self, config: InferenceServerConfig, inference_context: InferenceContext, app: "FastAPI"):
        self.config, self.inference_context, self.app = config, inference_context, app
        self._server = None

    @staticmethod
    def create(config: InferenceServerConfig, model: Optional[LmHeadModel] = None, tokenizer=None) -> "InferenceServer":
        """Build model, engine and app.  ``model``/``tokenizer`` may be passed in (tests, in-process serving during
        training); otherwise they are loaded from ``checkpoint_path`` / ``hf_checkpoint`` and ``tokenizer``."""
        if tokenizer is None:
            from ..compat.hf_checkpoints import load_tokenizer

            name = config.tokenizer or (str(config.hf_checkpoint) if config.hf_checkpoint is not None else None)
            if name is None:
                raise ValueError("a tokenizer is required")
            tokenizer = load_tokenizer(name)
        if model is None:
            model = _load_model(config, tokenizer)
        engine = InferenceEngine.from_model_with_config(model=model, tokenizer=tokenizer, config=config.service)
        ctx = InferenceContext(model, tokenizer, engine, config)
        ctx.start()
        return InferenceServer(config, ctx, InferenceServer._create_app(ctx))

    @staticmethod
    def _create_app(ctx: InferenceContext) -> "FastAPI":
        app = FastAPI(title="levanter_b200 inference", version="1.0.0")

        @app.get("/health")
        async def health_check():
            return _health_check()

        @app.post("/v1/completions")
        async def create_completion(request: CompletionRequest):
            return await _create_completion(ctx, request)

        @app.post("/v1/chat/completions")
        async def create_chat_completion(request: ChatCompletionRequest):
            return await _create_chat_completion(ctx, request)

        return app

    def unload(self) -> None:
        self.inference_context.unload()

    def reload(self, weight_callback: WeightSource) -> None:
        self.inference_context.reload(weight_callback)

    def serve(self) -> None:
        import uvicorn

        uvicorn.run(self.app, host=self.config.host, port=self.config.port)

    async def serve_async(self) -> None:
        import uvicorn

        self._server = uvicorn.Server(uvicorn.Config(self.app, host=self.config.host, port=self.config.port))
        await self._server.serve()

    def shutdown(self) -> None:
        if self._server is not None:
            self._server.should_exit = True
        self.inference_context.shutdown()


def _load_model(config: InferenceServerConfig, tokenizer) -> LmHeadModel:
    from ..main._common import load_model
    from ..parallel.mesh import local_device

    return load_model(config.model, tokenizer, checkpoint_path=config.checkpoint_path, hf_checkpoint=config.hf_checkpoint,
                      dtype=config.trainer.mp.compute_dtype, device=local_device()).eval()
