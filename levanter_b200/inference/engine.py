"""Generation engine: continuous batching over a paged KV cache (src/levanter/inference/engine.py:36-1258).

Division of labour.  The host owns all scheduling state (slots, pages, token buffers, stop sequences) and plans ahead; the
GPU runs whole decode *calls*: up to ``max_rounds`` rounds in which the tokens sampled in one round are fed straight into
the next on the device.  The host prepares every round's ``PageBatchInfo``, positions and sampling seeds before the call,
copies them in one transfer, and reads all sampled tokens back in one transfer afterwards; stop sequences and length limits
are then applied to the rounds in order and whatever a sequence produced after its end is discarded.  A finished sequence
therefore costs at most ``max_rounds - 1`` wasted token-steps, and a decode call has two host/device synchronisation points
instead of two per token.  (The reference keeps the same round structure inside a compiled ``while_loop``, :539-633.)

Admission follows the reference (:807-854): a request is admitted when a slot is free for each of its ``n_generations``
and the free pages cover its prompt plus one page per clone; prompts are prefilled in batches of at most
``max_seqs_in_prefill`` sequences / ``max_prefill_size`` tokens.  Clones (``n > 1``) share the parent's full pages; a
partially filled last page is copied (:423-535).  Outputs exclude the prompt."""
from __future__ import annotations

import dataclasses
import logging
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..layers.attention import KvPageCache
from ..layers.sampler import Sampler
from .jit_scheduler import DecodeState, SeqDecodingParams, _DecodeOutputs
from .page_table import PageBatchInfo, PageTable
from .utils import INVALID, is_valid

logger = logging.getLogger(__name__)


@dataclass(frozen=True)
class Request:
    """One prompt; ``n_generations`` independent continuations are sampled for it."""
    prompt_tokens: List[int]
    request_id: int
    decode_params: SeqDecodingParams
    n_generations: int
    enable_logprobs: bool = False


@dataclass
class DecodeResult:
    id: int
    choice: int
    token_list: List[int]
    tokens_decoded: int = 0
    done: bool = False
    logprobs: List[float] = field(default_factory=list)


@dataclass(frozen=True)
class InferenceEngineConfig:
    max_pages: Optional[int] = None  # default: max_seqs * max_pages_per_seq
    max_seqs: int = 16
    page_size: int = 128
    max_pages_per_seq: int = 64
    compute_dtype: torch.dtype = torch.bfloat16  # KV cache dtype
    max_queued_tokens: int = 512
    max_seqs_in_prefill: int = 16
    max_prefill_size: Optional[int] = None  # tokens per prefill batch; default: max sequence length
    max_tokens_per_round: Optional[int] = None  # accepted for compatibility: a round always holds one token per live sequence
    max_rounds: int = 8  # decode rounds per device call
    max_stop_seqs: int = 4
    max_stop_tokens: int = 16
    seed: int = 0
    enable_logprobs: bool = False
    use_cuda_graph: bool = False  # capture the decode call (fixed shapes) and replay it

    @property
    def imputed_max_pages(self) -> int:
        return int(self.max_pages) if self.max_pages is not None else int(self.max_seqs * self.max_pages_per_seq)


@dataclass
class GenState:
    cache: object  # what ``model.initial_cache`` returned (a KvPageCache or a list of them, one per layer)
    decode_state: DecodeState


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    logprobs: Optional[List[List[float]]]
    total_generated: int


PREFILL_PAD = 256  # packed prefill tokens are padded to this multiple (two query tiles of the flash-attention kernel)


class _DecodeGraph:
    """Static input/output buffers and the captured graph of one decode round."""

    def __init__(self, engine: "InferenceEngine", example: PageBatchInfo):
        from ..ops import lib

        dev = engine.device
        T = engine.config.max_seqs
        self.tok = torch.zeros(T, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(T, dtype=torch.int32, device=dev)
        self.seeds = torch.zeros(T, dtype=torch.int64, device=dev)
        self.temps = torch.zeros(T, dtype=torch.float32, device=dev)
        z = lambda t: torch.zeros(t.shape, dtype=t.dtype, device=dev)  # noqa: E731
        # warm-up and capture run on tables that address nothing: no sequences, every token destination invalid
        self.binfo = PageBatchInfo(z(example.slot_ids), z(example.page_indices), z(example.seq_lens), z(example.cu_q_lens),
                                   z(example.num_seqs), torch.full(example.new_token_dests.shape, INVALID, dtype=example.new_token_dests.dtype, device=dev),
                                   example.page_size)
        self._shapes = self._shape_key(example)
        if lib.available():
            lib.status_buffer()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):  # lazy initialisation (kernel attributes, scratch buffers, cuBLAS handles) happens here
                self._round(engine)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.out_tok, self.out_lp = self._round(engine)
            self.tok.copy_(self.out_tok)

    def _round(self, engine):
        logits = engine._forward(self.tok, self.binfo, self.pos)
        return engine.sampler(logits, self.temps, key=self.seeds)

    @staticmethod
    def _shape_key(b: PageBatchInfo):
        return tuple(tuple(t.shape) for t in (b.slot_ids, b.page_indices, b.seq_lens, b.cu_q_lens, b.num_seqs, b.new_token_dests))

    def matches(self, b: PageBatchInfo) -> bool:
        return self._shape_key(b) == self._shapes

    def load_round(self, b: PageBatchInfo, pos: torch.Tensor, seeds: torch.Tensor) -> None:
        s = self.binfo
        for dst, src in ((s.slot_ids, b.slot_ids), (s.page_indices, b.page_indices), (s.seq_lens, b.seq_lens), (s.cu_q_lens, b.cu_q_lens),
                         (s.num_seqs, b.num_seqs), (s.new_token_dests, b.new_token_dests)):
            dst.copy_(src, non_blocking=True)
        self.pos.copy_(pos)
        self.seeds.copy_(seeds)


def _caches(cache) -> List[KvPageCache]:
    if isinstance(cache, KvPageCache):
        return [cache]
    if isinstance(cache, (list, tuple)):
        return [c for x in cache for c in _caches(x)]
    return []


class InferenceEngine:
    def __init__(self, *, model, tokenizer, cache, decode_state: DecodeState, sampler: Sampler, config: InferenceEngineConfig, device=None):
        self.model = model
        self.tokenizer = tokenizer
        self.sampler = sampler
        self.gen_state = GenState(cache=cache, decode_state=decode_state)
        if config.max_prefill_size is None:
            config = dataclasses.replace(config, max_prefill_size=decode_state.page_table.max_len_per_seq)
        self.config = config
        if device is None:
            try:
                device = next(model.parameters()).device
            except (AttributeError, StopIteration, TypeError):
                device = torch.device("cpu")
        self.device = torch.device(device)
        self.free_slots: List[int] = [i for i, u in enumerate(decode_state.page_table.used_mask) if not u]
        self.local_map: Dict[int, Tuple[int, int]] = {}  # slot -> (request id, choice)
        self.request_queue: Deque[Request] = deque()
        self.results: Dict[int, Dict[int, DecodeResult]] = {}
        self._graph: Optional[_DecodeGraph] = None
        try:
            import inspect

            self._decode_takes_rows = "logit_rows" in inspect.signature(model.decode).parameters
        except (TypeError, ValueError):
            self._decode_takes_rows = False
        self.stats: Dict[str, float] = {"prefill_tokens": 0, "prefill_seconds": 0.0, "decode_tokens": 0, "decode_seconds": 0.0}

    # -- construction -------------------------------------------------------------------------------------------
    @classmethod
    def from_model(cls, model, tokenizer, *, max_pages: int, max_seqs: int, page_size: int, max_pages_per_seq: int, compute_dtype,
                   max_queued_tokens: int = 32, max_seqs_in_prefill: int = 16, max_prefill_size: Optional[int] = None) -> "InferenceEngine":
        cfg = InferenceEngineConfig(max_pages=max_pages, max_seqs=max_seqs, page_size=page_size, max_pages_per_seq=max_pages_per_seq,
                                    compute_dtype=compute_dtype, max_queued_tokens=max_queued_tokens,
                                    max_seqs_in_prefill=max_seqs_in_prefill, max_prefill_size=max_prefill_size)
        return cls.from_model_with_config(model=model, tokenizer=tokenizer, config=cfg)

    @classmethod
    def from_model_with_config(cls, model, tokenizer, config: InferenceEngineConfig) -> "InferenceEngine":
        table = PageTable.init(config.imputed_max_pages, config.max_seqs, config.page_size, config.max_pages_per_seq)
        try:
            device = next(model.parameters()).device
        except (AttributeError, StopIteration, TypeError):
            device = torch.device("cpu")
        try:
            cache = model.initial_cache(table, dtype=config.compute_dtype, device=device)
        except TypeError:
            cache = model.initial_cache(table, dtype=config.compute_dtype)
        ds = DecodeState.init(table, max_stop_seqs=config.max_stop_seqs, max_stop_tokens=config.max_stop_tokens,
                              max_queued_tokens=max(config.max_queued_tokens, config.max_seqs), enable_logprobs=config.enable_logprobs)
        return cls(model=model, tokenizer=tokenizer, cache=cache, decode_state=ds, sampler=Sampler(), config=config, device=device)

    def reset(self) -> None:
        """Drop every sequence and request.  The KV cache contents are left as they are: pages are rewritten before use."""
        cfg = self.config
        table = PageTable.init(cfg.imputed_max_pages, cfg.max_seqs, cfg.page_size, cfg.max_pages_per_seq)
        self.gen_state.decode_state = DecodeState.init(table, max_stop_seqs=cfg.max_stop_seqs, max_stop_tokens=cfg.max_stop_tokens,
                                                       max_queued_tokens=max(cfg.max_queued_tokens, cfg.max_seqs),
                                                       enable_logprobs=cfg.enable_logprobs)
        self.free_slots = list(range(cfg.max_seqs))
        self.local_map.clear()
        self.request_queue.clear()
        self.results = {}

    # -- invariants -----------------------------------------------------------------------------------------------
    def _verify_free_slot_view(self, *, context: str) -> None:
        used = self.gen_state.decode_state.page_table.used_mask
        free = set(self.free_slots)
        for s, u in enumerate(used):
            if u and s in free:
                raise RuntimeError(f"[free slot invariant] slot {s} marked used but present in free list during {context}")
            if not u and s not in free:
                raise RuntimeError(f"[free slot invariant] slot {s} free in page table but missing from free list during {context}")

    def _free_page_count(self) -> int:
        return self.gen_state.decode_state.page_table.num_free_pages

    def _pages_needed_for_prompt(self, prompt_len: int) -> int:
        ps = self.config.page_size
        return (prompt_len + 1 + ps - 1) // ps

    # -- model calls ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def _forward(self, tokens: torch.Tensor, binfo: PageBatchInfo, pos: torch.Tensor, logit_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if logit_rows is not None and self._decode_takes_rows:
            logits, cache = self.model.decode(tokens, self.gen_state.cache, binfo, pos, logit_rows=logit_rows)
        else:
            logits, cache = self.model.decode(tokens, self.gen_state.cache, binfo, pos)
            if logit_rows is not None:
                logits = logits.index_select(0, logit_rows)
        self.gen_state.cache = cache
        return logits

    # -- public API -----------------------------------------------------------------------------------------------
    def enqueue_requests(self, requests: Sequence[Request]) -> None:
        self.request_queue.extend(requests)

    def generate(self, requests: Sequence[Request]) -> GenerationResult:
        """Run the requests to completion; results are ordered by request, then by choice."""
        for r in requests:
            if r.n_generations > self.config.max_seqs:
                raise ValueError(f"request {r.request_id} wants {r.n_generations} generations but the engine has {self.config.max_seqs} slots")
            if len(r.prompt_tokens) + 1 > self.gen_state.decode_state.page_table.max_len_per_seq:
                raise ValueError(f"request {r.request_id}: prompt of {len(r.prompt_tokens)} tokens does not fit a sequence")
            if r.n_generations * self._pages_needed_for_prompt(len(r.prompt_tokens)) > self.config.imputed_max_pages:
                raise ValueError(f"request {r.request_id} can never be admitted: it needs more pages than the cache has")
        self.results = {r.request_id: {k: DecodeResult(r.request_id, k, []) for k in range(r.n_generations)} for r in requests}
        self.enqueue_requests(requests)
        t0 = time.time()
        total = 0
        stalled = 0
        while self.request_queue or self.local_map:
            t_a = self._now()
            before = sum(len(r.prompt_tokens) for r in self.request_queue)
            admitted = False
            while self._admit_from_queue():  # fill the batch before decoding: rounds over a half-empty batch cost the same
                admitted = True
            if admitted:
                self.stats["prefill_seconds"] += self._now() - t_a
                self.stats["prefill_tokens"] += before - sum(len(r.prompt_tokens) for r in self.request_queue)
            running = bool(self.local_map)
            if running:
                t_d = self._now()
                kept = self._decode_call()
                self.stats["decode_seconds"] += self._now() - t_d
                self.stats["decode_tokens"] += kept
                total += kept
            self._release_finished()
            if not admitted and not running:
                stalled += 1
                if stalled > 2:
                    raise RuntimeError("no request can be admitted and nothing is running: the page budget is too small")
            else:
                stalled = 0
        self._verify_free_slot_view(context="generate end")
        out_tokens, out_lps = [], []
        gen = 0
        for r in requests:
            for k in range(r.n_generations):
                dr = self.results[r.request_id][k]
                out_tokens.append(dr.token_list)
                out_lps.append(dr.logprobs)
                gen += len(dr.token_list)
        logger.debug(f"generated {gen} tokens in {time.time() - t0:.3f}s")
        want_lp = self.config.enable_logprobs or any(r.enable_logprobs for r in requests)
        return GenerationResult(out_tokens, out_lps if want_lp else None, gen)

    # -- admission and prefill ------------------------------------------------------------------------------------
    def _admit_from_queue(self) -> bool:
        """Admit as many queued requests as slots, pages and the prefill limits allow, and prefill them."""
        batch: List[Request] = []
        slots_left = len(self.free_slots)
        pages_left = self._free_page_count()
        toks = 0
        seqs = 0
        while self.request_queue:
            r = self.request_queue[0]
            need_pages = self._pages_needed_for_prompt(len(r.prompt_tokens)) + (r.n_generations - 1)
            if r.n_generations > slots_left or need_pages > pages_left:
                break
            if batch and (seqs + 1 > self.config.max_seqs_in_prefill or toks + len(r.prompt_tokens) > self.config.max_prefill_size):
                break
            batch.append(self.request_queue.popleft())
            slots_left -= r.n_generations
            pages_left -= need_pages
            toks += len(r.prompt_tokens)
            seqs += 1
        if not batch:
            return False
        self._prefill_prompts(batch)
        return True

    def _take_slot(self) -> int:
        ds = self.gen_state.decode_state
        slot = self.free_slots.pop(0)
        ds.page_table, got = ds.page_table.assign_seq_id_to_seq(slot)
        if got != slot:
            raise RuntimeError(f"slot {slot} was on the free list but the page table refused it")
        return slot

    def _prefill_prompts(self, batch: List[Request]) -> None:
        ds = self.gen_state.decode_state
        toks, slots, pos = [], [], []
        primary: List[Tuple[Request, int]] = []
        for r in batch:
            s = self._take_slot()
            prompt = list(r.prompt_tokens) or [0]
            params = dataclasses.replace(r.decode_params, max_num_tokens=int(min(int(r.decode_params.max_num_tokens),
                                                                                 ds.page_table.max_len_per_seq)))
            ds.assign_seq(s, np.asarray(prompt, np.int32), len(prompt), seq_params=params)
            self.local_map[s] = (r.request_id, 0)
            toks += prompt
            slots += [s] * len(prompt)
            pos += list(range(len(prompt)))
            primary.append((r, s))
        # every sequence of a prefill starts at position 0: attention runs densely over the packed tokens, one segment per
        # prompt; pad the packed length to the attention kernel's tile (padding: no slot, no page, segment -1)
        seg = [i for i, r in enumerate(batch) for _ in range(max(len(r.prompt_tokens), 1))]
        pad = (-len(toks)) % PREFILL_PAD
        slots_np = np.asarray(slots + [INVALID] * pad, np.int32)
        pos_alloc = np.asarray(pos + [INVALID] * pad, np.int32)
        ds.page_table, binfo = ds.page_table.allocate_for_seq(slots_np, pos_alloc)
        binfo = dataclasses.replace(binfo, prefill_segment_ids=torch.tensor(seg + [-1] * pad, dtype=torch.int32))
        dev = self.device
        # the last prompt token of each sequence predicts its first new token; clones sample the same row with their own key
        last_index, cursor = {}, 0
        for r, s in primary:
            cursor += max(len(r.prompt_tokens), 1)
            last_index[s] = cursor - 1
        # one logits row per generation: the primary and each of its clones read the row of the prompt's last token
        rows = [last_index[s] for r, s in primary for _ in range(r.n_generations)]
        logits = self._forward(torch.tensor(toks + [0] * pad, dtype=torch.int32, device=dev), binfo.to(dev),
                               torch.tensor(pos + [0] * pad, dtype=torch.int32, device=dev), torch.tensor(rows, dtype=torch.long, device=dev))
        # clones are made after the forward pass: they copy pages that the pass has just filled
        row_slots = []
        for r, s in primary:
            row_slots.append(s)
            for k in range(1, r.n_generations):
                c = self._take_slot()
                self._clone(s, c, r, k)
                row_slots.append(c)
        row_slots_np = np.asarray(row_slots, np.int32)
        sample_pos = ds.seq_lens[row_slots_np]
        tokens, lps = self._sample(logits, row_slots_np, sample_pos)
        ds.update_tokens(tokens, row_slots_np, lps, len(row_slots_np))
        self._ingest(tokens, row_slots_np, lps)

    def _clone(self, src: int, dst: int, r: Request, choice: int) -> None:
        """Slot ``dst`` becomes a copy of ``src`` (same prompt, own sampling key); full pages are shared, a partial last page
        is duplicated in every layer's cache."""
        ds = self.gen_state.decode_state
        before = ds.page_table.page_indices[src].copy()
        ds.page_table = ds.page_table.clone_pages_from(src, dst)
        after = ds.page_table.page_indices[dst]
        L = int(ds.page_table.seq_lens[src])
        if L % self.config.page_size != 0 and L > 0:
            last = (L - 1) // self.config.page_size
            if before[last] != after[last]:
                for c in _caches(self.gen_state.cache):
                    c.copy_page(int(before[last]), int(after[last]))
        params = dataclasses.replace(r.decode_params, key=int(r.decode_params.key) * 1000003 + choice,
                                     max_num_tokens=int(min(int(r.decode_params.max_num_tokens), ds.page_table.max_len_per_seq)))
        n = int(ds.seq_lens[src])
        ds.assign_seq(dst, ds.tokens[src, :n].copy(), n, seq_params=params)
        self.local_map[dst] = (r.request_id, choice)

    # -- sampling ---------------------------------------------------------------------------------------------------
    def _sample(self, logits: torch.Tensor, slots: np.ndarray, positions: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
        ds = self.gen_state.decode_state
        temps = torch.from_numpy(ds.temperature[slots].astype(np.float32)).to(logits.device)
        seeds = torch.from_numpy(ds.prng_keys_for(slots, positions)).to(logits.device)
        tok, lp = self.sampler(logits, temps, key=seeds)
        return tok.cpu().numpy().astype(np.int32), lp.float().cpu().numpy()

    # -- decode -----------------------------------------------------------------------------------------------------
    def _decode_call(self) -> int:
        """One device call of up to ``max_rounds`` rounds over every live sequence.  Returns the number of tokens kept."""
        t_plan = time.perf_counter()
        ds = self.gen_state.decode_state
        ds, packed = ds.pack_next_sequence(self.config.max_seqs)
        n = packed.num_tokens
        if n == 0:
            return 0
        slots = packed.slot_ids[:n].copy()
        first_tokens = packed.tokens[:n].copy()
        pos0 = packed.pos_ids[:n].copy()  # position of the queued token of each sequence
        max_len = ds.page_table.max_len_per_seq
        remaining = np.maximum(ds.max_num_tokens[slots] - ds.seq_lens[slots], 0)
        R = int(max(1, min(self.config.max_rounds, int(remaining.max()) if len(remaining) else 1)))
        T = self.config.max_seqs
        dev = self.device
        # plan all rounds on the host
        binfos: List[PageBatchInfo] = []
        pos_rounds = np.full((R, T), INVALID, np.int32)
        slot_pad = np.full(T, INVALID, np.int32)
        slot_pad[:n] = slots
        seeds = np.zeros((R, T), np.int64)
        pos_model = np.zeros((R, T), np.int32)  # positions as the model sees them (padding rows at 0)
        for r in range(R):
            # a sequence that reaches the end of its pages is finished by then; its later (discarded) rounds rewrite the last slot
            p = np.minimum(pos0 + r, max_len - 1)
            pos_rounds[r, :n] = p
            pos_model[r, :n] = p
            ds.page_table, binfo = ds.page_table.allocate_for_seq(slot_pad, pos_rounds[r])
            binfos.append(binfo)
            seeds[r, :n] = ds.prng_keys_for(slots, pos0 + r + 1)
        temps = np.zeros(T, np.float32)
        temps[:n] = ds.temperature[slots]
        tok_in = np.zeros(T, np.int32)
        tok_in[:n] = first_tokens
        # the device part: round r feeds the tokens sampled in round r - 1
        d_tok = torch.from_numpy(tok_in).to(dev)
        d_temps = torch.from_numpy(temps).to(dev)
        d_seeds = torch.from_numpy(seeds).to(dev)
        d_pos = torch.from_numpy(pos_model).to(dev)
        out_tok = torch.empty((R, T), dtype=torch.int32, device=dev)
        out_lp = torch.empty((R, T), dtype=torch.float32, device=dev)
        # the batch rows of a PageBatchInfo are in order of first appearance, and tokens are sorted by slot: row i = token i
        t_dev = time.perf_counter()
        self.stats["decode_rounds"] = self.stats.get("decode_rounds", 0) + R
        self.stats["decode_plan_seconds"] = self.stats.get("decode_plan_seconds", 0.0) + (t_dev - t_plan)
        graph = self._decode_graph(binfos[0]) if (self.config.use_cuda_graph and dev.type == "cuda") else None
        if graph is not None:
            # one captured round, replayed R times: only the small per-round tables are copied into its static inputs; the
            # sampled tokens are fed back to the token input inside the graph
            graph.tok.copy_(d_tok)
            graph.temps.copy_(d_temps)
            # the tables of all R rounds cross to the device in one copy per field; each round then refreshes the graph's static
            # inputs with device-to-device copies, so the host never waits for a round to finish before queueing the next
            fields = ("slot_ids", "page_indices", "seq_lens", "cu_q_lens", "num_seqs", "new_token_dests")
            staged = {f: torch.stack([getattr(b, f) for b in binfos]).to(dev, non_blocking=True) for f in fields}
            for r in range(R):
                graph.load_round(PageBatchInfo(*(staged[f][r] for f in fields), binfos[r].page_size), d_pos[r], d_seeds[r])
                graph.graph.replay()
                out_tok[r].copy_(graph.out_tok)
                out_lp[r].copy_(graph.out_lp)
        else:
            for r in range(R):
                b = binfos[r].to(dev)
                logits = self._forward(d_tok, b, d_pos[r])
                d_tok, lp = self.sampler(logits, d_temps, key=d_seeds[r])
                out_tok[r], out_lp[r] = d_tok, lp
        toks = out_tok.cpu().numpy()
        lps = out_lp.cpu().numpy()
        if dev.type == "cuda":
            from ..ops import lib as _lib

            _lib.check_status()  # e.g. a tensor-parallel all-reduce whose wait for a peer ran out: the tokens are not to be trusted
        t_post = time.perf_counter()
        self.stats["decode_device_seconds"] = self.stats.get("decode_device_seconds", 0.0) + (t_post - t_dev)
        # apply stop conditions round by round; a finished sequence's later tokens are dropped
        kept = 0
        alive = np.ones(n, dtype=bool)
        for r in range(R):
            idx = np.nonzero(alive)[0]
            if len(idx) == 0:
                break
            ds.update_tokens(toks[r, idx], slots[idx], lps[r, idx], len(idx), enqueue=(r == R - 1))
            self._ingest(toks[r, idx], slots[idx], lps[r, idx])
            kept += len(idx)
            alive[idx] = ~ds.finished[slots[idx]]
        self.stats["decode_post_seconds"] = self.stats.get("decode_post_seconds", 0.0) + (time.perf_counter() - t_post)
        return kept

    def _now(self) -> float:
        """Host time after the device has drained (phase timings for ``stats``)."""
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)
        return time.perf_counter()

    def _decode_graph(self, example: PageBatchInfo) -> Optional["_DecodeGraph"]:
        """The CUDA graph of one decode round (forward over ``max_seqs`` packed tokens, sampling, token feedback), captured
        on first use.  Returns None when the round's table shapes differ from the captured ones (the caller runs eagerly)."""
        g = self._graph
        if g is None:
            g = self._graph = _DecodeGraph(self, example)
        return g if g.matches(example) else None

    # -- outputs ----------------------------------------------------------------------------------------------------
    def _ingest(self, tokens: np.ndarray, slots: np.ndarray, lps: Optional[np.ndarray]) -> None:
        for i, (t, s) in enumerate(zip(tokens.tolist(), slots.tolist())):
            rid, choice = self.local_map[s]
            dr = self.results[rid][choice]
            dr.token_list.append(int(t))
            dr.tokens_decoded += 1
            if lps is not None:
                dr.logprobs.append(float(lps[i]))

    def _release_finished(self) -> None:
        ds = self.gen_state.decode_state
        fin = ds.finished.copy()
        if not fin.any():
            return
        slots = np.nonzero(fin)[0].tolist()
        logger.info(f"Releasing finished sequences: {slots}")
        for s in slots:
            rid, choice = self.local_map.pop(s)
            self.results[rid][choice].done = True
        ds.purge_queue_of_slot(np.asarray(slots, np.int32))
        ds.page_table = ds.page_table.free_pages_for_finished(fin)
        ds.invalidate_finished()
        ds.seq_lens[fin] = 0
        self.free_slots = sorted(set(self.free_slots) | set(slots))
