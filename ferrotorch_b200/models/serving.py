"""Continuous batching over the paged KV cache: many requests of different lengths share every forward pass.

The reference generates one sequence at a time (ferrotorch-llama/src/generation.rs:145-228 loops over a single
``LlamaKvCache``; its attention is ``batch = 1 only``, attention.rs:225-231) and its paged cache is a host
structure that no model reads (ferrotorch-nn/src/paged_attention.rs:447-532).  A server pays for a decode step by
the bytes of the weights it streams, not by the rows it multiplies, so this module keeps a set of running
sequences and gives every step one flat token batch:

* each running sequence contributes the tokens whose keys and values are not in the cache yet: one token when
  it is decoding, a chunk of its prompt (``prefill_chunk``) when it has just been admitted or was preempted;
* the projections, the MLP and the norms run once over the flat batch; attention reads the pages: decoding
  rows through :meth:`PagedKVCache.decode` (the paged-decode kernel on a device, row b reading the block table
  of the sequence that owns it), prompt chunks through flash attention over the sequence's gathered pages;
* pages are reserved as sequences grow; when the pool runs dry the most recently admitted sequence is preempted
  (its pages are freed, it re-enters the queue at the front and recomputes its prompt plus what it has generated),
  so the earliest requests always finish and the pool can be smaller than the sum of all contexts;
* waiting requests are admitted first come first served while there are sequence slots, step-token budget and
  pages above a watermark;
* a greedy request with ``lookahead`` decodes speculatively without a draft model: the continuation of the most
  recent earlier occurrence of its last few tokens (in its own prompt and output) is fed along with the last
  token, one forward pass scores all of them, and the longest run that equals the model's own choices is kept
  plus the token after it.  The output is the plain greedy output; repetitive text needs fewer steps.  Keys and
  values of rejected positions are simply overwritten later;
* with ``prefix_caching`` whole pages of finished (or still running) prompts stay in a table keyed by a hash chain
  of their tokens; a new request whose prompt starts with the same tokens adopts those pages (reference-counted
  in the pool) and computes only the rest.  Unused entries are evicted, deepest page of the least recently used
  chain first, before any sequence is preempted.

Greedy requests are sampled on the device in one ``argmax``; sampled requests carry their own generator, so
the tokens of a request do not depend on which other requests share its steps.
"""
from __future__ import annotations

import collections
import enum
import hashlib
import queue
import struct
import threading
import time
from dataclasses import dataclass, field
from typing import Callable

import torch

from ..nn.paged import OutOfPages, PagedAttentionManager, PagedKVCache
from ..ops.attention import flash_attention
from .generation import apply_repetition_penalty, filter_top_k_top_p


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class SamplingParams:
    """``temperature == 0`` is greedy; otherwise softmax sampling after top-k / top-p filtering with the
    request's own generator (``seed``)."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int | None = None
    repetition_penalty: float = 1.0

    def validate(self) -> None:
        if self.temperature < 0.0 or not 0.0 < self.top_p <= 1.0 or self.top_k < 0 or self.repetition_penalty <= 0.0:
            raise ValueError("SamplingParams: temperature >= 0, 0 < top_p <= 1, top_k >= 0, repetition_penalty > 0")


@dataclass
class Request:
    prompt: list
    max_new_tokens: int
    stop_ids: tuple = ()
    sampling: SamplingParams = field(default_factory=SamplingParams)
    on_token: Callable[[int], object] | None = None       # called with every new token; returning False stops the request
    logits_processor: Callable | None = None              # (generated ids [1, n], logits [1, V]) -> logits, before sampling
    lookahead: int = 0                                    # greedy requests: verify up to this many looked-up tokens per step
    ngram: int = 3                                        # longest suffix that the look-up matches
    # ---- filled in by the batcher
    id: int = -1
    output: list = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    finish_reason: str | None = None                      # "stop" | "length" | "cancelled"
    slot: int = -1
    computed: int = 0                                     # tokens of prompt + output whose keys / values are cached
    preemptions: int = 0
    submit_step: int = -1
    first_token_step: int = -1
    finish_step: int = -1
    submit_time: float = 0.0
    first_token_time: float = 0.0
    finish_time: float = 0.0

    def __post_init__(self):
        self.prompt = [int(t) for t in self.prompt]
        self._done = threading.Event()
        self._generator: torch.Generator | None = None
        self._admitted_at = -1

    def tokens(self) -> list:
        return self.prompt + self.output

    def is_finished(self) -> bool:
        return self.state is RequestState.FINISHED

    def result(self, timeout: float | None = None) -> list:
        """Block until the request has finished (for callers on another thread than the serving loop)."""
        if not self._done.wait(timeout):
            raise TimeoutError("request %d still running" % self.id)
        return self.output


@dataclass
class ServingStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    peak_running: int = 0
    peak_pages: int = 0
    prefix_hit_tokens: int = 0                            # prompt tokens that were adopted from the prefix table
    spec_proposed: int = 0                                # looked-up tokens that were verified
    spec_accepted: int = 0                                # ... and were what the model would have produced
    batch_tokens: list = field(default_factory=list)      # tokens of every step's flat batch

    def mean_batch_tokens(self) -> float:
        return sum(self.batch_tokens) / len(self.batch_tokens) if self.batch_tokens else 0.0


class PrefixCache:
    """Full pages of token prefixes, shared between sequences.  The key of page i of a sequence is a digest of
    the key of page i - 1 and of the page's tokens, so equal keys mean equal prefixes; the table holds one
    reference on every page it lists."""

    def __init__(self, pool, block_size: int):
        self.pool, self.block_size = pool, block_size
        self._table: collections.OrderedDict = collections.OrderedDict()      # digest -> page, least recently used first
        self.hits = self.misses = self.evictions = 0

    def __len__(self) -> int:
        return len(self._table)

    def keys_for(self, tokens: list) -> list:
        keys, prev, bs = [], b"", self.block_size
        for i in range(len(tokens) // bs):
            prev = hashlib.blake2b(prev + struct.pack("<%dq" % bs, *tokens[i * bs:(i + 1) * bs]), digest_size=16).digest()
            keys.append(prev)
        return keys

    def match(self, tokens: list) -> list:
        """Pages of the longest listed prefix of ``tokens`` (whole pages only)."""
        keys, pages = self.keys_for(tokens), []
        for k in keys:
            page = self._table.get(k)
            if page is None:
                break
            pages.append(page)
        for k in reversed(keys[:len(pages)]):             # the root of a chain is its most recently used entry
            self._table.move_to_end(k)
        self.hits += len(pages)
        self.misses += len(keys) - len(pages)
        return pages

    def insert(self, tokens: list, pages: list) -> int:
        """List the whole pages of ``tokens`` (``pages[i]`` holds tokens ``i * block_size ..``); returns how many were new."""
        keys, new = self.keys_for(tokens)[:len(pages)], 0
        for k, page in reversed(list(zip(keys, pages))):
            if k not in self._table:
                self._table[k] = self.pool.retain(page)
                new += 1
            self._table.move_to_end(k)
        return new

    def evictable(self) -> int:
        return sum(1 for page in self._table.values() if self.pool.ref_count(page) == 1)

    def evict(self, n_pages: int) -> int:
        """Drop up to ``n_pages`` entries that no sequence holds, least recently used first; returns how many."""
        done = 0
        for k in list(self._table):
            if done >= n_pages:
                break
            page = self._table[k]
            if self.pool.ref_count(page) == 1:
                del self._table[k]
                self.pool.free(page)
                done += 1
        self.evictions += done
        return done

    def clear(self) -> None:
        for page in self._table.values():
            self.pool.free(page)
        self._table.clear()


class ContinuousBatcher:
    """Serve requests on ``model`` (a :class:`~ferrotorch_b200.models.llama.LlamaForCausalLM`) with a paged cache
    of ``num_blocks`` pages of ``block_size`` tokens.

    ``max_running``: sequence slots; ``max_tokens_per_step``: size limit of a step's flat batch;
    ``prefill_chunk``: most prompt tokens one sequence contributes to one step (long prompts are spread over
    steps, so running sequences keep decoding meanwhile); ``watermark``: fraction of the pool that admission
    leaves free for the growth of the sequences that are already running."""

    def __init__(self, model, num_blocks: int, block_size: int = 16, max_running: int = 64, max_seq_len: int | None = None,
                 max_tokens_per_step: int = 2048, prefill_chunk: int = 512, watermark: float = 0.01,
                 prefix_caching: bool = False):
        cfg = model.config
        p = next(model.parameters())
        self.model = model
        self.max_seq_len = max_seq_len or cfg.max_position_embeddings
        self.cache = PagedKVCache(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, num_blocks, max_running,
                                  self.max_seq_len, block_size, device=p.device, dtype=p.dtype)
        self.manager = PagedAttentionManager(self.cache)
        self.max_running, self.max_tokens_per_step, self.prefill_chunk = max_running, max_tokens_per_step, prefill_chunk
        if max_tokens_per_step < 1 or prefill_chunk < 1:
            raise ValueError("ContinuousBatcher: max_tokens_per_step and prefill_chunk must be at least 1")
        self.watermark_pages = max(1, int(watermark * num_blocks)) if watermark > 0 else 0
        self.prefix = PrefixCache(self.cache.pool, block_size) if prefix_caching else None
        self._drafts: dict = {}
        self.waiting: collections.deque = collections.deque()
        self.running: list = []                           # in admission order
        self.stats = ServingStats()
        self._next_id = 0
        self._inbox: queue.Queue = queue.Queue()

    # ------------------------------------------------------------------ requests
    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.cache.block_size - 1) // self.cache.block_size

    def submit(self, request: Request | list, max_new_tokens: int | None = None, **kw) -> Request:
        """Queue a request (a :class:`Request`, or a prompt with ``max_new_tokens`` and ``Request`` fields).
        May be called from any thread; the request joins the queue at the next :meth:`step`."""
        if not isinstance(request, Request):
            request = Request(list(request), int(max_new_tokens), **kw)
        request.sampling.validate()
        total = len(request.prompt) + request.max_new_tokens
        if not request.prompt or request.max_new_tokens < 1:
            raise ValueError("submit: a request needs a prompt and max_new_tokens >= 1")
        if total > self.max_seq_len:
            raise ValueError("submit: prompt + max_new_tokens = %d exceeds max_seq_len %d" % (total, self.max_seq_len))
        if self._pages_for(total) > self.cache.num_blocks:
            raise OutOfPages("submit: the request needs %d pages, the pool has %d" % (self._pages_for(total), self.cache.num_blocks))
        request.submit_time = time.perf_counter()
        self._inbox.put(request)
        return request

    def cancel(self, request: Request) -> None:
        """Finish a request at the next step boundary with reason ``cancelled``."""
        request.finish_reason = "cancelled"

    def _drain_inbox(self) -> None:
        while True:
            try:
                r = self._inbox.get_nowait()
            except queue.Empty:
                return
            r.id, self._next_id = self._next_id, self._next_id + 1
            r.submit_step = self.stats.steps
            if r.sampling.temperature > 0.0:
                r._generator = torch.Generator()
                r._generator.manual_seed(r.sampling.seed if r.sampling.seed is not None else r.id)
            self.waiting.append(r)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or not self._inbox.empty())

    # ------------------------------------------------------------------ scheduling
    def _remember(self, r: Request) -> None:
        if self.prefix is not None and r.slot >= 0 and r.computed >= self.cache.block_size:
            self.prefix.insert(r.tokens()[:r.computed], self.cache.pages_of(r.slot))      # a slice: never past the tokens kept

    def _finish(self, r: Request, reason: str) -> None:
        if r.slot >= 0:
            self._remember(r)
            self.manager.remove_sequence(r.slot)
            r.slot = -1
        if r in self.running:
            self.running.remove(r)
        r.state, r.finish_reason = RequestState.FINISHED, reason
        r.finish_step, r.finish_time = self.stats.steps, time.perf_counter()
        self.stats.finished += 1
        r._done.set()

    def _preempt(self, r: Request) -> None:
        self._remember(r)
        self.manager.remove_sequence(r.slot)
        self.running.remove(r)
        r.slot, r.computed, r.state = -1, 0, RequestState.WAITING
        r.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(r)

    def _reserve(self, r: Request, new_len: int, protected: set) -> bool:
        """Pages for ``new_len`` tokens of ``r``; preempts later-admitted sequences while the pool is dry.
        False if ``r`` itself had to give way."""
        while True:
            try:
                self.cache.reserve(r.slot, new_len)
                self.manager.active[r.slot] = max(self.manager.active[r.slot], new_len)
                return True
            except OutOfPages:
                if self.prefix is not None and self.prefix.evict(1):
                    continue
                victims = [v for v in self.running if v is not r and v.id not in protected]
                if victims:
                    self._preempt(victims[-1])
                    continue
                if any(v is not r for v in self.running):  # everything else is already in this step's batch
                    self._preempt(r)
                    return False
                raise

    @staticmethod
    def _look_up(tokens: list, ngram: int, k: int) -> list:
        """Up to ``k`` tokens that followed the most recent earlier occurrence of the last ``ngram`` (or fewer) tokens."""
        L = len(tokens)
        for g in range(min(ngram, L - 1), 0, -1):
            tail = tokens[L - g:]
            for i in range(L - g - 1, -1, -1):
                if tokens[i:i + g] == tail:
                    return tokens[i + g:i + g + k]
        return []

    def _schedule(self) -> list:
        """This step's runs: ``(request, first position, number of tokens)``; ``self._drafts`` holds the looked-up
        tokens of the runs that speculate."""
        budget = self.max_tokens_per_step
        runs, scheduled, preempted = [], set(), False
        self._drafts = {}
        before = self.stats.preemptions
        for r in list(self.running):                      # admission order: the oldest sequences are served first
            if r not in self.running or budget == 0:
                continue
            n = min(len(r.prompt) + len(r.output) - r.computed, self.prefill_chunk, budget)
            draft = []
            if (r.lookahead > 0 and r.output and r.computed == len(r.prompt) + len(r.output) - 1 and r.sampling.temperature == 0.0
                    and r.sampling.repetition_penalty == 1.0 and r.logits_processor is None):
                k = min(r.lookahead, r.max_new_tokens - len(r.output) - 1, budget - 1, self.prefill_chunk - 1)
                draft = self._look_up(r.tokens(), r.ngram, k) if k > 0 else []
                n += len(draft)
            if self._reserve(r, r.computed + n, scheduled):
                if draft:
                    self._drafts[r.id] = draft
                runs.append((r, r.computed, n))
                scheduled.add(r.id)
                budget -= n
        preempted = self.stats.preemptions > before
        runs = [run for run in runs if run[0].state is RequestState.RUNNING and run[0].slot >= 0]
        while self.waiting and not preempted and budget > 0 and len(self.running) < self.max_running:
            r = self.waiting[0]
            seq = r.tokens()
            shared = self.prefix.match(seq[:-1]) if self.prefix is not None else []      # at least one token is computed
            start = len(shared) * self.cache.block_size
            n = min(len(seq) - start, self.prefill_chunk, budget)
            need = self._pages_for(start + n) - len(shared) + (self.watermark_pages if self.running else 0)
            if need > self.manager.free_pages and self.prefix is not None:
                for page in shared:                           # pages this request is about to adopt must survive the eviction
                    self.cache.pool.retain(page)
                self.prefix.evict(need - self.manager.free_pages)
                for page in shared:
                    self.cache.pool.free(page)
            if need > self.manager.free_pages:
                break
            self.waiting.popleft()
            r.slot = self.manager.add_sequence(0)
            if shared:
                self.cache.adopt(r.slot, shared, start)
                self.stats.prefix_hit_tokens += start
            self.cache.reserve(r.slot, start + n)
            self.manager.active[r.slot] = start + n
            r.computed = start
            r.state, r._admitted_at = RequestState.RUNNING, self.stats.steps
            self.running.append(r)
            runs.append((r, start, n))
            budget -= n
        return runs

    # ------------------------------------------------------------------ one forward over the flat batch
    def _attention(self, attn, layer: int, h: torch.Tensor, pos: torch.Tensor, sid: torch.Tensor, spans: list) -> torch.Tensor:
        T = h.shape[1]
        Hq, Hkv, D = attn.n_heads, attn.n_kv_heads, attn.head_dim
        qkv = attn.qkv_proj(h).view(1, T, Hq + 2 * Hkv, D)
        if attn.rope is not None:
            qkv = attn.rope(qkv, positions=pos, n_rot_heads=Hq + Hkv)
        q, k, v = qkv[0, :, :Hq], qkv[0, :, Hq:Hq + Hkv], qkv[0, :, Hq + Hkv:]
        self.cache.append(layer, k, v, pos, sid)
        out = torch.empty((T, Hq, D), device=h.device, dtype=h.dtype)
        single = [row for (_, row, _, n) in spans if n == 1]
        if single:
            idx = torch.tensor(single, device=h.device, dtype=torch.long)
            qd = q.index_select(0, idx).contiguous()
            out[idx] = self.cache.decode(layer, qd, (pos.index_select(0, idx) + 1).to(torch.int32), seq_ids=sid.index_select(0, idx))
        for slot, row, start, n in spans:
            if n > 1:
                kk, vv = self.cache.gather(layer, slot, start + n)
                out[row:row + n] = flash_attention(q[None, row:row + n].contiguous(), kk[None], vv[None], causal=True)[0]
        return attn.o_proj(out.reshape(1, T, Hq * D))

    @torch.no_grad()
    def _forward(self, runs: list) -> torch.Tensor:
        """Logits of the last token of every run (of its last ``1 + len(draft)`` tokens when it speculates), run after run."""
        dev = self.cache.device
        toks, poss, sids, spans, last, row = [], [], [], [], [], 0
        for r, start, n in runs:
            draft = self._drafts.get(r.id, [])
            seq = r.tokens() + draft
            toks += seq[start:start + n]
            poss += range(start, start + n)
            sids += [r.slot] * n
            spans.append((r.slot, row, start, n))
            row += n
            last += range(row - 1 - len(draft), row)
        tok = torch.tensor(toks, dtype=torch.long, device=dev)
        pos = torch.tensor(poss, dtype=torch.int32, device=dev)
        sid = torch.tensor(sids, dtype=torch.int32, device=dev)
        m = self.model.model
        x, delta = m.embed_tokens(tok[None]), None
        for li, layer in enumerate(m.layers):
            if delta is None:
                h = layer.input_layernorm(x)
            else:
                h, x = layer.input_layernorm(x, delta)
            a = self._attention(layer.self_attn, li, h, pos, sid, spans)
            h, x = layer.post_attention_layernorm(x, a)
            delta = layer.mlp(h)
        h, _ = m.norm(x, delta)
        return self.model.lm_head(h[0, torch.tensor(last, device=dev)])

    def _sample(self, requests: list, logits: torch.Tensor) -> list:
        greedy = [i for i, r in enumerate(requests)
                  if r.sampling.temperature == 0.0 and r.sampling.repetition_penalty == 1.0 and r.logits_processor is None]
        out = [0] * len(requests)
        if greedy:
            for i, t in zip(greedy, logits[greedy].float().argmax(-1).tolist()):
                out[i] = t
        for i, r in enumerate(requests):
            if i in greedy:
                continue
            s = r.sampling
            z = logits[i].float().cpu()[None]
            if r.logits_processor is not None:            # e.g. a grammar mask (models.generation.GrammarLogitsProcessor)
                z = r.logits_processor(torch.tensor([r.output], dtype=torch.long), z)
            z = apply_repetition_penalty(z, torch.tensor([r.tokens()], dtype=torch.long), s.repetition_penalty)
            if s.temperature == 0.0:
                out[i] = int(z.argmax(-1))
                continue
            z = filter_top_k_top_p(z / s.temperature, s.top_k, s.top_p)
            out[i] = int(torch.multinomial(z.softmax(-1), 1, generator=r._generator))
        return out

    # ------------------------------------------------------------------ the loop
    def step(self) -> list:
        """Schedule, run one forward pass, sample; returns ``(request, token)`` for every token produced."""
        self._drain_inbox()
        for r in [r for r in list(self.running) + list(self.waiting) if r.finish_reason == "cancelled"]:
            if r in self.waiting:
                self.waiting.remove(r)
            self._finish(r, "cancelled")
        runs = self._schedule()
        if not runs:
            if self.waiting and not self.running:
                raise OutOfPages("the pool cannot hold the first chunk of request %d" % self.waiting[0].id)
            return []
        logits = self._forward(runs)
        self.stats.steps += 1
        self.stats.batch_tokens.append(sum(n for _, _, n in runs))
        self.stats.peak_running = max(self.stats.peak_running, len(self.running))
        self.stats.peak_pages = max(self.stats.peak_pages, self.cache.pool.num_used)
        emit, rows, spec, at = [], [], [], 0
        for r, start, n in runs:
            draft = self._drafts.get(r.id)
            r.computed = start + n
            if draft or (n == 1 and r.output):
                self.stats.decode_tokens += n
            else:
                self.stats.prefill_tokens += n
            if draft:
                spec.append((r, start, draft, at))
            elif r.computed == len(r.prompt) + len(r.output):
                if n > 1:
                    self._remember(r)                         # a prompt that has just been computed can be shared at once
                emit.append(r)
                rows.append(at)
            at += 1 + len(draft or ())
        new_tokens = []
        if emit:
            new_tokens += [(r, [t]) for r, t in zip(emit, self._sample(emit, logits[rows]))]
        for r, start, draft, at in spec:
            choice = logits[at:at + len(draft) + 1].float().argmax(-1).tolist()
            kept = 0
            while kept < len(draft) and choice[kept] == draft[kept]:
                kept += 1
            self.stats.spec_proposed += len(draft)
            self.stats.spec_accepted += kept
            r.computed = start + 1 + kept                     # the last token and the drafts that were right
            new_tokens.append((r, choice[:kept + 1]))
        produced = []
        now = time.perf_counter()
        for r, toks in new_tokens:
            for t in toks:
                r.output.append(t)
                if r.first_token_step < 0:
                    r.first_token_step, r.first_token_time = self.stats.steps, now
                produced.append((r, t))
                stop = r.on_token is not None and r.on_token(t) is False
                if t in r.stop_ids or stop:
                    self._finish(r, "stop")
                    break
                if len(r.output) >= r.max_new_tokens:
                    self._finish(r, "length")
                    break
        return produced

    def run(self, max_steps: int | None = None) -> ServingStats:
        """Step until nothing is queued or running."""
        n = 0
        while self.has_work() and (max_steps is None or n < max_steps):
            self.step()
            n += 1
        return self.stats

    def serve_forever(self, stop: threading.Event, idle_sleep: float = 0.001) -> None:
        """The serving loop for a dedicated thread: steps while there is work, sleeps while idle, returns when
        ``stop`` is set and the work has drained."""
        while not (stop.is_set() and not self.has_work()):
            if self.has_work():
                self.step()
            else:
                time.sleep(idle_sleep)

    def generate(self, prompts: list, max_new_tokens: int, stop_ids: tuple = (), sampling: SamplingParams | None = None) -> list:
        """All prompts to completion; returns the generated tokens of each, in the order given."""
        reqs = [self.submit(Request(list(p), max_new_tokens, tuple(stop_ids),
                                    SamplingParams(**vars(sampling)) if sampling is not None else SamplingParams()))
                for p in prompts]
        self.run()
        return [r.output for r in reqs]
