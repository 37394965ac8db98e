"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier, and as
many batches one after another as there are requests.

One request is abacus's chat loop (src/main.c:171-182): prefill, then sample,
stop on a stop token (it is neither kept nor fed back), else keep the token and
run it. The decisions of the loop (who is in which batch, who goes on, who is
finished and why) are plain Python on the host, apart from the engine, so they
are tested without a GPU.

Where the engine can run a decode step from tokens that are still on the device (`step_ahead`), the loop
does not let the GPU wait for the host: as soon as a step's tokens are drawn it launches the next step for
the same sequences with them, and only then reads them (over a second stream, so that the read does not
queue behind that step). If the tokens stop nobody, the step it launched is the next step; if they stop
somebody, that sequence's row of it is dropped (its slot is given back anyway). A step is launched ahead
only when no sequence ends for a reason the host knows before it sees the token (its length, its context).
"""
import time
from dataclasses import dataclass, field

import torch

from ..cache.kv import TOKENS_PER_PAGE


@dataclass
class Request:
    index: int
    prompt: list
    max_new_tokens: int
    output: list = field(default_factory=list)
    finish_reason: str = ""  # "stop", "length" or "context"
    slot: int = -1


def pages(n):
    return -(-n // TOKENS_PER_PAGE)


def plan_batches(requests, max_tokens, max_slots, max_context, batch_size=None):
    """Cut the requests, in order, into batches that fit the cache.

    A request may grow to min(prompt + max_new_tokens, max_context) tokens; a batch holds requests
    while their pages fit max_tokens and their number fits max_slots (and batch_size, if given).
    """
    limit = min(max_slots, batch_size or max_slots)
    batches, current, used = [], [], 0
    for r in requests:
        if not r.prompt:
            raise ValueError(f"request {r.index} has an empty prompt")
        if len(r.prompt) > max_context:
            raise ValueError(f"request {r.index}: prompt of {len(r.prompt)} tokens is longer than the context "
                             f"of {max_context}")
        need = pages(min(len(r.prompt) + r.max_new_tokens, max_context))
        if need > pages(max_tokens):
            raise ValueError(f"request {r.index} needs {need * TOKENS_PER_PAGE} tokens of cache; "
                             f"the cache has {max_tokens}")
        if current and (len(current) >= limit or used + need > pages(max_tokens)):
            batches.append(current)
            current, used = [], 0
        current.append(r)
        used += need
    if current:
        batches.append(current)
    return batches


class LiveBatch:
    """The requests of one batch that are still running, and what happens to each sampled token."""

    def __init__(self, requests, stop_tokens, max_context):
        self.live = list(requests)
        self.stop_tokens = frozenset(stop_tokens)
        self.max_context = max_context

    def first_step(self):
        """The prefill: every prompt whole, logits wanted at its last token."""
        return [(r.slot, r.prompt, [len(r.prompt) - 1]) for r in self.live]

    def take(self, sampled):
        """sampled[i] is the token drawn for self.live[i]. Returns (finished requests, next step's
        entries): a request ends on a stop token (not kept), after max_new_tokens, or when its
        context is full (src/main.c:174-176)."""
        finished, entries, still = [], [], []
        for r, token in zip(self.live, sampled):
            token = int(token)
            if r.max_new_tokens <= 0:
                r.finish_reason = "length"
            elif token in self.stop_tokens:
                r.finish_reason = "stop"
            else:
                r.output.append(token)
                if len(r.output) >= r.max_new_tokens:
                    r.finish_reason = "length"
                elif len(r.prompt) + len(r.output) >= self.max_context:
                    r.finish_reason = "context"
            if r.finish_reason:
                finished.append(r)
            else:
                still.append(r)
                entries.append((r.slot, [token], [0]))
        self.live = still
        return finished, entries


class Generator:
    """Runs requests through an engine. `engine` needs open(), close(slot), step(entries) -> logits,
    max_context and a cache with n_pages and max_slots; `sampler` needs states() and sample()."""

    def __init__(self, engine, sampler, stop_tokens=(), on_token=None):
        """on_token(request, token): called for every token a request keeps, as soon as the host has it (the chat
        loop prints each piece as it comes, src/main.c:177-180)."""
        self.engine, self.sampler, self.stop_tokens, self.on_token = engine, sampler, tuple(stop_tokens), on_token
        self.stats = {"prefill_steps": 0, "decode_steps": 0, "batches": 0}
        self.rng = None

    def generate(self, prompts, max_new_tokens, batch_size=None):
        """prompts: list of token-id lists. Returns the Request objects, outputs filled, in order."""
        requests = [Request(i, [int(t) for t in p], max_new_tokens) for i, p in enumerate(prompts)]
        cache = self.engine.cache
        for batch in plan_batches(requests, cache.n_pages * TOKENS_PER_PAGE, cache.max_slots,
                                  self.engine.max_context, batch_size):
            self.run_batch(batch)
            self.stats["batches"] += 1
        return requests

    @staticmethod
    def _may_run_ahead(rows, engine, max_context):
        """Whether the next step may be launched before this step's tokens are seen: the engine can, and no
        sequence ends with this token for a reason that does not depend on the token."""
        if not hasattr(engine, "step_ahead"):
            return False
        return all(r.max_new_tokens > 0 and len(r.output) + 1 < r.max_new_tokens
                   and len(r.prompt) + len(r.output) + 1 < max_context for r in rows)

    def _read_beside(self, drawn):
        """Start copying `drawn` (int32 on the device) to the host on a stream of its own, ordered after what the
        current stream holds now but not after what is launched on it later. Returns a function that waits for
        the copy and gives the list."""
        if drawn.device.type != "cuda":
            return drawn.tolist
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(drawn.device)
            self._landing = torch.empty(4096, dtype=torch.int32).pin_memory()
        n = drawn.numel()
        if n > self._landing.numel():
            return drawn.tolist
        self._copy_stream.wait_stream(torch.cuda.current_stream(drawn.device))
        with torch.cuda.stream(self._copy_stream):
            self._landing[:n].copy_(drawn, non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        drawn.record_stream(self._copy_stream)

        def read():
            done.synchronize()
            return self._landing[:n].tolist()
        return read

    def run_batch(self, batch):
        engine = self.engine
        for r in batch:
            r.slot = engine.open()
        live = LiveBatch(batch, self.stop_tokens, engine.max_context)
        # one random stream per request, kept at the request's slot
        if self.rng is None:
            self.rng = torch.zeros(engine.cache.max_slots, dtype=torch.int64, device=self.sampler.device)
        slots = torch.tensor([r.slot for r in batch], dtype=torch.int64, device=self.sampler.device)
        self.rng.index_copy_(0, slots, self.sampler.states([r.index for r in batch]))
        try:
            entries = live.first_step()
            self.stats["prefill_steps"] += 1
            logits = engine.step(entries)
            index = engine.last_batch.seq_slot  # row -> slot, on the device: which random stream a row draws from
            while True:
                rows = list(live.live)
                drawn = self.sampler.sample(logits, self.rng, index=index)
                ahead = None
                if self._may_run_ahead(rows, engine, live.max_context):
                    read = self._read_beside(drawn)
                    ahead = engine.step_ahead([r.slot for r in rows], drawn)
                    sampled = read() if ahead is not None else drawn.tolist()
                else:
                    sampled = drawn.tolist()
                now = time.perf_counter()  # the tokens are on the host
                self.stats.setdefault("t_first_token", now)
                self.stats["t_end"] = now
                kept = [len(r.output) for r in rows]
                finished, entries = live.take(sampled)
                if self.on_token is not None:
                    for r, n in zip(rows, kept):
                        for token in r.output[n:]:
                            self.on_token(r, token)
                for r in finished:
                    engine.close(r.slot)
                    r.slot = -1
                if not entries:
                    break
                self.stats["decode_steps"] += 1
                if ahead is None:
                    logits = engine.step(entries)
                    index = engine.last_batch.seq_slot
                elif not finished:
                    logits, index = ahead, engine.last_batch.seq_slot
                else:  # the step that ran ahead carries rows of sequences that have ended: the others' are the next step's
                    keep = [i for i, r in enumerate(rows) if r.slot >= 0]
                    logits = ahead[torch.tensor(keep, device=ahead.device)]
                    index = torch.tensor([rows[i].slot for i in keep], dtype=torch.int32, device=ahead.device)
        finally:
            for r in batch:
                if r.slot >= 0:
                    engine.close(r.slot)
                    r.slot = -1
        if hasattr(engine, "check_status"):
            engine.check_status()
