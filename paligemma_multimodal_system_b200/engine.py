"""Ragged-step engine for the token-sequence decoders: one step runs, as ONE batch, the next tokens of every request
that has some -- whole prompts, portions of prompts and single decoded tokens side by side.

  SequenceEngine.step(entries, end)   the step function: entries = [(request id, new token ids, wanted positions)];
                                      admits unknown ids, finds pages, runs the model's step over the shared page pool and
                                      state slots, returns the wanted logits; `end` releases requests afterwards
  SequenceEngine.generate(prompts)    continuous batching on top of it: serving.StepScheduler plans the steps, the
                                      framework's samplers (pg_argmax / pg_sample_top_p) pick the tokens

The model supplies `cache_layout()`, `step(batch, store, want_rows)`, `prec` and `vocab_size` (modeling_mapedra.py).
"""
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .cache import SequenceStore
from .seq_ops import make_step_batch
from .serving import StepScheduler, TokenRequest


class SequenceEngine:
    def __init__(self, model, max_tokens: int, num_slots: int = 4):
        _lib.require_device()
        self.model = model
        self.store = SequenceStore(model.cache_layout(), max_tokens, num_slots, model.prec.dtype)
        self._step_no = torch.zeros(1, device="cuda", dtype=torch.int32)

    @torch.no_grad()
    def step(self, entries: Sequence[Tuple[object, Sequence[int], Sequence[int]]], end: Sequence[object] = (), trace=None):
        """Runs the new tokens of every entry; returns fp32 logits [sum(len(want)), vocab] in entry / want order (None when
        nothing is wanted).  A request id seen for the first time is admitted; ids in `end` are released after the step."""
        store, V = self.store, self.model.vocab_size
        batch, want, row = [], [], 0
        seen = set()
        for rid, toks, w in entries:
            if rid in seen:
                raise ValueError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            toks = [int(t) for t in toks]
            if not toks:
                raise ValueError(f"request {rid!r}: empty entry")
            if min(toks) < 0 or max(toks) >= V:
                raise IndexError(f"request {rid!r}: token id out of range")
            if rid not in store.live:
                store.admit(rid)
            rec = store.reserve(rid, len(toks))
            batch.append(dict(tokens=toks, ctx=rec.length, slot=rec.slot, pages=rec.pages))
            for k in w:
                if not 0 <= int(k) < len(toks):
                    raise IndexError(f"request {rid!r}: wanted position {k} outside its {len(toks)} tokens")
                want.append(row + int(k))
            row += len(toks)
        logits = None
        if batch:
            b = make_step_batch(batch)
            rows = torch.tensor(want, dtype=torch.int64).to("cuda", non_blocking=True) if want else None
            logits = self.model.step(b, store, rows, trace=trace)
            for (rid, toks, _w) in entries:
                store.commit(rid, len(toks))
        for rid in end:
            if rid in store.live:
                store.release(rid)
        return logits

    def release(self, rid):
        self.store.release(rid)

    # -- generation ------------------------------------------------------------------------------------------------
    def _sample(self, logits, do_sample, temperature, top_p, seed):
        n, V = logits.shape
        out = torch.empty(n, device="cuda", dtype=torch.int32)
        L = _lib.lib()
        if do_sample:
            _lib.check(L.pg_sample_top_p(logits.data_ptr(), logits.stride(0), out.data_ptr(), 0, n, V, 1.0 / float(temperature), float(top_p),
                                         int(seed), self._step_no.data_ptr(), _lib.stream()), "pg_sample_top_p")
            self._step_no += 1
        else:
            _lib.check(L.pg_argmax(logits.data_ptr(), logits.stride(0), out.data_ptr(), n, V, _lib.stream()), "pg_argmax")
        return out.tolist()

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, do_sample: bool = False, temperature: float = 0.8,
                 top_p: float = 0.9, eos_token_id: Optional[int] = None, seed: int = 0, step_tokens: int = 512) -> List[List[int]]:
        """Greedy (or temperature / top-p) continuation of every prompt; more prompts than slots queue up and take over slots
        and pages as earlier ones finish.  Returns the new tokens per prompt (EOS included when it was emitted)."""
        sched = StepScheduler(self.store.num_slots, self.store.pool.num_pages, self.store.page, step_tokens, eos_token_id)
        for i, pr in enumerate(prompts):
            sched.submit(TokenRequest(("gen", i), [int(t) for t in pr], int(max_new_tokens)))
        while not sched.idle():
            plan = sched.plan()
            if not plan:
                raise RuntimeError("scheduler made no progress")
            entries = [(req.rid, toks, [len(toks) - 1] if sample else []) for req, toks, sample in plan]
            logits = self.step(entries)
            picked = self._sample(logits, do_sample, temperature, top_p, seed) if logits is not None else []
            it = iter(picked)
            for req, toks, sample in plan:
                if sched.advance(req, len(toks), next(it) if sample else None):
                    self.store.release(req.rid)
        return [sched.finished[("gen", i)] for i in range(len(prompts))]
