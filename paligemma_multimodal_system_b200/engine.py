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
from .seq_ops import StaticDecodeBatch, make_step_batch
from .serving import StepScheduler, TokenRequest


class SequenceEngine:
    def __init__(self, model, max_tokens: int, num_slots: int = 4, use_cuda_graph: bool = True):
        _lib.require_device()
        self.model = model
        self.store = SequenceStore(model.cache_layout(), max_tokens, num_slots, model.prec.dtype)
        self._step_no = torch.zeros(1, device="cuda", dtype=torch.int32)
        # decode steps (every entry one token) replay a CUDA graph per (entries, page-table width, context bound); the second
        # step of a geometry captures it, the first ran eagerly (lazy kernel attributes are set by then)
        self.use_cuda_graph = use_cuda_graph
        self._decode_graphs = {}

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
        if batch and trace is None and self.use_cuda_graph and all(len(e["tokens"]) == 1 for e in batch):
            logits = self._decode_step(batch, want)
            for (rid, toks, _w) in entries:
                store.commit(rid, len(toks))
        elif batch:
            b = make_step_batch(batch)
            rows = torch.tensor(want, dtype=torch.int64).to("cuda", non_blocking=True) if want else None
            logits = self.model.step(b, store, rows, trace=trace)
            for (rid, toks, _w) in entries:
                store.commit(rid, len(toks))
        for rid in end:
            if rid in store.live:
                store.release(rid)
        return logits

    def _decode_step(self, batch, want):
        """A step of single-token entries through a captured graph (eagerly the first time a geometry is seen)."""
        E = len(batch)
        pages = max(len(e["pages"]) for e in batch)
        pages_cap = 4
        while pages_cap < pages:
            pages_cap *= 2
        ctx_cap = pages_cap * self.store.page  # every context of this page-table width; fixes the key split of the attention
        key = (E, pages_cap)
        slot = self._decode_graphs.get(key)
        if slot is None:
            slot = self._decode_graphs[key] = dict(static=StaticDecodeBatch(E, pages_cap, ctx_cap), graph=None, logits=None, seen=0)
        st = slot["static"]
        st.fill(batch)
        slot["seen"] += 1
        if slot["graph"] is None and slot["seen"] >= 2:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    slot["logits"] = self.model.step(st.batch, self.store, st.rows)
            torch.cuda.current_stream().wait_stream(side)
            slot["graph"] = g
        if slot["graph"] is not None:
            slot["graph"].replay()
            full = slot["logits"]
        else:
            full = self.model.step(st.batch, self.store, st.rows)
        if not want:
            return None
        return full.index_select(0, torch.tensor(want, dtype=torch.int64).to("cuda", non_blocking=True))

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
