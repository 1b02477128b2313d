"""Replay of a recorded serving trace: given token ids are fed step by step through the model's own step function
(``forward_infer``) and KV cache, and the logits at chosen places are returned.  Nothing is sampled.

A step is a list of entries ``{"id", "tokens", "want"}``: the next tokens of every request of that step and the places
(among these tokens) whose logits are asked for, plus the ids that end with the step.  All entries of a step form one
batch: either every request starts (context encoding, right-padded to the longest) or every request continues by one
token (token generation over the cache lines the requests hold).  A request keeps its cache line from its first step
until it ends; freed lines are handed out again (lowest first).  With a paged pool the lines' pages are reserved and
released through the cache's allocator.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch


class TraceReplayer:
    def __init__(self, model, pad_token_id: int = 0):
        self.model = model
        if model.kv_cache is None:
            model.init_kv_cache()
        self.cache = model.kv_cache
        self.pad = pad_token_id
        self.free_lines: List[int] = list(range(self.cache.lines))
        self.line_of: Dict[str, int] = {}
        self.length: Dict[str, int] = {}
        self.device = next(model.parameters()).device

    # -- cache lines ------------------------------------------------------------------------------------------------
    def _admit(self, rid: str) -> int:
        if not self.free_lines:
            raise RuntimeError(f"no free cache line for request {rid!r} ({self.cache.lines} lines)")
        line = min(self.free_lines)
        self.free_lines.remove(line)
        self.line_of[rid], self.length[rid] = line, 0
        return line

    def release(self, rid: str) -> None:
        line = self.line_of.pop(rid, None)
        self.length.pop(rid, None)
        if line is not None:
            self.cache.free(line)
            self.free_lines.append(line)

    # -- one step ---------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: List[dict], end: Iterable[str] = ()) -> Optional[torch.Tensor]:
        """Runs the entries as one batch; returns fp32 logits ``[wanted, vocab]`` in entry / want order (``None`` when
        nothing is wanted)."""
        entries = [e for e in entries if len(e["tokens"]) > 0]
        out = None
        if entries:
            for e in entries:
                if e["id"] not in self.line_of:
                    self._admit(e["id"])
            starts = [self.length[e["id"]] for e in entries]
            counts = [len(e["tokens"]) for e in entries]
            B, T = len(entries), max(counts)
            if T > 1 and any(s != 0 for s in starts) and not getattr(self.model, "supports_prefill_at_offset", False):
                raise ValueError("this model family cannot continue a prompt in portions")
            dev = self.device
            ids = torch.full((B, T), self.pad, dtype=torch.long)
            for b, e in enumerate(entries):
                ids[b, : counts[b]] = torch.tensor(e["tokens"], dtype=torch.long)
            pos = torch.tensor(starts, dtype=torch.long).unsqueeze(1) + torch.arange(T, dtype=torch.long).unsqueeze(0)
            lines = torch.tensor([self.line_of[e["id"]] for e in entries], dtype=torch.int32)
            for b, e in enumerate(entries):
                if starts[b] + counts[b] > self.cache.seq_len:
                    raise ValueError(f"request {e['id']!r} outgrows the cache ({self.cache.seq_len} tokens per line)")
                self.cache.reserve(self.line_of[e["id"]], starts[b] + counts[b])
            rows = [b for b, e in enumerate(entries) for _ in e["want"]]
            cols = [int(w) for e in entries for w in e["want"]]
            if not rows:                      # the step still has to run: it fills the cache
                rows, cols = [0], [0]
            last = torch.tensor(counts, dtype=torch.long) - 1
            _, logits = self.model.forward_infer(
                ids.to(dev), pos.to(dev), seq_ids=lines.to(dev), last_token_index=last.to(dev), return_logits=True,
                logit_index=(torch.tensor(rows, device=dev), torch.tensor(cols, device=dev)), sample=False,
                past_context=T > 1 and any(s != 0 for s in starts))
            for b, e in enumerate(entries):
                self.length[e["id"]] = starts[b] + counts[b]
            if any(e["want"] for e in entries):
                out = logits.float()
        for rid in end:
            self.release(rid)
        return out
