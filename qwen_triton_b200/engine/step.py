"""One step's work as the kernels see it, and how a step is cut into passes.

A step brings, for each of its sequences, the next tokens and the places whose logits are wanted.
``plan_passes`` cuts it into passes that fit the per-pass token limit and, where a cache group keeps
only a window of keys, the per-sequence chunk limit; ``StepContext`` is one pass: packed tokens with
their sequence and position, per-sequence offsets and lengths, page tables per cache group, all as
int32 arrays in one device buffer filled by a single copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    tokens: list[int]
    want: list[int] = field(default_factory=list)    # places among ``tokens`` whose logits are wanted


@dataclass
class PassPiece:
    entry: int          # index into the step's entries
    begin: int          # token range of the entry that this pass runs
    end: int


def plan_passes(lengths: list[int], max_tokens: int, chunk_limit: int | None) -> list[list[PassPiece]]:
    """Cut ``lengths`` tokens per entry into passes of at most ``max_tokens`` tokens in total and at
    most ``chunk_limit`` tokens per entry.  Within an entry the pieces keep their order, one per pass at most."""
    if max_tokens <= 0:
        raise ValueError("max_tokens must be positive")
    done = [0] * len(lengths)
    passes: list[list[PassPiece]] = []
    while any(done[i] < lengths[i] for i in range(len(lengths))):
        budget = max_tokens
        pieces: list[PassPiece] = []
        for i, total in enumerate(lengths):
            if done[i] >= total or budget == 0:
                continue
            take = min(total - done[i], budget, chunk_limit or total)
            pieces.append(PassPiece(i, done[i], done[i] + take))
            done[i] += take
            budget -= take
        passes.append(pieces)
    return passes


class StepContext:
    """Device-side description of one pass."""

    def __init__(self, *, device: torch.device, meta: torch.Tensor) -> None:
        self.device = device
        self._meta = meta          # int32 device buffer that holds every array below
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.max_q_len = 0
        self.max_context = 0       # longest sequence after this pass
        self.is_decode = False
        self.token_ids = self.token_seq = self.token_pos = None
        self.seq_start = self.seq_past = self.seq_len = self.slots = self.want_rows = None
        self._tables: dict[int, torch.Tensor] = {}
        self._decode_plans: dict[tuple, "_DecodePlan"] = {}

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    @staticmethod
    def meta_size(max_tokens: int, max_seqs: int, table_widths: list[int]) -> int:
        return 4 * max_tokens + 5 * max_seqs + 8 + max_seqs * sum(table_widths) + 64

    def fill(self, slots: list[int], tokens: list[list[int]], past: list[int], want_rows: list[int],
             tables: list[np.ndarray], max_context: int | None = None) -> None:
        """Pack the pass on the host and copy it to the device in one transfer.  For given counts of
        tokens, sequences, wanted rows and table widths every array lands at the same address, which is
        what lets a captured decode step be replayed on new contents."""
        n_seqs = len(slots)
        q_lens = [len(t) for t in tokens]
        n_tokens = sum(q_lens)
        parts: list[np.ndarray] = []
        token_ids = np.fromiter((tok for seq in tokens for tok in seq), dtype=np.int32, count=n_tokens)
        token_seq = np.repeat(np.arange(n_seqs, dtype=np.int32), q_lens)
        seq_start = np.zeros(n_seqs + 1, dtype=np.int32)
        np.cumsum(q_lens, out=seq_start[1:])
        past_arr = np.asarray(past, dtype=np.int32)
        token_pos = (np.arange(n_tokens, dtype=np.int32) - seq_start[token_seq]) + past_arr[token_seq]
        seq_len = past_arr + np.asarray(q_lens, dtype=np.int32)
        parts = [token_ids, token_seq, token_pos.astype(np.int32), seq_start, past_arr, seq_len,
                 np.asarray(slots, dtype=np.int32), np.asarray(want_rows, dtype=np.int32)]
        parts += [np.ascontiguousarray(t, dtype=np.int32).reshape(-1) for t in tables]
        total = sum(p.size for p in parts)
        if total > self._meta.numel():
            raise ValueError(f"step metadata of {total} words exceeds the buffer of {self._meta.numel()}")
        host = torch.empty(total, dtype=torch.int32, pin_memory=True)
        np.concatenate(parts, out=host.numpy())
        self._meta[:total].copy_(host, non_blocking=True)
        self.meta_bytes = 4 * total

        offset = 0
        views = []
        for p in parts:
            views.append(self._meta[offset:offset + p.size])
            offset += p.size
        (self.token_ids, self.token_seq, self.token_pos, self.seq_start, self.seq_past, self.seq_len,
         self.slots, self.want_rows) = views[:8]
        self._tables = {g: views[8 + g].view(n_seqs, tables[g].shape[1]) for g in range(len(tables))}
        self.n_tokens, self.n_seqs, self.n_want = n_tokens, n_seqs, len(want_rows)
        self.max_q_len = max(q_lens) if q_lens else 0
        self.max_context = max_context if max_context is not None else (int(seq_len.max()) if n_seqs else 0)
        self.is_decode = bool(q_lens) and all(q == 1 for q in q_lens)

    # ------------------------------------------------------------------ one token per sequence
    def prepare_decode(self, slots: list[int], past: list[int], tables: list[np.ndarray]):
        """The part of ``fill`` for a pass of one token per sequence (every row wanted) that does not need the
        tokens: the same layout at the same addresses, written into pinned buffers that are kept (a small ring,
        each guarded by an event, so that a caller who runs ahead of the device cannot overwrite a copy that has
        not happened yet) with the parts that never change filled in once.  Returns what ``commit_decode`` takes."""
        n = len(slots)
        key = (n, tuple(t.shape[1] for t in tables))
        plan = self._decode_plans.get(key)
        if plan is None:
            plan = self._decode_plans[key] = _DecodePlan(self._meta, n, key[1])
        host, array, event = plan.next_buffer()
        array[2 * n:3 * n] = past
        array[plan.at_past:plan.at_past + n] = past
        np.add(array[plan.at_past:plan.at_past + n], 1, out=array[plan.at_len:plan.at_len + n])
        array[plan.at_slots:plan.at_slots + n] = slots
        for offset, table in zip(plan.at_tables, tables):
            array[offset:offset + table.size] = table.reshape(-1)
        return plan, host, array, event

    def commit_decode(self, prepared, tokens: list[int], max_context: int, chosen: torch.Tensor | None = None,
                      vocab: int = 0) -> None:
        """Put the tokens in, copy the pass to the device in one transfer and make it the current pass.
        With ``chosen`` (int32 on the device) ``tokens`` are row numbers of it (negative: token 0): the ids are then
        filled in on the device, from what a sampling kernel has written or is about to write."""
        plan, host, array, event = prepared
        n = plan.n
        array[0:n] = tokens
        self._meta[:plan.total].copy_(host, non_blocking=True)
        event.record()
        if chosen is not None:
            from ..ops import kernels
            kernels.feed_tokens(plan.views[0], chosen, vocab)
        self.meta_bytes = 4 * plan.total
        (self.token_ids, self.token_seq, self.token_pos, self.seq_start, self.seq_past, self.seq_len,
         self.slots, self.want_rows) = plan.views[:8]
        self._tables = plan.tables
        self.n_tokens = self.n_seqs = self.n_want = n
        self.max_q_len = 1
        self.max_context = max_context
        self.is_decode = True


class _DecodePlan:
    """Offsets, device views and pinned host buffers of ``prepare_decode`` for one batch size and table widths."""

    RING = 4

    def __init__(self, meta: torch.Tensor, n: int, widths: tuple[int, ...]) -> None:
        self.n = n
        sizes = [n, n, n, n + 1, n, n, n, n] + [n * w for w in widths]
        offsets = np.concatenate(([0], np.cumsum(sizes))).tolist()
        self.total = offsets[-1]
        if self.total > meta.numel():
            raise ValueError(f"step metadata of {self.total} words exceeds the buffer of {meta.numel()}")
        self.at_past, self.at_len, self.at_slots = offsets[4], offsets[5], offsets[6]
        self.at_tables = offsets[8:8 + len(widths)]
        self.views = [meta[offsets[i]:offsets[i + 1]] for i in range(len(sizes))]
        self.tables = {g: self.views[8 + g].view(n, w) for g, w in enumerate(widths)}
        self.buffers = []
        for _ in range(self.RING):
            host = torch.zeros(self.total, dtype=torch.int32, pin_memory=True)
            array = host.numpy()
            array[offsets[1]:offsets[2]] = np.arange(n)              # token_seq
            array[offsets[3]:offsets[4]] = np.arange(n + 1)          # seq_start
            array[offsets[7]:offsets[8]] = np.arange(n)              # want_rows
            self.buffers.append((host, array, torch.cuda.Event()))
        self.turn = 0

    def next_buffer(self):
        host, array, event = self.buffers[self.turn % self.RING]
        if self.turn >= self.RING:
            event.synchronize()                                      # the copy that last used this buffer has happened
        self.turn += 1
        return host, array, event
