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
