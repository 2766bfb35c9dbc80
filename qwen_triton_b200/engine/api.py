"""The Python entry point, in the manner of the reference's ``QwenTritonForCausalLM``
(qwen_triton/models/core.py:250-409): ``from_pretrained_hf``, ``from_config``, a whole-sequence
``forward`` with ``logits_to_keep``, and ``greedy_generate``; plus ``generate`` for unequal prompts,
stop tokens and temperature sampling, which the reference does not have.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Sequence

import torch

from ..config import config_from_dict, load_config
from ..sampling import Sampler, SamplingParams
from .engine import Engine, parse_dtype
from .generate import BatchRun, GenerationResult, generate, stop_set
from .step import StepEntry


@dataclass
class CausalLMOutput:
    logits: torch.Tensor          # [batch, kept positions, vocab], float32; rows of padding are zero


class QwenB200ForCausalLM:
    """One model on one B200.  Token ids in, logits or token ids out."""

    def __init__(self, engine: Engine) -> None:
        self.engine = engine
        self.config = getattr(engine, "config", None)
        self.sampler = Sampler(engine.device)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained_hf(cls, model_id: str | Path, backend: str = "b200", device: str | torch.device = "cuda:0",
                           dtype: torch.dtype | str | None = None, **engine_options: Any) -> "QwenB200ForCausalLM":
        """``model_id`` is a local model folder (config.json + safetensors); nothing is downloaded.
        ``backend`` exists for the reference's signature; the only backend is the sm_100a kernels."""
        if backend not in ("b200", "cuda"):
            raise ValueError(f"backend {backend!r} is not built; this library has one backend, 'b200'")
        if not Path(model_id).exists():
            raise FileNotFoundError(f"{model_id} is not a local model folder (hub downloads are not part of this library)")
        engine = Engine.from_pretrained(model_id, dtype=parse_dtype(dtype or "bf16"), device=device, **engine_options)
        return cls(engine)

    @classmethod
    def from_config(cls, config: Mapping[str, Any] | Any, seed: int = 0, device: str | torch.device = "cuda:0",
                    dtype: torch.dtype | str | None = None, **engine_options: Any) -> "QwenB200ForCausalLM":
        """Random weights (seeded) for a config.json mapping or a typed configuration."""
        if isinstance(config, Mapping):
            config = config_from_dict(config)
        engine = Engine.from_config(config, seed=seed, dtype=parse_dtype(dtype or "bf16"), device=device,
                                    **engine_options)
        return cls(engine)

    # ------------------------------------------------------------------ forward
    @staticmethod
    def _rows(input_ids, attention_mask) -> list[list[int]]:
        ids = torch.as_tensor(input_ids).cpu()
        if ids.dim() == 1:
            ids = ids[None]
        if attention_mask is None:
            return [row.tolist() for row in ids]
        mask = torch.as_tensor(attention_mask).cpu().bool()
        rows = []
        for row, keep in zip(ids, mask):
            length = int(keep.sum())
            if not bool(keep[:length].all()):
                raise ValueError("attention_mask must mark a prefix of each row (right padding)")
            rows.append(row[:length].tolist())
        return rows

    @torch.no_grad()
    def forward(self, input_ids, attention_mask=None, logits_to_keep: int = 0) -> CausalLMOutput:
        """Whole sequences, no cache kept.  ``logits_to_keep`` = n > 0 keeps the last n positions of
        each sequence, 0 keeps all (qwen_triton/models/core.py:360-363)."""
        rows = self._rows(input_ids, attention_mask)
        slots = [self.engine.new_sequence() for _ in rows]
        try:
            wants = [list(range(len(r))) if logits_to_keep <= 0 else list(range(max(0, len(r) - logits_to_keep), len(r)))
                     for r in rows]
            flat = self.engine.step([StepEntry(s, r, w) for s, r, w in zip(slots, rows, wants)])
            self.engine.check_kernels()
        finally:
            for slot in slots:
                self.engine.release(slot)
        width = max(len(w) for w in wants)
        out = torch.zeros((len(rows), width, self.engine.vocab_size), dtype=torch.float32, device=flat.device)
        offset = 0
        for i, w in enumerate(wants):
            # all positions: left-aligned like the input; last n: right-aligned so that [:, -1] is each row's last token
            start = 0 if logits_to_keep <= 0 else width - len(w)
            out[i, start:start + len(w)] = flat[offset:offset + len(w)]
            offset += len(w)
        return CausalLMOutput(logits=out)

    __call__ = forward

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                 seed: int = 0, stop_token_ids: Sequence[int] | None = None, ignore_eos: bool = False,
                 max_batch_size: int | None = None, top_k: int = 0, top_p: float = 1.0) -> list[GenerationResult]:
        return generate(self.engine, prompts, max_new_tokens=max_new_tokens,
                        sampling=SamplingParams(temperature=temperature, seed=seed, top_k=top_k, top_p=top_p),
                        stop_token_ids=stop_token_ids, ignore_eos=ignore_eos, max_batch_size=max_batch_size, sampler=self.sampler)

    def start_batch(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                    seed: int = 0, stop_token_ids: Sequence[int] | None = None, ignore_eos: bool = False,
                    top_k: int = 0, top_p: float = 1.0) -> BatchRun:
        """Step-by-step generation of one batch: ``run.start()`` runs the prompts and returns each request's
        first token, every ``run.advance()`` one more token per request still going; ``run.results`` collects
        them and ``run.close()`` gives the cache back.  ``generate`` is this, looped over batches."""
        results = [GenerationResult() for _ in prompts]
        return BatchRun(self.engine, self.sampler, prompts, results, range(len(prompts)), max_new_tokens=max_new_tokens,
                        sampling=SamplingParams(temperature=temperature, seed=seed, top_k=top_k, top_p=top_p),
                        stop=stop_set(self.engine, stop_token_ids, ignore_eos))

    @torch.no_grad()
    def greedy_generate(self, input_ids, attention_mask=None, max_new_tokens: int = 16) -> torch.LongTensor:
        """As the reference's ``greedy_generate`` (qwen_triton/models/core.py:377-409): exactly
        ``max_new_tokens`` greedy tokens per row, no stop condition; returns prompt and new tokens.
        Rows shorter than the widest are padded on the right with 0 after their new tokens."""
        rows = self._rows(input_ids, attention_mask)
        results = self.generate(rows, max_new_tokens=max_new_tokens, temperature=0.0, ignore_eos=True)
        width = max(len(r) for r in rows) + max_new_tokens
        out = torch.zeros((len(rows), width), dtype=torch.long)
        for i, (row, result) in enumerate(zip(rows, results)):
            sequence = row + result.tokens
            out[i, :len(sequence)] = torch.tensor(sequence, dtype=torch.long)
        return out
