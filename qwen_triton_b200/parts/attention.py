"""Softmax attention over the paged cache with grouped kv heads, optional per-head q/k RMSNorm,
a position encoding part and an optional window.

Order as in the reference (qwen_triton/modules/attention.py:53-73,125-128): project, norm q and k
per head over head_dim *before* rotation, rotate, write k/v to the cache, attend, project out.
The three projections run as one product over the row-concatenated weight [q; k; v].
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, KVRequest, Runtime, part_class, register_mixer, to_device
from .linear import Linear

_DECODE_BLOCKS_PER_SM = 3           # blocks of the generic one-token kernel that are resident at once
_MAX_SPLIT_PAIRS = 640              # (sequence, split) pairs the scratch holds
_MIN_KEYS_PER_SPLIT = 128


@register_mixer("attention")
class Attention:
    graph_safe = True      # forward() only launches kernels: a decode step with this mixer can be captured in a CUDA graph

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.nq = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        self.scale = float(params.get("scale", self.d ** -0.5))
        self.window = params.get("window")
        self.own_kv = bool(params.get("own_kv", True))
        self.qk_norm = bool(params.get("qk_norm", False))
        self.bias = bool(params.get("bias", False))        # q, k, v and o projections with a bias (attention.py:38-41)
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.names = {k: params.get(k, k) for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
        if self.nq % self.nkv:
            raise ValueError(f"{prefix}: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d > 256:
            raise ValueError(f"{prefix}: head_dim={self.d} is beyond what the attention kernels take (256)")
        position_spec = params["position"]
        self.position = part_class("position", position_spec)(position_spec.params, runtime)
        self.interleaved = bool(getattr(self.position, "interleaved", False))      # which elements of a head form a rotation pair
        self.cos_sin: torch.Tensor | None = None
        self.q_weight = self.k_weight = None
        proj_rows = (self.nq + (2 * self.nkv if self.own_kv else 0)) * self.d
        self.qkv = Linear("attn.qkv" + (".biased" if self.bias else ""), proj_rows, self.hidden, runtime, role="qkv", bias=self.bias)
        self.o = Linear("attn.o" + (".biased" if self.bias else ""), self.hidden, self.nq * self.d, runtime, role="attn_out", bias=self.bias)
        ws = runtime.workspace
        ws.declare("attn.q", runtime.max_step_tokens * self.nq * self.d, runtime.dtype)
        ws.declare("attn.ctx", runtime.max_step_tokens * self.nq * self.d, runtime.dtype)
        ws.declare("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.d, torch.float32)
        ws.declare("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2, torch.float32)
        # few tokens: the projection takes rows whose norm factor is still to be applied (``ScaledRows``)
        self.takes_scaled_rows = self.qkv.fused_capable

    # ------------------------------------------------------------------ weights
    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, nq, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        n = {k: params.get(k, k) for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
        own_kv = bool(params.get("own_kv", True))
        out = {f"{prefix}.{n['q']}.weight": TensorSpec((nq * d, hidden)),
               f"{prefix}.{n['o']}.weight": TensorSpec((hidden, nq * d))}
        if own_kv:
            out[f"{prefix}.{n['k']}.weight"] = TensorSpec((nkv * d, hidden))
            out[f"{prefix}.{n['v']}.weight"] = TensorSpec((nkv * d, hidden))
        if params.get("bias", False):
            # the reference starts a bias at zero (models/core.py:269-270); random ones so that a bias that is skipped shows
            for name in ("q", "o") + (("k", "v") if own_kv else ()):
                rows = out[f"{prefix}.{n[name]}.weight"].shape[0]
                out[f"{prefix}.{n[name]}.bias"] = TensorSpec((rows,), role="vector", init_std=0.1, init_mean=0.0)
        if params.get("qk_norm", False):
            out[f"{prefix}.{n['q_norm']}.weight"] = TensorSpec((d,), role="vector", init_std=0.1, init_mean=1.0)
            if own_kv:
                out[f"{prefix}.{n['k_norm']}.weight"] = TensorSpec((d,), role="vector", init_std=0.1, init_mean=1.0)
        return out

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        rows = [source(f"{p}.{n['q']}.weight")]
        if self.own_kv:
            rows += [source(f"{p}.{n['k']}.weight"), source(f"{p}.{n['v']}.weight")]
        self.qkv.set_weight(torch.cat([r.to(self.runtime.dtype) for r in rows], dim=0))
        self.o.set_weight(source(f"{p}.{n['o']}.weight"))
        if self.bias:
            names = ("q", "k", "v") if self.own_kv else ("q",)
            self.qkv.set_bias(torch.cat([source(f"{p}.{n[name]}.bias").float() for name in names], dim=0))
            self.o.set_bias(source(f"{p}.{n['o']}.bias"))
        if self.qk_norm:
            self.q_weight = to_device(source(f"{p}.{n['q_norm']}.weight"), torch.float32, self.runtime.device)
            if self.own_kv:
                self.k_weight = to_device(source(f"{p}.{n['k_norm']}.weight"), torch.float32, self.runtime.device)
        tables = self.runtime.options.setdefault("position_tables", {})
        key = self.position.key() + (self.runtime.max_positions,)
        if key not in tables:
            tables[key] = self.position.table(self.runtime.max_positions)
        self.cos_sin = tables[key]

    # ------------------------------------------------------------------ cache
    def cache_request(self) -> KVRequest | None:
        return KVRequest(self.nkv, self.d, self.window)

    # ------------------------------------------------------------------ run
    def _splits(self, ctx, cache) -> tuple[int, int]:
        """How a one-token step cuts the keys of each sequence: (blocks per sequence and kv head, warps per block).

        The tensor-core kernel gives every warp a key range of its own.  Measured on the B200: with a moderate
        number of (sequence, kv head) pairs, about one block of four warps per SM and as few partial results as that
        allows; with very few pairs, blocks of six warps and a count weighed against the cost of merging them (below);
        with blocks for two per SM, three warps each and no cut at all.  Every range keeps at least
        two tiles of 32 keys.  The generic kernel (other element types and head sizes) takes one range per
        block: the count whose blocks fill whole waves of three blocks per SM nearly as well as the best one.
        """
        span = ctx.max_context if not self.window else min(ctx.max_context, self.window)
        group = self.nq // self.nkv
        most = max(1, min(_MAX_SPLIT_PAIRS // ctx.n_seqs, 32))
        if self.runtime.dtype == torch.bfloat16 and self.d % 16 == 0 and self.d <= 128 and cache.page_tokens == 64:
            pairs = ctx.n_seqs * self.nkv * math.ceil(group / 16)
            tiles = math.ceil(span / 32)
            sms = self.runtime.sm_count
            splits = max(1, min(sms // pairs, most))
            # blocks of four warps are one to an SM, of three two: three where that makes one wave of what would be two
            # with a nearly empty second one (160-192 blocks: 2-5 % shorter steps at batch 20-24 of the 8B shape), and
            # where there are blocks for three waves and more (batch 56-64: 6 %)
            warps = 3 if pairs * splits >= 3 * sms or sms < pairs * splits <= 2 * sms else 4
            if splits >= 4:
                # Few pairs (batch 1 to 4 with eight kv heads): blocks of six warps, and as many of them per pair as
                # pays: a block draws about 80 GB/s of keys and values, a merge through a cluster of up to four blocks
                # costs about 1.5 us, of six 3 us, and more blocks than a cluster holds (scratch memory and the combine
                # kernel) 13 us.  Clusters of five and seven, and more than eight clusters of eight, are left out: they
                # pack the SMs of a GPC badly beside the next product's clusters (batch 2, cache 8,192: 3.80 ms a step
                # with eight blocks per pair, 3.57 with five, 3.51 with six).  Timed in the model, 8B shape, batch 1: cache 2,048: 3.09 ms a step
                # with four blocks against 3.15 with eight; 8,192: 3.32 against 3.54 with four; 32,768: 3.99 with
                # eighteen against 4.23 with eight and 5.26 with four.
                warps = kernels.DECODE_WARPS_MAX
                pair_bytes = 4.0 * span * self.d                      # keys and values of one pair, bfloat16
                best = None
                for count in range(1, splits + 1):
                    if count > 1 and count * warps * 2 > tiles:
                        break
                    if count in (5, 7) or (count == 8 and pairs > 8):        # eight clusters of eight still find a GPC each
                        continue
                    merge = 0.0 if count == 1 else 1.5e-6 if count <= 4 else 3e-6 if count <= 8 else 13e-6
                    cost = merge + pair_bytes / (count * 80e9)
                    if best is None or cost < best[0]:
                        best = (cost, count)
                splits = best[1]
            while splits > 1 and splits * warps * 2 > tiles:
                splits -= 1
            while warps > 1 and splits * warps * 2 > tiles:
                warps -= 1
            return splits, warps
        heads_per_block = 8 if group > 4 else max(1, group)
        blocks = ctx.n_seqs * self.nkv * math.ceil(group / heads_per_block)
        most = max(1, min(span // _MIN_KEYS_PER_SPLIT, most))
        fills = []
        resident = _DECODE_BLOCKS_PER_SM * self.runtime.sm_count
        for splits in range(1, most + 1):
            total = blocks * splits
            fills.append(total / (math.ceil(total / resident) * resident))
        enough = max(fills) - 0.13
        return next(splits for splits, fill in enumerate(fills, start=1) if fill >= enough), 1

    def forward(self, x, ctx, cache):
        tokens = x.shape[0]
        ws = self.runtime.workspace
        q = ws.view("attn.q", tokens, self.nq, self.d)
        out = ws.view("attn.ctx", tokens, self.nq, self.d)
        table = ctx.block_table(cache.group)
        write = cache.writable and self.own_kv
        rotary_dim = 0 if self.cos_sin is None else self.cos_sin.shape[1]
        if self.qkv.fusable(tokens) and kernels.fused_qkv_supported(self.d, rotary_dim):
            # few tokens: per-head norm, rotation and the cache write in the projection's epilogue
            self.qkv.into_qkv(x, q, cache.k if write else None, cache.v if write else None, ctx.token_seq, ctx.token_pos,
                              table if write else None, self.q_weight, self.k_weight, self.eps, self.cos_sin, self.nq, self.nkv,
                              self.d, cache.page_tokens, cache.ring_tokens, write_kv=write, interleaved=self.interleaved)
        else:
            kernels.qk_norm_rope_write(
                self.qkv(x), q, cache.k if write else None, cache.v if write else None, ctx.token_seq, ctx.token_pos,
                table if write else None, self.q_weight, self.k_weight, self.eps, self.cos_sin, self.nq, self.nkv, self.d,
                cache.page_tokens, cache.ring_tokens, write_kv=write, kv_in_proj=self.own_kv, interleaved=self.interleaved)
        if ctx.is_decode:
            n_splits, warps = self._splits(ctx, cache)
            kernels.attention_decode(q, cache.k, cache.v, out, table, ctx.seq_len, self.nkv, cache.page_tokens,
                                     cache.ring_tokens, self.window, self.scale, n_splits,
                                     ws.view("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.d),
                                     ws.view("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2), warps=warps)
        else:
            kernels.attention_prefill(q, cache.k, cache.v, out, table, ctx.seq_start, ctx.seq_past, ctx.max_q_len,
                                      self.nkv, cache.page_tokens, cache.ring_tokens, self.window, self.scale)
        out = out.view(tokens, self.nq * self.d)
        return DeferredProduct(self.o, out) if self.o.fusable(tokens) else self.o(out)
