"""Grouped-query attention without a rotation, whose positions enter through the scores:

* every query head and every key head is rescaled to unit mean square, ``v / sqrt(mean(v^2) + eps)``
  with ``eps = qk_norm_eps`` and no learned gain (None: left as projected);
* the query at position ``p`` is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``
  (``q_temp = {"coef", "every"}``; None: no temperature);
* ``score(i, j) = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))``: a penalty that grows with
  the logarithm of the distance, two numbers per query head (``distance_bias``; False: neither the
  penalty nor the tensors ``r1``, ``r2``);
* the keys of a query at position ``i`` are those at ``i - window + 1 .. i`` (None: ``0 .. i``);
* keys and values may differ in size (``head_dim``, ``value_dim``).

A token keeps its key and value side by side in pages ``[kv_heads, page, head_dim + value_dim]``;
with a window the cache manager takes back the pages it has passed.  Scores, softmax and the
weighted sum are 32-bit; the projections give 32-bit sums, from which the norms are taken.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import BuildEnv, CacheNeed, LayerCache, Mixer, PartError, WeightSpec, register
from .linear import Linear


@register("mixer", "distance_biased_attention")
class DistanceBiasedAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``
    (None: ``head_dim``), ``scale``, ``window``, ``qk_norm_eps``, ``q_temp``, ``distance_bias``;
    tensors ``q``, ``k``, ``v``, ``o`` (``[out, in]``) and ``r1``, ``r2`` (``[num_heads]``)."""

    MAX_HEAD = 256

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "num_heads", "num_kv_heads", "head_dim", "scale")
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p["value_dim"]) if p.get("value_dim") is not None else self.hd
        if self.nkv <= 0 or self.nh % self.nkv:
            raise PartError(f"{self.nh} heads are not a multiple of {self.nkv} KV heads")
        if not (0 < self.hd <= self.MAX_HEAD and 0 < self.vd <= self.MAX_HEAD):
            raise PartError(f"head sizes {self.hd}/{self.vd} are not ones the kernel takes (1 to {self.MAX_HEAD})")
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        temp = p.get("q_temp")
        self.temp_coef = float(temp["coef"]) if temp else 0.0
        self.temp_every = int(temp["every"]) if temp else 0
        if temp and self.temp_every <= 0:
            raise PartError("q_temp.every must be positive")
        self.distance_bias = bool(p.get("distance_bias", True))
        self.q_size, self.k_size, self.v_size = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd
        self.qkv = Linear(env, self.q_size + self.k_size + self.v_size, self.hidden)
        self.o = Linear(env, self.hidden, self.nh * self.vd)
        self.r1 = self.r2 = None

    def weights(self) -> Dict[str, WeightSpec]:
        w = {"q": WeightSpec((self.q_size, self.hidden)), "k": WeightSpec((self.k_size, self.hidden)),
             "v": WeightSpec((self.v_size, self.hidden)), "o": WeightSpec((self.hidden, self.nh * self.vd))}
        if self.distance_bias:
            w["r1"] = WeightSpec((self.nh,), "positive")
            w["r2"] = WeightSpec((self.nh,), "positive")
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.qkv.load(torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0))
        self.o.load(tensors["o"])
        if self.distance_bias:
            self.r1 = tensors["r1"].float().contiguous()
            self.r2 = tensors["r2"].float().contiguous()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(outer=(self.nkv,), inner=(self.hd + self.vd,), window=self.window)

    def forward(self, h: torch.Tensor, step, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        ws = self.env.workspace
        qkv = self.qkv.forward(h, "battn.qkv", "float32")
        q = ws.get("battn.q", (T, self.q_size), self.env.dtype)
        table = step.block_tables[cache.group]
        ops.qk_norm_store(qkv, q, cache.pages if cache.writes else None, step.positions, step.token_seq, table,
                          self.nh, self.nkv, self.hd, self.vd, self.qk_norm_eps or 0.0,
                          normalise=self.qk_norm_eps is not None, temp_coef=self.temp_coef,
                          temp_every=self.temp_every)
        out = ws.get("battn.out", (T, self.nh * self.vd), self.env.dtype)
        # bfloat16: one-row sequences on the decode kernel (a step of such rows only is what a CUDA graph
        # records, and every replay is again such a step); 32-bit: one kernel for all rows, so that a
        # row has the same bits alone, in a portion and in a batch
        lens = step.host_query_lens
        single = self.env.dtype == torch.bfloat16 and (step.max_query_len == 1 or 1 in lens)
        ops.attention_window_bias(q, out, cache.pages, table, step.seq_start, step.positions, step.num_seqs,
                                  self.nh, self.nkv, self.hd, self.vd, self.scale, self.window or 0, self.r1, self.r2,
                                  single_rows=single, other_rows=step.max_query_len != 1)
        return self.o.forward(out, "battn.o", "delta")
