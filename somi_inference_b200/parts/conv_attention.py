"""Attention whose queries, keys and values pass a short causal convolution before they are rotated.

Per token, with h the mixer's input:
    q = Wq h + bq, k = Wk h + bk, v = Wv h + bv
    each channel of q, k, v: u_t <- sum_j taps[c, j] * u_(t - n + 1 + j)   (zeros before the start)
    q, k: neighbouring pairs (2i, 2i+1) below `rotary.dims` turn by position * base^(-2i/dims)
    q, k: divided by their root mean square over the head (`unit_norm`, eps inside the root)
    scores q.k * scale over the keys the mask leaves: all earlier ones, the last `size`
    ("window"), or those of the token's own chunk of `size` positions ("chunk"); softmax
    out = Wo (heads * sigmoid(Wg h))                                       (`gate`)
Key and value widths may differ; query head i reads key/value head i // (heads / kv_heads).

One product makes q, k, v and the gate's logits; the convolution reads the first three out of
it and keeps the last taps - 1 projected rows of every request as state; one kernel rotates,
normalises and writes keys and values to their pages; the attention kernel applies the mask
and the gate.  Norms, scores and softmax are float32; angles are formed in float64 (their
sines and cosines are float32).
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, PagedKVNeeds, StateNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import MIXERS


@MIXERS.register("conv_attention")
class ConvAttentionMixer:
    graph_safe = True
    STATE = "qkv_taps"

    @staticmethod
    def _sizes(params):
        heads, kv_heads = int(params["num_heads"]), int(params["num_kv_heads"])
        d, dv = int(params["key_dim"]), int(params["value_dim"])
        return heads, kv_heads, d, dv

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, taps = int(params["hidden_size"]), int(params["taps"])
        heads, kv_heads, d, dv = ConvAttentionMixer._sizes(params)
        decl = []
        for part, rows in (("q", heads * d), ("k", kv_heads * d), ("v", kv_heads * dv)):
            decl.append(TensorDecl(n[part + "_weight"], (rows, hidden)))
            if params.get("qkv_bias"):
                decl.append(TensorDecl(n[part + "_bias"], (rows,), init="zeros", matrix=False))
            decl.append(TensorDecl(n[part + "_taps"], (rows, taps), init="taps", matrix=False))
        if params.get("gate"):
            decl.append(TensorDecl(n["gate_weight"], (heads * dv, hidden)))
        decl.append(TensorDecl(n["o_weight"], (hidden, heads * dv)))
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads, self.kv_heads, self.key_dim, self.value_dim = self._sizes(params)
        if self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot be grouped over {self.kv_heads} "
                             "key/value heads")
        if not (1 <= self.key_dim <= 256 and 1 <= self.value_dim <= 256):
            raise ValueError("key and value widths of 1 to 256 are supported")
        self.scale = float(params["scale"])
        self.taps = int(params["taps"])
        ctx.ops.check_conv_taps(self.taps)
        self.unit_norm = bool(params.get("unit_norm"))
        self.eps = float(params.get("eps", 0.0))
        mask = params.get("mask") or {}
        kind, size = mask.get("kind"), mask.get("size")
        if kind not in (None, "chunk", "window") or (kind is not None and not (size and size > 0)):
            raise ValueError(f"unknown mask {mask!r} (kinds: 'chunk', 'window', each with a size)")
        self.chunk = int(size) if kind == "chunk" else None
        self.window = int(size) if kind == "window" else None
        rotary = params.get("rotary") or {}
        self.rotary_dim = int(rotary.get("dims", 0))
        if self.rotary_dim % 2 or self.rotary_dim > self.key_dim:
            raise ValueError("rotary dims must be even and at most the key width")
        if self.rotary_dim:
            i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
            inv = float(rotary["base"]) ** (-i / self.rotary_dim)
        else:
            inv = torch.zeros(1, dtype=torch.float64)
        # float64: the kernel forms position * frequency and reduces it to [-pi, pi] in float64, so
        # that the angle's error does not grow with the position
        self.inv_freq = inv.to(ctx.device)

        self.qkv_width = (self.heads + self.kv_heads) * self.key_dim + self.kv_heads * self.value_dim
        self.gate_width = self.heads * self.value_dim if params.get("gate") else 0
        parts = ("q", "k", "v")
        w = [tensors[n[p + "_weight"]] for p in parts]
        if self.gate_width:
            w.append(tensors[n["gate_weight"]])
        bias = None
        if params.get("qkv_bias"):
            b = [tensors[n[p + "_bias"]].float() for p in parts]
            if self.gate_width:
                b.append(torch.zeros(self.gate_width, dtype=torch.float32, device=b[0].device))
            bias = torch.cat(b, 0)
        self.proj = Linear(torch.cat(w, 0).contiguous(), bias, ctx.ops)
        # [taps, channels] float32, the newest input's tap last
        self.taps_weight = torch.cat([tensors[n[p + "_taps"]].float() for p in parts], 0).t().contiguous()
        self.out = Linear(tensors[n["o_weight"]], None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        # a token of a chunk never reads further back than the chunk's size: pages older than
        # that are given back like those behind a window
        reach = self.chunk if self.chunk is not None else self.window
        paged = PagedKVNeeds(self.kv_heads, self.key_dim, reach,
                             None if self.value_dim == self.key_dim else self.value_dim)
        state = None
        if self.taps > 1:
            state = StateNeeds({self.STATE: ((self.taps - 1, self.qkv_width), self.ctx.dtype)})
        return CacheNeeds(paged=paged, state=state)

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops, paged = self.ctx.ops, cache.paged
        T = x.shape[0]
        proj = self.proj(x)                                    # [T, q | k | v | gate logits]
        qkv = torch.empty((T, self.qkv_width), dtype=x.dtype, device=x.device)
        ops.causal_conv(proj, self.qkv_width, self.taps_weight, None, cache.state.get(self.STATE),
                        batch, qkv)
        group = batch.groups[paged.group]
        ops.rotary_pairs_store(qkv, batch.positions, self.inv_freq, self.heads, self.kv_heads,
                               self.key_dim, self.value_dim, self.rotary_dim, self.unit_norm,
                               self.eps, group.slot_map if owns_cache else None, paged.keys,
                               paged.values)
        out = torch.empty((T, self.heads * self.value_dim), dtype=x.dtype, device=x.device)
        gate = proj[:, self.qkv_width:] if self.gate_width else None
        ops.paged_attention(qkv, paged.keys, paged.values, batch, group, self.heads, self.kv_heads,
                            self.key_dim, self.scale, self.window, out, storage=paged.storage,
                            value_dim=self.value_dim, chunk=self.chunk, gate=gate)
        partial = self.out.partial_sums(out)
        return partial if partial is not None else self.out(out)
