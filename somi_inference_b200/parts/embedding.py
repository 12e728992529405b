"""Token embedding and the output head.

Embedding: x = E[ids] (somi_inference/models/qwen2.py:360,382), written straight
into the float32 residual stream.  Head: logits = h E^T when tied
(somi_inference/models/qwen2_adapter.py:60-62), else h W_lm^T with the file's
`lm_head.weight`; logits are produced in float32 for the wanted rows only.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .linear import Linear
from .registry import EMBEDDINGS, HEADS, NORMS


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"],
                           (int(params["vocab_size"]), int(params["hidden_size"])))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))     # x = E[ids] * scale, in float32

    def forward(self, batch) -> torch.Tensor:
        token_ids = batch.token_ids
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32,
                          device=token_ids.device)
        if self.scale != 1.0:
            self.ctx.ops.embed_scaled(token_ids, self.weight, self.scale, out)
        else:
            self.ctx.ops.embed(token_ids, self.weight, out)
        return out


@EMBEDDINGS.register("sinusoid_embedding")
class SinusoidEmbedding:
    """x = norm(E[token] + s(position)): s has sin(p * base^(-2i/H)) at entry 2i and the cosine
    of the same angle at entry 2i + 1 (an odd width ends on a sine); `norm` is a norm part (its weight is this part's).  The
    frequencies are made once on the host (float64, rounded to float32); angles, sine, cosine
    and the norm are float32 in the kernel, which writes the residual stream."""

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"],
                           (int(params["vocab_size"]), int(params["hidden_size"]))),
                *NORMS.declare(params["norm"])]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]
        self.hidden = int(params["hidden_size"])
        norm = params["norm"]
        if norm.kind != "layernorm":
            raise ValueError(f"the sinusoid embedding's kernel applies a layer norm, not {norm.kind!r}")
        self.norm_weight = tensors[names_of(norm.params)["weight"]]
        self.eps = float(norm.params["eps"])
        i = torch.arange(0, self.hidden, 2, dtype=torch.float64)
        self.inv_freq = (float(params["base"]) ** (-i / self.hidden)).to(torch.float32).to(ctx.device)

    def forward(self, batch) -> torch.Tensor:
        out = torch.empty((batch.token_ids.shape[0], self.hidden), dtype=torch.float32,
                          device=batch.token_ids.device)
        self.ctx.ops.embed_sinusoid_layernorm(batch.token_ids, batch.positions, self.weight,
                                              self.inv_freq, self.norm_weight, self.eps, out)
        return out


@HEADS.register("lm_head")
class LMHead:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        shape = (int(params["vocab_size"]), int(params["hidden_size"]))
        # a tied model's file may still carry the head's matrix (the reference drops it as well:
        # somi_inference/models/qwen2_adapter.py:161-162): tolerated, never read
        return [TensorDecl(names_of(params)["weight"], shape, optional=bool(params["tied"]),
                           ignored=bool(params["tied"]))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.proj = Linear(tensors[n["tied_to"] if params["tied"] else n["weight"]], None, ctx.ops)
        # logits <- cap * tanh(logits / cap) where the model has a cap
        self.softcap = float(params["softcap"]) if params.get("softcap") else None

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.proj.to_float32(h)
        if self.softcap is not None:
            self.ctx.ops.softcap(logits, self.softcap)
        return logits
