"""Mamba-2 mixer: a state-space recurrence per head with a short convolution in front.

With h the mixer's input, inner = heads * head width P, N the state size, G groups:
    [z | x | B | C | dt] = W_in h          (inner, inner, G N, G N, heads columns)
    x, B, C <- silu(conv(x, B, C) + b)     (causal, per channel, zeros before the start)
    dt <- softplus(dt + dt_bias)           (no clamp)
    per head i (group i // (heads / G)), state M [N, P] from zero:
        M <- exp(-exp(A_log_i) dt_i) M + dt_i B x_i^T;   y_i = M^T C + D_i x_i
    y <- y * silu(z); RMS norm in `norm_groups` equal parts, times a weight; W_o.
The state M is float32 and lives in the request's state slot with the convolution's last
taps - 1 inputs; softplus, decay, the recurrence and the norm are float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, StateNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import MIXERS


@MIXERS.register("mamba2")
class Mamba2Mixer:
    graph_safe = True
    STATE_SSM, STATE_CONV = "ssm", "conv_taps"

    @staticmethod
    def _sizes(params):
        heads, P = int(params["heads"]), int(params["head_dim"])
        N, G = int(params["state_size"]), int(params["groups"])
        return heads, P, N, G, heads * P, heads * P + 2 * G * N

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, taps = int(params["hidden_size"]), int(params["taps"])
        heads, P, N, G, inner, conv_ch = Mamba2Mixer._sizes(params)
        return [TensorDecl(n["in_weight"], (inner + conv_ch + heads, hidden)),
                TensorDecl(n["taps"], (conv_ch, taps), init="taps", matrix=False),
                TensorDecl(n["taps_bias"], (conv_ch,), init="zeros", matrix=False),
                TensorDecl(n["dt_bias"], (heads,), init="zeros", matrix=False),
                TensorDecl(n["a_log"], (heads,), init="zeros", matrix=False),
                TensorDecl(n["skip"], (heads,), init="ones", matrix=False),
                TensorDecl(n["norm"], (inner,), init="ones", matrix=False),
                TensorDecl(n["o_weight"], (hidden, inner))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.heads, self.head_dim, self.state_size, self.groups, self.inner, self.conv_ch = \
            self._sizes(params)
        self.taps = int(params["taps"])
        self.norm_groups = int(params["norm_groups"])
        self.eps = float(params["eps"])
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} columns cannot be normalised in {self.norm_groups} equal parts")
        ctx.ops.check_conv_taps(self.taps)
        ctx.ops.check_ssm_geometry(self.heads, self.groups, self.state_size)
        self.inp = Linear(tensors[n["in_weight"]], None, ctx.ops)
        self.taps_weight = tensors[n["taps"]].float().t().contiguous()      # [taps, channels]
        self.taps_bias = tensors[n["taps_bias"]].float().contiguous()
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.a_log = tensors[n["a_log"]].float().contiguous()
        self.skip = tensors[n["skip"]].float().contiguous()
        self.norm_weight = tensors[n["norm"]]
        self.out = Linear(tensors[n["o_weight"]], None, ctx.ops)

    def cache_needs(self) -> CacheNeeds:
        # [heads, head width, state size]: the state's rows of one column lie side by side
        state = {self.STATE_SSM: ((self.heads, self.head_dim, self.state_size), torch.float32)}
        if self.taps > 1:
            state[self.STATE_CONV] = ((self.taps - 1, self.conv_ch), self.ctx.dtype)
        return CacheNeeds(paged=None, state=StateNeeds(state))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        ops = self.ctx.ops
        T = x.shape[0]
        proj = self.inp(x)                                     # [T, z | x B C | dt]
        z = proj[:, :self.inner]
        dt = proj[:, self.inner + self.conv_ch:]
        xbc = torch.empty((T, self.conv_ch), dtype=x.dtype, device=x.device)
        ops.causal_conv(proj[:, self.inner:], self.conv_ch, self.taps_weight, self.taps_bias,
                        cache.state.get(self.STATE_CONV), batch, xbc, act="silu")
        y = torch.empty((T, self.inner), dtype=torch.float32, device=x.device)
        ops.ssm_scan(xbc, dt, self.dt_bias, self.a_log, self.skip, cache.state[self.STATE_SSM],
                     batch, y, self.heads, self.groups, self.state_size, self.head_dim)
        gated = torch.empty((T, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(y, z, self.norm_weight, self.eps, self.norm_groups, gated)
        partial = self.out.partial_sums(gated)
        return partial if partial is not None else self.out(gated)
