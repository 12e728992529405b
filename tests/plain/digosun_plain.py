"""A plain, slow restatement of the Digosun decoder, one function per mechanism.

Written from the design's equations, with whole-sequence tensors and Python loops; it shares
nothing with the engine (no cache, no pages, no kernels) and serves as the oracle of its tests.
`cfg` is the dictionary of the model's config.json, `w` maps tensor names to tensors; all
arithmetic runs in `dtype` (float64 by default).

Notation: S tokens of one sequence at positions 0..S-1, D the model width, x the residual stream.
"""

from __future__ import annotations

import torch


def sinusoid(positions: torch.Tensor, width: int, dtype=torch.float64) -> torch.Tensor:
    """[S, D]: column 2i holds sin(p * 10000^(-2i/D)), column 2i+1 the cosine of the same angle."""
    out = torch.zeros((positions.shape[0], width), dtype=dtype)
    p = positions.to(dtype)
    for c in range(width):
        i = c // 2
        angle = p * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(angle) if c % 2 == 0 else torch.cos(angle)
    return out


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight over the last axis, var = mean of squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * weight


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def causal_taps(h: torch.Tensor, taps_weight: torch.Tensor) -> torch.Tensor:
    """h + conv(h): conv(h)[t] = sum_j w[:, j] * h[t - (taps - 1) + j], zero before the start."""
    S, _ = h.shape
    taps = taps_weight.shape[1]
    out = h.clone()
    for t in range(S):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += taps_weight[:, j] * h[src]
    return out


def windowed_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                            window: int | None, sink: torch.Tensor, first: int = 0) -> torch.Tensor:
    """q, k [S, H, d], v [S, H, dv] -> [S, H, dv] (rows before `first` are left zero).  Token i
    reads j with 0 <= i - j < window; the softmax denominator of head h also holds exp(sink[h]),
    which carries no value."""
    S, H, _ = q.shape
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for i in range(first, S):
        lo = 0 if window is None else max(0, i - window + 1)
        s = torch.einsum("jhd,hd->jh", k[lo:i + 1], q[i]) * scale          # [keys, H]
        m = torch.maximum(s.max(dim=0).values, sink)
        e = torch.exp(s - m)
        denom = e.sum(dim=0) + torch.exp(sink - m)
        out[i] = torch.einsum("jh,jhd->hd", e, v[lo:i + 1]) / denom[:, None]
    return out


def kv_latent(h: torch.Tensor, w: dict, prefix: str, eps: float) -> torch.Tensor:
    """The cached latent of a layer that owns one: rms_norm(W_dkv h)."""
    return rms_norm(h @ w[f"{prefix}.mix.dkv"].T, w[f"{prefix}.mix.dkv.norm"], eps)


def latent_attention(h: torch.Tensor, latent: torch.Tensor, w: dict, prefix: str, mixer: dict,
                     eps: float) -> torch.Tensor:
    """Queries through their own latent, keys and values expanded from `latent` head by head."""
    H, d, dv = mixer["heads"], mixer["dim"], mixer["vdim"]
    S = h.shape[0]
    cq = rms_norm(h @ w[f"{prefix}.mix.dq"].T, w[f"{prefix}.mix.dq.norm"], eps)
    q = (cq @ w[f"{prefix}.mix.uq"].T).reshape(S, H, d)
    k = (latent @ w[f"{prefix}.mix.uk"].T).reshape(S, H, d)
    v = (latent @ w[f"{prefix}.mix.uv"].T).reshape(S, H, dv)
    mask = mixer.get("mask")
    window = None if not mask else mask.get("size")
    a = windowed_sink_attention(q, k, v, float(mixer["scale"]), window, w[f"{prefix}.mix.sink"])
    return a.reshape(S, H * dv) @ w[f"{prefix}.mix.o"].T


def dense_ff(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    act = w[f"{prefix}.mlp.act"]
    z = h @ w[f"{prefix}.mlp.up"].T + w[f"{prefix}.mlp.up.b"]
    return xielu(z, act[0], act[1]) @ w[f"{prefix}.mlp.down"].T + w[f"{prefix}.mlp.down.b"]


def gate(h: torch.Tensor, w: dict, name: str) -> torch.Tensor:
    return torch.sigmoid(h @ w[name].T + w[f"{name}.b"])


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [S, vocab] of one sequence from position 0 (and the residual after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    D, eps = cfg["width"], float(cfg["norm"]["eps"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    S = ids.shape[0]
    x = w["embed"][ids] + sinusoid(torch.arange(S), D, dtype)
    x = layer_norm(x, w["embed.norm"], eps)
    latents: dict[int, torch.Tensor] = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] != "latent_attention":
            raise ValueError(f"unknown mixer {layer['type']!r}")
        mixer = layer["mixer"]
        h = layer_norm(x, w[f"{p}.norm1"], eps)
        hc = causal_taps(h, w[f"{p}.canon1"])
        if mixer.get("kv_from") is None:
            latents[i] = kv_latent(hc, w, p, eps)
            c = latents[i]
        else:
            c = latents[int(mixer["kv_from"])]
        x = x + gate(h, w, f"{p}.rg1") * latent_attention(hc, c, w, p, mixer, eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward {layer['mlp']['kind']!r}")
            h = layer_norm(x, w[f"{p}.norm2"], eps)
            x = x + gate(h, w, f"{p}.rg2") * dense_ff(h, w, p)
        after.append(x.clone())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    if return_layers:
        return logits, torch.stack(after)
    return logits


def greedy(cfg: dict, weights: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, weights, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
