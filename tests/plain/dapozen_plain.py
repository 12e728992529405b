"""A plain, slow restatement of the Dapozen decoder, one function per mechanism.

Written from the design's equations with whole-sequence tensors and Python loops.  It shares
nothing with the engine (no cache, no pages, no kernels, no portions) and is the oracle of the
engine's tests.  `cfg` is the dictionary of a model's config.json, `w` maps tensor names to
tensors; all arithmetic runs in `dtype` (float64 by default).

Notation: S tokens of one sequence at positions 0..S-1, D the model width, x the residual stream.
"""

from __future__ import annotations

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def short_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """u [S, C], taps [C, n]: y[t] = sum_j taps[:, j] * u[t - (n - 1) + j] (+ bias); inputs before
    the sequence's start are zero.  The last column of `taps` multiplies the current token."""
    S, _ = u.shape
    n = taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(S):
        for j in range(n):
            src = t - (n - 1) + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y if bias is None else y + bias


def rotate_pairs(x: torch.Tensor, rot_dims: int, base: float) -> torch.Tensor:
    """x [S, H, d]: neighbouring entries (2i, 2i+1), i < rot_dims/2, of the token at position p turn
    by the angle p * base^(-2i/rot_dims); entries from rot_dims on are left as they are."""
    S = x.shape[0]
    out = x.clone()
    p = torch.arange(S, dtype=x.dtype)
    for i in range(rot_dims // 2):
        angle = p * (base ** (-2.0 * i / rot_dims))
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        a, b = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = a * c - b * s
        out[:, :, 2 * i + 1] = b * c + a * s
    return out


def chunked_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                              chunk: int | None) -> torch.Tensor:
    """q [S, H, d], k [S, G, d], v [S, G, dv] -> [S, H, dv].  Query head h reads key/value head
    h // (H / G).  Token i reads j <= i with i // chunk == j // chunk (no chunk: all j <= i)."""
    S, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for i in range(S):
        lo = 0 if chunk is None else (i // chunk) * chunk
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    """Projections with biases, a short convolution on each of q, k, v, rotation of q and k, unit
    root mean square per head, chunked softmax attention, a sigmoid gate from the mixer's input,
    output projection."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    p = prefix + ".mix."
    parts = {}
    for name in ("q", "k", "v"):
        u = h @ w[p + name].T + w[p + name + ".b"]
        parts[name] = short_conv(u, w[p + name + ".conv"])
    q = parts["q"].reshape(S, H, d)
    k = parts["k"].reshape(S, G, d)
    v = parts["v"].reshape(S, G, dv)
    rot = m.get("rot")
    if rot is not None and rot["dims"] > 0:
        q = rotate_pairs(q, rot["dims"], rot["base"])
        k = rotate_pairs(k, rot["dims"], rot["base"])
    q = rms_norm(q, None, eps)
    k = rms_norm(k, None, eps)
    mask = m.get("mask")
    chunk = None if not mask else mask.get("size")
    a = chunked_softmax_attention(q, k, v, m["scale"], chunk).reshape(S, H * dv)
    a = a * torch.sigmoid(h @ w[p + "g"].T)
    return a @ w[p + "o"].T


def ssm_scan(x: torch.Tensor, dt: torch.Tensor, a_log: torch.Tensor, B: torch.Tensor,
             C: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    """x [S, Hs, P], dt [S, Hs] (already positive), B and C [S, Gs, N] -> y [S, Hs, P].
    Per head, with its group g = head // (Hs / Gs), a state M [N, P] that starts at zero:
    M <- exp(-exp(a_log) dt_t) M + dt_t B_t x_t^T;  y_t = M^T C_t + D x_t."""
    S, Hs, P = x.shape
    Gs, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for hd in range(Hs):
        g = hd // (Hs // Gs)
        M = torch.zeros((N, P), dtype=x.dtype)
        rate = torch.exp(a_log[hd])
        for t in range(S):
            M = torch.exp(-rate * dt[t, hd]) * M + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = M.T @ C[t, g] + D[hd] * x[t, hd]
    return y


def grouped_rms_norm(y: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis in `groups` equal parts, each divided by its own root mean square; then `weight`."""
    S, C = y.shape
    parts = y.reshape(S, groups, C // groups)
    return rms_norm(parts, None, eps).reshape(S, C) * weight


def mamba2_mixer(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    S = h.shape[0]
    Hs, P, N, Gs = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hs * P
    p = prefix + ".mix."
    proj = h @ w[p + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * Gs * N]
    dt = proj[:, 2 * inner + 2 * Gs * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(S, Hs, P)
    B = xbc[:, inner:inner + Gs * N].reshape(S, Gs, N)
    C = xbc[:, inner + Gs * N:].reshape(S, Gs, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = ssm_scan(x, dt, w[p + "A_log"], B, C, w[p + "D"]).reshape(S, inner)
    y = y * silu(z)
    y = grouped_rms_norm(y, w[p + "norm"], m["norm_groups"], eps)
    return y @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    p = prefix + ".mlp."
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h: torch.Tensor, w: dict, p: str, limit: float) -> torch.Tensor:
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit);
    W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def table_moe_ff(h: torch.Tensor, tokens: torch.Tensor, w: dict, prefix: str, mlp: dict) -> torch.Tensor:
    """Each token id's row of the table names its experts; each counts 1/top.  A shared expert,
    where the layer has one, runs for every token and is added."""
    p = prefix + ".mlp."
    top = mlp["router"]["top"]
    table = w[p + "table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] += clamped_expert(h[t:t + 1], w, f"{p}e{int(e)}.", mlp["expert"]["limit"])[0] / top
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def schedule(cfg: dict) -> list[int]:
    """The order in which layers run: those before `loop.start` once, layers start..stop-1
    `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, w: dict, tokens, dtype=torch.float64, residuals: list | None = None) -> torch.Tensor:
    """Logits [S, vocab] of one sequence from position 0; with `residuals` a list, the residual
    stream after every layer run is appended to it."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    for i in schedule(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        h = rms_norm(x, w[p + ".norm1"], eps)
        if layer["type"] == "attention":
            a = attention_mixer(h, w, p, layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            a = mamba2_mixer(h, w, p, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(a, w[p + ".norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + ".norm2"], eps)
            f = dense_ff(h, w, p) if mlp["kind"] == "dense" else table_moe_ff(h, tokens, w, p, mlp)
            x = x + rms_norm(f, w[p + ".norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits



def greedy(cfg: dict, weights: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every new token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, weights, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
