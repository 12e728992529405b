"""Small Digosun configurations for the tests, with random weights that make faults show.

P: sizes that are no multiple of 16, two windows on one shared latent (the reader's shorter than
   the owner's), a layer without a feed-forward, a layer without a window, value width unlike
   the key width, three taps.
Q: one tap (no convolution state), one head, a window of one (a token sees only itself) beside
   a window longer than any test sequence.
R: five taps, a window that spans several pages, the reader's window longer than the owner's
   (the cache must be kept for the longer one), head sizes of 32 and 16.
S: an odd width and latent widths that are no multiple of 4 or 8 (none of the kernels' vector
   paths, the attention kernel on the CUDA cores in bfloat16 too), seven heads, two taps, pages
   of four positions.
"""

from __future__ import annotations

import torch

from somi_inference_b200.config import DigosunConfig
from somi_inference_b200.parts import declared_tensors


def _mixer(heads, dim, vdim, q_rank, kv_rank, scale, window=None, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, ff):
    return {"type": "latent_attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


TINY_P = dict(architecture="Digosun", vocab=131, width=48, norm={"eps": 1e-5}, canon={"taps": 3},
              layers=[_layer(_mixer(3, 12, 20, 20, 40, 0.35, window=9), 72),
                      _layer(_mixer(2, 8, 8, 28, 40, 0.5, window=5, kv_from=0), None),
                      _layer(_mixer(5, 4, 6, 12, 24, 0.6), 40),
                      _layer(_mixer(3, 12, 20, 20, 24, 0.3, window=21, kv_from=2), 56)])
TINY_Q = dict(architecture="Digosun", vocab=67, width=32, norm={"eps": 1e-6}, canon={"taps": 1},
              layers=[_layer(_mixer(1, 16, 16, 8, 16, 0.25, window=1), 32),
                      _layer(_mixer(1, 8, 24, 16, 16, 0.4, window=500, kv_from=0), 48),
                      _layer(_mixer(2, 16, 8, 16, 8, 0.3, window=2), 16)])
TINY_R = dict(architecture="Digosun", vocab=257, width=96, norm={"eps": 1e-6}, canon={"taps": 5},
              layers=[_layer(_mixer(4, 32, 16, 48, 64, 0.2, window=33), 160),
                      _layer(_mixer(2, 16, 32, 32, 64, 0.3, window=70, kv_from=0), 96),
                      _layer(_mixer(6, 16, 16, 24, 80, 0.25, window=16), None)])
TINY_S = dict(architecture="Digosun", vocab=90, width=45, norm={"eps": 1e-4}, canon={"taps": 2},
              layers=[_layer(_mixer(7, 6, 10, 9, 20, 0.45, window=12), 33),
                      _layer(_mixer(1, 5, 3, 7, 20, 0.7, window=12, kv_from=0), 21),
                      _layer(_mixer(2, 10, 2, 11, 12, 0.4), 50)])
TINY = {"P": TINY_P, "Q": TINY_Q, "R": TINY_R, "S": TINY_S}
PAGE_SIZES = {"P": 8, "Q": 16, "R": 16, "S": 4}


def random_weights(raw: dict, seed: int, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Tensors for `raw`, by name: matrices spread widely enough that attention is peaked and a
    wrong key or mask moves the logits; norm weights around one; sinks, gate biases, activation
    numbers and taps of order one."""
    g = torch.Generator().manual_seed(seed)
    cfg = DigosunConfig.from_dict(raw)
    out = {}
    for name, decl in declared_tensors(cfg.to_model_spec()).items():
        shape = tuple(decl.shape)
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".sink"):
            t = 1.5 * torch.randn(shape, generator=g)
        elif name.endswith(".act"):
            t = torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif "canon" in name:
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.6 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def stored_values(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The weights as float64, exactly the values that were stored."""
    return {k: v.double() for k, v in weights.items()}


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
