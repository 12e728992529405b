"""Small Dapozen configurations for the tests, with random weights that make faults show.

A: a loop of two layers run twice, grouped key/value heads, values wider than keys, rotation on
   part of the head, two experts per token with a shared expert, a layer without a feed-forward,
   state sizes above one warp's width, chunks (9, 21) that are no multiple of the page (8).
B: an odd width, one head everywhere, key and value widths that are no multiple of 2 or 4, one tap
   (no convolution state), no rotation, a chunk of one (a token sees only itself) beside a chunk
   longer than any test sequence, no loop, no soft cap, one norm group over everything.
C: keys and values of equal width (one cache tensor), a chunk of 64 over pages of 16, a loop run
   three times, three of eight experts, five taps, rotation on the whole head.
D: head sizes of 64 and 128, which the tensor-core attention kernels take in bfloat16, under
   chunks (48, 200) that are no multiple of a key tile, a page or a query tile.
"""

from __future__ import annotations

import torch

from somi_inference_b200.config import DapozenConfig
from somi_inference_b200.parts import declared_tensors


def attention(heads, kv_heads, dim, vdim, conv, scale, chunk, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=scale,
             mask={"size": chunk})
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def mamba(heads, vdim, state, groups, norm_groups, conv):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


TINY_A = dict(architecture="Dapozen", vocab=131, width=48, norm={"eps": 1e-5}, embedding={"scale": 3.0},
              logit_softcap=20.0, loop={"start": 1, "stop": 3, "times": 2},
              layers=[layer("attention", attention(4, 2, 12, 20, 3, 0.9, 9, rot=(8, 10000.0)), dense(72)),
                      layer("mamba2", mamba(3, 10, 12, 1, 3, 4), moe(5, 2, 24, 1.5, shared=(16, 3.0))),
                      layer("attention", attention(2, 1, 16, 8, 2, 0.7, 21, rot=(16, 500.0)), None),
                      layer("mamba2", mamba(4, 6, 40, 2, 1, 2), moe(3, 1, 20, 2.5))])
TINY_B = dict(architecture="Dapozen", vocab=67, width=45, norm={"eps": 1e-4}, embedding={"scale": 1.0},
              layers=[layer("attention", attention(1, 1, 5, 3, 1, 1.2, 1), dense(33)),
                      layer("mamba2", mamba(1, 5, 70, 1, 1, 1), None),
                      layer("attention", attention(3, 3, 10, 6, 1, 0.8, 500), moe(2, 2, 9, 0.7)),
                      layer("mamba2", mamba(2, 7, 3, 2, 2, 3), dense(21))])
TINY_C = dict(architecture="Dapozen", vocab=257, width=96, norm={"eps": 1e-6}, embedding={"scale": 7.5},
              logit_softcap=8.0, loop={"start": 0, "stop": 2, "times": 3},
              layers=[layer("mamba2", mamba(8, 8, 16, 4, 2, 5), moe(8, 3, 32, 1.0, shared=(48, 1.0))),
                      layer("attention", attention(4, 2, 32, 32, 5, 0.5, 64, rot=(32, 1e6)), dense(160)),
                      layer("attention", attention(6, 6, 16, 24, 2, 0.75, 16, rot=(4, 100.0)), moe(4, 1, 40, 4.0))])
TINY_D = dict(architecture="Dapozen", vocab=300, width=128, norm={"eps": 1e-6}, embedding={"scale": 2.0},
              logit_softcap=15.0,
              layers=[layer("attention", attention(4, 2, 64, 64, 2, 0.3, 48, rot=(32, 1e4)), dense(256)),
                      layer("mamba2", mamba(4, 16, 32, 2, 2, 4), moe(4, 2, 64, 2.0)),
                      layer("attention", attention(2, 1, 128, 128, 3, 0.2, 200, rot=(128, 1e4)), dense(192))])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZES = {"A": 8, "B": 4, "C": 16, "D": 16}


def random_weights(raw: dict, seed: int, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Tensors for `raw`, by name: matrices spread widely enough that attention is peaked and the
    recurrence forgets at a visible rate; norm weights around one; biases, taps, step biases and
    decay rates of order one; every row of a routing table names distinct experts."""
    g = torch.Generator().manual_seed(seed)
    cfg = DapozenConfig.from_dict(raw)
    out = {}
    for name, decl in declared_tensors(cfg.to_model_spec()).items():
        shape = tuple(decl.shape)
        last = name.split(".")[-1]
        if last == "table":
            n = int(decl.init.split(":")[1])
            rows = [torch.randperm(n, generator=g)[:shape[1]] for _ in range(shape[0])]
            out[name] = torch.stack(rows).to(torch.int32)
            continue
        if last.startswith("norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("b", "dt_bias", "D"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "A_log":
            t = 0.7 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.6 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def stored_values(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The weights as float64 (integer tables as they are), exactly the values that were stored."""
    return {k: (v.double() if v.is_floating_point() else v) for k, v in weights.items()}


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
