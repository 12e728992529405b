"""Typed configuration of the Digosun architecture: a decoder whose layers mix by latent
attention under a sliding window, with gated residual branches and a short causal convolution
in front of every mixer.

config.json names the architecture under `architecture` and gives `vocab`, `width`, `norm.eps`,
`canon.taps` (the convolution's length) and `layers`: per layer `type` (the mixer kind),
`mixer` (its sizes) and `mlp` (`{"kind": "dense", "ff": n}`, or null for a layer without a
feed-forward).  A `latent_attention` mixer gives `heads`, `dim` (query/key width per head), `vdim`
(value width per head), `q_rank` and `kv_rank` (widths of the two latents), `scale` (the factor on
q.k), `mask.size` (how many positions a token sees, itself included; no mask: all earlier ones)
and optionally `kv_from`: the index of an earlier layer whose cached key/value latent this layer
reads instead of making its own.  Every size comes from the file; the design's fixed constants
(the sinusoid's base, the sink in every softmax, biases in the feed-forward only) are stated here.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer `l<i>.`: `norm1`,
`norm2`, `canon1` [width, taps], `rg1` / `rg1.b` and `rg2` / `rg2.b` (gates of the two
branches), `mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o}`, `mlp.{up, up.b, down, down.b,
act}`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any

from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

ARCHITECTURE = "Digosun"
SINUSOID_BASE = 10000.0          # fixed by the design
DEFAULT_MAX_POSITIONS = 1 << 20  # positions are computed, not learned: a bound for tables only


def _positive_int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None
    kv_from: int | None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "LatentAttentionConfig":
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        if "scale" not in d:
            raise ConfigError(f"config.json: {where}mixer lacks scale")
        mask = d.get("mask")
        window = None
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"config.json: {where}mixer.mask must be an object or null")
            if mask.get("size") is not None:
                window = _positive_int(mask, "size", where + "mixer.mask.")
        kv_from = d.get("kv_from")
        if kv_from is not None and (not isinstance(kv_from, int) or isinstance(kv_from, bool)):
            raise ConfigError(f"config.json: {where}mixer.kv_from must be a layer index")
        return cls(heads=_positive_int(d, "heads", where + "mixer."),
                   dim=_positive_int(d, "dim", where + "mixer."),
                   vdim=_positive_int(d, "vdim", where + "mixer."),
                   q_rank=_positive_int(d, "q_rank", where + "mixer."),
                   kv_rank=_positive_int(d, "kv_rank", where + "mixer."),
                   scale=float(d["scale"]), window=window, kv_from=kv_from)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim,
                             "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DigosunLayerConfig:
    mixer_type: str
    mixer: LatentAttentionConfig
    ff: int | None               # None: the layer has no feed-forward


@dataclass(frozen=True)
class DigosunConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int
    layers: tuple[DigosunLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int | None = None

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "DigosunConfig":
        missing = [k for k in ("vocab", "width", "norm", "canon", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        norm, canon = d["norm"], d["canon"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json lacks: norm.eps")
        if not isinstance(canon, dict):
            raise ConfigError("config.json lacks: canon.taps")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(raw, dict) or "type" not in raw or "mixer" not in raw:
                raise ConfigError(f"config.json: {where[:-1]} needs 'type' and 'mixer'")
            if raw["type"] != "latent_attention":
                raise ConfigError(f"config.json: {where}type {raw['type']!r} is not a mixer of this "
                                  "architecture (known: 'latent_attention')")
            mlp = raw.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense'")
                ff = _positive_int(mlp, "ff", where + "mlp.")
            layers.append(DigosunLayerConfig(raw["type"],
                                             LatentAttentionConfig.from_dict(raw["mixer"], where), ff))
        cfg = cls(vocab=_positive_int(d, "vocab", ""), width=_positive_int(d, "width", ""),
                  norm_eps=float(norm["eps"]), taps=_positive_int(canon, "taps", "canon."),
                  layers=tuple(layers),
                  max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "DigosunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "canon": {"taps": self.taps},
            "layers": [{"type": l.mixer_type, "mixer": l.mixer.to_dict(),
                        "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}}
                       for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------- validation
    def validate(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError("norm.eps must be positive")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")
        for i, layer in enumerate(self.layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i:
                raise ConfigError(f"layers[{i}].mixer.kv_from = {j} must name an earlier layer")
            src = self.layers[j].mixer
            if src.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from = {j}, but layer {j} keeps no "
                                  "key/value latent of its own")
            if src.kv_rank != layer.mixer.kv_rank:
                raise ConfigError(f"layers[{i}] reads layer {j}'s latent but kv_rank differs "
                                  f"({layer.mixer.kv_rank} against {src.kv_rank})")

    # ------------------------------------------------------------ model spec
    def cache_window(self, layer: int) -> int | None:
        """How far back the cache of `layer` (which keeps its own latent) must reach: the
        widest window among the layer itself and the layers that read its latent."""
        windows = [self.layers[layer].mixer.window]
        windows += [l.mixer.window for l in self.layers if l.mixer.kv_from == layer]
        return None if any(w is None for w in windows) else max(windows)

    def to_model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("layernorm", {"size": D, "eps": eps, "names": {"weight": name}})

        def gate(p: str) -> PartSpec:
            return PartSpec("sigmoid_gate", {"in_features": D, "out_features": D,
                                             "names": {"weight": p, "bias": f"{p}.b"}})
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer.mixer
            owner = i if m.kv_from is None else m.kv_from
            names = {k: f"{p}.mix.{v}" for k, v in (
                ("q_down", "dq"), ("q_norm", "dq.norm"), ("q_up", "uq"), ("k_up", "uk"),
                ("v_up", "uv"), ("sink", "sink"), ("out", "o"))}
            if m.kv_from is None:
                names.update(kv_down=f"{p}.mix.dkv", kv_norm=f"{p}.mix.dkv.norm")
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window,
                "cache_window": self.cache_window(owner), "own_latent": m.kv_from is None,
                "sink": True, "eps": eps, "names": names})
            ff = None
            norms = {"mixer": norm(f"{p}.norm1")}
            extras = {"mixer_gate": gate(f"{p}.rg1"),
                      "mixer_taps": PartSpec("causal_taps", {"channels": D, "taps": self.taps,
                                                             "names": {"weight": f"{p}.canon1"}})}
            if layer.ff is not None:
                ff = PartSpec("dense_ff", {"hidden_size": D, "intermediate_size": layer.ff,
                                           "activation": "xielu", "bias": True,
                                           "names": {"up": f"{p}.mlp.up", "up_bias": f"{p}.mlp.up.b",
                                                     "down": f"{p}.mlp.down",
                                                     "down_bias": f"{p}.mlp.down.b",
                                                     "act": f"{p}.mlp.act"}})
                norms["feed_forward"] = norm(f"{p}.norm2")
                extras["feed_forward_gate"] = gate(f"{p}.rg2")
            layers.append(LayerSpec(prefix=p, mixer=mixer, feed_forward=ff, norms=norms,
                                    arrangement="gated_pre_norm", extras=extras))
            schedule.append(RunSpec(i, cache_of=m.kv_from))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=D, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("sinusoid_embedding", {
                "vocab_size": self.vocab, "hidden_size": D, "base": SINUSOID_BASE,
                "norm": norm("embed.norm"), "names": {"weight": "embed"}}),
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied": False,
                                      "names": {"weight": "head", "tied_to": "embed"}}))
        spec.validate()
        return spec
