"""Typed configuration of the Dapozen architecture: a decoder that interleaves attention layers
(short convolutions on q, k and v, pair rotation on part of the head, unit-norm queries and
keys, a chunked mask, a sigmoid output gate) with Mamba-2 layers, every branch between two RMS
norms, feed-forwards that are dense (SwiGLU) or a table-routed mixture of experts, and a block of
layers that may run several times in a row with the same weights.

config.json gives `architecture`, `vocab`, `width`, `norm.eps`, `embedding.scale`,
`logit_softcap`, optionally `loop` = {start, stop, times} and `layers`: per layer `type`
("attention" or "mamba2"), `mixer` (its sizes) and `mlp` (null, {"kind": "dense", "ff"} or
{"kind": "moe", "expert": {ff, limit}, "router": {experts, top}, "shared": {ff, limit} | absent}).
Attention: `heads`, `kv_heads`, `dim`, `vdim`, `conv` (taps), `rot` = {dims, base}, `scale`,
`mask.size` (the chunk).  Mamba-2: `heads`, `vdim`, `state`, `groups`, `norm_groups`, `conv`.
What the design fixes (the experts' activation constant, interleaved rotation pairs, softmax, the
gate, biases on q, k, v only) is stated here.

Tensor names: `embed`, `final.norm`, `head`; per layer `l<i>.`: `norm1`, `norm1b`, `norm2`,
`norm2b`; attention `mix.{q,k,v}` with `.b` and `.conv`, `mix.g`, `mix.o`; Mamba-2
`mix.{in, conv, conv.b, dt_bias, A_log, D, norm, o}`; `mlp.{gate,up,down}` (dense) or
`mlp.table`, `mlp.e<j>.{gate,up,down}`, `mlp.shared.{gate,up,down}`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any

from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

ARCHITECTURE = "Dapozen"
EXPERT_ACTIVATION_ALPHA = 1.702   # fixed by the design: g * sigmoid(1.702 g) * (u + 1)
DEFAULT_MAX_POSITIONS = 1 << 20   # positions are computed, not learned: a bound for tables only


def _int(d: dict, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"config.json: {where}{key} must be an integer >= {least}, got {v!r}")
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"config.json: {where}{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class DapozenLayerConfig:
    type: str                    # "attention" | "mamba2"
    mixer: dict[str, Any]        # the mixer's sizes, as the file gives them (validated)
    mlp: dict[str, Any] | None   # None: the layer has no feed-forward


@dataclass(frozen=True)
class DapozenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float | None
    layers: tuple[DapozenLayerConfig, ...]
    loop: tuple[int, int, int] | None = None      # (start, stop, times)
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
    @staticmethod
    def _mixer(kind: str, m: Any, where: str) -> dict[str, Any]:
        if not isinstance(m, dict):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        w = where + "mixer."
        if kind == "attention":
            out: dict[str, Any] = {k: _int(m, k, w) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            out["scale"] = _number(m, "scale", w)
            if out["heads"] % out["kv_heads"]:
                raise ConfigError(f"config.json: {w}heads must be a multiple of kv_heads")
            rot = m.get("rot")
            if rot is not None:
                out["rot"] = {"dims": _int(rot, "dims", w + "rot.", 0), "base": _number(rot, "base", w + "rot.")}
                if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
                    raise ConfigError(f"config.json: {w}rot.dims must be even and at most dim")
            mask = m.get("mask")
            if mask is not None:
                out["mask"] = {"size": _int(mask, "size", w + "mask.")}
            return out
        out = {k: _int(m, k, w) for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"config.json: {w}heads must be a multiple of groups")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"config.json: {w}heads * vdim must be a multiple of norm_groups")
        return out

    @staticmethod
    def _mlp(mlp: Any, where: str) -> dict[str, Any] | None:
        if mlp is None:
            return None
        w = where + "mlp."
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense' or 'moe'")
        if mlp["kind"] == "dense":
            return {"kind": "dense", "ff": _int(mlp, "ff", w)}
        out: dict[str, Any] = {"kind": "moe"}
        for part in ("expert", "shared"):
            if part == "shared" and mlp.get("shared") is None:
                continue
            out[part] = {"ff": _int(mlp.get(part), "ff", f"{w}{part}."),
                         "limit": _number(mlp.get(part), "limit", f"{w}{part}.")}
        out["router"] = {"experts": _int(mlp.get("router"), "experts", w + "router."),
                         "top": _int(mlp.get("router"), "top", w + "router.")}
        if out["router"]["top"] > out["router"]["experts"]:
            raise ConfigError(f"config.json: {w}router.top exceeds router.experts")
        return out

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "DapozenConfig":
        missing = [k for k in ("vocab", "width", "norm", "embedding", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(raw, dict) or "type" not in raw or "mixer" not in raw:
                raise ConfigError(f"config.json: {where[:-1]} needs 'type' and 'mixer'")
            if raw["type"] not in ("attention", "mamba2"):
                raise ConfigError(f"config.json: {where}type {raw['type']!r} is not a mixer of this "
                                  "architecture (known: 'attention', 'mamba2')")
            layers.append(DapozenLayerConfig(raw["type"], cls._mixer(raw["type"], raw["mixer"], where),
                                             cls._mlp(raw.get("mlp"), where)))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_int(lp, "start", "loop.", 0), _int(lp, "stop", "loop.", 0), _int(lp, "times", "loop."))
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_number(d["norm"], "eps", "norm."),
                  embedding_scale=_number(d["embedding"], "scale", "embedding."),
                  logit_softcap=None if cap is None else _number(d, "logit_softcap", ""),
                  layers=tuple(layers), loop=loop,
                  max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "DapozenConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": json.loads(json.dumps(l.mixer)),
                        "mlp": None if l.mlp is None else json.loads(json.dumps(l.mlp))}
                       for l in self.layers]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
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
        if self.logit_softcap is not None and not self.logit_softcap > 0.0:
            raise ConfigError("logit_softcap must be positive")
        if self.loop is not None:
            start, stop, _ = self.loop
            if not 0 <= start <= stop <= len(self.layers):
                raise ConfigError(f"loop {start}..{stop} does not lie within the {len(self.layers)} layers")

    # ------------------------------------------------------------ model spec
    def layer_order(self) -> list[int]:
        """Layers before the loop once, the looped layers `times` times in a row, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": D, "eps": eps, "names": {"weight": name}})

        layers = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer.mixer
            if layer.type == "attention":
                names = {"o_weight": f"{p}.mix.o", "gate_weight": f"{p}.mix.g"}
                for part in ("q", "k", "v"):
                    names.update({f"{part}_weight": f"{p}.mix.{part}", f"{part}_bias": f"{p}.mix.{part}.b",
                                  f"{part}_taps": f"{p}.mix.{part}.conv"})
                mask = m.get("mask")
                mixer = PartSpec("conv_attention", {
                    "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                    "key_dim": m["dim"], "value_dim": m["vdim"], "scale": m["scale"],
                    "taps": m["conv"], "qkv_bias": True, "gate": True, "unit_norm": True, "eps": eps,
                    "rotary": m.get("rot"),
                    "mask": None if mask is None else {"kind": "chunk", "size": mask["size"]},
                    "names": names})
            else:
                mixer = PartSpec("mamba2", {
                    "hidden_size": D, "heads": m["heads"], "head_dim": m["vdim"],
                    "state_size": m["state"], "groups": m["groups"], "norm_groups": m["norm_groups"],
                    "taps": m["conv"], "eps": eps,
                    "names": {"in_weight": f"{p}.mix.in", "taps": f"{p}.mix.conv",
                              "taps_bias": f"{p}.mix.conv.b", "dt_bias": f"{p}.mix.dt_bias",
                              "a_log": f"{p}.mix.A_log", "skip": f"{p}.mix.D",
                              "norm": f"{p}.mix.norm", "o_weight": f"{p}.mix.o"}})
            norms = {"mixer": norm(f"{p}.norm1"), "mixer_post": norm(f"{p}.norm1b")}
            ff, mlp = None, layer.mlp
            if mlp is not None:
                norms.update(feed_forward=norm(f"{p}.norm2"), feed_forward_post=norm(f"{p}.norm2b"))
                if mlp["kind"] == "dense":
                    ff = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": mlp["ff"],
                                             "names": {"gate_weight": f"{p}.mlp.gate",
                                                       "up_weight": f"{p}.mlp.up",
                                                       "down_weight": f"{p}.mlp.down"}})
                else:
                    E = mlp["router"]["experts"]
                    names = {"table": f"{p}.mlp.table",
                             "gate": [f"{p}.mlp.e{e}.gate" for e in range(E)],
                             "up": [f"{p}.mlp.e{e}.up" for e in range(E)],
                             "down": [f"{p}.mlp.e{e}.down" for e in range(E)],
                             "shared_gate": f"{p}.mlp.shared.gate", "shared_up": f"{p}.mlp.shared.up",
                             "shared_down": f"{p}.mlp.shared.down"}
                    ff = PartSpec("table_moe", {
                        "hidden_size": D, "vocab_size": self.vocab, "experts": E,
                        "top": mlp["router"]["top"], "expert_ff": mlp["expert"]["ff"],
                        "limit": mlp["expert"]["limit"], "alpha": EXPERT_ACTIVATION_ALPHA,
                        "shared": mlp.get("shared"), "names": names})
            layers.append(LayerSpec(prefix=p, mixer=mixer, feed_forward=ff, norms=norms,
                                    arrangement="sandwich_norm"))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=D, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D,
                                                   "scale": self.embedding_scale,
                                                   "names": {"weight": "embed"}}),
            layers=tuple(layers),
            # every run of a looped layer keeps a cache and a state of its own
            schedule=tuple(RunSpec(i) for i in self.layer_order()),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied": False,
                                      "softcap": self.logit_softcap,
                                      "names": {"weight": "head", "tied_to": "embed"}}))
        spec.validate()
        return spec
