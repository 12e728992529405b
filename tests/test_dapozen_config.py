"""Dapozen: reading config.json, what it refuses, the model spec it produces (the loop as a
schedule, cache and state needs); the plain implementation against itself where two settings
must agree."""

import copy
import json

import pytest
import torch

from somi_inference_b200.config import ConfigError, DapozenConfig, load_config
from somi_inference_b200.parts import declared_tensors
from somi_inference_b200.weights.random_init import random_tensors
from tests.dapozen_tiny import TINY, TINY_A, TINY_B, random_tokens, random_weights, stored_values
from tests.plain import dapozen_plain as plain


def test_round_trip_and_registry(tmp_path):
    for raw in TINY.values():
        cfg = DapozenConfig.from_dict(raw)
        assert DapozenConfig.from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, DapozenConfig) and cfg.vocab_size == 131 and cfg.loop == (1, 3, 2)


def test_spec_schedule_parts_and_names():
    cfg = DapozenConfig.from_dict(TINY_A)
    spec = cfg.to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert all(r.cache_of is None for r in spec.schedule)         # every run has a cache of its own
    assert [l.mixer.kind for l in spec.layers] == ["conv_attention", "mamba2", "conv_attention", "mamba2"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["swiglu", "table_moe", None, "table_moe"]
    assert set(spec.layers[2].norms) == {"mixer", "mixer_post"}
    assert spec.layers[0].mixer.params["mask"] == {"kind": "chunk", "size": 9}
    assert spec.embedding.params["scale"] == 3.0 and spec.head.params["softcap"] == 20.0
    names = declared_tensors(spec)
    assert names["l0.mix.q"].shape == (48, 48) and names["l0.mix.v"].shape == (40, 48)
    assert names["l0.mix.k.conv"].shape == (24, 3) and names["l0.mix.g"].shape == (80, 48)
    assert names["l1.mix.in"].shape == (2 * 30 + 2 * 12 + 3, 48) and names["l1.mix.conv"].shape == (54, 4)
    assert names["l1.mlp.table"].shape == (131, 2) and names["l1.mlp.e4.down"].shape == (48, 24)
    assert "l3.mlp.shared.up" not in names and "l2.norm2" not in names and "l2.mlp.gate" not in names
    no_loop = DapozenConfig.from_dict(TINY_B)
    assert no_loop.layer_order() == [0, 1, 2, 3] and no_loop.logit_softcap is None


def test_random_tables_name_distinct_experts():
    w = random_tensors(DapozenConfig.from_dict(TINY_A), 5)
    t = w["l1.mlp.table"]
    assert t.dtype == torch.int32 and t.shape == (131, 2) and int(t.min()) >= 0 and int(t.max()) < 5
    assert (t[:, 0] != t[:, 1]).all()


@pytest.mark.parametrize("change, message", [
    (lambda d: d.pop("vocab"), "lacks"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d["embedding"].pop("scale"), "embedding.scale"),
    (lambda d: d["layers"][0].update(type="mystery"), "not a mixer"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][1]["mixer"].update(groups=2), "multiple of groups"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=4), "norm_groups"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d.update(logit_softcap=0.0), "softcap"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(TINY_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        DapozenConfig.from_dict(raw)


def test_plain_chunks_and_limits():
    """A chunk longer than the sequence is plain causal attention; a chunk of one returns the
    token's own value; a token at a chunk's start sees only itself."""
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(11, 4, 6, generator=g).double(), torch.randn(11, 2, 6, generator=g).double()
    v = torch.randn(11, 2, 5, generator=g).double()
    a = plain.chunked_softmax_attention(q, k, v, 0.4, None)
    assert torch.equal(a, plain.chunked_softmax_attention(q, k, v, 0.4, 50))
    kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * 0.4
    s = s.masked_fill(torch.triu(torch.ones(11, 11, dtype=torch.bool), 1), float("-inf"))
    assert torch.allclose(a, torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vv), atol=1e-12)
    assert torch.allclose(plain.chunked_softmax_attention(q, k, v, 0.4, 1), vv, atol=1e-12)
    four = plain.chunked_softmax_attention(q, k, v, 0.4, 4)
    assert torch.allclose(four[[0, 4, 8]], vv[[0, 4, 8]], atol=1e-12)
    assert not torch.allclose(four[5], a[5])


def test_plain_recurrence_by_hand():
    """Two steps of a one-head recurrence, written out."""
    x = torch.tensor([[[1.0, 2.0]], [[3.0, -1.0]]], dtype=torch.float64)
    dt = torch.tensor([[0.5], [2.0]], dtype=torch.float64)
    B = torch.tensor([[[1.0, 0.0, 2.0]], [[0.0, 1.0, 1.0]]], dtype=torch.float64)
    C = torch.tensor([[[1.0, 1.0, 1.0]], [[2.0, 0.0, -1.0]]], dtype=torch.float64)
    a_log, D = torch.tensor([0.0], dtype=torch.float64), torch.tensor([0.25], dtype=torch.float64)
    y = plain.ssm_scan(x, dt, a_log, B, C, D)
    m1 = 0.5 * torch.outer(B[0, 0], x[0, 0])
    m2 = torch.exp(torch.tensor(-2.0, dtype=torch.float64)) * m1 + 2.0 * torch.outer(B[1, 0], x[1, 0])
    assert torch.allclose(y[0, 0], m1.T @ C[0, 0] + 0.25 * x[0, 0])
    assert torch.allclose(y[1, 0], m2.T @ C[1, 0] + 0.25 * x[1, 0])


def test_plain_prefix_property():
    """Causality of the whole plain model: logits of a prefix do not change when tokens follow."""
    w = stored_values(random_weights(TINY_A, 4))
    toks = random_tokens(30, 131, 1)
    full = plain.forward(TINY_A, w, toks)
    assert torch.allclose(plain.forward(TINY_A, w, toks[:17]), full[:17], atol=1e-10)
    assert full.abs().max() <= 20.0          # the cap bounds every logit
