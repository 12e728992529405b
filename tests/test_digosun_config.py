"""Digosun: reading config.json, what it refuses, the model spec it produces; the plain
implementation against itself where two settings must agree."""

import copy
import json

import pytest
import torch

from somi_inference_b200.config import ConfigError, DigosunConfig, load_config
from somi_inference_b200.parts import declared_tensors
from tests.digosun_tiny import TINY, TINY_P, random_tokens, random_weights, stored_values
from tests.plain import digosun_plain as plain


def test_round_trip_and_registry(tmp_path):
    for raw in TINY.values():
        cfg = DigosunConfig.from_dict(raw)
        assert DigosunConfig.from_dict(cfg.to_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(TINY_P))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, DigosunConfig) and cfg.vocab_size == 131 and cfg.taps == 3


def test_spec_schedule_windows_and_names():
    cfg = DigosunConfig.from_dict(TINY_P)
    spec = cfg.to_model_spec()
    assert [r.cache_of for r in spec.schedule] == [None, 0, None, 2]
    m = [l.mixer.params for l in spec.layers]
    assert [p["window"] for p in m] == [9, 5, None, 21]
    # a cache is kept for the widest window among its readers; without a window, for everything
    assert [p["cache_window"] for p in m] == [9, 9, None, None]
    names = declared_tensors(spec)
    assert "l0.mix.dkv" in names and "l1.mix.dkv" not in names and "l1.mix.dkv.norm" not in names
    assert "l1.mlp.up" not in names and "l1.norm2" not in names and "l1.rg2" not in names
    assert names["l0.canon1"].shape == (48, 3) and names["l2.mix.uv"].shape == (30, 24)
    assert spec.layers[1].feed_forward is None and "feed_forward_gate" not in spec.layers[1].extras


def test_reader_window_longer_than_owner():
    from tests.digosun_tiny import TINY_R
    cfg = DigosunConfig.from_dict(TINY_R)
    assert cfg.cache_window(0) == 70


@pytest.mark.parametrize("change, message", [
    (lambda d: d.pop("vocab"), "lacks"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "keeps no"),
    (lambda d: d["layers"][1]["mixer"].update(kv_rank=48), "kv_rank differs"),
    (lambda d: d["layers"][0].update(type="mystery"), "not a mixer"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["canon"].update(taps=0), "taps"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "size"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(TINY_P)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        DigosunConfig.from_dict(raw)


def test_plain_window_and_sink_limits():
    """A window longer than the sequence is no window; a sink far below every score is no sink
    (plain softmax); a sink far above takes all the weight."""
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(11, 2, 6, generator=g).double(), torch.randn(11, 2, 6, generator=g).double()
    v = torch.randn(11, 2, 5, generator=g).double()
    low = torch.full((2,), -1e4, dtype=torch.float64)
    a = plain.windowed_sink_attention(q, k, v, 0.4, None, low)
    b = plain.windowed_sink_attention(q, k, v, 0.4, 50, low)
    assert torch.equal(a, b)
    s = torch.einsum("ihd,jhd->hij", q, k) * 0.4
    s = s.masked_fill(torch.triu(torch.ones(11, 11, dtype=torch.bool), 1), float("-inf"))
    ref = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v)
    assert torch.allclose(a, ref, atol=1e-12)
    high = torch.full((2,), 50.0, dtype=torch.float64)
    assert plain.windowed_sink_attention(q, k, v, 0.4, None, high).abs().max() < 1e-12
    one = plain.windowed_sink_attention(q, k, v, 0.4, 1, low)       # a token sees only itself
    assert torch.allclose(one, v, atol=1e-12)


def test_plain_prefix_property():
    """Causality of the whole plain model: logits of a prefix do not change when tokens follow."""
    w = stored_values(random_weights(TINY_P, 4))
    toks = random_tokens(30, 131, 1)
    full = plain.forward(TINY_P, w, toks)
    assert torch.allclose(plain.forward(TINY_P, w, toks[:17]), full[:17], atol=1e-10)
