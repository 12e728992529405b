"""Digosun through the engine, against the plain implementation, under every way of cutting the
work: whole prompts; most of a prompt and then token by token; portions of changing size down to
two tokens; up to four live requests in one batch with so few pages and slots that both are
used again; long decoding past every window; greedy generation through `LLM` and the command
line.  float32 and bfloat16, three small configurations (tests/digosun_tiny.py)."""

import json
import os

import pytest
import torch

from somi_inference_b200.config import DigosunConfig
from somi_inference_b200.weights.safetensors_io import save_safetensors
from tests import replay
from tests.digosun_tiny import PAGE_SIZES, TINY, random_tokens, random_weights, stored_values
from tests.plain import digosun_plain as plain

pytestmark = pytest.mark.gpu

LENGTHS = {"P": [5, 97, 40, 70, 1, 33, 100, 64, 81, 2], "Q": [3, 50, 17, 64, 1, 30],
           "R": [150, 5, 129, 71, 200, 16, 90], "S": [30, 1, 77, 12, 13, 45]}
# float32: logits are of size 5-20 here; bfloat16: every activation between two kernels is
# rounded to 8 bits.  A wrong key, a window that is off by one or a lost state moves a logit by
# its own size.
ATOL = {"float32": lambda s: 4e-5 * max(1.0, s), "bfloat16": lambda s: 6e-2 * s}
RMS = {"float32": lambda s: 1e-5 * max(1.0, s), "bfloat16": lambda s: 8e-3 * s}
MODES = {"whole": replay.whole, "last32": replay.last_one_by_one, "portions": replay.portions,
         "mixed": replay.mixed}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("digosun")
    out = {}
    for k, (name, raw) in enumerate(TINY.items()):
        for dt in (torch.float32, torch.bfloat16):
            d = str(root / f"{name}_{str(dt).split('.')[-1]}")
            os.makedirs(d)
            w = random_weights(raw, 20 + k, dt)
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(raw, f)
            save_safetensors(w, os.path.join(d, "model.safetensors"))
            reqs = {f"r{i}": random_tokens(n, raw["vocab"], 50 + i) for i, n in enumerate(LENGTHS[name])}
            ref = {rid: plain.forward(raw, stored_values(w), toks) for rid, toks in reqs.items()}
            scale = max(v.abs().max().item() for v in ref.values())
            out[(name, str(dt).split(".")[-1])] = (d, raw, w, reqs, ref, scale)
    return out


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_in_process(models, name, dtype, mode):
    from somi_inference_b200.engine import Engine
    d, raw, w, reqs, ref, scale = models[(name, dtype)]
    steps, max_tokens = MODES[mode](reqs)
    eng = Engine(d, dtype=dtype, page_size=PAGE_SIZES[name], max_tokens=max_tokens, max_requests=4)
    got = replay.run_steps(eng, steps)
    eng.ops.check_errors()
    assert len(got) >= len(reqs)
    replay.compare(got, ref, ATOL[dtype](scale), f"{name}/{dtype}/{mode}", RMS[dtype](scale))
    assert all(f == eng.num_pages for f in eng.cache.free_pages()), "pages were lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(models, tmp_path, dtype):
    d, raw, w, reqs, ref, scale = models[("P", dtype)]
    for mode in ("mixed", "last32"):
        steps, max_tokens = MODES[mode](reqs)
        got = replay.run_trace_program(d, dtype, steps, max_tokens, str(tmp_path / mode), raw["vocab"])
        replay.compare(got, ref, ATOL[dtype](scale), f"trace_run P/{dtype}/{mode}", RMS[dtype](scale))


def test_cut_independence_float32(models):
    """The same position whole, token by token and in portions: equal beyond rounding, and the
    first tokens of a sequence (before any window or convolution is full) among them."""
    from somi_inference_b200.engine import Engine
    d, raw, w, reqs, ref, scale = models[("R", "float32")]
    sub = {"r0": reqs["r0"], "r1": reqs["r1"]}
    outs = []
    for mode in ("whole", "last32", "portions"):
        steps, mt = MODES[mode](sub)
        eng = Engine(d, dtype="float32", page_size=16, max_tokens=mt, max_requests=4)
        outs.append(replay.run_steps(eng, steps))
    for key in outs[0]:
        for o in outs[1:]:
            assert (outs[0][key] - o[key]).abs().max().item() < 2e-5 * max(1.0, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_in_a_small_pool(models, dtype):
    """Token by token from the first token on, far past every window, two requests side by side
    in a pool that holds a fraction of their length: the windowed caches give pages back as
    they go and take them again."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, raw, w, reqs, ref, scale = models[("Q", dtype)]      # every cache of Q has a window <= 500
    raw2 = TINY["R"]
    d2, _, w2, _, _, _ = models[("R", dtype)]
    toks = {"x": random_tokens(260, raw2["vocab"], 1), "y": random_tokens(190, raw2["vocab"], 2)}
    want = {k: plain.forward(raw2, stored_values(w2), v) for k, v in toks.items()}
    s2 = max(v.abs().max().item() for v in want.values())
    # R's caches are kept for 70 and 16 positions: 2 requests * (70 + 16 + 16) tokens, with room to spare
    eng = Engine(d2, dtype=dtype, page_size=16, num_pages=14, max_requests=2)
    got = {}
    for i in range(260):
        entries = [StepEntry(k, [v[i]], [0]) for k, v in toks.items() if i < len(v)]
        logits = eng.step(entries).float().cpu()
        for e, row in zip(entries, logits):
            got[(e.request, i)] = row
        for k, v in toks.items():
            if i == len(v) - 1:
                eng.end(k)
        eng.cache.check_consistency()
    eng.ops.check_errors()
    replay.compare(got, want, ATOL[dtype](s2), f"long decoding/{dtype}", RMS[dtype](s2))
    assert all(f == 14 for f in eng.cache.free_pages())


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_llm(models, name):
    """Greedy continuations through the scheduler (prompts in portions, several requests at once)
    equal the plain model's, which recomputes the whole sequence for every token."""
    from somi_inference_b200.engine import LLM
    from somi_inference_b200.sampling import SamplingParams
    d, raw, w, reqs, ref, scale = models[(name, "float32")]
    prompts = [random_tokens(n, raw["vocab"], 90 + n) for n in (3, 41, 18, 1, 66)]
    llm = LLM(d, num_blocks=64, block_size=PAGE_SIZES[name], dtype="float32", max_concurrent=3,
              chunk_size=16, max_num_batched_tokens=40)
    outs = llm.generate_many(prompts, max_new_tokens=12,
                             sampling_params=[SamplingParams(temperature=0.0)] * len(prompts),
                             ignore_eos=True)
    for p, o in zip(prompts, outs):
        assert list(o) == plain.greedy(raw, stored_values(w), p, 12), len(p)


def test_command_line_from_config_and_seed(tmp_path, capsys):
    from somi_inference_b200.entrypoints.generate import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY["P"]))
    rc = main(["--config", str(cfg), "--random-weights", "--seed", "3", "--prompt-lens", "4", "19",
               "--max-new-tokens", "5", "--temperature", "0", "--dtype", "float32", "--std", "0.2"])
    assert rc == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert [r["prompt_len"] for r in lines] == [4, 19] and all(len(r["output_ids"]) == 5 for r in lines)
    # the same weights written to a folder and read back give the same tokens
    folder = tmp_path / "model"
    assert main(["--write-random-model", str(folder), "--config", str(cfg), "--seed", "3",
                 "--std", "0.2"]) == 0
    capsys.readouterr()
    assert DigosunConfig.from_json(str(folder)).to_dict() == DigosunConfig.from_dict(TINY["P"]).to_dict()
