"""Rirusun on the GPU against the plain implementation (``plain_rirusun``): each mechanism alone, then whole models of
several made-up shapes stepped through the engine under every cutting, and generation through the scheduler.

The models' weights are drawn here, larger than a trained model's and with the attention sharpened, so that a key that is
wrongly seen or missed at a window's edge, a kept first token, a sink or a distance bias that is left out, a state or a
convolution input that is lost and a wrong expert all move the logits by much more than the tolerance."""
from __future__ import annotations

import json
import math

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_rirusun as plain
import trace_tools
from test_parts_gpu import step_view
from test_zemavik_gpu import assert_logits, engine_for, fresh_cache, make_requests, on, paged, run_part

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


# ---------------------------------------------------------------------------------------
# made-up models
# ---------------------------------------------------------------------------------------
def moe(ff, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def parallel_layer(left, bias, mask, right, scales, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale); bias: (rows, far); mask: (size, keep_first) or None; right: (width, blocks, taps)."""
    attention = dict(zip(("heads", "kv_heads", "dim", "vdim", "scale"), left), bias_max=bias[1], bias_rows=bias[0])
    if mask is not None:
        attention["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return {"type": "parallel", "mixer": {"left": attention, "left_scale": scales[0], "right": dict(zip(("width", "blocks", "conv"), right)), "right_scale": scales[1]},
            "mlp": mlp}


def memory_layer(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def latent_layer(heads, dim, rot_dim, vdim, rank, scale, rot, mlp=None):
    """rot: (dims, base, scaling or None) or None."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1], "scaling": rot[2]}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, loop, eps=1e-5, scale=3.0):
    config = {"architecture": "Rirusun", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    return config


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
CONFIGS = {
    # the loop in the middle, twice; all three mixers; a window of 11 with 3 kept first tokens over pages of 8; a bias table that ends
    # at distance 40; grouped heads; values wider than keys; three blocks of gates; experts in three groups of which two are kept, a
    # shared expert; rotation of part of the rotated elements with YaRN; a layer without feed-forward
    "mix": model(97, 64, [
        parallel_layer((4, 2, 16, 24, 0.3), (12, 40), (11, 3), (48, 3, 3), (0.8, 1.3), moe(32, 6, 2, (3, 2), 40)),
        memory_layer(2, 24, 16, 10.0, moe(24, 4, 2, (2, 1))),
        latent_layer(3, 16, 8, 12, 24, 0.2, (4, 500.0, YARN), moe(16, 5, 3, None, 24)),
        parallel_layer((2, 2, 8, 8, 0.5), (6, 9), (5, 7), (32, 2, 4), (1.0, 0.6)),
        memory_layer(3, 40, 8, 4.0, moe(16, 8, 3, (4, 3))),
    ], loop=(1, 3, 2)),
    # no loop; attention over every earlier key (no window); one kv head per head and one head; one block of gates; a convolution of
    # one tap (no inputs kept); one expert of three, every group kept, groups of one expert; no shared expert; rotation without
    # scaling over all rotated elements; kept first tokens beyond the window's reach; pages of 4
    "plain": model(61, 40, [
        parallel_layer((1, 1, 16, 16, 0.4), (4, 3), None, (24, 1, 1), (1.0, 1.0), moe(20, 3, 1)),
        latent_layer(1, 8, 8, 16, 12, 0.3, (8, 10000.0, None), moe(12, 4, 2, (4, 4))),
        memory_layer(1, 8, 24, 50.0, moe(20, 2, 1, (1, 1), 12)),
        parallel_layer((3, 1, 8, 12, 0.6), (16, 100), (2, 9), (40, 4, 2), (0.5, 2.0), moe(12, 6, 6, (2, 2))),
    ], loop=None),
    # the whole model is the loop, three times; sizes at which the bfloat16 steps run the tensor-core latent attention (rows of 128,
    # values of 96, pages of 64); a memory of 64 x 64 per head, more key elements than a warp has lanes; a window of 70 over pages of 64
    "looped": model(130, 128, [
        latent_layer(4, 32, 32, 32, 96, 0.15, (32, 10000.0, YARN), moe(48, 8, 2, (4, 2), 64)),
        memory_layer(2, 64, 64, 12.0),
        parallel_layer((4, 2, 64, 32, 0.12), (20, 150), (70, 4), (96, 2, 4), (1.1, 0.5), moe(32, 4, 1)),
    ], loop=(0, 3, 3)),
}
PAGE_SIZES = {"mix": 8, "plain": 4, "looped": 64}
LENGTHS = {"mix": (61, 23, 5, 38, 1, 44, 17), "plain": (70, 9, 35, 2, 41), "looped": (230, 70, 3, 129)}


def draw_mixer(rand, matrix, layer, width, name, w):
    p = layer["mixer"]
    if layer["type"] == "parallel":
        left, right = p["left"], p["right"]
        heads, groups, dim, vdim = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        w[name + "left.q"], w[name + "left.k"] = matrix(heads * dim, width, 1.5), matrix(groups * dim, width, 1.5)
        w[name + "left.v"], w[name + "left.o"] = matrix(groups * vdim, width), matrix(width, heads * vdim)
        w[name + "left.q.norm"], w[name + "left.k.norm"] = 2.0 + 0.5 * rand(heads * dim), 2.0 + 0.5 * rand(groups * dim)
        w[name + "left.rel"], w[name + "left.sink"] = 1.5 * rand(left["bias_rows"], heads), 1.0 + rand(heads)
        channels, blocks, taps = right["width"], right["blocks"], right["conv"]
        part = channels // blocks
        w[name + "right.y"], w[name + "right.x"] = matrix(channels, width, 1.5), matrix(channels, width, 1.5)
        w[name + "right.y.b"], w[name + "right.x.b"] = 0.3 * rand(channels), 0.3 * rand(channels)
        w[name + "right.conv"], w[name + "right.conv.b"] = 0.6 * rand(channels, taps), 0.2 * rand(channels)
        w[name + "right.ra"], w[name + "right.ri"] = rand(blocks, part, part) / math.sqrt(part), rand(blocks, part, part) / math.sqrt(part)
        w[name + "right.ra.b"], w[name + "right.ri.b"] = 0.5 * rand(blocks, part), 0.5 * rand(blocks, part)
        w[name + "right.lam"] = -3.0 + 2.0 * rand(channels)      # decays per step from quick to nearly none
        w[name + "right.o"] = matrix(width, channels)
        return
    if layer["type"] == "mlstm":
        heads, dim, vdim = p["heads"], p["dim"], p["vdim"]
        # queries that lean towards their own keys: a read-out whose normaliser is next to nothing would turn its sign with the rounding
        w[name + "k"] = matrix(heads * dim, width, 1.5)
        w[name + "q"] = w[name + "k"] + 0.5 * matrix(heads * dim, width, 1.5)
        w[name + "v"], w[name + "g"], w[name + "o"] = matrix(heads * vdim, width, 1.5), matrix(heads * vdim, width, 1.5), matrix(width, heads * vdim)
        w[name + "norm"] = 1 + 0.2 * rand(heads * vdim)
        w[name + "i"], w[name + "f"] = matrix(heads, width, 2.0), matrix(heads, width, 2.0)
        w[name + "i.b"], w[name + "f.b"] = rand(heads), 3.0 + rand(heads)
        return
    heads, dim, rot_dim, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    w[name + "q"], w[name + "dkv"] = matrix(heads * (dim + rot_dim), width, 2.0), matrix(rank + rot_dim, width, 2.0)
    w[name + "dkv.norm"] = 1 + 0.2 * rand(rank)
    w[name + "uk"], w[name + "uv"], w[name + "o"] = matrix(heads * dim, rank, 2.0), matrix(heads * vdim, rank), matrix(width, heads * vdim)


def draw_weights(config, seed):
    """Weights of a made-up model: matrices N(0, 1/in) times a gain, norm weights around one, biases, corrections and sinks
    that matter, decays from quick to nearly none."""
    g = torch.Generator().manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    rand.generator = g
    matrix = lambda out, inner, gain=1.0: rand(out, inner) * gain / math.sqrt(inner)
    width = config["width"]
    w = {"embed": rand(config["vocab"], width), "head": matrix(config["vocab"], width), "final.norm": 1 + 0.2 * rand(width),
         "final.norm.b": 0.2 * rand(width), "final.norm.alpha": torch.tensor(0.3) + 0.05 * rand(1)[0]}
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        w[name + "norm1"], w[name + "norm1.b"], w[name + "norm1.alpha"] = 1 + 0.2 * rand(width), 0.2 * rand(width), torch.tensor(0.25) + 0.05 * rand(1)[0]
        draw_mixer(rand, matrix, layer, width, name + "mix.", w)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
        # corrections that change who is chosen, under scores whose spread is wide: few choices are so close that rounding turns them
        w[name + "mlp.router"] = matrix(experts, width, 3.0)
        w[name + "mlp.correction"] = 0.3 * rand(experts)
        for e in range(experts):
            w[name + f"mlp.e{e}.up"], w[name + f"mlp.e{e}.down"] = matrix(ff, width, 1.5), matrix(width, ff, 1.5)
        if mlp.get("shared") is not None:
            shared = mlp["shared"]["ff"]
            w[name + "mlp.shared.up"], w[name + "mlp.shared.down"] = matrix(shared, width, 1.5), matrix(width, shared, 1.5)
            w[name + "mlp.shared.sg"] = matrix(1, width, 2.0)
    return {key: value.to(torch.bfloat16).contiguous() for key, value in w.items()}


def every_expert(config):
    """The same model with every token going through all of a layer's experts: no choice is left that rounding could turn."""
    out = json.loads(json.dumps(config))
    for layer in out["layers"]:
        if layer["mlp"] is not None:
            router = layer["mlp"]["router"]
            router["top"] = router["experts"]
            if router.get("groups") is not None:
                router["groups"]["keep"] = router["groups"]["count"]
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, weights as stored); under ``name + "/all"`` the same weights with a configuration in which
    every expert is used: a 16-bit run is compared on the latter, since a rounded input turns a close choice now and then."""
    made = {}
    for seed, (name, config) in enumerate(CONFIGS.items()):
        weights = draw_weights(config, 700 + seed)
        for key, stored in ((name, config), (name + "/all", every_expert(config))):
            folder = tmp_path_factory.mktemp("rirusun_" + name)
            save_file(weights, str(folder / "model.safetensors"), metadata={"format": "pt"})
            (folder / "config.json").write_text(json.dumps(stored))
            made[key] = (folder, stored, weights)
    return made


def plain_logits(config, weights, requests):
    logits = {name: plain.forward(config, weights, tokens).numpy() for name, tokens in requests.items()}
    return logits, {name: len(tokens) for name, tokens in requests.items()}


# ---------------------------------------------------------------------------------------
# whole models under every cutting
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_gives_the_plain_logits(models, name, dtype):
    folder, config, weights = models[name if dtype == "float32" else name + "/all"]
    requests = make_requests(config, LENGTHS[name], seed=7)
    want, sure = plain_logits(config, weights, requests)
    page = PAGE_SIZES[name]
    cuttings = {
        "whole": trace_tools.whole(requests),
        "tail one by one": trace_tools.tail_one_by_one(requests, tail=30),
        "changing portions": trace_tools.changing_portions(requests),
        "mixed": trace_tools.mixed(requests, seed=3, max_live=3, decode_tail=9, max_portion=19),
    }
    for what, steps in cuttings.items():
        pool = trace_tools.pool_tokens(steps, round_to=page)     # no page to spare: pages and slots are used again
        engine = engine_for(folder, dtype, page, pool, slots=3, prefill_chunk_size=pool)
        got = trace_tools.run_in_process(engine, steps)
        assert_logits(got, want, sure, dtype, f"{name}, {what}, {dtype}")
        assert engine.cache.free_slots() == 3 and all(group.pool.free_count == group.pool.num_pages for group in engine.cache.groups)
        del engine


def test_layer_by_layer_in_32_bit(models):
    """The residual stream after every layer run, the loop's passes included."""
    from pylon_b200.engine import StepEntry

    folder, config, weights = models["mix"]
    tokens = make_requests(config, (37,), seed=5)["r0"]
    want: list = []
    plain.forward(config, weights, tokens, taps=want)
    engine = engine_for(folder, "float32", 8, 64)
    taps: list = []
    forward = engine.model.forward
    engine.model.forward = lambda step, caches: forward(step, caches, taps)
    request = engine.open("a", len(tokens))
    engine.step([StepEntry(request, tokens, [0])])
    assert len(taps) == len(plain.run_order(config)) == 7
    for index, (got, expected) in enumerate(zip(taps, want)):
        torch.testing.assert_close(got.double().cpu(), expected, rtol=1e-4, atol=1e-4 * float(expected.abs().max()), msg=lambda m: f"run {index}: {m}")


def test_long_decoding_past_the_window_and_many_pages(models):
    """A short prompt, then 200 tokens one by one: the window passes over decoded tokens many times while the first tokens stay, pages
    are given back behind it, the states and the convolutions' inputs are carried 200 times."""
    folder, config, weights = models["mix"]
    requests = make_requests(config, (212,), seed=11)
    want, sure = plain_logits(config, weights, requests)
    steps = trace_tools.tail_one_by_one(requests, tail=200)
    engine = engine_for(folder, "float32", 8, 216)
    got = trace_tools.run_in_process(engine, steps)
    assert_logits(got, want, sure, "float32", "long decoding")
    assert any(group.need.keep_first for group in engine.cache.groups) and all(group.pool.free_count == group.pool.num_pages for group in engine.cache.groups)


def test_the_replay_program_runs_the_model(models, tmp_path):
    folder, config, weights = models["plain"]
    requests = make_requests(config, (33, 12, 20), seed=2)
    want, sure = plain_logits(config, weights, requests)
    steps = trace_tools.mixed(requests, seed=1, max_live=2, decode_tail=5, max_portion=9)
    got = trace_tools.run_program(folder, "float32", steps, tmp_path / "out", extra_args=("--page-size", "4"))
    assert_logits(got, want, sure, "float32", "bin/trace_run")


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(models, graphs):
    """Several prompts through ``Engine.generate`` with a small prompt budget and few slots: every generated token is the
    arg-max of the plain logits of its own prefix."""
    from pylon_b200.sampling.params import SamplingParams

    folder, config, weights = models["mix"]
    prompts = list(make_requests(config, (19, 3, 40, 11, 27, 8), seed=13).values())
    new_tokens = 12
    engine = engine_for(folder, "float32", PAGE_SIZES["mix"], 4 * 64, slots=3, prefill_chunk_size=16, cuda_graphs=graphs)
    results = engine.generate(prompts, SamplingParams(max_new_tokens=new_tokens, temperature=0.0, ignore_eos=True))
    for prompt, result in zip(prompts, results):
        assert len(result.output_ids) == new_tokens
        sequence = list(prompt) + list(result.output_ids)
        logits = plain.forward(config, weights, sequence[:-1])
        for place in range(len(prompt) - 1, len(sequence) - 1):
            row = logits[place]
            best = int(row.argmax())
            if sequence[place + 1] != best:   # a tie within rounding may go either way
                assert float(row[best] - row[sequence[place + 1]]) < 1e-3 * float(row.std()), f"token {place + 1} of a request is not the plain arg-max"
    engine.cache.check()
    assert engine.cache.free_slots() == 3


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
def mixer_case(name, rand, matrix, width, eps):
    """(the mixer's tensors, its part's description, the plain function) of a small made-up mixer."""
    from pylon_b200.parts import PartSpec

    bf = lambda t: t.to(torch.bfloat16)
    left = {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.35, "bias_max": 30, "mask": {"size": 9, "keep_first": 4}}
    right = {"width": 36, "blocks": 3, "conv": 3}
    w_left = {"q": matrix(48, width, 1.5), "k": matrix(24, width, 1.5), "v": matrix(40, width), "o": matrix(width, 80), "q.norm": bf(2 + 0.5 * rand(48)),
              "k.norm": bf(2 + 0.5 * rand(24)), "rel": bf(1.5 * rand(10, 4)), "sink": bf(1 + rand(4))}
    w_right = {"y": matrix(36, width, 1.5), "x": matrix(36, width, 1.5), "y.b": bf(0.3 * rand(36)), "x.b": bf(0.3 * rand(36)), "conv": bf(0.6 * rand(36, 3)),
               "conv.b": bf(0.2 * rand(36)), "ra": bf(rand(3, 12, 12) / 3.5), "ri": bf(rand(3, 12, 12) / 3.5), "ra.b": bf(0.5 * rand(3, 12)),
               "ri.b": bf(0.5 * rand(3, 12)), "lam": bf(-3 + 2 * rand(36)), "o": matrix(width, 36)}
    attention = PartSpec("gqa_attention", {
        "width": width, "n_heads": 4, "n_kv_heads": 2, "head_dim": 12, "value_dim": 20, "scale": 0.35, "window": 9, "keep_first": 4, "qk_norm": "whole",
        "qk_norm_eps": eps, "distance_bias": {"rows": 10, "far": 30}, "sink": True,
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "distance_bias": "rel", "sink": "sink"}})
    recurrent = PartSpec("gated_linear_recurrence", {"width": width, "channels": 36, "blocks": 3, "conv_taps": 3, "decay_factor": 8.0})
    if name == "window":
        return w_left, attention, lambda h, w: plain.sink_window_attention(h, w, "", left, eps)
    if name == "recurrence":
        return w_right, recurrent, lambda h, w: plain.gated_linear_recurrence(h, w, "", right)
    if name == "side_by_side":
        w = {**{"left." + k: v for k, v in w_left.items()}, **{"right." + k: v for k, v in w_right.items()}}
        spec = PartSpec("weighted_mixers", {"mixers": (attention, recurrent), "prefixes": ("left.", "right."), "scales": (1.3, 0.4)})
        return w, spec, lambda h, w: plain.side_by_side(h, w, "", {"left": left, "right": right, "left_scale": 1.3, "right_scale": 0.4}, eps)
    if name == "memory":
        heads, dim, vdim, cap = 3, 20, 12, 6.0
        keys = matrix(heads * dim, width, 1.5)
        w = {"q": (keys + 0.5 * matrix(heads * dim, width, 1.5)).to(torch.bfloat16), "k": keys, "v": matrix(heads * vdim, width, 1.5), "g": matrix(heads * vdim, width, 1.5),
             "o": matrix(width, heads * vdim), "norm": bf(1 + 0.2 * rand(heads * vdim)), "i": matrix(heads, width, 3.0), "f": matrix(heads, width, 3.0),
             "i.b": bf(rand(heads)), "f.b": bf(2 + rand(heads))}
        spec = PartSpec("matrix_memory", {"width": width, "n_heads": heads, "head_dim": dim, "value_dim": vdim, "gate_cap": cap, "norm_eps": eps})
        return w, spec, lambda h, w: plain.matrix_memory(h, w, "", {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, eps)
    heads, dim, rot_dim, vdim, rank = 3, 12, 8, 10, 20
    rot = {"dims": 6, "base": 300.0, "scaling": YARN}
    w = {"q": matrix(heads * (dim + rot_dim), width, 2.0), "dkv": matrix(rank + rot_dim, width, 2.0), "dkv.norm": bf(1 + 0.2 * rand(rank)),
         "uk": matrix(heads * dim, rank, 2.0), "uv": matrix(heads * vdim, rank), "o": matrix(width, heads * vdim)}
    spec = PartSpec("latent_attention", {
        "width": width, "n_heads": heads, "head_dim": dim, "rot_dim": rot_dim, "value_dim": vdim, "q_rank": None, "kv_rank": rank, "norm_eps": eps, "scale": 0.3,
        "position": PartSpec("rope", {"head_dim": rot_dim, "theta": 300.0, "max_positions": 128, "rotary_dim": 6, "scaling": {"kind": "yarn", **YARN}, "layout": "halves"})})
    return w, spec, lambda h, w: plain.latent_attention(h, w, "", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": 0.3, "rot": rot}, eps)


def built(name, dtype, seed=21, width=56, eps=1e-5):
    from pylon_b200.parts import MIXERS

    g = torch.Generator().manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    rand.generator = g
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w, spec, oracle = mixer_case(name, rand, matrix, width, eps)
    part = MIXERS.build(spec)
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w) and all(tuple(w[k].shape) == tuple(declared[k].shape) for k in w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    return part, w, oracle, rand


MIXER_NAMES = ["window", "recurrence", "side_by_side", "memory", "latent"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", MIXER_NAMES)
def test_each_mixer_alone_against_its_plain_statement(name, dtype):
    """A mixer part from its normalised input to its delta for the stream: a prompt in one step, then the same in portions
    down to single tokens (portions that end right at, before and behind the window's and the kept tokens' edges), and token by
    token from the start."""
    part, w, oracle, rand = built(name, dtype)
    count, page = 45, 8
    h = rand(count, 56).to(dtype)
    want = oracle(h.double(), {k: v.double() for k, v in w.items()})
    spread = float(want.std())
    limit = 0.06 * spread if dtype == torch.bfloat16 else 1e-4 * spread
    for cutting in ((count,), (20, 2, 1, 1, 13, 8), (1,) * 12 + (2, 2, 29), (9, 9, 9, 18), (8, 1, 9, 27), (4, 5, 1, 3, 32), (3, 2, 4, 36)):
        got = run_part(part, h, cutting, page, dtype)
        assert float((got - want).abs().max()) <= limit, f"{name}, {cutting}: off by {float((got - want).abs().max()):.3g} of {spread:.3g}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", MIXER_NAMES)
def test_unequal_requests_in_one_step_against_each_alone(name, dtype):
    """Three requests of 1, 17 and 6 new tokens at different places of their sequences in one step, in state slots and pages
    that another request used before: every request's result is the one it has alone."""
    part, w, oracle, rand = built(name, dtype, seed=8)
    page = 8
    before, new = (12, 0, 30), (1, 17, 6)
    inputs = [rand(b + n, 56).to(dtype) for b, n in zip(before, new)]
    want = [oracle(h.double(), {k: v.double() for k, v in w.items()}) for h in inputs]
    need = part.cache_need()
    cache = fresh_cache(need, page, dtype, table=tuple(range(15)), slots=4)
    slots = (2, 0, 3)
    if need.kv is not None:
        cache.block_table = torch.tensor([[9, 3, 12, 0, 7], [1, 14, 5, 10, 2], [6, 11, 4, 13, 8]], device=DEVICE, dtype=torch.int32)
        cache.k_pages.fill_(3.0)                               # what an earlier request left in the pages
        if cache.v_pages is not None:
            cache.v_pages.fill_(-2.0)

    def run(rows, sizes, starts):
        step = step_view(sizes, starts, dtype)
        step.slots = torch.tensor([slots[r] for r in rows], device=DEVICE, dtype=torch.int32)
        saved = cache.block_table
        if need.kv is not None:
            cache.block_table = saved[list(rows)].contiguous()
        out = part.forward(on(torch.cat([inputs[r][s : s + n] for r, n, s in zip(rows, sizes, starts)])), step, cache)
        cache.block_table = saved
        return (out.sum(dim=0) if out.dim() == 3 else out).double().cpu()

    if need.state is not None:
        cache.state.normal_()                                  # what an earlier request left in the slots ...
        cache.state[list(slots)] = 0.0                         # ... and a slot is handed out cleared
    for r in (0, 2):                                           # what the requests hold already, each alone
        run((r,), (before[r],), (0,))
    got = run((0, 1, 2), new, before)
    spread = float(torch.cat(want).std())
    limit = 0.06 * spread if dtype == torch.bfloat16 else 1e-4 * spread
    cursor = 0
    for r in range(3):
        mine = got[cursor : cursor + new[r]]
        cursor += new[r]
        worst = float((mine - want[r][before[r] :]).abs().max())
        assert worst <= limit, f"{name}: request {r} in the batch is off by {worst:.3g} of {spread:.3g}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_that_stand_out_at_the_windows_edge_among_the_first_and_far_away(dtype):
    """Keys far larger than the rest, each with a value of its own: the last kept first token and the one behind it (seen for ever;
    seen only while the window reaches it), and a key in the middle that a query sees up to the window's last position and not one
    later.  A bias table that ends far outside the window says how far the kept token is.  In a prompt, token by token across
    the edges, and in portions that end and start right at them; a window that is no multiple of the page."""
    from pylon_b200.kernels import ops
    from pylon_b200.parts.attention import distance_bucket

    g = torch.Generator().manual_seed(5)
    count, window, keep, page, heads, width, dv = 170, 37, 5, 16, 4, 32, 24
    kept, lost, middle = keep - 1, keep, 90
    rows = torch.randn(count, width, generator=g) * 0.3
    values = torch.randn(count, dv, generator=g) * 0.3
    for place, (low, high) in ((kept, (-4.0, 4.0)), (lost, (5.0, -5.0)), (middle, (-6.0, 6.0))):
        rows[place] = 3.0
        values[place] = torch.linspace(low, high, dv)
    queries = torch.randn(count, heads, width, generator=g) * 0.3 + 0.25
    table_rows, far = 12, 120
    rel = torch.randn(table_rows, heads, generator=g)
    rel[-1] = 2.0                                                # the far rows matter: a kept token is up to 165 positions back
    sink = torch.randn(heads, generator=g) + 1.0
    bias = torch.stack([rel[distance_bucket(n, table_rows, far)] for n in range(far + 1)])
    pages, table = paged(rows, page, dtype, seed=3)
    value_pages, _ = paged(values, page, dtype, seed=3)
    scale = 0.5
    q, keys, vals = queries.to(dtype).double(), rows.to(dtype).double(), values.to(dtype).double()
    index = torch.arange(count)
    distance = index[:, None] - index[None, :]
    visible = (distance >= 0) & ((distance < window) | (index[None, :] < keep))
    scores = torch.einsum("ihd,jd->hij", q, keys) * scale + bias.double()[distance.clamp(0, far)].permute(2, 0, 1)
    scores = scores.masked_fill(~visible[None], -math.inf)
    top = torch.maximum(scores.max(dim=-1).values, sink.double()[:, None])
    e = torch.exp(scores - top[..., None])
    weights = e / (e.sum(dim=-1) + torch.exp(sink.double()[:, None] - top))[..., None]
    want = torch.einsum("hij,jv->ihv", weights, vals).reshape(count, heads * dv)
    assert float(weights[:, 150, kept].min()) > 0.02 and float(weights[:, lost + window :, lost].max()) == 0.0 and float(weights[:, lost + window - 1, lost].min()) > 0.02
    assert float(weights[:, middle + window - 1, middle].min()) > 0.02 and float(weights[:, middle + window :, middle].max()) == 0.0

    def run(cutting):
        outs, cursor = [], 0
        for size in cutting:
            step = step_view((size,), (cursor,), dtype)
            outs.append(ops.paged_attention(on(queries[cursor : cursor + size].to(dtype)).view(size, heads * width), pages, value_pages, step.positions,
                                            step.token_row, step.q_start, step.kv_len, table, heads, step.max_q, step.max_kv, window=window, scale=scale,
                                            sinks=on(sink), keep_first=keep, distance_bias=on(bias)))
            cursor += size
        return torch.cat(outs).double().cpu()

    tolerance = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    edge = middle + window
    for cutting in ((count,), (edge - 3,) + (1,) * 6 + (count - edge - 3,), (edge - 1, 1, count - edge), (edge, count - edge), (keep, 1, 1, count - keep - 2),
                    (keep - 1, 2, count - keep - 1), (lost + window - 2,) + (1,) * 4 + (count - lost - window - 2,), (2,) * 85):
        assert sum(cutting) == count
        torch.testing.assert_close(run(cutting), want, **tolerance)


def test_the_distance_rows_of_the_bias_table():
    from pylon_b200.parts.attention import distance_bucket

    for rows, far in ((12, 120), (16, 64), (6, 9), (32, 128), (5, 40)):
        got = [distance_bucket(n, rows, far) for n in range(3 * far)]
        assert got == [plain.distance_bucket(n, rows, far) for n in range(3 * far)]
        assert got[: rows // 2] == list(range(rows // 2)) and all(a <= b for a, b in zip(got, got[1:])) and got[far] == rows - 1 == got[-1]
    assert distance_bucket(32, 16, 128) == 8 + 4      # a quotient of logarithms that is an integer counts as one: ln 4 / ln 16 * 8


def test_the_recurrence_and_the_memory_read_back_what_was_written_long_ago():
    """A channel that hardly decays keeps what one token wrote for 400 tokens, the channel beside it forgets within a few; a head of
    the matrix memory whose forget gate stays open hands a value back 400 tokens later.  The projections are unit matrices, so the
    layer's input is the products' columns themselves.  In one step and in portions."""
    from pylon_b200.parts import MIXERS, PartSpec

    count, write, read = 420, 3, 403
    # -- the recurrence: channels [y | x] = the input itself
    channels = 4
    h = torch.zeros(count, 2 * channels)
    h[:, :channels] = 3.0                                             # the gelu branch is open
    h[write, channels:] = 2.0
    w = {"y": torch.eye(2 * channels)[:channels], "x": torch.eye(2 * channels)[channels:], "y.b": torch.zeros(channels), "x.b": torch.zeros(channels),
         "conv": torch.ones(channels, 1), "conv.b": torch.zeros(channels), "ra": torch.zeros(1, channels, channels), "ri": torch.zeros(1, channels, channels),
         "ra.b": torch.zeros(1, channels), "ri.b": torch.full((1, channels), 20.0), "lam": torch.tensor([-10.6, -10.6, 2.0, 2.0]), "o": torch.eye(channels)}
    want = plain.gated_linear_recurrence(h.double(), {k: v.double() for k, v in w.items()}, "", {"width": channels, "blocks": 1})
    assert float(want[read, 2:].abs().max()) < 1e-6 and float(want[write + 1, 2].abs()) > 1e-3 and float(want[read, 0]) > 1e-3 and float(want[write - 1].abs().max()) == 0.0
    part = MIXERS.build(PartSpec("gated_linear_recurrence", {"width": 2 * channels, "channels": channels, "blocks": 1, "conv_taps": 1}))
    part.load({k: on(v) for k, v in w.items()}, torch.float32, torch.device(DEVICE))
    for cutting in ((count,), (2, 2) + (1,) * 399 + (17,), (write + 1, read - write - 1, 1, count - read - 1), (200, 203, 17)):
        got = run_part(part, h, cutting, 8, torch.float32)
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-7)
    # -- the memory: columns [q | k | v | g] = the input itself, one head
    dim, vdim = 4, 6
    columns = 2 * dim + 2 * vdim
    g = torch.Generator().manual_seed(4)
    h = torch.zeros(count, columns)
    h[:, 2 * dim + vdim :] = 4.0                                       # the output gate is open
    h[write, dim + 1] = 3.0                                            # k of the writing token: row 1
    h[write, 2 * dim : 2 * dim + vdim] = torch.randn(vdim, generator=g)
    h[read, 1] = 2.0                                                   # q of the reading token: row 1
    h[read - 1, 2] = 2.0                                               # the token before asks for the row beside it: nothing there
    w = {"q": torch.eye(columns)[:dim], "k": torch.eye(columns)[dim : 2 * dim], "v": torch.eye(columns)[2 * dim : 2 * dim + vdim], "g": torch.eye(columns)[2 * dim + vdim :],
         "o": torch.eye(vdim), "norm": torch.ones(vdim), "i": torch.zeros(1, columns), "f": torch.zeros(1, columns), "i.b": torch.zeros(1), "f.b": torch.full((1,), 30.0)}
    mixer = {"heads": 1, "dim": dim, "vdim": vdim, "gate_cap": 40.0}
    want = plain.matrix_memory(h.double(), {k: v.double() for k, v in w.items()}, "", mixer, 1e-6)
    far = plain.rms_unit(h[write, 2 * dim : 2 * dim + vdim].double(), 1e-6) * torch.sigmoid(torch.tensor(4.0, dtype=torch.float64))
    torch.testing.assert_close(want[read], far, rtol=1e-3, atol=1e-3)
    assert float(want[read - 1].abs().max()) < 1e-6
    part = MIXERS.build(PartSpec("matrix_memory", {"width": columns, "n_heads": 1, "head_dim": dim, "value_dim": vdim, "gate_cap": 40.0, "norm_eps": 1e-6}))
    part.load({k: on(v) for k, v in w.items()}, torch.float32, torch.device(DEVICE))
    for cutting in ((count,), (2, 2) + (1,) * 399 + (17,), (write + 1, read - write - 1, 1, count - read - 1), (200, 203, 17)):
        got = run_part(part, h, cutting, 8, torch.float32)
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_of_a_scaled_tanh(dtype):
    from pylon_b200.parts import NORMS, PartSpec, ResidualStream

    width = 200
    norm = NORMS.build(PartSpec("dynamic_tanh", {"width": width, "weight_name": "", "alpha_name": ".alpha", "bias_name": ".b"}))
    weight, bias, alpha = torch.rand(width) + 0.5, torch.randn(width), torch.tensor(0.37)
    norm.load({"": weight.to(DEVICE), ".b": bias.to(DEVICE), ".alpha": alpha.to(DEVICE)}, dtype, torch.device(DEVICE))
    residual = 3 * torch.randn(6, width, device=DEVICE)
    delta = torch.randn(6, width, device=DEVICE).to(dtype)
    stream = ResidualStream(residual.clone())
    stream.add(delta)
    out = norm.apply(stream)
    want_sum = residual.double() + delta.double()
    torch.testing.assert_close(stream.residual.double(), want_sum, rtol=1e-6, atol=1e-6)
    assert stream.pending is None
    want = plain.dynamic_tanh(want_sum.cpu(), alpha.double(), weight.double(), bias.double())
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.double().cpu(), want, **tol)
    rows = torch.tensor([4, 1], device=DEVICE, dtype=torch.int32)     # a selection: the stream stays as it is
    stream.add(delta)
    picked = norm.apply(stream, rows=rows)
    torch.testing.assert_close(stream.residual.double(), want_sum, rtol=1e-6, atol=1e-6)
    want = plain.dynamic_tanh((want_sum + delta.double()).cpu()[[4, 1]], alpha.double(), weight.double(), bias.double())
    torch.testing.assert_close(picked.double().cpu(), want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,experts,top,groups,shared,tokens", [
    (40, 12, 3, 1, None, None, 1), (56, 20, 6, 6, (3, 3), 24, 7), (48, 24, 12, 4, (4, 2), 16, 150), (128, 64, 33, 3, (11, 4), None, 70),
    (64, 40, 2, 1, (2, 1), 40, 40), (256, 136, 4, 2, (1, 1), 128, 700), (384, 256, 3, 1, None, 64, 600), (64, 32, 8, 2, (8, 3), None, 90)])
def test_the_mixture_of_experts_against_token_by_token(width, ff, experts, top, groups, shared, tokens, dtype):
    """Sigmoid scores in 32-bit, the choice by score plus correction inside the kept groups (negative choice scores, groups of one
    expert, one group, every group kept), weights without the correction, ungated experts with the exact gelu, the gated shared expert:
    one token, few and many, tiles that are partly filled; the last shapes but one have enough tokens an expert for the grouped
    tensor-core product.  Tokens whose choice hangs on a margin that 16-bit rounding of the input can turn are left out of the
    16-bit comparison."""
    from pylon_b200.parts import FEED_FORWARDS, PartSpec

    g = torch.Generator().manual_seed(17)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w = {"router": matrix(experts, width, 3.0), "correction": (0.4 * rand(experts) - 0.8).to(torch.bfloat16)}    # choice scores on both sides of zero
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = matrix(ff, width, 1.5), matrix(width, ff, 1.5)
    mlp = {"expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups is not None:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
        w["shared.up"], w["shared.down"], w["shared.sg"] = matrix(shared, width, 1.5), matrix(width, shared, 1.5), matrix(1, width, 2.0)
    part = FEED_FORWARDS.build(PartSpec("expert_mixture", {
        "width": width, "intermediate": ff, "experts": experts, "top": top, "activation": "gelu", "gated": False, "routing": "sigmoid", "correction": True,
        "groups": None if groups is None else groups[0], "groups_keep": None if groups is None else groups[1], "share_eps": 1e-20, "shared_intermediate": shared}))
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w) and all(tuple(w[k].shape) == tuple(declared[k].shape) for k in w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    h = rand(tokens, width).to(dtype)
    doubles = {k: v.double() for k, v in w.items()}
    want = plain.expert_mixture(h.double(), doubles, "", mlp)
    # a token is sure if nudging its scores by what rounding does changes nobody's place: compare the choice under two small nudges
    chosen, _ = plain.choose_experts(h.double(), doubles, "", mlp["router"])
    sure = torch.ones(tokens, dtype=torch.bool)
    margin = 1e-4 if dtype == torch.float32 else 0.03
    for sign in (-1.0, 1.0):
        nudged = dict(doubles)
        nudged["correction"] = doubles["correction"] + sign * margin * torch.cos(torch.arange(experts, dtype=torch.float64) * 2.4)
        other, _ = plain.choose_experts(h.double(), nudged, "", mlp["router"])
        sure &= (chosen.sort(dim=1).values == other.sort(dim=1).values).all(dim=1)
    assert int(sure.sum()) >= 0.7 * tokens
    out = part.forward(on(h), step_view((tokens,), (0,), dtype))
    assert out.dtype == torch.float32          # the stream takes it in 32-bit
    got = (out.sum(dim=0) if out.dim() == 3 else out).double().cpu()
    spread = float(want.std())
    limit = 0.05 * spread if dtype == torch.bfloat16 else 1e-4 * spread
    assert float((got - want)[sure].abs().max()) <= limit
    # the same tokens in another order and among others: a token's result does not depend on its place in the step
    order = torch.randperm(tokens, generator=g)
    both = torch.cat([h[order], rand(5, width).to(dtype)])
    again = part.forward(on(both), step_view((tokens + 5,), (0,), dtype))
    again = (again.sum(dim=0) if again.dim() == 3 else again).double().cpu()[:tokens]
    if tokens + 5 < 512 or tokens >= 512:      # (the same kernels either way)
        assert torch.equal(again, got[order])
