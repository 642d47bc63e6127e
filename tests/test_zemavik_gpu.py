"""Zemavik on the GPU against the plain implementation (``plain_zemavik``): each mechanism alone, then whole models of
several made-up shapes stepped through the engine under every cutting, and generation through the scheduler.

The models' weights are drawn here, larger than a trained model's and with the attention sharpened, so that a key that is
wrongly seen or missed across a chunk's edge, a state or a convolution input that is lost, a wrong expert and an embedding
that is not fed in again all move the logits by much more than the tolerance."""
from __future__ import annotations

import json
import math

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_zemavik as plain
import trace_tools
from test_parts_gpu import step_view

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


# ---------------------------------------------------------------------------------------
# made-up models
# ---------------------------------------------------------------------------------------
def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def parallel_layer(left, right, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale, chunk or None); right: (heads, vdim, state, groups, norm_groups, taps)."""
    attention = dict(zip(("heads", "kv_heads", "dim", "vdim", "scale"), left[:5]))
    if left[5] is not None:
        attention["mask"] = {"size": left[5]}
    return {"type": "parallel", "mixer": {"left": attention, "right": dict(zip(("heads", "vdim", "state", "groups", "norm_groups", "conv"), right))},
            "mlp": mlp}


def delta_layer(heads, kv_heads, dim, vdim, taps, ranks, mlp=None):
    """ranks: the widths of the decay's and the gate's narrow middles; the checkpoint's shapes carry them, not the configuration."""
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}, "mlp": mlp,
            "_ranks": ranks}


def model(vocab, width, layers, loop, max_positions=512, eps=1e-5):
    config = {"architecture": "Zemavik", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    return config


CONFIGS = {
    # the loop in the middle, twice; both mixers; grouped heads everywhere (attention 4 over 2, state space 4 over 2 groups, delta 4
    # over 2); the gated norm in two and three parts; values wider and narrower than keys; chunks that are no multiple of the page;
    # a layer without feed-forward; experts of which two and three of five and seven are used
    "mix": model(83, 48, [
        parallel_layer((4, 2, 16, 8, 0.6, 9), (4, 6, 10, 2, 2, 4), dense(80)),
        delta_layer(4, 2, 12, 10, 3, (8, 6), moe(24, 5, 2)),
        parallel_layer((3, 3, 8, 20, 0.9, 13), (3, 8, 7, 1, 3, 2)),
        delta_layer(2, 2, 20, 6, 2, (5, 9), dense(56)),
        parallel_layer((2, 1, 24, 12, 0.4, 30), (6, 4, 12, 3, 1, 3), moe(16, 7, 3)),
    ], loop=(1, 3, 2)),
    # no loop and no map into it; attention over every earlier key (no chunks) and in chunks of one and two positions; a
    # convolution of one tap (no inputs kept); one head everywhere; one expert of three, and every expert of four; pages of 4
    "plain": model(61, 40, [
        parallel_layer((1, 1, 16, 16, 0.5, None), (1, 16, 8, 1, 1, 1), moe(20, 3, 1)),
        delta_layer(1, 1, 16, 24, 1, (4, 4), dense(48)),
        parallel_layer((2, 2, 8, 8, 0.8, 1), (2, 8, 5, 2, 2, 5), moe(12, 4, 4)),
        parallel_layer((3, 1, 8, 12, 0.9, 2), (4, 4, 16, 4, 4, 2), dense(40)),
    ], loop=None),
    # the whole model is the loop, three times; head size 64 with pages of 64: the bfloat16 steps run the tensor-core attention
    # inside chunks; states of 64 x 64 per head, the delta rule's heads as large as a real model's
    "looped": model(130, 64, [
        parallel_layer((4, 2, 64, 64, 0.16, 70), (2, 64, 64, 1, 1, 4), dense(96)),
        delta_layer(2, 1, 64, 64, 4, (16, 8), moe(32, 8, 2)),
    ], loop=(0, 2, 3)),
    # a width at which the decode steps' products come as partial sums over slices of k and prompts run on the tcgen05 kernels;
    # the loop at the end, once (the map into it still applies); values narrower than keys; experts wide enough for the tensor cores
    "wide": model(300, 1024, [
        delta_layer(8, 4, 64, 128, 4, (32, 48), dense(512)),
        parallel_layer((8, 4, 64, 32, 0.16, 80), (16, 32, 128, 2, 4, 4), moe(256, 6, 2)),
        parallel_layer((4, 2, 128, 128, 0.08, 200), (8, 64, 32, 8, 1, 3), dense(512)),
    ], loop=(2, 3, 1)),
    # no attention at all: no page is ever held, the state slots are all a request has
    "delta_only": model(45, 32, [
        delta_layer(2, 1, 8, 16, 3, (4, 6), dense(48)),
        delta_layer(4, 4, 16, 8, 2, (6, 3), moe(8, 3, 2)),
    ], loop=(0, 1, 2)),
}
PAGE_SIZES = {"mix": 8, "plain": 4, "looped": 64, "wide": 64, "delta_only": 16}
LENGTHS = {"mix": (61, 23, 5, 38, 1, 44, 17), "plain": (70, 9, 35, 2, 41), "looped": (230, 70, 3, 129), "delta_only": (40, 3, 25, 31, 1), "wide": (330, 45, 150)}


def stored_config(config):
    """What goes into config.json: the layers without the sizes that only the checkpoint's shapes give."""
    out = dict(config)
    out["layers"] = [{key: value for key, value in layer.items() if key != "_ranks"} for layer in config["layers"]]
    return out


def draw_mixer(rand, matrix, layer, width, name, w):
    p = layer["mixer"]
    if layer["type"] == "parallel":
        left, right = p["left"], p["right"]
        heads, groups, dim, vdim = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        w[name + "left.q"], w[name + "left.k"] = matrix(heads * dim, width, 1.5), matrix(groups * dim, width, 1.5)
        w[name + "left.v"], w[name + "left.o"] = matrix(groups * vdim, width), matrix(width, heads * vdim)
        heads, vdim, state, groups, taps = right["heads"], right["vdim"], right["state"], right["groups"], right["conv"]
        inner, channels = heads * vdim, heads * vdim + 2 * groups * state
        w[name + "right.in"] = matrix(inner + channels + heads, width, 1.5)
        w[name + "right.conv"], w[name + "right.conv.b"] = 0.6 * rand(channels, taps), 0.2 * rand(channels)
        w[name + "right.dt_bias"], w[name + "right.D"] = 0.5 * rand(heads), 1 + 0.3 * rand(heads)
        w[name + "right.A_log"] = -4.5 * torch.rand(heads, generator=rand.generator)      # decays per step from about 0.5 to nearly one
        w[name + "right.norm"], w[name + "right.o"] = 1 + 0.2 * rand(inner), matrix(width, inner)
        w[name + "left.out"], w[name + "right.out"] = 1 + 0.3 * rand(width), 1 + 0.3 * rand(width)
        return
    heads, groups, dim, vdim, taps = p["heads"], p["kv_heads"], p["dim"], p["vdim"], p["conv"]
    decay_rank, gate_rank = layer["_ranks"]
    for key, rows in (("q", groups * dim), ("k", groups * dim), ("v", heads * vdim)):
        w[name + key] = matrix(rows, width, 1.5)
        w[name + key + ".conv"] = 0.6 * rand(rows, taps)
    w[name + "b"] = matrix(heads, width, 2.0)
    w[name + "A_log"] = -3.0 * torch.rand(heads, generator=rand.generator)
    w[name + "a1"], w[name + "a2"], w[name + "dt_bias"] = matrix(decay_rank, width), matrix(heads * dim, decay_rank, 1.5), 0.5 * rand(heads * dim)
    w[name + "g1"], w[name + "g2"] = matrix(gate_rank, width), matrix(heads * vdim, gate_rank, 2.0)
    w[name + "norm"], w[name + "o"] = 1 + 0.2 * rand(vdim), matrix(width, heads * vdim)


def draw_weights(config, seed):
    """Weights of a made-up model: matrices N(0, 1/in) times a gain, norm weights around one, biases and router offsets that
    matter, decays from quick to nearly none."""
    g = torch.Generator().manual_seed(seed)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    rand.generator = g
    matrix = lambda out, inner, gain=1.0: rand(out, inner) * gain / math.sqrt(inner)
    width = config["width"]
    w = {"embed": rand(config["vocab"], width), "pos": 0.7 * rand(config["max_positions"], width), "final.norm": 1 + 0.2 * rand(width)}
    if config.get("loop") is not None:
        w["loop.in"] = matrix(width, 2 * width, 1.4)
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        w[name + "norm1"] = 1 + 0.2 * rand(width)
        draw_mixer(rand, matrix, layer, width, name + "mix.", w)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        w[name + "norm2"] = 1 + 0.2 * rand(width)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            w[name + "mlp.gate"], w[name + "mlp.up"], w[name + "mlp.down"] = matrix(ff, width, 1.5), matrix(ff, width, 1.5), matrix(width, ff)
            w[name + "mlp.gate.b"], w[name + "mlp.up.b"], w[name + "mlp.down.b"] = 0.5 * rand(ff), 0.5 * rand(ff), 0.5 * rand(width)
        else:
            ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
            # offsets a unit apart under logits of about that spread: who is chosen changes from token to token, and few
            # choices are so close that rounding the input turns them
            w[name + "mlp.router"] = matrix(experts, width, 0.7)
            w[name + "mlp.router.b"] = torch.randperm(experts, generator=g).float() + 0.1 * rand(experts)
            for e in range(experts):
                w[name + f"mlp.e{e}.gate"], w[name + f"mlp.e{e}.up"] = matrix(ff, width, 1.5), matrix(ff, width, 1.5)
                w[name + f"mlp.e{e}.down"] = matrix(width, ff, 1.5)
    return {key: value.to(torch.bfloat16).contiguous() for key, value in w.items()}


def every_expert(config):
    """The same model with every token going through all of a layer's experts: no choice is left that rounding could turn."""
    out = json.loads(json.dumps(config))
    for layer in out["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, weights as stored); under ``name + "/all"`` the same weights with a configuration in which
    every expert is used.  A 16-bit run is compared on the latter: with few of the experts, one choice in thirty is so close
    that the rounded input turns it, and everything after it in the request rightly differs."""
    made = {}
    for seed, (name, config) in enumerate(CONFIGS.items()):
        weights = draw_weights(config, 900 + seed)
        for key, stored in ((name, stored_config(config)), (name + "/all", every_expert(stored_config(config)))):
            folder = tmp_path_factory.mktemp("zemavik_" + name)
            save_file(weights, str(folder / "model.safetensors"), metadata={"format": "pt"})
            (folder / "config.json").write_text(json.dumps(stored))
            made[key] = (folder, stored, weights)
    return made


def make_requests(config, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, config["vocab"], size=n)] for i, n in enumerate(lengths)}


CLOSE_CALL = 0.05      # a router's margin under which a bfloat16 run may choose otherwise (the logits' spread is about one)


def plain_logits(config, weights, requests):
    """name -> logits, and name -> the number of leading positions none of whose routers' choices was a close call."""
    logits, sure = {}, {}
    for name, tokens in requests.items():
        margins: list = []
        logits[name] = plain.forward(config, weights, tokens, margins=margins).numpy()
        close = torch.stack(margins).min(dim=0).values < CLOSE_CALL if margins else torch.zeros(len(tokens), dtype=torch.bool)
        sure[name] = int(close.nonzero()[0]) if bool(close.any()) else len(tokens)
    return logits, sure


def engine_for(folder, dtype, page_size, pool, slots=4, **options):
    from pylon_b200.config import EngineConfig
    from pylon_b200.engine import Engine

    return Engine(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool, max_context=pool, max_batch_size=slots, **options))


def assert_logits(got, want, sure, dtype, what):
    """float32: every logit within 2e-4 of the logits' spread.  bfloat16: per position the root mean square of the
    difference within 0.08 of the spread and the largest within 0.35 - a key, a state or an expert that is lost shows as
    several times that; a request is compared up to its first close call of a router, since from there on a 16-bit run may
    rightly have chosen another expert (nine tenths of all positions must remain; a 32-bit run is compared everywhere)."""
    spread = float(np.std(np.concatenate(list(want.values()))))
    compared = 0
    for name in want:
        count = want[name].shape[0] if dtype == "float32" else sure[name]
        compared += count
        if count == 0:
            continue
        difference = (got[name] - want[name])[:count]
        largest = np.abs(difference).max(axis=1)
        if dtype == "float32":
            worst = int(largest.argmax())
            assert largest[worst] <= 2e-4 * spread, f"{what}: request {name}, position {worst}: off by {largest[worst]:.3g} (spread of the logits {spread:.3g})"
        else:
            rms = np.sqrt((difference ** 2).mean(axis=1))
            worst = int(rms.argmax())
            assert rms[worst] <= 0.08 * spread and largest.max() <= 0.35 * spread, \
                f"{what}: request {name}, position {worst}: rms {rms[worst]:.3g}, largest {largest.max():.3g} (spread of the logits {spread:.3g})"
    total = sum(rows.shape[0] for rows in want.values())
    assert compared >= 0.9 * total, f"{what}: only {compared} of {total} positions are free of close calls: draw other weights or requests"


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
        engine = engine_for(folder, dtype, page, pool, slots=3)
        got = trace_tools.run_in_process(engine, steps)
        assert_logits(got, want, sure, dtype, f"{name}, {what}, {dtype}")
        assert engine.cache.free_slots() == 3 and all(group.pool.free_count == group.pool.num_pages for group in engine.cache.groups)
        assert (len(engine.cache.groups) == 0) == (name == "delta_only")
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


def test_long_decoding_across_many_chunks_and_pages(models):
    """A short prompt, then 200 tokens one by one: many chunks and pages pass, the states and the convolutions' inputs are
    carried 200 times."""
    folder, config, weights = models["mix"]
    requests = make_requests(config, (212,), seed=11)
    want, sure = plain_logits(config, weights, requests)
    steps = trace_tools.tail_one_by_one(requests, tail=200)
    engine = engine_for(folder, "float32", 8, 216)
    got = trace_tools.run_in_process(engine, steps)
    assert_logits(got, want, sure, "float32", "long decoding")


def test_the_replay_program_runs_the_model(models, tmp_path):
    folder, config, weights = models["plain"]
    requests = make_requests(config, (33, 12, 20), seed=2)
    want, sure = plain_logits(config, weights, requests)
    steps = trace_tools.mixed(requests, seed=1, max_live=2, decode_tail=5, max_portion=9)
    got = trace_tools.run_program(folder, "float32", steps, tmp_path / "out", extra_args=("--page-size", "4"))
    assert_logits(got, want, sure, "float32", "bin/trace_run")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["mix", "looped"])
def test_greedy_generation_through_the_scheduler(models, name, graphs):
    """Several prompts through ``Engine.generate`` with a small prompt budget and few slots: every generated token is the
    arg-max of the plain logits of its own prefix."""
    from pylon_b200.sampling.params import SamplingParams

    folder, config, weights = models[name]
    prompts = list(make_requests(config, (19, 3, 40, 11, 27, 8), seed=13).values())
    new_tokens = 12
    # with graphs, decode steps replay at their batch size and steps with prompt portions padded to captured sizes (rows
    # without tokens, tokens without a row): nothing of the padding may touch a state slot, a page or an expert's share
    engine = engine_for(folder, "float32", PAGE_SIZES[name], 4 * 64, slots=3, prefill_chunk_size=16, cuda_graphs=graphs)
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
    if graphs:
        replays = engine.step_function.graphs.replays
        assert replays["decode"] > 0 and replays["padded"] > 0, replays


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
def on(tensor, dtype=None):
    return tensor.to(device=DEVICE, dtype=dtype) if dtype is not None else tensor.to(DEVICE)


def fresh_cache(need, page, dtype, table=(4, 0, 6, 2, 5, 1, 3, 7), slots=2):
    from pylon_b200.parts.base import LayerCache

    cache = LayerCache(page_size=page)
    if need.kv is not None:
        cache.k_pages = torch.zeros(len(table), need.kv.n_kv_heads, page, need.kv.head_dim, device=DEVICE, dtype=dtype)
        cache.v_pages = torch.zeros(len(table), need.kv.n_kv_heads, page, need.kv.value_width, device=DEVICE, dtype=dtype) if need.kv.value_width else None
        cache.block_table = torch.tensor([list(table)], device=DEVICE, dtype=torch.int32)
    if need.state is not None:
        cache.state = torch.zeros(slots, *need.state.shape, device=DEVICE)
    return cache


def paged(rows, page_size, dtype, seed=0, spare=3):
    """Lays the rows ``[tokens, width]`` of one request into shuffled pages: (pages [P, 1, page_size, width], block table)."""
    count = -(-rows.shape[0] // page_size)
    order = torch.randperm(count + spare, generator=torch.Generator().manual_seed(seed)).tolist()[:count]
    pages = torch.full((count + spare, 1, page_size, rows.shape[1]), 7.0)
    for logical, page in enumerate(order):
        part = rows[logical * page_size : (logical + 1) * page_size]
        pages[page, 0, : part.shape[0]] = part
    return on(pages, dtype), on(torch.tensor([order], dtype=torch.int32))


def run_part(part, h, cutting, page, dtype, slot=1):
    """The part over one request's tokens in portions; pages in a shuffled order, the second of two state slots."""
    cache = fresh_cache(part.cache_need(), page, dtype)
    outs, cursor = [], 0
    for size in cutting:
        step = step_view((size,), (cursor,), dtype)
        step.slots = torch.tensor([slot], device=DEVICE, dtype=torch.int32)
        out = part.forward(on(h[cursor : cursor + size]), step, cache)
        outs.append(out.sum(dim=0) if out.dim() == 3 else out)
        cursor += size
    return torch.cat(outs).double().cpu()


def mixer_case(name, rand, matrix, width, eps):
    """(the mixer's configuration, its tensors, its part's description, the plain function) of a small made-up mixer."""
    from pylon_b200.parts import PartSpec

    bf = lambda t: t.to(torch.bfloat16)
    left = {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.7, "mask": {"size": 9}}
    right = {"heads": 6, "vdim": 5, "state": 9, "groups": 3, "norm_groups": 2, "conv": 3}
    w_left = {"q": matrix(48, width, 1.5), "k": matrix(24, width, 1.5), "v": matrix(40, width), "o": matrix(width, 80)}
    channels = 30 + 2 * 27
    w_right = {"in": matrix(30 + channels + 6, width, 1.5), "conv": bf(0.6 * rand(channels, 3)), "conv.b": bf(0.2 * rand(channels)), "dt_bias": bf(0.5 * rand(6)),
               "A_log": bf(-4.0 * torch.rand(6, generator=rand.generator)), "D": bf(1 + 0.3 * rand(6)), "norm": bf(1 + 0.2 * rand(30)), "o": matrix(width, 30)}
    attention = PartSpec("gqa_attention", {"width": width, "n_heads": 4, "n_kv_heads": 2, "head_dim": 12, "value_dim": 20, "scale": 0.7, "chunk": 9,
                                           "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
    recurrent = PartSpec("state_space", {"width": width, "n_heads": 6, "value_dim": 5, "state_dim": 9, "groups": 3, "norm_groups": 2, "conv_taps": 3,
                                         "norm_eps": eps})
    if name == "chunked":
        oracle = lambda h, w: plain.chunked_attention(h, w["q"], w["k"], w["v"], w["o"], 4, 2, 12, 20, 0.7, 9)
        return w_left, attention, oracle
    if name == "state_space":
        return w_right, recurrent, lambda h, w: plain.state_space(h, w, "", 6, 5, 9, 3, 2, eps)
    if name == "parallel":
        w = {**{"left." + k: v for k, v in w_left.items()}, **{"right." + k: v for k, v in w_right.items()},
             "left.out": bf(1 + 0.3 * rand(width)), "right.out": bf(1 + 0.3 * rand(width))}
        spec = PartSpec("parallel_mixers", {"width": width, "mixers": (attention, recurrent), "prefixes": ("left.", "right."),
                                            "norm_names": ("left.out", "right.out"), "norm_eps": eps})
        return w, spec, lambda h, w: plain.parallel_mixer(h, w, "", {"left": left, "right": right}, width, eps)
    heads, groups, dim, vdim, taps, decay_rank, gate_rank = 4, 2, 10, 14, 3, 7, 5
    w = {"q": matrix(groups * dim, width, 1.5), "k": matrix(groups * dim, width, 1.5), "v": matrix(heads * vdim, width, 1.5), "b": matrix(heads, width, 2.0),
         "q.conv": bf(0.6 * rand(groups * dim, taps)), "k.conv": bf(0.6 * rand(groups * dim, taps)), "v.conv": bf(0.6 * rand(heads * vdim, taps)),
         "A_log": bf(-3.0 * torch.rand(heads, generator=rand.generator)), "a1": matrix(decay_rank, width), "a2": matrix(heads * dim, decay_rank, 1.5),
         "dt_bias": bf(0.5 * rand(heads * dim)), "g1": matrix(gate_rank, width), "g2": matrix(heads * vdim, gate_rank, 2.0), "norm": bf(1 + 0.2 * rand(vdim)),
         "o": matrix(width, heads * vdim)}
    spec = PartSpec("gated_delta", {
        "width": width, "n_heads": heads, "n_kv_heads": groups, "head_dim": dim, "value_dim": vdim, "conv_taps": taps, "norm_eps": eps, "unit_eps": 1e-6,
        "decay": "channel", "decay_rank": decay_rank, "gate_rank": gate_rank, "gate_activation": "sigmoid",
        "names": {"decay_in": "a1", "decay": "a2", "gate_in": "g1", "gate": "g2"}})
    return w, spec, lambda h, w: plain.channel_delta(h, w, "", heads, groups, dim, vdim, eps)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["chunked", "state_space", "parallel", "channel_delta"])
def test_each_mixer_alone_against_its_plain_statement(name, dtype):
    """A mixer part from its normalised input to its delta for the stream: a prompt in one step, then the same in portions
    down to single tokens, and token by token from the start."""
    from pylon_b200.parts import MIXERS

    g = torch.Generator().manual_seed(21)
    width, eps, count, page = 56, 1e-5, 45, 8
    rand = lambda *shape: torch.randn(*shape, generator=g)
    rand.generator = g
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w, spec, oracle = mixer_case(name, rand, matrix, width, eps)
    part = MIXERS.build(spec)
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w) and all(tuple(w[k].shape) == tuple(declared[k].shape) for k in w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    h = rand(count, width).to(dtype)
    want = oracle(h.double(), {k: v.double() for k, v in w.items()})
    spread = float(want.std())
    limit = 0.06 * spread if dtype == torch.bfloat16 else 1e-4 * spread
    for cutting in ((count,), (20, 2, 1, 1, 13, 8), (1,) * 12 + (2, 2, 29), (9, 9, 9, 18), (8, 1, 9, 27)):
        got = run_part(part, h, cutting, page, dtype)
        assert float((got - want).abs().max()) <= limit, f"{name}, {cutting}: off by {float((got - want).abs().max()):.3g} of {spread:.3g}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_key_that_stands_out_at_both_ends_of_a_chunk(dtype):
    """Two keys far larger than the rest, each with a value of its own: one on the first position of a chunk, seen by the
    whole chunk and by nobody after it; one on the last position of a chunk, seen by its own token alone.  In a prompt, token
    by token across the edges, and in portions that end and start right at them; chunks that are no multiple of the page."""
    from pylon_b200.kernels import ops

    g = torch.Generator().manual_seed(5)
    count, chunk, page, heads, width, dv = 150, 37, 16, 4, 64, 24
    first, last = 2 * chunk, 3 * chunk - 1                       # positions 74 and 110
    rows = torch.randn(count, width, generator=g) * 0.3
    values = torch.randn(count, dv, generator=g) * 0.3
    rows[first], rows[last] = 3.0, 3.0
    values[first], values[last] = torch.linspace(-4.0, 4.0, dv), torch.linspace(5.0, -5.0, dv)
    queries = torch.randn(count, heads, width, generator=g) * 0.3 + 0.25
    pages, table = paged(rows, page, dtype, seed=3)
    value_pages, _ = paged(values, page, dtype, seed=3)
    scale = 0.5
    q, keys, vals = queries.to(dtype).double(), rows.to(dtype).double(), values.to(dtype).double()
    index = torch.arange(count)
    visible = (index[None, :] <= index[:, None]) & (index[None, :] // chunk == index[:, None] // chunk)
    scores = (torch.einsum("ihd,jd->hij", q, keys) * scale).masked_fill(~visible[None], -math.inf)
    weights = torch.softmax(scores, dim=-1)
    want = torch.einsum("hij,jv->ihv", weights, vals).reshape(count, heads * dv)
    assert float(weights[:, first : last, first].min()) > 0.8 and float(weights[:, last + 1 :, first].max()) == 0.0
    assert float(weights[:, last, last].min()) > 0.4 and float(weights[:, last + 1 :, last].max()) == 0.0 and float(weights[:, :first, first].max()) == 0.0

    def run(cutting):
        outs, cursor = [], 0
        for size in cutting:
            step = step_view((size,), (cursor,), dtype)
            outs.append(ops.paged_attention(on(queries[cursor : cursor + size].to(dtype)).view(size, heads * width), pages, value_pages, step.positions,
                                            step.token_row, step.q_start, step.kv_len, table, heads, step.max_q, step.max_kv, chunk=chunk, scale=scale))
            cursor += size
        return torch.cat(outs).double().cpu()

    tolerance = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    edge = last + 1
    for cutting in ((count,), (edge - 3,) + (1,) * 6 + (count - edge - 3,), (edge - 1, 1, count - edge), (edge, count - edge), (first, 1, 1, count - first - 2),
                    (first + 1, 2, count - first - 3), (first - 2,) + (1,) * (chunk + 4) + (count - first - chunk - 2,)):
        assert sum(cutting) == count
        torch.testing.assert_close(run(cutting), want, **tolerance)


def test_the_state_space_layer_reads_back_a_value_written_long_ago():
    """A head that does not decay: one token writes a row of its state, 400 tokens later one token reads that row, and
    nothing else touches it in between; the head beside it forgets within a few tokens.  The projections are unit matrices,
    so the layer's input is the columns [z | x | B | C | dt] themselves.  In one step and in portions."""
    from pylon_b200.parts import MIXERS, PartSpec

    heads, vdim, state, count, write, read, row = 2, 8, 16, 420, 3, 403, 5
    inner, columns = heads * vdim, 2 * heads * vdim + 2 * state + heads
    g = torch.Generator().manual_seed(2)
    h = torch.zeros(count, columns)
    h[:, :inner] = 2.0                                                   # z: the gate is open
    h[:, inner : 2 * inner] = torch.randn(count, inner, generator=g)      # x
    h[:, 2 * inner + 2 * state :] = 1.0                                   # dt
    h[write, 2 * inner + row] = 4.0                                       # B of the writing token
    h[read, 2 * inner + state + row] = 4.0                                # C of the reading token
    h[read - 1, 2 * inner + state + row + 1] = 4.0                        # the token before reads the row beside it: nothing there
    h = h.to(torch.bfloat16).float()
    w = {"in": torch.eye(columns), "o": torch.eye(inner), "conv": torch.ones(inner + 2 * state, 1), "conv.b": torch.zeros(inner + 2 * state),
         "dt_bias": torch.zeros(heads), "A_log": torch.tensor([-30.0, 1.0]), "D": torch.zeros(heads), "norm": torch.ones(inner)}
    # the plain statement without its closing norm, to see the read-out itself: the far value comes back whole in head 0
    x3 = plain.silu(h[write, inner : inner + vdim].double())
    want = plain.state_space(h.double(), {k: v.double() for k, v in w.items()}, "", heads, vdim, state, 1, heads, 1e-5)
    step_size = float(plain.softplus(torch.tensor(1.0, dtype=torch.float64)))
    far = float(plain.silu(torch.tensor(4.0, dtype=torch.float64))) ** 2 * step_size * x3 * float(plain.silu(torch.tensor(2.0, dtype=torch.float64)))
    torch.testing.assert_close(want[read, :vdim], plain.rms_unit(far, 1e-5), rtol=1e-6, atol=1e-6)
    assert float(want[read, vdim:].abs().max()) < 1e-3 and float(want[read - 1].abs().max()) < 1e-3 and float(want[read + 1].abs().max()) == 0.0
    part = MIXERS.build(PartSpec("state_space", {"width": columns, "n_heads": heads, "value_dim": vdim, "state_dim": state, "groups": 1, "norm_groups": heads,
                                                 "conv_taps": 1, "norm_eps": 1e-5}))
    part.load({k: on(v) for k, v in w.items()}, torch.float32, torch.device(DEVICE))
    for cutting in ((count,), (2, 2) + (1,) * 399 + (17,), (write + 1, read - write - 1, 1, count - read - 1), (200, 203, 17)):
        assert sum(cutting) == count
        got = run_part(part, h, cutting, 8, torch.float32)
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["state_space", "channel_delta", "parallel"])
def test_unequal_requests_in_one_step_against_each_alone(name, dtype):
    """Three requests of 1, 17 and 6 new tokens at different places of their sequences in one step, in state slots and pages
    that another request used before: every request's result is the one it has alone."""
    from pylon_b200.parts import MIXERS

    g = torch.Generator().manual_seed(8)
    width, eps, page = 56, 1e-5, 8
    rand = lambda *shape: torch.randn(*shape, generator=g)
    rand.generator = g
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w, spec, oracle = mixer_case(name, rand, matrix, width, eps)
    part = MIXERS.build(spec)
    declared = {d.name: d for d in part.tensors()}
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    before, new = (12, 0, 30), (1, 17, 6)                      # tokens each request already holds, and brings
    inputs = [rand(b + n, width).to(dtype) for b, n in zip(before, new)]
    want = [oracle(h.double(), {k: v.double() for k, v in w.items()}) for h in inputs]
    need = part.cache_need()
    pages_each = 5
    cache = fresh_cache(need, page, dtype, table=tuple(range(3 * pages_each)), slots=4)
    slots = (2, 0, 3)
    if need.kv is not None:
        cache.block_table = torch.tensor([[9, 3, 12, 0, 7], [1, 14, 5, 10, 2], [6, 11, 4, 13, 8]], device=DEVICE, dtype=torch.int32)
        cache.k_pages.fill_(3.0)                               # what an earlier request left in the pages
        cache.v_pages.fill_(-2.0)

    def step_for(rows, sizes, starts):
        step = step_view(sizes, starts, dtype)
        step.slots = torch.tensor([slots[r] for r in rows], device=DEVICE, dtype=torch.int32)
        return step

    def run(rows, sizes, starts):
        step = step_for(rows, sizes, starts)
        saved = cache.block_table
        if need.kv is not None:
            cache.block_table = saved[list(rows)].contiguous()
        out = part.forward(on(torch.cat([inputs[r][s : s + n] for r, n, s in zip(rows, sizes, starts)])), step, cache)
        cache.block_table = saved
        return (out.sum(dim=0) if out.dim() == 3 else out).double().cpu()

    if need.state is not None:
        cache.state.zero_()                                    # a slot is handed out cleared; the pages are not
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
@pytest.mark.parametrize("width,ff,tokens", [(40, 24, 1), (56, 100, 9), (256, 136, 300)])
def test_the_gated_unit_with_relu_and_biases(width, ff, tokens, dtype):
    from pylon_b200.parts import FEED_FORWARDS, PartSpec

    g = torch.Generator().manual_seed(3)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w = {"gate": matrix(ff, width, 1.5), "up": matrix(ff, width, 1.5), "down": matrix(width, ff), "gate.b": rand(ff).to(torch.bfloat16),
         "up.b": rand(ff).to(torch.bfloat16), "down.b": rand(width).to(torch.bfloat16)}
    part = FEED_FORWARDS.build(PartSpec("gated_unit", {"width": width, "intermediate": ff, "activation": "relu", "bias": True, "bias_suffix": ".b",
                                                       "names": {"gate": "gate", "up": "up", "down": "down"}}))
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    h = rand(tokens, width).to(dtype)
    want = plain.dense_relu_glu(h.double(), *(w[k].double() for k in ("gate", "gate.b", "up", "up.b", "down", "down.b")))
    out = part.forward(on(h), step_view((tokens,), (0,), dtype))
    got = (out.sum(dim=0) if out.dim() == 3 else out).double().cpu()
    spread = float(want.std())
    limit = 0.05 * spread if dtype == torch.bfloat16 else 1e-4 * spread
    assert float((got - want).abs().max()) <= limit


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,experts,top,tokens", [(40, 12, 3, 1, 1), (56, 20, 5, 5, 7), (48, 24, 10, 4, 150), (256, 128, 6, 2, 200), (128, 64, 33, 3, 70),
                                                          (64, 40, 2, 1, 40), (256, 136, 4, 2, 700), (384, 256, 3, 1, 600), (128, 520, 5, 3, 333)])
def test_the_mixture_of_experts_against_token_by_token(width, ff, experts, top, tokens, dtype):
    """Router logits in 32-bit with a bias, the largest ``top``, the softmax over just those, the chosen experts' gated units:
    one token, few and many, fewer tokens than experts and more, every expert used, tiles that are partly filled; the last shapes
    have enough tokens an expert for the grouped tensor-core product (inner widths that are and are not whole column tiles).  Tokens
    whose choice hangs on a margin that 16-bit rounding of the input can turn are left out of the 16-bit comparison."""
    from pylon_b200.parts import FEED_FORWARDS, PartSpec

    g = torch.Generator().manual_seed(17)
    rand = lambda *shape: torch.randn(*shape, generator=g)
    matrix = lambda out, inner, gain=1.0: (rand(out, inner) * gain / math.sqrt(inner)).to(torch.bfloat16)
    w = {"router": matrix(experts, width, 2.0), "router.b": rand(experts).to(torch.bfloat16)}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = matrix(ff, width, 1.5), matrix(ff, width, 1.5), matrix(width, ff, 1.5)
    part = FEED_FORWARDS.build(PartSpec("expert_mixture", {"width": width, "intermediate": ff, "experts": experts, "top": top, "activation": "silu",
                                                           "router_bias": True}))
    declared = {d.name: d for d in part.tensors()}
    assert set(declared) == set(w) and all(tuple(w[k].shape) == tuple(declared[k].shape) for k in w)
    part.load({k: on(v, torch.float32 if declared[k].role == "vector" else dtype) for k, v in w.items()}, dtype, torch.device(DEVICE))
    h = rand(tokens, width).to(dtype)
    doubles = {k: v.double() for k, v in w.items()}
    want = plain.expert_mixture(h.double(), doubles, "", experts, top)
    margin = plain.route_margin(h.double(), doubles["router"], doubles["router.b"], top)
    sure = margin > (1e-4 if dtype == torch.float32 else 0.02)
    assert int(sure.sum()) >= 0.9 * tokens
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
    assert torch.equal(again, got[order])
