"""Zemavik without a GPU: its configuration, the model description built from it (the looped run order and where a pass is
entered, tensor names and shapes, what each run keeps between steps), the sizes that only a checkpoint's shapes give, and
the cache manager over its chunked groups and state slots."""
from __future__ import annotations

import copy
import json

import pytest
import torch

import plain_zemavik as plain
from pylon_b200.cache.manager import CacheManager
from pylon_b200.config.model_config import ConfigError, ZemavikConfig
from pylon_b200.config.registry import ARCHITECTURES, architecture_of, read_config
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.parts.base import KVNeed, StateNeed

CONFIG = {
    "architecture": "Zemavik", "vocab": 50, "width": 24, "max_positions": 96, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.5, "mask": {"size": 12}},
                                       "right": {"heads": 6, "vdim": 2, "state": 5, "groups": 3, "norm_groups": 2, "conv": 3}},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "conv": 4, "decay_rank": 5, "gate_rank": 7},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 2}}},
        {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.25},
                                       "right": {"heads": 2, "vdim": 4, "state": 3, "groups": 1, "norm_groups": 1, "conv": 1}},
         "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 8, "conv": 2, "decay_rank": 2, "gate_rank": 2}, "mlp": None},
    ],
}


def built(data=CONFIG, max_positions=64):
    config = ZemavikConfig.from_dict(data)
    return config, ARCHITECTURES["Zemavik"].build_spec(config, max_positions)


def test_the_configuration_reads_every_key_and_writes_it_back():
    config = ZemavikConfig.from_dict(CONFIG)
    assert (config.vocab, config.width, config.max_positions, config.norm_eps, config.loop) == (50, 24, 96, 1e-6, (1, 3, 3))
    first, second, third, fourth = config.layers
    assert first.kind == "parallel" and first.delta is None
    assert (first.left.heads, first.left.kv_heads, first.left.dim, first.left.vdim, first.left.scale, first.left.chunk) == (4, 2, 8, 4, 0.5, 12)
    assert (first.right.heads, first.right.vdim, first.right.state, first.right.groups, first.right.norm_groups, first.right.conv) == (6, 2, 5, 3, 2, 3)
    assert (first.mlp.kind, first.mlp.ff, first.mlp.experts) == ("dense", 40, None)
    assert second.kind == "channel_delta" and second.left is None
    assert (second.delta.heads, second.delta.kv_heads, second.delta.dim, second.delta.vdim, second.delta.conv, second.delta.decay_rank,
            second.delta.gate_rank) == (4, 2, 6, 3, 4, 5, 7)
    assert (second.mlp.kind, second.mlp.ff, second.mlp.experts, second.mlp.top) == ("moe", 16, 3, 2)
    assert third.left.chunk is None and third.mlp is None and fourth.mlp is None
    assert config.to_dict() == CONFIG
    assert ZemavikConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config


def test_the_registry_finds_the_architecture(tmp_path):
    assert architecture_of(CONFIG) is ARCHITECTURES["Zemavik"]
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    architecture, config = read_config(tmp_path)
    assert architecture.name == "Zemavik" and isinstance(config, ZemavikConfig)


@pytest.mark.parametrize("loop,order", [
    ({"start": 1, "stop": 3, "times": 3}, [0, -1, 2, -1, 2, -1, 2, 3]),
    ({"start": 0, "stop": 4, "times": 2}, [-0.5, 1, 2, 3, -0.5, 1, 2, 3]),
    ({"start": 3, "stop": 4, "times": 2}, [0, 1, 2, -3, -3]),
    ({"start": 2, "stop": 2, "times": 5}, [0, 1, 2, 3]),
    ({"start": 0, "stop": 2, "times": 1}, [-0.5, 1, 2, 3]),
    (None, [0, 1, 2, 3]),
])
def test_the_run_order_repeats_the_loop_and_marks_where_a_pass_is_entered(loop, order):
    """A negative entry: that layer runs behind the map of stream and embedding output (-0.5 stands for layer 0).  The first
    pass is entered through the map too, and a loop that runs once still has it."""
    data = {key: value for key, value in CONFIG.items() if key != "loop"}
    if loop is not None:
        data["loop"] = loop
    config, spec = built(data)
    got = [(-run.layer if run.layer else -0.5) if run.reenter else run.layer for run in spec.order]
    assert got == order
    assert [(run.layer, run.reenter) for run in spec.order] == plain.run_order(data)
    assert all(run.cache_of is None and not run.add_embedding for run in spec.order)   # every pass has caches of its own
    assert (spec.reentry_name == "loop.in") == any(entry < 0 for entry in order)


def test_the_description_names_the_checkpoints_tensors():
    config, spec = built()
    assert spec.position_name == "pos" and spec.position_rows == 96 and spec.max_positions == 64 and spec.lm_head_name is None
    decls = DecoderModel(spec).tensor_decls()
    shapes = {name: tuple(decl.shape) for name, decl in decls.items()}
    experts = {f"l1.mlp.e{e}.{key}": shape for e in range(3) for key, shape in (("gate", (16, 24)), ("up", (16, 24)), ("down", (24, 16)))}
    assert shapes == {
        "embed": (50, 24), "pos": (96, 24), "loop.in": (24, 48), "final.norm": (24,),
        "l0.norm1": (24,), "l0.norm2": (24,), "l0.mix.left.q": (32, 24), "l0.mix.left.k": (16, 24), "l0.mix.left.v": (8, 24), "l0.mix.left.o": (24, 16),
        "l0.mix.right.in": (12 + 12 + 30 + 6, 24), "l0.mix.right.conv": (42, 3), "l0.mix.right.conv.b": (42,), "l0.mix.right.dt_bias": (6,),
        "l0.mix.right.A_log": (6,), "l0.mix.right.D": (6,), "l0.mix.right.norm": (12,), "l0.mix.right.o": (24, 12), "l0.mix.left.out": (24,),
        "l0.mix.right.out": (24,), "l0.mlp.gate": (40, 24), "l0.mlp.gate.b": (40,), "l0.mlp.up": (40, 24), "l0.mlp.up.b": (40,), "l0.mlp.down": (24, 40),
        "l0.mlp.down.b": (24,),
        "l1.norm1": (24,), "l1.norm2": (24,), "l1.mix.q": (12, 24), "l1.mix.q.conv": (12, 4), "l1.mix.k": (12, 24), "l1.mix.k.conv": (12, 4),
        "l1.mix.v": (12, 24), "l1.mix.v.conv": (12, 4), "l1.mix.b": (4, 24), "l1.mix.A_log": (4,), "l1.mix.norm": (3,), "l1.mix.a1": (5, 24),
        "l1.mix.a2": (24, 5), "l1.mix.dt_bias": (24,), "l1.mix.g1": (7, 24), "l1.mix.g2": (12, 7), "l1.mix.o": (24, 12),
        "l1.mlp.router": (3, 24), "l1.mlp.router.b": (3,), **experts,
        "l2.norm1": (24,), "l2.mix.left.q": (16, 24), "l2.mix.left.k": (16, 24), "l2.mix.left.v": (16, 24), "l2.mix.left.o": (24, 16),
        "l2.mix.right.in": (8 + 8 + 6 + 2, 24), "l2.mix.right.conv": (14, 1), "l2.mix.right.conv.b": (14,), "l2.mix.right.dt_bias": (2,),
        "l2.mix.right.A_log": (2,), "l2.mix.right.D": (2,), "l2.mix.right.norm": (8,), "l2.mix.right.o": (24, 8), "l2.mix.left.out": (24,),
        "l2.mix.right.out": (24,),
        "l3.norm1": (24,), "l3.mix.q": (4, 24), "l3.mix.q.conv": (4, 2), "l3.mix.k": (4, 24), "l3.mix.k.conv": (4, 2), "l3.mix.v": (8, 24),
        "l3.mix.v.conv": (8, 2), "l3.mix.b": (1, 24), "l3.mix.A_log": (1,), "l3.mix.norm": (8,), "l3.mix.a1": (2, 24), "l3.mix.a2": (4, 2),
        "l3.mix.dt_bias": (4,), "l3.mix.g1": (2, 24), "l3.mix.g2": (8, 2), "l3.mix.o": (24, 8),
    }
    vectors = ("l0.norm1", "l0.mix.right.conv", "l0.mix.right.A_log", "l0.mix.left.out", "l0.mlp.gate.b", "l1.mix.q.conv", "l1.mix.dt_bias", "l1.mix.norm",
               "l1.mlp.router", "l1.mlp.router.b", "final.norm")
    assert all(decls[name].role == "vector" for name in vectors)     # kept in 32-bit whatever the compute dtype


def test_the_checkpoints_shapes_give_the_widths_of_the_narrow_middles():
    data = copy.deepcopy(CONFIG)
    for index in (1, 3):
        del data["layers"][index]["mixer"]["decay_rank"], data["layers"][index]["mixer"]["gate_rank"]
    config = ZemavikConfig.from_dict(data)
    with pytest.raises(ConfigError, match="middles"):
        ARCHITECTURES["Zemavik"].build_spec(config, 64)
    shapes = {"l1.mix.a1": (9, 24), "l1.mix.g1": (11, 24), "l3.mix.a1": (3, 24), "l3.mix.g1": (1, 24)}
    sized = config.with_checkpoint_sizes(shapes.get)
    assert [(layer.delta.decay_rank, layer.delta.gate_rank) for layer in sized.layers if layer.delta] == [(9, 11), (3, 1)]
    decls = DecoderModel(ARCHITECTURES["Zemavik"].build_spec(sized, 64)).tensor_decls()
    assert tuple(decls["l1.mix.a2"].shape) == (24, 9) and tuple(decls["l1.mix.g2"].shape) == (12, 11) and tuple(decls["l3.mix.g2"].shape) == (8, 1)


def test_what_each_run_keeps_between_steps():
    config, spec = built()
    model = DecoderModel(spec)
    needs = model.cache_needs()
    assert len(needs) == 8
    # both halves of a layer of two mixers keep something: pages for the attention, a slot for the state-space layer (its
    # heads' matrices and the convolution's last two inputs)
    assert needs[0].kv == KVNeed(2, 8, None, 4, 12) and needs[0].state == StateNeed((6 * 5 * 2 + 2 * 42,), torch.float32)
    for run in (1, 3, 5):
        assert needs[run].kv is None and needs[run].state.dtype == torch.float32
    for run in (2, 4, 6):   # no chunks: every earlier key stays; one tap: no inputs kept
        assert needs[run].kv == KVNeed(2, 8, None, None, None) and needs[run].state == StateNeed((2 * 3 * 4,), torch.float32)
    assert needs[7].kv is None
    manager = CacheManager(needs, [None] * 8, page_size=4, num_pages=40, max_requests=2)
    assert [len(group.runs) for group in manager.groups] == [1, 3]
    request = manager.open("a", 100)
    for _ in range(10):
        manager.prepare([(request, 5)])
        manager.commit(request)
    # 50 tokens held, pages of 4: the chunked layer reads back to position 48 only, the others keep every page
    assert [len(request.held(g)) for g in range(2)] == [1, 13]
    manager.close(request)
    manager.check()
    assert manager.free_pages() == [40, 40]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("heads", 3), "cannot be grouped"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("groups", 4), "cannot be grouped"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("norm_groups", 5), "equal parts"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "cannot be grouped"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv"), "unknown feed-forward"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 4), "cannot use"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda c: c["loop"].__setitem__("stop", 5), "loop"),
    (lambda c: c["loop"].__setitem__("start", 3) or c["loop"].__setitem__("stop", 2), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "times"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("max_positions"), "max_positions"),
])
def test_what_the_configuration_refuses(change, message):
    data = copy.deepcopy(CONFIG)
    change(data)
    with pytest.raises(ConfigError, match=message):
        ZemavikConfig.from_dict(data)
