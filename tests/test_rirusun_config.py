"""Rirusun without a GPU: its configuration, the model description built from it (the looped run order, tensor names and
shapes, what each run keeps between steps), the size that only a checkpoint's shape gives, the rows of the bias table, and the
cache manager over a windowed group whose first pages stay."""
from __future__ import annotations

import copy
import json

import pytest
import torch

import plain_rirusun as plain
from pylon_b200.cache.manager import CacheManager
from pylon_b200.config.model_config import ConfigError, RirusunConfig
from pylon_b200.config.registry import ARCHITECTURES, architecture_of, read_config
from pylon_b200.models.decoder import DecoderModel
from pylon_b200.parts.attention import distance_bucket
from pylon_b200.parts.base import KVNeed, StateNeed

CONFIG = {
    "architecture": "Rirusun", "vocab": 50, "width": 24, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.5, "bias_max": 30, "bias_rows": 10,
                                                "mask": {"size": 12, "keep_first": 5}},
                                       "left_scale": 0.7, "right": {"width": 12, "blocks": 3, "conv": 3}, "right_scale": 1.5},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": 20}}},
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 6, "vdim": 10, "gate_cap": 12.0}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "scale": 0.3,
                                               "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 1}}},
        {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.25, "bias_max": 9, "bias_rows": 4},
                                       "left_scale": 1.0, "right": {"width": 8, "blocks": 1, "conv": 1}, "right_scale": 1.0},
         "mlp": None},
    ],
}


def built(data=CONFIG, max_positions=64):
    config = RirusunConfig.from_dict(data)
    return config, ARCHITECTURES["Rirusun"].build_spec(config, max_positions)


def test_the_configuration_reads_every_key_and_writes_it_back():
    config = RirusunConfig.from_dict(CONFIG)
    assert (config.vocab, config.width, config.embedding_scale, config.norm_eps, config.loop) == (50, 24, 2.5, 1e-6, (1, 3, 3))
    first, second, third, fourth = config.layers
    assert first.kind == "parallel" and first.memory is None and first.latent is None
    left = first.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.bias_max, left.bias_rows, left.window, left.keep_first) == (4, 2, 8, 4, 0.5, 30, 10, 12, 5)
    assert (first.right.width, first.right.blocks, first.right.conv, first.left_scale, first.right_scale) == (12, 3, 3, 0.7, 1.5)
    assert (first.mlp.ff, first.mlp.experts, first.mlp.top, first.mlp.groups, first.mlp.groups_keep, first.mlp.shared_ff) == (16, 6, 2, 3, 2, 20)
    assert second.memory == (2, 6, 10, 12.0) and second.mlp is None
    assert third.latent[:6] == (3, 8, 4, 6, 10, 0.3) and third.latent[6].dims == 4 and dict(third.latent[6].scaling)["factor"] == 4.0
    assert (third.mlp.groups, third.mlp.shared_ff) == (None, None)
    assert fourth.left.window is None and fourth.left.keep_first == 0
    assert config.to_dict() == CONFIG
    assert RirusunConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config
    assert config.run_order() == plain.run_order(CONFIG) == [0, 1, 2, 1, 2, 1, 2, 3]


def test_the_registry_finds_the_architecture(tmp_path):
    assert architecture_of(CONFIG) is ARCHITECTURES["Rirusun"]
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    architecture, config = read_config(tmp_path)
    assert architecture.name == "Rirusun" and isinstance(config, RirusunConfig)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="other"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "cannot be grouped"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5), "equal parts"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot use"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=6), "exceeds rot_dim"),
    (lambda c: c["loop"].update(stop=7), "does not fit"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
])
def test_what_the_configuration_refuses(change, text):
    data = copy.deepcopy(CONFIG)
    change(data)
    with pytest.raises(ConfigError, match=text):
        RirusunConfig.from_dict(data)


def test_the_model_description():
    config, spec = built()
    assert [run.layer for run in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3] and all(run.cache_of is None and not run.add_embedding and not run.reenter for run in spec.order)
    assert spec.embedding_scale == 2.5 and spec.lm_head_name == "head" and spec.final_norm.kind == "dynamic_tanh"
    model = DecoderModel(spec)
    decls = model.tensor_decls()
    expected = {
        "embed": (50, 24), "head": (50, 24), "final.norm": (24,), "final.norm.alpha": (), "final.norm.b": (24,),
        "l0.norm1": (24,), "l0.norm1.alpha": (), "l0.norm1.b": (24,),
        "l0.mix.left.q": (32, 24), "l0.mix.left.k": (16, 24), "l0.mix.left.v": (8, 24), "l0.mix.left.o": (24, 16), "l0.mix.left.q.norm": (32,),
        "l0.mix.left.k.norm": (16,), "l0.mix.left.rel": (10, 4), "l0.mix.left.sink": (4,),
        "l0.mix.right.y": (12, 24), "l0.mix.right.y.b": (12,), "l0.mix.right.x": (12, 24), "l0.mix.right.x.b": (12,), "l0.mix.right.conv": (12, 3),
        "l0.mix.right.conv.b": (12,), "l0.mix.right.ra": (3, 4, 4), "l0.mix.right.ra.b": (3, 4), "l0.mix.right.ri": (3, 4, 4), "l0.mix.right.ri.b": (3, 4),
        "l0.mix.right.lam": (12,), "l0.mix.right.o": (24, 12),
        "l0.mlp.router": (6, 24), "l0.mlp.correction": (6,), "l0.mlp.shared.up": (20, 24), "l0.mlp.shared.down": (24, 20), "l0.mlp.shared.sg": (1, 24),
        "l1.mix.q": (12, 24), "l1.mix.k": (12, 24), "l1.mix.v": (20, 24), "l1.mix.g": (20, 24), "l1.mix.o": (24, 20), "l1.mix.norm": (20,),
        "l1.mix.i": (2, 24), "l1.mix.i.b": (2,), "l1.mix.f": (2, 24), "l1.mix.f.b": (2,),
        "l2.mix.q": (36, 24), "l2.mix.dkv": (14, 24), "l2.mix.dkv.norm": (10,), "l2.mix.uk": (24, 10), "l2.mix.uv": (18, 10), "l2.mix.o": (24, 18),
        "l2.mlp.router": (3, 24), "l2.mlp.correction": (3,),
    }
    for name, shape in expected.items():
        assert tuple(decls[name].shape) == shape, name
    assert {f"l0.mlp.e{e}.{key}" for e in range(6) for key in ("up", "down")} <= set(decls) and "l0.mlp.e0.gate" not in decls
    assert not any(name.startswith("l1.mlp.") or name.startswith("l3.mlp.") or name.endswith("norm2") for name in decls)
    needs = model.cache_needs()
    assert needs[0].kv == KVNeed(2, 8, 12, 4, None, 5) and needs[0].state == StateNeed((12 * 3,))
    assert needs[1].kv is None and needs[1].state == StateNeed((2 * (6 * 10 + 6 + 1),)) and needs[3] == needs[1] == needs[5]
    assert needs[2].kv == KVNeed(1, 14, None, 0) and needs[2].state is None
    assert needs[7].kv == KVNeed(2, 8, None, None, None, 0) and needs[7].state == StateNeed((8,))
    assert model.takes_padding()


def test_the_rows_of_the_bias_table_come_from_the_checkpoints_shape():
    data = copy.deepcopy(CONFIG)
    for layer in (data["layers"][0], data["layers"][3]):
        del layer["mixer"]["left"]["bias_rows"]
    config = RirusunConfig.from_dict(data)
    with pytest.raises(ConfigError, match="rows of the bias table"):
        ARCHITECTURES["Rirusun"].build_spec(config, 64)
    shapes = {"l0.mix.left.rel": (10, 4), "l3.mix.left.rel": (4, 2)}
    sized = config.with_checkpoint_sizes(lambda name: shapes.get(name))
    assert sized.layers[0].left.bias_rows == 10 and sized.layers[3].left.bias_rows == 4
    assert sized == RirusunConfig.from_dict(CONFIG)


def test_a_distance_finds_its_row_of_the_bias_table():
    assert [distance_bucket(n, 10, 30) for n in (0, 4, 5, 6, 29, 30, 500)] == [plain.distance_bucket(n, 10, 30) for n in (0, 4, 5, 6, 29, 30, 500)]
    assert [distance_bucket(n, 10, 30) for n in (0, 4, 5, 30, 500)] == [0, 4, 5, 9, 9]
    assert [distance_bucket(n, 4, 9) for n in range(12)] == [0, 1, 2, 2, 2, 3, 3, 3, 3, 3, 3, 3]


def test_the_first_pages_of_a_windowed_group_stay():
    """A window of 12 with 5 kept first tokens over pages of 4: the two pages that hold the first five positions are never given back,
    the pages behind them are, one after the other, as the window passes."""
    need = KVNeed(2, 8, 12, 4, None, 5)
    from pylon_b200.parts.base import CacheNeed

    manager = CacheManager([CacheNeed(kv=need)], [None], page_size=4, num_pages=40, max_requests=2)
    request = manager.open("a", 200)
    manager.prepare([(request, 30)])
    manager.commit(request)
    table = request.tables[0]
    assert table[0] >= 0 and table[1] >= 0            # positions 0..7: the kept tokens' pages
    assert table[2] == table[3] == -1                 # positions 8..15: wholly behind the window of the next token (it reads from 19 on)
    assert all(page >= 0 for page in table[4:])
    for _ in range(40):
        manager.prepare([(request, 1)])
        manager.commit(request)
        manager.check()
    table = request.tables[0]
    assert table[0] >= 0 and table[1] >= 0 and all(page == -1 for page in table[2 : (70 - 12 + 1) // 4])
    assert len(request.held(0)) <= 2 + 4
    assert manager.groups[0].lifetime_pages(200, 1) >= len(request.held(0))
    manager.close(request)
    assert manager.groups[0].pool.free_count == 40
