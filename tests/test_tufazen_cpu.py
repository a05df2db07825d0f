"""The Tufazen decoder without a GPU: configuration (round trip, errors that name the key), the layout's parts, tensor names
and schedule, state needs, the rotation table against the plain statement's frequencies, and the plain statement against
values worked by hand."""
import copy
import json
import math

import pytest
import torch

import plain_tufazen as plain
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.config.base import ConfigError
from scriptling_llm_lib_b200.config.registry import architecture_for
from scriptling_llm_lib_b200.config.tufazen import TufazenConfig
from scriptling_llm_lib_b200.engine.layout import looped_schedule
from scriptling_llm_lib_b200.engine.model import DecoderModel

RAW = {
    "architecture": "Tufazen", "vocab": 70, "width": 40, "norm": {"eps": 1e-5}, "logit_scale": 0.25,
    "embedding": {"bigram": {"buckets": 29, "mul_cur": 3, "mul_prev": 11}}, "token_side": {"dim": 6},
    "loop": {"start": 1, "stop": 2, "times": 3},
    "layers": [
        {"type": "attention", "mixer": {"dim": 8, "heads": 4, "kv_heads": 2, "scale": 0.3, "softcap": 7.0, "vdim": 8,
                                        "rot": {"base": 500.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 4.0, "original": 32, "slow": 1.0}}},
         "mlp": {"ff": 20, "kind": "dense", "limit": 1.5}},
        {"type": "latent_attention", "mixer": {"dim": 6, "heads": 3, "kv_rank": 10, "q_rank": 12, "rot_dim": 4, "scale": 0.3, "vdim": 5,
                                               "rot": {"base": 100.0, "dims": 4}},
         "mlp": {"expert": {"ff": 8}, "kind": "moe", "router": {"experts": 6, "groups": {"count": 3, "keep": 2}, "top": 2},
                 "shared": {"ff": 12}}},
        {"type": "attention", "mixer": {"dim": 4, "heads": 2, "kv_heads": 1, "scale": 0.5, "vdim": 4}, "mlp": None},
    ],
}


def test_the_configuration_reads_back_as_it_was_written():
    cfg = TufazenConfig.from_dict(RAW, "t")
    assert cfg.to_json_dict() == RAW
    assert cfg.layers[2].mixer.rot is None and cfg.layers[2].mixer.softcap is None and cfg.layers[2].mlp is None
    assert TufazenConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())), "t") == cfg
    bare = {k: v for k, v in RAW.items() if k not in ("embedding", "token_side", "loop", "logit_scale")}
    c2 = TufazenConfig.from_dict(bare, "t")
    assert c2.bigram is None and c2.side_dim is None and c2.loop is None and c2.logit_scale == 1.0


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "vdim"), 6, "vdim"),
    (("layers", 0, "mixer", "rot", "dims"), 5, "dims"), (("layers", 1, "mlp", "router", "top"), 5, "router"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "router"), (("loop", "stop"), 4, "loop"),
    (("layers", 1, "type"), "scan", "type"), (("norm", "eps"), 0, "eps"), (("embedding", "bigram", "buckets"), 0, "buckets"),
])
def test_errors_name_the_key(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        TufazenConfig.from_dict(raw, "t")
    assert word in str(e.value)


def test_the_layout_names_the_designs_tensors_and_schedule():
    arch = architecture_for("Tufazen")
    layout = arch.layout(arch.config_class.from_dict(RAW, "t"))
    model = DecoderModel(layout)
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert shapes["embed"] == (70, 40) and shapes["bigram"] == (30, 40) and shapes["loop.step"] == (3, 40)
    assert shapes["side.embed"] == (70, 18) and shapes["head"] == (70, 40)
    assert shapes["l0.mix.q"] == (32, 40) and shapes["l0.mix.k"] == (16, 40) and shapes["l0.mix.g"] == (32, 40)
    assert shapes["l0.mix.sink"] == (4,) and shapes["l0.mix.o"] == (40, 32) and "l0.mix.v" not in shapes
    assert shapes["l0.norm1.alpha"] == () and shapes["l0.norm1.b"] == (40,) and "l0.norm2" not in shapes
    assert shapes["l1.mix.dq"] == (12, 40) and shapes["l1.mix.uq"] == (30, 12) and shapes["l1.mix.dkv"] == (14, 40)
    assert shapes["l1.mix.dkv.norm"] == (10,) and shapes["l1.mix.uk"] == (18, 10) and shapes["l1.mix.uv"] == (15, 10)
    assert shapes["l1.mix.g"] == (3, 40) and shapes["l1.mlp.router"] == (6, 40) and shapes["l1.mlp.e5.down"] == (40, 8)
    assert shapes["l1.mlp.shared.gate"] == (12, 40) and shapes["l2.side.proj"] == (40, 6) and "l2.mlp.gate" not in shapes
    # layer 1 three times, a cache unit for every appearance, the pass vectors before its appearances
    assert [(e.layer, e.cache_unit, e.before) for e in layout.schedule] == [(0, 0, ()), (1, 1, (0,)), (1, 2, (1,)), (1, 3, (2,)), (2, 4, ())]
    needs = model.cache_needs()
    assert needs[0].kv_heads == 2 and needs[0].head_dim == 8 and needs[0].value_dim == 8
    assert needs[1] == needs[2] == needs[3] and needs[1].head_dim == 14 and needs[1].value_dim == 0
    assert model.state_needs()["embedding"].dtype == torch.int32 and model.graph_safe()


def test_a_looped_schedule():
    s = looped_schedule(5, 1, 3, 2, before_pass=lambda t: (t,))
    assert [e.layer for e in s] == [0, 1, 2, 1, 2, 3, 4] and [e.cache_unit for e in s] == list(range(7))
    assert [e.before for e in s] == [(), (0,), (), (1,), (), (), ()]
    assert plain.run_order(5, {"start": 1, "stop": 3, "times": 2}) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None), (4, None)]
    with pytest.raises(ValueError):
        looped_schedule(3, 2, 5, 2)


def test_the_rotation_table_has_the_ramped_frequencies():
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding, YarnScaling
    sc = {"factor": 6.0, "fast": 16.0, "original": 256, "slow": 1.0}
    for dims, base in ((16, 20000.0), (8, 300.0), (32, 250000.0)):
        f, amp = plain.frequencies(dims, base, sc)
        enc = RotaryEncoding(dims, dims, base, YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]), "interleaved")
        enc.prepare(50, "cpu")
        table, width, interleaved = enc.rotation()
        assert width == dims and interleaved and abs(amp - (0.1 * math.log(6.0) + 1.0)) < 1e-12
        for p in (0, 1, 7, 49):
            for i in (0, 1, dims // 2 - 1):
                assert abs(float(table[p, i, 0]) - math.cos(p * f[i]) * amp) < 1e-6
                assert abs(float(table[p, i, 1]) - math.sin(p * f[i]) * amp) < 1e-6
    assert f[0] == 1.0 and abs(f[-1] - 250000.0 ** (-30.0 / 32) / 6.0) < 1e-12       # the fastest pair kept, the slowest slowed down


def test_the_plain_statement_by_hand():
    assert plain.bigram_rows([5, 2, 9], 7, 3, 4) == [7, (5 * 3 + 2 * 4) % 7, (2 * 3 + 9 * 4) % 7]
    # a group is rated by its best member: experts 4, 5 win their group over 2, 3 although 2 + 3 add up to more
    z = torch.log(torch.tensor([0.30, 0.01, 0.14, 0.14, 0.25, 0.01, 0.08, 0.07], dtype=torch.float64))
    picked, weights = plain.route(z, 4, 2, 3)
    assert picked == [0, 4, 1] and abs(float(sum(weights)) - 0.56) < 1e-9
    # the sink takes its share and nothing else changes
    s = torch.tensor([0.0, math.log(3.0)], dtype=torch.float64)
    w = plain.softmax_with_sink(s, torch.tensor(math.log(4.0), dtype=torch.float64))
    assert torch.allclose(w, torch.tensor([1 / 8, 3 / 8], dtype=torch.float64))
    # the two pairings turn the same planes when the dims are permuted
    v = torch.arange(1.0, 7.0, dtype=torch.float64)
    a = plain.rotate(v, 5, 4, 10.0, None, "half")
    b = plain.rotate(v[[0, 2, 1, 3, 4, 5]], 5, 4, 10.0, None, "interleaved")[[0, 2, 1, 3, 4, 5]]
    assert torch.allclose(a, b) and torch.equal(a[4:], v[4:])
    g = plain.clamped_glu_ff(torch.eye(2, dtype=torch.float64), torch.tensor([[5.0, -1.0]], dtype=torch.float64),
                             torch.tensor([[-9.0, 0.5]], dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64), 2.0)
    assert abs(float(g[0, 0]) - 2.0 / (1 + math.exp(-3.404)) * (-2.0 + 1.0)) < 1e-12
    assert abs(float(g[1, 0]) - (-1.0) / (1 + math.exp(1.702)) * 1.5) < 1e-12
