"""What of the Belasun decoder needs no GPU: its configuration, its layout and tensor names, which pages a
chunked cache gives back, the rescaled rotation table, and the plain statement against second statements of
the same formulas."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_belasun as plain
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.cache.needs import PAGE, CacheNeed
from scriptling_llm_lib_b200.config.base import ConfigError
from scriptling_llm_lib_b200.config.registry import architecture_for, architecture_name
from scriptling_llm_lib_b200.engine.model import DecoderModel

SCALING = {"factor": 8.0, "high": 4.0, "low": 1.0, "original": 256}
RAW = {
    "architecture": "Belasun", "norm": {"eps": 1e-6}, "vocab": 70, "width": 40, "logit_softcap": 12.5, "token_side": {"dim": 6},
    "layers": [
        {"type": "attention",
         "mixer": {"conv": 3, "dim": 16, "heads": 4, "kv_heads": 2, "mask": {"size": 20}, "scale": 0.3, "vdim": 12,
                   "rot": {"base": 500.0, "dims": 8, "scaling": SCALING}},
         "mlp": {"expert": {"ff": 24, "limit": 2.5}, "kind": "moe", "router": {"experts": 5, "top": 2}}},
        {"type": "attention", "mlp": None,
         "mixer": {"conv": 1, "dim": 8, "heads": 3, "kv_heads": 3, "scale": 0.5, "vdim": 8, "rot": {"base": 100.0, "dims": 8}}},
    ],
}


def test_the_configuration_reads_back_and_names_the_model():
    arch = architecture_for(architecture_name(RAW))
    cfg = arch.config_class.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_softcap, cfg.side_dim) == (70, 40, 1e-6, 12.5, 6)
    a, b = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.conv, a.chunk) == (4, 2, 16, 12, 0.3, 3, 20)
    assert (a.rot.dims, a.rot.base, a.rot.scaling.factor, a.rot.scaling.original_max_position_embeddings) == (8, 500.0, 8.0, 256)
    assert (b.conv, b.chunk, b.rot.scaling) == (1, None, None)
    e = cfg.layers[0].mlp
    assert (e.ff, e.limit, e.experts, e.top) == (24, 2.5, 5, 2) and cfg.layers[1].mlp is None
    assert arch.config_class.from_dict(cfg.to_json_dict()) == cfg
    assert cfg.to_json_dict() == RAW
    bare = {k: v for k, v in RAW.items() if k not in ("logit_softcap", "token_side")}
    cfg2 = arch.config_class.from_dict(bare)
    assert cfg2.logit_softcap is None and cfg2.side_dim is None and cfg2.to_json_dict() == bare


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "scan", "type"), (("layers", 0, "mixer", "kv_heads"), 3, "heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "dims"), (("layers", 0, "mixer", "rot", "dims"), 18, "dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"), (("layers", 0, "mlp", "router", "top"), 6, "experts"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("layers", 0, "mlp", "expert", "limit"), -1.0, "limit"),
    (("layers",), [], "layers"), (("norm",), 3, "norm"), (("token_side",), {"dim": 0}, "dim"), (("logit_softcap",), -2.0, "logit_softcap"),
    (("layers", 0, "mixer", "conv"), 0, "conv"),
])
def test_a_wrong_configuration_names_its_key(path, value, word):
    raw = copy.deepcopy(RAW)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        architecture_for("Belasun").config_class.from_dict(raw)
    assert word in str(e.value)


def test_the_layout_asks_for_every_tensor_once():
    arch = architecture_for("Belasun")
    model = DecoderModel(arch.layout(arch.config_class.from_dict(RAW)))
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    want = {"embed": (70, 40), "side.embed": (70, 12), "final.norm": (40,),
            "l0.norm1": (40,), "l0.norm2": (40,), "l0.mix.q": (64, 40), "l0.mix.k": (32, 40), "l0.mix.v": (24, 40), "l0.mix.g": (4, 40),
            "l0.mix.o": (40, 48), "l0.mix.q.conv": (64, 3), "l0.mix.k.conv": (32, 3), "l0.mix.v.conv": (24, 3), "l0.mix.q.norm": (64,),
            "l0.mix.k.norm": (32,), "l0.mlp.router": (5, 40), "l0.mlp.router.b": (5,), "l0.side.gate": (6, 40), "l0.side.proj": (40, 6),
            "l0.side.norm": (40,), "l1.norm1": (40,), "l1.mix.q": (24, 40), "l1.mix.k": (24, 40), "l1.mix.v": (24, 40),
            "l1.mix.g": (3, 40), "l1.mix.o": (40, 24), "l1.mix.q.norm": (24,), "l1.mix.k.norm": (24,), "l1.side.gate": (6, 40),
            "l1.side.proj": (40, 6), "l1.side.norm": (40,)}
    for j in range(5):
        want.update({f"l0.mlp.e{j}.gate": (24, 40), f"l0.mlp.e{j}.up": (24, 40), f"l0.mlp.e{j}.down": (40, 24)})
    assert shapes == want
    needs = model.cache_needs()
    assert (needs[0].kind, needs[0].window, needs[0].kv_heads, needs[0].head_dim, needs[0].value_dim) == ("chunk", 20, 2, 16, 12)
    assert (needs[1].kind, needs[1].window, needs[1].value_dim) == ("full", None, 8)
    states = model.state_needs()
    assert tuple(states[0]["conv"].shape) == (2, 64 + 32 + 24) and states[1] is None     # one tap: nothing to remember
    assert model.graph_safe()


def test_a_chunked_cache_gives_back_the_pages_of_chunks_that_have_passed():
    from scriptling_llm_lib_b200.cache.store import SequenceCache
    for size in (PAGE, 2 * PAGE, PAGE + 7, 5):
        need = CacheNeed("chunk", 1, 4, size)
        for length in (0, 1, size - 1, size, size + 1, 3 * size - 1, 3 * size, 3 * size + 2):
            first = need.first_needed(length)
            assert first == (length // size) * size                      # the start of the chunk the next query lies in
        cache = SequenceCache({0: need}, {0: None}, 2, 16, torch.float32, "cpu")
        slot = cache.open()
        held = 0
        for step in (3, PAGE - 3, 1, PAGE, 2 * PAGE + 9, 1, 1, 40):
            cache.reserve([(slot, step)])
            cache.advance([(slot, step)])
            held += step
            first = (held // size) * size
            pages = cache.groups[0].pages[slot]
            for i, pg in enumerate(pages):
                wholly_before = (i + 1) * PAGE - 1 < first
                assert (pg < 0) == wholly_before, (size, held, i)
        cache.close(slot)
        assert cache.groups[0].pool.n_held == 0
    with pytest.raises(ValueError):
        CacheNeed("chunk", 1, 4)


def test_the_rescaled_rotation_table_against_values_worked_by_hand():
    from scriptling_llm_lib_b200.config.llama import RopeScaling
    from scriptling_llm_lib_b200.parts.rotary import RotaryEncoding, inverse_frequencies
    dims, base = 8, 500.0
    f = [1.0, 500.0 ** -0.25, 500.0 ** -0.5, 500.0 ** -0.75]
    # wavelengths 6.28, 29.7, 140.5, 664.4 against the bands 256 / 4 = 64 and 256 / 1 = 256: keep, keep, blend, slow down
    s = (256.0 / (2 * math.pi / f[2]) - 1.0) / 3.0
    want = [f[0], f[1], (1 - s) * f[2] / 8.0 + s * f[2], f[3] / 8.0]
    got = inverse_frequencies(dims, base, RopeScaling("llama3", 8.0, 1.0, 4.0, 256))
    assert np.allclose(got, want, rtol=1e-12)
    assert np.allclose(plain.rotary_frequencies(dims, base, SCALING), want, rtol=1e-12)
    enc = RotaryEncoding(16, dims, base, RopeScaling("llama3", 8.0, 1.0, 4.0, 256), "half")
    enc.prepare(300, "cpu")
    table, rot, interleaved = enc.rotation()
    assert rot == 8 and not interleaved and tuple(table.shape) == (300, 4, 2)
    assert abs(float(table[299, 2, 0]) - math.cos(299 * want[2])) < 1e-6 and abs(float(table[299, 3, 1]) - math.sin(299 * want[3])) < 1e-6


def test_plain_convolution_rotation_and_mask_against_second_statements():
    g = torch.Generator().manual_seed(1)
    u, w = torch.randn(11, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    y = plain.short_conv(u, w)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(y, ref, atol=1e-12)
    assert torch.allclose(y[0], w[:, 3] * u[0])                          # the last column multiplies the row itself
    # a rotation keeps lengths, leaves the tail alone, and q . k depends on the distance only
    x = torch.randn(6, 2, 10, generator=g, dtype=torch.float64)
    f = plain.rotary_frequencies(6, 50.0)
    r = plain.rotate(x, list(range(6)), f, 6)
    assert torch.allclose(r[..., 6:], x[..., 6:]) and torch.allclose(r.norm(dim=-1), x.norm(dim=-1))
    a, b = torch.randn(1, 1, 6, generator=g, dtype=torch.float64), torch.randn(1, 1, 6, generator=g, dtype=torch.float64)
    d1 = (plain.rotate(a, [9], f, 6) * plain.rotate(b, [4], f, 6)).sum()
    d2 = (plain.rotate(a, [25], f, 6) * plain.rotate(b, [20], f, 6)).sum()
    assert abs(float(d1 - d2)) < 1e-12
    vis = plain.chunk_visible(10, 4)
    assert vis[3, 0] and not vis[4, 3] and vis[4, 4] and vis[7, 4] and not vis[8, 7] and not vis[2, 3]
    assert plain.chunk_visible(5, None).sum() == 15


def test_plain_router_and_expert_against_second_statements():
    z = torch.tensor([[0.1, 2.0, -1.0, 1.5, 0.3], [5.0, 5.0, 1.0, 0.0, -3.0]], dtype=torch.float64)
    idx, w = plain.route(z, 2)
    assert idx[0].tolist() == [1, 3] and sorted(idx[1].tolist()) == [0, 1]
    assert abs(float(w[0, 0]) - 1.0 / (1.0 + math.exp(-0.5))) < 1e-12 and torch.allclose(w.sum(-1), torch.ones(2, dtype=torch.float64))
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    gate, up, down = torch.tensor([[3.0, 0.0], [0.0, 1.0]]), torch.tensor([[0.0, 4.0], [0.5, 0.0]]), torch.eye(2)
    y = plain.expert(h, gate, up, down, 2.0)[0]
    # gate sums 3 -> 2 (capped above only) and -2 (kept); up sums -8 -> -2 and 0.5
    want0 = 2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0)
    want1 = -2.0 / (1.0 + math.exp(1.702 * 2.0)) * 1.5
    assert abs(float(y[0]) - want0) < 1e-12 and abs(float(y[1]) - want1) < 1e-12
    assert abs(float(plain.softcap(torch.tensor(100.0, dtype=torch.float64), 5.0)) - 5.0) < 1e-9
