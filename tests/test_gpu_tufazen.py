"""The Tufazen decoder on the GPU against the plain statement in plain_tufazen.py: each mechanism alone, the residual
stream layer by layer, whole prompts against token-by-token decoding and against portions, unequal batches, slots and
pages used again, keys far back and at page borders, the sink, the first tokens, long decoding through several passes,
other sizes, greedy generation through the entry point. Configurations and weights are made here; weights are larger
than a trained model's so that every branch moves the logits."""
import json
import math

import numpy as np
import pytest
import torch

import plain_tufazen as plain

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-4       # of a row's largest logit
TOL_BF16 = 6e-2
RAMP = {"factor": 4.0, "fast": 8.0, "original": 64, "slow": 1.0}


def attention(heads=4, kv_heads=2, dim=8, scale=0.4, softcap=5.0, dims=4, base=300.0, scaling=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": dim}
    if softcap is not None:
        m["softcap"] = softcap
    if dims:
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=10, q_rank=12, scale=0.35, base=200.0):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot_dim >= 2:
        m["rot"] = {"base": base, "dims": rot_dim}
    return {"type": "latent_attention", "mixer": m}


def dense(ff=24, limit=1.2):
    return {"ff": ff, "kind": "dense", "limit": limit}


def moe(ff=10, experts=6, top=2, groups=3, keep=2, shared=14):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if groups is not None:
        out["router"]["groups"] = {"count": groups, "keep": keep}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def with_ff(layer, mlp):
    return dict(layer, mlp=mlp)


def config(layers, width=48, vocab=90, eps=1e-6, side=None, bigram=None, loop=None, logit_scale=None):
    cfg = {"architecture": "Tufazen", "layers": [dict({"mlp": None}, **l) for l in layers], "norm": {"eps": eps}, "vocab": vocab,
           "width": width}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if bigram is not None:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


# Sizes that differ from one another in every number. A: a loop over the two middle layers, three times; groups of experts;
# a layer without a feed-forward, rotation or cap. B: no pair table, no loop, no token input, no scale; the latent layer
# first; as many key/value heads as heads; one group; one expert a token; no shared expert. C: widths that are multiples of
# nothing; the whole model gone through twice; every open expert chosen. D: sizes the tensor-core kernels take (bfloat16).
CFG_A = config([with_ff(attention(scaling=RAMP), dense()), with_ff(latent(), moe()), attention(2, 1, 16, 0.3, None, 0),
                with_ff(latent(2, 4, 8, 8, 6, 5, 0.5, 50.0), dense(16, 0.8))],
               side=5, bigram=(53, 31, 7), loop=(1, 3, 3), logit_scale=0.7)
CFG_B = config([with_ff(latent(5, 12, 6, 10, 20, 16, 0.2, 5000.0), moe(12, 5, 1, None, None, None)),
                with_ff(attention(6, 6, 12, 0.25, 9.0, 12, 1000.0), dense(40, 2.5))], width=96, vocab=130, eps=1e-5)
CFG_C = config([with_ff(attention(3, 1, 6, 0.6, 2.0, 2, 30.0, RAMP), moe(6, 9, 6, 3, 2, 7)), latent(1, 5, 2, 3, 7, 9, 0.6, 10.0),
                with_ff(attention(5, 5, 2, 1.0, 50.0, 2, 7.0), dense(9, 0.5))], width=50, vocab=61, side=3, bigram=(17, 5, 3),
               loop=(0, 3, 2), logit_scale=1.5)
CFG_D = config([with_ff(attention(4, 2, 64, 0.125, 15.0, 32, 10000.0, RAMP), dense(128, 1.5)),
                with_ff(latent(4, 32, 16, 32, 64, 64, 0.15, 10000.0), moe(64, 8, 2, 4, 2, 64)),
                with_ff(attention(2, 1, 128, 0.09, 30.0, 128, 10000.0), moe(32, 4, 3, 1, 1, 32))], width=128, vocab=200, side=16,
               bigram=(251, 131, 11), loop=(0, 2, 2), logit_scale=0.6)


def random_weights(cfg, seed, std=0.25):
    """Weights by tensor name for `cfg`, bfloat16-representable (the folder stores bfloat16)."""
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    arch = architecture_for("Tufazen")
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(cfg, "test"))).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    W = {}
    for s in specs:
        t = torch.randn(s.shape, generator=g)
        if s.init == "norm_weight":
            t = 1.0 + 0.2 * t
        elif s.init == "matrix":
            t = t * std * (4.0 / math.sqrt(s.shape[-1]))
        elif s.init == "slope":
            t = 0.6 + 0.1 * t
        else:
            t = 0.5 * t
        W[s.name] = t.to(torch.bfloat16)
    for name in ("embed", "side.embed", "bigram"):
        if name in W:
            W[name] = (torch.randn(W[name].shape, generator=g) * (0.5 if name == "bigram" else 1.0)).to(torch.bfloat16)
    return W


def write_folder(path, cfg, W):
    from scriptling_llm_lib_b200.weights.safetensors_io import write_safetensors
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", W)
    return path


def ids(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def engine(folder, dtype="float32", max_tokens=2048, max_seqs=8, **kw):
    from scriptling_llm_lib_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, max_seqs=max_seqs, **kw)


def run(eng, pieces):
    """Feed one sequence in the given pieces; logits of every position [T, vocab]."""
    from scriptling_llm_lib_b200.engine.step import StepEntry
    seq = eng.open()
    out = []
    for p in pieces:
        out.append(eng.step([StepEntry(seq, list(p), list(range(len(p))))]))
    eng.check_errors()
    seq.close()
    return torch.cat(out).cpu().double()


def cut(tokens, sizes):
    out, at = [], 0
    for s in sizes:
        out.append(tokens[at:at + s])
        at += s
    if at < len(tokens):
        out.append(tokens[at:])
    return [p for p in out if p]


def rel(got, want):
    return float(((got - want).abs().amax(-1) / want.abs().amax(-1).clamp_min(1e-30)).max())


def mostly(got, want, tol, part=0.04):
    """bfloat16 against the 32-bit statement: a router's close call may go the other way in a row or two and
    carry that row's logits off, so all but a small part of the rows must be within `tol`."""
    err = (got - want).abs().amax(-1) / want.abs().amax(-1).clamp_min(1e-30)
    return float((err > tol).double().mean()) <= part and float(err.median()) < tol / 2


def plain_logits(cfg, W, tokens, layers_out=None):
    logits, streams = plain.plain_model(cfg, W, tokens)
    if layers_out is not None:
        layers_out.extend(streams)
    return logits


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("tufazen")
    out = {}
    for name, cfg, seed in (("A", CFG_A, 1), ("B", CFG_B, 2), ("C", CFG_C, 3), ("D", CFG_D, 4)):
        W = random_weights(cfg, seed)
        out[name] = (write_folder(root / name, cfg, W), cfg, W)
    return out


# --------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_a_whole_prompt_equals_the_plain_statement_in_32_bit(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(150, cfg["vocab"], 10)
    want = plain_logits(cfg, W, tokens)
    got = run(engine(folder), [tokens])
    assert rel(got, want) < TOL_F32


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_bfloat16_stays_near_the_plain_statement(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(230, cfg["vocab"], 11)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder, "bfloat16")
    got = run(eng, [tokens])
    assert mostly(got, want, 2 * TOL_BF16)
    step = run(eng, [tokens[:180]] + [[t] for t in tokens[180:]])
    assert mostly(step, want, 2 * TOL_BF16)
    assert mostly(run(eng, cut(tokens, [64, 3, 70, 2])), want, 2 * TOL_BF16)


def test_the_residual_stream_after_every_layer_run(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    from scriptling_llm_lib_b200.parts.norm import take_into_stream
    for name in ("A", "C"):
        folder, cfg, W = folders[name]
        tokens = ids(57, cfg["vocab"], 12)
        want = []
        plain_logits(cfg, W, tokens, layers_out=want)
        eng = engine(folder)
        assert len(eng.layout.schedule) == len(want)
        seq = eng.open()
        arr = np.asarray(tokens, dtype=np.int64)
        eng.cache.reserve([(seq.slot, len(tokens))])
        ctx = eng._context([StepEntry(seq, tokens, [])], arr, [len(tokens)], [0], [])
        x = eng.model.embedding.forward(ctx.token_ids, ctx)
        delta = None
        for i, e in enumerate(eng.layout.schedule):
            for j in e.before:
                delta = eng.model.stream_parts[j].forward(x, delta, ctx)
            delta = eng.model.blocks[e.layer].forward(x, delta, ctx, e.cache_unit, e.writes_cache)
            full = x.clone()                         # what is pending is taken in by the next norm
            take_into_stream(full, delta, ctx)
            assert float((full.double().cpu() - want[i]).abs().max()) < 1e-4 * float(want[i].abs().max()), f"layer run {i}"
        seq.close()


@pytest.mark.parametrize("layer,extra", [
    (attention(3, 3, 8, 0.5, None, 0), {}), (attention(4, 2, 8, 0.5, None, 8, 100.0), {}),
    (attention(4, 1, 8, 0.5, None, 6, 100.0, RAMP), {}), (attention(4, 2, 8, 0.8, 1.5, 0), {}),
    (latent(2, 6, 0, 6, 8, 8, 0.5), {}), (latent(3, 4, 6, 5, 9, 7, 0.5, 40.0), {}),
    (with_ff(attention(1, 1, 4, 1.0, None, 0), dense(20, 0.6)), {}), (with_ff(attention(1, 1, 4, 1.0, None, 0), moe(8, 8, 3, 4, 2, None)), {}),
    (with_ff(attention(1, 1, 4, 1.0, None, 0), moe(8, 4, 2, None, None, 12)), {}),
    (attention(1, 1, 4, 1.0, None, 0), {"side": 7}), (attention(1, 1, 4, 1.0, None, 0), {"bigram": (23, 3, 5)}),
    (attention(1, 1, 4, 1.0, None, 0), {"loop": (0, 1, 3)}), (attention(1, 1, 4, 1.0, None, 0), {"logit_scale": 3.0}),
], ids=["sink-and-gate", "rotation", "ramp", "cap", "latent", "latent-rotation", "dense", "experts-in-groups", "shared-expert",
        "token-input", "pair-table", "passes", "logit-scale"])
def test_each_mechanism_alone(tmp_path, layer, extra):
    cfg = config([layer], width=32, vocab=50, **extra)
    W = random_weights(cfg, 5, std=0.4)
    folder = write_folder(tmp_path / "m", cfg, W)
    tokens = ids(75, 50, 13)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder)
    assert rel(run(eng, [tokens]), want) < TOL_F32
    assert rel(run(eng, [tokens[:20]] + [[t] for t in tokens[20:]]), want) < TOL_F32


# --------------------------------------------------------------------------- cutting, batches, slots
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_token_by_token_and_portions_equal_the_whole_prompt(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(210, cfg["vocab"], 14)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder)
    for sizes in ([1] * 210, [2] * 105, [3, 2, 31, 33, 1, 64, 7, 41], [64, 64, 64], [63, 2, 63, 2], [140] + [1] * 70):
        got = run(eng, cut(tokens, sizes))
        assert rel(got, want) < TOL_F32, sizes


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "float32"), ("D", "bfloat16")])
def test_unequal_requests_in_a_batch_equal_each_alone_and_slots_are_used_again(folders, name, dtype):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders[name]
    V = cfg["vocab"]
    reqs = [ids(n, V, 20 + i) for i, n in enumerate((70, 3, 139, 1, 40, 200))]
    prompt = [60, 2, 100, 1, 33, 190]
    want = [plain_logits(cfg, W, r) for r in reqs]
    eng = engine(folder, dtype, max_seqs=6, max_tokens=1024)
    tol = TOL_F32 if dtype == "float32" else 2 * TOL_BF16
    for round_ in range(3):                     # the same slots and pages again, after other requests held them
        seqs = [eng.open() for _ in reqs]
        out = eng.step([StepEntry(s, r[:p], list(range(p))) for s, r, p in zip(seqs, reqs, prompt)]).cpu().double()
        got, at = [[] for _ in reqs], 0
        for i, p in enumerate(prompt):
            got[i].append(out[at:at + p])
            at += p
        pos = list(prompt)
        live = [i for i in range(len(reqs)) if pos[i] < len(reqs[i])]
        for i in range(len(reqs)):
            if i not in live:
                seqs[i].close()
        while live:
            out = eng.step([StepEntry(seqs[i], [reqs[i][pos[i]]], [0]) for i in live]).cpu().double()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
                if pos[i] == len(reqs[i]):
                    seqs[i].close()
            live = [i for i in live if pos[i] < len(reqs[i])]
        if dtype == "float32":
            for i in range(len(reqs)):
                assert rel(torch.cat(got[i]), want[i]) < tol, (round_, i)
        else:
            assert mostly(torch.cat([torch.cat(g) for g in got]), torch.cat(want), tol)
        reqs, prompt, want = reqs[::-1], prompt[::-1], want[::-1]
    assert eng.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in eng.cache.groups)


def test_the_first_tokens_of_a_sequence(folders):
    for name in ("A", "C"):
        folder, cfg, W = folders[name]
        eng = engine(folder)
        for n in (1, 2, 3, 4, 5, 6):
            tokens = ids(n, cfg["vocab"], 30 + n)
            want = plain_logits(cfg, W, tokens)
            assert rel(run(eng, [tokens]), want) < TOL_F32
            assert rel(run(eng, [[t] for t in tokens]), want) < TOL_F32


def test_the_previous_token_of_a_slot_used_again_is_the_new_sequences_own(folders):
    """The pair table's row depends on the token before: a slot's last token must not leak into the sequence that takes the
    slot next, and a portion's first row must find the token the portion before it ended on."""
    folder, cfg, W = folders["A"]
    eng = engine(folder, max_seqs=1)
    a, b = ids(40, cfg["vocab"], 50), ids(33, cfg["vocab"], 51)
    for tokens in (a, b, a):
        assert rel(run(eng, cut(tokens, [11, 1, 1, 9])), plain_logits(cfg, W, tokens)) < TOL_F32


def test_long_decoding_through_all_passes(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders["C"]
    tokens = ids(300, cfg["vocab"], 15)
    want = plain_logits(cfg, W, tokens)
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype, max_tokens=1024)
        seq = eng.open()
        got = [eng.step([StepEntry(seq, tokens[:5], list(range(5)))])]
        for t in tokens[5:]:
            got.append(eng.step([StepEntry(seq, [t], [0])]))
        got = torch.cat(got).cpu().double()
        assert rel(got, want) < TOL_F32 if dtype == "float32" else mostly(got, want, 2 * TOL_BF16)
        assert all(sum(p >= 0 for p in g.pages[seq.slot]) == 5 for g in eng.cache.groups)     # every pass keeps its own keys
        seq.close()


# --------------------------------------------------------------------------- far keys, page borders, the sink
def loud_attention(tmp_path, dim=8, heads=2, kv_heads=1, softcap=None, dims=0, name="loud"):
    """One attention layer whose queries all look for one token (the last id): that token lights channel 0 of the stream,
    the key projection's first row reads it, and every query has a positive number there (it reads channel 1, a constant
    of the embedding). Whoever sees that token's key takes its output from it; the value is the key itself."""
    cfg = config([attention(heads, kv_heads, dim, 3.0 * math.sqrt(8.0 / dim), softcap, dims, 100.0)], width=32, vocab=40)
    W = random_weights(cfg, 7, std=0.5)
    W["embed"][:, 0] = 0.0
    W["embed"][39, 0] = 8.0
    W["embed"][:, 1] = 2.0
    for n, v in (("l0.norm1", 1.0), ("l0.norm1.b", 0.0)):
        W[n][0], W[n][1] = v, v
    W["l0.norm1.alpha"].fill_(1.0)
    W["l0.mix.k"][0, :] = 0.0
    W["l0.mix.k"][0, 0] = 10.0
    for h in range(heads):
        W["l0.mix.q"][h * dim, :] = 0.0
        W["l0.mix.q"][h * dim, 1] = 6.0
    W["l0.mix.sink"].fill_(0.0)
    return write_folder(tmp_path / f"{name}{dim}_{softcap}_{dims}", cfg, W), cfg, W


@pytest.mark.parametrize("dim,softcap,dims,dtype", [(8, None, 0, "float32"), (8, 12.0, 0, "float32"), (6, None, 0, "float32"),
                                                    (64, 12.0, 0, "bfloat16"), (128, None, 0, "bfloat16")])
def test_one_loud_key_far_back_and_at_page_borders(tmp_path, dim, softcap, dims, dtype):
    folder, cfg, W = loud_attention(tmp_path, dim, softcap=softcap, dims=dims)
    eng = engine(folder, dtype)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    base = ids(200, 39, 16)                          # never the loud token
    other = plain_logits(cfg, W, base)
    for p in (0, 1, 63, 64, 65, 127, 128, 150):
        tokens = list(base)
        tokens[p] = 39
        want = plain_logits(cfg, W, tokens)
        assert rel(want[190:], other[190:]) > 100 * TOL_F32         # the far key shows in the last rows
        assert rel(run(eng, [tokens]), want) < tol
        assert rel(run(eng, [tokens[:170]] + [[t] for t in tokens[170:]]), want) < tol
        assert rel(run(eng, cut(tokens, [63, 2, 64, 41])), want) < tol


def test_a_loud_key_behind_the_latent(tmp_path):
    """The same through the cached latent: the shared key part's first dim reads the loud channel, every head's first rotated
    query dim reads a constant through the query latent (no rotation, so the product of the two is the score)."""
    cfg = config([latent(2, 4, 4, 6, 8, 6, 3.0)], width=32, vocab=40)
    del cfg["layers"][0]["mixer"]["rot"]
    W = random_weights(cfg, 8, std=0.5)
    W["embed"][:, 0] = 0.0
    W["embed"][39, 0] = 8.0
    W["embed"][:, 1] = 2.0
    for n, v in (("l0.norm1", 1.0), ("l0.norm1.b", 0.0)):
        W[n][0], W[n][1] = v, v
    W["l0.norm1.alpha"].fill_(1.0)
    W["l0.mix.dkv"][8, :] = 0.0
    W["l0.mix.dkv"][8, 0] = 10.0
    W["l0.mix.dq"][0, :] = 0.0
    W["l0.mix.dq"][0, 1] = 6.0
    W["l0.mix.dq.norm"][0] = 1.0
    for h in range(2):
        W["l0.mix.uq"][h * 8 + 4, :] = 0.0
        W["l0.mix.uq"][h * 8 + 4, 0] = 4.0
    folder = write_folder(tmp_path / "loudlatent", cfg, W)
    eng = engine(folder)
    base = ids(200, 39, 16)
    other = plain_logits(cfg, W, base)
    for p in (0, 1, 63, 64, 65, 128, 150):
        tokens = list(base)
        tokens[p] = 39
        want = plain_logits(cfg, W, tokens)
        assert rel(want[190:], other[190:]) > 100 * TOL_F32
        assert rel(run(eng, [tokens]), want) < TOL_F32
        assert rel(run(eng, [tokens[:170]] + [[t] for t in tokens[170:]]), want) < TOL_F32
        assert rel(run(eng, cut(tokens, [20, 44, 2, 70])), want) < TOL_F32


def test_the_sink_takes_its_share_once(tmp_path):
    """A large sink on one head empties that head's output whatever the number of keys or the way they are split; a sink
    that is left out, or counted once per split, shows."""
    folder, cfg, W = loud_attention(tmp_path, 8, heads=4, kv_heads=2, name="sink")
    tokens = ids(300, 39, 18)
    quiet = plain_logits(cfg, W, tokens)
    W["l0.mix.sink"][0], W["l0.mix.sink"][1], W["l0.mix.sink"][3] = 6.0, -3.0, 1.5
    folder = write_folder(tmp_path / "sink_on", cfg, W)
    want = plain_logits(cfg, W, tokens)
    assert rel(want, quiet) > 100 * TOL_F32
    for dtype, tol in (("float32", TOL_F32), ("bfloat16", TOL_BF16)):
        eng = engine(folder, dtype)
        assert rel(run(eng, [tokens]), want) < tol
        assert rel(run(eng, [tokens[:250]] + [[t] for t in tokens[250:]]), want) < tol      # the keys of a decode step are split over blocks


# --------------------------------------------------------------------------- kernels by themselves
def test_the_router_rates_groups_by_their_best_and_weighs_by_the_scores_as_they_are():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).mix
    g = torch.Generator().manual_seed(3)
    for E, groups, keep, top in ((8, 4, 2, 3), (12, 4, 3, 4), (6, 1, 1, 6), (9, 3, 1, 1), (64, 8, 3, 6), (5, 5, 2, 2), (10, 2, 2, 7)):
        z = torch.randn(50, E, generator=g) * 2.0
        idx = torch.empty((50, top), dtype=torch.int32, device="cuda")
        wgt = torch.empty((50, top), dtype=torch.float32, device="cuda")
        k.moe_route(z.cuda().contiguous(), None, idx, wgt, groups, keep, top, 1.0, router="grouped_softmax")
        for t in range(50):
            picked, weights = plain.route(z[t].double(), groups, keep, top)
            got = dict(zip(idx[t].tolist(), wgt[t].tolist()))
            assert set(got) == set(picked), (E, t)
            assert all(abs(got[e] - float(w)) < 1e-6 for e, w in zip(picked, weights))


def test_the_small_kernels_against_their_formulas():
    from types import SimpleNamespace
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(6)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        ks = KernelSet(dtype)
        # the gate without a clamp, stacked and in tiles
        gu = (torch.randn(9, 2 * 16, generator=g) * 2.0).to(dtype)
        want = torch.nn.functional.silu(gu[:, :16].double()) * gu[:, 16:].double()
        out = torch.zeros((9, 16), dtype=dtype, device="cuda")
        ks.mix.glu_clamp(gu.cuda(), out, 0.0, 1.0)
        assert float((out.cpu().double() - want).abs().max()) < tol * 4
        tiled = torch.stack([gu[:, :16].view(9, 2, 8), gu[:, 16:].view(9, 2, 8)], dim=2).reshape(9, 32)
        ks.mix.glu_clamp(tiled.contiguous().cuda(), out, 0.0, 1.0, tiled=True)
        assert float((out.cpu().double() - want).abs().max()) < tol * 4
        # a gate per element
        o = torch.randn(7, 15, generator=g).to(dtype)
        lg = torch.randn(7, 15, generator=g).to(dtype)
        od = o.clone().cuda()
        ks.gate.head_gate(od, lg.cuda(), 15, 1)
        assert float((od.cpu().double() - o.double() * torch.sigmoid(lg.double())).abs().max()) < tol
        o, wide = torch.randn(7, 32, generator=g).to(dtype), torch.randn(7, 48, generator=g).to(dtype).cuda()     # eight columns a thread
        od = o.clone().cuda()
        ks.gate.head_gate(od, wide[:, 16:], 32, 1)
        assert float((od.cpu().double() - o.double() * torch.sigmoid(wide[:, 16:].cpu().double())).abs().max()) < tol
        # several addends and a row vector in one pass; the rounded copy
        for T, d in ((5, 72), (6, 50)):
            x = torch.randn(T, d, generator=g)
            a1, a2 = torch.randn(3, T, d, generator=g), torch.randn(T, d, generator=g).to(dtype)
            vec = torch.randn(d, generator=g)
            xd, xb = x.clone().cuda(), torch.empty((T, d), dtype=dtype, device="cuda")
            ks.gate.add_list_cast(xd, [a1.cuda(), a2.cuda()], xb, vec.cuda())
            want = x.double() + a1.double().sum(0) + a2.double() + vec.double()
            assert float((xd.cpu().double() - want).abs().max()) < 1e-5
            assert float((xb.cpu().double() - want).abs().max()) < tol * 4
            # x += y / rms(y) w + vec, then the norm without statistics, on all rows and on picked rows
            y, w = torch.randn(2, T, d, generator=g), torch.randn(d, generator=g)
            w2, b2 = torch.randn(d, generator=g), torch.randn(d, generator=g)
            after = x.double() + plain.rms_div(y.double().sum(0), 1e-3) * w.double() + vec.double()
            normed = plain.dyn_tanh(after, w2.double(), b2.double(), 0.7)
            xd, out = x.clone().cuda(), torch.empty((T, d), dtype=dtype, device="cuda")
            ks.gate.add_rms_normed(xd, y.cuda(), w.cuda(), 1e-3, vec=vec.cuda(), dyt=(w2.cuda(), b2.cuda(), 0.7, out))
            assert float((xd.cpu().double() - after).abs().max()) < 1e-5
            assert float((out.cpu().double() - normed).abs().max()) < tol * 4
            pick = torch.tensor([4, 1], dtype=torch.int32)
            xd, out = x.clone().cuda(), torch.empty((2, d), dtype=dtype, device="cuda")
            ks.gate.add_rms_normed(xd, y.cuda(), w.cuda(), 1e-3, rows=pick.cuda(), dyt=(w2.cuda(), b2.cuda(), 0.7, out))
            no_vec = plain.dyn_tanh(after - vec.double(), w2.double(), b2.double(), 0.7)
            assert float((out.cpu().double() - no_vec[pick.long()]).abs().max()) < tol * 4
        # scale and cap of the logits
        lgt = (torch.randn(5, 33, generator=g) * 20.0).cuda()
        want = lgt.cpu().double() * 0.3
        ks.gate.softcap(lgt, None, 0.3)
        assert float((lgt.cpu().double() - want).abs().max()) < 1e-5
        # the embedding with the pair table: a prompt step of three sequences, two of them with a past
        table, pair = torch.randn(30, 12, generator=g).to(dtype), torch.randn(12, 12, generator=g).to(dtype)
        last = torch.tensor([7, 0, 21, 3, 0], dtype=torch.int32).cuda()
        lens, pos0, slots = [3, 1, 2], [5, 0, 9], [2, 4, 0]
        tok = [4, 29, 8, 11, 0, 17]
        ctx = SimpleNamespace(tok_pos=torch.tensor([5, 6, 7, 0, 9, 10], dtype=torch.int32).cuda(),
                              tok_seq=torch.tensor([0, 0, 0, 1, 2, 2], dtype=torch.int32).cuda(),
                              seq_start=torch.tensor([0, 3, 4, 6], dtype=torch.int32).cuda(),
                              slots=torch.tensor(slots, dtype=torch.int32).cuda())
        out = torch.empty((6, 12), dtype=torch.float32, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ks.embed_pair_rows(torch.tensor(tok, dtype=torch.int32).cuda(), ctx, table.cuda(), pair.cuda(), 11, 13, 5, last, out, err)
        prev = [21, 4, 29, None, 7, 0]
        rows = [11 if p is None else (p * 13 + t * 5) % 11 for p, t in zip(prev, tok)]
        want = table.double()[torch.tensor(tok)] + pair.double()[torch.tensor(rows)]
        assert float((out.cpu().double() - want).abs().max()) < 1e-6 and int(err) == 0
        assert last.tolist() == [17, 0, 8, 3, 11]


def test_attention_kernels_with_a_cap_and_a_sink():
    """Prompt (tiled and scalar kernel) and decode (split and merged) kernels of the generic set against the formula, on pages
    in scattered order, for head widths that take the wide loads and for one that does not."""
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(9)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        ks = KernelSet(dtype)
        for H, G, hd, cap in ((4, 2, 16, 3.0), (3, 1, 6, 1.5), (2, 2, 64, None), (8, 1, 64, 4.0)):
            L = 150
            q = (torch.randn(L, H * hd, generator=g)).to(dtype)
            kk = torch.randn(L, G, hd, generator=g).to(dtype)
            vv = torch.randn(L, G, hd, generator=g).to(dtype)
            sink = torch.randn(H, generator=g) * 2.0
            order = [3, 0, 2]
            kp = torch.zeros(4, G, 64, hd, dtype=dtype)
            vp = torch.zeros(4, G, 64, hd, dtype=dtype)
            for p in range(L):
                kp[order[p // 64], :, p % 64] = kk[p]
                vp[order[p // 64], :, p % 64] = vv[p]
            want = torch.zeros(L, H, hd, dtype=torch.float64)
            for t in range(L):
                for h in range(H):
                    s = (kk[:t + 1, h // (H // G)].double() @ q[t, h * hd:(h + 1) * hd].double()) * 0.3
                    if cap:
                        s = cap * torch.tanh(s / cap)
                    want[t, h] = plain.softmax_with_sink(s, sink[h].double()) @ vv[:t + 1, h // (H // G)].double()
            want = want.view(L, H * hd)
            bt = torch.tensor([order], dtype=torch.int32).cuda()
            kpd, vpd, qd, sd = kp.cuda(), vp.cuda(), q.cuda(), sink.cuda()
            out = torch.zeros(L, H * hd, dtype=dtype, device="cuda")
            ks.attn_paged(qd, out, torch.tensor([0, L], dtype=torch.int32).cuda(), torch.tensor([0], dtype=torch.int32).cuda(), bt, kpd,
                          vpd, 1, L, H, G, hd, 0, 0.3, cap, sd)
            assert float((out.cpu().double() - want).abs().max()) < tol * 5
            # the last three rows as a portion on a cache (the scalar kernel), then the last row as a decode step in 1 and 3 splits
            out3 = torch.zeros(3, H * hd, dtype=dtype, device="cuda")
            ks.attn_paged(qd[L - 3:].contiguous(), out3, torch.tensor([0, 3], dtype=torch.int32).cuda(),
                          torch.tensor([L - 3], dtype=torch.int32).cuda(), bt, kpd, vpd, 1, 3, H, G, hd, 0, 0.3, cap, sd)
            assert float((out3.cpu().double() - want[L - 3:]).abs().max()) < tol * 5
            if ks.attn_decode_split_takes(hd, H * hd):
                for n_split in (1, 3):
                    out1 = torch.zeros(1, H * hd, dtype=dtype, device="cuda")
                    part = torch.empty(H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
                    ks.attn_decode_split(qd[L - 1:].contiguous(), out1, torch.tensor([L - 1], dtype=torch.int32).cuda(), bt, kpd, vpd, part,
                                         1, H, G, hd, 0, 0.3, n_split, cap, sd)
                    assert float((out1.cpu().double() - want[L - 1:]).abs().max()) < tol * 5, (H, hd, n_split)


@pytest.mark.parametrize("H,G,hd,cap", [(4, 2, 64, 3.0), (8, 1, 64, 4.0), (4, 2, 128, None), (6, 3, 128, 5.0), (3, 3, 128, 2.0), (2, 2, 64, 6.0)])
def test_the_tensor_core_attention_kernels_with_a_cap_and_a_sink(H, G, hd, cap):
    """The tcgen05 prompt kernels (a head width each; pairs of heads and pairs of query tiles) and the decode kernel that puts
    a group's heads on the tensor cores, against the formula on bfloat16-rounded inputs, on pages in scattered order."""
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(11)
    ks = KernelSet(torch.bfloat16)
    L, scale = 800, 2.0 / math.sqrt(hd)
    q = torch.randn(L, H * hd, generator=g).to(torch.bfloat16)
    kk = torch.randn(L, G, hd, generator=g).to(torch.bfloat16)
    vv = torch.randn(L, G, hd, generator=g).to(torch.bfloat16)
    sink = torch.randn(H, generator=g) * 2.0
    order = [5, 0, 3, 1, 6, 2, 12, 9, 7, 13, 4, 8, 10]
    kp = torch.zeros(14, G, 64, hd, dtype=torch.bfloat16)
    vp = torch.zeros(14, G, 64, hd, dtype=torch.bfloat16)
    for p in range(L):
        kp[order[p // 64], :, p % 64] = kk[p]
        vp[order[p // 64], :, p % 64] = vv[p]
    rows = [0, 1, 63, 64, 127, 128, 129, 200, 255, 256, 300, 511, 640, L - 2, L - 1]
    want = torch.zeros(len(rows), H, hd, dtype=torch.float64)
    for i, t in enumerate(rows):
        for h in range(H):
            s = (kk[:t + 1, h // (H // G)].double() @ q[t, h * hd:(h + 1) * hd].double()) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            want[i, h] = plain.softmax_with_sink(s, sink[h].double()) @ vv[:t + 1, h // (H // G)].double()
    want = want.view(len(rows), H * hd)
    bt = torch.tensor([order], dtype=torch.int32).cuda()
    kpd, vpd, qd, sd = kp.cuda(), vp.cuda(), q.cuda(), sink.cuda()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(L, H * hd, dtype=torch.bfloat16, device="cuda")
    ks.prefill_attention_tc.attn(qd, out, torch.tensor([0, L], dtype=torch.int32).cuda(), torch.tensor([0], dtype=torch.int32).cuda(), bt,
                                 kpd, vpd, 1, L, H, G, hd, 0, scale, err, cap, sd)
    assert int(err) == 0
    assert float((out.cpu().double()[rows] - want).abs().max()) < 2e-2
    # a portion of 160 rows that lands on a cache of 640
    out2 = torch.zeros(160, H * hd, dtype=torch.bfloat16, device="cuda")
    ks.prefill_attention_tc.attn(qd[640:].contiguous(), out2, torch.tensor([0, 160], dtype=torch.int32).cuda(),
                                 torch.tensor([640], dtype=torch.int32).cuda(), bt, kpd, vpd, 1, 160, H, G, hd, 0, scale, err, cap, sd)
    assert float((out2.cpu().double()[[0, 158, 159]] - want[[12, 13, 14]]).abs().max()) < 2e-2
    dec = ks.decode
    if dec.uses_tensor_cores(1, H, G, hd):
        for n_split in (1, 3, 6, 12):                 # more than eight splits are merged a warp a head
            out1 = torch.zeros(1, H * hd, dtype=torch.bfloat16, device="cuda")
            scratch = torch.empty(H * n_split * (hd + 2), dtype=torch.float32, device="cuda")
            tickets = torch.zeros(64, dtype=torch.int32, device="cuda")
            dec.attn_decode_capped(qd[L - 1:].contiguous(), out1, torch.tensor([L - 1], dtype=torch.int32).cuda(), bt, kpd, vpd, scratch,
                                   tickets, 1, H, G, hd, 0, scale, n_split, cap, sd)
            assert float((out1.cpu().double() - want[-1:]).abs().max()) < 2e-2, n_split
            assert int(tickets.abs().sum()) == 0


@pytest.mark.parametrize("H,G,kd,vd,width,cap,sinks", [(4, 2, 96, 64, 96, None, False), (3, 3, 192, 128, 192, None, False),
                                                         (2, 1, 64, 64, 64, 4.0, True), (2, 2, 256, 128, 256, 8.0, True),
                                                         (5, 5, 128, 64, 136, None, True)])
def test_the_prompt_attention_kernel_for_keys_and_values_of_different_widths(H, G, kd, vd, width, cap, sinks):
    """The mma.sync prompt kernel against the formula: rows in storage `width` wide of which the keys use kd and the values
    vd, pages in scattered order, a whole prompt and a portion that lands on a cache."""
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(12)
    ks = KernelSet(torch.bfloat16)
    L, scale = 420, 2.0 / math.sqrt(kd)
    q = torch.zeros(L, H, width)
    q[:, :, :kd] = torch.randn(L, H, kd, generator=g)
    kk, vv = torch.zeros(L, G, width), torch.zeros(L, G, width)
    kk[:, :, :kd] = torch.randn(L, G, kd, generator=g)
    vv[:, :, :vd] = torch.randn(L, G, vd, generator=g)
    vv[:, :, vd:] = 7.0                                     # columns past the values used are not read
    q, kk, vv = q.to(torch.bfloat16), kk.to(torch.bfloat16), vv.to(torch.bfloat16)
    sink = torch.randn(H, generator=g) * 2.0 if sinks else None
    order = [5, 0, 3, 1, 6, 2, 4]
    kp = torch.full((8, G, 64, width), float("nan"), dtype=torch.bfloat16)      # what a page held before must not show
    vp = torch.full((8, G, 64, width), float("nan"), dtype=torch.bfloat16)
    for p in range(L):
        kp[order[p // 64], :, p % 64] = kk[p]
        vp[order[p // 64], :, p % 64] = vv[p]
    rows = [0, 1, 15, 16, 63, 64, 65, 127, 128, 200, 300, 383, 384, L - 1]
    want = torch.zeros(len(rows), H, vd, dtype=torch.float64)
    for i, t in enumerate(rows):
        for h in range(H):
            s = (kk[:t + 1, h // (H // G)].double() @ q[t, h].double()) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            want[i, h] = plain.softmax_with_sink(s, sink[h].double() if sinks else None) @ vv[:t + 1, h // (H // G), :vd].double()
    bt = torch.tensor([order], dtype=torch.int32).cuda()
    kpd, vpd, qd = kp.cuda(), vp.cuda(), q.view(L, H * width).cuda()
    sd = sink.cuda() if sinks else None
    out = torch.full((L, H * width), float("nan"), dtype=torch.bfloat16, device="cuda")
    ks.prefill_attention_mma.attn(qd, width, out, width, torch.tensor([0, L], dtype=torch.int32).cuda(),
                                  torch.tensor([0], dtype=torch.int32).cuda(), bt, kpd, vpd, 1, L, H, G, kd, vd, 0, scale, cap, sd)
    got = out.cpu().double().view(L, H, width)
    assert float((got[rows][:, :, :vd] - want).abs().max()) < 2e-2
    assert float(got[:, :, vd:].abs().max()) == 0.0 if width > vd else True
    out2 = torch.zeros(100, H * width, dtype=torch.bfloat16, device="cuda")
    ks.prefill_attention_mma.attn(qd[320:].contiguous(), width, out2, width, torch.tensor([0, 100], dtype=torch.int32).cuda(),
                                  torch.tensor([320], dtype=torch.int32).cuda(), bt, kpd, vpd, 1, 100, H, G, kd, vd, 0, scale, cap, sd)
    got2 = out2.cpu().double().view(100, H, width)
    assert float((got2[[63, 64, 99]][:, :, :vd] - want[[11, 12, 13]]).abs().max()) < 2e-2


def test_experts_one_by_one_and_grouped_agree(folders):
    """A step of few rows runs every (token, expert) pair by itself, a longer one groups them by expert."""
    for name, dtype, tol in (("A", "float32", TOL_F32), ("D", "bfloat16", TOL_BF16)):
        folder, cfg, W = folders[name]
        tokens = ids(160, cfg["vocab"], 18)
        eng = engine(folder, dtype)
        whole = run(eng, [tokens])                       # grouped (on the tensor cores in bfloat16)
        small = run(eng, cut(tokens, [7] * 23))          # 7 rows a step: one by one
        assert rel(small, whole) < tol if dtype == "float32" else mostly(small, whole, tol)


# --------------------------------------------------------------------------- the entry point
def test_greedy_generation_through_the_entry_point(folders):
    from scriptling_llm_lib_b200 import llm
    folder, cfg, W = folders["A"]
    prompt = ids(41, cfg["vocab"], 19)
    for dtype in ("float32", "bfloat16"):
        out = llm.generate(str(folder), prompt, max_tokens=20, strategy="greedy", dtype=dtype)
        tokens = list(prompt)
        for t in out:
            lg = plain_logits(cfg, W, tokens)[-1]
            top2 = lg.topk(2).values
            if dtype == "float32" or float(top2[0] - top2[1]) > 0.2 * float(lg.abs().max()):
                assert int(lg.argmax()) == t
            tokens.append(t)
        assert len(out) == 20
        llm.unload()


def test_a_batch_of_unequal_prompts_generates_what_each_alone_does(folders):
    from scriptling_llm_lib_b200 import llm
    folder, cfg, W = folders["C"]
    prompts = [ids(n, cfg["vocab"], 60 + n) for n in (3, 70, 1, 18)]
    alone = [llm.generate(str(folder), p, max_tokens=12, strategy="greedy", dtype="float32") for p in prompts]
    together = llm.generate(str(folder), prompts, max_tokens=12, strategy="greedy", dtype="float32")
    assert together == alone
    llm.unload()


def test_random_weights_mode_and_the_command_line(tmp_path):
    import subprocess
    import sys
    from pathlib import Path
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CFG_B))
    eng = engine(f"random:{cfg_path}:3", "bfloat16")
    got = run(eng, [ids(40, CFG_B["vocab"], 1)])
    assert torch.isfinite(got).all() and float(got.abs().max()) > 0
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "scriptling_llm_lib_b200", "-model", f"random:{cfg_path}:3", "-prompt", "1,2,3",
                        "-tokens", "4"], cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_trace_replay_writes_the_logits_of_the_wanted_places(folders, tmp_path):
    import subprocess
    import sys
    from pathlib import Path
    folder, cfg, W = folders["C"]
    V = cfg["vocab"]
    a, b = ids(30, V, 40), ids(9, V, 41)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}, {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[26:27], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[27:], "want": [2]}], "end": ["a"]}]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb = plain_logits(cfg, W, a), plain_logits(cfg, W, b)
    read = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V).copy()).double()
    assert rel(read(0), wa[[0, 24]]) < TOL_F32
    assert rel(read(1), torch.stack([wa[25], wb[8]])) < TOL_F32
    assert not (out / "2.f32").exists()
    assert rel(read(3), wa[29:30]) < TOL_F32
