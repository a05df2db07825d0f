"""The Belasun decoder on the GPU against the plain statement in plain_belasun.py: each mechanism alone, the
residual stream layer by layer, whole prompts against token-by-token decoding and against portions, unequal
batches, slots and pages used again, keys far back, at page borders and on either side of a chunk's edge, the
first tokens, long decoding, other sizes, greedy generation through the entry point. Configurations and weights
are made here; weights are larger than a trained model's so that every branch moves the logits."""
import json
import math

import numpy as np
import pytest
import torch

import plain_belasun as plain

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-4       # of a row's largest logit
TOL_BF16 = 6e-2
BANDS = {"factor": 4.0, "high": 4.0, "low": 1.0, "original": 64}


def attention(heads=4, kv_heads=2, dim=16, vdim=16, conv=4, chunk=48, scale=0.3, dims=8, base=300.0, scaling=None):
    m = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": m}


def moe(ff=24, experts=6, top=2, limit=1.5):
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top}}


def with_ff(layer, mlp):
    return dict(layer, mlp=mlp)


def config(layers, width=64, vocab=96, eps=1e-6, side=None, cap=None):
    cfg = {"architecture": "Belasun", "layers": [dict({"mlp": None}, **l) for l in layers], "norm": {"eps": eps}, "vocab": vocab,
           "width": width}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if cap is not None:
        cfg["logit_softcap"] = cap
    return cfg


# Sizes that differ from one another in every number. A: chunks that are no multiple of a page, values narrower
# than keys, a layer without a feed-forward, every expert chosen. B: ten heads, chunks longer than two pages,
# a head width the fast decode kernels know, a layer without convolution, rotation or token input, no cap.
# C: widths that are multiples of nothing, one expert a token, a layer that sees every earlier key.
# D: sizes the tensor-core kernels take (bfloat16).
CFG_A = config([with_ff(attention(scaling=BANDS), moe()), attention(6, 3, 8, 12, 2, 100, 0.45, 8, 50.0),
                with_ff(attention(2, 1, 32, 32, 3, 64, 0.2, 16, 1000.0, BANDS), moe(16, 4, 4, 0.7))], side=6, cap=10.0)
CFG_B = config([with_ff(attention(10, 5, 12, 12, 5, 130, 0.25, 6, 5000.0), moe(40, 9, 3, 1.0)),
                with_ff(attention(3, 3, 64, 64, 1, 16, 0.12, 0), moe(8, 5, 1, 3.0))], width=96, vocab=130, eps=1e-5)
CFG_C = config([with_ff(attention(3, 1, 5, 3, 2, 7, 0.6, 4, 30.0), moe(6, 3, 1, 0.9)), attention(1, 1, 6, 6, 3, None, 0.4, 2, 10.0),
                with_ff(attention(5, 5, 2, 7, 6, 33, 1.0, 2, 7.0, BANDS), moe(10, 7, 5, 2.0))], width=50, vocab=61, side=5, cap=3.0)
CFG_D = config([with_ff(attention(4, 2, 64, 64, 4, 128, 0.125, 32, 10000.0, BANDS), moe(64, 8, 2, 1.2)),
                with_ff(attention(2, 1, 128, 128, 3, 192, 0.09, 128, 10000.0), moe(32, 4, 3, 1.0))], width=128, vocab=200, side=16,
               cap=20.0)


def random_weights(cfg, seed, std=0.25):
    """Weights by tensor name for `cfg`, bfloat16-representable (the folder stores bfloat16)."""
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    arch = architecture_for("Belasun")
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(cfg, "test"))).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    W = {}
    for s in specs:
        t = torch.randn(s.shape, generator=g)
        if s.init == "norm_weight":
            t = 1.0 + 0.2 * t
        elif s.init == "matrix":
            t = t * std * (4.0 / math.sqrt(s.shape[-1]))
        elif s.init == "bias":
            t = 0.5 * t
        else:
            t = 0.5 * t
        W[s.name] = t.to(torch.bfloat16)
    for name in ("embed", "side.embed"):
        if name in W:
            W[name] = torch.randn(W[name].shape, generator=g).to(torch.bfloat16)
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
    return plain.model_forward(cfg, W, tokens, layers_out)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("belasun")
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


def test_the_residual_stream_after_every_layer(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders["A"]
    tokens = ids(57, cfg["vocab"], 12)
    want = []
    plain_logits(cfg, W, tokens, layers_out=want)
    eng = engine(folder)
    seq = eng.open()
    arr = np.asarray(tokens, dtype=np.int64)
    eng.cache.reserve([(seq.slot, len(tokens))])
    ctx = eng._context([StepEntry(seq, tokens, [])], arr, [len(tokens)], [0], [])
    x = eng.model.embedding.forward(ctx.token_ids, ctx)
    delta = None
    for i, e in enumerate(eng.layout.schedule):
        delta = eng.model.blocks[e.layer].forward(x, delta, ctx, e.cache_unit, e.writes_cache)
        full = x.clone()                         # the token input's addend is pending: the next norm adds it
        assert delta is not None
        delta.apply(full, ctx)
        assert float((full.double().cpu() - want[i]).abs().max()) < 1e-4 * float(want[i].abs().max()), f"layer {i}"
    seq.close()


@pytest.mark.parametrize("layer,side,cap", [
    (attention(conv=1, chunk=None, dims=0), None, None), (attention(conv=5, chunk=None, dims=0), None, None),
    (attention(conv=1, chunk=None, dims=16, scaling=BANDS), None, None), (attention(conv=1, chunk=24, dims=0), None, None),
    (attention(3, 1, 8, 20, 1, None, 0.4, 0), None, None), (with_ff(attention(1, 1, 4, 4, 1, None, 1.0, 0), moe(12, 5, 2, 0.8)), None, None),
    (attention(1, 1, 4, 4, 1, None, 1.0, 0), 7, None), (attention(1, 1, 4, 4, 1, None, 1.0, 0), None, 2.0),
], ids=["norm-and-gate", "convolution", "rotation", "chunks", "wide-values", "experts", "token-input", "cap"])
def test_each_mechanism_alone(tmp_path, layer, side, cap):
    cfg = config([layer], width=32, vocab=50, side=side, cap=cap)
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
    for sizes in ([1] * 210, [2] * 105, [3, 2, 31, 33, 1, 64, 7, 41], [64, 64, 64], [63, 2, 63, 2], [47, 1, 48, 49], [140] + [1] * 70):
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


def test_long_decoding_over_many_chunks_gives_pages_back(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders["C"]                 # chunks of 7 and 33 positions beside a layer that keeps everything
    tokens = ids(400, cfg["vocab"], 15)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder, max_tokens=1024)
    seq = eng.open()
    got = [eng.step([StepEntry(seq, tokens[:5], list(range(5)))])]
    for t in tokens[5:]:
        got.append(eng.step([StepEntry(seq, [t], [0])]))
    assert rel(torch.cat(got).cpu().double(), want) < TOL_F32
    held = {g.need.kind + str(g.need.window): sum(p >= 0 for p in g.pages[seq.slot]) for g in eng.cache.groups}
    assert held["chunk7"] == 1 and held["chunk33"] == 1 and held["fullNone"] == 7
    seq.close()


# --------------------------------------------------------------------------- far keys, page borders, chunk edges
def loud_model(tmp_path, chunk, heads=2, kv_heads=1, dim=8):
    """One layer without convolution whose queries all look for one token of its own (the last id): that token
    lights channel 0 of the stream, the key projection's first row reads it, and every query has a positive
    number there (it reads channel 1, a constant of the embedding). Whoever sees that token's key takes its
    output from it."""
    cfg = config([attention(heads, kv_heads, dim, dim, 1, chunk, 4.0 * math.sqrt(8.0 / dim), 0)], width=32, vocab=40)
    W = random_weights(cfg, 7, std=0.5)
    W["embed"][:, 0] = 0.0
    W["embed"][39, 0] = 8.0
    W["embed"][:, 1] = 2.0
    W["l0.norm1"][0], W["l0.norm1"][1] = 1.0, 1.0
    W["l0.mix.k"][0, :] = 0.0
    W["l0.mix.k"][0, 0] = 10.0
    W["l0.mix.k.norm"][0] = 1.0
    W["l0.mix.q"][0, :] = 0.0
    W["l0.mix.q"][0, 1] = 6.0
    W["l0.mix.q.norm"][0] = 1.0
    return write_folder(tmp_path / f"loud{chunk}_{dim}", cfg, W), cfg, W


def test_one_loud_key_far_back_and_at_page_borders(tmp_path):
    folder, cfg, W = loud_model(tmp_path, None)
    eng = engine(folder)
    base = ids(200, 39, 16)                          # never the loud token
    other = plain_logits(cfg, W, base)
    for p in (0, 1, 63, 64, 65, 127, 128, 150):
        tokens = list(base)
        tokens[p] = 39
        want = plain_logits(cfg, W, tokens)
        assert rel(want[190:], other[190:]) > 100 * TOL_F32         # the far key shows in the last rows
        assert rel(run(eng, [tokens]), want) < TOL_F32
        assert rel(run(eng, [tokens[:170]] + [[t] for t in tokens[170:]]), want) < TOL_F32


@pytest.mark.parametrize("chunk,dim,dtype", [(7, 8, "float32"), (64, 8, "float32"), (100, 8, "float32"), (150, 8, "float32"),
                                             (7, 64, "bfloat16"), (64, 128, "bfloat16"), (100, 64, "bfloat16"), (150, 64, "bfloat16")])
def test_a_loud_key_just_inside_and_just_outside_a_chunk(tmp_path, chunk, dim, dtype):
    """In bfloat16 with heads of 64 and 128 the prompt runs the tensor-core attention kernel and single tokens
    the decode kernels that split a sequence's keys."""
    folder, cfg, W = loud_model(tmp_path, chunk, dim=dim)
    eng = engine(folder, dtype)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    n = 2 * chunk + chunk // 2 + 1
    base = ids(n, 39, 17)
    other = plain_logits(cfg, W, base)
    edge = 2 * chunk                                   # the first position of the third chunk
    for p, seen_by in ((chunk, range(chunk, 2 * chunk)), (edge - 1, range(edge - 1, edge)), (edge, range(edge, n)),
                       (edge + 1, range(edge + 1, n))):
        tokens = list(base)
        tokens[p] = 39
        want = plain_logits(cfg, W, tokens)
        rows = torch.tensor(list(seen_by))
        others = torch.tensor([i for i in range(n) if i not in seen_by])
        assert rel(want[rows[-1:]], other[rows[-1:]]) > 100 * TOL_F32 or len(rows) == 1     # the last row of the chunk hears it
        assert torch.equal(want[others], other[others])                                    # and no row of another chunk does
        for pieces in ([tokens], [tokens[:edge - 2]] + [[t] for t in tokens[edge - 2:]], cut(tokens, [edge - 1, 2, 5]),
                       cut(tokens, [chunk + 3, chunk - 3, 1, 1, 1])):
            got = run(eng, pieces)
            assert rel(got, want) < tol, (p, [len(x) for x in pieces][:4])


# --------------------------------------------------------------------------- kernels by themselves
def test_the_router_picks_the_largest_logits_and_weighs_by_their_softmax():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).mix
    g = torch.Generator().manual_seed(3)
    for E, top in ((8, 2), (12, 4), (6, 6), (9, 1), (64, 6), (5, 5), (3, 2)):
        z = torch.randn(50, E, generator=g) * 3.0
        bias = torch.randn(E, generator=g) * 1.5
        want_idx, want_w = plain.route(z.double() + bias.double(), top)
        idx = torch.empty((50, top), dtype=torch.int32, device="cuda")
        wgt = torch.empty((50, top), dtype=torch.float32, device="cuda")
        k.moe_route(z.cuda().contiguous(), bias.cuda(), idx, wgt, 1, 1, top, 1.0, top_softmax=True)
        for t in range(50):
            got = dict(zip(idx[t].tolist(), wgt[t].tolist()))
            want = dict(zip(want_idx[t].tolist(), want_w[t].tolist()))
            assert set(got) == set(want), (E, t)
            assert all(abs(got[e] - want[e]) < 1e-5 for e in want)


def test_the_small_kernels_against_their_formulas():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(6)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        ks = KernelSet(dtype)
        # the clamped gate
        gu = (torch.randn(9, 2 * 14, generator=g) * 2.0).to(dtype)
        out = torch.zeros((9, 14), dtype=dtype, device="cuda")
        ks.mix.glu_clamp(gu.cuda(), out, 1.3, 1.702)
        gg, uu = gu[:, :14].double().clamp(max=1.3), gu[:, 14:].double().clamp(-1.3, 1.3)
        assert float((out.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)).abs().max()) < tol
        # a gate per head
        o = torch.randn(7, 3 * 5, generator=g).to(dtype)
        lg = torch.randn(7, 3, generator=g).to(dtype)
        od = o.clone().cuda()
        ks.gate.head_gate(od, lg.cuda(), 3, 5)
        want = (o.double().view(7, 3, 5) * torch.sigmoid(lg.double())[:, :, None]).view(7, 15)
        assert float((od.cpu().double() - want).abs().max()) < tol
        # the same over widths that take the four-wide kernels
        for hh, vv in ((4, 8), (2, 12)):     # eight and four columns a thread
            o = torch.randn(9, hh * vv, generator=g).to(dtype)
            lg = torch.randn(9, hh, generator=g).to(dtype)
            od = o.clone().cuda()
            ks.gate.head_gate(od, lg.cuda(), hh, vv)
            want = (o.double().view(9, hh, vv) * torch.sigmoid(lg.double())[:, :, None]).view(9, hh * vv)
            assert float((od.cpu().double() - want).abs().max()) < tol
        x = torch.randn(5, 72, generator=g)
        y = torch.randn(2, 5, 72, generator=g)
        w = torch.randn(72, generator=g)
        xd = x.clone().cuda()
        ks.gate.add_rms_normed(xd, y.cuda(), w.cuda(), 1e-3)
        assert float((xd.cpu().double() - x.double() - plain.rms_norm(y.double().sum(0), w, 1e-3)).abs().max()) < 1e-5
        # the same with the next norm's output in the pass, on all rows and on picked rows, at both widths
        for xx, yy, ww in ((x, y, w), (torch.randn(6, 50, generator=g), torch.randn(3, 6, 50, generator=g), torch.randn(50, generator=g))):
            w2 = (torch.rand(xx.shape[1], generator=g) + 0.5).to(dtype)
            after = xx.double() + plain.rms_norm(yy.double().sum(0), ww, 1e-3)
            normed = plain.rms_norm(after, w2.double(), 1e-2)
            xd = xx.clone().cuda()
            out = torch.empty(xx.shape, dtype=dtype, device="cuda")
            ks.gate.add_rms_normed(xd, yy.cuda(), ww.cuda(), 1e-3, norm=(w2.cuda(), 1e-2, out))
            assert float((xd.cpu().double() - after).abs().max()) < 1e-5
            assert float((out.cpu().double() - normed).abs().max()) < tol * float(normed.abs().max())
            pick = torch.tensor([4, 1], dtype=torch.int32)
            xd = xx.clone().cuda()
            out = torch.empty((2, xx.shape[1]), dtype=dtype, device="cuda")
            ks.gate.add_rms_normed(xd, yy.cuda(), ww.cuda(), 1e-3, norm=(w2.cuda(), 1e-2, out), rows=pick.cuda())
            assert float((out.cpu().double() - normed[pick.long()]).abs().max()) < tol * float(normed.abs().max())
        xd = x.clone().cuda()
        xb = torch.empty((5, 72), dtype=dtype, device="cuda")
        ks.gate.add_cast(xd, y.cuda(), xb)
        assert float((xd.cpu().double() - x.double() - y.double().sum(0)).abs().max()) < 1e-5
        assert float((xb.cpu().double() - xd.cpu().double()).abs().max()) < tol
        # stream += y / rms(y) * w, y as partial sums
        x = torch.randn(7, 50, generator=g)
        y = torch.randn(3, 7, 50, generator=g)
        w = torch.randn(50, generator=g)
        xd = x.clone().cuda()
        ks.gate.add_rms_normed(xd, y.cuda(), w.cuda(), 1e-3)
        assert float((xd.cpu().double() - x.double() - plain.rms_norm(y.double().sum(0), w, 1e-3)).abs().max()) < 1e-5
        # the stream takes its addend and is copied in the element type
        xd = x.clone().cuda()
        xb = torch.empty((7, 50), dtype=dtype, device="cuda")
        ks.gate.add_cast(xd, y.cuda(), xb)
        assert float((xd.cpu().double() - x.double() - y.double().sum(0)).abs().max()) < 1e-5
        assert float((xb.cpu().double() - xd.cpu().double()).abs().max()) < tol
        # gelu(a) * the token's table columns
        a = torch.randn(7, 6, generator=g).to(dtype)
        table = torch.randn(11, 20, generator=g).to(dtype)
        tok = torch.tensor([3, 0, 10, 3, 7, 1, 9], dtype=torch.int32)
        outg = torch.empty((7, 6), dtype=dtype, device="cuda")
        ks.gate.gelu_mul_rows(a.cuda(), tok.cuda(), table.cuda(), 8, outg)
        assert float((outg.cpu().double() - plain.gelu_tanh(a.double()) * table.double()[tok.long()][:, 8:14]).abs().max()) < tol
        # the cap
        lgt = (torch.randn(5, 33, generator=g) * 20.0).cuda()
        want = plain.softcap(lgt.cpu().double(), 7.5)
        ks.gate.softcap(lgt, 7.5)
        assert float((lgt.cpu().double() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("H,G,hd,vd,rot,taps,gate_cols,interleaved", [
    (4, 2, 16, 16, 8, 4, 4, False),      # four channels a thread, two dims a store
    (4, 2, 16, 8, 16, 3, 0, True),       # neighbouring pairs
    (2, 2, 12, 4, 6, 2, 0, False),       # an odd number of pairs a head: one dim a store
    (3, 1, 5, 3, 4, 5, 3, False),        # widths that are multiples of nothing
    (2, 1, 8, 8, 0, 4, 0, False)])       # nothing turns
def test_convolution_norm_and_store_in_one_kernel_equal_the_two_kernels(H, G, hd, vd, rot, taps, gate_cols, interleaved):
    """A prompt step of three sequences that have a past (one of a single row), then a decode step of the three: the
    queries, the cache pages and the convolution's state of the one-kernel path against the convolution and the
    norm-and-store kernel run one behind the other."""
    from types import SimpleNamespace
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    g = torch.Generator().manual_seed(31)
    QW, KW, VW = H * hd, G * hd, G * vd
    C = QW + KW + VW
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        ks = KernelSet(dtype)
        wc = (torch.randn(C, taps, generator=g) * 0.5).to(dtype).cuda()
        qn, kn = (torch.rand(QW, generator=g) + 0.5).cuda(), (torch.rand(KW, generator=g) + 0.5).cuda()
        cs = torch.randn(300, max(rot // 2, 1), 2, generator=g).cuda()
        slots = torch.tensor([2, 0, 3], dtype=torch.int32).cuda()
        table = torch.tensor([[4, 1], [0, 5], [2, 3]], dtype=torch.int32).cuda()
        state0 = torch.randn(5, taps - 1, C, generator=g).cuda()
        outs = []
        for fused in (False, True):
            st = state0.clone()
            kp = torch.zeros(7, G, 64, hd, dtype=dtype, device="cuda")
            vp = torch.zeros(7, G, 64, vd, dtype=dtype, device="cuda")
            got = []
            for lens, pos0 in (([5, 1, 9], [60, 3, 17]), ([1, 1, 1], [65, 4, 26])):
                T = sum(lens)
                start = [0]
                for n in lens:
                    start.append(start[-1] + n)
                ctx = SimpleNamespace(
                    seq_start=torch.tensor(start, dtype=torch.int32).cuda(), n_seqs=3, slots=slots, is_decode=max(lens) == 1,
                    tok_seq=torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32).cuda(),
                    tok_pos=torch.tensor([pos0[b] + i for b, n in enumerate(lens) for i in range(n)], dtype=torch.int32).cuda())
                y = torch.randn(T, C + gate_cols, generator=torch.Generator().manual_seed(T)).to(dtype).cuda()
                q = torch.zeros(T, QW, dtype=dtype, device="cuda")
                if fused:
                    ks.gate.conv_qk_norm_store(y[:, :C], wc, taps, st, ctx, q, table, cs if rot else None, kp, vp, H, G, hd, vd, rot,
                                               interleaved, qn, kn, 1e-4)
                else:
                    c = torch.empty(T, C, device="cuda")
                    ks.seq.causal_conv(y[:, :C], wc, st, ctx, c, taps)
                    ks.gate.qk_norm_store(c, q, ctx.tok_pos, ctx.tok_seq, table, cs if rot else None, kp, vp, H, G, hd, vd, rot,
                                          interleaved, qn, kn, 1e-4)
                got.append(q.float().cpu())
            outs.append(got + [kp.float().cpu(), vp.float().cpu(), st.cpu()])
        for a, b in zip(*outs):
            assert float((a - b).abs().max()) <= tol * max(1.0, float(a.abs().max()))
        assert float(outs[1][2].abs().max()) > 0 and float((outs[1][4] - state0.cpu()).abs().max()) > 0


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
