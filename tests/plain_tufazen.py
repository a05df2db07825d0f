"""A plain statement of the Tufazen decoder in float64: one function per mechanism, whole sequences, explicit
loops, keys and values formed per head and position. It shares no code with the library; the tests compare the
library's numbers with these.

`plain_model(raw, W, tokens)` takes the configuration as the dict that config.json holds, the weights as a
dict name -> float64 tensor, and one sequence's token ids; it returns the logits of every position and the
residual stream after every layer run.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_div(x, eps):
    """x divided by its root mean square (eps inside the root), along the last dim."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyn_tanh(x, w, b, alpha):
    return torch.tanh(alpha * x) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every position: the hash of (previous, current), the last row for a first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embed(tokens, table, pair_table=None, buckets=0, mul_prev=0, mul_cur=0):
    x = table[torch.tensor(tokens)]
    if pair_table is not None:
        x = x + pair_table[torch.tensor(bigram_rows(tokens, buckets, mul_prev, mul_cur))]
    return x


def frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with a scaling, pairs between index(fast) and index(slow) are slowed down along a ramp.
    Returns (frequencies, amplitude of cos and sin)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return f, 1.0
    factor, original, fast, slow = scaling["factor"], scaling["original"], scaling["fast"], scaling["slow"]

    def index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index(fast)), 0)
    hi = min(math.ceil(index(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(v, pos, dims, base, scaling, layout):
    """Turns the first `dims` entries of the vector v (float64 [d]) for position `pos`; `layout` "half" pairs
    entry i with i + dims/2, "interleaved" entry 2i with 2i + 1."""
    f, amp = frequencies(dims, base, scaling)
    out = v.clone()
    for i in range(dims // 2):
        a, b = (i, i + dims // 2) if layout == "half" else (2 * i, 2 * i + 1)
        ang = pos * f[i]
        c, s = math.cos(ang) * amp, math.sin(ang) * amp
        out[a] = v[a] * c - v[b] * s
        out[b] = v[b] * c + v[a] * s
    return out


def softmax_with_sink(scores, sink=None):
    """Weights of the visible keys; a sink adds exp(sink) to the denominator and nothing else."""
    m = scores.max() if sink is None else torch.maximum(scores.max(), sink)
    e = torch.exp(scores - m)
    den = e.sum() if sink is None else e.sum() + torch.exp(sink - m)
    return e / den


def attention_mixer(h, W, p, m):
    """Grouped-query attention whose values are the unrotated keys; capped scores, a sink per head, an elementwise gate."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    q = (h @ W[p + "q"].T).view(T, H, d)
    k = (h @ W[p + "k"].T).view(T, G, d)
    v = k.clone()
    assert vd == d, "the values are the keys"
    if rot is not None and rot.get("dims", 0) >= 2:
        qr, kr = q.clone(), k.clone()
        for t in range(T):
            for i in range(H):
                qr[t, i] = rotate(q[t, i], t, rot["dims"], rot["base"], rot.get("scaling"), "interleaved")
            for g in range(G):
                kr[t, g] = rotate(k[t, g], t, rot["dims"], rot["base"], rot.get("scaling"), "interleaved")
        q, k = qr, kr
    cap = m.get("softcap")
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        for i in range(H):
            g = i // (H // G)
            s = (k[:t + 1, g] @ q[t, i]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            w = softmax_with_sink(s, W[p + "sink"][i] if p + "sink" in W else None)
            out[t, i] = w @ v[:t + 1, g]
    out = out.reshape(T, H * vd) * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def latent_attention_mixer(h, W, p, m, eps):
    """Attention whose keys and values are made from a normed latent, with one rotated key part for all heads,
    queries through a latent of their own, and a gate per head."""
    T = h.shape[0]
    H, d, r, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot")
    cq = rms_div(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, d + r)
    dkv = h @ W[p + "dkv"].T
    c = rms_div(dkv[:, :R], eps) * W[p + "dkv.norm"]
    kr = dkv[:, R:].clone()
    q = q.clone()
    if rot is not None and r >= 2:
        for t in range(T):
            kr[t] = rotate(dkv[t, R:], t, r, rot["base"], rot.get("scaling"), "half")
            for i in range(H):
                q[t, i, d:] = rotate(q[t, i, d:].clone(), t, r, rot["base"], rot.get("scaling"), "half")
    ku = (c @ W[p + "uk"].T).view(T, H, d)
    vu = (c @ W[p + "uv"].T).view(T, H, vd)
    gate = torch.sigmoid(h @ W[p + "g"].T)          # [T, H]
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        for i in range(H):
            s = (ku[:t + 1, i] @ q[t, i, :d] + kr[:t + 1] @ q[t, i, d:]) * m["scale"]
            out[t, i] = softmax_with_sink(s) @ vu[:t + 1, i] * gate[t, i]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def clamped_glu_ff(h, wg, wu, wd, limit):
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def silu_glu_ff(h, wg, wu, wd):
    g = h @ wg.T
    return (g * torch.sigmoid(g) * (h @ wu.T)) @ wd.T


def route(z, n_groups, keep, top):
    """For one token's router logits: softmax over all experts; a group counts as its best member; only the best
    `keep` groups are open; the `top` best open experts are taken, weighted by their scores as they are."""
    s = torch.softmax(z, -1)
    E = s.shape[0]
    size = E // n_groups
    rating = [float(s[g * size:(g + 1) * size].max()) for g in range(n_groups)]
    open_groups = sorted(range(n_groups), key=lambda g: -rating[g])[:keep]
    cand = [e for e in range(E) if e // size in open_groups]
    cand.sort(key=lambda e: -float(s[e]))
    picked = cand[:top]
    return picked, [s[e] for e in picked]


def moe_ff(h, W, p, f):
    r = f["router"]
    E = r["experts"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        picked, weights = route(W[p + "router"] @ h[t], groups["count"], groups["keep"], r["top"])
        for e, w in zip(picked, weights):
            out[t] += w * silu_glu_ff(h[t:t + 1], W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"], W[f"{p}e{e}.down"])[0]
    if f.get("shared") is not None:
        out = out + silu_glu_ff(h, W[p + "shared.gate"], W[p + "shared.up"], W[p + "shared.down"])
    assert E == sum(1 for n in W if n.startswith(p + "e") and n.endswith(".gate"))
    return out


def token_side(x, tokens, W, p, layer, dim, eps):
    e = W["side.embed"][torch.tensor(tokens)][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ W[p + "side.gate"].T) * e
    y = g @ W[p + "side.proj"].T
    return x + rms_div(y, eps) * W[p + "side.norm"]


def run_order(n_layers, loop):
    """(layer, pass number or None when the layer opens no pass) for every layer run."""
    if not loop:
        return [(i, None) for i in range(n_layers)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n_layers)]


def plain_model(raw, W, tokens):
    W = {n: w.to(F64) for n, w in W.items()}
    eps = raw["norm"]["eps"]
    bi = (raw.get("embedding") or {}).get("bigram")
    if bi:
        x = embed(tokens, W["embed"], W["bigram"], bi["buckets"], bi["mul_prev"], bi["mul_cur"])
    else:
        x = embed(tokens, W["embed"])
    side = (raw.get("token_side") or {}).get("dim")
    streams = []
    for i, t in run_order(len(raw["layers"]), raw.get("loop")):
        layer, p = raw["layers"][i], f"l{i}."
        if t is not None:
            x = x + W["loop.step"][t]
        h = dyn_tanh(x, W[p + "norm1"], W[p + "norm1.b"], W[p + "norm1.alpha"])
        if layer["type"] == "attention":
            a = attention_mixer(h, W, p + "mix.", layer["mixer"])
        else:
            a = latent_attention_mixer(h, W, p + "mix.", layer["mixer"], eps)
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                a = a + clamped_glu_ff(h, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"], f["limit"])
            else:
                a = a + moe_ff(h, W, p + "mlp.", f)
        x = x + a
        if side:
            x = token_side(x, tokens, W, p, i, side, eps)
        streams.append(x.clone())
    n = dyn_tanh(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    return (n @ W["head"].T) * raw.get("logit_scale", 1.0), torch.stack(streams)
