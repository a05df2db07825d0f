"""The Belasun decoder stated plainly: whole sequences, float64, one function per mechanism.

Written from the equations alone; shares nothing with the library. No cache and no state: every
function sees the whole sequence, so whatever the library does with pages, slots, portions and
batches has to come out as these numbers.

A layer: x += attention(rms(x) w1); x += experts(rms(x) w2) where the layer has a feed-forward; then the
per-layer token input x += rms(P (gelu(G x) * e_token)) ws where the model has one. Output:
cap * tanh((rms(x) wf) E^T / cap).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F64)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros in front of the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros((T, C), dtype=F64)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j].to(F64) * u[s].to(F64)
    return y


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with `scaling` (factor, low, high, original) long wavelengths are slowed down."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f:
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out.append(fi)
        elif wavelength > original / low:
            out.append(fi / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return out


def rotate(x, positions, freqs, dims):
    """x [T, heads, width]: dimension i < dims/2 turns with dimension i + dims/2 by positions * freqs[i]."""
    x = x.to(F64).clone()
    half = dims // 2
    ang = torch.tensor(positions, dtype=F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half].clone(), x[..., half:dims].clone()
    x[..., :half] = a * c - b * s
    x[..., half:dims] = b * c + a * s
    return x


def chunk_visible(T, size):
    """[T, T] of booleans: position i sees position j when j is not later and lies in the same chunk
    (chunks counted from position 0; size None: every earlier position)."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    vis = j <= i
    if size is not None:
        vis = vis & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return vis


def attention_heads(q, k, v, scale, chunk):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; softmax over the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    vis = chunk_visible(T, chunk)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = torch.where(vis, s, torch.full_like(s, -math.inf))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g].to(F64)
    return out


def attention_mixer(h, W, m, eps, prefix):
    """The whole mixer on its input h [T, width]; `m` the layer's mixer sizes, `W` name -> tensor."""
    T = h.shape[0]
    h = h.to(F64)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = lambda n: W[prefix + n].to(F64)
    q, k, v = h @ t("q").T, h @ t("k").T, h @ t("v").T
    if m.get("conv", 1) > 1 or (prefix + "q.conv") in W:
        q, k, v = short_conv(q, t("q.conv")), short_conv(k, t("k.conv")), short_conv(v, t("v.conv"))
    q = rms_norm(q, t("q.norm"), eps).view(T, H, d)
    k = rms_norm(k, t("k.norm"), eps).view(T, G, d)
    rot = m.get("rot")
    if rot is not None and rot["dims"] >= 2:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, list(range(T)), f, rot["dims"]), rotate(k, list(range(T)), f, rot["dims"])
    mask = m.get("mask")
    o = attention_heads(q, k, v.view(T, G, dv), m["scale"], mask["size"] if mask else None)
    gate = torch.sigmoid(h @ t("g").T)                      # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ t("o").T


def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.to(F64).T, max=limit)
    u = torch.clamp(h @ up.to(F64).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.to(F64).T


def route(z, top):
    """z [T, E] -> (indices [T, top], weights [T, top]): the largest logits, softmax over those alone."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routed_experts(h, W, f, prefix):
    h = h.to(F64)
    E, top = f["router"]["experts"], f["router"]["top"]
    limit = float(f["expert"]["limit"])
    z = h @ W[prefix + "router"].to(F64).T + W[prefix + "router.b"].to(F64)
    idx, wgt = route(z, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            p = f"{prefix}e{e}."
            out[t] += wgt[t, c] * expert(h[t:t + 1], W[p + "gate"], W[p + "up"], W[p + "down"], limit)[0]
    return out


def token_side(x, tokens, W, layer, dim, eps):
    """The per-layer token input: what it adds to the stream x [T, width]."""
    x = x.to(F64)
    e = W["side.embed"].to(F64)[torch.tensor(tokens)][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ W[f"l{layer}.side.gate"].to(F64).T) * e
    y = g @ W[f"l{layer}.side.proj"].to(F64).T
    return rms_norm(y, W[f"l{layer}.side.norm"], eps)


def softcap(logits, cap):
    return cap * torch.tanh(logits / cap) if cap else logits


def model_forward(cfg: dict, W: dict, tokens: list[int], layers_out: list | None = None):
    """Logits [T, vocab] of every position of one sequence; `layers_out` collects the stream after each layer."""
    eps = float(cfg["norm"]["eps"])
    side = cfg.get("token_side")
    x = W["embed"].to(F64)[torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + attention_mixer(rms_norm(x, W[p + "norm1"], eps), W, layer["mixer"], eps, p + "mix.")
        if layer.get("mlp") is not None:
            x = x + routed_experts(rms_norm(x, W[p + "norm2"], eps), W, layer["mlp"], p + "mlp.")
        if side is not None:
            x = x + token_side(x, tokens, W, i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].to(F64).T
    return softcap(logits, cfg.get("logit_softcap"))
