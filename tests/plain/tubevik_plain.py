"""A plain, slow implementation of the Tubevik decoder: whole sequences, no cache, one function
per mechanism, PyTorch on the CPU only (float64 by default).

Written from the design's equations in this file's own notation; it shares no code with
``scratch_llm_b200``.  It takes ``config.json`` as a plain dict and the tensors as a dict by
name.

Notation: ``T`` tokens of one sequence at positions ``0 .. T-1``; ``x`` is the residual
stream ``[T, width]``; a layer is ``x <- x + m * (mixer(LN(x)) + ff(LN(x)))`` with ONE layer
norm in front of both branches.
"""

from __future__ import annotations

import math

import torch

#: constants the design fixes
SWISH_SLOPE = 1.702        # the feed-forward's gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6            # inside the root when the recurrence's q and k are made unit vectors
YARN_MAG_COEF = 0.1        # cos and sin are multiplied by 0.1 ln(factor) + 1


# ------------------------------------------------------------------------------ small pieces

def layer_norm(x, weight, bias, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = (x - mu).pow(2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))


# ---------------------------------------------------------------------------------- rotation

def plain_frequencies(base, dims):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(base, dims, scaling):
    """The frequencies blended between themselves and themselves / factor by a ramp over the
    pair index, and the factor that cos and sin are multiplied by."""
    factor, original = scaling["factor"], scaling["original"]

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(scaling["fast"])), 0)
    hi = min(math.ceil(pair_of(scaling["slow"])), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, YARN_MAG_COEF * math.log(factor) + 1.0


def rotate(x, rot, layout):
    """``x`` [T, heads, dim]: the first ``rot['dims']`` entries of every head turn by the
    position's angles.  ``layout`` "pairs": entry 2i with 2i+1; "halves": entry i with
    i + dims/2."""
    dims = rot["dims"]
    if rot.get("scaling"):
        freqs, mag = yarn_frequencies(rot["base"], dims, rot["scaling"])
    else:
        freqs, mag = plain_frequencies(rot["base"], dims), 1.0
    out = x.clone()
    for p in range(x.shape[0]):
        for i, f in enumerate(freqs):
            a, b = (2 * i, 2 * i + 1) if layout == "pairs" else (i, i + dims // 2)
            c, s = math.cos(p * f) * mag, math.sin(p * f) * mag
            u, v = x[p, :, a], x[p, :, b]
            out[p, :, a] = u * c - v * s
            out[p, :, b] = v * c + u * s
    return out


# -------------------------------------------------------------------------- attention proper

def attend(q, k, v, scale, visible, softcap=None, zero_sink=False):
    """``q`` [T, H, D], ``k`` [T, G, D], ``v`` [T, G, V]; ``visible(i, j)`` says whether the
    query at i sees the key at j <= i.  ``zero_sink``: one more term exp(0) in the softmax's
    denominator, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j)]
            s = (k[js, g] @ q[i, head]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            top = max(float(s.max()), 0.0) if zero_sink else float(s.max())
            e = torch.exp(s - top)
            den = e.sum() + (math.exp(-top) if zero_sink else 0.0)
            out[i, head] = (e / den) @ v[js, g]
    return out


def window_visible(size):
    return lambda i, j: 0 <= i - j < size


def chunk_visible(size):
    return lambda i, j: j <= i and i // size == j // size


# ---------------------------------------------------------------- mixer: windowed attention

def attention_keys_values(h, w, m, eps):
    """The keys (normed over the whole projection, then rotated by halves) and values of an
    attention layer, as a later layer that borrows them sees them."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w["k"].T + w["k.b"]
    k = rms_unit(k, eps) * w["k.norm"]
    k = rotate(k.view(T, G, D), m["rot"], "halves")
    v = (h @ w["v"].T + w["v.b"]).view(T, G, V)
    return k, v


def attention_mixer(h, w, m, eps, borrowed=None):
    """``borrowed``: (k, v) of the layer this one takes its keys and values from."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    q = h @ w["q"].T + w["q.b"]
    q = rms_unit(q, eps) * w["q.norm"]
    q = rotate(q.view(T, H, D), m["rot"], "halves")
    k, v = borrowed if borrowed is not None else attention_keys_values(h, w, m, eps)
    o = attend(q, k, v, m["scale"], window_visible(m["mask"]["size"]), softcap=m.get("softcap"))
    o = o * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, -1) @ w["o"].T


# --------------------------------------------------- mixer: chunked attention beside a delta rule

def chunked_attention(h, w, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w["q"].T).view(T, H, D), m["rot"], "pairs")
    k = rotate((h @ w["k"].T).view(T, G, D), m["rot"], "pairs")
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    v = (h @ w["v"].T).view(T, G, V)
    o = attend(q, k, v, m["scale"], chunk_visible(m["mask"]["size"]), zero_sink=True)
    return o.reshape(T, -1) @ w["o"].T


def short_conv(x, taps):
    """Causal convolution over time per channel: ``x`` [T, C], ``taps`` [C, K] whose last
    column meets the current token; zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1 - j)
            if src >= 0:
                out[t] = out[t] + taps[:, j] * x[src]
    return out


def unit_vector(x):
    return x / torch.sqrt(x.pow(2).sum(dim=-1, keepdim=True) + UNIT_EPS)


def delta_recurrence(q, k, v, beta, decay):
    """``q``, ``k`` [T, D]; ``v`` [T, V]; ``beta`` [T]; ``decay`` [T, D] (one factor per key
    channel).  The state S is [D, V] and starts at zero; the read-out sees the current
    token's write."""
    T, D = q.shape
    S = torch.zeros((D, v.shape[1]), dtype=q.dtype)
    out = torch.zeros_like(v)
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, V)
    q, k = unit_vector(q) * D ** -0.5, unit_vector(k)
    beta = sigmoid(h @ w["b"].T)                                             # [T, H]
    rate = softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * rate)           # [T, H, D]
    gate = sigmoid((h @ w["g1"].T) @ w["g2"].T).view(T, H, V)
    o = torch.zeros((T, H, V), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        o[:, head] = delta_recurrence(q[:, g], k[:, g], v[:, head], beta[:, head],
                                      decay[:, head])
    o = rms_unit(o, eps) * w["norm"] * gate
    return o.reshape(T, -1) @ w["o"].T


def parallel_mixer(h, w_left, w_right, m, eps):
    return m["left_scale"] * chunked_attention(h, w_left, m["left"], eps) + \
        m["right_scale"] * delta_mixer(h, w_right, m["right"], eps)


# ------------------------------------------------------------------------------ feed-forward

def feed_forward(h, w, m):
    limit = m["limit"]
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, min=-limit, max=limit)
    return (g * sigmoid(SWISH_SLOPE * g) * (u + 1.0)) @ w["down"].T


# --------------------------------------------------------------------------------- the model

def sub(tensors, prefix):
    """The tensors below ``prefix.`` by their short names."""
    return {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}


def forward(config, tensors, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence.  ``streams`` (a list): receives the residual
    stream after every layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = layer_norm(x, t["embed.norm"], t["embed.norm.b"], eps)
    kept = {}       # layer -> (k, v) of attention layers, for layers that borrow them
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        h = layer_norm(x, t[f"l{i}.norm1"], t[f"l{i}.norm1.b"], eps)
        w = sub(t, f"l{i}.mix")
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, w, m, eps)
            branch = attention_mixer(h, w, m, eps, kept[i if src is None else src])
        elif layer["type"] == "parallel":
            branch = parallel_mixer(h, sub(t, f"l{i}.mix.left"), sub(t, f"l{i}.mix.right"), m, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        if layer.get("mlp") is not None:
            branch = branch + feed_forward(h, sub(t, f"l{i}.mlp"), layer["mlp"])
        x = x + mult * branch
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    logits = x @ t["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
