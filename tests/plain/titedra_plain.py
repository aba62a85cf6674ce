"""A plain, slow Titedra: whole sequences, no cache, 64-bit, one function per mechanism.  It
shares no code with the package; the tests compare the engine with it.

``w`` maps tensor names to 64-bit tensors; a mixer's and a feed-forward's functions take the
tensors below their own prefix (``dq``, ``uq``, ..., ``router``, ``e0.up``, ...).
"""

import math

import torch


def rms_unit(x, eps):
    """x over its root mean square, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, gain, eps):
    """RMS norm whose gain is stored around zero."""
    return rms_unit(x, eps) * (1.0 + gain)


def rotate_split_half(v, positions, dims, base):
    """v: [T, ..., n]; the first ``dims`` entries turn: entry i with entry i + dims / 2 by the
    angle position * base^(-2i / dims); the rest pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    angle = positions.double()[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = angle.cos().view(shape), angle.sin().view(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def latent_attention(h, w, m, eps):
    """h: [T, width] (already normed).  Keys and values per head are formed from the latent, as
    the definition has them (not absorbed into the queries)."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, d + r)
    down = h @ w["dkv"].T
    c = rms_unit(down[:, :R], eps) * w["dkv.norm"]
    k_rot = rotate_split_half(down[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])     # [T, r]
    q_rot = rotate_split_half(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"])      # [T, H, r]
    k = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=torch.float64)
    gate = torch.sigmoid(h @ w["g"].T)                                                 # [T, H]
    for head in range(H):
        s = (q[:, head, :d] @ k[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, head] * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ w["o"].T


def dense_ff(h, w):
    z = h @ w["gate"].T
    return (z * torch.sigmoid(z) * (h @ w["up"].T)) @ w["down"].T


def route(h, w, router):
    """(chosen experts per token in the order they are taken, their weights)."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w["router"].T)
    chosen, weights = [], []
    per = E // groups["count"]
    for t in range(h.shape[0]):
        choice = (s[t] + w["correction"]).tolist()
        if groups["keep"] < groups["count"]:
            score = []
            for g in range(groups["count"]):
                best = sorted(choice[g * per:(g + 1) * per], reverse=True)
                score.append(best[0] + best[1] if per > 1 else best[0])
            kept = sorted(range(groups["count"]), key=lambda g: (-score[g], g))[:groups["keep"]]
            choice = [c if e // per in kept else -math.inf for e, c in enumerate(choice)]
        ids = sorted(range(E), key=lambda e: (-choice[e], e))[:top]
        chosen.append(ids)
        weights.append(torch.stack([s[t, e] for e in ids]))
    return chosen, weights


def moe_ff(h, w, mlp):
    chosen, weights = route(h, w, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t], weights[t]):
            hidden = torch.relu(w[f"e{e}.up"] @ h[t]).pow(2)
            out[t] += weight * (w[f"e{e}.down"] @ hidden)
    return out


def below(w, prefix):
    return {k[len(prefix) + 1:]: v for k, v in w.items() if k.startswith(prefix + ".")}


def run_order(cfg):
    """(layer, whether a pass of the loop starts there) in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    order = [(i, False) for i in range(a)]
    for _ in range(loop["times"]):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, tensors, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; ``streams`` (a list) receives the residual
    stream after every layer run."""
    w = {k: v.double() for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    first = x
    for i, starts in run_order(cfg):
        if starts:
            x = torch.cat([x, first], -1) @ w["loop.in"].T
        layer, p = cfg["layers"][i], f"l{i}"
        y = latent_attention(norm_around_zero(x, w[p + ".norm1"], eps), below(w, p + ".mix"),
                             layer["mixer"], eps)
        x = x + norm_around_zero(y, w[p + ".norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_around_zero(x, w[p + ".norm2"], eps)
            y = dense_ff(h, below(w, p + ".mlp")) if mlp["kind"] == "dense" \
                else moe_ff(h, below(w, p + ".mlp"), mlp)
            x = x + norm_around_zero(y, w[p + ".norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
