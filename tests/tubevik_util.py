"""Small Tubevik configurations with random tensors of every kind (norms with offsets, biases,
wide q/k gains, head gates, convolutions, low-rank decays and gates), written as model folders,
for the tests of that architecture."""

import torch

from nilevik_util import relative_error, write_model  # noqa: F401  (shared test helpers)


def attention(heads, kv_heads, dim, vdim, window, rot_dims=None, base=10000.0, scale=None,
              softcap=None, scaling=None, kv_from=None, mlp=None):
    rot = {"base": base, "dims": rot_dims if rot_dims is not None else dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window},
             "rot": rot}
    if softcap is not None:
        mixer["softcap"] = softcap
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def parallel(left, right, left_scale=1.0, right_scale=1.0, mlp=None):
    """``left``: (heads, kv_heads, dim, vdim, chunk, rot_dims, base, scale); ``right``: (heads,
    kv_heads, dim, vdim, conv)."""
    lh, lg, ld, lv, chunk, rot_dims, base, scale = left
    rh, rg, rd, rv, conv = right
    return {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": scale,
                 "mask": {"size": chunk}, "rot": {"base": base, "dims": rot_dims}},
        "right": {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": conv},
        "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(vocab, width, layers, eps=1e-5, residual_mult=1.0, logit_softcap=0.0):
    return {"architecture": "Tubevik", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "residual_mult": residual_mult, "logit_softcap": logit_softcap, "layers": layers}


# Sizes differ from one configuration to the next in everything: a parallel layer first and an
# attention layer first; head counts from 1 to 6 with groups of 1, 2 and 3; value sizes smaller
# and larger than key sizes; head sizes that are no multiple of 16; rotations of a part of a
# head and of all of it, with and without blended frequencies; windows and chunks of 1, of a
# few tokens and longer than most prompts; a borrowed cache entry read through a wider and
# through a narrower window than its owner's; one, two and four convolution taps; layers
# without a feed-forward; with and without caps.
CONFIGS = {
    "P": config(97, 48, [
        parallel((3, 1, 12, 20, 7, 8, 500.0, 0.4), (4, 2, 6, 10, 3), 0.7, 1.3, mlp=dense(40, 0.8)),
        attention(4, 2, 16, 8, 9, rot_dims=8, base=300.0, softcap=4.0,
                  scaling=(3.0, 16, 4.0, 0.5), mlp=dense(72, 2.5)),
        parallel((2, 2, 8, 8, 1, 8, 50.0, 0.5), (2, 1, 16, 12, 1), 1.0, 0.5, mlp=None),
        attention(4, 2, 16, 8, 21, rot_dims=8, base=300.0, softcap=4.0,
                  scaling=(3.0, 16, 4.0, 0.5), kv_from=1, mlp=dense(24, 1.0)),
    ], eps=1e-5, residual_mult=0.6, logit_softcap=12.0),
    "Q": config(131, 64, [
        attention(2, 1, 24, 24, 1, base=10000.0, scale=0.3, mlp=None),
        attention(6, 2, 8, 16, 30, rot_dims=4, base=40.0, softcap=50.0, mlp=dense(80, 1.0)),
        attention(6, 2, 8, 16, 5, rot_dims=4, base=40.0, softcap=50.0, kv_from=1, mlp=dense(56, 7.0)),
        parallel((1, 1, 32, 16, 200, 32, 1e6, 0.2), (3, 3, 20, 7, 2), -0.9, 1.0, mlp=dense(33, 0.5)),
    ], eps=3e-6, residual_mult=1.0, logit_softcap=0.0),
    # head sizes 64 and 128: the shapes of the tensor-core attention kernels; a key size of 128
    # in the recurrence
    "R": config(300, 128, [
        attention(4, 2, 64, 64, 100, base=2e5, softcap=20.0, scaling=(4.0, 128, 16.0, 2.0),
                  mlp=dense(192, 1.5)),
        parallel((4, 1, 128, 128, 64, 64, 1e5, 0.09), (2, 1, 128, 64, 4), 0.9, 1.2,
                 mlp=dense(160, 2.0)),
        attention(4, 2, 64, 64, 130, base=2e5, softcap=20.0, scaling=(4.0, 128, 16.0, 2.0),
                  kv_from=0, mlp=dense(96, 1.5)),
    ], eps=1e-5, residual_mult=0.4, logit_softcap=25.0),
}


def random_tensors(cfg, seed):
    """{name: tensor} for every tensor of the architecture, as bfloat16-exact values in 32-bit
    (so that both precisions and the plain model hold the same numbers)."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std=1.0, mean=0.0):
        t = torch.randn(shape, generator=g) * std + mean
        return t.to(torch.bfloat16).float()

    def norm(name, t, d):
        t[name] = normal((d,), 0.2, 1.0)
        t[name + ".b"] = normal((d,), 0.2)

    d, V = cfg["width"], cfg["vocab"]
    t = {"embed": normal((V, d)), "head": normal((V, d), d ** -0.5)}
    norm("embed.norm", t, d)
    norm("final.norm", t, d)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        norm(p + "norm1", t, d)
        if layer["type"] == "attention":
            H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            names = ["q"] + ([] if m.get("kv_from") is not None else ["k", "v"])
            for n in names:
                rows = {"q": H * D, "k": G * D, "v": G * Vd}[n]
                t[p + f"mix.{n}"] = normal((rows, d), d ** -0.5)
                t[p + f"mix.{n}.b"] = normal((rows,), 0.3)
                if n != "v":
                    t[p + f"mix.{n}.norm"] = normal((rows,), 0.3, 1.0)
            t[p + "mix.g"] = normal((H, d), 2.0 * d ** -0.5)
            t[p + "mix.o"] = normal((d, H * Vd), (H * Vd) ** -0.5)
        else:
            L, R = m["left"], m["right"]
            H, G, D, Vd = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            t[p + "mix.left.q"] = normal((H * D, d), d ** -0.5)
            t[p + "mix.left.k"] = normal((G * D, d), d ** -0.5)
            t[p + "mix.left.v"] = normal((G * Vd, d), d ** -0.5)
            t[p + "mix.left.o"] = normal((d, H * Vd), (H * Vd) ** -0.5)
            H, G, D, Vd, K = R["heads"], R["kv_heads"], R["dim"], R["vdim"], R["conv"]
            ra, rg = 5 + i, 3 + 2 * i        # the low ranks: the tensors alone say them
            q = p + "mix.right."
            t[q + "q"] = normal((G * D, d), d ** -0.5)
            t[q + "k"] = normal((G * D, d), d ** -0.5)
            t[q + "v"] = normal((H * Vd, d), d ** -0.5)
            t[q + "q.conv"] = normal((G * D, K), 0.6)
            t[q + "k.conv"] = normal((G * D, K), 0.6)
            t[q + "v.conv"] = normal((H * Vd, K), 0.6)
            t[q + "b"] = normal((H, d), d ** -0.5)
            t[q + "A_log"] = normal((H,), 0.7, -1.0)
            t[q + "a1"] = normal((ra, d), d ** -0.5)
            t[q + "a2"] = normal((H * D, ra), 1.5 * ra ** -0.5)
            t[q + "dt_bias"] = normal((H * D,), 0.7)
            t[q + "g1"] = normal((rg, d), d ** -0.5)
            t[q + "g2"] = normal((H * Vd, rg), 2.0 * rg ** -0.5)
            t[q + "norm"] = normal((Vd,), 0.2, 1.0)
            t[q + "o"] = normal((d, H * Vd), (H * Vd) ** -0.5)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            t[p + "mlp.gate"] = normal((f, d), 1.5 * d ** -0.5)
            t[p + "mlp.up"] = normal((f, d), 1.5 * d ** -0.5)
            t[p + "mlp.down"] = normal((d, f), f ** -0.5)
    return t
