"""Small Titedra configurations with random tensors of every kind (latent projections with their
norms, gates, norms stored around zero, routers with corrections, the loop's joining matrix),
written as model folders, for the tests of that architecture."""

import math

import torch

from nilevik_util import relative_error, write_model  # noqa: F401  (shared test helpers)


def layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, scale=None, rot_dims=None,
          mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
             "kv_rank": kv_rank,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim),
             "rot": {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(vocab, width, layers, loop=None, eps=1e-5, embedding_scale=1.0, logit_scale=1.0):
    cfg = {"architecture": "Titedra", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Sizes differ from one configuration to the next in everything: head counts from 1 to 9, rotated
# parts larger and smaller than the unrotated ones, value sizes other than key sizes, latents
# whose cached vector is and is not a multiple of 16 (and of 64), layers without a feed-forward,
# routers with and without groups, groups of one expert, every group kept, one choice and several,
# a loop in the middle, one that starts at the first layer, one over all layers, one that runs
# once, and no loop at all.
CONFIGS = {
    "X": config(97, 48, [layer(3, 8, 4, 10, 20, 24, base=500.0, mlp=dense(72)),
                         layer(5, 12, 6, 6, 16, 21, base=30.0, scale=0.3,
                               mlp=moe(40, 6, 2, groups=(3, 2))),
                         layer(2, 16, 16, 24, 40, 32, mlp=None),
                         layer(1, 4, 28, 16, 8, 36, base=100000.0, mlp=moe(24, 5, 5))],
                loop=(1, 3, 3), eps=1e-5, embedding_scale=7.0, logit_scale=0.5),
    "Y": config(131, 64, [layer(4, 16, 8, 16, 32, 40, base=10000.0, mlp=moe(32, 4, 1, groups=(4, 2))),
                          layer(9, 6, 2, 5, 24, 14, base=50.0, mlp=dense(80)),
                          layer(2, 20, 12, 32, 48, 52, mlp=moe(16, 8, 3, groups=(2, 2)))],
                eps=3e-6, embedding_scale=0.5, logit_scale=3.0),
    # cached vectors of 128 and 64 entries: the shapes of the tensor-core attention kernels
    "Z": config(300, 128, [layer(6, 24, 32, 40, 64, 96, base=150000.0, mlp=moe(64, 9, 3, groups=(3, 1))),
                           layer(4, 64, 16, 64, 96, 48, base=300.0, mlp=dense(192))],
                loop=(0, 2, 2), eps=1e-6, embedding_scale=11.0, logit_scale=1.5),
}


def random_tensors(cfg, seed):
    """{name: tensor} for every tensor of the architecture, as bfloat16-exact values in 32-bit
    (so that both precisions and the plain model hold the same numbers)."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std=1.0, mean=0.0):
        t = torch.randn(shape, generator=g) * std + mean
        return t.to(torch.bfloat16).float()

    d, V = cfg["width"], cfg["vocab"]
    # the stream is the embedding times its scale: keep the product of order 1
    t = {"embed": normal((V, d), 1.0 / abs(cfg["embedding"]["scale"])),
         "head": normal((V, d), d ** -0.5), "final.norm": normal((d,), 0.2)}
    if cfg.get("loop") is not None:
        t["loop.in"] = normal((d, 2 * d), (2 * d) ** -0.5)
    for i, one in enumerate(cfg["layers"]):
        m, p = one["mixer"], f"l{i}."
        H, dim, r, dv, Rq, R = (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"],
                                m["kv_rank"])
        for name in ("norm1", "norm1b"):
            t[p + name] = normal((d,), 0.2)           # stored around zero
        t[p + "mix.dq"] = normal((Rq, d), d ** -0.5)
        t[p + "mix.dq.norm"] = normal((Rq,), 0.2, 1.0)  # a plain gain
        t[p + "mix.uq"] = normal((H * (dim + r), Rq), Rq ** -0.5)
        t[p + "mix.dkv"] = normal((R + r, d), d ** -0.5)
        t[p + "mix.dkv.norm"] = normal((R,), 0.2, 1.0)
        t[p + "mix.uk"] = normal((H * dim, R), R ** -0.5)
        t[p + "mix.uv"] = normal((H * dv, R), R ** -0.5)
        t[p + "mix.g"] = normal((H, d), 2.0 * d ** -0.5)
        t[p + "mix.o"] = normal((d, H * dv), (H * dv) ** -0.5)
        mlp = one["mlp"]
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            t[p + name] = normal((d,), 0.2)
        if mlp["kind"] == "dense":
            f = mlp["ff"]
            t[p + "mlp.gate"] = normal((f, d), d ** -0.5)
            t[p + "mlp.up"] = normal((f, d), d ** -0.5)
            t[p + "mlp.down"] = normal((d, f), f ** -0.5)
            continue
        E, f = mlp["router"]["experts"], mlp["expert"]["ff"]
        t[p + "mlp.router"] = normal((E, d), 2.0 * d ** -0.5)
        # corrections large enough to change the choice, most below zero: sigmoid scores lie in
        # (0, 1), so choice scores of both signs occur
        t[p + "mlp.correction"] = normal((E,), 0.4, -0.5)
        for e in range(E):
            t[p + f"mlp.e{e}.up"] = normal((f, d), d ** -0.5)
            t[p + f"mlp.e{e}.down"] = normal((d, f), f ** -0.5)
    return t
