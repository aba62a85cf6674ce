"""Tubevik configurations drawn at random with fixed seeds (every size, head counts and groups,
value sizes, rotated parts, windows and chunks, taps, caps, the order of layers, borrowed cache
entries with windows of their own, layers without a feed-forward, page sizes), each through a
whole and a mixed trace in both precisions against the plain implementation, free pages
poisoned."""

import random

import pytest
import torch

import trace_util as T
import tubevik_util as U
from plain import tubevik_plain as P
from test_tubevik_model_gpu import compare, make_runner

pytestmark = pytest.mark.gpu


def draw_mlp(rng):
    if rng.random() < 0.25:
        return None
    return U.dense(rng.choice([24, 56, 100, 160]), rng.choice([0.5, 1.0, 3.0, 7.0]))


def draw_attention(rng, kv_from=None, like=None):
    if like is not None:         # a layer that borrows keys: same heads, sizes and rotation
        m = like["mixer"]
        rot = m["rot"]
        sc = rot.get("scaling")
        return U.attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"],
                           rng.choice([1, 3, 17, 40, 200]), rot_dims=rot["dims"], base=rot["base"],
                           scale=rng.choice([0.1, 0.3]), softcap=rng.choice([None, 5.0, 25.0]),
                           scaling=None if sc is None else tuple(sc[k] for k in
                                                                  ("factor", "original", "fast", "slow")),
                           kv_from=kv_from, mlp=draw_mlp(rng))
    # (head sizes are drawn so that the attention kernels are compiled for few: the padded size
    # is 16, 32, 64 or 128)
    dim, vdim = rng.choice([(8, 16), (12, 10), (32, 32), (20, 32), (64, 48), (64, 64), (128, 128)])
    kv = rng.choice([1, 2, 3])
    rot_dims = rng.choice([dim, 2 * rng.randint(1, dim // 2)])
    scaling = None
    if rng.random() < 0.6:
        scaling = (rng.choice([1.5, 2.0, 8.0]), rng.choice([16, 64, 512]),
                   rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0]))
    return U.attention(kv * rng.choice([1, 2, 4]), kv, dim, vdim, rng.choice([1, 5, 24, 60, 300]),
                       rot_dims=rot_dims, base=rng.choice([30.0, 10000.0, 2e6]),
                       scale=rng.choice([0.1, 0.3, dim ** -0.5]),
                       softcap=rng.choice([None, 3.0, 25.0]), scaling=scaling, mlp=draw_mlp(rng))


def draw_parallel(rng):
    dim, vdim = rng.choice([(8, 16), (12, 10), (32, 32), (64, 64), (64, 24)])
    kv = rng.choice([1, 2])
    left = (kv * rng.choice([1, 2, 3]), kv, dim, vdim, rng.choice([1, 4, 19, 64, 250]),
            2 * rng.randint(1, dim // 2), rng.choice([50.0, 3e5]), rng.choice([0.15, 0.4]))
    rkv = rng.choice([1, 2, 3])
    right = (rkv * rng.choice([1, 2]), rkv, rng.choice([8, 16, 33, 64]),
             rng.choice([4, 16, 24, 64]), rng.choice([1, 2, 4]))
    return U.parallel(left, right, rng.choice([1.0, 0.75, -0.5]), rng.choice([1.0, 1.25, 0.3]),
                      mlp=draw_mlp(rng))


def draw(seed):
    rng = random.Random(5000 + seed)
    layers = []
    for i in range(rng.randint(1, 5)):
        owners = [j for j, l in enumerate(layers)
                  if l["type"] == "attention" and "kv_from" not in l["mixer"]]
        kind = rng.choice(["attention", "parallel", "borrow" if owners else "parallel"])
        if kind == "attention":
            layers.append(draw_attention(rng))
        elif kind == "parallel":
            layers.append(draw_parallel(rng))
        else:
            j = rng.choice(owners)
            layers.append(draw_attention(rng, kv_from=j, like=layers[j]))
    cfg = U.config(rng.choice([50, 128, 301]), rng.choice([32, 40, 64, 96, 128, 256]), layers,
                   eps=rng.choice([1e-5, 1e-6, 3e-4]), residual_mult=rng.choice([1.0, 0.5, 0.3]),
                   logit_softcap=rng.choice([0.0, 10.0, 20.0]))
    lengths = [rng.randint(1, 140) for _ in range(5)] + [rng.choice([1, 2])]
    return cfg, lengths, rng.choice([8, 16, 32, 64])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(seed, dtype, tmp_path):
    from scratch_llm_b200.kernels import ops
    cfg, lengths, page = draw(seed)
    tensors = U.random_tensors(cfg, 600 + seed)
    folder = U.write_model(cfg, tensors, tmp_path / "m")
    reqs = T.make_requests(cfg["vocab"], lengths, seed=seed)
    want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    for steps in (T.whole(reqs), T.mixed(reqs, seed=seed)):
        runner = make_runner(folder, dtype, page, T.peak_tokens(steps, round_to=max(64, page)),
                             max_requests=4, poison_free_pages=True)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        ops.check_kernel_errors()
        assert len(got) == sum(lengths)
        compare(got, want, dtype)
