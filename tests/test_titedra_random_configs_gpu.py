"""Titedra configurations drawn at random with fixed seeds (every size, head counts, latent
sizes, rotated parts, scales, routers with and without groups, layers without a feed-forward,
loops anywhere, page sizes), each through a whole and a mixed trace in both precisions against
the plain implementation, free pages poisoned."""

import random

import pytest
import torch

import titedra_util as U
import trace_util as T
from plain import titedra_plain as P
from test_titedra_model_gpu import compare, make_runner

pytestmark = pytest.mark.gpu


def draw_mlp(rng):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return U.dense(rng.choice([24, 56, 100, 160]))
    groups = rng.choice([None, 2, 3, 4])
    if groups is None:
        experts = rng.randint(1, 10)
        return U.moe(rng.choice([8, 24, 40, 64, 136]), experts, rng.randint(1, min(4, experts)))
    per = rng.randint(1, 4)
    keep = rng.randint(1, groups)
    return U.moe(rng.choice([8, 24, 40, 64, 136]), groups * per,
                 rng.randint(1, min(4, keep * per)), groups=(groups, keep))


def draw(seed):
    rng = random.Random(3000 + seed)
    width = rng.choice([32, 40, 64, 96, 128, 256])
    layers = []
    for _ in range(rng.randint(1, 5)):
        dim = rng.choice([4, 8, 16, 24, 32, 64])
        # the cached vector (latent, rotated part, zeros up to a multiple of 16) has one of a few
        # sizes, so that the attention kernels are compiled for few
        cached = rng.choice([16, 32, 48, 64, 80, 128, 192, 256, 288])
        rot_dim = 2 * rng.randint(1, min(24, cached // 2 - 1))
        kv_rank = max(1, cached - rot_dim - rng.randint(0, 15))
        layers.append(U.layer(
            rng.choice([1, 2, 3, 4, 8, 12]), dim, rot_dim, rng.choice([8, 16, 24, 48, 64]),
            rng.choice([8, 24, 32, 64, 100]), kv_rank,
            base=rng.choice([30.0, 10000.0, 200000.0]), scale=rng.choice([None, 0.05, 0.3]),
            mlp=draw_mlp(rng)))
    loop = None
    if rng.random() < 0.7:
        a = rng.randrange(len(layers))
        b = rng.randint(a + 1, len(layers))
        # (at most eight layer runs: bfloat16 is compared with an exact model, and every routed
        # layer on the way may take another expert for a token whose choice scores are close)
        loop = (a, b, min(rng.randint(1, 3), max(1, (8 - len(layers)) // (b - a) + 1)))
    cfg = U.config(rng.choice([50, 128, 301]), width, layers, loop=loop,
                   eps=rng.choice([1e-5, 1e-6, 3e-4]),
                   embedding_scale=rng.choice([1.0, 4.0, 0.25, 13.0]),
                   logit_scale=rng.choice([1.0, 2.0, 0.3]))
    lengths = [rng.randint(1, 140) for _ in range(5)] + [rng.choice([1, 2])]
    return cfg, lengths, rng.choice([8, 16, 32, 64])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(seed, dtype, tmp_path):
    from scratch_llm_b200.kernels import ops
    cfg, lengths, page = draw(seed)
    tensors = U.random_tensors(cfg, 400 + seed)
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
