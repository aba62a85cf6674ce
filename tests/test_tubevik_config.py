"""The Tubevik configuration without a GPU: config.json keys to layers as data, tensor names,
which run reads whose cache entry and through which window, what the configuration refuses,
and the plain implementation's own properties (causality, windows, chunks, the state)."""

import copy

import pytest
import torch

import tubevik_util as U
from plain import tubevik_plain as P


def build(cfg):
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine.model import build_model
    return build_model(config_from_dict(cfg))


@pytest.mark.parametrize("name", list(U.CONFIGS))
def test_tensor_names_are_those_of_the_random_model(name):
    cfg = U.CONFIGS[name]
    specs = build(cfg).param_specs()
    tensors = U.random_tensors(cfg, 0)
    assert set(specs) == set(tensors)
    for key, spec in specs.items():
        got = tuple(tensors[key].shape)
        assert len(got) == len(spec.shape)
        assert all(w in (-1, g) for g, w in zip(got, spec.shape)), key


def test_a_borrowing_layer_reads_its_owner_s_entry_and_widens_its_window():
    model = build(U.CONFIGS["P"])       # parallel, attention, parallel, attention from layer 1
    order = model.spec.order
    assert [(r.layer, r.cache, r.write) for r in order] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    kv, st = model.cache_specs()
    assert len(kv) == 3
    # chunks are kept like windows; the borrowed entry keeps what its farthest reader sees
    # (the owner's window is 9, the borrower's 21)
    assert [k.window for k in kv] == [7, 21, 1]
    assert kv[1].n_kv_heads == 2 and kv[1].head_dim == 16
    assert "l3.mix.k" not in model.param_specs() and "l3.mix.q" in model.param_specs()
    # the parallel layers carry the recurrence's matrix and the convolution's inputs
    assert st[1] is None
    assert [tuple(s.shape) for s in st[0]] == [(4, 10, 6), (2, 2 * 2 * 6 + 4 * 10)]
    assert len(st[2]) == 1               # one tap: nothing to carry beside the matrix
    q = build(U.CONFIGS["Q"])            # the borrower's window (5) is inside the owner's (30)
    assert [k.window for k in q.cache_specs()[0]] == [1, 30, 200]


def test_round_trip_and_refusals():
    from scratch_llm_b200.config import TubevikConfig, config_from_dict
    cfg = config_from_dict(U.CONFIGS["P"])
    assert isinstance(cfg, TubevikConfig)
    again = config_from_dict(cfg.to_dict())
    assert again == cfg and again.model_spec() == cfg.model_spec()

    def broken(change):
        c = copy.deepcopy(U.CONFIGS["P"])
        change(c)
        return c

    bad = [lambda c: c["layers"][3]["mixer"].update(kv_from=3),          # not an earlier layer
           lambda c: c["layers"][3]["mixer"].update(kv_from=0),          # not an attention layer
           lambda c: c["layers"][3]["mixer"].update(kv_heads=4),         # other heads than its owner
           lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18),     # beyond the head
           lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5),
           lambda c: c["layers"][0]["mixer"]["left"].update(heads=4, kv_heads=3),
           lambda c: c["layers"][0].update(type="delta"),
           lambda c: c["layers"][1]["mlp"].update(limit=0.0),
           lambda c: c["layers"][1]["mlp"].update(kind="moe"),
           lambda c: c.pop("residual_mult"),
           lambda c: c["norm"].update(eps=0.0)]
    for change in bad:
        with pytest.raises(ValueError):
            config_from_dict(broken(change))


def test_plain_model_is_causal_and_forgets_behind_its_masks():
    cfg = U.CONFIGS["P"]
    tensors = U.random_tensors(cfg, 3)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    base = P.forward(cfg, tensors, toks)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab"]
    changed = P.forward(cfg, tensors, other)
    assert torch.equal(changed[:30], base[:30])
    assert (changed[30:] - base[30:]).abs().max() > 1e-3     # the recurrence carries it on


def test_plain_pieces():
    # a window of w keys: itself and the w - 1 before it; chunks count from position 0
    assert [j for j in range(10) if P.window_visible(3)(7, j)] == [5, 6, 7]
    assert [j for j in range(10) if j <= 8 and P.chunk_visible(4)(8, j)] == [8]
    assert [j for j in range(10) if j <= 7 and P.chunk_visible(4)(7, j)] == [4, 5, 6, 7]
    # a sink of score 0 takes its share of the weights
    q = torch.zeros((1, 1, 4), dtype=torch.float64)
    k = torch.zeros((1, 1, 4), dtype=torch.float64)
    v = torch.ones((1, 1, 2), dtype=torch.float64)
    assert torch.allclose(P.attend(q, k, v, 1.0, P.window_visible(5), zero_sink=True),
                          torch.full((1, 1, 2), 0.5, dtype=torch.float64))
    # blended frequencies: the fastest pairs keep theirs, the slowest are divided by the factor
    f, mag = P.yarn_frequencies(10000.0, 64, {"factor": 4.0, "original": 256, "fast": 32.0,
                                              "slow": 1.0})
    plain = P.plain_frequencies(10000.0, 64)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 4.0) < 1e-12 and mag > 1.0
    # the convolution's last tap meets the current token
    x = torch.arange(1.0, 5.0)[:, None]
    taps = torch.tensor([[100.0, 10.0, 1.0]])
    assert P.short_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0]
    # the recurrence reads the token's own write: one token, beta 1, unit key = query
    k1 = torch.tensor([[1.0, 0.0]])
    out = P.delta_recurrence(k1, k1, torch.tensor([[3.0, 5.0]]), torch.ones(1),
                             torch.full((1, 2), 0.5))
    assert out.tolist() == [[3.0, 5.0]]
