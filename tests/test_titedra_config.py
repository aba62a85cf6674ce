"""The Titedra configuration without a GPU: config.json keys to layers as data, tensor names,
the order in which looped layers run and the cache entry each run holds, and the plain
implementation's own properties (causality, the router's groups, the join of every pass)."""

import copy
import math

import pytest
import torch

import titedra_util as U
from plain import titedra_plain as P


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


def test_looped_layers_run_again_with_cache_entries_of_their_own():
    cfg = U.CONFIGS["X"]                     # four layers, layers 1 and 2 three times
    model = build(cfg)
    assert len(model.spec.layers) == 4
    order = model.spec.order
    assert [r.layer for r in order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [r.cache for r in order] == list(range(8))
    # the stream meets the embedding output before the first layer of every pass, the first too
    assert [r.join for r in order] == [None, 0, None, 0, None, 0, None, None]
    kv, st = model.cache_specs()
    assert len(kv) == 8 and all(s is None for s in st)
    # one vector per token: one kv head, one plane, latent + rotated part up to a multiple of 16
    assert all(k.planes == 1 and k.n_kv_heads == 1 for k in kv)
    assert [k.head_dim for k in kv] == [32, 32, 48, 32, 48, 32, 48, 64]
    assert kv[1] == kv[3] == kv[5]


def test_loops_at_the_start_over_everything_once_and_absent():
    z = build(U.CONFIGS["Z"]).spec.order      # both layers twice
    assert [(r.layer, r.join) for r in z] == [(0, 0), (1, None), (0, 0), (1, None)]
    y = build(U.CONFIGS["Y"])                 # no loop: no join and no joining matrix
    assert [(r.layer, r.join) for r in y.spec.order] == [(0, None), (1, None), (2, None)]
    assert "loop.in" not in y.param_specs()
    once = copy.deepcopy(U.CONFIGS["Y"])
    once["loop"] = {"start": 2, "stop": 3, "times": 1}
    m = build(once)                           # a loop that runs once still joins
    assert [(r.layer, r.join) for r in m.spec.order] == [(0, None), (1, None), (2, 0)]
    assert m.param_specs()["loop.in"].shape == (64, 128)


def test_config_errors_name_the_key():
    from scratch_llm_b200.config import config_from_dict
    base = U.CONFIGS["X"]
    for path, value, word in [(("layers", 1, "mixer", "rot", "dims"), 5, "rot.dims"),
                              (("layers", 1, "mixer", "rot", "dims"), 8, "rot.dims"),
                              (("layers", 0, "mixer", "kv_rank"), 0, "kv_rank"),
                              (("layers", 1, "mlp", "router", "top"), 0, "top"),
                              (("layers", 0, "type"), "other", "type"),
                              (("layers", 0, "mlp", "kind"), "glu", "kind"),
                              (("loop", "stop"), 9, "loop"),
                              (("loop", "times"), 0, "loop"),
                              (("vocab",), -3, "vocab")]:
        cfg = copy.deepcopy(base)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ValueError, match=word):
            config_from_dict(cfg)
    cfg = copy.deepcopy(base)
    cfg["layers"][1]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}   # 6 experts, 4 groups
    with pytest.raises(ValueError, match="groups"):
        build(cfg)


def test_round_trip_of_the_configuration():
    from scratch_llm_b200.config import config_from_dict
    for cfg in U.CONFIGS.values():
        first = config_from_dict(cfg)
        assert first.architecture == "Titedra"
        again = config_from_dict(first.to_dict())
        assert again.to_dict() == first.to_dict()
        assert again.to_dict()["layers"] == cfg["layers"]
        assert again.to_dict().get("loop") == cfg.get("loop")


def test_random_model_folder_opens(tmp_path):
    """The package's own random weights for this architecture: every tensor it names is written
    and read back, gains stored around zero among them."""
    from scratch_llm_b200.config import config_from_dict, load_config
    from scratch_llm_b200.weights import write_random_model
    from scratch_llm_b200.weights import SafetensorsFile
    cfg = config_from_dict(U.CONFIGS["Y"])
    write_random_model(cfg, tmp_path, 3)
    assert load_config(tmp_path).to_dict() == cfg.to_dict()
    file = SafetensorsFile(tmp_path / "model.safetensors")
    assert set(file) == set(build(U.CONFIGS["Y"]).param_specs())
    file.close()


# ------------------------------------------------------------------ the plain model itself

def test_plain_model_is_causal():
    cfg = U.CONFIGS["X"]
    tensors = U.random_tensors(cfg, 3)
    toks = [5, 9, 90, 3, 77, 20, 1, 64]
    full = P.forward(cfg, tensors, toks)
    part = P.forward(cfg, tensors, toks[:5])
    torch.testing.assert_close(full[:5], part, rtol=1e-9, atol=1e-9)


def test_plain_rotation_turns_pairs_half_apart_and_passes_the_rest():
    v = torch.arange(1.0, 9.0, dtype=torch.float64).repeat(3, 1)          # [3, 8]
    out = P.rotate_split_half(v, torch.tensor([0, 1, 7]), 4, 100.0)
    torch.testing.assert_close(out[0], v[0])                               # position 0: no turn
    torch.testing.assert_close(out[:, 4:], v[:, 4:])                       # beyond dims: unchanged
    for row, p in ((1, 1.0), (2, 7.0)):
        for i, f in ((0, 1.0), (1, 100.0 ** -0.5)):
            a, u, w = p * f, v[row, i], v[row, i + 2]
            assert out[row, i].item() == pytest.approx(u * math.cos(a) - w * math.sin(a))
            assert out[row, i + 2].item() == pytest.approx(w * math.cos(a) + u * math.sin(a))


def test_plain_router_scores_groups_by_their_two_best_and_bars_the_rest_below_any_score():
    # six experts in three groups of two, one group stays; every choice score is negative, so a
    # barred expert that counted as 0 would be chosen
    w = {"router": torch.eye(6, dtype=torch.float64),
         "correction": torch.tensor([-2.0, -2.0, -1.2, -3.0, -1.9, -1.9], dtype=torch.float64)}
    h = torch.tensor([[0.0, 0.0, 4.0, -4.0, 0.5, 0.5]], dtype=torch.float64)
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    s = torch.sigmoid(h[0])
    # group sums: (-1.5, -1.5), (s2 - 1.2 ~ -0.22, s3 - 3 ~ -2.98), (~ -1.28, ~ -1.28):
    # group 2 wins by its sum although group 1 holds the single best expert
    chosen, weights = P.route(h, w, r)
    assert chosen[0] == [4, 5]
    torch.testing.assert_close(weights[0], s[[4, 5]])          # plain scores, not renormalised
    r["groups"] = {"count": 3, "keep": 3}
    chosen, weights = P.route(h, w, r)
    assert chosen[0] == [2, 4]
    torch.testing.assert_close(weights[0], s[[2, 4]])


def test_plain_model_joins_the_embedding_output_before_every_pass():
    """With a joining matrix [0 | I] every pass starts from the embedding output again: three
    passes give what one gives."""
    cfg = copy.deepcopy(U.CONFIGS["X"])
    tensors = U.random_tensors(cfg, 5)
    d = cfg["width"]
    tensors["loop.in"] = torch.cat([torch.zeros(d, d), torch.eye(d)], 1)
    toks = [3, 50, 7, 7, 12]
    three = P.forward(cfg, tensors, toks)
    cfg["loop"]["times"] = 1
    one = P.forward(cfg, tensors, toks)
    torch.testing.assert_close(three, one, rtol=1e-9, atol=1e-9)
    streams = []
    P.forward(U.CONFIGS["X"], tensors, toks, streams)
    assert len(streams) == 8 and streams[0].shape == (5, d)
