"""The Tubevik architecture through the engine: every way of cutting requests into steps gives
the logits of the plain implementation (tests/plain/tubevik_plain.py), in 32-bit and in
bfloat16, with small page pools whose free pages hold NaN and are used again; the residual
stream after every layer; greedy generation through the scheduler; the trace program."""

import copy

import pytest
import torch

import trace_util as T
import tubevik_util as U
from plain import tubevik_plain as P

pytestmark = pytest.mark.gpu

SEED = {"P": 51, "Q": 52, "R": 53}
# across several pages, windows and chunks; some of one or two tokens
LENGTHS = {"P": [1, 2, 50, 23, 77, 9, 64, 31], "Q": [3, 90, 41, 16, 130, 2, 57],
           "R": [150, 2, 71, 260, 33, 97]}
PAGE = {"P": 8, "Q": 16, "R": 16}
#: root mean square of the difference over that of the logits.  32-bit differs by the order of
#: its sums; in bfloat16 (the matrices are bfloat16-exact, the activations are rounded) the
#: bound is what rounding of the activations gives, which a fault in a mechanism exceeds by far.
BOUND = {"float32": 1e-4, "bfloat16": 0.06}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in U.CONFIGS.items():
        tensors = U.random_tensors(cfg, SEED[name])
        folder = U.write_model(cfg, tensors, tmp_path_factory.mktemp(f"tubevik_{name}"))
        reqs = T.make_requests(cfg["vocab"], LENGTHS[name], seed=SEED[name])
        want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
        out[name] = (cfg, tensors, folder, reqs, want)
    return out


def make_runner(folder, dtype, page, max_tokens, max_requests=4, **kw):
    from scratch_llm_b200.engine import ModelRunner, load_model
    model = load_model(folder, dtype, verbose=False)
    return ModelRunner(model, page, -(-max_tokens // page), max_requests, **kw)


def compare(got, want, dtype):
    assert got
    for (rid, pos), row in sorted(got.items()):
        err = U.relative_error(row, want[rid][pos])
        assert err < BOUND[dtype], f"request {rid} position {pos}: relative error {err:.3g}"


WAYS = {"whole": T.whole, "tail": lambda r: T.tail_one_by_one(r, tail=40),
        "portions": T.changing_portions, "mixed": T.mixed,
        "pairs": lambda r: T.chunks_of(r, 2), "ones": lambda r: T.chunks_of(r, 1)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("way", list(WAYS))
def test_replay_matches_plain(way, name, dtype, models):
    from scratch_llm_b200.kernels import ops
    cfg, _, folder, reqs, want = models[name]
    steps = WAYS[way](reqs)
    peak = T.peak_tokens(steps, round_to=64)
    # pages and state slots are used again by later requests
    runner = make_runner(folder, dtype, PAGE[name], peak, max_requests=4 if way == "mixed" else 2,
                         poison_free_pages=True)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    ops.check_kernel_errors()
    assert len(got) == sum(len(t) for t in reqs.values())
    compare(got, want, dtype)
    assert not runner.cache.requests
    assert all(g.pool.n_free == g.pool.n_pages for g in runner.cache.groups)


@pytest.mark.parametrize("name", ["P", "R"])
def test_residual_stream_after_every_layer(name, models):
    """The stream after each layer (what is pending added in), against the plain model's, for a
    prompt fed in two portions."""
    from scratch_llm_b200.engine import RowInput
    from scratch_llm_b200.parts.stream import Terms
    cfg, tensors, folder, reqs, _ = models[name]
    toks = max(reqs.values(), key=len)[:45]
    want = []
    P.forward(cfg, tensors, toks, streams=want)
    runner = make_runner(folder, "float32", PAGE[name], 64, max_requests=1)
    assert runner.admit("a")
    seen = []

    def probe(run, resid, pending):
        x = resid.float().clone()
        assert isinstance(pending, Terms)
        for t, coef in pending.items:
            x += coef * t.float()
        seen.append(x.cpu())

    runner.model.stream_probe = probe
    with torch.no_grad():
        runner.step([RowInput("a", toks[:30], [])])
        runner.step([RowInput("a", toks[30:], [])])
    runner.model.stream_probe = None
    n_runs = len(want)
    assert len(seen) == 2 * n_runs
    for k in range(n_runs):
        got = torch.cat([seen[k][:30], seen[n_runs + k][:len(toks) - 30]], 0)   # (steps are padded)
        err = (got - want[k].float()).norm() / want[k].float().norm()
        assert err < 1e-5, f"layer {k}: relative error {float(err):.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_steps_replayed_as_padded_graphs(dtype, models):
    """Steps of portions beside single tokens are padded to a few shapes and captured as CUDA
    graphs once a shape has come often enough: padding tokens and rows without tokens reach
    every kernel, the norms over whole projections and the recurrence among them."""
    cfg, _, folder, reqs, want = models["P"]
    steps = T.mixed(reqs, seed=9, sizes=(2, 3, 5))
    runner = make_runner(folder, dtype, PAGE["P"], T.peak_tokens(steps), poison_free_pages=True)
    assert runner.pad_small_steps
    runner.capture_padded_after = 2
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert runner.replayed_steps > len(steps) // 3
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_multiples_of_nothing(dtype, tmp_path):
    """A width, a vocabulary and feed-forward sizes that are multiples of neither 8 nor 4, head
    sizes that are no multiple of 16 or of 4, a rotation of two entries, one head, five taps:
    every kernel's plain path."""
    cfg = U.config(77, 50, [
        U.attention(3, 1, 6, 5, 11, rot_dims=2, base=7.0, scale=0.37, softcap=3.0,
                    scaling=(1.7, 8, 3.0, 0.7), mlp=U.dense(30, 1.3)),
        U.parallel((1, 1, 10, 3, 13, 6, 9.0, 0.21), (3, 1, 9, 5, 5), 1.2, 0.9, mlp=U.dense(13, 0.4)),
        U.attention(3, 1, 6, 5, 4, rot_dims=2, base=7.0, scale=0.37, softcap=3.0,
                    scaling=(1.7, 8, 3.0, 0.7), kv_from=0, mlp=None)],
        eps=2e-5, residual_mult=0.9, logit_softcap=5.0)
    tensors = U.random_tensors(cfg, 8)
    folder = U.write_model(cfg, tensors, tmp_path / "m")
    reqs = T.make_requests(cfg["vocab"], [37, 2, 60], seed=4)
    want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    for steps in (T.whole(reqs), T.mixed(reqs, seed=1, max_live=3)):
        runner = make_runner(folder, dtype, 16, T.peak_tokens(steps), max_requests=3,
                             poison_free_pages=True)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        compare(got, want, dtype)


def test_constants_matter(models, tmp_path):
    """Values that a model may happen to set to 1, to 0 or to equal each other: the multiplier
    on what a layer adds, the two sides' weights, the caps, the feed-forward's limit, the
    rotation's blend, a borrowed entry's own window: each changes the logits as in the plain
    model."""
    cfg0, tensors, _, reqs, _ = models["P"]
    toks = reqs["r4"]

    def changed(path, value):
        cfg = copy.deepcopy(cfg0)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        return cfg

    variants = [changed(("residual_mult",), 1.0), changed(("logit_softcap",), 0.0),
                changed(("layers", 0, "mixer", "left_scale"), 1.0),
                changed(("layers", 0, "mixer", "right_scale"), 0.25),
                changed(("layers", 1, "mlp", "limit"), 0.3),
                changed(("layers", 3, "mixer", "mask", "size"), 3),
                changed(("layers", 0, "mixer", "left", "mask", "size"), 30),
                changed(("layers", 0, "mixer", "left", "scale"), 1.5)]
    base = P.forward(cfg0, tensors, toks).float()
    for k, cfg in enumerate(variants):
        folder = U.write_model(cfg, tensors, tmp_path / f"m{k}")
        want = P.forward(cfg, tensors, toks).float()
        assert U.relative_error(want, base) > 1e-3, f"variant {k} changes nothing"
        runner = make_runner(folder, "float32", 8, 128, max_requests=1)
        with torch.no_grad():
            got = T.run_in_process(runner, T.whole({"a": toks}))
        compare(got, {"a": want}, "float32")


def test_cutting_does_not_change_logits_beyond_rounding(models):
    cfg, _, folder, reqs, _ = models["P"]
    ways = [T.whole(reqs), T.chunks_of(reqs, 2), T.mixed(reqs, seed=5)]
    runner = make_runner(folder, "float32", 8, max(T.peak_tokens(w) for w in ways))
    with torch.no_grad():
        a, b, c = (T.run_in_process(runner, w) for w in ways)
    for key in a:
        assert U.relative_error(b[key], a[key]) < 1e-4
        assert U.relative_error(c[key], a[key]) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, models):
    """A short prompt and then 300 tokens one by one, across many pages, windows and chunks:
    decode steps replay captured graphs, pages behind the windows are given back on the way."""
    cfg, tensors, folder, _, _ = models["R"]
    reqs = T.make_requests(cfg["vocab"], [310, 305], seed=77)
    want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    steps = T.tail_one_by_one(reqs, tail=300)
    runner = make_runner(folder, dtype, 16, T.peak_tokens(steps), max_requests=1,
                         poison_free_pages=True)
    with torch.no_grad():
        got = T.run_in_process(runner, steps)
    assert runner.replayed_steps > 500
    compare(got, want, dtype)


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_scheduler(name, models):
    """LLM.generate (scheduler, portions, decode steps replayed as graphs, sampling kernel)
    gives the plain model's greedy continuation."""
    from scratch_llm_b200 import LLM, SamplingParams
    cfg, tensors, folder, reqs, _ = models[name]
    prompts = [toks for toks in reqs.values() if len(toks) >= 2][:5]
    n_new = 12

    def plain_greedy(prompt):
        toks = list(prompt)
        for _ in range(n_new):
            toks.append(int(P.forward(cfg, tensors, toks)[-1].argmax()))
        return toks[len(prompt):]

    llm = LLM(str(folder), dtype="float32", max_tokens=1024, page_size=PAGE[name], max_requests=3,
              max_batch_tokens=64, chunk_size=24)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new))
    assert got == [plain_greedy(p) for p in prompts]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(dtype, models, tmp_path):
    cfg, _, folder, reqs, want = models["P"]
    steps = T.mixed(reqs, seed=3)
    for s in steps[::3]:                      # some steps want nothing, some only a few places
        for e in s["entries"]:
            e["want"] = []
    for s in steps[1::3]:
        for e in s["entries"]:
            e["want"] = e["want"][-1:]
    got = T.run_program(folder, dtype, steps, tmp_path / "out", T.peak_tokens(steps), cfg["vocab"])
    compare(got, want, dtype)
