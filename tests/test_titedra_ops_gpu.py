"""Each mechanism of the Titedra architecture alone: the engine's kernel or part against the
plain function of tests/plain/titedra_plain.py, in 32-bit and (where rounding allows a sharp
bound) in bfloat16.  Inputs are made so that a fault shows: a query is built to meet ONE far
token's latent, whose value differs from its own, so that a lost key changes the output by
its whole size; every choice score of a router is pushed below zero; a neighbour request
shares the steps."""

import math

import pytest
import torch

from plain import titedra_plain as P
from test_vobosun_ops_gpu import DEV, bf16_exact, feed, i32, ops

pytestmark = pytest.mark.gpu


def ctx(dtype):
    from scratch_llm_b200.parts import BuildContext
    return BuildContext(dtype=dtype, device=torch.device(DEV))


# ------------------------------------------------------------------------------------ norms

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [10, 33, 256])
def test_norms_around_a_branch_with_gains_stored_around_zero(dtype, width):
    """x + norm_b(branch(norm_a(x))): the norm before a branch and the one on its output, both
    with the gain 1 + w."""
    from scratch_llm_b200.parts.norm import RMSNorm
    g = torch.Generator().manual_seed(width)
    n, eps = 9, 1e-3
    x = torch.randn((n, width), generator=g) * 3
    y = (torch.randn((n, width), generator=g) * 5).to(dtype)
    wa, wb = (bf16_exact(torch.randn((width,), generator=g) * 0.3) for _ in range(2))
    before, after = RMSNorm(width, eps, "", offset=1.0), RMSNorm(width, eps, "", offset=1.0)
    before.load({"": wa.clone()}, ctx(dtype))
    after.load({"": wb.clone()}, ctx(dtype))
    resid = x.clone().to(DEV)
    got = before.forward(resid, None).float().cpu()
    want = P.norm_around_zero(x.double(), wa.double(), eps).float()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)
    after.add_normed(resid, y.to(DEV))
    want = (x.double() + P.norm_around_zero(y.double(), wb.double(), eps)).float()
    torch.testing.assert_close(resid.cpu(), want, rtol=1e-5, atol=1e-5)   # the stream is 32-bit
    # the norm on a branch's output and the norm in front of the next branch in one launch
    r3 = x.clone().to(DEV)
    assert after.chains_with(before) and not after.chains_with(RMSNorm(width + 1, eps, ""))
    h = after.add_normed(r3, y.to(DEV), then=before)
    assert torch.equal(r3, resid)
    torch.testing.assert_close(h.float().cpu(), P.norm_around_zero(want.double(), wa.double(),
                                                                   eps).float(), rtol=tol, atol=tol)
    # a gain of exactly -1 stored: the branch adds nothing
    zero = RMSNorm(width, eps, "", offset=1.0)
    zero.load({"": torch.full((width,), -1.0)}, ctx(dtype))
    r2 = x.clone().to(DEV)
    zero.add_normed(r2, y.to(DEV))
    assert torch.equal(r2.cpu(), x)


# -------------------------------------------------------------- the latent attention's steps

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Rq, R, r, rot, page, extra, d", [
    (20, 24, 8, 8, 4, 3, 5), (16, 21, 6, 4, 8, 3, 5), (8, 36, 28, 28, 16, 3, 5),
    (64, 96, 32, 32, 16, 3, 5), (5, 3, 2, 2, 4, 3, 5),
    # rows that move 16 bytes at a time: every size a multiple of 8, a query latent of more
    # than one vector a thread, a rotated part with an unrotated rest and zeros behind it
    (64, 96, 32, 32, 16, 0, 8), (2304, 48, 16, 16, 8, 8, 16), (24, 32, 24, 16, 4, 0, 8)])
def test_latents_are_normed_rotated_and_stored_as_one_vector(Rq, R, r, rot, page, extra, d,
                                                             dtype):
    """The kernel behind the down projections: the query latent's norm, the cached vector
    [normed latent | rotated shared key part | zeros] at the token's page place; tokens of
    padding rows store nothing.  ``extra``: gate columns behind, a wider buffer."""
    from scratch_llm_b200.parts.position import Rotary
    g = torch.Generator().manual_seed(R)
    base, eps, n = 300.0, 1e-4, 6
    pos = Rotary(r + r % 2, base, 64, interleaved=False, rot_dims=rot)
    pos.load({}, ctx(torch.float32))
    assert pos.cos.shape == (64, rot // 2)
    Dp = -(-(R + r) // 16) * 16
    a = (torch.randn((n, Rq + R + r + extra), generator=g) * 2).to(dtype)
    gq, gkv = torch.randn((Rq,), generator=g), torch.randn((R,), generator=g)
    positions = [0, 1, 2, 3, 41, 7]
    rows = [0, 0, 0, 0, 0, -1]                       # the last token belongs to no request
    pages = torch.full((12, 1, 1, page, Dp), float("nan"), device=DEV, dtype=dtype)
    table = i32([[7, 2, 9, 1, 0, 3, 4, 5, 6, 8, 10]])
    cq = torch.empty((n, Rq), dtype=dtype, device=DEV)
    ops().latent_prep(a.to(DEV), Rq, Rq, R, r, gq.to(DEV), gkv.to(DEV), eps, i32(positions),
                      i32(rows), pos.cos, pos.sin, cq, pages, table, page, True)
    ad = a.double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(cq.float().cpu(), (P.rms_unit(ad[:, :Rq], eps) * gq.double()).float(),
                               rtol=tol, atol=tol)
    c = P.rms_unit(ad[:, Rq:Rq + R], eps) * gkv.double()
    kr = P.rotate_split_half(ad[:, Rq + R:Rq + R + r], torch.tensor(positions), rot, base)
    for t, p in enumerate(positions[:-1]):
        slot = pages[int(table[0, p // page]), 0, 0, p % page].float().cpu()
        torch.testing.assert_close(slot[:R], c[t].float(), rtol=tol, atol=tol)
        torch.testing.assert_close(slot[R:R + r], kr[t].float(), rtol=tol, atol=tol)
        assert torch.equal(slot[R + r:], torch.zeros(Dp - R - r))
    p = positions[-1]
    assert pages[int(table[0, p // page]), 0, 0, p % page].isnan().all()
    # the queries' rotated parts land behind the absorbed part of each head
    H = 3
    q = (torch.randn((n, H * (d + r)), generator=g)).to(dtype)
    out = torch.full((n, H * Dp), float("nan"), dtype=dtype, device=DEV)
    ops().latent_q_rot(q.to(DEV), H, d, r, i32(positions), pos.cos, pos.sin, out, R)
    qr = P.rotate_split_half(q.double().view(n, H, d + r)[..., d:], torch.tensor(positions), rot,
                             base)
    got = out.view(n, H, Dp).float().cpu()
    torch.testing.assert_close(got[..., R:R + r], qr.float(), rtol=tol, atol=tol)
    assert torch.equal(got[..., R + r:], torch.zeros(n, H, Dp - R - r))
    assert got[..., :R].isnan().all()                # the absorbed part is somebody else's


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_and_gates_per_head(dtype):
    g = torch.Generator().manual_seed(8)
    n, H, K, J = 45, 3, 21, 37
    x = bf16_exact(torch.randn((n, H * (K + 4)), generator=g))
    w = bf16_exact(torch.randn((H, J, K), generator=g) * K ** -0.5)
    out = torch.zeros((n, H * (J + 2)), dtype=dtype, device=DEV)
    ops().head_product(x.to(DEV, dtype), K + 4, w.to(DEV, dtype), out, J + 2)
    want = torch.einsum("nhk,hjk->nhj", x.view(n, H, K + 4)[..., :K].double(), w.double())
    got = out.view(n, H, J + 2).float().cpu()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got[..., :J], want.float(), rtol=tol, atol=tol)
    assert torch.equal(got[..., J:], torch.zeros(n, H, 2))
    # a token alone gets what it got in the batch, bit for bit
    alone = torch.zeros((1, H * (J + 2)), dtype=dtype, device=DEV)
    ops().head_product(x[17:18].to(DEV, dtype), K + 4, w.to(DEV, dtype), alone, J + 2)
    assert torch.equal(alone[0], out[17])
    # one gate per head, read from a slice of a wider buffer (16: rows that move 16 bytes at a
    # time)
    for V in (10, 16):
        o = torch.randn((n, H * V), generator=g).to(dtype)
        wide = torch.randn((n, 7 + H), generator=g).to(dtype)
        got = ops().head_gate(o.clone().to(DEV), wide.to(DEV)[:, 7:], H).float().cpu()
        want = o.double().view(n, H, V) * torch.sigmoid(wide[:, 7:].double())[..., None]
        torch.testing.assert_close(got, want.reshape(n, H * V).float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, H, K, J", [(8, 3, 16, 192), (13, 2, 192, 64), (1, 5, 21, 10),
                                        (64, 1, 7, 300), (5, 4, 100, 96)])
def test_products_per_head_of_steps_of_few_tokens(n, H, K, J, dtype):
    """The kernel that steps of few tokens use instead of a batched product: alone, with the
    gate, and with the rotated tail behind its outputs."""
    from scratch_llm_b200.parts.position import Rotary
    g = torch.Generator().manual_seed(n * K + J)
    r, pad, base = 6, 3, 90.0
    x = bf16_exact(torch.randn((n, H * (K + r)), generator=g))
    w = bf16_exact(torch.randn((H, K, J), generator=g) * K ** -0.5)
    gate = bf16_exact(torch.randn((n, 4 + H), generator=g))
    want = torch.einsum("nhk,hkj->nhj", x.view(n, H, K + r)[..., :K].double(), w.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    xd, wdev = x.to(DEV, dtype), w.to(DEV, dtype)
    assert ops().latent_small_supports(K, J)
    out = torch.full((n, H * J), float("nan"), dtype=dtype, device=DEV)
    ops().latent_small(xd, K + r, wdev, out, J)
    torch.testing.assert_close(out.view(n, H, J).float().cpu(), want.float(), rtol=tol, atol=tol)
    gated = torch.full((n, H * J), float("nan"), dtype=dtype, device=DEV)
    ops().latent_small(xd, K + r, wdev, gated, J, gate=gate.to(DEV, dtype)[:, 4:])
    torch.testing.assert_close(
        gated.view(n, H, J).float().cpu(),
        (want * torch.sigmoid(gate[:, 4:].double())[..., None]).float(), rtol=tol, atol=tol)
    pos = Rotary(r, base, 64, interleaved=False, rot_dims=4)
    pos.load({}, ctx(torch.float32))
    positions = [(7 * i) % 60 for i in range(n)]
    tailed = torch.full((n, H * (J + r + pad)), float("nan"), dtype=dtype, device=DEV)
    ops().latent_small(xd, K + r, wdev, tailed, J + r + pad, rot=(r, i32(positions), pos.cos,
                                                                  pos.sin))
    got = tailed.view(n, H, J + r + pad).float().cpu()
    assert torch.equal(got[..., :J], out.view(n, H, J).float().cpu())
    turned = P.rotate_split_half(x.double().view(n, H, K + r)[..., K:], torch.tensor(positions), 4,
                                 base)
    torch.testing.assert_close(got[..., J:J + r], turned.float(), rtol=tol, atol=tol)
    assert torch.equal(got[..., J + r:], torch.zeros(n, H, pad))
    # a token alone gets what it got in the batch, bit for bit
    alone = torch.empty((1, H * J), dtype=dtype, device=DEV)
    ops().latent_small(xd[n - 1:], K + r, wdev, alone, J)
    assert torch.equal(alone[0], out[n - 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [40, 37])      # rows that move 16 bytes at a time, and not
def test_stream_joins_the_embedding_output(d, dtype):
    from scratch_llm_b200.parts.stream_join import ConcatLinear
    g = torch.Generator().manual_seed(2)
    n = 13
    x, first = torch.randn((n, d), generator=g), torch.randn((n, d), generator=g) * 4
    w = bf16_exact(torch.randn((d, 2 * d), generator=g) * (2 * d) ** -0.5)
    join = ConcatLinear(d, "")
    join.load({"": w}, ctx(dtype))
    got = join.forward(x.to(DEV), first.to(DEV))
    assert got.dtype == torch.float32
    want = (torch.cat([x, first], 1).double() @ w.double().T).float()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(got.cpu(), want, rtol=tol, atol=tol)
    # the stream's half comes first
    w2 = torch.cat([torch.eye(d), torch.zeros(d, d)], 1)
    join.load({"": w2}, ctx(torch.float32))
    assert torch.equal(join.forward(x.to(DEV), first.to(DEV)).cpu(), x)


# -------------------------------------------------------------------------- latent attention

def seeking_case(H, d, r, dv, Rq, R, width, T, pairs, seed, base=5000.0, boost=8.0):
    """Weights and inputs of one latent attention in which token i of every pair (i, j) looks
    for token j.  The shared key part is not normed, so x_j times ``boost`` gives j a long one
    (its latent, and so its value, keeps its size); every head's rotated query rows are one
    matrix M, and x_i is solved so that M c_q(i) is j's shared key part turned by the angle of
    j - i: after both are rotated by their positions they are parallel, and the score is the
    product of their lengths, which no other key can reach.  i's own latent has nothing to do
    with j's, so its output is j's value only if it finds j."""
    assert width >= Rq >= r and r % 2 == 0
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape, std=1.0: bf16_exact(torch.randn(shape, generator=g) * std)  # noqa: E731
    w = {"dq": rnd(Rq, width, std=width ** -0.5), "dq.norm": rnd(Rq, std=0.1) + 1.0,
         "dkv": rnd(R + r, width, std=width ** -0.5), "dkv.norm": rnd(R, std=0.1) + 1.0,
         "uk": rnd(H * d, R, std=R ** -0.5), "uv": rnd(H * dv, R, std=R ** -0.5),
         "g": rnd(H, width, std=2 * width ** -0.5), "o": rnd(width, H * dv, std=(H * dv) ** -0.5)}
    rows = rnd(r, Rq, std=Rq ** -0.5).double()                                   # M
    x = rnd(T, width)
    assert not {i for i, _ in pairs} & {j for _, j in pairs}
    for _, j in pairs:
        x[j] *= boost
    solve, back = torch.linalg.pinv(w["dq"].double()), torch.linalg.pinv(rows)
    dkv, gq = w["dkv"].double(), w["dq.norm"].double()
    raw = []
    for i, j in pairs:
        key = dkv[R:] @ x[j].double()
        turned = P.rotate_split_half(key[None], torch.tensor([j - i]), r, base)[0]
        t = solve @ ((back @ turned) / gq)
        x[i] = bf16_exact((t / t.pow(2).mean().sqrt()).float())
        cq = P.rms_unit(w["dq"].double() @ x[i].double(), 1e-5) * gq
        raw.append(float(P.rotate_split_half((rows @ cq)[None], torch.tensor([i]), r, base)[0]
                         @ P.rotate_split_half(key[None], torch.tensor([j]), r, base)[0]))
    scale = 30.0 / min(raw)                 # every sought key scores 30 or more, in every head
    uq = torch.zeros((H, d + r, Rq), dtype=torch.float64)
    # (unrotated products of a few units)
    uq[:, :d] = torch.randn((H, d, Rq), generator=g, dtype=torch.float64) \
        * 2.0 / (scale * math.sqrt(Rq * d))
    uq[:, d:] = rows
    w["uq"] = bf16_exact(uq.reshape(H * (d + r), Rq).float())
    m = {"heads": H, "dim": d, "rot_dim": r, "vdim": dv, "q_rank": Rq, "kv_rank": R,
         "scale": scale, "rot": {"base": base, "dims": r}}
    return m, w, x


def latent_part(m, width, w, eps, dtype, max_position=4096):
    from scratch_llm_b200.parts.latent_attention import LatentAttention
    from scratch_llm_b200.parts.position import Rotary
    mixer = LatentAttention(width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"],
                            m["kv_rank"], m["scale"], eps)
    mixer.load(w, ctx(dtype))
    pos = Rotary(m["rot_dim"] + m["rot_dim"] % 2, m["rot"]["base"], max_position,
                 interleaved=False, rot_dims=m["rot"]["dims"])
    pos.load({}, ctx(dtype))
    return mixer, pos


LATENT = [  # heads, dim, rot_dim, vdim, q_rank, kv_rank, width, page
    (4, 16, 16, 24, 48, 48, 64, 16),       # a cached vector of 64 entries
    (3, 8, 8, 10, 40, 20, 48, 8),          # of 28, kept as 32
    (2, 20, 10, 12, 64, 48, 72, 16),       # of 58, kept as 64; a value size below the key's
    (16, 32, 32, 32, 96, 96, 128, 16),     # of 128, many heads on one cached vector
    (20, 16, 16, 24, 64, 48, 96, 16),      # of 64, more heads than one tile of queries holds
    (1, 8, 28, 16, 36, 36, 40, 32),        # one head, a rotated part larger than the rest
    (2, 16, 32, 40, 48, 256, 64, 64)]      # of 288: beyond the tensor-core kernels' sizes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, r, dv, Rq, R, width, page", LATENT)
@pytest.mark.parametrize("cut", ["whole", "decode", "portions"])
def test_latent_attention_sees_far_keys_and_page_borders(cut, H, d, r, dv, Rq, R, width, page,
                                                         dtype):
    """Queries near the end look for one token each: the first of the sequence, the second, a
    page's last place and the next page's first, one in the middle, and their own neighbour."""
    T, eps = 330, 1e-5
    pairs = [(T - 1, 1), (T - 2, page - 1), (T - 3, page), (T - 4, 5 * page + 1), (T - 5, 0),
             (T - 6, T - 7)]
    m, w, x = seeking_case(H, d, r, dv, Rq, R, width, T, pairs, seed=H * d + r)
    wd = {k: v.double() for k, v in w.items()}
    want = P.latent_attention(x.double(), wd, m, eps).float()
    if cut == "whole" and dtype == torch.float32:
        # the construction holds: without the sought token the seeker's output is another one
        x2 = x.clone()
        x2[1] = bf16_exact(torch.randn((width,), generator=torch.Generator().manual_seed(1)))
        other = P.latent_attention(x2.double(), wd, m, eps).float()
        assert (other[T - 1] - want[T - 1]).norm() > 0.5 * want[T - 1].norm()
    mixer, pos = latent_part(m, width, w, eps, dtype)
    portions = {"whole": [T], "decode": [T - 8] + [1] * 8,
                "portions": [7, 2, 100, 1, 33, 2, 152, 3, 20, 2, 1, 1, 2, 1, 1, 1, 1]}[cut]
    other = {"portions": [3, 1, 40, 2, 1, 1, 9]}.get(cut)
    assert sum(portions) == T
    xb = bf16_exact(torch.randn((60, width), generator=torch.Generator().manual_seed(3)))
    seen = []

    def run(batch, view, t0, t1, off):
        rows = torch.cat([xb[sum(seen):][:off], x[t0:t1]], 0) if off else x[t0:t1]
        seen.append(off)
        return mixer.forward(rows.to(DEV, dtype), batch, view, True, pos)[off:].float().cpu()

    got = feed([mixer.kv_spec()], [None], dtype, page, portions, run, other=other)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    else:
        # (scores of 30 carry bfloat16 errors of a tenth: where two long keys compete for an
        # ordinary query, and one head averages nothing, a row moves by that much; the seekers
        # have a margin, and 32-bit above is sharp for every row)
        err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert err.median() < 0.02 and err.max() < 0.25, (err.median(), err.max())
        assert err[[i for i, _ in pairs]].max() < 0.06


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_alone_and_beside_others_is_the_same(dtype):
    """What a request gets does not depend on its neighbours in the step nor on how it was cut."""
    T, eps, page = 90, 1e-5, 8
    m, w, x = seeking_case(3, 8, 8, 12, 32, 24, 48, T, [(T - 1, 2), (T - 2, page)], seed=4)
    mixer, pos = latent_part(m, 48, w, eps, dtype)
    xb = bf16_exact(torch.randn((60, 48), generator=torch.Generator().manual_seed(3)))

    def once(portions, other):
        seen = []

        def run(batch, view, t0, t1, off):
            rows = torch.cat([xb[sum(seen):][:off], x[t0:t1]], 0) if off else x[t0:t1]
            seen.append(off)
            return mixer.forward(rows.to(DEV, dtype), batch, view, True, pos)[off:].float().cpu()
        return feed([mixer.kv_spec()], [None], dtype, page, portions, run, other=other)

    whole = once([T], None)
    cut = once([50, 2, 30] + [1] * 8, [5, 1, 20, 1, 1, 1])
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(cut, whole, rtol=tol, atol=tol)


def test_latent_attention_without_a_gate_and_with_part_of_the_key_part_rotated():
    """Constructor arguments beyond what the Titedra reader passes: no output gate, a rotation
    over fewer entries than the shared key part has."""
    from scratch_llm_b200.parts.latent_attention import LatentAttention
    from scratch_llm_b200.parts.position import Rotary
    T, eps, width = 40, 1e-5, 48
    m, w, x = seeking_case(3, 8, 12, 10, 32, 24, width, T, [(T - 1, 3)], seed=6)
    m["rot"]["dims"] = 8
    wd = {k: v.double() for k, v in w.items()}
    wd["g"] = torch.zeros_like(wd["g"])                     # sigmoid(0) = 1/2 in the plain model
    want = 2.0 * P.latent_attention(x.double(), wd, m, eps).float()
    mixer = LatentAttention(width, 3, 8, 12, 10, 32, 24, m["scale"], eps, gate=False)
    assert "g" not in mixer.param_specs()
    mixer.load({k: v for k, v in w.items() if k != "g"}, ctx(torch.float32))
    pos = Rotary(12, m["rot"]["base"], 128, interleaved=False, rot_dims=8)
    pos.load({}, ctx(torch.float32))

    def run(batch, view, t0, t1, off):
        return mixer.forward(x[t0:t1].to(DEV), batch, view, True, pos).float().cpu()

    got = feed([mixer.kv_spec()], [None], torch.float32, 8, [30, 2] + [1] * 8, run)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


# ------------------------------------------------------------------------- routed experts

ROUTERS = [  # experts, top, groups (count, keep), expert size
    (6, 2, (3, 2), 40), (10, 4, (2, 1), 24), (5, 5, None, 33), (8, 3, (2, 2), 16),
    (4, 1, (4, 2), 32), (9, 3, (3, 1), 64), (64, 6, (8, 3), 8), (1, 1, None, 20)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, groups, ff", ROUTERS)
def test_sigmoid_router_with_squared_relu_experts(experts, top, groups, ff, dtype):
    routed_case(experts, top, groups, ff, dtype, width=40, n=150)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_with_many_tokens_per_expert(dtype):
    """Experts with several hundred tokens each and sizes beyond one tile of the grouped
    products in both directions."""
    routed_case(4, 2, (2, 1), 200, dtype, width=320, n=700)


def routed_case(experts, top, groups, ff, dtype, width, n):
    from scratch_llm_b200.parts.routed import RoutedExperts
    g = torch.Generator().manual_seed(experts * 10 + top)
    rnd = lambda *shape, std=1.0: bf16_exact(torch.randn(shape, generator=g) * std)  # noqa: E731
    # corrections around -0.6 beside scores in (0, 1): most choice scores are below zero, where
    # a barred expert that counted as 0 would win, and some above
    w = {"router": rnd(experts, width, std=2 * width ** -0.5),
         "correction": rnd(experts, std=0.3) - 0.6}
    for e in range(experts):
        w[f"e{e}.up"] = rnd(ff, width, std=width ** -0.5)
        w[f"e{e}.down"] = rnd(width, ff, std=ff ** -0.5)
    x = rnd(n, width)
    mlp = {"router": {"experts": experts, "top": top}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    wd = {k: v.double() for k, v in w.items()}
    want = P.moe_ff(x.double(), wd, mlp).float()
    part = RoutedExperts(width, ff, experts, top, 0, *(groups or (1, 1)), None, score="sigmoid",
                         group_score="top2", renormalize=False, expert="sqrelu")
    part.load(w, ctx(dtype))
    assert "e0.gate" not in part.param_specs()
    got = part.forward(x.to(DEV, dtype)).float().cpu()
    # the choice itself, in 32-bit from the same logits: the experts in the order they are
    # taken, and their plain scores as weights (the correction only chooses; no division)
    chosen, weights = P.route(x.double(), wd, mlp["router"])
    flags = ops().MOE_SIGMOID | ops().MOE_GROUP_TOP2 | ops().MOE_RAW_WEIGHTS
    logits = (x.double() @ wd["router"].T).float()
    ids, wts = ops().moe_route(logits.to(DEV), w["correction"].to(DEV), None, experts,
                               *(groups or (1, 1)), top, flags=flags)[:2]
    assert ids.cpu().tolist() == chosen
    torch.testing.assert_close(wts.cpu().double(), torch.stack(weights), rtol=1e-5, atol=1e-7)
    assert float(torch.stack(weights).sum(-1).sub(1).abs().mean()) > 0.05     # not renormalised
    # steps of few tokens take the router that does everything in one launch
    few = slice(40, 40 + max(1, 48 // top))
    ids_few, wts_few = ops().moe_route(logits[few].to(DEV), w["correction"].to(DEV), None,
                                       experts, *(groups or (1, 1)), top, flags=flags)[:2]
    assert ids_few.cpu().tolist() == chosen[few]
    torch.testing.assert_close(wts_few.cpu().double(), torch.stack(weights[few]), rtol=1e-5,
                               atol=1e-7)
    got_few = part.forward(x[few].to(DEV, dtype)).float().cpu()
    if dtype == torch.float32:
        assert torch.equal(got_few, got[few])
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
        alone = part.forward(x[17:18].to(DEV, dtype)).float().cpu()
        assert torch.equal(alone[0], got[17])
    else:
        torch.testing.assert_close(got_few, got[few], rtol=2e-2, atol=2e-2)
        err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert err.median() < 0.02 and err.quantile(0.9) < 0.05


def test_groups_are_scored_by_their_two_best_and_barred_experts_lose_to_negative_scores():
    """The router kernel on the hand-made case of the plain model's own test: the group with
    the best single expert loses to the group with the best pair; with every choice score
    below zero a barred expert must not come back as a 0."""
    corr = torch.tensor([-2.0, -2.0, -1.2, -3.0, -1.9, -1.9])
    z = torch.tensor([[0.0, 0.0, 4.0, -4.0, 0.5, 0.5], [3.0, 3.0, 9.0, -9.0, -1.0, 2.0]])
    wd = {"router": torch.eye(6, dtype=torch.float64), "correction": corr.double()}
    flags = ops().MOE_SIGMOID | ops().MOE_GROUP_TOP2 | ops().MOE_RAW_WEIGHTS
    for keep, first in ((1, [4, 5]), (3, [2, 4])):
        r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": keep}}
        chosen, weights = P.route(z.double(), wd, r)
        assert chosen[0] == first
        ids, wts = ops().moe_route(z.to(DEV), corr.to(DEV), None, 6, 3, keep, 2, flags=flags)[:2]
        assert ids.cpu().tolist() == chosen
        torch.testing.assert_close(wts.cpu().double(), torch.stack(weights), rtol=1e-6, atol=1e-7)
    # the same logits with the largest-member group score: the other group wins
    ids, _ = ops().moe_route(z.to(DEV), corr.to(DEV), None, 6, 3, 1, 2,
                             flags=ops().MOE_SIGMOID | ops().MOE_RAW_WEIGHTS)[:2]
    assert sorted(ids.cpu().tolist()[0]) == [2, 3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward(dtype):
    from scratch_llm_b200.parts.feed_forward import SwiGLU
    g = torch.Generator().manual_seed(4)
    width, ff, n = 24, 50, 11
    w = {"gate": bf16_exact(torch.randn((ff, width), generator=g) * width ** -0.5),
         "up": bf16_exact(torch.randn((ff, width), generator=g) * width ** -0.5),
         "down": bf16_exact(torch.randn((width, ff), generator=g) * ff ** -0.5)}
    x = bf16_exact(torch.randn((n, width), generator=g) * 2)
    want = P.dense_ff(x.double(), {k: v.double() for k, v in w.items()}).float()
    part = SwiGLU(width, ff, names={"gate": "gate", "up": "up", "down": "down"})
    part.load(w, ctx(dtype))
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(part.forward(x.to(DEV, dtype)).float().cpu(), want, rtol=tol,
                               atol=tol)
