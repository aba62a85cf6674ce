"""Each mechanism of the Tubevik architecture alone: the engine's kernel against the plain
function of tests/plain/tubevik_plain.py, in 32-bit and (where rounding allows a sharp bound)
in bfloat16.  Inputs are made so that a fault shows: a key just inside and just outside a window
or a chunk gets a score that stands out, as does one key far back among hundreds; the sink's
share is large; decays are strong enough that a forgotten one changes everything; a row's state
is carried over portions of two tokens and its slot is used again."""

import math

import pytest
import torch

from plain import tubevik_plain as P
from test_nilevik_ops_gpu import fill_pages, i32

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from scratch_llm_b200.kernels import ops as o
    return o


def rnd(g, shape, std=1.0, dtype=torch.float32):
    return (torch.randn(shape, generator=g) * std).to(dtype).float()


# -------------------------------------------------------------------------------- layer norm

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [10, 33, 256, 1000])
def test_layer_norm_with_pending_terms(dtype, d):
    g = torch.Generator().manual_seed(d)
    n, eps = 6, 1e-3
    resid = rnd(g, (n, d), 2.0) + 3.0            # a mean far from zero
    terms = [(rnd(g, (n, d), 1.5, dtype), c) for c in (0.5, -1.25, 2.0)]
    w, b = rnd(g, (d,)) + 1.0, rnd(g, (d,))
    x = resid.double() + sum(c * t.double() for t, c in terms)
    want = P.layer_norm(x, w.double(), b.double(), eps)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    r = resid.clone().to(DEV)
    out = torch.empty((n, d), dtype=dtype, device=DEV)
    ops().add_layernorm(r, [(t.to(DEV, dtype), c) for t, c in terms], w.to(DEV), b.to(DEV), eps, out)
    torch.testing.assert_close(out.float().cpu(), want.float(), **tol)
    torch.testing.assert_close(r.cpu(), x.float(), rtol=1e-6, atol=1e-6)     # the stream got the sum
    # only some rows, the stream untouched
    r2 = resid.clone().to(DEV)
    rows = [4, 0, 3]
    out2 = torch.empty((3, d), dtype=dtype, device=DEV)
    ops().add_layernorm(r2, [(t.to(DEV, dtype), c) for t, c in terms[:1]], w.to(DEV), b.to(DEV),
                        eps, out2, i32(rows))
    x1 = resid.double() + terms[0][1] * terms[0][0].double()
    torch.testing.assert_close(out2.float().cpu(),
                               P.layer_norm(x1, w.double(), b.double(), eps)[rows].float(), **tol)
    assert torch.equal(r2.cpu(), resid)
    # the stream normed in place, in 32-bit
    r3 = resid.clone().to(DEV)
    ops().add_layernorm(r3, [], w.to(DEV), b.to(DEV), eps, r3)
    torch.testing.assert_close(r3.cpu(), P.layer_norm(resid.double(), w.double(), b.double(),
                                                      eps).float(), rtol=1e-5, atol=1e-5)


def test_clamped_gate_and_low_rank_products():
    g = torch.Generator().manual_seed(2)
    gu = rnd(g, (6, 2 * 37), 3.0)
    wide = torch.zeros((6, 50), device=DEV)
    for limit in (0.7, 7.0):
        ops().clamped_gate(gu.to(DEV), wide[:, 5:42], limit, 1.702)
        gate = torch.clamp(gu[:, :37], max=limit)
        up = torch.clamp(gu[:, 37:], -limit, limit)
        want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
        torch.testing.assert_close(wide[:, 5:42].cpu(), want, rtol=1e-5, atol=1e-6)
    assert float(wide[:, :5].abs().max()) == 0.0 and float(wide[:, 42:].abs().max()) == 0.0
    # the second product of a low-rank pair, plain and as the logarithm of a decay per channel
    n, r, heads, per = 11, 7, 3, 5
    pre = rnd(g, (n, 4 + r + 2))
    w2 = rnd(g, (heads * per, r))
    bias, rate = rnd(g, (heads * per,)), rnd(g, (heads,), 0.7) - 1.0
    z = pre[:, 4:4 + r].double() @ w2.double().T
    out = torch.empty((n, heads * per), device=DEV)
    ops().lowrank_expand(pre.to(DEV), 4, w2.t().contiguous().to(DEV), out)
    torch.testing.assert_close(out.cpu(), z.float(), rtol=1e-5, atol=1e-5)
    ops().lowrank_expand(pre.to(DEV), 4, w2.t().contiguous().to(DEV), out, bias=bias.to(DEV),
                         rate_log=rate.to(DEV), per_rate=per)
    want = -torch.exp(rate.double()).repeat_interleave(per) * P.softplus(z + bias.double())
    torch.testing.assert_close(out.cpu(), want.float(), rtol=1e-5, atol=1e-5)
    half = torch.empty((n, heads * per), dtype=torch.bfloat16, device=DEV)
    ops().lowrank_expand(pre.to(DEV), 4, w2.t().contiguous().to(DEV), half)
    torch.testing.assert_close(half.float().cpu(), z.float(), rtol=1e-2, atol=1e-2)
    # two products of the same hidden values' buffer in one launch, of other ranks and widths
    w3 = rnd(g, (9, 3))
    out.zero_()
    second = torch.empty((n, 9), dtype=torch.bfloat16, device=DEV)
    ops().lowrank_expand(pre.to(DEV), 4, w2.t().contiguous().to(DEV), out, bias=bias.to(DEV),
                         rate_log=rate.to(DEV), per_rate=per,
                         also=(1, w3.t().contiguous().to(DEV), second))
    torch.testing.assert_close(out.cpu(), want.float(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(second.float().cpu(), (pre[:, 1:4].double() @ w3.double().T).float(),
                               rtol=1e-2, atol=1e-2)


# --------------------------------------------------- norms and rotation in front of attention

def rotary_tables(dims, base, layout, positions, scaling=None):
    from scratch_llm_b200.parts.position import Rotary
    rot = Rotary(dims, base, positions, interleaved=layout == "pairs", rot_dims=dims,
                 yarn=None if scaling is None else dict(zip(("factor", "original", "fast", "slow"),
                                                            scaling)))
    cos, sin = rot.tables()
    return cos.to(DEV).contiguous(), sin.to(DEV).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["wide_halves", "unit_pairs", "borrowed"])
def test_norms_and_rotation_before_attention(mode, dtype):
    """A head size of 12 padded to 16 (the norms divide by 12), a rotation of the first 8
    entries, tokens at positions up to 700 of two rows, pages in a shuffled order."""
    g = torch.Generator().manual_seed(5)
    H, G, dim, hd, rot_dims, page_size, eps = 3, 1, 12, 16, 8, 8, 1e-4
    has_kv = mode != "borrowed"
    positions = [0, 1, 2, 699, 700]
    rows = [0, 0, 0, 1, 1]
    n = len(positions)
    scaling = (3.0, 64, 8.0, 0.5) if mode != "unit_pairs" else None
    layout = "pairs" if mode == "unit_pairs" else "halves"
    rot = {"base": 300.0, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    cols = (H + (2 * G if has_kv else 0)) * hd
    x = torch.zeros((n, cols + 8))
    true = rnd(g, (n, H + 2 * G, dim), 1.0, dtype)
    x.view(n, -1)[:, :cols].view(n, -1, hd)[:, :, :dim] = true[:, :H + (2 * G if has_kv else 0)]
    x[:, cols:] = 7.0                                            # other columns: not touched
    bias = rnd(g, (H + 2 * G, dim), 0.3)
    q_gain, k_gain = rnd(g, (H, dim), 0.3) + 1.0, rnd(g, (G, dim), 0.3) + 1.0

    def padded(t):
        out = torch.zeros(t.shape[:-1] + (hd,))
        out[..., :dim] = t
        return out.reshape(-1).to(DEV)

    cos, sin = rotary_tables(rot_dims, rot["base"], layout, 701, scaling)
    n_pages = 200
    pages = torch.full((n_pages, 2, G, page_size, hd), float("nan"), dtype=dtype, device=DEV)
    table = torch.full((2, 100), -1, dtype=torch.int32, device=DEV)
    table[0, 0], table[1, 87] = 5, 9
    xd = x.to(DEV, dtype)
    wide = mode != "unit_pairs"
    ops().norm_rope_kv_write(
        xd, i32(positions), i32(rows), pages, table, page_size, H, G, hd, dim, eps,
        has_kv=has_kv, write=has_kv,
        bias=padded(bias[:H + (2 * G if has_kv else 0)]) if wide else None,
        q_gain=padded(q_gain) if wide else None, k_gain=padded(k_gain) if wide and has_kv else None,
        unit_after=not wide, cos=cos, sin=sin, interleaved=layout == "pairs")
    t64 = true.double()
    q, k, v = t64[:, :H], t64[:, H:H + G], t64[:, H + G:]
    if wide:
        q, k, v = q + bias[:H].double(), k + bias[H:H + G].double(), v + bias[H + G:].double()
        q = (P.rms_unit(q.reshape(n, -1), eps) * q_gain.reshape(-1).double()).view(n, H, dim)
        k = (P.rms_unit(k.reshape(n, -1), eps) * k_gain.reshape(-1).double()).view(n, G, dim)

    def turned(t):
        out = torch.empty_like(t)
        for a, p in enumerate(positions):
            full = torch.zeros((p + 1,) + tuple(t.shape[1:]), dtype=t.dtype)
            full[p] = t[a]
            out[a] = P.rotate(full, rot, layout)[p]
        return out

    q, k = turned(q), turned(k)
    if not wide:
        q, k = P.rms_unit(q, eps), P.rms_unit(k, eps)
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    got = xd.float().cpu()
    torch.testing.assert_close(got[:, :H * hd].view(n, H, hd)[:, :, :dim], q.float(), **tol)
    assert float(got[:, :H * hd].view(n, H, hd)[:, :, dim:].abs().max()) == 0.0
    assert torch.equal(got[:, cols:], torch.full((n, 8), 7.0))
    if not has_kv:
        assert torch.isnan(pages).all()
        return
    for a, (p, row) in enumerate(zip(positions, rows)):
        page, off = int(table[row, p // page_size]), p % page_size
        torch.testing.assert_close(pages[page, 0, :, off, :dim].float().cpu(), k[a].float(), **tol)
        torch.testing.assert_close(pages[page, 1, :, off, :dim].float().cpu(), v[a].float(), **tol)
    assert int((~torch.isnan(pages)).sum()) == n * 2 * G * hd      # nothing else was written


# ------------------------------------------------------------------------------- attention

def run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, n_splits=1, **kw):
    o = ops()
    n = q.shape[0]
    dtype = pages.dtype
    qd = q.reshape(n, H * hd).to(DEV, dtype).contiguous()
    out = torch.empty_like(qd)
    row_start, row_pos0 = i32([0, n]), i32([pos0])
    sinks = torch.zeros(H, device=DEV) if kw.pop("zero_sink", False) else None
    window = kw.pop("window", None)
    if kind == "simt":
        o.attention_simt(qd, pages, table, page_size, row_start, row_pos0, out, 1, n, H, G, hd,
                         scale, window, None, sinks, **kw)
    elif kind == "tc":
        o.attention_tc(qd, pages, table, page_size, row_start, row_pos0, out, i32([0]), 1, n, H, G,
                       hd, scale, window, None, sinks, biased=True, **kw)
        assert o.attention_tc_error(hd) == 0
    else:
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(o.attention_mma_scratch_floats(n, H, hd, n_splits),
                                  dtype=torch.float32, device=DEV)
        gate = kw.pop("gate", None)
        o.attention_mma(qd, pages, table, page_size, row_start, row_pos0, out, i32([0]), 1, n, H,
                        G, hd, scale, window, split=(kind == "split"), n_splits=n_splits,
                        scratch=scratch, sinks=sinks,
                        gate=None if gate is None else gate.to(DEV, dtype), **kw)
    return out.float().cpu().view(n, H, hd)


CASES = [  # kind, dtype, head size, new tokens, splits
    ("simt", torch.float32, 16, 70, 1), ("simt", torch.float32, 24, 1, 1),
    ("simt", torch.bfloat16, 40, 7, 1),
    ("wide", torch.bfloat16, 64, 70, 1), ("wide", torch.bfloat16, 32, 90, 1),
    ("wide", torch.bfloat16, 128, 2, 1),
    ("split", torch.bfloat16, 64, 1, 1), ("split", torch.bfloat16, 64, 1, 3),
    ("split", torch.bfloat16, 32, 1, 2), ("split", torch.bfloat16, 128, 1, 2),
    # tcgen05: query tiles of 64 tokens x 2 heads, a ragged second one
    ("tc", torch.bfloat16, 64, 64, 1), ("tc", torch.bfloat16, 64, 100, 1),
    ("tc", torch.bfloat16, 128, 130, 1),
]


@pytest.mark.parametrize("kind, dtype, hd, n_new, n_splits", CASES)
@pytest.mark.parametrize("mask", [("chunk", 37), ("chunk", 64), ("chunk", 1), ("chunk", 500),
                                  ("window", 37), ("window", 200)])
def test_attention_with_chunks_cap_and_zero_sink(kind, dtype, hd, n_new, n_splits, mask):
    """The last query's first visible key and the key just before it both get scores that stand
    out, as does one key far back: a mask that is one token off moves the output by much."""
    H, G, page_size, T = 4, 2, 16, 300
    g = torch.Generator().manual_seed(hd + n_new + mask[1])
    k = rnd(g, (T, G, hd), 1.0, dtype)
    v = rnd(g, (T, G, hd), 1.0, dtype)
    pos0 = T - n_new
    q = rnd(g, (n_new, H, hd), 1.0, dtype)
    what, size = mask
    last = T - 1
    first_seen = last // size * size if what == "chunk" else max(0, last - size + 1)
    unit = q[-1] / q[-1].norm(dim=-1, keepdim=True)
    for j in {first_seen, first_seen - 1, 3} - {-1}:
        for kv_head in range(G):            # aligned with the last query of the group's first head
            k[j, kv_head] = (unit[kv_head * (H // G)] * 6.0 * math.sqrt(hd)).to(dtype).float()
    pages, table = fill_pages(k, v, page_size, 24, G, hd, dtype)
    scale = 0.5 / math.sqrt(hd)
    visible = P.chunk_visible(size) if what == "chunk" else P.window_visible(size)
    kw = {"chunk": size} if what == "chunk" else {"window": size}
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for cap, sink in ((0.0, True), (2.5, False), (2.5, True)):
        full_q = torch.zeros((T, H, hd), dtype=torch.float64)
        full_q[pos0:] = q.double()
        want = P.attend(full_q, k.double(), v.double(), scale, visible, softcap=cap or None,
                        zero_sink=sink)[pos0:].float()
        got = run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, n_splits,
                            softcap=cap, zero_sink=sink, **kw)
        torch.testing.assert_close(got, want, **tol)
    if kind in ("wide", "split"):
        # one gate per token and head in the kernel's epilogue, and where the last CTA merges
        gate = rnd(g, (n_new, H), 2.0, dtype)
        for inside in (False, True):
            got = run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, n_splits,
                                softcap=2.5, zero_sink=True, gate=gate, merge_inside=inside, **kw)
            torch.testing.assert_close(got, want * torch.sigmoid(gate)[:, :, None], **tol)
    if first_seen == 0:
        return
    # one token more in the mask would show
    off_by_one = P.attend(full_q, k.double(), v.double(), scale,
                          lambda i, j: visible(i, j) or visible(i, j + 1),
                          softcap=2.5, zero_sink=True)[pos0:].float()
    assert (off_by_one[-1] - want[-1]).abs().max() > 0.03


# ------------------------------------------------------- the delta rule, a decay per channel

def delta_inputs(g, T, H, G, D, V, dtype):
    """Activations after the convolution (q heads, k heads, v heads), step inputs among other
    narrow columns, and log decays strong enough to matter (some channels forget within a few
    tokens, some keep nearly everything)."""
    act = rnd(g, (T, 2 * G * D + H * V), 1.0, dtype)
    narrow = rnd(g, (T, 3 + H + 2), 1.5)
    log_decay = -torch.exp(rnd(g, (T, H * D), 1.5) - 1.0)
    log_decay[:, ::7] *= 20.0
    return act, narrow, log_decay


def plain_delta(act, narrow, log_decay, H, G, D, V):
    T = act.shape[0]
    a = act.double()
    q = P.unit_vector(a[:, :G * D].view(T, G, D)) * D ** -0.5
    k = P.unit_vector(a[:, G * D:2 * G * D].view(T, G, D))
    v = a[:, 2 * G * D:].view(T, H, V)
    beta = P.sigmoid(narrow[:, 3:3 + H].double())
    decay = torch.exp(log_decay.double()).view(T, H, D)
    out = torch.zeros((T, H, V), dtype=torch.float64)
    for h in range(H):
        gq = h // (H // G)
        out[:, h] = P.delta_recurrence(q[:, gq], k[:, gq], v[:, h], beta[:, h], decay[:, h])
    return out.view(T, H * V)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, V", [(4, 2, 16, 10), (2, 2, 33, 5), (3, 1, 64, 64), (2, 1, 128, 24),
                                        (1, 1, 6, 3)])
def test_delta_rule_with_a_decay_per_channel(H, G, D, V, dtype):
    """Whole rows (chunks of 16 and a ragged tail), the same in portions of 2, 1 and 21 tokens,
    two rows side by side in slots that the first launch left dirty."""
    g = torch.Generator().manual_seed(D + V)
    T = 53
    rows = [delta_inputs(g, T, H, G, D, V, dtype) for _ in range(2)]
    want = [plain_delta(*r, H, G, D, V).float() for r in rows]
    state = torch.full((3, H, V, D), float("nan"), device=DEV)
    slots = [2, 0]
    tol = dict(rtol=2e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)

    def run(cuts, tables=False):
        state[slots] = 0.0
        got = [[], []]
        at = 0
        for size in cuts:
            part = [tuple(t[at:at + size] for t in r) for r in rows]
            act = torch.cat([p[0] for p in part]).to(DEV, dtype)
            narrow = torch.cat([p[1] for p in part]).to(DEV)
            logd = torch.cat([p[2] for p in part]).to(DEV)
            n = act.shape[0] // 2
            out = torch.empty((2 * n, H * V), device=DEV)
            ops().delta_rule(act, narrow, None, None, state, i32([0, n, 2 * n]), i32(slots), out,
                             2, H, G, D, V, max_new=1 if n == 1 else 0, log_decay=logd, b_col=3,
                             longest=n if tables else 0)
            got[0].append(out[:n].cpu())
            got[1].append(out[n:].cpu())
            at += size
        return [torch.cat(x) for x in got]

    # (the chunks' tables of weights formed by every CTA itself, and by the kernel that forms
    # them all before the scan)
    for cuts in ([T], [2] * 26 + [1], [21, 1, 1, 16, 14]):
        for tables in (False, True):
            got = run(cuts, tables)
            for a, b in zip(got, want):
                torch.testing.assert_close(a, b, **tol)
    # a decay that is left out, or taken per head instead of per channel, would show
    flat = [(r[0], r[1], r[2].view(T, H, D).mean(-1, keepdim=True).expand(T, H, D).reshape(T, H * D))
            for r in rows]
    assert (plain_delta(*flat[0], H, G, D, V).float() - want[0]).abs().max() > 1e-2
