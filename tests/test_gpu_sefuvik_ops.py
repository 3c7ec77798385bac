"""Sefuvik's mechanisms one at a time, each kernel (or the few kernels of one mechanism) against the plain model's
function for it: the residual stream in several copies, the rotation that pairs an element with the one half the
rotated dims further on, attention with chunks, windows that keep first tokens, sinks and pairs of maps (over pages
in a shuffled order; whole prompts and single queries), the difference of two maps under a unit norm, and the gated
delta rule behind its convolutions, carried from step to step."""
import math

import numpy as np
import pytest
import torch

import plain_sefuvik as P
from qstream_b200.csrc import ops
from qstream_b200.parts.rotary import _table

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def r32(a):
    """Rounded to 32-bit, as float64: what the kernels are given."""
    return np.asarray(a, dtype=np.float32).astype(np.float64)


@pytest.mark.parametrize("S,D", [(1, 50), (2, 64), (3, 200), (4, 1024), (8, 48)])
def test_the_stream_in_several_copies(S, D):
    """A write with two branches and their factors, the read of the next sublayer and its norm, in one call; then
    the pieces alone."""
    rng = np.random.default_rng(S * D)
    T = 5
    xs = r32(rng.normal(0, 2.0, (T, S, D)))
    y1, y2 = r32(rng.normal(0, 1.0, (T, D))), r32(rng.normal(0, 1.0, (T, D)))
    ls, w = r32(1 + rng.normal(0, 0.3, D)), r32(rng.normal(0, 0.2, D))
    mix, w_in, w_out = r32(rng.normal(0, 0.5, (S, S))), r32(rng.normal(0.3, 0.5, S)), r32(rng.normal(1, 0.5, S))
    y = (0.7 * y1 + 1.3 * y2) * ls
    new = np.stack([sum(mix[s, t] * xs[:, s] for s in range(S)) + w_out[t] * y for t in range(S)], axis=1)
    u = sum(w_in[s] * new[:, s] for s in range(S))
    want_h = P.norm_around_zero(u, w, 1e-5)
    x = dev(xs.reshape(T, S * D))
    h = ops.hyper_mix_norm(x, S, D, y=dev(y1), y_scale=0.7, y2=dev(y2), y2_scale=1.3, layer_scale=dev(ls), mix=dev(mix),
                           out_weights=dev(w_out), in_weights=dev(w_in), norm_weight=dev(w), offset=1.0, eps=1e-5,
                           out_dtype=torch.float32)
    np.testing.assert_allclose(x.cpu().numpy().reshape(T, S, D), new, rtol=0, atol=3e-5)
    np.testing.assert_allclose(h.cpu().numpy(), want_h, rtol=0, atol=3e-5)
    # a read alone leaves the stream as it is; a write alone returns nothing; the sum of the copies
    x = dev(xs.reshape(T, S * D))
    h = ops.hyper_mix_norm(x, S, D, in_weights=dev(w_in), norm_weight=dev(w), offset=1.0, eps=1e-5, out_dtype=torch.float32)
    np.testing.assert_array_equal(x.cpu().numpy(), xs.reshape(T, S * D).astype(np.float32))
    np.testing.assert_allclose(h.cpu().numpy(), P.norm_around_zero(sum(w_in[s] * xs[:, s] for s in range(S)), w, 1e-5), rtol=0, atol=3e-5)
    assert ops.hyper_mix_norm(x, S, D, y=dev(y1), layer_scale=dev(ls), mix=dev(mix), out_weights=dev(w_out)) is None
    one = np.stack([sum(mix[s, t] * xs[:, s] for s in range(S)) + w_out[t] * y1 * ls for t in range(S)], axis=1)
    np.testing.assert_allclose(x.cpu().numpy().reshape(T, S, D), one, rtol=0, atol=3e-5)
    total = ops.hyper_mix_norm(x, S, D, out_dtype=torch.float32, plain_sum=True)
    np.testing.assert_allclose(total.cpu().numpy(), one.sum(1), rtol=0, atol=5e-5)
    spread = ops.hyper_spread(dev(y1), S)
    np.testing.assert_array_equal(spread.cpu().numpy().reshape(T, S, D), np.repeat(y1[:, None].astype(np.float32), S, 1))


@pytest.mark.parametrize("H,d,dims,base", [(3, 16, 8, 1e4), (1, 10, 10, 200.0), (4, 64, 32, 1e6), (2, 12, 0, 1.0)])
def test_the_rotation_by_halves(H, d, dims, base):
    rng = np.random.default_rng(H * d)
    pos = np.array([0, 1, 2, 63, 64, 65, 1000, 30000])
    T = len(pos)
    q, k = r32(rng.normal(size=(T, H, d))), r32(rng.normal(size=(T, H, d)))
    table = _table(dims, base, 32768, DEV) if dims else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for x in (q, k):
        xd = dev(x.reshape(T, H * d))
        ops.rope_store(xd, None, None, H, 0, d, dims, table, i32(np.zeros(T)), i32(pos), None, 64, None, None, status,
                       settled=True, half_layout=True)
        np.testing.assert_allclose(xd.cpu().numpy().reshape(T, H, d), P.rotate_half(x, pos, dims, base), rtol=0, atol=2e-6)
    assert int(status.item()) == 0


class Pages:
    """Keys and values of one sequence in a paged cache entry whose pages lie in a shuffled order among pages full of
    NaN that no query may read."""

    def __init__(self, k, v, page_tokens=64, dtype=torch.float32, seed=0):
        T, G, dk = k.shape
        dv = v.shape[2]
        n = -(-T // page_tokens)
        order = np.random.default_rng(seed).permutation(n + 3)[:n]
        self.k = torch.full((n + 3, G, page_tokens, dk), float("nan"), dtype=dtype, device=DEV)
        self.v = torch.full((n + 3, G, page_tokens, dv), float("nan"), dtype=dtype, device=DEV)
        for p in range(T):
            self.k[order[p // page_tokens], :, p % page_tokens] = dev(k[p], dtype)
            self.v[order[p // page_tokens], :, p % page_tokens] = dev(v[p], dtype)
        # values past the sequence's end, in its last page, are read by no one but must be numbers
        self.v[order[-1], :, T % page_tokens or page_tokens:] = 0
        self.k[order[-1], :, T % page_tokens or page_tokens:] = 0
        self.table = i32(np.concatenate([order, [-1] * 4])[None, :])
        self.page_tokens = page_tokens
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)


MASKS = [dict(chunk=37), dict(chunk=64), dict(chunk=3), dict(chunk=128, sink=True), dict(chunk=21, sink=True),
         dict(window=23, keep=3), dict(window=64, keep=70), dict(window=7, keep=11), dict(window=50, keep=0),
         dict(window=19, keep=2, maps=2), dict(window=0, keep=0, maps=2), dict(sink=True)]


@pytest.mark.parametrize("mask", MASKS, ids=lambda m: "-".join(f"{k}{v}" for k, v in m.items()))
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24), (3, 1, 10, 6), (2, 2, 64, 32)])
def test_attention_with_chunks_windows_sinks_and_pairs_of_maps(mask, sizes):
    """A prompt of 200 tokens at once, and single queries at places of their own (as a decode step asks), over the
    same pages.  The scores are sharp, so that a query rests on few keys."""
    H, G, d, dv = sizes
    chunk, window, keep = mask.get("chunk", 0), mask.get("window", 0), mask.get("keep", 0)
    maps = mask.get("maps", 1)
    rng = np.random.default_rng(H * d + chunk + window)
    T, scale = 200, 2.0 / math.sqrt(d)
    q = r32(rng.normal(size=(T, H, maps, d)))
    k = r32(rng.normal(size=(T, G, maps, d)))
    v = r32(rng.normal(size=(T, G, dv)))
    sink = r32(rng.normal(2.0, 2.0, H)) if mask.get("sink") else None
    see = (lambda i, j: P.visible_chunk(i, j, chunk)) if chunk else (lambda i, j: P.visible_window(i, j, window, keep))
    want = np.stack([P.masked_softmax_attention(q[:, :, m], k[:, :, m], v, scale, see, sink=sink) for m in range(maps)], axis=2)
    pages = Pages(k.reshape(T, G, maps * d), v)
    sink_dev = None
    if sink is not None:                                 # one per query head
        sink_dev = dev(sink)

    def run(rows):
        return ops.attention(dev(q[rows].reshape(len(rows), H * maps * d)), H * maps, G, d, scale, window, i32(np.zeros(len(rows))),
                             i32(rows), pages.table, pages.page_tokens, pages.k, pages.v, pages.status, v_head_dim=dv,
                             chunk=chunk, keep_first=keep, sink=sink_dev, maps=maps, out_dtype=torch.float32)
    got = run(np.arange(T)).cpu().numpy().reshape(T, H, maps, dv)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5)
    for p in (0, 1, 63, 64, 65, 127, 128, 199):
        one = run(np.array([p])).cpu().numpy().reshape(H, maps, dv)
        np.testing.assert_allclose(one, want[p], rtol=0, atol=2e-5)
    assert int(pages.status.item()) == 0


def test_one_key_that_stands_out_just_inside_and_just_outside():
    """One key has a score far above all others: a query sees its value alone while the key is inside the window
    (the chunk, the kept first tokens), and nothing of it from the next place on."""
    d, dv, T = 16, 8, 160
    rng = np.random.default_rng(5)
    for star, rule in ((70, dict(window=30, keep=4)), (2, dict(window=9, keep=3)), (3, dict(window=9, keep=3)), (64, dict(chunk=40))):
        q, k, v = r32(rng.normal(size=(T, 1, d))), r32(rng.normal(size=(T, 1, d))) * 0.1, r32(rng.normal(size=(T, 1, dv)))
        q[:, 0, 0], k[:, 0, 0] = 6.0, 0.0
        k[star, 0, 0] = 6.0                               # 36 above the others' scores
        pages = Pages(k, v)
        got = ops.attention(dev(q.reshape(T, d)), 1, 1, d, 1.0, rule.get("window", 0), i32(np.zeros(T)), i32(np.arange(T)),
                            pages.table, 64, pages.k, pages.v, pages.status, v_head_dim=dv, chunk=rule.get("chunk", 0),
                            keep_first=rule.get("keep", 0), out_dtype=torch.float32).cpu().numpy()
        chunk, window, keep = rule.get("chunk", 0), rule.get("window", 0), rule.get("keep", 0)
        for i in range(star, T):
            seen = P.visible_chunk(i, star, chunk) if chunk else P.visible_window(i, star, window, keep)
            near = np.abs(got[i] - v[star, 0]).max() < 1e-3
            assert near == seen, (rule, star, i)
        last = star + window - 1 if window and star >= keep else (star // chunk + 1) * chunk - 1 if chunk else T - 1
        assert np.abs(got[last] - v[star, 0]).max() < 1e-3
        if last + 1 < T:
            assert np.abs(got[last + 1] - v[star, 0]).max() > 0.1


@pytest.mark.parametrize("H,dv", [(3, 8), (1, 6), (4, 64), (2, 200)])
def test_the_difference_of_two_maps_under_a_unit_norm(H, dv):
    rng = np.random.default_rng(H * dv)
    a = r32(rng.normal(size=(9, H, 2, dv)))
    lam, diff, eps = 0.37, 0.2, 1e-5
    want = P.rms_unit(a[:, :, 0] - lam * a[:, :, 1], eps) * (1.0 - diff)
    got = ops.pair_diff_norm(dev(a.reshape(9, H * 2 * dv)), H, dv, lam, 1.0 - diff, eps, torch.float32)
    np.testing.assert_allclose(got.cpu().numpy().reshape(9, H, dv), want, rtol=0, atol=3e-6)
    half = ops.pair_diff_norm(dev(a.reshape(9, H * 2 * dv)), H, dv, lam, 1.0 - diff, eps, torch.bfloat16)
    np.testing.assert_allclose(half.float().cpu().numpy().reshape(9, H, dv), want, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("sizes", [(4, 2, 8, 12, 4), (5, 5, 6, 4, 1), (3, 1, 10, 14, 5), (2, 1, 64, 64, 4), (4, 4, 32, 128, 2)])
def test_the_gated_delta_rule_step_after_step(sizes):
    """Convolutions with silu, unit vectors, decays and step sizes, the scan and the normed, gated read-out: two
    sequences of unequal lengths in steps of 1 to 40 tokens from states that earlier steps left, in slots 2 and 0 of
    four; against the plain mixer's walk over each whole sequence."""
    H, G, d, dv, taps = sizes
    D, ra, rg, eps = 24, 5, 7, 1e-5
    rng = np.random.default_rng(H * d + taps)
    nq, nv = G * d, H * dv
    W = {"m." + n: r32(rng.normal(0, 1.5 / math.sqrt(s[1]), s)) for n, s in (
        ("q", (nq, D)), ("k", (nq, D)), ("v", (nv, D)), ("b", (H, D)), ("a1", (ra, D)), ("a2", (H * d, ra)), ("g1", (rg, D)),
        ("g2", (nv, rg)), ("o", (nv, nv)))}
    W["m.o"] = np.eye(nv)
    W.update({"m.q.conv": r32(rng.normal(0, 0.7, (nq, taps))), "m.k.conv": r32(rng.normal(0, 0.7, (nq, taps))),
              "m.v.conv": r32(rng.normal(0, 0.7, (nv, taps))), "m.A_log": r32(rng.uniform(-4, -0.5, H)),
              "m.dt_bias": r32(rng.uniform(-3, 1, H * d)), "m.norm": r32(1 + rng.normal(0, 0.2, dv))})
    lens = (93, 41)
    hs = [r32(rng.normal(size=(n, D))) for n in lens]
    want = [P.gated_delta({"heads": H, "kv_heads": G, "dim": d, "vdim": dv}, W, "m.", h, eps) for h in hs]
    slots = (2, 0)
    state = torch.zeros((4, H, dv, d), dtype=torch.float32, device=DEV)
    held = torch.zeros((4, max(taps - 1, 1), 2 * nq + nv), dtype=torch.float32, device=DEV)
    got = [[], []]
    at = [0, 0]
    for step_len in (1, 2, 40, 1, 7, 40, 40):
        seqs = [(i, min(step_len, lens[i] - at[i])) for i in range(2) if at[i] < lens[i]]
        h = np.concatenate([hs[i][at[i]:at[i] + n] for i, n in seqs])
        T = len(h)
        tok_slot = np.concatenate([[slots[i]] * n for i, n in seqs])
        tok_pos = np.concatenate([np.arange(at[i], at[i] + n) for i, n in seqs])
        seq_start = np.concatenate([[0], np.cumsum([n for _, n in seqs])])
        p = dev(np.concatenate([h @ W["m.q"].T, h @ W["m.k"].T, h @ W["m.v"].T], axis=1))
        q, k, v = p[:, :nq], p[:, nq:2 * nq], p[:, 2 * nq:]
        a = dev((h @ W["m.a1"].T) @ W["m.a2"].T + W["m.dt_bias"])
        b = dev(h @ W["m.b"].T)
        conv = [dev(W[f"m.{n}.conv"]) for n in "qkv"]
        cs = held if taps > 1 else None
        qo, ko, vo, decay, beta = ops.delta_prepare(q, k, v, *conv, cs, a, b, dev(W["m.A_log"]), i32(tok_slot), i32(tok_pos),
                                                    G, H, d, dv, d ** -0.5, 1e-6)
        if cs is not None:
            ops.conv_state_update(cs, q, k, v, nq, nv, taps, i32(seq_start), i32([slots[i] for i, _ in seqs]), len(seqs))
        o = ops.state_scan("delta", qo, ko, vo, state, i32(seq_start), i32([slots[i] for i, _ in seqs]), len(seqs), H, d, dv,
                           key_decay=decay, token_weight=beta, qk_group=H // G)
        gate = dev((h @ W["m.g1"].T) @ W["m.g2"].T)
        y = ops.gated_group_norm(o, dv, dev(np.tile(W["m.norm"], H)), gate, "sigmoid", eps, torch.float32).cpu().numpy()
        for j, (i, n) in enumerate(seqs):
            got[i].append(y[seq_start[j]:seq_start[j] + n])
            at[i] += n
    for i in range(2):
        g = np.concatenate(got[i])
        assert g.shape == want[i].shape
        np.testing.assert_allclose(g, want[i], rtol=0, atol=1e-4 * max(1.0, np.abs(want[i]).max()))
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0    # the other slots were not touched


def rbf(a):
    """Rounded to bfloat16, as float64."""
    return torch.tensor(np.asarray(a), dtype=torch.bfloat16).to(torch.float64).numpy()


@pytest.mark.parametrize("mask", MASKS, ids=lambda m: "-".join(f"{k}{v}" for k, v in m.items()))
@pytest.mark.parametrize("sizes", [(4, 2, 16, 32), (2, 2, 64, 32), (4, 1, 128, 128), (2, 1, 128, 256)])
def test_the_bfloat16_kernels_take_the_same_masks(mask, sizes):
    """The tensor-core kernel for prompts (whole, and as a second portion that starts in the middle of a page) and the
    split-key kernel for single queries, with a gate where the form has one map; 330 keys, so that queries lie beyond
    the first split of 256 keys and windows leave whole pages (and splits) behind."""
    from qstream_b200.csrc import attention_bf16
    H, G, d, dv = sizes
    chunk, window, keep = mask.get("chunk", 0), mask.get("window", 0), mask.get("keep", 0)
    maps = mask.get("maps", 1)
    rng = np.random.default_rng(H * d + chunk + window + 1)
    T, scale = 330, 2.0 / math.sqrt(d)
    q = rbf(rng.normal(size=(T, H, maps, d)))
    k = rbf(rng.normal(size=(T, G, maps, d)))
    v = rbf(rng.normal(size=(T, G, dv)))
    sink = r32(rng.normal(2.0, 2.0, H)) if mask.get("sink") else None
    gate = rbf(rng.normal(size=(T, H * dv))) if maps == 1 else None
    see = (lambda i, j: P.visible_chunk(i, j, chunk)) if chunk else (lambda i, j: P.visible_window(i, j, window, keep))
    want = np.stack([P.masked_softmax_attention(q[:, :, m], k[:, :, m], v, scale, see, sink=sink) for m in range(maps)], axis=2)
    want = want.reshape(T, H * maps * dv)
    if gate is not None:
        want = want * P.sigmoid(gate)
    pages = Pages(k.reshape(T, G, maps * d), v, dtype=torch.bfloat16)
    bf = torch.bfloat16
    qd = dev(q.reshape(T, H * maps * d), bf)
    gd = dev(gate, bf) if gate is not None else None
    opts = dict(v_head_dim=dv, chunk=chunk, keep_first=keep, sink=dev(sink) if sink is not None else None, maps=maps,
                out_dtype=torch.float32 if maps > 1 else None)
    for start in (0, 100):
        rows = T - start
        tiles = i32([(a - start, min(128, T - a), a, 0) for a in range(start, T, 128)][::-1])
        got = attention_bf16.prefill(qd[start:], H * maps, G, d, scale, window, tiles, pages.table, 64, pages.k, pages.v, pages.status,
                                     gate=gd[start:] if gd is not None else None, **opts)
        assert got.dtype == (torch.float32 if maps > 1 else bf) and got.shape[0] == rows
        np.testing.assert_allclose(got.float().cpu().numpy(), want[start:], rtol=0, atol=3e-2)
    places = np.array([0, 1, 63, 64, 65, 127, 128, 255, 256, 257, 300, 329])
    got = attention_bf16.decode(qd[places].contiguous(), H * maps, G, d, scale, window, i32(np.zeros(len(places))), i32(places),
                                pages.table.expand(1, -1).contiguous(), 64, pages.k, pages.v, 512, pages.status,
                                gate=gd[places].contiguous() if gd is not None else None, **opts)
    np.testing.assert_allclose(got.float().cpu().numpy(), want[places], rtol=0, atol=1e-4 if maps > 1 else 1e-2)
    assert int(pages.status.item()) == 0


@pytest.mark.parametrize("sizes", [(4, 2, 8, 12), (2, 1, 64, 64), (3, 3, 10, 14), (2, 2, 128, 96)])
def test_the_delta_rule_in_chunks_equals_the_walk_in_order(sizes):
    """Two prompts of unequal lengths cut into chunks of 64 (the last ones ragged), from states that a first step
    left, against the same kernel's walk in order; small decays among them (a chunk's product of decays underflows
    nothing, since nothing is divided by it)."""
    H, G, d, dv = sizes
    rng = np.random.default_rng(H * d)
    lens, first = (333, 200), 17
    T = sum(lens)
    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)      # noqa: E731
    q = dev(unit(rng.normal(size=(T, G, d))).reshape(T, G * d) * d ** -0.5)
    k = dev(unit(rng.normal(size=(T, G, d))).reshape(T, G * d))
    v = dev(rng.normal(size=(T, H * dv)))
    decay = dev(np.where(rng.random((T, H * d)) < 0.1, rng.uniform(1e-3, 0.5, (T, H * d)), rng.uniform(0.9, 1.0, (T, H * d))))
    beta = dev(rng.uniform(0.0, 1.0, (T, H)))
    walk = dict(key_decay=decay, token_weight=beta, qk_group=H // G)
    slots, n_slots = (2, 0), 3
    starts = [0, lens[0], T]

    def run(chunked):
        state = torch.zeros((n_slots, H, dv, d), dtype=torch.float32, device=DEV)
        outs = [None, None]
        # a first step of 17 tokens each in order, then the rest in one step
        rows1 = np.concatenate([np.arange(starts[i], starts[i] + first) for i in range(2)])
        rows2 = np.concatenate([np.arange(starts[i] + first, starts[i + 1]) for i in range(2)])
        for rows, n_each in ((rows1, [first, first]), (rows2, [n - first for n in lens])):
            sel = torch.tensor(rows, device=DEV)
            seq_start = np.concatenate([[0], np.cumsum(n_each)])
            chunks = None
            if chunked and max(n_each) > 64:
                cs, owners, row = [0], [0], 0
                for n in n_each:
                    cs += [row + min(n, a + 64) for a in range(0, n, 64)]
                    row += n
                    owners.append(len(cs) - 1)
                chunks = (i32(cs), i32(np.arange(len(cs) - 1)), i32(owners), len(cs) - 1)
            o = ops.state_scan("delta", q[sel].contiguous(), k[sel].contiguous(), v[sel].contiguous(), state, i32(seq_start), i32(slots), 2,
                               H, d, dv, chunks=chunks, key_decay=decay[sel].contiguous(), token_weight=beta[sel].contiguous(),
                               qk_group=H // G)
            outs[0 if rows is rows1 else 1] = o.cpu().numpy()
        return outs, state.cpu().numpy()
    (a1, a2), sa = run(False)
    (b1, b2), sb = run(True)
    np.testing.assert_array_equal(a1, b1)
    scale = max(1.0, np.abs(a2).max())
    np.testing.assert_allclose(b2, a2, rtol=0, atol=2e-5 * scale)
    np.testing.assert_allclose(sb, sa, rtol=0, atol=2e-5 * max(1.0, np.abs(sa).max()))
    assert np.abs(sa[1]).max() == 0.0 and np.abs(sb[1]).max() == 0.0
