"""Nutatar's mechanisms one at a time, each kernel (or kernel option) against the plain model's function for it: the
stream read as it is behind a normed branch, the gate per head, the clamped gated unit, the softmax router with group
maxima, gated experts through the routing table, the linear attention's walk (in order, carried from step to step, and
in chunks), the latent's rotation by neighbours with scaled frequencies, and attention whose values are its keys under
one norm over all heads, with a sink of score zero."""
import numpy as np
import pytest
import torch

import plain_nutatar as P
from qstream_b200.csrc import ops
from qstream_b200.parts.rotary import scaled_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def r32(a):
    """Rounded to 32-bit, as float64: what the kernels are given."""
    return np.asarray(a, dtype=np.float32).astype(np.float64)


@pytest.mark.parametrize("D", [50, 64, 1000])
def test_a_normed_branch_joins_the_stream_and_the_stream_is_read_as_it_is(D):
    rng = np.random.default_rng(D)
    T = 7
    x, y, w = r32(rng.normal(0, 2.0, (T, D))), r32(rng.normal(0, 3.0, (T, D))), r32(1 + rng.normal(0, 0.3, D))
    new = x + P.rms_norm(y, w, 1e-5)
    xd = dev(x)
    h = ops.branch_norm(xd, None, 1e-5, False, out_dtype=torch.bfloat16, branch=dev(y), branch_weight=dev(w))
    np.testing.assert_allclose(xd.cpu().numpy(), new, rtol=0, atol=3e-6)
    assert h.dtype == torch.bfloat16
    np.testing.assert_array_equal(h.float().cpu().numpy(), xd.to(torch.bfloat16).float().cpu().numpy())
    h = ops.branch_norm(xd, None, 1e-5, False, out_dtype=torch.bfloat16)           # the read alone changes nothing
    np.testing.assert_allclose(xd.cpu().numpy(), new, rtol=0, atol=3e-6)
    np.testing.assert_array_equal(h.float().cpu().numpy(), xd.to(torch.bfloat16).float().cpu().numpy())


@pytest.mark.parametrize("H,dv", [(3, 12), (1, 7), (6, 64)])
def test_one_gate_value_per_head(H, dv):
    rng = np.random.default_rng(H * dv)
    T = 5
    o, g = r32(rng.normal(size=(T, H, dv))), r32(rng.normal(0, 2.0, (T, H)))
    got = ops.gated_group_norm(dev(o.reshape(T, H * dv)), 0, None, dev(g), "sigmoid", 0.0, torch.float32, gate_span=dv)
    np.testing.assert_allclose(got.cpu().numpy().reshape(T, H, dv), o * P.sigmoid(g)[:, :, None], rtol=0, atol=1e-6)


@pytest.mark.parametrize("F,limit", [(20, 1.0), (7, 0.5), (256, 2.5)])
def test_the_clamped_gated_unit(F, limit):
    rng = np.random.default_rng(F)
    a, b = r32(rng.normal(0, 2.0, (9, F))), r32(rng.normal(0, 2.0, (9, F)))
    g, u = np.minimum(a, limit), np.clip(b, -limit, limit)
    want = g * P.sigmoid(1.702 * g) * (u + 1.0)
    assert (a > limit).any() and (b < -limit).any() and (a < -limit).any()
    got = ops.clamped_glu(dev(np.concatenate([a, b], 1)), limit, 1.702, 1.0)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=0, atol=2e-6)


@pytest.mark.parametrize("E,top,count,keep", [(6, 2, 3, 2), (16, 4, 4, 2), (4, 4, 4, 4), (5, 1, 1, 1), (12, 3, 3, 1), (40, 2, 8, 3)])
def test_the_softmax_router_with_group_maxima(E, top, count, keep):
    rng = np.random.default_rng(E * top)
    T = 200
    z = r32(rng.normal(0, 2.0, (T, E)))
    chosen, weights = P.route(z, top, count, keep)
    idx, wts, gate = ops.moe_route(dev(z), None, E, top, count, keep, 1.0, scores="softmax", group_score="max")
    assert gate is None
    np.testing.assert_array_equal(idx.cpu().numpy(), chosen)
    np.testing.assert_allclose(wts.cpu().numpy(), weights, rtol=0, atol=1e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
def test_gated_experts_through_the_routing_table(dtype, tol):
    rng = np.random.default_rng(3)
    T, D, F, E, top, limit = 11, 40, 12, 5, 2, 0.8
    rnd = (lambda a: dev(a, dtype).double().cpu().numpy())
    x = rnd(rng.normal(size=(T, D)))
    w = {}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (rnd(rng.normal(0, D ** -0.5, (F, D))), rnd(rng.normal(0, D ** -0.5, (F, D))),
                                                            rnd(rng.normal(0, F ** -0.5, (D, F))))
    idx = np.stack([rng.permutation(E)[:top] for _ in range(T)])
    wts = r32(rng.uniform(0.1, 0.9, (T, top)))
    want = np.zeros((T, D))
    for t in range(T):
        for e, c in zip(idx[t], wts[t]):
            want[t] += c * P.expert(w, f"e{e}.", x[t:t + 1], limit)[0]
    w_up = torch.stack([torch.cat([dev(w[f"e{e}.gate"], dtype), dev(w[f"e{e}.up"], dtype)]) for e in range(E)]).contiguous()
    w_down = torch.stack([dev(w[f"e{e}.down"], dtype) for e in range(E)]).contiguous()
    got = ops.moe_experts_indirect(dev(x, dtype), w_up, w_down, i32(idx), dev(wts), i32(np.zeros(T)), None,
                                   glu=(limit, 1.702, 1.0))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=0, atol=tol)


def plain_walk(q, k, v, z, power, S):
    """The linear attention's walk in float64 from the state S [H, dk, dv]; returns (o [T, H, dv], S)."""
    T, H, _ = q.shape
    o = np.zeros((T, H, v.shape[2]))
    alpha = P.sigmoid(z) ** power
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    return o, S


@pytest.mark.parametrize("H,dk,dv,tau", [(3, 8, 12, 4.0), (1, 10, 14, 1.0), (2, 64, 32, 16.0), (5, 6, 4, 30.0)])
def test_the_linear_attention_s_walk_in_order_in_steps_and_in_chunks(H, dk, dv, tau):
    rng = np.random.default_rng(H * dk)
    T = 300
    q, k, v = (r32(rng.normal(0, 0.7, (T, H, n))) for n in (dk, dk, dv))
    target = rng.uniform(0.5, 0.9999, (H, dk)) ** tau
    z = r32(np.log(target / (1 - target))[None] + rng.normal(0, 1.0, (T, H, dk)))
    want, S_end = plain_walk(q * dk ** -0.5, k, v, z, 1.0 / tau, np.zeros((H, dk, dv)))

    def run(pieces, chunked):
        state = torch.zeros((2, H, dv, dk), dtype=torch.float32, device=DEV)
        out, at = [], 0
        for n in pieces:
            sl = slice(at, at + n)
            chunks = None
            if chunked:
                starts = list(range(0, n, 64)) + [n]
                nc = len(starts) - 1
                chunks = (i32(starts), i32(np.arange(nc)), i32([0, nc]), nc)
            out.append(ops.state_scan("gla", dev(q[sl].reshape(n, -1)), dev(k[sl].reshape(n, -1)), dev(v[sl].reshape(n, -1)), state,
                                      i32([0, n]), i32([1]), 1, H, dk, dv, decay_logits=dev(z[sl].reshape(n, -1)),
                                      decay_power=1.0 / tau, q_scale=dk ** -0.5, chunks=chunks).cpu().numpy())
            at += n
        assert float(state[0].abs().max()) == 0.0                                   # another sequence's slot is untouched
        return np.concatenate(out).reshape(T, H, dv), state[1].cpu().numpy().transpose(0, 2, 1)

    scale = np.abs(want).max()
    for pieces, chunked in (((T,), False), ((1,) * 40 + (2, 3, 64, 65, 126), False), ((T,), True), ((130, 170), True)):
        o, S = run(pieces, chunked)
        assert np.abs(o - want).max() <= 3e-5 * scale, (pieces, chunked, np.abs(o - want).max() / scale)
        assert np.abs(S - S_end).max() <= 3e-5 * np.abs(S_end).max(), (pieces, chunked)


def test_a_far_token_reaches_the_end_through_channels_that_do_not_forget():
    """One key channel keeps everything, the others forget fast; a value written at the first token under the keeping
    channel alone is read back 500 tokens later, in chunks as in order."""
    H, dk, dv, T = 1, 8, 4, 500
    q, k, v = np.zeros((T, H, dk)), np.zeros((T, H, dk)), np.zeros((T, H, dv))
    rng = np.random.default_rng(0)
    k[:, 0, 1:], v[:] = rng.normal(size=(T, dk - 1)), rng.normal(size=(T, H, dv))
    k[0, 0, 0], v[0, 0] = 1.0, [1.0, -2.0, 3.0, -4.0]
    q[T - 1, 0, 0] = 1.0
    z = np.zeros((T, H, dk))
    z[:, :, 0], z[:, :, 1:] = 40.0, -3.0
    for chunked in (False, True):
        state = torch.zeros((1, H, dv, dk), dtype=torch.float32, device=DEV)
        starts = list(range(0, T, 64)) + [T]
        chunks = (i32(starts), i32(np.arange(len(starts) - 1)), i32([0, len(starts) - 1]), len(starts) - 1) if chunked else None
        o = ops.state_scan("gla", dev(q.reshape(T, -1)), dev(k.reshape(T, -1)), dev(v.reshape(T, -1)), state, i32([0, T]), i32([0]), 1,
                           H, dk, dv, decay_logits=dev(z.reshape(T, -1)), decay_power=1.0, q_scale=1.0, chunks=chunks).cpu().numpy()
        np.testing.assert_allclose(o[T - 1], [1.0, -2.0, 3.0, -4.0], rtol=0, atol=1e-5)


@pytest.mark.parametrize("dims,rot_dim,scaling", [(8, 8, (2.0, 32, 4.0, 1.0)), (4, 6, None), (32, 32, (4.0, 128, 8.0, 0.5))])
def test_the_latent_s_rotation_by_neighbours(dims, rot_dim, scaling):
    """The shared key part as the cache holds it and every head's rotated query part, at positions across pages."""
    rng = np.random.default_rng(dims)
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    f, mag = P.yarn_frequencies(dims, 1e3, sc)
    freq, mag_lib = scaled_frequencies(dims, 1e3, sc)
    np.testing.assert_allclose(freq.numpy(), f, rtol=1e-14)
    assert mag_lib == pytest.approx(mag)
    pos = np.array([0, 1, 63, 64, 65, 130, 191])
    T, r, H, dn, rq = len(pos), 10, 3, 4, 6
    dq, dkv = r32(rng.normal(size=(T, rq))), r32(rng.normal(size=(T, r + rot_dim)))
    wq, wkv = r32(1 + rng.normal(0, 0.2, rq)), r32(1 + rng.normal(0, 0.2, r))
    k_cache = torch.zeros((4, 1, 64, r + rot_dim), dtype=torch.float32, device=DEV)
    v_cache = torch.zeros((4, 1, 64, r), dtype=torch.float32, device=DEV)
    table = i32([[2, 0, 3, -1]])                             # the sequence's pages in a shuffled order
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    cq = ops.latent_prepare(dev(dq), dev(wq), rq, dev(dkv), dev(wkv), r, rot_dim, dims, freq.to(DEV), mag, 1e-5, i32(np.zeros(T)),
                            i32(pos), table, 64, k_cache, v_cache, status, interleaved=True)
    np.testing.assert_allclose(cq.cpu().numpy(), P.rms_norm(dq, wq, 1e-5), rtol=0, atol=2e-6)
    c = P.rms_norm(dkv[:, :r], wkv, 1e-5)
    kr = P.rotate(dkv[:, None, r:], pos, dims, f, mag, True)[:, 0]
    pages = [2, 0, 3]
    for t, p in enumerate(pos):
        row = k_cache[pages[p // 64], 0, p % 64].cpu().numpy()
        np.testing.assert_allclose(row, np.concatenate([c[t], kr[t]]), rtol=0, atol=3e-6)
        np.testing.assert_allclose(v_cache[pages[p // 64], 0, p % 64].cpu().numpy(), c[t], rtol=0, atol=3e-6)
    q = r32(rng.normal(size=(T, H, dn + rot_dim)))
    q_abs = torch.zeros((T, H * (r + rot_dim)), dtype=torch.float32, device=DEV)
    ops.latent_q_rotate(q_abs, dev(q.reshape(T, -1)), H, dn, rot_dim, r, dims, freq.to(DEV), mag, i32(np.zeros(T)), i32(pos), interleaved=True)
    got = q_abs.cpu().numpy().reshape(T, H, r + rot_dim)[:, :, r:]
    np.testing.assert_allclose(got, P.rotate(q[:, :, dn:], pos, dims, f, mag, True), rtol=0, atol=3e-6)
    assert int(status.item()) == 0


@pytest.mark.parametrize("H,G,d,dims,half", [(4, 2, 16, 8, True), (1, 1, 10, 10, True), (3, 3, 6, 0, True), (6, 2, 64, 32, True), (2, 1, 8, 4, False)])
def test_one_norm_over_all_heads_then_rotation_and_cache_write(H, G, d, dims, half):
    """q and k normed over their whole rows, rotated by halves (or neighbours), k kept in the pages with the raw k as
    values; positions across pages in a shuffled page order; a row of no sequence."""
    from qstream_b200.parts.rotary import _table
    rng = np.random.default_rng(H * d)
    pos = np.array([0, 1, 63, 64, 65, 130, 191, 5])
    slots = np.array([0, 0, 0, 0, 0, 0, 0, -1])
    T = len(pos)
    qk = r32(rng.normal(size=(T, (H + G) * d)))
    wq, wk = r32(1 + rng.normal(0, 0.3, H * d)), r32(1 + rng.normal(0, 0.3, G * d))
    base = 1e3
    f = P.plain_frequencies(dims, base) if dims else np.zeros(0)
    want_q = P.rotate(P.rms_norm(qk[:, :H * d], wq, 1e-5).reshape(T, H, d), pos, dims, f, 1.0, not half)
    want_k = P.rotate(P.rms_norm(qk[:, H * d:], wk, 1e-5).reshape(T, G, d), pos, dims, f, 1.0, not half)
    k_cache = torch.zeros((4, G, 64, d), dtype=torch.float32, device=DEV)
    v_cache = torch.zeros((4, G, 64, d), dtype=torch.float32, device=DEV)
    table = i32([[2, 0, 3, -1]])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = dev(qk)
    ops.norm_rope_store(x[:, :H * d], x[:, H * d:], x[:, H * d:], dev(wq), dev(wk), 1e-5, H, G, d, dims,
                        _table(dims, base, 4096, DEV) if dims else None, i32(slots), i32(pos), table, 64, k_cache, v_cache, status,
                        half_layout=half)
    got = x.cpu().numpy()
    np.testing.assert_allclose(got[:7, :H * d].reshape(7, H, d), want_q[:7], rtol=0, atol=3e-6)
    np.testing.assert_array_equal(got[7, :H * d], 0.0)
    np.testing.assert_array_equal(got[:, H * d:], qk[:, H * d:].astype(np.float32))      # k itself stays as projected
    pages = [2, 0, 3]
    for t in range(7):
        p = pos[t]
        np.testing.assert_allclose(k_cache[pages[p // 64], :, p % 64].cpu().numpy(), want_k[t], rtol=0, atol=3e-6)
        np.testing.assert_array_equal(v_cache[pages[p // 64], :, p % 64].cpu().numpy(), qk[t, H * d:].reshape(G, d).astype(np.float32))
    assert int(status.item()) == 0


@pytest.mark.parametrize("H,G,d,dims,half", [(6, 2, 64, 32, True), (4, 2, 16, 16, True), (2, 1, 8, 8, False), (4, 4, 128, 64, True),
                                             (2, 2, 32, 0, True), (3, 1, 24, 8, True)])
def test_the_same_in_bfloat16_in_16_byte_pieces(H, G, d, dims, half):
    """Sizes that take the kernel's 16-byte form (and one that does not), against the plain functions on the rounded
    inputs; the result is rounded once."""
    from qstream_b200.parts.rotary import _table
    rng = np.random.default_rng(H * d + dims)
    bf = torch.bfloat16
    pos = np.array([0, 1, 63, 64, 65, 130, 191, 5])
    slots = np.array([0, 0, 0, 0, 0, 0, 0, -1])
    T = len(pos)
    x = dev(rng.normal(size=(T, (H + G) * d)), bf)
    wq, wk = dev(1 + rng.normal(0, 0.3, H * d), bf), dev(1 + rng.normal(0, 0.3, G * d), bf)
    qk = x.double().cpu().numpy()
    f = P.plain_frequencies(dims, 1e3) if dims else np.zeros(0)
    want_q = P.rotate(P.rms_norm(qk[:, :H * d], wq.double().cpu().numpy(), 1e-5).reshape(T, H, d), pos, dims, f, 1.0, not half)
    want_k = P.rotate(P.rms_norm(qk[:, H * d:], wk.double().cpu().numpy(), 1e-5).reshape(T, G, d), pos, dims, f, 1.0, not half)
    k_cache = torch.zeros((4, G, 64, d), dtype=bf, device=DEV)
    v_cache = torch.zeros((4, G, 64, d), dtype=bf, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.norm_rope_store(x[:, :H * d], x[:, H * d:], x[:, H * d:], wq, wk, 1e-5, H, G, d, dims,
                        _table(dims, 1e3, 4096, DEV) if dims else None, i32(slots), i32(pos), i32([[2, 0, 3, -1]]), 64, k_cache, v_cache,
                        status, half_layout=half)
    got = x.double().cpu().numpy()
    np.testing.assert_allclose(got[:7, :H * d].reshape(7, H, d), want_q[:7], rtol=2 ** -8, atol=1e-3)
    np.testing.assert_array_equal(got[7, :H * d], 0.0)
    np.testing.assert_array_equal(got[:, H * d:], qk[:, H * d:])
    pages = [2, 0, 3]
    for t in range(7):
        p = pos[t]
        np.testing.assert_allclose(k_cache[pages[p // 64], :, p % 64].double().cpu().numpy(), want_k[t], rtol=2 ** -8, atol=1e-3)
        np.testing.assert_array_equal(v_cache[pages[p // 64], :, p % 64].double().cpu().numpy(), qk[t, H * d:].reshape(G, d))
    assert int(status.item()) == 0
