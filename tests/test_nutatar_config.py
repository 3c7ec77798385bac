"""Nutatar's configuration: reading, validation, the model it describes; and the plain model's own pieces on inputs
whose results are known."""
import copy
import math

import numpy as np
import pytest

import qstream_b200 as qs
from qstream_b200.config.nutatar import NutatarConfig
from qstream_b200.engine.model import declared_tensors
from qstream_b200.errors import QStreamError

import plain_nutatar as P
from nutatar_util import CONFIGS, make_weights


@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_the_declared_tensors_are_the_checkpoint_s(which):
    cfg = qs.config_from_dict(CONFIGS[which])
    assert isinstance(cfg, NutatarConfig)
    decl = declared_tensors(cfg.model_spec())
    weights = make_weights(CONFIGS[which], 0, decay_rank=5)
    assert set(decl) == set(weights)
    for name, d in decl.items():
        assert len(d.shape) == weights[name].ndim, name
        assert all(a in (-1, b) for a, b in zip(d.shape, weights[name].shape)), name    # -1: the checkpoint's own size (a rank)
    assert qs.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_the_schedule_and_the_parts_follow_the_layers():
    spec = qs.config_from_dict(CONFIGS["A"]).model_spec()
    assert [r.cache for r in spec.schedule] == [0, 1, 2, 2, 4, 2]           # layers 3 and 5 read layer 2's latents
    assert [b.arrangement for b in spec.layers] == ["post_norm"] * 6
    assert spec.layers[2].ffn is None and set(spec.layers[2].norms) == {"post_input"}
    assert set(spec.layers[0].norms) == {"post_input", "post_ffn"} and not spec.head.tied
    gla, windowed, latent, sharing, plain = (spec.layers[i].mixer for i in (0, 1, 2, 3, 4))
    assert (gla.kind, gla.tau, gla.key_dim, gla.value_dim) == ("gla", 4.0, 8, 12)
    assert (windowed.window, windowed.qk_norm, windowed.values_from_keys, windowed.fixed_sink) == (37, "whole", True, 0.0)
    assert windowed.position.rotary_dim == 8 and plain.window == 0
    assert latent.position.layout == "interleaved" and latent.position.scaling["factor"] == 8.0
    assert (latent.shares_cache, sharing.shares_cache, latent.sink, latent.head_gate) == (False, True, True, True)
    experts = spec.layers[0].ffn
    assert (experts.scores, experts.group_score, experts.groups, experts.keep, experts.top) == ("softmax", "max", 3, 2, 2)
    assert (experts.gated, experts.limit, experts.shared_limit, experts.shared_gate, experts.correction) == (True, 1.0, 2.5, False, False)
    assert spec.layers[1].ffn.activation == "relu2" and spec.embedding.scale == 3.0


def test_a_layer_that_reads_another_s_latents_may_leave_their_sizes_out():
    cfg = copy.deepcopy(CONFIGS["A"])
    for key in ("kv_rank", "rot_dim", "rot"):
        del cfg["layers"][3]["mixer"][key]
    spec = qs.config_from_dict(cfg).model_spec()
    assert spec.layers[3].mixer == qs.config_from_dict(CONFIGS["A"]).model_spec().layers[3].mixer


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=-1), "mask"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=4), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "router"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, needle):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises(QStreamError) as e:
        qs.config_from_dict(cfg)
    assert needle in str(e.value)


def test_the_plain_softmax_with_a_sink_on_a_hand_made_case():
    """Two equal scores and a sink of the same size: each key weighs a third, and a third of the weight is lost; with
    one key, a half."""
    scores = np.ones((2, 2))
    visible = np.array([[True, False], [True, True]])
    p = P.softmax_with_sink(scores, visible, 1.0)
    np.testing.assert_allclose(p, [[0.5, 0.0], [1 / 3, 1 / 3]])
    np.testing.assert_allclose(P.softmax_with_sink(scores, visible, None), [[1.0, 0.0], [0.5, 0.5]])


def test_the_plain_rotations_pair_halves_or_neighbours():
    x = np.zeros((1, 1, 6))
    x[0, 0] = [1.0, 2.0, 0.0, 0.0, 5.0, 6.0]
    f = P.plain_frequencies(4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    np.testing.assert_allclose(f, [1.0, 100.0 ** -0.5])
    out = P.rotate(x, [3], 4, f, 1.0, False)[0, 0]
    np.testing.assert_allclose(out, [math.cos(a0), 2 * math.cos(a1), math.sin(a0), 2 * math.sin(a1), 5.0, 6.0], atol=1e-12)
    out = P.rotate(x, [3], 4, f, 2.0, True)[0, 0]           # pairs (1, 2) and (0, 0); cos and sin doubled
    np.testing.assert_allclose(out, [2 * (math.cos(a0) - 2 * math.sin(a0)), 2 * (2 * math.cos(a0) + math.sin(a0)), 0.0, 0.0, 5.0, 6.0], atol=1e-12)


def test_the_plain_scaled_frequencies_blend_between_the_two_ends():
    """Fast dimensions keep their frequency, slow ones are divided by the factor, the ramp between them is linear."""
    f0 = P.plain_frequencies(16, 1e4)
    f, mag = P.yarn_frequencies(16, 1e4, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    dim = lambda t: 16 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(1e4))      # noqa: E731
    lo, hi = max(math.floor(dim(8.0)), 0), min(math.ceil(dim(1.0)), 15)
    assert (lo, hi) == (0, 3)
    np.testing.assert_allclose(f[0], f0[0])
    np.testing.assert_allclose(f[3:], f0[3:] / 4.0)
    np.testing.assert_allclose(f[1], f0[1] * (1 - 1 / 3) + f0[1] / 4 / 3)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert P.yarn_frequencies(16, 1e4, None)[1] == 1.0


def test_the_plain_router_keeps_the_best_groups_and_does_not_renormalise():
    z = np.log(np.array([[0.05, 0.30, 0.25, 0.02, 0.28, 0.10]]))           # three groups of two: maxima 0.30, 0.25, 0.28
    chosen, weights = P.route(z, top=2, count=3, keep=2)
    assert chosen.tolist() == [[1, 4]]                                      # group 1 (0.25, 0.02) is dropped
    np.testing.assert_allclose(weights, [[0.30, 0.28]])
    chosen, weights = P.route(z, top=3, count=1, keep=1)
    assert chosen.tolist() == [[1, 4, 2]]


def test_the_plain_expert_clamps_before_it_gates():
    w = {"e.gate": np.array([[10.0], [-10.0]]), "e.up": np.array([[10.0], [-10.0]]), "e.down": np.eye(2)}
    out = P.expert(w, "e.", np.array([[1.0]]), 2.0)[0]
    g = np.array([2.0, -10.0])                               # the gate is cut from above only
    np.testing.assert_allclose(out, g * P.sigmoid(1.702 * g) * (np.array([2.0, -2.0]) + 1.0))


def test_the_plain_linear_attention_forgets_by_channel():
    """One head, two key channels, one of which forgets everything at every token: the kept channel answers with the sum
    of what was written under it, the other with the last value only."""
    T, D = 3, 8
    h = np.eye(T, D)
    W = {"m." + n: np.zeros(s) for n, s in (("q", (2, D)), ("k", (2, D)), ("v", (1, D)), ("g", (1, D)), ("a1", (1, D)), ("a2", (2, 1)))}
    W.update({"m.a2.b": np.array([60.0, -60.0]), "m.norm": np.ones(1), "m.o": np.eye(1)})
    W["m.k"][:, :] = 1.0
    W["m.v"][0, :3] = [1.0, 2.0, 4.0]
    W["m.q"][0, 1], W["m.q"][1, 2] = 1.0, 1.0               # token 1 asks channel 0, token 2 channel 1
    m = {"heads": 1, "dim": 2, "vdim": 1, "tau": 1.0}
    T_, H, dk = 3, 1, 2
    q = (h @ W["m.q"].T).reshape(T_, H, dk) * dk ** -0.5
    z = (h @ W["m.a1"].T) @ W["m.a2"].T + W["m.a2.b"]
    alpha = P.sigmoid(z)
    np.testing.assert_allclose(alpha[0], [1.0, 0.0], atol=1e-20)
    # walk by hand: S[c] after token t
    S = np.zeros(2)
    seen = []
    for t, v in enumerate([1.0, 2.0, 4.0]):
        S = alpha[t] * S + v
        seen.append(S @ q[t, 0])
    np.testing.assert_allclose(seen, [0.0, 3.0 * 2 ** -0.5, 4.0 * 2 ** -0.5])
    W["m.g"][0, :] = 30.0                                    # silu(30) = 30 up to 1e-11
    out = P.gla_mixer(m, W, "m.", h, 1e-30)                  # the norm over one value leaves its sign
    np.testing.assert_allclose(out[:, 0], [0.0, 30.0, 30.0], atol=1e-9)
