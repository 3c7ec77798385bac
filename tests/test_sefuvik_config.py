"""Sefuvik's configuration: reading, validation, the model it describes; and the plain model's own pieces on inputs
whose results are known."""
import copy
import math

import numpy as np
import pytest

import qstream_b200 as qs
from qstream_b200.config.sefuvik import SefuvikConfig
from qstream_b200.engine.model import declared_tensors
from qstream_b200.errors import QStreamError

import plain_sefuvik as P
from sefuvik_util import CONFIGS, make_weights


@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_the_declared_tensors_are_the_checkpoint_s(which):
    cfg = qs.config_from_dict(CONFIGS[which])
    assert isinstance(cfg, SefuvikConfig)
    decl = declared_tensors(cfg.model_spec())
    weights = make_weights(CONFIGS[which], 0, decay_rank=5, gate_rank=7)
    assert set(decl) == set(weights)
    for name, d in decl.items():
        assert len(d.shape) == weights[name].ndim, name
        assert all(a in (-1, b) for a, b in zip(d.shape, weights[name].shape)), name    # -1: the checkpoint's own size (a rank)
    assert qs.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_one_copy_without_mixing_tensors_is_the_plain_stream():
    cfg = copy.deepcopy(CONFIGS["B"])
    del cfg["streams"]
    decl = declared_tensors(qs.config_from_dict(cfg).model_spec())
    assert not [n for n in decl if ".hc" in n] and "l0.ls1" in decl


def test_the_schedule_gives_a_pair_of_mixers_two_entries():
    spec = qs.config_from_dict(CONFIGS["A"]).model_spec()
    assert [r.cache for r in spec.schedule] == [(0, 1), 2, 3, 4, (5, 6)]
    assert spec.layers[1].ffn is None and spec.layers[0].ffn is not None and spec.head.tied
    left, window = spec.layers[0].mixer.left, spec.layers[1].mixer
    assert (left.chunk, left.window, left.sink, left.gate) == (37, 0, True, True)
    assert (window.window, window.keep_first, window.maps, window.chunk) == (50, 5, 2, 0)
    assert spec.layers[4].mixer.left.position is None and left.position.rotary_dim == 8


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=9), "conv"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=-1), "mask"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, needle):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises(QStreamError) as e:
        qs.config_from_dict(cfg)
    assert needle in str(e.value)


def test_the_plain_visibility_rules():
    """A window of 4 that keeps 2 first tokens, and chunks of 4, at position 9."""
    assert [j for j in range(12) if P.visible_window(9, j, 4, 2)] == [0, 1, 6, 7, 8, 9]
    assert [j for j in range(12) if P.visible_window(9, j, 0, 0)] == list(range(10))
    assert [j for j in range(12) if P.visible_chunk(9, j, 4)] == [8, 9]
    assert [j for j in range(12) if P.visible_chunk(8, j, 4)] == [8]
    assert [j for j in range(12) if P.visible_chunk(7, j, 4)] == [4, 5, 6, 7]


def test_the_plain_softmax_with_a_sink_on_a_hand_made_case():
    """Two equal scores and a sink of the same size: each key weighs a third, and a third of the weight is lost."""
    q, k = np.ones((2, 1, 1)), np.ones((2, 1, 1))
    v = np.array([[[3.0]], [[9.0]]])
    out = P.masked_softmax_attention(q, k, v, 1.0, lambda i, j: j <= i, sink=np.array([1.0]))
    np.testing.assert_allclose(out[:, 0, 0], [1.5, 4.0])


def test_the_plain_rotation_pairs_an_element_with_the_one_half_the_rotated_dims_on():
    x = np.zeros((1, 1, 6))
    x[0, 0] = [1.0, 2.0, 0.0, 0.0, 5.0, 6.0]
    out = P.rotate_half(x, [3], 4, 100.0)[0, 0]
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    np.testing.assert_allclose(out, [math.cos(a0), 2 * math.cos(a1), math.sin(a0), 2 * math.sin(a1), 5.0, 6.0], atol=1e-12)


def test_the_plain_delta_rule_overwrites_what_a_key_held():
    """No decay, a step size of one, unit keys: writing a second value under the same key replaces the first, and an
    orthogonal key reads nothing of it."""
    d, dv = 4, 3
    k1, k2 = np.eye(d)[0], np.eye(d)[1]
    S = np.zeros((d, dv))
    for k, v in ((k1, np.array([1.0, 2.0, 3.0])), (k2, np.array([5.0, 5.0, 5.0])), (k1, np.array([7.0, 8.0, 9.0]))):
        S = S + np.outer(k, 1.0 * (v - S.T @ k))
    np.testing.assert_allclose(S.T @ k1, [7.0, 8.0, 9.0])
    np.testing.assert_allclose(S.T @ k2, [5.0, 5.0, 5.0])
    # the same through the mixer's function: inputs that are one-hot rows pick weight columns
    T, D = 3, 8
    h = np.eye(T, D)
    W = {"m." + n: np.zeros(s) for n, s in (("q", (d, D)), ("k", (d, D)), ("v", (dv, D)), ("b", (1, D)), ("a1", (1, D)),
                                             ("a2", (d, 1)), ("g1", (1, D)), ("g2", (dv, 1)))}
    W.update({"m.q.conv": np.ones((d, 1)), "m.k.conv": np.ones((d, 1)), "m.v.conv": np.ones((dv, 1)), "m.A_log": np.zeros(1),
              "m.dt_bias": np.full(d, -60.0), "m.norm": np.ones(dv), "m.o": np.eye(dv)})
    W["m.b"][0, :] = 60.0                                # beta = 1
    big = 30.0                                           # silu(30) = 30: keys become unit vectors anyway
    W["m.k"][0, 0], W["m.k"][1, 1], W["m.k"][0, 2] = big, big, big
    W["m.q"][0, 2] = big                                 # the last token asks for key 1
    W["m.v"][:, 0], W["m.v"][:, 1], W["m.v"][:, 2] = [1.0, 2.0, 3.0], [5.0, 5.0, 5.0], [7.0, 8.0, 9.0]
    out = P.gated_delta({"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv}, W, "m.", h, 1e-30)
    sv = P.silu(np.array([7.0, 8.0, 9.0]))
    np.testing.assert_allclose(out[2], 0.5 * sv / np.sqrt((sv ** 2).mean()), rtol=1e-6)      # 0.5: the gate, sigmoid(0)
