"""Nutatar through the engine, against the plain float64 model: whole prompts, token-by-token decoding, prompts cut
into portions, batches of unequal requests, slots and pages used again, long decoding across pages and windows, sharp
scores that rest on single keys at the edges, greedy generation through the library's entry point."""
import copy

import numpy as np
import pytest

import qstream_b200 as qs
import plain_nutatar as P
from nutatar_util import (CONFIGS, assert_close, attention_layer, gla_layer, latent_layer, load_plain, logits_error,
                          make_folder, make_weights, model as model_config, write_folder)
from util import random_tokens

pytestmark = pytest.mark.gpu

CASES = [(which, dtype) for dtype in ("float32", "bfloat16") for which in "ABC"]
SINGLE = [(which, dtype) for dtype in ("float32", "bfloat16") for which in "TGLM"]
_REFS = {}


def reference(key, pcfg, w, toks):
    """The plain model's logits of a sequence, computed once per (model, sequence)."""
    k = (key, tuple(toks))
    if k not in _REFS:
        _REFS[k] = P.forward(pcfg, w, toks)
    return _REFS[k]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(key, plain config, plain weights, library model) per configuration and type, made once."""
    made = {}

    def get(which, dtype):
        if (which, dtype) not in made:
            folder, _ = make_folder(tmp_path_factory.mktemp("nutatar"), which, dtype)
            pcfg, w = load_plain(folder)
            made[which, dtype] = ((which, dtype), pcfg, w, qs.load_model(folder, dtype=dtype, device="cuda"))
        return made[which, dtype]
    return get


def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_layer_by_layer(models, which):
    """The residual stream after every layer, in 32-bit."""
    key, pcfg, w, model = models(which, "float32")
    toks = random_tokens(np.random.default_rng(0), 90, pcfg["vocab"])
    _, after = P.forward(pcfg, w, toks, want_layers=True)
    engine = qs.Engine(model, max_tokens=256, max_batch=1, use_graphs=False)
    got = []

    def watched(block, forward):
        def run(x, step, cache_id):
            x = forward(x, step, cache_id)
            got.append(step.pending.apply(x.clone()))       # the layer's last branch is still pending: add it to a copy
            return x
        return run
    for block in model.blocks:
        block.forward = watched(block, block.forward)
    try:
        slot = engine.acquire()
        engine.step([slot], [toks], [[len(toks) - 1]])
        engine.release(slot)
    finally:
        for block in model.blocks:
            del block.forward
    assert len(got) == len(after)
    for i, (g, ref) in enumerate(zip(got, after)):      # typical rows are off by 1e-6, single ones (a norm of small values) by 6e-5
        err = np.abs(g.cpu().numpy() - ref).max(1) / np.abs(ref).max()
        assert err.max() <= 2e-4 and np.median(err) <= 5e-6, f"layer {i} ({pcfg['layers'][i]['type']}): {err.max():.3e}, median {np.median(err):.3e} of the largest value"


@pytest.mark.parametrize("which,dtype", CASES + SINGLE)
def test_whole_prompts(models, which, dtype):
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=512, max_batch=2)
    rng = np.random.default_rng(1)
    for n in (1, 2, 33, 64, 65, 389):       # from 256 tokens on the linear attention cuts the prompt into chunks
        toks = random_tokens(rng, n, pcfg["vocab"])
        slot = engine.acquire()
        got = engine.step([slot], [toks], [all_places(n)]).cpu().numpy()
        engine.release(slot)
        assert_close(got, reference(key, pcfg, w, toks), dtype, f"{n} tokens")
    engine.check_status()
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", CASES + SINGLE)
@pytest.mark.parametrize("graphs", [True, False])
def test_token_by_token_equals_the_prompt(models, which, dtype, graphs):
    """The first tokens of a sequence one by one from an empty state (fewer than a window holds), then on across a
    page border and every window's edge."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2, use_graphs=graphs)
    toks = random_tokens(np.random.default_rng(2), 140, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([slot], [[t]], [[0]]).cpu().numpy()[0] for t in toks]
    engine.release(slot)
    assert_close(np.stack(got), ref, dtype, "one by one")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 65])
def test_portions(models, which, dtype, portion):
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2)
    toks = random_tokens(np.random.default_rng(3), 150, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = []
    for a in range(0, len(toks), portion):
        piece = toks[a:a + portion]
        got.append(engine.step([slot], [piece], [all_places(len(piece))]).cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, f"portions of {portion}")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_a_long_prompt_in_long_portions(models, which, dtype):
    """Portions beyond 256 tokens run the linear attention's chunks from a state that earlier portions left; the
    windows of attention are counted from the sequence's start, not the portion's."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=1024, max_batch=1)
    toks = random_tokens(np.random.default_rng(9), 700, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([slot], [toks[a:b]], [all_places(b - a)]).cpu().numpy() for a, b in ((0, 300), (300, 301), (301, 700))]
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, "portions of 300, 1 and 399")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
def test_batches_of_unequal_requests_and_reused_slots(models, which, dtype):
    """Prompts of unequal lengths in one step, then one token each until the shorter ones end; a second batch
    takes the slots and pages the first gave back (fewer pages than the two batches need together)."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=3)
    rng = np.random.default_rng(4)
    for lens, prompt in (((130, 1, 67), (100, 1, 40)), ((64, 129, 3), (33, 128, 2)), ((300, 20, 5), (290, 3, 1))):
        reqs = [random_tokens(rng, n, pcfg["vocab"]) for n in lens]
        refs = [reference(key, pcfg, w, t) for t in reqs]
        slots = [engine.acquire() for _ in reqs]
        got = [[] for _ in reqs]
        first = engine.step(slots, [t[:p] for t, p in zip(reqs, prompt)], [all_places(p) for p in prompt]).cpu().numpy()
        at = 0
        for i, p in enumerate(prompt):
            got[i].append(first[at:at + p])
            at += p
        pos = list(prompt)
        live = list(range(len(reqs)))
        for i in [i for i in live if pos[i] == len(reqs[i])]:       # a request that was all prompt
            engine.release(slots[i])
            live.remove(i)
        while live:
            out = engine.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], [[0]] * len(live)).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(reqs[i])]:
                engine.release(slots[i])
                live.remove(i)
        for i, ref in enumerate(refs):
            assert_close(np.concatenate(got[i]), ref, dtype, f"request {i} of lengths {lens}")
        engine.cache.check()
    engine.check_status()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_long_decoding(models, which, dtype):
    """300 tokens one by one after a short prompt: across page borders, every window several times over
    (pages fall out of the windows and are handed out again) and the 256-token border at which the engine changes
    to another captured step; a second sequence runs along and ends early."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=2)
    rng = np.random.default_rng(5)
    a, b = random_tokens(rng, 330, pcfg["vocab"]), random_tokens(rng, 90, pcfg["vocab"])
    ra, rb = reference(key, pcfg, w, a), reference(key, pcfg, w, b)
    sa, sb = engine.acquire(), engine.acquire()
    first = engine.step([sa, sb], [a[:30], b[:5]], [[29], [4]]).cpu().numpy()
    ga, gb = [first[0]], [first[1]]
    for i in range(300):
        both = 5 + i < len(b)
        out = engine.step([sa, sb] if both else [sa], [[a[30 + i]], [b[5 + i]]] if both else [[a[30 + i]]]).cpu().numpy()
        ga.append(out[0])
        if both:
            gb.append(out[1])
        elif sb is not None:
            engine.release(sb)
            sb = None
    engine.release(sa)
    assert_close(np.stack(ga), ra[29:], dtype, "long sequence")
    assert_close(np.stack(gb), rb[4:], dtype, "short sequence")
    engine.check_status()
    engine.cache.check()


# Sharp scores: with a large factor on q.k a query's softmax rests on one or two of the keys it sees, so a window being
# one place off, a key read from the wrong page or a sink left out moves many rows' logits by much of their spread;
# decays close to one let the first tokens weigh on the last ones.
def sharp_config(window=23, wide=70, factor=1.0):
    return model_config(80, 64, 1e-5, 2.0, [
        attention_layer(4, 2, 8, window, 3.0 * factor, rot=(4, 1e3), mlp=None),
        latent_layer(3, 8, 8, 16, 24, 16, 2.0 * factor, (8, 1e3), (2.0, 32, 4.0, 1.0), mlp=None),
        gla_layer(2, 16, 16, 64.0, mlp=None),
        attention_layer(8, 4, 8, wide, 2.5 * factor, rot=(8, 1e4), mlp=None)])


def sharp_weights(cfg, seed=11, gain_all=1.0):
    weights = make_weights(cfg, seed, gain_all=gain_all)
    weights["l1.mix.sink"] = np.array([3.0, 1.0, 4.0], dtype=np.float32)               # of the order of the largest scores
    weights["l2.mix.a2.b"] = np.full_like(weights["l2.mix.a2.b"], 5.0)                 # forgets a ten-thousandth per token
    return weights


def plain_logits(tmp_path, name, cfg, weights, toks, dtype):
    pcfg, w = load_plain(write_folder(tmp_path / name, cfg, weights, dtype))
    return P.forward(pcfg, w, toks)


def test_the_sharp_model_shows_every_edge(tmp_path):
    """The plain model itself: each window moved by one place, the learned sink left out, and the sequence's first
    page cut off change a good part of the rows by far more than the limits the library is held to below."""
    cfg, toks = sharp_config(), random_tokens(np.random.default_rng(12), 330, 80)
    weights = sharp_weights(cfg)
    ref = plain_logits(tmp_path, "ref", cfg, weights, toks, "float32")
    for what, other in (("window + 1", sharp_config(window=24)), ("window - 1", sharp_config(window=22)),
                        ("wide + 1", sharp_config(wide=71)), ("wide - 1", sharp_config(wide=69))):
        e = logits_error(plain_logits(tmp_path, what.replace(" ", ""), other, weights, toks, "float32"), ref)
        assert (e > 0.03).sum() >= 30, (what, (e > 0.03).sum())
    no_sink = dict(weights)
    no_sink["l1.mix.sink"] = np.full(3, -80.0, dtype=np.float32)
    e = logits_error(plain_logits(tmp_path, "nosink", cfg, no_sink, toks, "float32"), ref)
    assert (e > 0.03).sum() >= 100
    cut = plain_logits(tmp_path, "cut", cfg, weights, toks[64:], "float32")
    assert np.median(logits_error(cut[-100:], ref[-100:])) > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("prompt", [200, 64, 3])
def test_sharp_edges_in_prompts_and_in_decoding(tmp_path, dtype, prompt):
    """A prompt, then token by token: every edge of `sharp_config` passes over keys of the prompt and over decoded
    ones (the window of 23 many times, the window of 70 across pages)."""
    # bfloat16 rounds large scores coarsely: smaller matrices there
    cfg = sharp_config(factor=1.0)
    folder = write_folder(tmp_path / "sharp", cfg, sharp_weights(cfg, gain_all=1.0 if dtype == "float32" else 0.5), dtype)
    pcfg, w = load_plain(folder)
    toks = random_tokens(np.random.default_rng(12), 330, cfg["vocab"])
    ref = P.forward(pcfg, w, toks)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    engine = qs.Engine(model, max_tokens=512, max_batch=2)
    slot = engine.acquire()
    got = [engine.step([slot], [toks[:prompt]], [all_places(prompt)]).cpu().numpy()]
    got += [engine.step([slot], [[t]], [[0]]).cpu().numpy() for t in toks[prompt:]]
    engine.release(slot)
    e = logits_error(np.concatenate(got), ref)
    if dtype == "float32":
        assert e.max() <= 2e-3 and np.median(e) <= 1e-4, (e.max(), int(e.argmax()), np.median(e))
    else:                                               # sharp scores amplify the rounding of q and k as well
        assert np.median(e) <= 0.05 and np.quantile(e, 0.95) <= 0.2, (np.median(e), np.quantile(e, 0.95), e.max(), int(e.argmax()))
    engine.check_status()
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", CASES)
def test_greedy_generation_through_the_entry_point(models, which, dtype):
    """More requests than slots, so batches follow one another through the generation loop and the scheduler
    hands slots on.  Every token must be the plain model's choice given the tokens before it."""
    key, pcfg, w, model = models(which, dtype)
    rng = np.random.default_rng(6)
    prompts = [random_tokens(rng, n, pcfg["vocab"]) for n in (5, 1, 40, 2, 66)]
    engine = qs.Engine(model, max_tokens=64 * 6, max_batch=2)
    res = qs.generate(engine, prompts, max_new_tokens=8, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert len(res.batches) >= 3 and all(len(t) == 8 for t in res.tokens)
    for prompt, got in zip(prompts, res.tokens):
        toks = list(prompt)
        for g in got:
            logits = P.forward(pcfg, w, toks)[-1]
            best = int(np.argmax(logits))
            if g != best:
                assert dtype == "bfloat16" and logits[best] - logits[g] < 0.1 * (logits.max() - logits.min()), (toks, g, best)
            toks.append(g)
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


def test_a_model_made_from_a_seed_runs_and_saves(tmp_path):
    """`CausalLM.random` and the folder that `write_model_folder` writes hold the same model."""
    cfg = copy.deepcopy(CONFIGS["A"])
    for layer in cfg["layers"]:                          # the bottleneck's rank: the library's key for a model made here
        if layer["type"] == "gla":
            layer["mixer"]["decay_rank"] = 6
    config = qs.config_from_dict(cfg)
    scales = qs.InitScales(0.2, 0.1, 0.1)
    folder = qs.write_model_folder(tmp_path / "made", config, seed=3, dtype="float32", scales=scales)
    pcfg, w = load_plain(folder)
    assert w["l0.mix.a1"].shape[0] == 6 and w["l0.mix.a2"].shape[1] == 6
    toks = random_tokens(np.random.default_rng(7), 50, pcfg["vocab"])
    ref = P.forward(pcfg, w, toks)
    for model in (qs.load_model(folder, dtype="float32"), qs.CausalLM.random(config, 3, "float32", "cuda", scales)):
        engine = qs.Engine(model, max_tokens=128, max_batch=1)
        slot = engine.acquire()
        assert_close(engine.step([slot], [toks], [all_places(50)]).cpu().numpy(), ref, "float32", "seeded model")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_long_requests(models, dtype):
    """Sizes that the tensor-core kernels take, requests of up to 900 tokens: a whole prompt; a prompt and 260 tokens
    one by one (the windows pass over decoded tokens, pages fall out); three unequal
    requests in one batch, decoded together until each ends."""
    key, pcfg, w, model = models("E", dtype)
    rng = np.random.default_rng(21)
    reqs = [random_tokens(rng, n, pcfg["vocab"]) for n in (900, 300, 70)]
    refs = [reference(key, pcfg, w, t) for t in reqs]
    engine = qs.Engine(model, max_tokens=64 * 24, max_batch=3)
    slot = engine.acquire()
    got = engine.step([slot], [reqs[0]], [all_places(900)]).cpu().numpy()
    engine.release(slot)
    assert_close(got, refs[0], dtype, "whole")
    slot = engine.acquire()
    got = [engine.step([slot], [reqs[0][:640]], [all_places(640)]).cpu().numpy()]
    got += [engine.step([slot], [[t]], [[0]]).cpu().numpy() for t in reqs[0][640:]]
    engine.release(slot)
    assert_close(np.concatenate(got), refs[0], dtype, "a prompt, then one by one")
    prompt = (830, 290, 1)
    slots = [engine.acquire() for _ in reqs]
    first = engine.step(slots, [t[:p] for t, p in zip(reqs, prompt)], [[p - 1] for p in prompt]).cpu().numpy()
    rows = [[first[i]] for i in range(3)]
    pos, live = list(prompt), [0, 1, 2]
    while live:
        for i in [i for i in live if pos[i] == len(reqs[i])]:
            engine.release(slots[i])
            live.remove(i)
        if not live:
            break
        out = engine.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], [[0]] * len(live)).cpu().numpy()
        for j, i in enumerate(live):
            rows[i].append(out[j])
            pos[i] += 1
    for i in range(3):
        assert_close(np.stack(rows[i]), refs[i][prompt[i] - 1:], dtype, f"request {i} in a batch")
    engine.check_status()
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_weighs_on_the_last_tokens(tmp_path, dtype):
    """Latent attention alone (a layer and one that reads its latents): one early token whose embedding is six times
    the others' gives a key that many later queries rest on (or shun).  The plain model first shows that the last
    rows change when that token is another one; the library must agree with it 700 tokens on, in a whole prompt, in
    portions that start behind the token's page, and token by token."""
    cfg = CONFIGS["L"]
    weights = make_weights(cfg, 5, gain_all=1.0 if dtype == "float32" else 0.5)
    special = 7
    weights["embed"][special] *= 6.0
    folder = write_folder(tmp_path / "far", cfg, weights, dtype)
    pcfg, w = load_plain(folder)
    rng = np.random.default_rng(31)
    toks = [int(t) for t in rng.integers(8, cfg["vocab"], 700)]
    toks[2] = special
    ref = P.forward(pcfg, w, toks)
    other = list(toks)
    other[2] = 9
    moved = logits_error(P.forward(pcfg, w, other)[-100:], ref[-100:])
    assert (moved > 0.03).sum() >= 50, (moved > 0.03).sum()
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    engine = qs.Engine(model, max_tokens=1024, max_batch=2)
    slot = engine.acquire()
    got = engine.step([slot], [toks], [all_places(700)]).cpu().numpy()
    engine.release(slot)
    assert_close(got, ref, dtype, "whole")
    slot = engine.acquire()
    got = [engine.step([slot], [toks[a:b]], [all_places(b - a)]).cpu().numpy() for a, b in ((0, 70), (70, 400), (400, 640))]
    got += [engine.step([slot], [[t]], [[0]]).cpu().numpy() for t in toks[640:]]
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, "portions, then one by one")
    engine.check_status()
