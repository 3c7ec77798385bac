"""Prefill and decode throughput of a Lutelorn model beside a GPT-J model of equal size, and the kernels that
Lutelorn adds, each against its roofline (`bench.py --design lutelorn`); the same for a Fofinex model beside a
Lutelorn model, the library's closest design (a 32-bit stream, matrix-state mixers among attention layers), with
the kernels that Fofinex adds (`bench.py --design fofinex`); and for a Sefuvik model beside a Lutelorn model
(`bench.py --design sefuvik`); and for a Nutatar model beside a Fofinex model, the library's closest design (attention
through a latent, routed experts, a matrix-state mixer, branches normed on their way into a 32-bit stream)
(`bench.py --design nutatar`).

Sizes resemble a real model's layers: a width, heads of 128 (attention: a quarter as many key heads), a gated
feed-forward of 8/3 width on every layer, the mixers in the order lightning, attention, lightning, wkv; the
GPT-J model beside it has the same width, number of layers and heads and a feed-forward of 4 width, which gives
nearly the same number of weights per layer.  Weights are random, tokens uniform.

Timing: CUDA events on the launching stream, three warm-up runs, a buffer larger than L2 written between timed
kernels (per-kernel table) or steps that read more than L2 holds (models).
"""
from __future__ import annotations

import json

SIZES = {"w2048": dict(width=2048, layers=8), "w4096": dict(width=4096, layers=4)}
VOCAB = 32000
FP32_LANES_PER_SM, SMS = 128, 148


def lutelorn_config(width: int, layers: int) -> dict:
    heads = width // 128
    ff = (width * 8 // 3 + 255) // 256 * 256
    mlp = {"kind": "dense", "ff": ff}
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * i / max(heads - 1, 1)) for i in range(heads)]
    kinds = {
        "lightning": {"type": "lightning", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": decay}, "mlp": mlp},
        "attention": {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128,
                                                     "rot": {"dims": 64, "base": 10000.0}, "scale": 128 ** -0.5, "softcap": 50.0,
                                                     "v_mix": True}, "mlp": mlp},
        "wkv": {"type": "wkv", "mixer": {"heads": width // 64, "dim": 64, "decay_rank": 64}, "mlp": mlp},
    }
    order = ["lightning", "attention", "lightning", "wkv"]
    return {"architecture": "Lutelorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31337, "mul_cur": 7919}},
            "layers": [kinds[order[i % 4]] for i in range(layers)], "max_positions": 8192}


def fofinex_config(width: int, layers: int) -> dict:
    """Heads of 128 values; the matrix memory with keys of 64; the latent of 192 + 64 rotated dims (what the tensor-core
    attention takes as one key head), queries through a latent of 3/4 width; feed-forwards in turn dense (8/3 width)
    and 16 routed experts of 1/3 width, 4 per token out of the best 2 of 4 groups, beside a shared one of 1/2 width."""
    heads = width // 128
    dense = {"kind": "dense", "ff": (width * 8 // 3 + 255) // 256 * 256}
    routed = {"kind": "moe", "expert": {"ff": (width // 3 + 63) // 64 * 64}, "shared": {"ff": width // 2},
              "router": {"experts": 16, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    memory = {"heads": heads, "dim": 64, "vdim": 128, "gate_cap": 15.0}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": width * 3 // 4, "kv_rank": 192, "scale": 192 ** -0.5,
              "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    out = []
    for i in range(layers):
        kind = ("mlstm", "latent_attention", "mlstm", "latent_attention")[i % 4]
        mixer = dict(memory) if kind == "mlstm" else dict(latent)
        if i % 4 == 3:
            mixer["kv_from"] = i - 2                    # every second latent layer reads the latents of the one before
        out.append({"type": kind, "mixer": mixer, "mlp": dense if i % 2 == 0 else routed})
    return {"architecture": "Fofinex", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "layers": out, "max_positions": 8192}


def sefuvik_config(width: int, layers: int) -> dict:
    """Heads of 128; the residual stream in four copies; mixers in the order retention, pair (attention in chunks of
    512 with sinks beside the gated delta rule with four taps and bottlenecks of 64), retention, differential attention
    (half as many heads, each with two maps of 128 and values of 256; a window of 1,024 that keeps the first four
    tokens); a gated feed-forward of 8/3 width on every layer."""
    heads = width // 128
    mlp = {"kind": "dense", "ff": (width * 8 // 3 + 255) // 256 * 256}
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * i / max(heads - 1, 1)) for i in range(heads)]
    kinds = {
        "retention": {"type": "retention", "mlp": mlp,
                      "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": decay, "rot": {"dims": 64, "base": 10000.0}}},
        "parallel": {"type": "parallel", "mlp": mlp, "mixer": {
            "left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "rot": {"dims": 64, "base": 10000.0},
                     "scale": 128 ** -0.5, "mask": {"size": 512}},
            "right": {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64,
                      "gate_rank": 64},
            "left_scale": 0.5, "right_scale": 0.5}},
        "attention": {"type": "attention", "mlp": mlp,
                      "mixer": {"heads": heads // 2, "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 256, "scale": 128 ** -0.5,
                                "diff": 0.3, "mask": {"size": 1024, "keep_first": 4}}},
    }
    order = ["retention", "parallel", "retention", "attention"]
    return {"architecture": "Sefuvik", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "streams": 4,
            "layers": [kinds[order[i % 4]] for i in range(layers)], "max_positions": 8192}


def nutatar_config(width: int, layers: int) -> dict:
    """Heads of 128; mixers in the order latent attention (a latent of 192 + 64 rotated dims, queries through 3/4 width),
    windowed attention (a quarter as many key heads, a window of 1,024), gated linear attention (keys of 64, values of
    128, a bottleneck of 64), latent attention that reads the first one's latents; feed-forwards in turn dense (4 width,
    ungated: as many weights as Fofinex's gated one of 8/3) and 16 gated experts of 1/3 width, 4 per token out of the best
    2 of 4 groups, beside a shared one of 1/2 width."""
    heads = width // 128
    dense = {"kind": "dense", "ff": 4 * width}
    routed = {"kind": "moe", "expert": {"ff": (width // 3 + 63) // 64 * 64, "limit": 7.0}, "shared": {"ff": width // 2, "limit": 7.0},
              "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}}}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": width * 3 // 4, "kv_rank": 192, "scale": 192 ** -0.5,
              "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    windowed = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024},
                "rot": {"dims": 64, "base": 10000.0}}
    linear = {"heads": heads, "dim": 64, "vdim": 128, "tau": 16.0, "decay_rank": 64}
    out = []
    for i in range(layers):
        kind = ("latent_attention", "attention", "gla", "latent_attention")[i % 4]
        mixer = dict({"latent_attention": latent, "attention": windowed, "gla": linear}[kind])
        if i % 4 == 3:
            mixer["kv_from"] = i - 3                    # every second latent layer reads the latents of the one before
        out.append({"type": kind, "mixer": mixer, "mlp": dense if i % 2 == 0 else routed})
    return {"architecture": "Nutatar", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": out,
            "max_positions": 8192}


def gptj_config(width: int, layers: int) -> dict:
    return dict(n_layer=layers, n_embd=width, n_head=width // 128, n_positions=8192, vocab_size=VOCAB, rotary_dim=64,
                n_inner=4 * width, activation_function="gelu_new", layer_norm_epsilon=1e-5, architectures=["GPTJForCausalLM"])


class Timer:
    def __init__(self, torch):
        self.torch = torch
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def kernel(self, fn, repeats=10, warmup=3) -> float:
        """Milliseconds of one call, L2 flushed before each timed call."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        total = 0.0
        for _ in range(repeats):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / repeats


def model_throughput(qs, torch, np, model, vocab, prompt_len, batch, ctx, steps, warmup):
    """Tokens per second of one prompt of `prompt_len` tokens, and of decode steps of `batch` sequences that end at
    a context of `ctx`."""
    from .csrc import ops
    from .engine import TokenFeed
    rng = np.random.default_rng(0)
    engine = qs.Engine(model, max_tokens=max(batch * ctx, prompt_len) + 64, max_batch=batch, max_context=max(ctx, prompt_len))
    times = []
    for _ in range(3 + 3):
        slot = engine.acquire()
        toks = [int(t) for t in rng.integers(0, vocab, prompt_len)]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([slot], [toks])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.release(slot)
    prefill_ms = sum(times[3:]) / 3
    slots = [engine.acquire() for _ in range(batch)]
    start = ctx - steps - warmup
    logits = None
    per = max(1, 4096 // start)
    outs = []
    for i in range(0, batch, per):
        outs.append(engine.step(slots[i:i + per], [[int(t) for t in rng.integers(0, vocab, start)] for _ in slots[i:i + per]]).clone())
    tokens = ops.argmax(torch.cat(outs))
    rows = list(range(batch))

    def one():
        nonlocal tokens
        tokens = ops.argmax(engine.step(slots, TokenFeed(tokens, rows)))
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    engine.check_status()
    ms = a.elapsed_time(b) / steps
    launches = ops.launch_count() - n0
    del engine
    torch.cuda.empty_cache()
    return {"prefill_tokens": prompt_len, "prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(prompt_len * 1e3 / prefill_ms, 1),
            "decode_batch": batch, "decode_context": ctx, "decode_ms": round(ms, 4), "decode_tok_s": round(batch * 1e3 / ms, 1),
            "launches": launches}


def kernel_table(torch, np, pk, width=2048, T=4096, batch=32, ctx=2048):
    """Each kernel of the new parts and the like kernel of the GPT-J parts by itself: milliseconds and the fraction
    of its roofline (copy bandwidth, bfloat16 tensor peak, or 32-bit multiply-add peak of the CUDA cores)."""
    from .csrc import attention_bf16, ops
    t = Timer(torch)
    bf, f32 = torch.bfloat16, torch.float32
    dev = "cuda"
    H, d = width // 128, 128
    G = max(1, H // 4)
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32 = 2.0 * FP32_LANES_PER_SM * SMS * pk.get("sm_max_mhz", 1965.0) * 1e6
    rows = []

    def add(name, like, ms, nbytes=0, flops=0, bound="hbm"):
        peak = {"hbm": hbm, "tensor": tens, "fp32": fp32}[bound]
        done = (nbytes if bound == "hbm" else flops) / (ms * 1e-3)
        rows.append({"kernel": name, "like": like, "ms": round(ms, 4), "bound": bound, "frac": round(done / peak, 4)})

    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)          # noqa: E731
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        x = torch.randn(n_rows, width, device=dev)
        y = torch.randn(n_rows, width, device=dev)
        w = torch.randn(width, device=dev, dtype=bf)
        xb = x.to(bf)
        add(f"rmsnorm {tag}", "layernorm", t.kernel(lambda: ops.rmsnorm(x, w, 1e-6, 1.0, out_dtype=bf)), n_rows * width * 6)
        add(f"rmsnorm + update {tag}", "layernorm", t.kernel(lambda: ops.rmsnorm(x, w, 1e-6, 1.0, out_dtype=bf, update=y, mult=0.0)),
            n_rows * width * 14)
        add(f"layernorm {tag} (GPT-J)", "", t.kernel(lambda: ops.layernorm(xb, w, w, 1e-5, settled=True)), n_rows * width * 4)
        o = torch.randn(n_rows, width, device=dev)
        g = torch.randn(n_rows, width, device=dev, dtype=bf)
        add(f"gated group norm {tag}", "layernorm", t.kernel(lambda: ops.gated_group_norm(o, width, w, g, "sigmoid", 1e-6, bf)),
            n_rows * width * 8)
        mu = torch.rand(5, width, device=dev)
        last = torch.zeros(batch, width, device=dev, dtype=bf)
        slot = i32([0] * n_rows) if tag == "prompt" else i32(list(range(batch)))
        pos = i32(list(range(n_rows))) if tag == "prompt" else i32([ctx - 1] * batch)
        add(f"token shift {tag}", "layernorm", t.kernel(lambda: ops.token_shift(xb, mu, last, slot, pos)), n_rows * width * 12)
        ab = torch.randn(n_rows, 2 * ((width * 8 // 3 + 255) // 256 * 256), device=dev, dtype=bf)     # the models' feed-forward width
        add(f"gated activation {tag}", "(in GPT-J's product)", t.kernel(lambda: ops.gated_act(ab, "silu")), ab.numel() * 3)

    # matrix states: one prompt of T tokens (cut into chunks, as the mixers do from 256 tokens on), and `batch` single tokens
    from .parts.recurrent import CHUNK_TOKENS
    n_chunks = T // CHUNK_TOKENS
    chunks = (i32(list(range(0, T + 1, CHUNK_TOKENS))), i32(list(range(n_chunks))), i32([0, n_chunks]), n_chunks)
    one_start, one_slot = i32([0, T]), i32([0])
    dec_start, dec_slot = i32(list(range(batch + 1))), i32(list(range(batch)))
    for mode, heads, dk in (("decay", H, d), ("wkv", width // 64, 64)):
        n = heads * dk
        q, k, v = (torch.randn(T, n, device=dev, dtype=bf) for _ in range(3))
        state = torch.zeros(batch, heads, dk, dk, device=dev)
        extra = dict(head_decay=torch.full((heads,), 0.99, device=dev)) if mode == "decay" else \
            dict(decay_logits=torch.randn(T, n, device=dev), bonus=torch.randn(heads, dk, device=dev, dtype=bf))
        ms = t.kernel(lambda: ops.state_scan(mode, q, k, v, state, one_start, one_slot, 1, heads, dk, dk, chunks=chunks, **extra))
        # the chunks' own part and the part of the state they start from: 2 + 1 multiply-adds per state element and token
        add(f"state scan {mode} prompt {T} (4 kernels)", "attention prompt", ms, flops=6.0 * T * heads * dk * dk, bound="fp32")
        qd, kd, vd = q[:batch], k[:batch], v[:batch]
        if mode == "wkv":
            extra["decay_logits"] = extra["decay_logits"][:batch]
        ms = t.kernel(lambda: ops.state_scan(mode, qd, kd, vd, state, dec_start, dec_slot, batch, heads, dk, dk, **extra))
        add(f"state scan {mode} decode {batch}", "attention decode", ms, 2 * state.numel() * 4)

    # attention: prompt of T tokens, decode of `batch` tokens at context ctx; GPT-J's form (values as wide as keys, no
    # cap, no gate, a key head per query head) and Lutelorn's (grouped keys, capped scores, gate)
    dslot, dpos = i32(list(range(batch))), i32([ctx - 1] * batch)
    for name, g_heads, cap, gated in (("(GPT-J)", H, 0.0, False), ("capped, gated, grouped", G, 50.0, True)):
        n_pages = batch * ctx // 64
        kc = torch.randn(n_pages, g_heads, 64, d, device=dev, dtype=bf)
        vc = torch.randn(n_pages, g_heads, 64, d, device=dev, dtype=bf)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, ctx // 64)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        q = torch.randn(T, H * d, device=dev, dtype=bf)
        gate = torch.randn(T, H * d, device=dev, dtype=bf) if gated else None
        tl = min(T, ctx)
        tiles = torch.tensor([(a, min(128, tl - a), a, 0) for a in range(0, tl, 128)][::-1], dtype=torch.int32, device=dev)
        qp, gp = q[:tl], (gate[:tl] if gated else None)
        ms = t.kernel(lambda: attention_bf16.prefill(qp, H, g_heads, d, d ** -0.5, 0, tiles, table, 64, kc, vc, status,
                                                     softcap=cap, gate=gp))
        add(f"attention prompt {tl} {name}", "" if not gated else "attention prompt (GPT-J)", ms, flops=4.0 * H * d * tl * tl / 2, bound="tensor")
        qd = q[:batch].contiguous()
        gd = gate[:batch].contiguous() if gated else None
        ms = t.kernel(lambda: attention_bf16.decode(qd, H, g_heads, d, d ** -0.5, 0, dslot, dpos, table, 64, kc, vc, ctx, status,
                                                    softcap=cap, gate=gd))
        add(f"attention decode {batch} x {ctx} {name}", "" if not gated else "attention decode (GPT-J)", ms, batch * ctx * g_heads * d * 4)
    return rows


def kernel_table_fofinex(torch, np, pk, width=2048, T=4096, batch=32, ctx=2048):
    """The kernels that Fofinex adds, each by itself beside the like kernel of the Lutelorn parts: milliseconds and the
    fraction of its roofline."""
    from .csrc import attention_bf16, ops
    from .parts.recurrent import CHUNK_TOKENS
    t = Timer(torch)
    bf = torch.bfloat16
    dev = "cuda"
    H = width // 128
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32 = 2.0 * FP32_LANES_PER_SM * SMS * pk.get("sm_max_mhz", 1965.0) * 1e6
    rows = []

    def add(name, like, ms, nbytes=0, flops=0, bound="hbm"):
        peak = {"hbm": hbm, "tensor": tens, "fp32": fp32}[bound]
        done = (nbytes if bound == "hbm" else flops) / (ms * 1e-3)
        rows.append({"kernel": name, "like": like, "ms": round(ms, 4), "bound": bound, "frac": round(done / peak, 4)})

    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)          # noqa: E731
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        x, y = torch.randn(n_rows, width, device=dev), torch.randn(n_rows, width, device=dev)
        w = torch.randn(width, device=dev, dtype=bf)
        add(f"branch norm + update + norm {tag}", "rmsnorm + update",
            t.kernel(lambda: ops.branch_norm(x, w, 1e-5, True, out_dtype=bf, branch=y, branch_weight=w)), n_rows * width * 14)
        add(f"rmsnorm + update {tag} (Lutelorn)", "", t.kernel(lambda: ops.rmsnorm(x, w, 1e-6, 1.0, out_dtype=bf, update=y, mult=0.0)),
            n_rows * width * 14)
    # the matrix memory: gates, scan (keys of 64, values of 128 and the normaliser's column), output
    dk, dv = 64, 128
    n_chunks = T // CHUNK_TOKENS
    chunks = (i32(list(range(0, T + 1, CHUNK_TOKENS))), i32(list(range(n_chunks))), i32([0, n_chunks]), n_chunks)
    one_start, one_slot = i32([0, T]), i32([0])
    dec_start, dec_slot = i32(list(range(batch + 1))), i32(list(range(batch)))
    raw = torch.randn(T, 2 * H, device=dev)
    m_state = torch.zeros(batch, H, device=dev)
    add(f"mlstm gates prompt {T}", "(none)", t.kernel(lambda: ops.mlstm_gates(raw, 15.0, m_state, one_start, one_slot, 1, H)), T * H * 20)
    add(f"mlstm gates decode {batch}", "(none)", t.kernel(lambda: ops.mlstm_gates(raw[:batch], 15.0, m_state, dec_start, dec_slot, batch, H)), batch * H * 20)
    a, b, m = ops.mlstm_gates(raw, 15.0, m_state, one_start, one_slot, 1, H)
    q, k = (torch.randn(T, H * dk, device=dev, dtype=bf) for _ in range(2))
    v, g = (torch.randn(T, H * dv, device=dev, dtype=bf) for _ in range(2))
    state = torch.zeros(batch, H, dv + 1, dk, device=dev)
    ms = t.kernel(lambda: ops.state_scan("gated", q, k, v, state, one_start, one_slot, 1, H, dk, dv + 1, token_decay=a, token_weight=b,
                                         q_scale=0.125, chunks=chunks))
    add(f"state scan gated prompt {T} (4 kernels)", "state scan decay prompt", ms, flops=6.0 * T * H * dk * (dv + 1), bound="fp32")
    ms = t.kernel(lambda: ops.state_scan("gated", q[:batch], k[:batch], v[:batch], state, dec_start, dec_slot, batch, H, dk, dv + 1,
                                         token_decay=a[:batch], token_weight=b[:batch], q_scale=0.125))
    add(f"state scan gated decode {batch}", "state scan decay decode", ms, 2 * state.numel() * 4)
    hd, n = H, H * 128
    ql, kl, vl = (torch.randn(T, n, device=dev, dtype=bf) for _ in range(3))
    st2 = torch.zeros(batch, hd, 128, 128, device=dev)
    dec = torch.full((hd,), 0.99, device=dev)
    ms = t.kernel(lambda: ops.state_scan("decay", ql, kl, vl, st2, one_start, one_slot, 1, hd, 128, 128, head_decay=dec, chunks=chunks))
    add(f"state scan decay prompt {T} (Lutelorn)", "", ms, flops=6.0 * T * hd * 128 * 128, bound="fp32")
    ms = t.kernel(lambda: ops.state_scan("decay", ql[:batch], kl[:batch], vl[:batch], st2, dec_start, dec_slot, batch, hd, 128, 128, head_decay=dec))
    add(f"state scan decay decode {batch} (Lutelorn)", "", ms, 2 * st2.numel() * 4)
    o = torch.randn(T, H * (dv + 1), device=dev)
    wn = torch.randn(H * dv, device=dev, dtype=bf)
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        add(f"mlstm output {tag}", "gated group norm", t.kernel(lambda: ops.mlstm_output(o[:n_rows], m[:n_rows], wn, g[:n_rows], H, dv, 1e-5, bf)),
            n_rows * H * dv * 8)
        og = torch.randn(n_rows, width, device=dev)
        add(f"gated group norm {tag} (Lutelorn)", "", t.kernel(lambda: ops.gated_group_norm(og, width, wn, g[:n_rows], "sigmoid", 1e-6, bf)),
            n_rows * width * 8)
    # the latent: preparation and cache write, the queries' rotation, the per-head maps, attention with one key head
    r, dr, dn, rq = 192, 64, 128, width * 3 // 4
    from .parts.rotary import scaled_frequencies
    f, mag = scaled_frequencies(dr, 10000.0, dict(factor=4.0, original=4096, fast=32.0, slow=1.0))
    f = f.to(dev)
    n_pages = batch * ctx // 64
    kc = torch.randn(n_pages, 1, 64, r + dr, device=dev, dtype=bf)
    vc = torch.randn(n_pages, 1, 64, r, device=dev, dtype=bf)
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, ctx // 64)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    d = torch.randn(T, rq + r + dr, device=dev, dtype=bf)
    wq, wkv = torch.randn(rq, device=dev, dtype=bf), torch.randn(r, device=dev, dtype=bf)
    qh = torch.randn(T, H * (dn + dr), device=dev, dtype=bf)
    q_abs = torch.zeros(T, H * (r + dr), device=dev, dtype=bf)
    w_uk = torch.randn(H, r, dn, device=dev, dtype=bf)
    for n_rows, tag, slot, pos in ((min(T, ctx), "prompt", i32([0] * min(T, ctx)), i32(list(range(min(T, ctx))))),
                                   (batch, "decode", i32(list(range(batch))), i32([ctx - 1] * batch))):
        add(f"latent prepare {tag}", "rmsnorm", t.kernel(lambda: ops.latent_prepare(d[:n_rows, :rq], wq, rq, d[:n_rows, rq:], wkv, r, dr, dr, f, mag,
                                                                                    1e-5, slot, pos, table, 64, kc, vc, status)),
            n_rows * (2 * rq + 3 * r + 2 * dr) * 2)
        add(f"latent query rotation {tag}", "rmsnorm", t.kernel(lambda: ops.latent_q_rotate(q_abs[:n_rows], qh[:n_rows], H, dn, dr, r, dr, f, mag, slot, pos)),
            n_rows * H * dr * 4)
    add(f"per-head maps decode {batch}", "(none)", t.kernel(lambda: ops.head_linear(q_abs[:batch], qh[:batch], w_uk, H)), w_uk.numel() * 2)
    tl = min(T, ctx)
    tiles = torch.tensor([(s0, min(128, tl - s0), s0, 0) for s0 in range(0, tl, 128)][::-1], dtype=torch.int32, device=dev)
    qa = torch.randn(T, H * (r + dr), device=dev, dtype=bf)
    ms = t.kernel(lambda: attention_bf16.prefill(qa[:tl], H, 1, r + dr, 0.07, 0, tiles, table, 64, kc, vc, status, v_head_dim=r))
    add(f"latent attention prompt {tl}", "attention prompt", ms, flops=2.0 * H * (2 * r + dr) * tl * tl / 2, bound="tensor")
    dslot, dpos = i32(list(range(batch))), i32([ctx - 1] * batch)
    qd = qa[:batch].contiguous()
    ms = t.kernel(lambda: attention_bf16.decode(qd, H, 1, r + dr, 0.07, 0, dslot, dpos, table, 64, kc, vc, ctx, status, v_head_dim=r))
    add(f"latent attention decode {batch} x {ctx}", "attention decode", ms, batch * ctx * (2 * r + dr) * 2)
    G = max(1, H // 4)
    kg, vg = (torch.randn(n_pages, G, 64, 128, device=dev, dtype=bf) for _ in range(2))
    qg = torch.randn(T, H * 128, device=dev, dtype=bf)
    ms = t.kernel(lambda: attention_bf16.prefill(qg[:tl], H, G, 128, 0.09, 0, tiles, table, 64, kg, vg, status))
    add(f"attention prompt {tl}, {G} key heads (Lutelorn's sizes)", "", ms, flops=4.0 * H * 128 * tl * tl / 2, bound="tensor")
    qgd = qg[:batch].contiguous()
    ms = t.kernel(lambda: attention_bf16.decode(qgd, H, G, 128, 0.09, 0, dslot, dpos, table, 64, kg, vg, ctx, status))
    add(f"attention decode {batch} x {ctx}, {G} key heads (Lutelorn's sizes)", "", ms, batch * ctx * G * 128 * 4)
    # routed experts: the router's choice; few tokens through the routing table; many tokens ordered by expert
    E, top, F = 16, 4, (width // 3 + 63) // 64 * 64
    z = torch.randn(T, E + 1, device=dev)
    corr = torch.randn(E, device=dev) * 0.1
    add(f"router choice prompt {T}", "(none)", t.kernel(lambda: ops.moe_route(z, corr, E, top, 4, 2, 2.5, E)), T * (E + 1 + 2 * top + 1) * 4)
    idx, wts, gate = ops.moe_route(z, corr, E, top, 4, 2, 2.5, E)
    w_up, w_down = torch.randn(E, F, width, device=dev, dtype=bf) * 0.02, torch.randn(E, width, F, device=dev, dtype=bf) * 0.02
    h = torch.randn(T, width, device=dev, dtype=bf)
    slot_all = i32([0] * T)
    for nb in (8, batch):
        used = len(set(idx[:nb].flatten().tolist()))
        ms = t.kernel(lambda: ops.moe_experts_indirect(h[:nb], w_up, w_down, idx[:nb].contiguous(), wts[:nb].contiguous(), slot_all[:nb], "relu2"))
        add(f"experts through the routing table, {nb} tokens ({used} experts read)", "weight-streaming product", ms, used * 2 * F * width * 2)

    def grouped():
        from .parts.linear import linear
        offsets, place_token, pair_place = ops.moe_sort(idx, E)
        rows_ = ops.gather_rows(h, place_token)
        yy = torch.empty((rows_.shape[0], width), dtype=torch.float32, device=dev)
        hid = torch.empty((rows_.shape[0], F), dtype=bf, device=dev)
        bounds = offsets.tolist()
        ops.expert_products(hid, rows_, w_up, bounds)
        ops.activate(hid, "relu2")
        ops.expert_products(yy, hid, w_down, bounds)
        return ops.moe_combine(yy, pair_place, wts, slot_all)
    add(f"experts ordered by expert, {T} tokens (sort, gather, {2 * E} products, activation, combine)", "feed-forward products",
        t.kernel(grouped, repeats=5), flops=4.0 * T * top * F * width, bound="tensor")
    wg = torch.randn(2 * 5632, width, device=dev, dtype=bf) * 0.02
    from .parts.linear import linear as lin
    add(f"gate and up product, {T} tokens (Lutelorn's feed-forward)", "", t.kernel(lambda: lin(h, wg)), flops=2.0 * T * wg.shape[0] * width, bound="tensor")
    return rows


def kernel_table_sefuvik(torch, np, pk, width=2048, T=4096, batch=32, ctx=2048):
    """The kernels that Sefuvik adds, each by itself beside the like kernel of the Lutelorn parts: milliseconds and the
    fraction of its roofline."""
    from .csrc import attention_bf16, ops
    from .parts.recurrent import CHUNK_TOKENS
    from .parts.rotary import _table
    t = Timer(torch)
    bf, f32 = torch.bfloat16, torch.float32
    dev = "cuda"
    H, d, S = width // 128, 128, 4
    G = max(1, H // 4)
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32 = 2.0 * FP32_LANES_PER_SM * SMS * pk.get("sm_max_mhz", 1965.0) * 1e6
    rows = []

    def add(name, like, ms, nbytes=0, flops=0, bound="hbm"):
        peak = {"hbm": hbm, "tensor": tens, "fp32": fp32}[bound]
        done = (nbytes if bound == "hbm" else flops) / (ms * 1e-3)
        rows.append({"kernel": name, "like": like, "ms": round(ms, 4), "bound": bound, "frac": round(done / peak, 4)})

    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)          # noqa: E731
    # the stream in four copies: a sublayer's write, the next one's read and its norm in one pass
    mix, w_in, w_out = torch.randn(S, S, device=dev), torch.randn(S, device=dev), torch.randn(S, device=dev)
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        xs, y = torch.randn(n_rows, S * width, device=dev), torch.randn(n_rows, width, device=dev)
        x1, w, ls = torch.randn(n_rows, width, device=dev), torch.randn(width, device=dev, dtype=bf), torch.randn(width, device=dev, dtype=bf)
        add(f"stream of {S} copies: write + read + norm {tag}", "rmsnorm + update",
            t.kernel(lambda: ops.hyper_mix_norm(xs, S, width, y=y, layer_scale=ls, mix=mix, out_weights=w_out, in_weights=w_in,
                                                norm_weight=w, offset=1.0, eps=1e-5, out_dtype=bf)), n_rows * width * (8 * S + 6))
        add(f"rmsnorm + update {tag} (Lutelorn)", "", t.kernel(lambda: ops.rmsnorm(x1, w, 1e-6, 1.0, out_dtype=bf, update=y, mult=0.0)),
            n_rows * width * 14)
    # attention in chunks with sinks (grouped keys), and differential attention in a window that keeps first tokens
    n_pages = batch * ctx // 64
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, ctx // 64)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tl = min(T, ctx)
    pslot, ppos = i32([0] * tl), i32(list(range(tl)))
    dslot, dpos = i32(list(range(batch))), i32([ctx - 1] * batch)
    tiles = torch.tensor([(s0, min(128, tl - s0), s0, 0) for s0 in range(0, tl, 128)][::-1], dtype=torch.int32, device=dev)
    kg, vg = (torch.randn(n_pages, G, 64, d, device=dev, dtype=bf) for _ in range(2))
    q = torch.randn(tl, H * d, device=dev, dtype=bf)
    sink = torch.randn(H, device=dev)
    chunk = 512
    seen = sum(p % chunk + 1 for p in range(tl))
    gate = torch.randn(tl, H * d, device=dev, dtype=bf)
    ms = t.kernel(lambda: attention_bf16.prefill(q, H, G, d, d ** -0.5, 0, tiles, table, 64, kg, vg, status, chunk=chunk, sink=sink, gate=gate))
    add(f"attention in chunks of {chunk} with sinks, gated, prompt {tl}", "attention prompt", ms, flops=4.0 * H * d * seen, bound="tensor")
    ms = t.kernel(lambda: ops.attention(q, H, G, d, d ** -0.5, 0, pslot, ppos, table, 64, kg, vg, status, chunk=chunk, sink=sink))
    add(f"the same by the generic kernel (the 32-bit engine's), prompt {tl}", "", ms, flops=4.0 * H * d * seen, bound="fp32")
    qd, gd = q[:batch].contiguous(), gate[:batch].contiguous()
    ms = t.kernel(lambda: attention_bf16.decode(qd, H, G, d, d ** -0.5, 0, dslot, dpos, table, 64, kg, vg, ctx, status, chunk=chunk,
                                                sink=sink, gate=gd))
    add(f"attention in chunks of {chunk} with sinks, gated, decode {batch} x {ctx}", "attention decode", ms,
        batch * ((ctx - 1) % chunk + 1) * G * d * 4)
    H2, G2, dv2, window, keep = H // 2, max(1, H // 8), 256, 1024, 4
    k2 = torch.randn(n_pages, G2, 64, 2 * d, device=dev, dtype=bf)
    v2 = torch.randn(n_pages, G2, 64, dv2, device=dev, dtype=bf)
    q2 = torch.randn(tl, H2 * 2 * d, device=dev, dtype=bf)
    seen = sum(min(p + 1, window + keep) for p in range(tl))
    ms = t.kernel(lambda: attention_bf16.prefill(q2, H2 * 2, G2, d, d ** -0.5, window, tiles, table, 64, k2, v2, status, v_head_dim=dv2,
                                                 keep_first=keep, maps=2, out_dtype=f32))
    add(f"two maps in a window of {window} + {keep}, prompt {tl}", "attention prompt", ms, flops=2.0 * 2 * H2 * (d + dv2) * seen, bound="tensor")
    q2d = q2[:batch].contiguous()
    ms = t.kernel(lambda: attention_bf16.decode(q2d, H2 * 2, G2, d, d ** -0.5, window, dslot, dpos, table, 64, k2, v2, ctx, status,
                                                v_head_dim=dv2, keep_first=keep, maps=2, out_dtype=f32))
    add(f"two maps in a window of {window} + {keep}, decode {batch} x {ctx}", "attention decode", ms,
        batch * (window + keep) * G2 * (2 * d + dv2) * 2)
    ms = t.kernel(lambda: attention_bf16.prefill(q, H, G, d, d ** -0.5, 0, tiles, table, 64, kg, vg, status))
    add(f"attention prompt {tl}, {G} key heads (Lutelorn's sizes)", "", ms, flops=4.0 * H * d * tl * tl / 2, bound="tensor")
    ms = t.kernel(lambda: attention_bf16.decode(qd, H, G, d, d ** -0.5, 0, dslot, dpos, table, 64, kg, vg, ctx, status))
    add(f"attention decode {batch} x {ctx}, {G} key heads (Lutelorn's sizes)", "", ms, batch * ctx * G * d * 4)
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        a2 = torch.randn(n_rows, H2 * 2 * dv2, device=dev)
        add(f"difference of the maps, unit norm {tag}", "gated group norm",
            t.kernel(lambda: ops.pair_diff_norm(a2, H2, dv2, 0.4, 0.7, 1e-5, bf)), n_rows * H2 * dv2 * 10)
        og, g = torch.randn(n_rows, width, device=dev), torch.randn(n_rows, width, device=dev, dtype=bf)
        wn = torch.randn(width, device=dev, dtype=bf)
        add(f"gated group norm {tag} (Lutelorn)", "", t.kernel(lambda: ops.gated_group_norm(og, width, wn, g, "sigmoid", 1e-6, bf)),
            n_rows * width * 8)
    # retention: q and k leave their product in 32-bit and are rotated in 32-bit; the scan is Lutelorn's
    table_r = _table(64, 10000.0, 8192, dev)
    for n_rows, tag, slot, pos in ((T, "prompt", i32([0] * T), i32(list(range(T)))), (batch, "decode", dslot, dpos)):
        qr = torch.randn(n_rows, H * d, device=dev)
        add(f"rotation of q or k in 32-bit {tag}", "(in attention's cache write)",
            t.kernel(lambda: ops.rope_store(qr, None, None, H, 0, d, 64, table_r, slot, pos, None, 64, None, None, status, settled=True,
                                            half_layout=True)), n_rows * H * d * 8)
    # the gated delta rule: preparation, the convolutions' state, the scan in order
    Gq, taps, nq, nv = max(1, H // 2), 4, max(1, H // 2) * d, H * d
    conv = [torch.randn(n, taps, device=dev, dtype=bf) for n in (nq, nq, nv)]
    held = torch.zeros(batch, taps - 1, 2 * nq + nv, device=dev, dtype=bf)
    a_log = torch.full((H,), -3.0, device=dev)
    n_chunks = T // CHUNK_TOKENS
    chunks = (i32(list(range(0, T + 1, CHUNK_TOKENS))), i32(list(range(n_chunks))), i32([0, n_chunks]), n_chunks)
    one_start, one_slot = i32([0, T]), i32([0])
    dec_start, dec_slot = i32(list(range(batch + 1))), i32(list(range(batch)))
    state = torch.zeros(batch, H, d, d, device=dev)
    for n_rows, tag, slot, pos, starts, slots, n_seq in ((T, "prompt", i32([0] * T), i32(list(range(T))), one_start, one_slot, 1),
                                                         (batch, "decode", dslot, dpos, dec_start, dec_slot, batch)):
        p = torch.randn(n_rows, 2 * nq + nv, device=dev, dtype=bf)
        qq, kk, vv = p[:, :nq], p[:, nq:2 * nq], p[:, 2 * nq:]
        a, b = torch.randn(n_rows, H * d, device=dev), torch.randn(n_rows, H, device=dev)
        add(f"delta rule: convolutions, unit vectors, decays {tag}", "token shift",
            t.kernel(lambda: ops.delta_prepare(qq, kk, vv, *conv, held, a, b, a_log, slot, pos, Gq, H, d, d, d ** -0.5, 1e-6)),
            n_rows * ((2 * nq + nv) * 6 + H * d * 8 + H * 8))
        add(f"delta rule: the convolutions' state {tag}", "(none)",
            t.kernel(lambda: ops.conv_state_update(held, qq, kk, vv, nq, nv, taps, starts, slots, n_seq)), n_seq * (taps - 1) * (2 * nq + nv) * 4)
        qo, ko, vo, decay, beta = ops.delta_prepare(qq, kk, vv, *conv, held, a, b, a_log, slot, pos, Gq, H, d, d, d ** -0.5, 1e-6)
        ms = t.kernel(lambda: ops.state_scan("delta", qo, ko, vo, state, starts, slots, n_seq, H, d, d, key_decay=decay, token_weight=beta,
                                             qk_group=H // Gq), repeats=5)
        if tag == "prompt":                             # decay, S^T k, the write and the read-out: 4 multiply-adds per element and token
            add(f"state scan delta prompt {T} (in order: what short prompts take)", "", ms, flops=8.0 * T * H * d * d, bound="fp32")
            ms = t.kernel(lambda: ops.state_scan("delta", qo, ko, vo, state, starts, slots, n_seq, H, d, d, key_decay=decay, token_weight=beta,
                                                 qk_group=H // Gq, chunks=chunks), repeats=5)
            add(f"state scan delta prompt {T} (chunks: three walks and a prefix)", "state scan decay prompt", ms, flops=8.0 * T * H * d * d, bound="fp32")
        else:
            add(f"state scan delta decode {batch}", "state scan decay decode", ms, 2 * state.numel() * 4)
    ql, kl, vl = (torch.randn(T, H * d, device=dev, dtype=bf) for _ in range(3))
    dec = torch.full((H,), 0.99, device=dev)
    ms = t.kernel(lambda: ops.state_scan("decay", ql, kl, vl, state, one_start, one_slot, 1, H, d, d, head_decay=dec, chunks=chunks))
    add(f"state scan decay prompt {T} (Lutelorn)", "", ms, flops=6.0 * T * H * d * d, bound="fp32")
    ms = t.kernel(lambda: ops.state_scan("decay", ql[:batch], kl[:batch], vl[:batch], state, dec_start, dec_slot, batch, H, d, d, head_decay=dec))
    add(f"state scan decay decode {batch} (Lutelorn)", "", ms, 2 * state.numel() * 4)
    xb, mu, last = torch.randn(T, width, device=dev, dtype=bf), torch.rand(5, width, device=dev), torch.zeros(batch, width, device=dev, dtype=bf)
    add("token shift prompt (Lutelorn)", "", t.kernel(lambda: ops.token_shift(xb, mu, last, i32([0] * T), i32(list(range(T))))), T * width * 12)
    return rows


def kernel_table_nutatar(torch, np, pk, width=2048, T=4096, batch=32, ctx=2048):
    """The kernels (and kernel options) that Nutatar adds, each by itself beside the like kernel of the Fofinex or Lutelorn
    parts: milliseconds and the fraction of its roofline."""
    from .csrc import attention_bf16, ops
    from .parts.recurrent import CHUNK_TOKENS
    from .parts.rotary import _table
    t = Timer(torch)
    bf = torch.bfloat16
    dev = "cuda"
    H, d = width // 128, 128
    G = max(1, H // 4)
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32 = 2.0 * FP32_LANES_PER_SM * SMS * pk.get("sm_max_mhz", 1965.0) * 1e6
    rows = []

    def add(name, like, ms, nbytes=0, flops=0, bound="hbm"):
        peak = {"hbm": hbm, "tensor": tens, "fp32": fp32}[bound]
        done = (nbytes if bound == "hbm" else flops) / (ms * 1e-3)
        rows.append({"kernel": name, "like": like, "ms": round(ms, 4), "bound": bound, "frac": round(done / peak, 4)})

    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)          # noqa: E731
    # the stream: a normed branch joins it and the next sublayer reads it as it is, in one pass
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        x, y = torch.randn(n_rows, width, device=dev), torch.randn(n_rows, width, device=dev)
        w = torch.randn(width, device=dev, dtype=bf)
        add(f"branch norm + update + read {tag}", "branch norm + update + norm",
            t.kernel(lambda: ops.branch_norm(x, None, 1e-5, False, out_dtype=bf, branch=y, branch_weight=w)), n_rows * width * 14)
        add(f"branch norm + update + norm {tag} (Fofinex)", "",
            t.kernel(lambda: ops.branch_norm(x, w, 1e-5, True, out_dtype=bf, branch=y, branch_weight=w)), n_rows * width * 14)
        F = (width // 3 + 63) // 64 * 64
        ab = torch.randn(n_rows * 4, 2 * F, device=dev, dtype=bf)           # four experts' rows per token
        add(f"clamped gated unit {tag}", "gated activation", t.kernel(lambda: ops.clamped_glu(ab, 7.0)), ab.numel() * 3)
        add(f"gated activation {tag} at the experts' sizes", "", t.kernel(lambda: ops.gated_act(ab, "silu")), ab.numel() * 3)
        ab2 = torch.randn(n_rows, 2 * ((width * 8 // 3 + 255) // 256 * 256), device=dev, dtype=bf)
        add(f"gated activation {tag} (Lutelorn)", "", t.kernel(lambda: ops.gated_act(ab2, "silu")), ab2.numel() * 3)
        o, g = torch.randn(n_rows, H * d, device=dev, dtype=bf), torch.randn(n_rows, H, device=dev, dtype=bf)
        add(f"gate per head {tag}", "gated group norm", t.kernel(lambda: ops.gated_group_norm(o, 0, None, g, "sigmoid", 0.0, bf, gate_span=d)),
            n_rows * H * d * 4)
        og, gg, wn = torch.randn(n_rows, width, device=dev), torch.randn(n_rows, width, device=dev, dtype=bf), torch.randn(width, device=dev, dtype=bf)
        add(f"gated group norm {tag} (Lutelorn)", "", t.kernel(lambda: ops.gated_group_norm(og, width, wn, gg, "sigmoid", 1e-6, bf)),
            n_rows * width * 8)
    # gated linear attention: keys of 64, values of 128, a decay per token and key channel taken from its logits in the walk
    dk, dv = 64, 128
    n_chunks = T // CHUNK_TOKENS
    chunks = (i32(list(range(0, T + 1, CHUNK_TOKENS))), i32(list(range(n_chunks))), i32([0, n_chunks]), n_chunks)
    one_start, one_slot = i32([0, T]), i32([0])
    dec_start, dec_slot = i32(list(range(batch + 1))), i32(list(range(batch)))
    q, k = (torch.randn(T, H * dk, device=dev, dtype=bf) for _ in range(2))
    v = torch.randn(T, H * dv, device=dev, dtype=bf)
    z = torch.randn(T, H * dk, device=dev) + 4.0
    state = torch.zeros(batch, H, dv, dk, device=dev)
    ms = t.kernel(lambda: ops.state_scan("gla", q, k, v, state, one_start, one_slot, 1, H, dk, dv, decay_logits=z, decay_power=1 / 16,
                                         q_scale=0.125, chunks=chunks))
    add(f"state scan gla prompt {T} (4 kernels)", "state scan gated prompt", ms, flops=6.0 * T * H * dk * dv, bound="fp32")
    ms = t.kernel(lambda: ops.state_scan("gla", q[:batch], k[:batch], v[:batch], state, dec_start, dec_slot, batch, H, dk, dv,
                                         decay_logits=z[:batch], decay_power=1 / 16, q_scale=0.125))
    add(f"state scan gla decode {batch}", "state scan gated decode", ms, 2 * state.numel() * 4)
    raw = torch.randn(T, 2 * H, device=dev)
    m_state = torch.zeros(batch, H, device=dev)
    a, b, _ = ops.mlstm_gates(raw, 15.0, m_state, one_start, one_slot, 1, H)
    st1 = torch.zeros(batch, H, dv + 1, dk, device=dev)
    ms = t.kernel(lambda: ops.state_scan("gated", q, k, v, st1, one_start, one_slot, 1, H, dk, dv + 1, token_decay=a, token_weight=b,
                                         q_scale=0.125, chunks=chunks))
    add(f"state scan gated prompt {T} (Fofinex)", "", ms, flops=6.0 * T * H * dk * (dv + 1), bound="fp32")
    ms = t.kernel(lambda: ops.state_scan("gated", q[:batch], k[:batch], v[:batch], st1, dec_start, dec_slot, batch, H, dk, dv + 1,
                                         token_decay=a[:batch], token_weight=b[:batch], q_scale=0.125))
    add(f"state scan gated decode {batch} (Fofinex)", "", ms, 2 * st1.numel() * 4)
    # windowed attention: one norm over the whole q and k, rotation and cache write, then a window of 1,024 with a sink
    n_pages = batch * ctx // 64
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, ctx // 64)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tl = min(T, ctx)
    dslot, dpos = i32(list(range(batch))), i32([ctx - 1] * batch)
    tiles = torch.tensor([(s0, min(128, tl - s0), s0, 0) for s0 in range(0, tl, 128)][::-1], dtype=torch.int32, device=dev)
    kg, vg = (torch.randn(n_pages, G, 64, d, device=dev, dtype=bf) for _ in range(2))
    window = 1024
    sink = torch.zeros(H, device=dev)
    rope = _table(64, 10000.0, 8192, dev)
    wq, wk = torch.randn(H * d, device=dev, dtype=bf), torch.randn(G * d, device=dev, dtype=bf)
    for n_rows, tag, slot, pos in ((tl, "prompt", i32([0] * tl), i32(list(range(tl)))), (batch, "decode", dslot, dpos)):
        qk = torch.randn(n_rows, (H + G) * d, device=dev, dtype=bf)

        add(f"norms of q and k, rotation, cache write {tag}", "rotation and cache write",
            t.kernel(lambda: ops.norm_rope_store(qk[:, :H * d], qk[:, H * d:], qk[:, H * d:], wq, wk, 1e-5, H, G, d, 64, rope, slot, pos,
                                                 table, 64, kg, vg, status, half_layout=True)), n_rows * (H * d * 4 + G * d * 6))
        qs_, ks_, vs_ = (torch.randn(n_rows, n * d, device=dev, dtype=bf) for n in (H, G, G))
        add(f"rotation and cache write {tag} (Lutelorn)", "",
            t.kernel(lambda: ops.rope_store(qs_, ks_, vs_, H, G, d, 64, rope, slot, pos, table, 64, kg, vg, status, settled=True)),
            n_rows * (H * d * 4 + G * d * 8))
    qw = torch.randn(tl, H * d, device=dev, dtype=bf)
    seen = sum(min(p + 1, window) for p in range(tl))
    ms = t.kernel(lambda: attention_bf16.prefill(qw, H, G, d, d ** -0.5, window, tiles, table, 64, kg, vg, status, sink=sink))
    add(f"attention in a window of {window} with a sink, prompt {tl}", "attention prompt", ms, flops=4.0 * H * d * seen, bound="tensor")
    qd = qw[:batch].contiguous()
    ms = t.kernel(lambda: attention_bf16.decode(qd, H, G, d, d ** -0.5, window, dslot, dpos, table, 64, kg, vg, ctx, status, sink=sink))
    add(f"attention in a window of {window} with a sink, decode {batch} x {ctx}", "attention decode", ms, batch * window * G * d * 4)
    ms = t.kernel(lambda: attention_bf16.prefill(qw, H, G, d, d ** -0.5, 0, tiles, table, 64, kg, vg, status))
    add(f"attention prompt {tl}, {G} key heads (Lutelorn's sizes)", "", ms, flops=4.0 * H * d * tl * tl / 2, bound="tensor")
    ms = t.kernel(lambda: attention_bf16.decode(qd, H, G, d, d ** -0.5, 0, dslot, dpos, table, 64, kg, vg, ctx, status))
    add(f"attention decode {batch} x {ctx}, {G} key heads (Lutelorn's sizes)", "", ms, batch * ctx * G * d * 4)
    # the latent with a sink per head: Fofinex's kernels with the sink's term (and the rotation by neighbours)
    r, dr, dn, rq = 192, 64, 128, width * 3 // 4
    from .parts.rotary import scaled_frequencies
    f, mag = scaled_frequencies(dr, 10000.0, dict(factor=4.0, original=4096, fast=32.0, slow=1.0))
    f = f.to(dev)
    kc = torch.randn(n_pages, 1, 64, r + dr, device=dev, dtype=bf)
    vc = torch.randn(n_pages, 1, 64, r, device=dev, dtype=bf)
    dd = torch.randn(T, rq + r + dr, device=dev, dtype=bf)
    wql, wkv = torch.randn(rq, device=dev, dtype=bf), torch.randn(r, device=dev, dtype=bf)
    for n_rows, tag, slot, pos in ((tl, "prompt", i32([0] * tl), i32(list(range(tl)))), (batch, "decode", dslot, dpos)):
        for inter, who in ((True, ""), (False, " (Fofinex)")):
            add(f"latent prepare {tag}{who}", "" if who else "latent prepare",
                t.kernel(lambda: ops.latent_prepare(dd[:n_rows, :rq], wql, rq, dd[:n_rows, rq:], wkv, r, dr, dr, f, mag, 1e-5, slot, pos,
                                                    table, 64, kc, vc, status, interleaved=inter)), n_rows * (2 * rq + 3 * r + 2 * dr) * 2)
    qa = torch.randn(tl, H * (r + dr), device=dev, dtype=bf)
    sinks = torch.randn(H, device=dev)
    for sk, who in ((sinks, ""), (None, " (Fofinex)")):
        ms = t.kernel(lambda: attention_bf16.prefill(qa, H, 1, r + dr, 0.07, 0, tiles, table, 64, kc, vc, status, v_head_dim=r, sink=sk))
        add(f"latent attention prompt {tl}{who}", "" if who else "latent attention prompt", ms, flops=2.0 * H * (2 * r + dr) * tl * tl / 2, bound="tensor")
        qad = qa[:batch].contiguous()
        ms = t.kernel(lambda: attention_bf16.decode(qad, H, 1, r + dr, 0.07, 0, dslot, dpos, table, 64, kc, vc, ctx, status, v_head_dim=r, sink=sk))
        add(f"latent attention decode {batch} x {ctx}{who}", "" if who else "latent attention decode", ms, batch * ctx * (2 * r + dr) * 2)
    # routed experts: the router's choice (softmax, group maxima); gated experts through the routing table and ordered by expert
    E, top, F = 16, 4, (width // 3 + 63) // 64 * 64
    zr = torch.randn(T, E + 1, device=dev)
    corr = torch.randn(E, device=dev) * 0.1
    add(f"router choice prompt {T}", "router choice", t.kernel(lambda: ops.moe_route(zr, None, E, top, 4, 2, 1.0, scores="softmax", group_score="max")),
        T * (E + 1 + 2 * top) * 4)
    add(f"router choice prompt {T} (Fofinex)", "", t.kernel(lambda: ops.moe_route(zr, corr, E, top, 4, 2, 2.5, E)), T * (E + 1 + 2 * top + 1) * 4)
    idx, wts, _ = ops.moe_route(zr, None, E, top, 4, 2, 1.0, scores="softmax", group_score="max")
    w_gu = torch.randn(E, 2 * F, width, device=dev, dtype=bf) * 0.02
    w_up, w_down = torch.randn(E, F, width, device=dev, dtype=bf) * 0.02, torch.randn(E, width, F, device=dev, dtype=bf) * 0.02
    h = torch.randn(T, width, device=dev, dtype=bf)
    slot_all = i32([0] * T)
    glu = (7.0, 1.702, 1.0)
    for nb in (8, batch):
        used = len(set(idx[:nb].flatten().tolist()))
        ix, wt = idx[:nb].contiguous(), wts[:nb].contiguous()
        ms = t.kernel(lambda: ops.moe_experts_indirect(h[:nb], w_gu, w_down, ix, wt, slot_all[:nb], None, glu=glu))
        add(f"gated experts through the routing table, {nb} tokens ({used} experts read; 3 kernels)", "experts through the routing table", ms,
            used * 3 * F * width * 2)
        ms = t.kernel(lambda: ops.moe_experts_indirect(h[:nb], w_up, w_down, ix, wt, slot_all[:nb], "relu2"))
        add(f"experts through the routing table, {nb} tokens (Fofinex; 2 kernels)", "", ms, used * 2 * F * width * 2)

    def grouped(gated):
        offsets, place_token, pair_place = ops.moe_sort(idx, E)
        rows_ = ops.gather_rows(h, place_token)
        yy = torch.empty((rows_.shape[0], width), dtype=torch.float32, device=dev)
        hid = torch.empty((rows_.shape[0], 2 * F if gated else F), dtype=bf, device=dev)
        bounds = offsets.tolist()
        ops.expert_products(hid, rows_, w_gu if gated else w_up, bounds)
        hid = ops.clamped_glu(hid, *glu) if gated else ops.activate(hid, "relu2")
        ops.expert_products(yy, hid, w_down, bounds)
        return ops.moe_combine(yy, pair_place, wts, slot_all)
    add(f"gated experts ordered by expert, {T} tokens (sort, gather, {2 * E} products, gated unit, combine)", "experts ordered by expert",
        t.kernel(lambda: grouped(True), repeats=5), flops=6.0 * T * top * F * width, bound="tensor")
    add(f"experts ordered by expert, {T} tokens (Fofinex)", "", t.kernel(lambda: grouped(False), repeats=5), flops=4.0 * T * top * F * width, bound="tensor")
    return rows


def run_nutatar(args, pk) -> int:
    import numpy as np
    import torch
    import qstream_b200 as qs
    out = {"impl": "ours", "design": "nutatar", "beside": "fofinex", "dtype": "bf16", "data": "synthetic token ids, random weights",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    for name, size in SIZES.items():
        entry = {}
        for which, cfg in (("nutatar", nutatar_config(**size)), ("fofinex", fofinex_config(**size))):
            model = qs.CausalLM.random(qs.config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
            r = model_throughput(qs, torch, np, model, VOCAB, 2048, 8, 1024, min(args.steps, 32), max(3, min(args.warmup, 4)))
            r["weights_mb"] = round(model.weight_bytes / 2**20, 1)
            entry[which] = r
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = entry
    out["kernels"] = kernel_table_nutatar(torch, np, pk)
    print(json.dumps(out))
    return 0


def run_fofinex(args, pk) -> int:
    import numpy as np
    import torch
    import qstream_b200 as qs
    out = {"impl": "ours", "design": "fofinex", "beside": "lutelorn", "dtype": "bf16", "data": "synthetic token ids, random weights",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    for name, size in SIZES.items():
        entry = {}
        for which, cfg in (("fofinex", fofinex_config(**size)), ("lutelorn", lutelorn_config(**size))):
            model = qs.CausalLM.random(qs.config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
            r = model_throughput(qs, torch, np, model, VOCAB, 2048, 8, 1024, min(args.steps, 32), max(3, min(args.warmup, 4)))
            r["weights_mb"] = round(model.weight_bytes / 2**20, 1)
            entry[which] = r
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = entry
    out["kernels"] = kernel_table_fofinex(torch, np, pk)
    print(json.dumps(out))
    return 0


def run_sefuvik(args, pk) -> int:
    import numpy as np
    import torch
    import qstream_b200 as qs
    out = {"impl": "ours", "design": "sefuvik", "beside": "lutelorn", "dtype": "bf16", "data": "synthetic token ids, random weights",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    for name, size in SIZES.items():
        entry = {}
        for which, cfg in (("sefuvik", sefuvik_config(**size)), ("lutelorn", lutelorn_config(**size))):
            model = qs.CausalLM.random(qs.config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
            r = model_throughput(qs, torch, np, model, VOCAB, 2048, 8, 1024, min(args.steps, 32), max(3, min(args.warmup, 4)))
            r["weights_mb"] = round(model.weight_bytes / 2**20, 1)
            entry[which] = r
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = entry
    out["kernels"] = kernel_table_sefuvik(torch, np, pk)
    print(json.dumps(out))
    return 0


def run(args, pk) -> int:
    if getattr(args, "design", "") == "fofinex":
        return run_fofinex(args, pk)
    if getattr(args, "design", "") == "sefuvik":
        return run_sefuvik(args, pk)
    if getattr(args, "design", "") == "nutatar":
        return run_nutatar(args, pk)
    import numpy as np
    import torch
    import qstream_b200 as qs
    out = {"impl": "ours", "design": "lutelorn", "beside": "gptj", "dtype": "bf16", "data": "synthetic token ids, random weights",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    for name, size in SIZES.items():
        entry = {}
        for which, cfg in (("lutelorn", lutelorn_config(**size)), ("gptj", gptj_config(**size))):
            model = qs.CausalLM.random(qs.config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
            r = model_throughput(qs, torch, np, model, VOCAB, 2048, 8, 1024, min(args.steps, 32), max(3, min(args.warmup, 4)))
            r["weights_mb"] = round(model.weight_bytes / 2**20, 1)
            entry[which] = r
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = entry
    out["kernels"] = kernel_table(torch, np, pk)
    print(json.dumps(out))
    return 0
