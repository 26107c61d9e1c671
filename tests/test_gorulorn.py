"""The Gorulorn decoder through the engine against the plain implementation (tests/plain_gorulorn.py).

Small configurations of their own sizes and random weights, made here.  On a GPU the engine runs its CUDA kernels in
float32 and bfloat16; without one the same tests run the host-side logic (configuration, loader, cache manager with
pages and state slots, step function) over the kernels' plain references.  Covered: each mechanism alone; a prompt
whole, against its last tokens decoded one by one, against portions down to two tokens; unequal requests in one batch
against each alone, with pages and slots that are given back and used again; keys just inside and just outside the
window and the kept first tokens, at page borders, with one score made to stand out, in prompts and in decoding; a
token far back that only the kept first keys reach; the sink; the looped span; long decoding from captured steps;
greedy generation through the front end; each new kernel against its plain reference.
"""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_gorulorn as P
from helpers import bf16_round, random_tokens

CUDA = torch.cuda.is_available()
DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]
DTYPES = ["float32", "bfloat16"]


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads=6, kv=2, dim=16, vdim=32, conv=4, window=11, keep=3, rot=8, base=900.0, scale=0.31, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": window, "keep_first": keep},
         "rot": {"dims": rot, "base": base}, "scale": scale}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads=3, dim=16, vdim=24, q_rank=24, kv_rank=40, window=7, scale=0.29, mlp=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window}, "scale": scale}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, loop=None):
    cfg = {"architecture": "Gorulorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


CONFIGS = {
    # everything at once, no two sizes alike: value heads wider and narrower than key heads, three query heads per key
    # head, a latent that is no multiple of 16, two and four taps, several experts per token, a layer without
    # feed-forward, a looped span that starts at the first layer
    "mixed": config([
        latent(mlp=moe(5, 2, 24)),
        attention(mlp=moe(3, 1, 40)),
        attention(heads=2, kv=2, dim=32, vdim=16, conv=2, window=33, keep=1, rot=32, base=10000.0, scale=0.2, mlp=None),
        latent(heads=2, dim=8, vdim=8, q_rank=16, kv_rank=16, window=20, scale=0.4, mlp=moe(4, 4, 16)),
    ], width=48, vocab=97, loop=(0, 2, 2)),
    # each mechanism alone
    "attention_only": config([attention(mlp=None)], width=32, vocab=61),
    "latent_only": config([latent(mlp=None)], width=32, vocab=61),
    "experts_only": config([latent(heads=1, dim=8, vdim=8, q_rank=8, kv_rank=8, window=1, mlp=moe(6, 3, 20))], width=40, vocab=50, eps=1e-6),
    "loop_only": config([latent(heads=2, window=5, mlp=None), attention(heads=2, kv=1, dim=16, vdim=16, conv=3, window=6, keep=2, rot=16, mlp=None)],
                        width=32, vocab=33, loop=(1, 2, 3)),
    # values that a model may happen to make equal or 1: one head, one expert, one tap, no kept tokens, a window of one
    "ones": config([attention(heads=1, kv=1, dim=16, vdim=16, conv=1, window=1, keep=0, rot=2, mlp=moe(1, 1, 8)),
                    latent(heads=1, dim=16, vdim=16, q_rank=16, kv_rank=16, window=1, mlp=None)], width=16, vocab=17, loop=(0, 2, 1)),
}


def make_weights(cfg, seed):
    """Random tensors for every declared name, large enough that each part moves the logits."""
    from litinfer_b200.config import config_from_dict
    from litinfer_b200.models.decoder import declared_params

    g = torch.Generator().manual_seed(seed)
    out = {}
    for p in declared_params(config_from_dict(cfg).to_model_spec()):
        n, shape = p.name, tuple(p.shape)
        r = torch.randn(shape, generator=g)
        last = n.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            out[n] = 1.0 + 0.2 * r
        elif last == "b":
            out[n] = 0.3 * r
        elif last == "conv":
            out[n] = 0.6 * r
        elif last == "sink":
            out[n] = 1.0 + r
        elif n == "loop.step":
            out[n] = 0.7 * r
        elif last == "router":
            out[n] = r * (3.0 / math.sqrt(shape[-1]))
        elif n == "embed":
            out[n] = r
        else:
            out[n] = r * (1.5 / math.sqrt(shape[-1]))
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from litinfer_b200.weights.safetensors_io import write_file

    out = {}
    for k, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp("gorulorn_" + name)
        w = make_weights(cfg, 91 + k)
        (d / "config.json").write_text(json.dumps(cfg))
        write_file(d / "model.safetensors", w)
        out[name] = (d, cfg, w)
    return out


def use_device(device, request):
    if device == "cpu":
        request.getfixturevalue("cpu_kernels")
    return torch.device("cuda:0" if device == "cuda" else "cpu")


def oracle(cfg, w, tokens, dtype):
    w = {k: v.double() for k, v in (bf16_round(w) if dtype == "bfloat16" else w).items()}
    return P.forward(cfg, w, tokens).float()


def assert_close(got, ref, dtype, what):
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std(dim=-1).clamp_min(1e-3)
    worst = int(err.argmax())
    if dtype == "float32":
        assert err.max() <= 2e-4, f"{what}: relative error {float(err.max()):.3e} at row {worst}"
        return
    # bfloat16: activations are rounded to 8 bits at a dozen places a layer.  A row may be unlucky, and a token whose two
    # best experts score within that rounding of each other may go to the other one than in the plain model; most rows may
    # not (a wrong key, window, state or sink moves every row behind it by tens of percent)
    assert err.median() <= 0.05, f"{what}: median relative error {float(err.median()):.3e}"
    assert (err > 0.2).float().mean() <= 0.15, f"{what}: {int((err > 0.2).sum())} of {err.numel()} rows are off, the worst ({worst}) by {float(err.max()):.3e}"


class Run:
    """Feeds requests to a Replayer step by step and keeps every position's logits."""

    def __init__(self, folder, dtype, device, max_tokens, max_live=4, graphs=None):
        from litinfer_b200.engine.replay import Replayer
        from litinfer_b200.models import DecoderModel

        self.model = DecoderModel.from_dir(folder, dtype, device)
        self.rp = Replayer(self.model, max_tokens, max_live=max_live, use_graphs=device.type == "cuda" if graphs is None else graphs)
        self.fed = {}
        self.got = {}
        self.n = 0

    def step(self, entries, end=()):
        """entries: (request, all its tokens, how many of them now)."""
        es = []
        for rid, tokens, count in entries:
            lo = self.fed.get(rid, 0)
            es.append({"id": rid, "tokens": tokens[lo:lo + count], "want": list(range(count))})
            self.fed[rid] = lo + count
        logits = self.rp.step({"step": self.n, "entries": es, "end": list(end)}).float().cpu()
        self.n += 1
        row = 0
        for (rid, tokens, count), e in zip(entries, es):
            self.got.setdefault(rid, []).append(logits[row:row + count])
            row += count
        for rid in end:
            self.fed.pop(rid)

    def logits(self, rid):
        return torch.cat(self.got[rid])


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention_only", "latent_only", "experts_only", "loop_only", "ones"])
def test_each_mechanism_alone(name, dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders[name]
    toks = random_tokens(45, cfg["vocab"], 5)
    ref = oracle(cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 128)
    run.step([("a", toks, 45)], end=["a"])
    assert_close(run.logits("a"), ref, dtype, f"{name} whole")
    run.step([("b", toks, 30)])
    for _ in range(15):
        run.step([("b", toks, 1)])
    assert_close(run.logits("b"), ref, dtype, f"{name} decoded")


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_decoded_and_in_portions(dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    n = 150 if device == "cuda" else 70
    toks = random_tokens(n, cfg["vocab"], 11)
    ref = oracle(cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 192)
    run.step([("whole", toks, n)], end=["whole"])
    assert_close(run.logits("whole"), ref, dtype, "whole")
    # most of it at once, then token by token across the windows (7 to 33 keys) and page borders (16)
    run.step([("tail", toks, n - 50)])
    for i in range(50):
        run.step([("tail", toks, 1)], end=["tail"] if i == 49 else [])
    assert_close(run.logits("tail"), ref, dtype, "decoded")
    # portions of changing size, down to two tokens and one; the first tokens of a sequence on their own
    fed, i, sizes = 0, 0, [1, 2, 7, 16, 2, 33, 5, 2, 17, 3, 1, 2, 11, 2, 29]
    while fed < n:
        c = min(sizes[i % len(sizes)], n - fed)
        run.step([("cut", toks, c)], end=["cut"] if fed + c == n else [])
        fed += c
        i += 1
    assert_close(run.logits("cut"), ref, dtype, "portions")
    # token by token from the very first one: the convolution's state and the kept first keys from the start
    for i in range(40):
        run.step([("one", toks, 1)], end=["one"] if i == 39 else [])
    assert_close(run.logits("one"), ref[:40], dtype, "token by token from the start")
    if dtype == "float32":
        assert (run.logits("whole") - run.logits("cut")).abs().max() < 5e-5
    run.rp.manager.check()
    assert run.rp.manager.num_free_slots() == 4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    lens = [90, 37, 1, 64, 23, 2, 55, 48] if device == "cuda" else [40, 17, 1, 33, 2, 21]
    reqs = {f"r{j}": random_tokens(n, cfg["vocab"], 40 + j) for j, n in enumerate(lens)}
    # a pool for the most tokens that are live at a time, each request rounded up to 64: pages and slots come back
    run = Run(folder, dtype, dev, 64 * 5, max_live=3)
    queue, live, step_no = list(reqs), [], 0
    portions = [5, 2, 16, 9, 3, 21, 2, 13]
    while queue or live:
        while queue and len(live) < 3:
            live.append(queue.pop(0))
        entries, ending = [], []
        for k, rid in enumerate(live):
            toks, fed = reqs[rid], run.fed.get(rid, 0)
            if (step_no + k) % 5 == 4 and fed > 0:
                continue                                    # left out of this step, goes on later
            c = min(portions[(step_no + k) % len(portions)], len(toks) - fed) if fed < 0.6 * len(toks) else 1
            entries.append((rid, toks, c))
            if fed + c == len(toks):
                ending.append(rid)
        if entries:
            run.step(entries, end=ending)
        live = [r for r in live if r not in ending]
        step_no += 1
    if dtype == "float32":
        for rid, toks in reqs.items():
            assert_close(run.logits(rid), oracle(cfg, w, toks, dtype), dtype, f"{rid} of {len(toks)} tokens in mixed batches")
    else:
        # bfloat16: against each request alone through the same engine (the kernels' choice by the step's size differs);
        # against the plain model all rows together, since a request in which one token's experts are a close call
        # differs from there on
        alone = Run(folder, dtype, dev, 64 * 5, max_live=3)
        for rid, toks in reqs.items():
            alone.step([(rid, toks, len(toks))], end=[rid])
            assert_close(run.logits(rid), alone.logits(rid), dtype, f"{rid} of {len(toks)} tokens: in mixed batches against alone")
        assert_close(torch.cat([run.logits(r) for r in reqs]), torch.cat([oracle(cfg, w, t, dtype) for t in reqs.values()]), dtype, "all requests")
    m = run.rp.manager
    m.check()
    assert m.num_free_slots() == 3 and all(m.num_free_pages(g) == m.num_pages for g in range(len(m.groups)))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_captured_steps(dtype, folders):
    """300 tokens one by one (steps replayed from a captured graph: the convolution's state, the windows and the pages
    behind them moving on) against the prompt whole."""
    folder, cfg, w = folders["mixed"]
    toks = random_tokens(330, cfg["vocab"], 3)
    ref = oracle(cfg, w, toks, dtype)
    run = Run(folder, dtype, torch.device("cuda:0"), 384)
    run.step([("a", toks, 30)])
    for _ in range(300):
        run.step([("a", toks, 1)])
    assert run.rp.runner.graph_replays >= 290
    assert_close(run.logits("a"), ref, dtype, "long decoding")


# --------------------------------------------------------------------------
# the window's edges, the kept first keys and the sink, with one key made to stand out
# --------------------------------------------------------------------------

def _attention_case(K, dev, dtype, window, keep, ctx, q_len, page_size, hot_key, sinks=None, implementation=None, copies=1, dh=32):
    """One sequence of ``ctx`` keys whose last ``q_len`` tokens are this step's.  Keys and queries are small noise, except
    that every query has a large component along one key: the key ``hot_key`` positions behind it (an int), or the key
    at an absolute position (``("at", j)``); that key's value is a marker.  Returns the kernel's output and the operands."""
    torch.manual_seed(ctx * 31 + q_len)
    nh, nkv = 4, 2
    T, pages = q_len, -(-ctx // page_size)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    k = 0.05 * torch.randn(ctx, nkv, dh)
    v = 0.05 * torch.randn(ctx, nkv, dh)
    q = 0.05 * torch.randn(T, nh, dh)
    for t in range(T):
        j = hot_key[1] if isinstance(hot_key, tuple) else ctx - T + t - hot_key
        if 0 <= j <= ctx - T + t:
            k[j, :, (3 * j) % dh] += 6.0
            q[t, :, (3 * j) % dh] += 6.0
            if t == T - 1:
                v[j, :, 0] = 10.0                                   # the marker: only the last token's hot key carries it
    order = torch.randperm(pages)                                   # pages in any order
    kc = torch.zeros(pages + 1, nkv, page_size, dh)
    vc = torch.zeros(pages + 1, nkv, dh, page_size)
    for j in range(ctx):
        kc[order[j // page_size], :, j % page_size] = k[j]
        vc[order[j // page_size], :, :, j % page_size] = v[j]
    qkv = torch.cat([q.reshape(T, -1), torch.zeros(T, 2 * nkv * dh)], dim=1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    S = copies
    assert S == 1 or T == 1
    args = dict(k_cache=kc.to(dev, dt), v_cache=vc.to(dev, dt), block_table=order.to(torch.int32).view(1, -1).repeat(S, 1).to(dev).contiguous(),
                q_start=i32(list(range(0, S * T + 1, T))), ctx_lens=i32([ctx] * S), seq_of_token=i32([s for s in range(S) for _ in range(T)]),
                positions=i32(list(range(ctx - T, ctx)) * S), num_heads=nh, num_kv_heads=nkv, head_dim=dh, scale=1.0, window=window,
                max_q_len=T, max_ctx_len=ctx)
    out = torch.empty(S * T, nh * dh, dtype=dt, device=dev)
    if implementation == "prefill_tcgen05":
        # with the work list the engine makes: few tiles of tokens behind a long context have their keys shared out among CTAs
        from litinfer_b200.engine.batch import attention_units

        units = attention_units([T], [ctx], work_budget=148 // nh)
        args.update(units=torch.from_numpy(units).to(dev), unit_slots=(int(units[0]), int(units[1])))
    K.paged_attention(qkv.repeat(S, 1).to(dev, dt).contiguous(), out, **args, keep_first=keep, sinks=sinks.to(dev) if sinks is not None else None,
                      implementation=implementation)
    out = out.float().cpu()
    assert S == 1 or (out - out[:1]).abs().max() <= 1e-2 * out.abs().max(), "equal sequences of one step differ"
    return out[:T], (q, k, v)


def _plain_attention(q, k, v, window, keep, sinks=None):
    T, nh, dh = q.shape
    ctx, nkv = k.shape[0], k.shape[1]
    out = torch.zeros(T, nh, dh, dtype=torch.float64)
    for t in range(T):
        i = ctx - T + t
        seen = [j for j in range(i + 1) if i - j < window or j < keep]
        for h in range(nh):
            s = k[seen, h // (nh // nkv)].double() @ q[t, h].double()
            if sinks is not None:
                p = torch.softmax(torch.cat([s, sinks[h:h + 1].double()]), 0)[:-1]
            else:
                p = torch.softmax(s, 0)
            out[t, h] = p @ v[seen, h // (nh // nkv)].double()
    return out.reshape(T, nh * dh).float()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 7, 70])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_first_tokens(q_len, dtype, device, request):
    dev = use_device(device, request)
    from litinfer_b200 import kernels as K

    window, keep, page = 37, 5, 16
    rnd = (lambda x: x.to(torch.bfloat16).float()) if dtype == "bfloat16" else (lambda x: x)
    tol = 2e-4 if dtype == "float32" else 0.03
    for ctx in ([75, 200] if device == "cuda" else [75]):
        if q_len > ctx:
            continue
        cases = [(window - 1, True), (window, False), (0, True), (window + 1, False), (15, True), (16, True),
                 (("at", 0), True), (("at", keep - 1), True), (("at", keep), False), (("at", keep + 1), False)]
        for hot, seen in cases:
            out, (q, k, v) = _attention_case(K, dev, dtype, window, keep, ctx, q_len, page, hot)
            ref = _plain_attention(rnd(q), rnd(k), rnd(v), window, keep)
            assert (out - ref).abs().max() <= tol * ref.abs().max(), f"ctx {ctx}, {q_len} tokens, hot key {hot}"
            # the marker (10 in column 0 of the value) reaches the last token's output only if its key is seen
            last = out[-1].view(4, 32)[:, 0].abs().max()
            assert (last > 1.0) == seen, f"ctx {ctx}, {q_len} tokens: key {hot} {'is' if seen else 'is not'} seen (window {window}, first {keep} kept)"


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 9])
def test_the_sink_takes_its_share_of_the_softmax(q_len, dtype, device, request):
    dev = use_device(device, request)
    from litinfer_b200 import kernels as K

    rnd = (lambda x: x.to(torch.bfloat16).float()) if dtype == "bfloat16" else (lambda x: x)
    tol = 2e-4 if dtype == "float32" else 0.03
    # per head: a sink far below the scores changes nothing; one far above them takes nearly everything; one as large as
    # the hot key's score (6 * 6) takes about half
    sinks = torch.tensor([-30.0, 0.5, 60.0, 36.0])
    out, (q, k, v) = _attention_case(K, dev, dtype, 20, 0, 50, q_len, 16, 3, sinks=sinks)
    ref = _plain_attention(rnd(q), rnd(k), rnd(v), 20, 0, sinks)
    assert (out - ref).abs().max() <= tol * ref.abs().max()
    plain, _ = _attention_case(K, dev, dtype, 20, 0, 50, q_len, 16, 3)
    heads, without = out.view(q_len, 4, 32), plain.view(q_len, 4, 32)
    assert (heads[:, 0] - without[:, 0]).abs().max() <= tol * ref.abs().max()
    assert heads[:, 2].abs().max() < 1e-3
    assert without[-1, 3, 0] > 9.0 and 2.0 < heads[-1, 3, 0] < 8.0


@pytest.mark.gpu
@pytest.mark.parametrize("implementation,q_len,ctx,copies", [
    ("general", 1, 700, 1), ("general", 45, 700, 1),
    ("decode", 1, 700, 1),             # a unit of 256 keys per CTA, merged by the last one
    ("decode", 1, 700, 80),            # many sequences: a CTA walks the whole context
    ("decode", 1, 3000, 10),           # units of several rounds
    ("prefill", 7, 700, 1), ("prefill", 130, 700, 1), ("prefill", 200, 333, 1),
    ("prefill_tcgen05", 130, 700, 1), ("prefill_tcgen05", 300, 333, 1), ("prefill_tcgen05", 64, 3000, 1), ("prefill_tcgen05", 520, 1500, 1)])
def test_each_attention_kernel_alone_keeps_the_first_keys_and_takes_the_sink(implementation, q_len, ctx, copies):
    """Kept first keys (more of them than a tile of keys holds) and the sink in each bfloat16 attention kernel by itself,
    over a context of several pages, tiles and split units, with the hot key at every edge."""
    from litinfer_b200 import kernels as K

    dev, window, keep = torch.device("cuda:0"), 300, 70
    dh = 32
    if implementation == "prefill_tcgen05":
        dh = 64                                                     # (heads of 64 or 128)
    rnd = lambda x: x.to(torch.bfloat16).float()
    sinks = torch.tensor([0.5, 36.0, -3.0, 2.0])
    for hot, seen in ((window - 1, True), (window, ctx - 1 - window < keep), (5, True), (("at", 0), True), (("at", keep - 1), True), (("at", keep), ctx - 1 - keep < window),
                      (("at", 64), True), (("at", 63), True)):
        if isinstance(hot, tuple) and keep == 0:
            seen = ctx - 1 - hot[1] < window
        out, (q, k, v) = _attention_case(K, dev, "bfloat16", window, keep, ctx, q_len, 16, hot, sinks=sinks, implementation=implementation, copies=copies,
                                         dh=dh)
        ref = _plain_attention(rnd(q), rnd(k), rnd(v), window, keep, sinks)
        assert (out - ref).abs().max() <= 0.03 * ref.abs().max(), f"{implementation}: ctx {ctx}, {q_len} tokens, hot key {hot}"
        last = out[-1].view(4, dh)[0, 0].abs()                      # head 0: its sink is negligible
        assert (last > 1.0) == seen, f"{implementation}: ctx {ctx}, {q_len} tokens: key {hot} {'is' if seen else 'is not'} seen"


@pytest.mark.parametrize("device", DEVICES)
def test_a_far_token_is_seen_only_through_the_kept_first_keys(device, folders, request):
    """One attention layer: changing a token among the kept first ones changes the last token's logits far beyond the
    window; changing the first token behind them does not.  The same whether the prompt is fed whole or in portions and
    single tokens (pages behind the window are given back on the way; the kept ones stay)."""
    dev = use_device(device, request)
    folder, cfg, w = folders["attention_only"]
    keep = cfg["layers"][0]["mixer"]["mask"]["keep_first"]
    n = 260 if device == "cuda" else 90
    a = random_tokens(n, cfg["vocab"], 9)
    b, c = list(a), list(a)
    b[keep - 1] = (a[keep - 1] + 17) % cfg["vocab"]
    c[keep] = (a[keep] + 17) % cfg["vocab"]
    ra, rb, rc = (oracle(cfg, w, t, "float32")[-1] for t in (a, b, c))
    assert (ra - rb).abs().max() > 1e-3 and (ra - rc).abs().max() < 1e-9
    run = Run(folder, "float32", dev, 64 * 10)
    run.step([("a", a, n)], end=["a"])
    for rid, toks in (("b", b), ("c", c)):
        fed = 0
        for cnt in [3, 60, 2, 1, 100, 31, 1, 1]:
            cnt = min(cnt, n - fed)
            if cnt:
                run.step([(rid, toks, cnt)])
                fed += cnt
        while fed < n:
            run.step([(rid, toks, 1)])
            fed += 1
    got = run.logits("a")[-1] - run.logits("b")[-1]
    assert (got - (ra - rb)).abs().max() <= 0.02 * (ra - rb).abs().max() + 2e-5
    assert (run.logits("a")[-1] - run.logits("c")[-1]).abs().max() <= 2e-5
    # pages behind the window went back while the request was live; the kept first page did not
    m = run.rp.manager
    rc_b = run.rp.live["b"]
    table = m.table(rc_b, 0)
    assert table[0] >= 0 and table[1] == m.RELEASED and table[-1] >= 0


# --------------------------------------------------------------------------
# the front end
# --------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_front_end(device, folders, request):
    dev = use_device(device, request)
    from litinfer_b200.api import CausalLM
    from litinfer_b200.models import DecoderModel

    folder, cfg, w = folders["mixed"]
    w64 = {k: v.double() for k, v in w.items()}
    lm = CausalLM(folder, dtype="float32") if device == "cuda" else CausalLM(folder, device="cpu", model=DecoderModel.from_dir(folder, "float32", dev),
                                                                            use_graphs=False)
    for n, new in ((1, 6), (13, 20), (50, 12)):
        prompt = random_tokens(n, cfg["vocab"], 60 + n)
        toks, margins = list(prompt), []
        for _ in range(new):
            top = torch.topk(P.forward(cfg, w64, toks)[-1], 2)
            margins.append(float(top.values[0] - top.values[1]))
            toks.append(int(top.indices[0]))
        assert min(margins) > 1e-4, "the plain model's own choice is a near-tie; pick another seed"
        out = lm.generate(prompt, max_new_tokens=new)
        assert list(out)[-new:] == toks[n:], f"prompt of {n} tokens"


def test_configuration_is_read_and_refused():
    from litinfer_b200.config import ConfigError, config_from_dict

    cfg = CONFIGS["mixed"]
    spec = config_from_dict(cfg).to_model_spec()
    assert len(spec.blocks) == 4 and [e.block for e in spec.schedule] == [0, 1, 0, 1, 2, 3]
    assert [e.add for e in spec.schedule] == [("loop.step", 0), None, ("loop.step", 1), None, None, None]
    assert spec.stream_tables == {"loop.step": 2}
    att = spec.blocks[1].parts["mixer"]
    assert att["window"] == 11 and att["keep_first"] == 3 and att["conv"] == 4 and att["value_dim"] == 32 and att["position"]["rotary_dim"] == 8
    lat = spec.blocks[0].parts["mixer"]
    assert lat["kv_rank"] == 40 and lat["window"] == 7
    ff = spec.blocks[0].parts["feed_forward"]
    assert ff["experts"] == 5 and ff["top"] == 2 and ff["weight_on"] == "input" and "feed_forward" not in spec.blocks[2].parts
    for path, bad in ((("layers", 0, "type"), "mamba2"), (("layers", 1, "mlp", "kind"), "dense"), (("layers", 1, "mixer", "kv_heads"), 4),
                      (("layers", 1, "mixer", "rot", "dims"), 7), (("layers", 0, "mlp", "router", "top"), 9), (("loop", "stop"), 7),
                      (("norm",), None), (("width",), 0)):
        broken = json.loads(json.dumps(cfg))
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = bad
        with pytest.raises(ConfigError):
            config_from_dict(broken)


def test_random_weights_and_a_written_folder(tmp_path, cpu_kernels):
    """Random-weights mode knows the design's tensors: a folder written from the configuration loads and steps."""
    from litinfer_b200.weights import write_model_folder
    from litinfer_b200.weights.safetensors_io import iter_tensors, read_header

    cfg = CONFIGS["mixed"]
    d = write_model_folder(tmp_path / "m", dict(cfg), seed=5)
    header, _ = read_header(d / "model.safetensors")
    w = {n: t.double() for n, t in iter_tensors(d / "model.safetensors", set(header))}
    assert w["loop.step"].shape == (2, 48) and w["l1.mix.q.conv"].shape == (96, 4) and w["l0.mix.sink"].shape == (3,)
    toks = random_tokens(20, cfg["vocab"], 1)
    run = Run(d, "float32", torch.device("cpu"), 64)
    run.step([("a", toks, 20)])
    assert_close(run.logits("a"), P.forward(cfg, w, toks).float(), "float32", "written folder")


def test_pages_behind_the_window_go_back_and_the_kept_first_ones_stay():
    """The host runtime's bookkeeping alone: a group with a window of 40 keys that keeps its first 20."""
    from litinfer_b200.cache.manager import CacheManager
    from litinfer_b200.parts.base import PagedKV

    m = CacheManager([PagedKV(1, 16, 40, 20), PagedKV(1, 16, 40)], [None, None], 32, 16, 2, torch.float32, "cpu", allocate=False)
    rc = m.admit(7)
    m.extend(rc, 200)
    m.commit(rc, 200)
    kept, plain = m.table(rc, 0), m.table(rc, 1)
    # a query at position 200 reads keys 161 .. 200 (pages 10 ..) and, in the first group, keys 0 .. 19 (pages 0 and 1)
    assert [p >= 0 for p in kept] == [True, True] + [False] * 8 + [True] * 3
    assert [p >= 0 for p in plain] == [False] * 10 + [True] * 3
    m.check()
    m.release(rc)
    assert m.num_free_pages(0) == 32 and m.num_free_pages(1) == 32


# --------------------------------------------------------------------------
# each new kernel alone against its plain float32 reference (tests/kernel_refs.py)
# --------------------------------------------------------------------------

def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(a, b, dtype, what):
    a, b = a.float().cpu(), b.float().cpu()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (a - b).abs().max() <= tol * max(1.0, float(b.abs().max())), f"{what}: {float((a - b).abs().max()):.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [48, 100, 1000, 4096])
def test_norms_on_both_sides_of_a_sublayer_kernel(H, dtype):
    from litinfer_b200 import kernels as K
    import kernel_refs as R

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(H)
    T = 37
    x = (3.0 + torch.randn(T, H)).to(dev)                     # a mean far from zero: the variance must be of the deviations
    y = (2.0 * torch.randn(T, H) - 1.0).to(dev, dt)
    wp, wn = (1 + 0.2 * torch.randn(H)).to(dev), (1 + 0.2 * torch.randn(H)).to(dev)
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=dev)
    for post, nxt in (((wp, True, 1e-5), (wn, True, 1e-5)), ((wp, True, 1e-5), None), (None, (wn, False, 1e-6)), ((wp, False, 1e-5), (wn, True, 1e-5))):
        xa, xb = x.clone(), x.clone()
        oa, ob = (torch.empty(T, H, dtype=dt, device=dev) for _ in range(2))
        K.norm_add_norm(xa, y, post, nxt, oa if nxt else None)
        R.norm_add_norm(xb, y, post, nxt, ob if nxt else None)
        _close(xa, xb, "float32", "stream")
        if nxt:
            _close(oa, ob, dtype, "normalised")
    # the sublayer's output as a sum of rows that lie elsewhere (a token's experts), with and without weights
    top = 3
    pool = torch.randn(T * top + 5, H).to(dev, dt)
    place = torch.randperm(T * top + 5)[:T * top].to(torch.int32).to(dev)
    wts = torch.rand(T, top).to(dev)
    for weights in (None, wts):
        xa, xb = x.clone(), x.clone()
        oa, ob = (torch.empty(T, H, dtype=dt, device=dev) for _ in range(2))
        K.norm_add_norm(xa, K.RowSum(pool, place, top, weights), (wp, True, 1e-5), (wn, True, 1e-5), oa)
        R.norm_add_norm(xb, K.RowSum(pool, place, top, weights), (wp, True, 1e-5), (wn, True, 1e-5), ob)
        _close(xa, xb, "float32", "stream (sum of rows)")
        _close(oa, ob, dtype, "normalised (sum of rows)")
    oa, ob = (torch.empty(4, H, dtype=dt, device=dev) for _ in range(2))
    K.norm_add_norm(x, None, None, (wn, True, 1e-5), oa, rows=rows)
    R.norm_add_norm(x, None, None, (wn, True, 1e-5), ob, rows=rows)
    _close(oa, ob, dtype, "gathered rows")
    xa, xb = x.clone(), x.clone()
    K.add_row(xa, wp)
    R.add_row(xb, wp)
    assert torch.equal(xa, xb)
    src = torch.randn(T, 100).to(dev, dt)
    oa = torch.zeros(T, 90, dtype=dt, device=dev)
    ob = torch.zeros(T, 90, dtype=dt, device=dev)
    wc = torch.cat([1 + 0.2 * torch.randn(24), torch.zeros(8)]).to(dev)
    src[:, 10 + 24:10 + 32] = 0
    K.rmsnorm_cols(src, 10, 32, 24, wc, 1e-5, oa, 3, 50)
    R.rmsnorm_cols(src, 10, 32, 24, wc, 1e-5, ob, 3, 50)
    _close(oa, ob, dtype, "norm of columns")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,rot,norm", [(4, 8, True), (1, 0, True), (3, 48, False), (2, 16, True)])
def test_convolution_norm_rotation_and_cache_write_kernel(taps, rot, norm, dtype):
    from litinfer_b200 import kernels as K
    import kernel_refs as R

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(taps * 7 + rot)
    nh, nkv, dh, page = 3, 1, 48, 16
    N = (nh + 2 * nkv) * dh
    lens, slots = [5, 1, 40, 2], [2, 0, 3, 1]
    T = sum(lens)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    first = [9, 30, 0, 3]                                      # positions the portions start at
    pos = [first[s] + j for s, n in enumerate(lens) for j in range(n)]
    seq = [s for s, n in enumerate(lens) for _ in range(n)]
    slot_map = torch.randperm(10 * page)[:T].to(torch.int32).to(dev)
    proj = torch.randn(T, N).to(dev, dt)
    conv = (0.5 * torch.randn(N, taps)).to(dev) if taps > 1 else None
    state = torch.randn(5, 7 + max(taps - 1, 0) * N).to(dt).float().to(dev)
    qn, kn = ((1 + 0.2 * torch.randn(dh)).to(dev), (1 + 0.2 * torch.randn(dh)).to(dev)) if norm else (None, None)
    den = torch.pow(torch.tensor(700.0), 2.0 * torch.arange(rot // 2) / max(rot, 1)).to(dev) if rot else None
    res = []
    for F in (K, R):
        out = torch.zeros(T, N, dtype=dt, device=dev)
        kc = torch.zeros(11, nkv, page, dh, dtype=dt, device=dev)
        vc = torch.zeros(11, nkv, dh, page, dtype=dt, device=dev)
        st = state.clone()
        F.conv_norm_rope_kv(proj, out, conv, st, 7, i32(starts), i32(seq), i32(slots), qn, kn, 1e-5, dh, i32(pos), den, rot, slot_map, kc, vc, nh, nkv, dh)
        if taps > 1:
            F.conv_state_shift(proj, 0, N, taps, st, 7, i32(starts), i32(slots))
        res.append((out[:, :nh * dh], kc, vc, st))
    for a, b, what in zip(res[0], res[1], ("queries", "keys", "values", "state")):
        _close(a, b, dtype, what)
    # keys and values left in the row for another kernel to store
    rows_out = []
    for F in (K, R):
        out = torch.zeros(T, N, dtype=dt, device=dev)
        kc = torch.zeros(11, nkv, page, dh, dtype=dt, device=dev)
        vc = torch.zeros(11, nkv, dh, page, dtype=dt, device=dev)
        F.conv_norm_rope_kv(proj, out, conv, state.clone(), 7, i32(starts), i32(seq), i32(slots), qn, kn, 1e-5, dh, i32(pos), den, rot, slot_map, kc, vc, nh, nkv,
                            dh, to_cache=False)
        F.rope_kv_write(out, i32(pos), None, 0, slot_map, kc, vc, nh, nkv, dh)
        rows_out.append((out, kc, vc))
    for a, b, what in zip(rows_out[0], rows_out[1], ("rows", "keys", "values")):
        _close(a, b, dtype, what + " (stored apart)")
    _close(rows_out[0][1], res[0][1], dtype, "keys stored apart against stored at once")
    _close(rows_out[0][2], res[0][2], dtype, "values stored apart against stored at once")
    # a step of single tokens: the state moves on in the same launch
    S = 4
    res = []
    for F in (K, R):
        out = torch.zeros(S, N, dtype=dt, device=dev)
        kc = torch.zeros(11, nkv, page, dh, dtype=dt, device=dev)
        vc = torch.zeros(11, nkv, dh, page, dtype=dt, device=dev)
        st = state.clone()
        F.conv_norm_rope_kv(proj[:S].contiguous(), out, conv, st, 7, i32(list(range(S + 1))), i32(list(range(S))), i32(slots), qn, kn, 1e-5, dh,
                            i32(first), den, rot, slot_map[:S].contiguous(), kc, vc, nh, nkv, dh, shift=True)
        res.append((out[:, :nh * dh], kc, vc, st))
    for a, b, what in zip(res[0], res[1], ("queries", "keys", "values", "state")):
        _close(a, b, dtype, what + " (single tokens)")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_products_in_groups_and_routing_kernels(dtype):
    from litinfer_b200 import kernels as K
    import kernel_refs as R

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(3)
    for T, E, top, H, F in ((1, 4, 2, 40, 32), (150, 7, 3, 72, 96), (64, 1, 1, 32, 16), (333, 40, 4, 48, 8), (9, 8, 2, 64, 100)):
        logits = (2.0 * torch.randn(T, E)).to(dev)
        ids = [torch.empty(T, top, dtype=torch.int32, device=dev) for _ in range(2)]
        wts = [torch.empty(T, top, dtype=torch.float32, device=dev) for _ in range(2)]
        K.moe_route(logits, top, ids[0], wts[0])
        R.moe_route(logits, top, ids[1], wts[1])
        assert torch.equal(ids[0], ids[1]) and (wts[0] - wts[1]).abs().max() < 1e-6
        srt = [[torch.empty(E + 1, dtype=torch.int32, device=dev), torch.empty(T * top, dtype=torch.int32, device=dev),
                torch.empty(T * top, dtype=torch.int32, device=dev)] for _ in range(2)]
        K.moe_sort(ids[0], E, *srt[0])
        R.moe_sort(ids[0], E, *srt[1])
        for a, b in zip(*srt):
            assert torch.equal(a, b)
        offsets, pair_at, place_of = srt[0]
        h = torch.randn(T, H).to(dev, dt)
        w1 = (torch.randn(E, F, H) / math.sqrt(H)).to(dev, dt)
        rows = [torch.empty(T * top, H, dtype=dt, device=dev) for _ in range(2)]
        outs = [torch.empty(T * top, F, dtype=dt, device=dev) for _ in range(2)]
        ys = [torch.empty(T, F, dtype=dt, device=dev) for _ in range(2)]
        for i, Fn in enumerate((K, R)):
            Fn.moe_gather(h, pair_at, wts[0], top, rows[i])
            Fn.grouped_linear(rows[i], w1, outs[i], offsets)
            Fn.moe_combine(outs[i], place_of, wts[0], top, ys[i])
        _close(rows[0], rows[1], dtype, "gathered rows")
        _close(outs[0], outs[1], dtype, "rows in groups")
        _close(ys[0], ys[1], dtype, "combined")
        if dtype == "bfloat16" and F % 16 == 0:                 # the gated activation as the product's epilogue
            acts = [torch.empty(T * top, F // 2, dtype=dt, device=dev) for _ in range(2)]
            K.grouped_linear(rows[0], w1, acts[0], offsets, epilogue="swiglu")
            R.grouped_linear(rows[0], w1, acts[1], offsets, epilogue="swiglu")
            _close(acts[0], acts[1], dtype, "gated rows in groups")
    # many rows: every expert's run starts at a multiple of 128 and the products take tensor-core tiles of one expert each
    for T, E, top, H, F in ((700, 5, 2, 64, 144), (2048, 8, 1, 256, 1056), (300, 16, 3, 72, 40)):
        logits = (2.0 * torch.randn(T, E)).to(dev)
        if E == 16:
            logits[:, 3] = -30.0                              # an expert nobody chooses: an empty run
        ids = torch.empty(T, top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, top, dtype=torch.float32, device=dev)
        K.moe_route(logits, top, ids, wts)
        n_rows = K.sorted_rows(T * top, E, 128)
        assert n_rows % 128 == 0 and n_rows >= T * top
        srt = [[torch.empty(E + 1, dtype=torch.int32, device=dev), torch.empty(n_rows, dtype=torch.int32, device=dev),
                torch.empty(T * top, dtype=torch.int32, device=dev), torch.empty(n_rows // 128, dtype=torch.int32, device=dev)] for _ in range(2)]
        K.moe_sort(ids, E, srt[0][0], srt[0][1], srt[0][2], 128, srt[0][3])
        R.moe_sort(ids, E, srt[1][0], srt[1][1], srt[1][2], 128, srt[1][3])
        upto = int(srt[1][0][-1])
        assert torch.equal(srt[0][0], srt[1][0]) and torch.equal(srt[0][2], srt[1][2]) and torch.equal(srt[0][3], srt[1][3])
        assert torch.equal(srt[0][1], srt[1][1])
        offsets, pair_at, place_of, tiles = srt[0]
        h = torch.randn(T, H).to(dev, dt)
        w1 = (torch.randn(E, F, H) / math.sqrt(H)).to(dev, dt)
        rows = [torch.empty(n_rows, H, dtype=dt, device=dev) for _ in range(2)]
        outs = [torch.zeros(n_rows, F, dtype=dt, device=dev) for _ in range(2)]
        ys = [torch.empty(T, F, dtype=dt, device=dev) for _ in range(2)]
        for i, Fn in enumerate((K, R)):
            Fn.moe_gather(h, pair_at, wts, top, rows[i])
            Fn.grouped_linear(rows[i], w1, outs[i], offsets, tile_group=tiles)
            Fn.moe_combine(outs[i], place_of, None, top, ys[i])
        if dtype == "bfloat16" and F % 16 == 0:
            acts = [torch.zeros(n_rows, F // 2, dtype=dt, device=dev) for _ in range(2)]
            K.grouped_linear(rows[0], w1, acts[0], offsets, tile_group=tiles, epilogue="swiglu")
            R.grouped_linear(rows[0], w1, acts[1], offsets, tile_group=tiles, epilogue="swiglu")
            _close(acts[0][:upto], acts[1][:upto], dtype, "gated rows in groups (padded runs)")
        _close(rows[0], rows[1], dtype, "gathered rows (padded runs)")
        _close(outs[0][:upto], outs[1][:upto], dtype, "rows in groups (padded runs)")
        _close(ys[0], ys[1], dtype, "combined (padded runs)")
    # a map per head: columns in groups
    G, M, Kd, N = 5, 77, 24, 40
    a = torch.randn(M, G * Kd + 3).to(dev, dt)
    w = (torch.randn(G, N, Kd) / math.sqrt(Kd)).to(dev, dt)
    outs = [torch.zeros(M, G * N + 9, dtype=dt, device=dev) for _ in range(2)]
    K.grouped_linear(a, w, outs[0], None, Kd, N)
    R.grouped_linear(a, w, outs[1], None, Kd, N)
    _close(outs[0], outs[1], dtype, "columns in groups")
