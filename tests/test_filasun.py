"""The Filasun decoder through the engine against the plain implementation (tests/plain_filasun.py).

Small configurations of its own sizes and random weights, made here.  On a GPU the engine runs its CUDA kernels in
float32 and bfloat16; without one the same tests run the host-side logic (configuration, loader, cache manager with
pages and state slots, step function) over the kernels' plain references.  Covered: each mixer alone; a prompt whole,
against its last tokens decoded one by one, against portions down to two tokens; unequal requests in one batch against
each alone, with pages and state slots that are given back and used again; keys just inside and just outside the
window and at page borders, with one score made to stand out; long decoding; greedy generation through the front end.
"""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_filasun as P
from helpers import bf16_round, random_tokens

CUDA = torch.cuda.is_available()
DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]
DTYPES = ["float32", "bfloat16"]


def left(heads=4, kv=2, dim=16, vdim=16, window=9, scale=0.3, softcap=5.0):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale, "softcap": softcap}


def right(heads=2, dim=16, vdim=16, decay=(0.7, 0.97)):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(l=None, r=None, ls=0.8, rs=1.1, ff=64, limit=0.9):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right(), "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def mamba(heads=2, vdim=8, state=12, groups=1, conv=3, norm_groups=1, ff=None, limit=1.5):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(layers, width=48, vocab=97, streams=2, positions=400, eps=1e-5, cap=12.0):
    return {"architecture": "Filasun", "layers": layers, "logit_softcap": cap, "max_positions": positions, "norm": {"eps": eps},
            "streams": streams, "vocab": vocab, "width": width}


CONFIGS = {
    # everything at once, no two sizes alike: value heads wider than key heads, three query heads per key head, groups
    # of B and C, norm groups, a layer without feed-forward of either kind, three streams
    "mixed": config([
        parallel(left(heads=6, kv=2, dim=16, vdim=32, window=9), right(heads=3, dim=8, vdim=24, decay=(0.5, 0.9, 0.995)), ff=80),
        mamba(heads=4, vdim=8, state=12, groups=2, conv=4, norm_groups=2, ff=56),
        parallel(left(heads=2, kv=2, dim=32, vdim=16, window=33, scale=0.2, softcap=3.0), right(heads=1, dim=16, vdim=16, decay=(0.98,)), ff=None),
        mamba(heads=2, vdim=16, state=8, groups=1, conv=2),
    ], width=48, vocab=97, streams=3),
    # each mechanism alone
    "window_only": config([parallel(ls=1.0, rs=0.0, ff=None)], width=32, vocab=61, streams=1),
    "decay_only": config([parallel(ls=0.0, rs=1.0, ff=None)], width=32, vocab=61, streams=2),
    "ssm_only": config([mamba(heads=3, vdim=8, state=6, conv=4)], width=40, vocab=50, streams=2),
    "glu_only": config([mamba(heads=1, vdim=8, state=4, conv=1, ff=72, limit=0.25)], width=26, vocab=33, streams=4, cap=4.0),
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
        if ".hc" in n:
            s = shape[0]
            out[n] = {"in": 1.0 / s + 0.2 * r, "out": 1.0 + 0.2 * r, "mix": (torch.eye(s) if len(shape) == 2 else 0) + 0.2 * r}[last]
        elif last in ("norm", "norm1", "norm2", "D"):
            out[n] = 1.0 + 0.2 * r
        elif last == "b":
            out[n] = 0.3 * r
        elif last in ("A_log", "dt_bias"):
            out[n] = 0.7 * r
        elif last == "conv":
            out[n] = 0.5 * r
        elif n in ("embed", "pos"):
            out[n] = r
        else:
            out[n] = r * (1.5 / math.sqrt(shape[-1]))
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from litinfer_b200.weights.safetensors_io import write_file

    out = {}
    for k, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp("filasun_" + name)
        w = make_weights(cfg, 77 + k)
        (d / "config.json").write_text(json.dumps(cfg))
        write_file(d / "model.safetensors", w)
        out[name] = (d, cfg, w)
    return out


def use_device(device, request):
    if device == "cpu":
        request.getfixturevalue("cpu_kernels")
    return torch.device("cuda:0" if device == "cuda" else "cpu")


def oracle(cfg, w, tokens, dtype):
    return P.forward(cfg, bf16_round(w) if dtype == "bfloat16" else w, tokens).float()


def assert_close(got, ref, dtype, what):
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std(dim=-1).clamp_min(1e-3)
    # float32: two implementations differ by rounding only.  bfloat16: activations are rounded to 8 bits at about ten
    # places a layer; a row may be unlucky, the mean may not (a wrong key, state or window moves logits by tens of percent)
    bound = 2e-4 if dtype == "float32" else 0.15
    worst = int(err.argmax())
    assert err.max() <= bound, f"{what}: relative error {float(err.max()):.3e} at row {worst} (bound {bound})"
    assert dtype == "float32" or err.mean() <= 0.03, f"{what}: mean relative error {float(err.mean()):.3e}"


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
@pytest.mark.parametrize("name", ["window_only", "decay_only", "ssm_only", "glu_only"])
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
    # most of it at once, then token by token across the window (9 and 33 keys) and page borders (16)
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
    # token by token from the very first one
    for i in range(40):
        run.step([("one", toks, 1)], end=["one"] if i == 39 else [])
    assert_close(run.logits("one"), ref[:40], dtype, "token by token from the start")
    if dtype == "float32" and device == "cuda":
        # the 32-bit path sums in one order whatever the cut
        assert torch.equal(run.logits("whole"), run.logits("cut")) or (run.logits("whole") - run.logits("cut")).abs().max() < 2e-5
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
    for rid, toks in reqs.items():
        assert_close(run.logits(rid), oracle(cfg, w, toks, dtype), dtype, f"{rid} of {len(toks)} tokens in mixed batches")
    m = run.rp.manager
    m.check()
    assert m.num_free_slots() == 3 and all(m.num_free_pages(g) == m.num_pages for g in range(len(m.groups)))


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_of_several_requests_in_one_step(dtype, device, folders, request):
    """Portions long enough for the scans to run in chunks (of 64 tokens, side by side), of requests that begin, go on and
    decode in the same step: chunk borders in the middle of a portion, states carried over them and into the next step."""
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    lens = {"x": 333, "y": 140, "z": 205} if device == "cuda" else {"x": 150, "y": 140, "z": 140}
    reqs = {r: random_tokens(n, cfg["vocab"], 70 + n) for r, n in lens.items()}
    run = Run(folder, dtype, dev, 64 * 14)
    run.step([("x", reqs["x"], 129), ("y", reqs["y"], 3)])
    run.step([("x", reqs["x"], 1), ("y", reqs["y"], 128), ("z", reqs["z"], lens["z"] - 1)])
    run.step([("x", reqs["x"], lens["x"] - 130), ("y", reqs["y"], 1), ("z", reqs["z"], 1)])
    for _ in range(lens["y"] - 132):
        run.step([("y", reqs["y"], 1)])
    for r, toks in reqs.items():
        assert_close(run.logits(r), oracle(cfg, w, toks, dtype), dtype, f"{r} of {len(toks)} tokens")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_captured_steps(dtype, folders):
    """300 tokens one by one (steps replayed from a captured graph, states and windows moving on) against the prompt whole."""
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
# the window's edges, with one key made to stand out
# --------------------------------------------------------------------------

def _attention_case(K, dev, dtype, window, ctx, q_len, page_size, hot_distance, implementation=None):
    """One sequence of ``ctx`` keys whose last ``q_len`` tokens are this step's.  All keys and queries are small noise,
    except that every query has a large component along the key at distance ``hot_distance`` behind it; that key's
    value is a marker.  Returns the kernel's output and the marker's share of it, for head 0 of the last token."""
    torch.manual_seed(ctx * 31 + hot_distance)
    nh, nkv, dh = 4, 2, 32
    T, pages = q_len, -(-ctx // page_size)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    k = 0.05 * torch.randn(ctx, nkv, dh)
    v = 0.05 * torch.randn(ctx, nkv, dh)
    q = 0.05 * torch.randn(T, nh, dh)
    for t in range(T):
        j = ctx - T + t - hot_distance
        if j >= 0:
            k[j, :, t % dh] += 6.0
            q[t, :, t % dh] += 6.0
            v[j, :, 0] += 10.0 * (t + 1)
    order = torch.randperm(pages)                                   # pages in any order
    kc = torch.zeros(pages + 1, nkv, page_size, dh)
    vc = torch.zeros(pages + 1, nkv, dh, page_size)
    for j in range(ctx):
        kc[order[j // page_size], :, j % page_size] = k[j]
        vc[order[j // page_size], :, :, j % page_size] = v[j]
    qkv = torch.cat([q.reshape(T, -1), torch.zeros(T, 2 * nkv * dh)], dim=1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    args = dict(k_cache=kc.to(dev, dt), v_cache=vc.to(dev, dt), block_table=order.to(torch.int32).view(1, -1).to(dev).contiguous(),
                q_start=i32([0, T]), ctx_lens=i32([ctx]), seq_of_token=i32([0] * T), positions=i32(list(range(ctx - T, ctx))),
                num_heads=nh, num_kv_heads=nkv, head_dim=dh, scale=1.0, window=window, max_q_len=T, max_ctx_len=ctx)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)], dtype=torch.float32, device=dev)
    gate = (0.5 * torch.randn(T, nh)).to(dev, dt)
    out = torch.empty(T, nh * dh, dtype=dt, device=dev)
    K.paged_attention(qkv.to(dev, dt), out, **args, softcap=25.0, slopes=slopes, gate=gate, implementation=implementation)
    return out.float().cpu(), (q, k, v, gate.float().cpu(), slopes.cpu())


def _plain_attention(q, k, v, gate, slopes, window, softcap):
    T, nh, dh = q.shape
    ctx, nkv = k.shape[0], k.shape[1]
    out = torch.zeros(T, nh, dh, dtype=torch.float64)
    for t in range(T):
        i = ctx - T + t
        lo = max(0, i - window + 1)
        for h in range(nh):
            s = (k[lo:i + 1, h // (nh // nkv)].double() @ q[t, h].double())
            s = softcap * torch.tanh(s / softcap) - slopes[h].double() * torch.arange(i - lo, -1, -1, dtype=torch.float64)
            out[t, h] = (torch.softmax(s, 0) @ v[lo:i + 1, h // (nh // nkv)].double()) * torch.sigmoid(gate[t, h].double())
    return out.reshape(T, nh * dh).float()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 7, 70])
def test_keys_just_inside_and_just_outside_the_window(q_len, dtype, device, request):
    dev = use_device(device, request)
    from litinfer_b200 import kernels as K

    window, page = 37, 16
    for ctx in ([75, 200] if device == "cuda" else [75]):
        if q_len > ctx:
            continue
        for hot, seen in ((window - 1, True), (window, False), (0, True), (window - 2, True), (window + 1, False), (15, True), (16, True)):
            out, (q, k, v, gate, slopes) = _attention_case(K, dev, dtype, window, ctx, q_len, page, hot)
            rnd = (lambda x: x.to(torch.bfloat16).float()) if dtype == "bfloat16" else (lambda x: x)
            ref = _plain_attention(rnd(q), rnd(k), rnd(v), rnd(gate), slopes, window, 25.0)
            tol = 2e-4 if dtype == "float32" else 0.03
            assert (out - ref).abs().max() <= tol * ref.abs().max(), f"ctx {ctx}, {q_len} tokens, hot key at distance {hot}"
            # the marker (10 (t + 1) in column 0 of the value) reaches the output only if the key is inside the window
            last = out[-1].view(4, 32)[:, 0].abs().max()
            if ctx - 1 - hot >= 0:
                assert (last > 1.0) == seen, f"ctx {ctx}, {q_len} tokens: key at distance {hot} {'is' if seen else 'is not'} inside a window of {window}"


@pytest.mark.gpu
@pytest.mark.parametrize("implementation,q_len", [("general", 1), ("general", 45), ("decode", 1), ("prefill", 7), ("prefill", 130)])
def test_each_attention_kernel_alone_takes_the_changed_scores(implementation, q_len):
    """The cap, the distance penalty and the head gate in each bfloat16 attention kernel by itself, over a context that
    spans several pages and split units, with a hot key at the window's edge."""
    from litinfer_b200 import kernels as K

    dev, window = torch.device("cuda:0"), 300
    for ctx, hot in ((700, window - 1), (700, window), (333, 5)):
        out, (q, k, v, gate, slopes) = _attention_case(K, dev, "bfloat16", window, ctx, q_len, 16, hot, implementation=implementation)
        rnd = lambda x: x.to(torch.bfloat16).float()
        ref = _plain_attention(rnd(q), rnd(k), rnd(v), rnd(gate), slopes, window, 25.0)
        assert (out - ref).abs().max() <= 0.03 * ref.abs().max(), f"{implementation}: ctx {ctx}, {q_len} tokens, hot key at distance {hot}"


# --------------------------------------------------------------------------
# a key far back, through the states
# --------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_a_far_token_is_remembered_by_the_states_across_portions(device, folders, request):
    """Changing the second token of a long prompt changes the last token's logits (a slow decay keeps it; no window
    reaches it), and by the same amount whether the prompt is fed whole or in portions and single tokens."""
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    n = 260 if device == "cuda" else 80
    a = random_tokens(n, cfg["vocab"], 9)
    b = list(a)
    b[1] = (a[1] + 17) % cfg["vocab"]
    ra, rb = oracle(cfg, w, a, "float32")[-1], oracle(cfg, w, b, "float32")[-1]
    assert (ra - rb).abs().max() > 1e-3, "the plain model forgets the far token: choose other weights"
    run = Run(folder, "float32", dev, 64 * 10)
    run.step([("a", a, n)], end=["a"])
    fed = 0
    for c in [3, 60, 2, 1, 100, 31, 1, 1]:
        c = min(c, n - fed)
        if c:
            run.step([("b", b, c)])
            fed += c
    while fed < n:
        run.step([("b", b, 1)])
        fed += 1
    got = run.logits("a")[-1] - run.logits("b")[-1]
    assert (got - (ra - rb)).abs().max() <= 0.02 * (ra - rb).abs().max() + 2e-5


# --------------------------------------------------------------------------
# the front end
# --------------------------------------------------------------------------

@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_front_end(device, folders, request):
    dev = use_device(device, request)
    from litinfer_b200.api import CausalLM
    from litinfer_b200.models import DecoderModel

    folder, cfg, w = folders["mixed"]
    # (without a GPU the front end is handed the model, built over the kernels' references; with one it loads the folder)
    lm = CausalLM(folder, dtype="float32") if device == "cuda" else CausalLM(folder, device="cpu", model=DecoderModel.from_dir(folder, "float32", dev),
                                                                            use_graphs=False)
    for n, new in ((1, 6), (13, 20), (50, 12)):
        prompt = random_tokens(n, cfg["vocab"], 60 + n)
        toks, margins = list(prompt), []
        for _ in range(new):
            top = torch.topk(P.forward(cfg, w, toks)[-1], 2)
            margins.append(float(top.values[0] - top.values[1]))
            toks.append(int(top.indices[0]))
        assert min(margins) > 1e-4, "the plain model's own choice is a near-tie; pick another seed"
        out = lm.generate(prompt, max_new_tokens=new)
        assert list(out)[-new:] == toks[n:], f"prompt of {n} tokens"


def test_configuration_is_read_and_refused():
    from litinfer_b200.config import ConfigError, config_from_dict

    cfg = CONFIGS["mixed"]
    spec = config_from_dict(cfg).to_model_spec()
    assert spec.streams == 3 and spec.logit_cap == 12.0 and len(spec.blocks) == 4
    att = spec.blocks[0].parts["mixer"]["left"]
    assert att["window"] == 9 and att["value_dim"] == 32 and len(att["distance_slopes"]) == 6
    assert abs(att["distance_slopes"][-1] - 2.0 ** -8) < 1e-12
    for path, bad in ((("layers", 0, "type"), "conv"), (("layers", 1, "mlp", "kind"), "experts"), (("layers", 0, "mixer", "right", "decay"), [0.5]),
                      (("layers", 0, "mixer", "left", "kv_heads"), 4), (("norm",), None), (("width",), 0)):
        broken = json.loads(json.dumps(cfg))
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = bad
        with pytest.raises(ConfigError):
            config_from_dict(broken)


def test_random_weights_and_a_written_folder(tmp_path, cpu_kernels):
    """Random-weights mode knows the design's tensors: a folder written from the configuration loads and steps."""
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder
    from litinfer_b200.weights.safetensors_io import iter_tensors, read_header

    cfg = CONFIGS["mixed"]
    d = write_model_folder(tmp_path / "m", dict(cfg), seed=5)
    header, _ = read_header(d / "model.safetensors")
    w = {n: t.float() for n, t in iter_tensors(d / "model.safetensors", set(header))}
    assert (w["l0.hc1.mix"] - torch.eye(3)).abs().max() < 0.5 and w["l1.mix.A_log"].shape == (4,)
    toks = random_tokens(20, cfg["vocab"], 1)
    run = Run(d, "float32", torch.device("cpu"), 64)
    run.step([("a", toks, 20)])
    assert_close(run.logits("a"), P.forward(cfg, w, toks).float(), "float32", "written folder")


# --------------------------------------------------------------------------
# each new kernel alone against its plain float32 reference (tests/kernel_refs.py)
# --------------------------------------------------------------------------

def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(a, b, dtype, what):
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (a.float() - b.float()).abs().max() <= tol * max(1.0, float(b.float().abs().max())), what


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,d,dv", [(3, 24, 40), (2, 128, 64), (1, 160, 72), (5, 8, 8)])
def test_decay_scan_kernel(heads, d, dv, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(heads * d + dv)
    lens = [1, 200, 0, 67, 130]                                      # a single token, long portions, an empty sequence
    q_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    T = sum(lens)
    slots = torch.tensor([3, 0, 5, 1, 4], dtype=torch.int32, device=dev)
    stride = 2 * heads * d + heads * dv + 7
    qkv = torch.randn(T, stride, device=dev).to(dt)
    decay = torch.tensor([0.5, 0.9, 0.99, 0.999, 0.95][:heads], dtype=torch.float32, device=dev)
    state0 = 0.3 * torch.randn(6, heads * d * dv + 5, device=dev)
    got_s, ref_s = state0.clone(), state0.clone()
    ref_o = torch.zeros(T, heads * dv, device=dev)
    R.decay_scan(qkv, 3, 3 + heads * d, 3 + 2 * heads * d, decay, ref_s, q_start, slots, ref_o, heads, d, dv)
    for chunks in (None, K.ScanChunks(q_start.tolist(), slots.tolist(), dev)):
        s, o = state0.clone(), torch.zeros(T, heads * dv, device=dev)
        K.decay_scan(qkv, 3, 3 + heads * d, 3 + 2 * heads * d, decay, s, q_start, slots, o, heads, d, dv, chunks=chunks)
        _close(o, ref_o, "float32", f"outputs, chunks {chunks is not None}")
        _close(s, ref_s, "float32", f"states, chunks {chunks is not None}")
        assert torch.equal(s[2], state0[2]) and torch.equal(s[:, -5:], state0[:, -5:]), "a slot nobody named, or the words behind the state, changed"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,P,N,groups", [(4, 24, 12, 2), (2, 64, 128, 1), (3, 66, 200, 3), (1, 8, 33, 1)])
def test_ssm_scan_kernel(heads, P, N, groups, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(heads * P + N)
    lens = [130, 1, 0, 70, 1]
    q_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    T = sum(lens)
    slots = torch.tensor([2, 0, 1, 4, 3], dtype=torch.int32, device=dev)
    C = heads * P + 2 * groups * N
    xbc = (0.5 * torch.randn(T, C, device=dev)).to(dt)
    proj = torch.randn(T, 5 + heads, device=dev).to(dt)
    dt_bias, A_log, D = (0.5 * torch.randn(heads, device=dev) for _ in range(3))
    state0 = 0.3 * torch.randn(5, heads * P * N + 9, device=dev)
    ref_s, ref_y = state0.clone(), torch.zeros(T, heads * P, device=dev)
    R.ssm_scan(xbc, proj, 5, dt_bias, A_log, D, ref_s, q_start, slots, ref_y, heads, P, N, groups)
    for chunks in (None, K.ScanChunks(q_start.tolist(), slots.tolist(), dev)):
        s, y = state0.clone(), torch.zeros(T, heads * P, device=dev)
        K.ssm_scan(xbc, proj, 5, dt_bias, A_log, D, s, q_start, slots, y, heads, P, N, groups, chunks=chunks)
        _close(y, ref_y, "float32", f"outputs, chunks {chunks is not None}")
        _close(s, ref_s, "float32", f"states, chunks {chunks is not None}")
        assert torch.equal(s[:, -9:], state0[:, -9:])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_convolution_kernels(taps, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(taps)
    C, col, off = 150, 11, 40
    w, b = torch.randn(C, taps, device=dev), torch.randn(C, device=dev)
    for lens in ([5, 1, 0, 2, 30], [1, 1, 1]):
        q_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
        T = sum(lens)
        seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).to(torch.int32).to(dev)
        slots = torch.arange(len(lens), dtype=torch.int32, device=dev).flip(0).contiguous()
        x = torch.randn(T, col + C + 3, device=dev).to(dt)
        state0 = torch.randn(len(lens), off + (taps - 1) * C + 2, device=dev)
        ref_s, ref_o = state0.clone(), torch.zeros(T, C, device=dev, dtype=dt)
        R.causal_conv_silu(x, col, w, b, ref_s, off, q_start, seq, slots, ref_o)
        R.conv_state_shift(x, col, C, taps, ref_s, off, q_start, slots)
        for fused in ([False, True] if max(lens) == 1 else [False]):
            s, o = state0.clone(), torch.zeros(T, C, device=dev, dtype=dt)
            K.causal_conv_silu(x, col, w, b, s, off, q_start, seq, slots, o, shift=fused)
            if not fused:
                K.conv_state_shift(x, col, C, taps, s, off, q_start, slots)
            _close(o, ref_o, dtype, f"outputs, fused {fused}")
            _close(s, ref_s, "float32", f"states, fused {fused}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_norm_and_gated_kernels(dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(4)
    for T, s, H in ((37, 3, 100), (5, 1, 26), (64, 8, 256)):
        xs0 = torch.randn(T, s, H, device=dev)
        y, y2 = torch.randn(T, H, device=dev).to(dt), torch.randn(T, H, device=dev).to(dt)
        mix, wo, wi, nw = torch.randn(s, s, device=dev), torch.randn(s, device=dev), torch.randn(s, device=dev), torch.randn(H, device=dev)
        rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=dev)
        for read, rr in ((wi, None), (None, rows)):
            a, b = (torch.empty((T if rr is None else 3, H), device=dev, dtype=dt) for _ in range(2))
            K.hc_read_norm(xs0, read, rr, nw, 1e-5, a)
            R.hc_read_norm(xs0, read, rr, nw, 1e-5, b)
            _close(a, b, dtype, "read and norm")
        for out, nxt in ((y, True), (K.WeightedPair(y, y2, 0.7, 1.3), True), (y, False)):
            xa, xb = xs0.clone(), xs0.clone()
            na, nb = (torch.empty(T, H, device=dev, dtype=dt) for _ in range(2))
            K.hc_update(xa, out, mix, wo, wi if nxt else None, nw if nxt else None, 1e-5, na if nxt else None)
            R.hc_update(xb, out, mix, wo, wi if nxt else None, nw if nxt else None, 1e-5, nb if nxt else None)
            _close(xa, xb, "float32", "streams after the write-back")
            if nxt:
                _close(na, nb, dtype, "the next read")
    for T, n, groups in ((33, 96, 3), (4, 50, 1)):
        y32 = torch.randn(T, n, device=dev)
        gate = torch.randn(T, n + 9, device=dev).to(dt)
        w = torch.randn(n, device=dev)
        for first in (True, False):
            a, b = (torch.empty(T, n, device=dev, dtype=dt) for _ in range(2))
            K.gated_rmsnorm(y32, gate, 4, w, 1e-5, groups, first, a)
            R.gated_rmsnorm(y32, gate, 4, w, 1e-5, groups, first, b)
            _close(a, b, dtype, f"gated norm, gate first {first}")
    # the gated unit with bounded operands: as a kernel of its own and as the epilogue of every product kernel that has one
    for M, I, Kd in ((5, 64, 96), (40, 136, 64), (300, 256, 128), (2048, 4096, 128)):          # (the last: the persistent tcgen05 product)
        gate_w, up_w = (torch.randn(I, Kd, device=dev) / Kd ** 0.5 * 3 for _ in range(2))
        a_in = torch.randn(M, Kd, device=dev).to(dt)
        both = torch.empty(M, 2 * I, device=dev, dtype=dt)
        K.linear(a_in, torch.cat([gate_w, up_w]).to(dt).contiguous(), None, both)
        ref = torch.empty(M, I, device=dev, dtype=dt)
        R.glu_clamped(both, ref, 0.8, 1.702)
        got = torch.empty_like(ref)
        K.glu_clamped(both, got, 0.8, 1.702)
        _close(got, ref, dtype, "gated unit")
        if dtype == "bfloat16":
            params = torch.tensor([0.8, 1.702], dtype=torch.float32, device=dev)
            inter = K.interleave_gate_up(gate_w.to(dt), up_w.to(dt))
            for which in ("gemv", "gemv_tcgen05", "tcgen05"):
                if (which != "tcgen05") == (M <= 64):
                    fused = torch.empty_like(ref)
                    K.linear_with(which, a_in, inter, None, fused, epilogue="glu_clamped", epilogue_params=params)
                    _close(fused, ref, dtype, f"gated unit as the epilogue of {which}, {M} rows")
