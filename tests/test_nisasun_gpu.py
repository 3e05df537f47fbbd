"""Nisasun on the step engine against the plain float64 restatement (tests/nisasun_plain.py): every mechanism alone,
then whole prompts, token-by-token decoding, portions of many sizes, mixed batches, reused pages and slots, window
edges, long decoding, and greedy generation through the scheduler.  Small random configurations made here; f32 mode is
held to f32 rounding, bf16 mode to bf16 rounding."""
import copy

import numpy as np
import pytest
import torch

import nisasun_plain as P
from mistralrs_b200 import engine, mixers, nisasun, seq_ops as K

pytestmark = pytest.mark.gpu
F64 = torch.float64


def lightning_layer(heads=3, dim=24, vdim=40, decay=(0.5, 0.9, 1.0), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def parallel_layer(heads=6, kv_heads=2, dim=40, vdim=24, window=10, scale=0.3, s_heads=4, s_vdim=20, state=12, groups=2, norm_groups=2,
                   conv=3, left_scale=0.7, right_scale=1.3, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale},
                      "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv},
                      "left_scale": left_scale, "right_scale": right_scale}}


DENSE = {"kind": "dense", "ff": 112}


def moe(experts=8, top=3, count=4, keep=2, ff=48):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def make_cfg(layers, width=72, vocab=131, streams=3, eps=1e-5):
    return {"architecture": "Nisasun", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps}, "layers": layers}


FULL = make_cfg([lightning_layer(mlp=DENSE), parallel_layer(mlp=moe()), lightning_layer(mlp=moe(experts=6, top=2, count=1, keep=1)),
                 parallel_layer(mlp=None), parallel_layer(kv_heads=6, groups=1, norm_groups=1, conv=5, window=17, mlp=DENSE)])
DENSE_ONLY = make_cfg([lightning_layer(mlp=DENSE), parallel_layer(mlp=DENSE), parallel_layer(mlp=None, conv=2)], streams=1)


def build(cj, dtype, device, seed=0, page_size=16, edit=None):
    cfg = nisasun.NisasunConfig(copy.deepcopy(cj))
    tensors = nisasun.random_tensors(cfg, seed)
    if edit:
        edit(tensors)
    model = nisasun.NisasunModel(cfg, tensors, device, dtype, page_size=page_size)
    return model, {k: v.to(F64) for k, v in tensors.items()}


def rel_err(got, want):
    """Per row: rms of the difference (mean taken off) over the rms of the wanted logits."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean())


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def assert_close(got, want, dtype, what=""):
    e = rel_err(got, want)
    if dtype == torch.float32:
        assert e.max() < TOL[dtype], (what, float(e.max()), int(e.argmax()))
    else:   # a router decision may flip under bf16 rounding of its input: a few rows may differ, none wildly
        assert (e > TOL[dtype]).mean() <= 0.03 and np.median(e) < TOL[dtype] / 3, (what, float(e.max()), float(np.median(e)))


def replay(eng, prompts, schedule):
    """schedule: steps, each a list of (name, n_tokens).  Returns name -> logits of every position [T, vocab]."""
    live, rows = {}, {k: [] for k in prompts}
    for step in schedule:
        plan, want = [], []
        for name, n in step:
            if name not in live:
                live[name] = eng.new_request([])
            r = live[name]
            at = r.n_computed
            r.tokens.extend(prompts[name][at:at + n])
            plan.append((r, n))
            want.append(list(range(n)))
        lg = eng.execute(plan, want).cpu().numpy()
        at = 0
        for name, n in step:
            rows[name].append(lg[at:at + n])
            at += n
            if live[name].n_computed == len(prompts[name]):
                eng.finish(live.pop(name))
    return {k: np.concatenate(v) for k, v in rows.items() if v}


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


# ---- mechanisms alone ------------------------------------------------------------------------------------------------
def one_seq_batch(device, n, past=0, slot=0, page_size=16, first_page=1):
    pages = list(range(first_page, first_page + -(-(past + n) // page_size)))
    slots = [pages[(past + i) // page_size] * page_size + (past + i) % page_size for i in range(n)]
    return engine.StepBatch(device, [0] * n, [n], [past], [slot], [pages], np.asarray(slots, dtype=np.int64), [])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,W", [(3, 50), (1, 64), (2, 136), (4, 24), (6, 40), (11, 9)])
def test_streams_read_write_norm(cuda, dtype, S, W):
    g = torch.Generator().manual_seed(1)
    T = 9
    xs = torch.randn(T, S, W, generator=g)
    w_in, w_out, w_mix, nw, nw2 = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(S, S, generator=g), 0.2 * torch.randn(W, generator=g), 0.2 * torch.randn(W, generator=g)
    y = torch.randn(T, W, generator=g).to(dtype)
    d = lambda t: t.to(cuda)
    got_h = K.streams_read_norm(d(xs), d(w_in), d(nw), 1e-5, 1.0, dtype)
    want_h = P.norm_around_zero(P.streams_read(xs.double(), w_in.double()), nw.double(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (got_h.double().cpu() - want_h).abs().max() < tol
    xd = d(xs).clone()
    got_n = K.streams_write(xd, d(w_mix), d(w_out), d(y), d(w_in), d(nw2), 1e-5, 1.0)
    want_x = P.streams_write(xs.double(), w_mix.double(), w_out.double(), y.double())
    assert (xd.double().cpu() - want_x).abs().max() < 1e-5                       # the streams stay f32 in either mode
    want_n = P.norm_around_zero(P.streams_read(want_x, w_in.double()), nw2.double(), 1e-5)
    assert (got_n.double().cpu() - want_n).abs().max() < tol
    rows = torch.tensor([4, 0, 8], dtype=torch.int32, device=cuda)               # plain sum + row selection (the output head's read)
    got_s = K.streams_read_norm(xd, None, d(nw), 1e-5, 1.0, torch.float32, rows=rows)
    want_s = P.norm_around_zero(want_x.sum(1), nw.double(), 1e-5)[[4, 0, 8]]
    assert (got_s.double().cpu() - want_s).abs().max() < 1e-5


def mixer_case(cuda, layer, dtype, T, portions, seed=3, edit=None, width=72):
    """Run layer 0's mixer alone over `portions` of one sequence; returns (got [T, W], want [T, W])."""
    cj = make_cfg([layer], width=width)
    model, w = build(cj, dtype, cuda, seed, edit=edit)
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, width, generator=g).to(dtype)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(2, 16 * 40, dtype, cuda)
    out, at = [], 0
    for n in portions:
        b = one_seq_batch(cuda, n, past=at, slot=1)
        out.append(mixer.forward(h[at:at + n].to(cuda).contiguous(), b, cache).float().cpu())
        at += n
    assert at == T
    eps = cj["norm"]["eps"]
    if layer["type"] == "lightning":
        want = P.lightning_mixer(h.double(), w, "l0.mix.", layer["mixer"], eps)
    else:
        want = P.parallel_mixer(h.double(), w, "l0.mix.", layer["mixer"], eps)
    return torch.cat(out).double(), want


def close_rows(got, want, tol):
    e = (got - want).norm(dim=-1) / want.norm(dim=-1).mean()
    assert e.max() < tol, (float(e.max()), int(e.argmax()))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[150], [1] * 40, [7, 2, 33, 1, 64, 2, 41]])
def test_lightning_mixer(cuda, dtype, tol, portions):
    got, want = mixer_case(cuda, lightning_layer(decay=(0.4, 0.97, 1.0)), dtype, sum(portions), portions)
    close_rows(got, want, tol)


def test_scan_in_segments(cuda, monkeypatch, full32):
    """Long portions are scanned as segments side by side (zero-state pass, chaining, output pass): made to happen on
    short ones here, with ragged last segments, a state carried in from an earlier portion, and a short sequence beside."""
    monkeypatch.setattr(K, "SCAN_SEGMENT", 16)
    monkeypatch.setattr(K, "SCAN_SEGMENT_MIN_TOKENS", 40)
    for layer in (lightning_layer(decay=(0.4, 0.97, 1.0)), parallel_layer(left_scale=0.0, right_scale=1.0)):
        got, want = mixer_case(cuda, layer, torch.float32, 150, [70, 3, 77])
        close_rows(got, want, 3e-5)
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 14, max_seqs=2)
    got = replay(eng, prompts, [[("a", 99), ("b", 37)], [("a", 51)]])
    for name in ("a", "b"):
        assert_close(got[name], want[name], torch.float32, name)


def test_lightning_wide_keys(cuda):
    got, want = mixer_case(cuda, lightning_layer(heads=2, dim=136, vdim=72, decay=(0.9, 0.99)), torch.float32, 40, [13, 1, 26])
    close_rows(got, want, 2e-5)


def test_lightning_first_token_survives_far(cuda):
    """A head with decay 1 keeps the first token for ever: make that token's key / value huge and look 300 tokens later."""
    def edit(t):
        t["l0.mix.norm"].fill_(1.0)
    layer = lightning_layer(heads=2, dim=16, vdim=16, decay=(1.0, 0.5))
    cj = make_cfg([layer], width=32)
    model, w = build(cj, torch.float32, cuda, 5, edit=edit)
    h = torch.randn(300, 32, generator=torch.Generator().manual_seed(5)) * 0.1
    h[0] *= 60.0
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16, torch.float32, cuda)
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), one_seq_batch(cuda, b - a, past=a), cache).cpu()
                     for a, b in ((0, 250), (250, 251), (251, 300))]).double()
    want = P.lightning_mixer(h.double(), w, "l0.mix.", layer["mixer"], cj["norm"]["eps"])
    close_rows(got, want, 2e-4)      # the huge first token costs the f32 state a few digits on everything after it
    without = P.lightning_mixer(h.double()[1:], w, "l0.mix.", layer["mixer"], cj["norm"]["eps"])
    assert (want[1:] - without).norm(dim=-1)[-1] > 0.1 * want[-1].norm()      # the test would see a lost first token


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("scales", [(1.0, 0.0), (0.0, 1.0), (0.7, 1.3)])
@pytest.mark.parametrize("portions", [[90], [1] * 30, [5, 2, 17, 1, 33, 2]])
def test_parallel_mixer_branches(cuda, dtype, tol, scales, portions):
    layer = parallel_layer(left_scale=scales[0], right_scale=scales[1])
    got, want = mixer_case(cuda, layer, dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("kw", [dict(kv_heads=6), dict(kv_heads=1, heads=4), dict(groups=1, norm_groups=4), dict(groups=4, norm_groups=1, conv=6),
                                dict(conv=1), dict(dim=8, vdim=136), dict(dim=72, vdim=8, window=1), dict(s_vdim=8, state=80)])
def test_parallel_mixer_other_sizes(cuda, kw):
    got, want = mixer_case(cuda, parallel_layer(**kw), torch.float32, 45, [20, 1, 1, 3, 20])
    close_rows(got, want, 3e-5)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("portions", [[90], [40, 1, 30, 19], [3, 87]])
def test_parallel_mixer_prompt_kernels(cuda, d, portions):
    """bf16 with equal head sizes of 64 / 128: a sequence's first portion of 32 tokens or more runs on the package's
    prompt-attention kernels over the fresh q / k / v; the pages must still be filled for what follows."""
    layer = parallel_layer(heads=4, kv_heads=2, dim=d, vdim=d, window=23, scale=d ** -0.5, s_heads=4, s_vdim=16, state=16, groups=1)
    got, want = mixer_case(cuda, layer, torch.bfloat16, 90, portions, width=64)
    close_rows(got, want, 3e-2)


@pytest.mark.parametrize("distance", [-2, -1, 0, 1])
@pytest.mark.parametrize("decoded", [False, True])
def test_window_edge_shows(cuda, distance, decoded):
    """One earlier token shares the query's direction, all others are near-orthogonal, and the score scale is large: the
    output is that token's value while it is inside the window and something else one step later."""
    window, T = 24, 70
    target = T - 1 - (window - 1) - distance          # distance <= 0: inside the window of the last token
    layer = parallel_layer(heads=2, kv_heads=1, dim=32, vdim=16, window=window, scale=1.5, left_scale=1.0, right_scale=0.0)

    def edit(t):
        for n in ("l0.mix.left.q", "l0.mix.left.k"):
            t[n].zero_()
        eye = torch.eye(32, 64).to(torch.bfloat16)
        t["l0.mix.left.q"][:32], t["l0.mix.left.q"][32:], t["l0.mix.left.k"][:] = eye, eye, eye
        t["l0.mix.left.q.norm"].fill_(1.0)
        t["l0.mix.left.k.norm"].fill_(1.0)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.float32, cuda, 9, edit=edit)
    g = torch.Generator().manual_seed(9)
    h = torch.randn(T, 64, generator=g)
    h[target, :32] = h[T - 1, :32]                    # same direction in the q / k subspace
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 8, torch.float32, cuda)
    cuts = [(0, T - 3), (T - 3, T - 2), (T - 2, T - 1), (T - 1, T)] if decoded else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), one_seq_batch(cuda, b - a, past=a), cache).cpu() for a, b in cuts]).double()
    want = P.parallel_mixer(h.double(), w, "l0.mix.", layer["mixer"], cj["norm"]["eps"])
    close_rows(got, want, 3e-5)
    m2 = copy.deepcopy(layer["mixer"])
    m2["left"]["mask"]["size"] = window + distance if distance > 0 else window - 1 + distance     # the target crosses the edge
    other = P.parallel_mixer(h.double(), w, "l0.mix.", m2, cj["norm"]["eps"])
    assert (other[-1] - want[-1]).norm() > 0.2 * want[-1].norm()               # an edge that is one off would show


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_dense_ff(cuda, dtype, tol):
    cj = make_cfg([lightning_layer(mlp=DENSE)])
    model, w = build(cj, dtype, cuda, 2)
    h = torch.randn(21, 72, generator=torch.Generator().manual_seed(2)).to(dtype)
    got = model.layers[0].mlp.forward(h.to(cuda)).double().cpu()
    close_rows(got, P.dense_ff(h.double(), w, "l0.mlp."), tol)


@pytest.mark.parametrize("kw", [dict(), dict(experts=12, top=4, count=2, keep=1), dict(experts=6, top=6, count=3, keep=3), dict(experts=5, top=1, count=1, keep=1),
                                dict(experts=16, top=2, count=8, keep=3)])
@pytest.mark.parametrize("T", [3, 150])     # few pairs per expert: weight-streaming kernels; many: rows sorted by expert
def test_routed_experts(cuda, kw, T):
    mlp = moe(**kw)

    def edit(t):      # a correction large enough to change who is chosen, negative for some experts
        t["l0.mlp.correction"].copy_((torch.randn(t["l0.mlp.correction"].shape, generator=torch.Generator().manual_seed(4)) * 0.2).to(torch.bfloat16))
    cj = make_cfg([lightning_layer(mlp=mlp)])
    model, w = build(cj, torch.float32, cuda, 4, edit=edit)
    h = torch.randn(T, 72, generator=torch.Generator().manual_seed(T)).to(torch.bfloat16).float()
    ff = model.layers[0].mlp
    idx, wt = ff.route(h.to(cuda))
    want_idx, want_wt = P.route(h.double(), w, "l0.mlp.", mlp["router"])
    assert torch.equal(idx.cpu().long().sort(-1).values, want_idx.sort(-1).values)
    assert (wt.double().cpu().sort(-1).values - want_wt.sort(-1).values).abs().max() < 1e-6
    plain_idx = torch.softmax(h.double() @ w["l0.mlp.router"].T, -1).topk(mlp["router"]["top"]).indices
    if kw.get("count", 4) > kw.get("keep", 2) and T > 3:
        assert not torch.equal(plain_idx.sort(-1).values, want_idx.sort(-1).values)     # groups and correction matter in this case
    close_rows(ff.forward(h.to(cuda)).double().cpu(), P.moe_ff(h.double(), w, "l0.mlp.", mlp), 2e-5)


# ---- the model on the engine ----------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full32(cuda):
    model, w = build(FULL, torch.float32, cuda, 11)
    prompts = {"a": tokens(150, 131, 1), "b": tokens(37, 131, 2), "c": tokens(2, 131, 3), "d": tokens(75, 131, 4), "e": tokens(1, 131, 5)}
    want = {k: P.forward(v, w, FULL).numpy() for k, v in prompts.items()}
    return model, prompts, want


def test_whole_prompts_and_layers(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    for name in prompts:
        got = replay(eng, prompts, [[(name, len(prompts[name]))]])[name]
        assert_close(got, want[name], torch.float32, name)
    _, w = build(FULL, torch.float32, cuda, 11)
    _, layers = P.forward(prompts["b"], w, FULL, return_layers=True)
    seen = {}
    r = eng.new_request(prompts["b"])
    eng.execute([(r, 37)], after_layer=lambda i, xs: seen.__setitem__(i, xs.sum(1).double().cpu()))
    eng.finish(r)
    for i in range(len(FULL["layers"])):
        assert (seen[i] - layers[i]).abs().max() < 2e-4 * layers[i].abs().max(), i


def test_decode_token_by_token_equals_prefill(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    got = replay(eng, prompts, [[("b", 1)] for _ in range(37)])["b"]
    assert_close(got, want["b"], torch.float32)
    got = replay(eng, prompts, [[("a", 100)]] + [[("a", 1)] for _ in range(50)])["a"]      # long decoding across windows and pages
    assert_close(got, want["a"], torch.float32)


@pytest.mark.parametrize("sizes", [[2] * 75, [3, 16, 1, 15, 17, 2, 32, 31, 2, 2, 29], [149, 1], [16] * 9 + [6]])
def test_portions(cuda, full32, sizes):
    model, prompts, want = full32
    assert sum(sizes) == 150
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    got = replay(eng, prompts, [[("a", n)] for n in sizes])["a"]
    assert_close(got, want["a"], torch.float32)


def test_mixed_batches_and_reuse(cuda, full32):
    """Unequal requests side by side, portions beside single tokens; the pools are too small for all of them at once, so
    pages and state slots of finished requests are taken again (by requests that must not see what was left there)."""
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 16, max_seqs=3)
    schedule = [[("a", 40), ("b", 30)], [("a", 1), ("b", 7), ("c", 2)], [("a", 60), ("d", 5)], [("d", 1), ("a", 1)], [("d", 69), ("a", 48), ("e", 1)]]
    got = replay(eng, prompts, schedule)
    for name in prompts:
        assert_close(got[name], want[name], torch.float32, name)
    assert eng.slots.num_free() == 3 and eng.pages.num_free_blocks() == 16
    again = replay(eng, prompts, [[("d", 75), ("b", 37), ("c", 2)], [("a", 100)], [("a", 50)]])    # every slot and page has been used before
    for name in ("a", "b", "d"):
        assert_close(again[name], want[name], torch.float32, name)


def test_batch_of_decodes_matches_each_alone(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 20, max_seqs=4)
    schedule = [[("a", 140), ("b", 27), ("d", 65)]] + [[("a", 1), ("b", 1), ("d", 1)] for _ in range(10)]
    got = replay(eng, prompts, schedule)
    for name in ("a", "b", "d"):
        assert_close(got[name], want[name], torch.float32, name)


@pytest.mark.parametrize("page_size", [4, 64])
def test_other_page_sizes(cuda, page_size):
    model, w = build(DENSE_ONLY, torch.float32, cuda, 21, page_size=page_size)
    p = {"x": tokens(90, 131, 8), "y": tokens(33, 131, 9)}
    eng = engine.Engine(model, max_tokens=192, max_seqs=2)
    got = replay(eng, p, [[("x", 50), ("y", 3)], [("x", 1), ("y", 30)], [("x", 39)]])
    for k in p:
        assert_close(got[k], P.forward(p[k], w, DENSE_ONLY).numpy(), torch.float32, k)


def test_bfloat16_model(cuda):
    model, w = build(FULL, torch.bfloat16, cuda, 11)
    p = {"a": tokens(120, 131, 1), "b": tokens(40, 131, 2)}
    eng = engine.Engine(model, max_tokens=176, max_seqs=2)
    got = replay(eng, p, [[("a", 70), ("b", 5)], [("a", 1), ("b", 35)], [("a", 49)]])
    for k in p:
        assert_close(got[k], P.forward(p[k], w, FULL).numpy(), torch.bfloat16, k)


def test_greedy_generation_through_the_scheduler(cuda):
    """engine.generate: waiting queue, admission by free slots and pages, chunked prefill under a small step budget,
    device top-1 sampling.  The plain model must make the same greedy choices (checked where its margin is clear)."""
    model, w = build(DENSE_ONLY, torch.float32, cuda, 31)
    prompts = [tokens(n, 131, 40 + n) for n in (30, 5, 61, 1, 17)]
    eng = engine.Engine(model, max_tokens=16 * 8, max_seqs=2, max_step_tokens=24)
    outs = eng.generate(prompts, engine.SamplingParams(max_new_tokens=6))
    assert eng.slots.num_free() == 2 and eng.pages.num_free_blocks() == 8 and not eng.scheduler.running
    for p, out in zip(prompts, outs):
        assert len(out) == 6
        seq = list(p)
        for t in out:
            lg = P.forward(seq, w, DENSE_ONLY)[-1]
            top2 = lg.topk(2).values
            if top2[0] - top2[1] > 1e-3:
                assert int(lg.argmax()) == t
            seq.append(t)


def test_config_rejects_unknown_branches():
    bad = make_cfg([lightning_layer()])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(NotImplementedError):
        nisasun.NisasunConfig(bad)
