"""Kilizen on the step engine against the plain float64 restatement (tests/kilizen_plain.py): every mechanism alone,
then whole prompts, token-by-token decoding, portions of many sizes, mixed batches, reused pages and slots, edges of the
window and of the kept first tokens, far keys, sinks, long decoding, and greedy generation through the scheduler.
Small random configurations made here; f32 mode is held to f32 rounding, bf16 mode to bf16 rounding."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kilizen_plain as P
from mistralrs_b200 import engine, kilizen, mixers, seq_ops as K

pytestmark = pytest.mark.gpu
F64 = torch.float64

YARN = {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}


def attention_layer(heads=6, kv_heads=2, dim=40, rot_dims=16, base=10000.0, scaling=YARN, window=10, keep_first=3, scale=0.3, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def attention2_layer(heads=4, kv_heads=2, dim=24, vdim=40, rot_dims=24, base=5000.0, scale=0.25, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def mlstm_layer(heads=3, dim=24, vdim=40, cap=8.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


DENSE = {"kind": "dense", "ff": 112}


def moe(experts=8, top=3, ff=48, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def make_cfg(layers, width=72, vocab=131, eps=1e-5, loop=None):
    cj = {"architecture": "Kilizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cj["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cj


FULL = make_cfg([mlstm_layer(mlp=DENSE), attention_layer(mlp=moe()), attention2_layer(mlp=moe(experts=6, top=2, shared=0)),
                 mlstm_layer(heads=2, dim=16, vdim=16, cap=3.0, mlp=None), attention_layer(kv_heads=6, window=17, keep_first=0, scaling=None, mlp=DENSE),
                 attention2_layer(kv_heads=1, rot_dims=8, mlp=DENSE)], loop=(1, 4, 3))
DENSE_ONLY = make_cfg([attention2_layer(mlp=DENSE), mlstm_layer(mlp=DENSE), attention_layer(mlp=None)])


def build(cj, dtype, device, seed=0, page_size=16, edit=None):
    cfg = kilizen.KilizenConfig(copy.deepcopy(cj))
    tensors = kilizen.random_tensors(cfg, seed)
    if edit:
        edit(tensors)
    model = kilizen.KilizenModel(cfg, tensors, device, dtype, page_size=page_size)
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
        assert (e > TOL[dtype]).sum() <= max(1, 0.03 * e.size) and np.median(e) < TOL[dtype] / 3, (what, float(e.max()), float(np.median(e)))


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


def close_rows(got, want, tol):
    """Every row within tol.  At bf16 tolerances a row or two may sit where the mechanism is ill-conditioned (a unit norm
    of a nearly cancelled sum amplifies the rounding of its inputs): 2 % of the rows may reach three times tol."""
    e = (got - want).norm(dim=-1) / want.norm(dim=-1).mean()
    if tol >= 1e-2:
        assert (e > tol).double().mean() <= 0.02 and e.max() < 3 * tol, (float(e.max()), int(e.argmax()))
    else:
        assert e.max() < tol, (float(e.max()), int(e.argmax()))


# ---- mechanisms alone ------------------------------------------------------------------------------------------------
def seq_batch(device, portions, page_size=16):
    """One step of several sequences: portions = [(n_new, past, slot, first_page)]."""
    counts, pasts, slots, tables, slot_map = [], [], [], [], []
    for n, past, slot, first_page in portions:
        pages = list(range(first_page, first_page + -(-(past + n) // page_size)))
        counts.append(n), pasts.append(past), slots.append(slot), tables.append(pages)
        slot_map += [pages[(past + i) // page_size] * page_size + (past + i) % page_size for i in range(n)]
    return engine.StepBatch(device, [0] * sum(counts), counts, pasts, slots, tables, np.asarray(slot_map, dtype=np.int64), [])


def plain_mixer(layer, h, w, eps):
    return P.MIXERS[layer["type"]](h, w, "l0.mix.", layer["mixer"], eps)


def mixer_case(cuda, layer, dtype, T, portions, seed=3, edit=None, width=72, h=None, pages=80):
    """Run layer 0's mixer alone over `portions` of one sequence; returns (got [T, W], want [T, W])."""
    cj = make_cfg([layer], width=width)
    model, w = build(cj, dtype, cuda, seed, edit=edit)
    if h is None:
        h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    h = h.to(dtype)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(2, 16 * pages, dtype, cuda)
    out, at = [], 0
    for n in portions:
        out.append(mixer.forward(h[at:at + n].to(cuda).contiguous(), seq_batch(cuda, [(n, at, 1, 1)]), cache).float().cpu())
        at += n
    assert at == T
    return torch.cat(out).double(), plain_mixer(layer, h.double(), w, cj["norm"]["eps"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [50, 64, 136, 9])
def test_tanh_norm_residual(cuda, dtype, W):
    g = torch.Generator().manual_seed(W)
    T = 9
    x, x0 = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g)
    y = (3.0 * torch.randn(T, W, generator=g)).to(dtype)
    norms = [(torch.rand((), generator=g) + 0.3, torch.randn(W, generator=g), torch.randn(W, generator=g)) for _ in range(2)]
    d = lambda n: tuple(t.to(cuda) for t in n)
    dyt = lambda z, n: torch.tanh(n[0].double() * z) * n[1].double() + n[2].double()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    rows = torch.tensor([4, 0, 8], dtype=torch.int32, device=cuda)
    got = K.tanh_norm_rows(x.to(cuda), d(norms[0]), dtype, rows=rows)
    assert (got.double().cpu() - dyt(x.double(), norms[0])[[4, 0, 8]]).abs().max() < tol
    xd = x.to(cuda).clone()
    got_n = K.residual_tanh_norm(xd, y.to(cuda), post=d(norms[0]), extra=x0.to(cuda), nxt=d(norms[1]))
    want_x = x.double() + dyt(y.double(), norms[0]) + x0.double()
    assert (xd.double().cpu() - want_x).abs().max() < 1e-5                       # the residual stays f32 in either mode
    assert (got_n.double().cpu() - dyt(want_x, norms[1])).abs().max() < tol
    xe = x.to(cuda).clone()                                                      # the same in two passes, parts left out
    K.residual_tanh_norm(xe, y.to(cuda), post=d(norms[0]))
    got_2 = K.residual_tanh_norm(xe, extra=x0.to(cuda), nxt=d(norms[1]), dtype=dtype)
    assert torch.equal(xe, xd) and torch.equal(got_2, got_n)


def test_rotation_table_with_scaled_frequencies(cuda):
    for rot in ({"base": 10000.0, "dims": 16, "scaling": YARN}, {"base": 500.0, "dims": 6}, {"base": 1e6, "dims": 64, "scaling": {"factor": 3.0, "original": 4096, "fast": 32.0, "slow": 2.0}}):
        r = mixers.Rotation(rot["dims"], rot["base"], rot.get("scaling"), cuda)
        pos = torch.tensor([0, 1, 63, 64, 1000, 70000], dtype=torch.int32, device=cuda)
        b = type("B", (), {})()
        b.pos_of_tok = pos
        got = r.table(b).double().cpu()
        f, mag = P.rotation_frequencies(rot)
        a = pos.cpu().double()[:, None] * f[None, :]
        assert (got[..., 0] - torch.cos(a) * mag).abs().max() < 2e-7 and (got[..., 1] - torch.sin(a) * mag).abs().max() < 2e-7
        if rot.get("scaling"):
            plain, _ = P.rotation_frequencies({"base": rot["base"], "dims": rot["dims"]})
            assert (f != plain).any() and (f == plain).any() and mag > 1.0      # the ramp has both ends inside these sizes


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[90], [1] * 30, [5, 2, 17, 1, 33, 2]])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_attention_mixers(cuda, dtype, tol, portions, kind):
    layer = attention_layer() if kind == "attention" else attention2_layer()
    got, want = mixer_case(cuda, layer, dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [attention_layer(kv_heads=6), attention_layer(kv_heads=1, heads=4), attention_layer(rot_dims=40), attention_layer(rot_dims=0),
                                   attention_layer(dim=8, rot_dims=2), attention_layer(dim=136, rot_dims=64, window=1, keep_first=1),
                                   attention_layer(window=0), attention_layer(window=7, keep_first=40), attention_layer(keep_first=0, scaling=None),
                                   attention2_layer(kv_heads=4), attention2_layer(kv_heads=1), attention2_layer(dim=8, vdim=136, rot_dims=4),
                                   attention2_layer(dim=72, vdim=8, rot_dims=0), attention2_layer(dim=33, vdim=7, rot_dims=32)])
def test_attention_other_sizes(cuda, layer):
    got, want = mixer_case(cuda, layer, torch.float32, 45, [20, 1, 1, 3, 20])
    close_rows(got, want, 3e-5)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
@pytest.mark.parametrize("portions", [[300], [70, 1, 200, 29], [3, 297]])
def test_attention_prompt_kernels(cuda, d, kind, portions):
    """bf16 with equal head sizes of 64 / 128: portions of 32 tokens or more, first or later, run on the tensor-core
    prompt kernel (sink, window and kept first tokens included), which reads keys and values — with values that are the
    keys: the unnormed keys — from the pages; single tokens in between take the (token, head) kernel."""
    if kind == "attention":
        layer = attention_layer(heads=4, kv_heads=2, dim=d, rot_dims=32, window=40, keep_first=5, scale=d ** -0.5)   # later query tiles: kept tile + window tiles
    else:
        layer = attention2_layer(heads=4, kv_heads=2, dim=d, vdim=d, rot_dims=d, scale=d ** -0.5)
    got, want = mixer_case(cuda, layer, torch.bfloat16, 300, portions, width=64)
    close_rows(got, want, 3e-2)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (40, 1), (64, 64), (65, 100), (200, 130), (17, 300)])
def test_prompt_kernel_tile_borders(cuda, d, window, keep):
    """The tensor-core prompt kernel alone against the plain softmax: windows and kept counts on, beside and across its
    64-key tiles and 128-row query tiles; portions of 33 / 128 / 129 / 400 rows in one flat batch, two of which continue a
    sequence whose earlier keys are only in the pages (70 and 130 of them, neither a multiple of a tile or a page); a
    sink on one head only; rows of short portions in between stay untouched."""
    g = torch.Generator().manual_seed(window * 7 + keep)
    H, G, page = 4, 2, 16
    seqs = [(33, 0), (128, 70), (3, 9), (129, 0), (400, 130)]            # (new rows, cached before)
    portions, first_page = [], 1
    for i, (n, past) in enumerate(seqs):
        portions.append((n, past, i, first_page))
        first_page += -(-(past + n) // page)
    batch = seq_batch(cuda, portions, page_size=page)
    assert [x[1] for x in batch.long] == [33, 128, 129, 400]
    n_rows = sum(n for n, _ in seqs)
    q = torch.randn(n_rows, H * d + 8, generator=g).to(torch.bfloat16)      # a row stride of its own
    k_cache = torch.zeros(first_page * page, G, d, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    ks, vs = [], []
    for n, past, _, fp in portions:
        kk, vv = torch.randn(past + n, G, d, generator=g).to(torch.bfloat16), torch.randn(past + n, G, d, generator=g).to(torch.bfloat16)
        k_cache[fp * page:fp * page + past + n], v_cache[fp * page:fp * page + past + n] = kk, vv      # its pages are consecutive here
        ks.append(kk), vs.append(vv)
    sink = torch.tensor([1.5, -50.0, 0.0, -1.0])
    out = torch.zeros(n_rows, H * d, dtype=torch.bfloat16, device=cuda)
    K.prompt_attention(q.to(cuda), 0, k_cache.to(cuda), v_cache.to(cuda), batch, page, H, G, d, d ** -0.5, window, keep, sink.to(cuda), out)
    mask = {"size": window, "keep_first": keep} if window else None
    row0 = 0
    for (n, past), kk, vv in zip(seqs, ks, vs):
        got = out[row0:row0 + n].double().cpu()
        if n < 32:
            assert (got == 0).all()
        else:
            qq = torch.zeros(past + n, H, d, dtype=F64)
            qq[past:] = q[row0:row0 + n, :H * d].double().view(n, H, d)
            want = P.sink_attention(qq, kk.double(), vv.double(), d ** -0.5, sink.double(), P.visible(past + n, mask))[past:]
            close_rows(got, want, 2e-2)
        row0 += n


def test_prompt_kernel_takes_several_sequences(cuda):
    """Two sequences start in one step beside a long portion that continues a third: one launch covers all three."""
    layer = attention_layer(heads=2, kv_heads=1, dim=64, rot_dims=16, window=40, keep_first=70, scale=0.125)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.bfloat16, cuda, 7)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(3, 16 * 40, torch.bfloat16, cuda)
    g = torch.Generator().manual_seed(7)
    hs = [torch.randn(n, 64, generator=g).to(torch.bfloat16) for n in (150, 33, 60)]
    mixer.forward(hs[2][:20].to(cuda).contiguous(), seq_batch(cuda, [(20, 0, 2, 30)]), cache)
    b = seq_batch(cuda, [(150, 0, 0, 1), (40, 20, 2, 30), (33, 0, 1, 12)])
    assert len(b.fresh) == 2 and len(b.long) == 3
    got = mixer.forward(torch.cat([hs[0], hs[2][20:], hs[1]]).to(cuda).contiguous(), b, cache).double().cpu()
    want = [plain_mixer(layer, h.double(), w, 1e-5) for h in hs]
    close_rows(got, torch.cat([want[0], want[2][20:], want[1]]), 3e-2)


def aligned_pair_edit(kind, dk, width, rot_dims, heads, kv_heads):
    """Projections that copy the input's entries [rot_dims, dk) into every query and key head (rotated entries stay 0) and
    unit norm weights: a query then scores high with exactly the keys whose input shares its direction there."""
    def edit(t):
        eye = torch.zeros(dk, width)
        for i in range(rot_dims, dk):
            eye[i, i] = 1.0
        t["l0.mix.q"].copy_(eye.repeat(heads, 1).to(torch.bfloat16))
        t["l0.mix.k"].copy_(eye.repeat(kv_heads, 1).to(torch.bfloat16))
        t["l0.mix.q.norm"].fill_(1.0)
        t["l0.mix.k.norm"].fill_(1.0)
        for n in ("l0.mix.q.b", "l0.mix.k.b"):
            if n in t:
                t[n].zero_()
    return edit


@pytest.mark.parametrize("edge", ["window", "keep_first"])
@pytest.mark.parametrize("distance", [-2, -1, 0, 1])
@pytest.mark.parametrize("decoded", [False, True])
def test_window_and_kept_edges_show(cuda, edge, distance, decoded):
    """One earlier token shares the last query's direction, all others are near-orthogonal, and the score scale is large:
    the output is that token's value while it is in sight and something else one step later.  The token sits around the
    window's far edge, or around the end of the kept first tokens far outside the window."""
    window, keep, T = 24, 9, 120
    target = T - 1 - (window - 1) - distance if edge == "window" else keep - 1 + distance     # distance <= 0: in sight
    layer = attention_layer(heads=2, kv_heads=1, dim=32, rot_dims=8, window=window, keep_first=keep, scale=1.5)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.float32, cuda, 9, edit=aligned_pair_edit("attention", 32, 64, 8, 2, 1))
    h = torch.randn(T, 64, generator=torch.Generator().manual_seed(9))
    h[target, :32] = 3.0 * h[T - 1, :32]             # the same key once normed; as a value (the key as projected) three times as long
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 10, torch.float32, cuda)
    cuts = [(0, T - 3), (T - 3, T - 2), (T - 2, T - 1), (T - 1, T)] if decoded else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), seq_batch(cuda, [(b - a, a, 0, 1)]), cache).cpu() for a, b in cuts]).double()
    want = plain_mixer(layer, h.double(), w, 1e-5)
    close_rows(got, want, 3e-5)
    other = copy.deepcopy(layer)
    if edge == "window":
        other["mixer"]["mask"]["size"] = window + distance if distance > 0 else window - 1 + distance     # the target crosses the edge
    else:
        other["mixer"]["mask"]["keep_first"] = keep + distance if distance > 0 else keep - 1 + distance
    assert (plain_mixer(other, h.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()   # an edge one off would show


@pytest.mark.parametrize("target", [0, 15, 16, 17, 333])
@pytest.mark.parametrize("decoded", [False, True])
def test_far_key_among_hundreds(cuda, target, decoded):
    """Causal attention: one key far back (the first token, the two sides of a page border, somewhere in the middle)
    matches the last query; hundreds of others do not."""
    T = 700
    layer = attention2_layer(heads=2, kv_heads=1, dim=32, vdim=24, rot_dims=8, scale=1.5)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.float32, cuda, 13, edit=aligned_pair_edit("attention_2", 32, 64, 8, 2, 1))
    h = torch.randn(T, 64, generator=torch.Generator().manual_seed(13))
    h[target, :32] = h[T - 1, :32]
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 50, torch.float32, cuda)
    cuts = [(0, T - 2), (T - 2, T - 1), (T - 1, T)] if decoded else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), seq_batch(cuda, [(b - a, a, 0, 1)]), cache).cpu() for a, b in cuts]).double()
    want = plain_mixer(layer, h.double(), w, 1e-5)
    close_rows(got[-3:], want[-3:], 3e-5)
    h2 = h.clone()
    h2[target, :32] = torch.randn(32, generator=torch.Generator().manual_seed(1))
    assert (plain_mixer(layer, h2.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()     # a lost key would show


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_sink_shows(cuda, kind):
    """A large sink on one head takes most of that head's softmax mass; no sink on the other.  Left out, or scaled like a
    score, the output would differ by far."""
    def edit(t):
        t["l0.mix.sink"].copy_(torch.tensor([6.0, -30.0]).to(torch.bfloat16))
    layer = attention_layer(heads=2, kv_heads=1, dim=24, rot_dims=8, scale=0.1) if kind == "attention" else attention2_layer(heads=2, kv_heads=2, scale=0.1)
    for portions in ([40], [30] + [1] * 10):
        got, want = mixer_case(cuda, layer, torch.float32, 40, portions, edit=edit)
        close_rows(got, want, 3e-5)
    cj = make_cfg([layer])
    _, w = build(cj, torch.float32, cuda, 3, edit=edit)
    h = torch.randn(40, 72, generator=torch.Generator().manual_seed(3)).double()
    w2 = dict(w)
    w2["l0.mix.sink"] = torch.full((2,), -1e4, dtype=F64)
    diff = (plain_mixer(layer, h, w2, 1e-5) - plain_mixer(layer, h, w, 1e-5)).norm(dim=-1)
    assert diff.min() > 0.2 * plain_mixer(layer, h, w, 1e-5).norm(dim=-1).mean()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[150], [1] * 40, [7, 2, 33, 1, 64, 2, 41]])
def test_mlstm_mixer(cuda, dtype, tol, portions):
    got, want = mixer_case(cuda, mlstm_layer(), dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [mlstm_layer(heads=1, dim=8, vdim=8), mlstm_layer(heads=2, dim=136, vdim=72, cap=30.0), mlstm_layer(heads=5, dim=16, vdim=7, cap=0.5),
                                   mlstm_layer(heads=2, dim=40, vdim=127, cap=2.0)])
def test_mlstm_other_sizes(cuda, layer):
    got, want = mixer_case(cuda, layer, torch.float32, 45, [20, 1, 1, 3, 20])
    close_rows(got, want, 3e-5)


def test_mlstm_gates_that_saturate(cuda):
    """Large gate pre-activations: the soft cap and the running maximum keep everything finite, the maximum starts from 0
    (not from the first input gate), and a portion that continues must pick the carried maximum up."""
    def edit(t):
        t["l0.mix.i"].mul_(40.0)
        t["l0.mix.f"].mul_(40.0)
        t["l0.mix.i.b"].copy_(torch.tensor([-6.0, 0.0, 6.0]).to(torch.bfloat16))
    for portions in ([60], [1] * 12 + [48], [33, 2, 25]):
        got, want = mixer_case(cuda, mlstm_layer(cap=12.0), torch.float32, 60, portions, edit=edit)
        assert torch.isfinite(got).all()
        close_rows(got, want, 1e-4)


def test_mlstm_first_token_survives_far(cuda):
    """Forget gates held open (a large forget bias) and input gates shut after the first token: 300 tokens later the
    output still is the first token's value, through portions, single tokens and segment-wise scanning."""
    def edit(t):
        t["l0.mix.f"].zero_()
        t["l0.mix.f.b"].fill_(30.0)
        t["l0.mix.i"].zero_()
        t["l0.mix.i"][:, 0] = 4.0
        t["l0.mix.i.b"].fill_(-20.0)
    layer = mlstm_layer(heads=2, dim=16, vdim=16, cap=50.0)
    T = 300
    h = torch.randn(T, 32, generator=torch.Generator().manual_seed(5)) * 0.1
    h[:, 0] = 0.0
    h[0, 0] = 8.0                                   # only the first token opens its input gate
    got, want = mixer_case(cuda, layer, torch.float32, T, [250, 1, 49], seed=5, edit=edit, width=32, h=h)
    close_rows(got, want, 1e-4)
    _, w = build(make_cfg([layer], width=32), torch.float32, cuda, 5, edit=edit)
    without = plain_mixer(layer, h.double()[1:], w, 1e-5)
    assert (want[1:] - without).norm(dim=-1)[-1] > 0.1 * want[-1].norm()      # the test would see a lost first token


def test_scan_in_segments(cuda, monkeypatch):
    """Long portions are scanned as segments side by side: made to happen on short ones here, with ragged last segments
    and a state (and running maximum) carried in from an earlier portion."""
    monkeypatch.setattr(K, "SCAN_SEGMENT", 16)
    monkeypatch.setattr(K, "SCAN_SEGMENT_MIN_TOKENS", 40)
    got, want = mixer_case(cuda, mlstm_layer(), torch.float32, 150, [70, 3, 77])
    close_rows(got, want, 5e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_dense_ff(cuda, dtype, tol):
    cj = make_cfg([mlstm_layer(mlp=DENSE)])
    model, w = build(cj, dtype, cuda, 2)
    h = torch.randn(21, 72, generator=torch.Generator().manual_seed(2)).to(dtype)
    got = model.layers[0].mlp.forward(h.to(cuda)).double().cpu()
    close_rows(got, P.dense_ff(h.double(), w, "l0.mlp."), tol)


@pytest.mark.parametrize("kw", [dict(), dict(experts=12, top=4, shared=0), dict(experts=6, top=6), dict(experts=5, top=1, shared=8), dict(experts=33, top=2, ff=8)])
@pytest.mark.parametrize("T", [3, 150])     # few pairs per expert: weight-streaming kernels; many: rows sorted by expert
def test_routed_experts(cuda, kw, T):
    mlp = moe(**kw)
    cj = make_cfg([mlstm_layer(mlp=mlp)])
    model, w = build(cj, torch.float32, cuda, 4)
    h = torch.randn(T, 72, generator=torch.Generator().manual_seed(T)).to(torch.bfloat16).float()
    ff = model.layers[0].mlp
    idx, wt = ff.route(h.to(cuda))
    want_idx, want_wt = P.route(h.double(), w, "l0.mlp.", mlp["router"])
    assert torch.equal(idx.cpu().long(), want_idx)                              # in the order of their logits
    assert (wt.double().cpu() - want_wt).abs().max() < 1e-6
    if 1 < mlp["router"]["top"] < mlp["router"]["experts"]:                   # softmax over the chosen ones only
        every = torch.softmax(h.double() @ w["l0.mlp.router"].T, -1).gather(1, want_idx)
        assert (every - want_wt).abs().max() > 0.05
    close_rows(ff.forward(h.to(cuda)).double().cpu(), P.moe_ff(h.double(), w, "l0.mlp.", mlp), 2e-5)


# ---- the model on the engine ----------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full32(cuda):
    model, w = build(FULL, torch.float32, cuda, 11)
    prompts = {"a": tokens(150, 131, 1), "b": tokens(37, 131, 2), "c": tokens(2, 131, 3), "d": tokens(75, 131, 4), "e": tokens(1, 131, 5)}
    want = {k: P.forward(v, w, FULL).numpy() for k, v in prompts.items()}
    return model, prompts, want


def test_layer_order_with_a_repeated_range():
    cfg = kilizen.KilizenConfig(copy.deepcopy(FULL))
    assert cfg.runs() == P.layer_runs(FULL) == [(0, False), (1, False), (2, False), (3, False), (1, True), (2, False), (3, False), (1, True),
                                                (2, False), (3, False), (4, False), (5, False)]
    once = kilizen.KilizenConfig(copy.deepcopy(DENSE_ONLY))
    assert once.runs() == [(0, False), (1, False), (2, False)]


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
    hooked = eng.execute([(r, 37)], after_layer=lambda i, x: seen.__setitem__(i, x.double().cpu())).cpu().numpy()
    eng.finish(r)
    assert len(seen) == len(layers) == 12                     # one per layer RUN: the repeated range counts every time
    for i in range(len(layers)):
        assert (seen[i] - layers[i]).abs().max() < 2e-4 * layers[i].abs().max(), i
    assert_close(hooked, want["b"][-1:], torch.float32)       # the split residual pass gives what the fused one gives


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
    """Also the captured-graph path: from its second occurrence a batch of single tokens replays a CUDA graph."""
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 20, max_seqs=4)
    schedule = [[("a", 140), ("b", 27), ("d", 65)]] + [[("a", 1), ("b", 1), ("d", 1)] for _ in range(10)]
    got = replay(eng, prompts, schedule)
    for name in ("a", "b", "d"):
        assert_close(got[name], want[name], torch.float32, name)
    assert 3 in eng._graphs or not eng.decode_graphs


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


AWKWARD = make_cfg([attention2_layer(heads=3, kv_heads=3, dim=9, vdim=5, rot_dims=4, mlp={"kind": "dense", "ff": 51}),
                    mlstm_layer(heads=2, dim=7, vdim=3, cap=1.5, mlp=moe(experts=3, top=2, ff=13, shared=11)),
                    attention_layer(heads=2, kv_heads=1, dim=10, rot_dims=10, window=5, keep_first=2, mlp=moe(experts=4, top=1, ff=6, shared=0))],
                   width=45, vocab=77, loop=(0, 3, 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_align_with_nothing(cuda, dtype):
    """Odd width, odd head sizes, odd feed-forward sizes: every kernel falls back to its unvectorised path, rows of the
    activations start on 2-byte boundaries in bf16; the whole list of layers runs twice."""
    model, w = build(AWKWARD, dtype, cuda, 17)
    p = {"x": tokens(70, 77, 8), "y": tokens(33, 77, 9)}
    eng = engine.Engine(model, max_tokens=128, max_seqs=2)
    got = replay(eng, p, [[("x", 40), ("y", 3)], [("x", 1), ("y", 30)], [("x", 29)]])
    for k in p:
        assert_close(got[k], P.forward(p[k], w, AWKWARD).numpy(), dtype, k)


def test_model_folder_through_the_command_lines(cuda, tmp_path):
    """config.json + model.safetensors on disk -> the registry picks the class; the step-trace replay tool writes the
    logits it is asked for (requests cut into portions, a finished request's pages reused), and the generate command
    decodes greedily through the scheduler."""
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cj = copy.deepcopy(DENSE_ONLY)
    cj["loop"] = {"start": 0, "stop": 2, "times": 2}
    tensors = kilizen.random_tensors(kilizen.KilizenConfig(copy.deepcopy(cj)), 41)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cj))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    w = {k: v.to(F64) for k, v in tensors.items()}
    a, b = tokens(50, 131, 1), tokens(20, 131, 2)
    want_a, want_b = P.forward(a, w, cj).numpy(), P.forward(b, w, cj).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": []}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}, {"id": "a", "tokens": a[31:], "want": [18]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [19]}], "end": ["c"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == ["done %d" % i for i in range(4)]
    read = lambda i: np.fromfile(out / ("%d.f32" % i), dtype="<f4").reshape(-1, 131)
    assert_close(read(0), want_a[[0, 29]], torch.float32)
    assert_close(read(1), want_b[[18]], torch.float32)
    assert_close(read(2), np.stack([want_b[19], want_a[49]]), torch.float32)
    assert_close(read(3), want_b[[19]], torch.float32)
    g = subprocess.run([sys.executable, os.path.join(root, "bin", "mrs-b200"), "generate", "--model", str(folder), "--dtype", "float32", "--max-new", "3",
                        "--prompt", " ".join(map(str, b))], capture_output=True, text=True, timeout=900)
    assert g.returncode == 0, g.stderr[-2000:]
    gen = json.loads(g.stdout.strip().split("\n")[-1])["generated"]
    seq = list(b)
    for t in gen:
        lg = torch.from_numpy(P.forward(seq, w, cj).numpy()[-1])
        top2 = lg.topk(2).values
        if top2[0] - top2[1] > 1e-3:
            assert int(lg.argmax()) == t
        seq.append(t)
    assert len(gen) == 3


def test_config_rejects_unknown_branches():
    bad = make_cfg([mlstm_layer()])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(NotImplementedError):
        kilizen.KilizenConfig(bad)
    bad = make_cfg([mlstm_layer(), mlstm_layer()], loop=(1, 1, 2))
    with pytest.raises(ValueError):
        kilizen.KilizenConfig(bad)
