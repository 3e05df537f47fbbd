"""Plain, slow restatement of the Kilizen design in float64 on the CPU: one function per mechanism, whole
sequences at once, no cache, no batching.  TEST INFRASTRUCTURE: it shares no code with the package; the GPU tests
compare the package's kernels, cache and scheduler with it.

Weights are a dict name -> float64 tensor with the checkpoint's names (`l<i>.mix.q`, `l<i>.norm1.alpha`, ...); the
configuration is the parsed config.json."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def tanh_norm(x, w, name):
    """Dynamic Tanh: no statistics of x at all."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


# ---- rotation ----------------------------------------------------------------------------------------
def rotation_frequencies(rot):
    """Angular frequency per rotated pair and the factor on cos / sin (1 without scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    turn = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(turn(float(sc["fast"]))), 0), min(math.ceil(turn(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x, rot, first_pos=0):
    """x [T, heads, d]: the first rot.dims entries of every head turn in pairs (i, i + dims/2); the rest pass."""
    if not rot:
        return x
    T, dims = x.shape[0], int(rot["dims"])
    half = dims // 2
    f, mag = rotation_frequencies(rot)
    a = (torch.arange(T, dtype=F64) + first_pos)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- softmax attention with a sink -------------------------------------------------------------------
def visible(T, mask):
    """[T, T] boolean: query i sees key j.  mask None: causal; else a window of mask.size plus the first keep_first."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if mask:
        seen &= (i - j < int(mask["size"])) | (j < int(mask.get("keep_first", 0)))
    return seen


def sink_attention(q, k, v, scale, sink, seen):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], sink [H]; the softmax denominator holds exp(sink) once more."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[a])
        e = torch.exp(s - top)
        out.append((e / (e.sum(-1, keepdim=True) + torch.exp(sink[a] - top))) @ v[:, g])
    return torch.cat(out, dim=1)


def attention_values_are_keys(h, w, pre, m, eps):
    """Mixer `attention`: no value projection (values = keys as projected), per-head query / key norm, partial rotation
    with scaled frequencies, window + kept first tokens, sink."""
    T = h.shape[0]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).view(T, H, dk)
    k = (h @ w[pre + "k"].T).view(T, G, dk)
    v = k
    q = rotate(unit_rms(q, eps) * w[pre + "q.norm"], m.get("rot"))
    k = rotate(unit_rms(k, eps) * w[pre + "k.norm"], m.get("rot"))
    o = sink_attention(q, k, v, float(m["scale"]), w[pre + "sink"], visible(T, m.get("mask")))
    return o @ w[pre + "o"].T


def attention_with_biases(h, w, pre, m, eps):
    """Mixer `attention_2`: biased projections, query / key norm over the whole projection, rotation, causal, sink."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    q = rotate((unit_rms(q, eps) * w[pre + "q.norm"]).view(T, H, dk), m.get("rot"))
    k = rotate((unit_rms(k, eps) * w[pre + "k.norm"]).view(T, G, dk), m.get("rot"))
    o = sink_attention(q, k, v, float(m["scale"]), w[pre + "sink"], visible(T, m.get("mask")))
    return o @ w[pre + "o"].T + w[pre + "o.b"]


# ---- matrix memory -----------------------------------------------------------------------------------
def stabilised_matrix_memory(q, k, v, log_in, log_forget):
    """One head.  q, k [T, dk], v [T, dv], gates [T] (logarithms).  Running maximum from 0."""
    T, dk = k.shape
    S, n, m = torch.zeros(dk, v.shape[1], dtype=F64), torch.zeros(dk, dtype=F64), torch.zeros((), dtype=F64)
    out = []
    for t in range(T):
        m_new = torch.maximum(log_forget[t] + m, log_in[t])
        keep, take = torch.exp(log_forget[t] + m - m_new), torch.exp(log_in[t] - m_new)
        S = keep * S + take * torch.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        out.append(S.T @ q[t] / (torch.maximum(torch.abs(n @ q[t]), torch.exp(-m)) + 1e-6))
    return torch.stack(out)


def mlstm_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[pre + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, dk)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    o = torch.stack([stabilised_matrix_memory(q[:, a], k[:, a], v[:, a], gi[:, a], gf[:, a]) for a in range(H)], dim=1)
    o = unit_rms(o, eps).reshape(T, H * dv) * w[pre + "norm"]
    return (o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


# ---- feed-forwards -----------------------------------------------------------------------------------
def dense_ff(h, w, pre):
    return gelu_erf(h @ w[pre + "up"].T) @ w[pre + "down"].T


def small_expert(h, w, pre):
    return relu_squared(h @ w[pre + "up"].T) @ w[pre + "down"].T


def route(h, w, pre, r):
    """-> (experts [T, top], weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ w[pre + "router"].T
    val, idx = torch.topk(z, int(r["top"]), dim=-1)
    return idx, torch.softmax(val, -1)


def moe_ff(h, w, pre, mlp):
    idx, wt = route(h, w, pre, mlp["router"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t].tolist(), wt[t]):
            out[t] += g * small_expert(h[t:t + 1], w, pre + f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + small_expert(h, w, pre + "shared.")
    return out


# ---- the model ---------------------------------------------------------------------------------------
MIXERS = {"attention": attention_values_are_keys, "attention_2": attention_with_biases, "mlstm": mlstm_mixer}


def layer_runs(cfg):
    """The order in which layers run: the looped range `times` times in a row, then the rest.  -> [(layer, starts_pass)]
    where starts_pass is True for the first layer of every pass but the first."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop or int(loop.get("times", 1)) <= 1:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for p in range(times):
        runs += [(i, p > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(tokens, w, cfg, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x, seen = x0.clone(), []
    for i, starts_pass in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if starts_pass:
            x = x + x0
        y = MIXERS[L["type"]](tanh_norm(x, w, p + "norm1"), w, p + "mix.", L["mixer"], eps)
        x = x + tanh_norm(y, w, p + "norm1b")
        if L.get("mlp") is not None:
            hin = tanh_norm(x, w, p + "norm2")
            y = dense_ff(hin, w, p + "mlp.") if L["mlp"]["kind"] == "dense" else moe_ff(hin, w, p + "mlp.", L["mlp"])
            x = x + tanh_norm(y, w, p + "norm2b")
        seen.append(x)
    logits = tanh_norm(x, w, "final.norm") @ w["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits
