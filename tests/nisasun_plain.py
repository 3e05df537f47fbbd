"""Plain, slow restatement of the Nisasun design in float64 on the CPU: one function per mechanism, whole
sequences at once or token by token, no cache, no batching.  TEST INFRASTRUCTURE: it shares no code with the
package; the GPU tests compare the package's kernels, cache and scheduler with it.

Weights are a dict name -> float64 tensor with the checkpoint's names (`l<i>.mix.q`, `l<i>.hc1.mix`, ...);
the configuration is the parsed config.json."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def norm_around_zero(x, w, eps):
    """The layer norms and the final norm: the stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


# ---- hyper-connections -------------------------------------------------------------------------------
def streams_read(xs, w_in):
    """xs [T, S, W] -> the sublayer's input [T, W]."""
    return torch.einsum("s,tsw->tw", w_in, xs)


def streams_write(xs, w_mix, w_out, y):
    """All streams at once from the old ones; w_mix is [from, to]."""
    return torch.einsum("sr,tsw->trw", w_mix, xs) + w_out[None, :, None] * y[:, None, :]


# ---- lightning attention -----------------------------------------------------------------------------
def decayed_outer_recurrence(q, k, v, decay):
    """One head: S_t = decay_t S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, dk], v [T, dv], decay [T]."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    out = []
    for t in range(T):
        S = decay[t] * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def lightning_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T).view(T, H, dk)
    k = silu(h @ w[pre + "k"].T).view(T, H, dk)
    v = silu(h @ w[pre + "v"].T).view(T, H, dv)
    o = torch.stack([decayed_outer_recurrence(q[:, i], k[:, i], v[:, i], torch.full((T,), float(m["decay"][i]), dtype=F64))
                     for i in range(H)], dim=1).reshape(T, H * dv)
    o = unit_rms(o, eps) * w[pre + "norm"]
    return (o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


# ---- sliding-window attention with query/key norm ----------------------------------------------------
def window_attention(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, dk)
    k = (h @ w[pre + "k"].T).view(T, G, dk)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    q = unit_rms(q, eps) * w[pre + "q.norm"]
    k = unit_rms(k, eps) * w[pre + "k.norm"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    out = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out.append(torch.softmax(s, -1) @ v[:, g])
    return torch.cat(out, dim=1) @ w[pre + "o"].T


# ---- Mamba-2 ----------------------------------------------------------------------------------------
def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K] (last column multiplies the current token), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=F64), x])
    return sum(pad[j:j + T] * taps[:, j] for j in range(K)) + bias


def mamba2_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = h @ w[pre + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) * dt)
    ys = []
    for a in range(H):
        g = a // (H // G)
        y = decayed_outer_recurrence(C[:, g], B[:, g] * dt[:, a:a + 1], x[:, a], decay[:, a])
        ys.append(y + w[pre + "D"][a] * x[:, a])
    y = torch.cat(ys, dim=1) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    return (m["left_scale"] * window_attention(h, w, pre + "left.", m["left"], eps)
            + m["right_scale"] * mamba2_mixer(h, w, pre + "right.", m["right"], eps))


# ---- feed-forward -----------------------------------------------------------------------------------
def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """-> (chosen experts [T, top], their weights [T, top])."""
    s = torch.softmax(h @ w[pre + "router"].T, -1)
    choice = s + w[pre + "correction"]
    E, cnt, keep = r["experts"], r["groups"]["count"], r["groups"]["keep"]
    by_group = choice.view(-1, cnt, E // cnt)
    best = by_group.max(-1).values.topk(keep, dim=-1).indices
    allowed = torch.zeros(h.shape[0], cnt, dtype=torch.bool).scatter_(1, best, True)
    choice = by_group.masked_fill(~allowed[:, :, None], float("-inf")).reshape(-1, E)
    idx = choice.topk(r["top"], dim=-1).indices
    return idx, s.gather(1, idx)


def moe_ff(h, w, pre, mlp):
    idx, wt = route(h, w, pre, mlp["router"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            p = f"{pre}e{e}."
            out[t] += a * ((silu(h[t] @ w[p + "gate"].T) * (h[t] @ w[p + "up"].T)) @ w[p + "down"].T)
    return out


# ---- the model --------------------------------------------------------------------------------------
def forward(tokens, w, cfg, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the summed streams after every layer)."""
    eps = cfg["norm"]["eps"]
    S = cfg["streams"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = x[:, None, :].repeat(1, S, 1)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        u = norm_around_zero(streams_read(xs, w[L + "hc1.in"]), w[L + "norm1"], eps)
        if layer["type"] == "lightning":
            y = lightning_mixer(u, w, L + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(u, w, L + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        xs = streams_write(xs, w[L + "hc1.mix"], w[L + "hc1.out"], y)
        if layer["mlp"] is not None:
            u = norm_around_zero(streams_read(xs, w[L + "hc2.in"]), w[L + "norm2"], eps)
            y = dense_ff(u, w, L + "mlp.") if layer["mlp"]["kind"] == "dense" else moe_ff(u, w, L + "mlp.", layer["mlp"])
            xs = streams_write(xs, w[L + "hc2.mix"], w[L + "hc2.out"], y)
        after.append(xs.sum(1))
    logits = norm_around_zero(xs.sum(1), w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
