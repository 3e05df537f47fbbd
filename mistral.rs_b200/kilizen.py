"""Kilizen: a decoder-only model with ONE f32 residual whose norms are Dynamic Tanh, placed before and after every
sublayer (x <- x + norm_b(sublayer(norm(x)))), and whose layers mix — in any order given by the configuration —

  * `attention`:   grouped-query attention without a value projection (values = keys as projected), per-head
                   query / key RMS norm, rotary positions on part of each head with YaRN-scaled frequencies, a sliding
                   window that keeps the first tokens in sight, a per-head sink in the softmax;
  * `attention_2`: biased projections, query / key RMS norm over the whole projection, rotary positions, causal, sink;
  * `mlstm`:       a stabilised matrix memory with capped log gates;

each followed by a plain feed-forward (erf-gelu), routed experts (squared-relu, top-k logits with a softmax over the
chosen ones, plus a shared expert) or nothing.  A range of layers may run several times in a row with the same weights
(`loop`): every pass has its own cache / state, and the embedding output is added to the residual before each pass
but the first.

Everything size-like comes from config.json: `vocab`, `width`, `norm.eps`, `loop` {start, stop, times} and per layer
`type`, `mixer` (its sizes and constants) and `mlp` (`kind` dense / moe, or null).  Tensor names: `embed`,
`l<i>.norm1|norm1b|norm2|norm2b` (+ `.alpha`, `.b`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.  The model is a
composition of the mechanisms in `mixers`; it has no cache or loop of its own — the engine owns pages, state slots
and the step."""
import json
import os

import torch

from . import mixers as M
from . import seq_ops as K

ARCHITECTURE = "Kilizen"
MIXER_TYPES = ("attention", "attention_2", "mlstm")


class KilizenConfig:
    def __init__(self, cj: dict):
        if cj.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = cj
        self.vocab, self.width = int(cj["vocab"]), int(cj["width"])
        self.eps = float(cj["norm"]["eps"])
        self.layers = cj["layers"]
        for i, L in enumerate(self.layers):
            if L["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"layer {i}: unknown mixer type {L['type']!r}")
            if L.get("mlp") is not None and L["mlp"]["kind"] not in ("dense", "moe"):
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {L['mlp']['kind']!r}")
        loop = cj.get("loop") or {}
        self.loop_start, self.loop_stop, self.loop_times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if self.loop_times > 1 and not 0 <= self.loop_start < self.loop_stop <= len(self.layers):
            raise ValueError("loop: start < stop must lie inside the layer list")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def runs(self):
        """[(layer index, re-enter)] in execution order: the looped range `times` times in a row, then the rest; re-enter
        marks the first layer of every pass but the first (the embedding output is added right before it)."""
        n = len(self.layers)
        if self.loop_times <= 1:
            return [(i, False) for i in range(n)]
        a, b = self.loop_start, self.loop_stop
        out = [(i, False) for i in range(a)]
        for p in range(self.loop_times):
            out += [(i, p > 0 and i == a) for i in range(a, b)]
        return out + [(i, False) for i in range(b, n)]

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (used to make random weights and to check a checkpoint)."""
        W, out = self.width, {}
        norm = lambda name: {name: (W,), name + ".b": (W,), name + ".alpha": ()}
        out["embed"], out["head"] = (self.vocab, W), (self.vocab, W)
        out.update(norm("final.norm"))
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            for q in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") is not None else ()):
                out.update(norm(p + q))
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "mlstm":
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (H * dk, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                            p + "mix.f": (H, W), p + "mix.f.b": (H,)})
            else:
                G = int(m.get("kv_heads", H))
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (G * dk, W), p + "mix.sink": (H,), p + "mix.o": (W, H * dv)})
                if L["type"] == "attention":
                    out.update({p + "mix.q.norm": (dk,), p + "mix.k.norm": (dk,)})
                else:
                    out.update({p + "mix.v": (G * dv, W), p + "mix.q.b": (H * dk,), p + "mix.k.b": (G * dk,), p + "mix.v.b": (G * dv,),
                                p + "mix.o.b": (W,), p + "mix.q.norm": (H * dk,), p + "mix.k.norm": (G * dk,)})
            mlp = L.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                out.update({p + "mlp.up": (int(mlp["ff"]), W), p + "mlp.down": (W, int(mlp["ff"]))})
            else:
                E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
                out[p + "mlp.router"] = (E, W)
                for e in range(E):
                    out.update({p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
                if mlp.get("shared"):
                    sf = int(mlp["shared"]["ff"])
                    out.update({p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
        return out


class _Layer:
    pass


class KilizenModel:
    """Device-resident weights arranged for the kernels: projections that read the same input are one matrix, the
    experts are stacked, norm parameters, sinks, gate projections and every constant of a recurrence are f32."""

    def __init__(self, cfg: KilizenConfig, tensors: dict, device, dtype=torch.bfloat16, page_size=16):
        if dtype not in K.DTYPE_CODE:
            raise ValueError("activation dtype must be bfloat16 or float32")
        self.cfg, self.device, self.dtype, self.page_size = cfg, device, dtype, page_size
        for name, shape in cfg.tensor_shapes().items():
            if name not in tensors:
                raise KeyError(f"checkpoint lacks tensor `{name}`")
            if tuple(tensors[name].shape) != tuple(shape):
                raise ValueError(f"tensor `{name}` has shape {tuple(tensors[name].shape)}, the configuration needs {tuple(shape)}")
        mat = lambda *names: torch.cat([tensors[n].to(device=device, dtype=dtype) for n in names], dim=0).contiguous()
        vec = lambda *names: torch.cat([tensors[n].to(device=device, dtype=torch.float32).reshape(-1) for n in names]).contiguous()
        norm = lambda n: M.TanhNorm(vec(n + ".alpha"), vec(n), vec(n + ".b")).t
        self.embed, self.head, self.final_norm = mat("embed"), mat("head"), norm("final.norm")
        self.layers, rotations = [], {}

        def rotation(rot):
            if not rot:
                return None
            r = M.Rotation(rot["dims"], rot["base"], rot.get("scaling"), device)
            return rotations.setdefault(r.key, r)          # layers with equal constants share one table per step

        for i, L in enumerate(cfg.layers):
            p, m, lay = f"l{i}.", L["mixer"], _Layer()
            lay.norm1, lay.norm1b = norm(p + "norm1"), norm(p + "norm1b")
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "mlstm":
                w_gates = torch.cat([tensors[p + "mix.i"], tensors[p + "mix.f"]]).to(device=device, dtype=torch.float32).contiguous()
                lay.mixer = M.MatrixMemoryMixer(mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), w_gates, vec(p + "mix.i.b", p + "mix.f.b"),
                                                mat(p + "mix.o"), vec(p + "mix.norm"), H, dk, dv, float(m.get("gate_cap", 0.0)), cfg.eps)
            else:
                G, mask = int(m.get("kv_heads", H)), m.get("mask") or {}
                keys_are_values = L["type"] == "attention"
                attn = M.WindowAttention(H, G, dk, dv, float(m["scale"]), int(mask.get("size", 0)), vec(p + "mix.q.norm"), vec(p + "mix.k.norm"),
                                         cfg.eps, norm_mode=K.QK_NORM_HEAD if keys_are_values else K.QK_NORM_WHOLE, rotation=rotation(m.get("rot")),
                                         keep_first=int(mask.get("keep_first", 0)), sink=vec(p + "mix.sink"), values_from_keys=keys_are_values)
                if keys_are_values:
                    lay.mixer = M.AttentionMixer(attn, mat(p + "mix.q", p + "mix.k"), mat(p + "mix.o"), page_size)
                else:
                    b_in = torch.cat([tensors[p + n] for n in ("mix.q.b", "mix.k.b", "mix.v.b")]).to(device=device, dtype=dtype).contiguous()
                    lay.mixer = M.AttentionMixer(attn, mat(p + "mix.q", p + "mix.k", p + "mix.v"), mat(p + "mix.o"), page_size, b_in=b_in,
                                                 b_out=tensors[p + "mix.o.b"].to(device=device, dtype=dtype).contiguous())
            mlp, lay.mlp = L.get("mlp"), None
            if mlp is not None:
                lay.norm2, lay.norm2b = norm(p + "norm2"), norm(p + "norm2b")
                if mlp["kind"] == "dense":
                    lay.mlp = M.DenseMLP(mat(p + "mlp.up"), mat(p + "mlp.down"), K.ACT_GELU_ERF)
                else:
                    E = int(mlp["router"]["experts"])
                    up = torch.stack([mat(p + f"mlp.e{e}.up") for e in range(E)]).contiguous()
                    dn = torch.stack([mat(p + f"mlp.e{e}.down") for e in range(E)]).contiguous()
                    shared = M.DenseMLP(mat(p + "mlp.shared.up"), mat(p + "mlp.shared.down"), K.ACT_RELU_SQ) if mlp.get("shared") else None
                    lay.mlp = M.RoutedExperts(vec(p + "mlp.router").view(E, cfg.width), None, up, dn, int(mlp["router"]["top"]), 1, 1,
                                              K.ACT_RELU_SQ, rule="top_softmax", gated=False, shared=shared)
            self.layers.append(lay)
        self.runs = cfg.runs()

    # ---- loading ------------------------------------------------------------------------------------
    @classmethod
    def from_dir(cls, path, device, dtype=torch.bfloat16, page_size=16):
        from .nisasun import load_safetensors
        return cls(KilizenConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), device, dtype, page_size)

    @classmethod
    def random(cls, cfg: KilizenConfig, device, dtype=torch.bfloat16, seed=0, page_size=16):
        return cls(cfg, random_tensors(cfg, seed), device, dtype, page_size)

    # ---- the engine's interface ---------------------------------------------------------------------
    @property
    def vocab(self):
        return self.cfg.vocab

    def capturable(self, n_tok):
        """True when a step of n_tok tokens launches a fixed sequence of kernels with no host read in between (the
        routed-expert layers then take their weight-streaming path), so it can be captured as a CUDA graph."""
        return all(lay.mlp is None or not isinstance(lay.mlp, M.RoutedExperts) or lay.mlp.streams_weights(n_tok) for lay in self.layers)

    def alloc_caches(self, n_state_slots, n_token_slots):
        """One cache per layer RUN: a layer inside the looped range has one per pass."""
        return [self.layers[i].mixer.alloc_cache(n_state_slots, n_token_slots, self.dtype, self.device) for i, _ in self.runs]

    def forward(self, batch, caches, after_layer=None):
        """Logits f32 [len(batch.rows), vocab] of one step's flat batch; advances `caches`.  after_layer(r, x) is called
        with the f32 residual after every layer run (inspection only; the fused residual pass is then split in two)."""
        T, W = batch.ids.numel(), self.cfg.width
        x0 = K.embed_streams(self.embed, batch.ids, 1).view(T, W)
        x = x0.clone() if any(again for _, again in self.runs) else x0
        h = K.tanh_norm_rows(x, self.layers[self.runs[0][0]].norm1, self.dtype)
        for r, (i, _) in enumerate(self.runs):
            lay = self.layers[i]
            y = lay.mixer.forward(h, batch, caches[r])
            post = lay.norm1b
            if lay.mlp is not None:
                h = K.residual_tanh_norm(x, y, post=post, nxt=lay.norm2)
                y, post = lay.mlp.forward(h), lay.norm2b
            if r + 1 == len(self.runs):
                K.residual_tanh_norm(x, y, post=post)
                if after_layer is not None:
                    after_layer(r, x)
                break
            j, again = self.runs[r + 1]
            extra, nxt = (x0 if again else None), self.layers[j].norm1
            if after_layer is None:
                h = K.residual_tanh_norm(x, y, post=post, extra=extra, nxt=nxt)
            else:
                K.residual_tanh_norm(x, y, post=post)
                after_layer(r, x)
                h = K.residual_tanh_norm(x, extra=extra, nxt=nxt, dtype=self.dtype)
        hn = K.tanh_norm_rows(x, self.final_norm, self.dtype, rows=batch.rows)
        return M.linear(hn, self.head).float()


def random_tensors(cfg: KilizenConfig, seed=0):
    """Random bf16-representable weights with activations of order one (throughput runs and tests)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        leaf = name.split(".")[-1]
        if leaf == "alpha":
            t = 0.5 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "b":
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b", "norm") and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out
