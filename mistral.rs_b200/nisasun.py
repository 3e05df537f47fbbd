"""Nisasun: a decoder-only model whose layers carry `streams` f32 residual copies (hyper-connections) and alternate,
in any order given by the configuration, linear attention with per-head decay ("lightning") and a pair of windowed
attention + Mamba-2 mixers side by side ("parallel"), each followed by a dense GLU or a routed-expert feed-forward.

Everything size-like comes from config.json: `vocab`, `width`, `streams`, `norm.eps` and per layer `type`, `mixer`
(sizes of the mixer) and `mlp` (`kind` dense / moe, or null).  Tensor names: `embed`, `l<i>.norm1|norm2`,
`l<i>.hc1|hc2.{in,out,mix}`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.  The model is a composition of the
mechanisms in `mixers`; it has no cache or loop of its own — the engine owns pages, state slots and the step."""
import json
import os

import numpy as np
import torch

from . import mixers as M
from . import seq_ops as K

ARCHITECTURE = "Nisasun"


class NisasunConfig:
    def __init__(self, cj: dict):
        if cj.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = cj
        self.vocab, self.width, self.streams = int(cj["vocab"]), int(cj["width"]), int(cj.get("streams", 1))
        self.eps = float(cj["norm"]["eps"])
        self.layers = cj["layers"]
        for i, L in enumerate(self.layers):
            if L["type"] not in ("lightning", "parallel"):
                raise NotImplementedError(f"layer {i}: unknown mixer type {L['type']!r}")
            if L.get("mlp") is not None and L["mlp"]["kind"] not in ("dense", "moe"):
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {L['mlp']['kind']!r}")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (used to make random weights and to check a checkpoint)."""
        W, S, out = self.width, self.streams, {}
        out["embed"], out["head"], out["final.norm"] = (self.vocab, W), (self.vocab, W), (W,)
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            subs = ["1"] + (["2"] if L.get("mlp") is not None else [])
            for q in subs:
                out[p + "norm" + q] = (W,)
                out[p + f"hc{q}.in"], out[p + f"hc{q}.out"], out[p + f"hc{q}.mix"] = (S,), (S,), (S, S)
            if L["type"] == "lightning":
                H, dk, dv = m["heads"], m["dim"], m["vdim"]
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (H * dk, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,)})
            else:
                a, r = m["left"], m["right"]
                H, G, dk, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"]
                out.update({p + "mix.left.q": (H * dk, W), p + "mix.left.k": (G * dk, W), p + "mix.left.v": (G * dv, W),
                            p + "mix.left.q.norm": (dk,), p + "mix.left.k.norm": (dk,), p + "mix.left.o": (W, H * dv)})
                inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
                out.update({p + "mix.right.in": (2 * inner + 2 * gn + r["heads"], W), p + "mix.right.conv": (inner + 2 * gn, r["conv"]),
                            p + "mix.right.conv.b": (inner + 2 * gn,), p + "mix.right.dt_bias": (r["heads"],),
                            p + "mix.right.A_log": (r["heads"],), p + "mix.right.D": (r["heads"],), p + "mix.right.norm": (inner,),
                            p + "mix.right.o": (W, inner)})
            mlp = L.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                out[p + "mlp.router"], out[p + "mlp.correction"] = (E, W), (E,)
                for e in range(E):
                    out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
        return out


def load_safetensors(path):
    """name -> torch tensor (CPU) through the package's safetensors reader (host/safetensors_reader.hpp)."""
    from .uqff_file import SafetensorsFile
    K.ensure_host_lib()
    f = SafetensorsFile(path)
    try:
        out = {}
        for name, (dt, _, _, _) in f.entries.items():
            t = torch.from_numpy(np.array(f.array(name)))           # a copy: the mapping goes away with the file
            out[name] = t.view(torch.bfloat16) if dt == "BF16" else t
        return out
    finally:
        f.close()


class _Layer:
    pass


class NisasunModel:
    """Device-resident weights arranged for the kernels: projections that read the same input are one matrix, the
    experts are stacked, small vectors and every constant of a recurrence are f32."""

    def __init__(self, cfg: NisasunConfig, tensors: dict, device, dtype=torch.bfloat16, page_size=16):
        if dtype not in K.DTYPE_CODE:
            raise ValueError("activation dtype must be bfloat16 or float32")
        self.cfg, self.device, self.dtype, self.page_size = cfg, device, dtype, page_size
        want = cfg.tensor_shapes()
        for name, shape in want.items():
            if name not in tensors:
                raise KeyError(f"checkpoint lacks tensor `{name}`")
            if tuple(tensors[name].shape) != tuple(shape):
                raise ValueError(f"tensor `{name}` has shape {tuple(tensors[name].shape)}, the configuration needs {tuple(shape)}")
        mat = lambda *names: torch.cat([tensors[n].to(device=device, dtype=dtype) for n in names], dim=0).contiguous()
        vec = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        self.embed, self.head, self.final_norm = mat("embed"), mat("head"), vec("final.norm")
        self.layers = []
        for i, L in enumerate(cfg.layers):
            p, m, lay = f"l{i}.", L["mixer"], _Layer()
            lay.norm1 = vec(p + "norm1")
            lay.hc1 = M.StreamResidual(vec(p + "hc1.in"), vec(p + "hc1.out"), vec(p + "hc1.mix"))
            if L["type"] == "lightning":
                per_head = m["decay"] if isinstance(m["decay"], (list, tuple)) else [m["decay"]] * m["heads"]   # one value: every head
                decay = torch.tensor([float(d) for d in per_head], dtype=torch.float32, device=device)
                if decay.numel() != m["heads"]:
                    raise ValueError(f"layer {i}: one decay per head is needed")
                lay.mixer = M.LinearAttentionMixer(mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), mat(p + "mix.o"),
                                                   vec(p + "mix.norm"), decay, m["heads"], m["dim"], m["vdim"], cfg.eps)
            else:
                a, r = m["left"], m["right"]
                attn = M.WindowAttention(a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"], float(a["scale"]),
                                         int((a.get("mask") or {}).get("size", 0)),      # no mask entry: every earlier position
                                         vec(p + "mix.left.q.norm"), vec(p + "mix.left.k.norm"), cfg.eps)
                ssm = M.StateSpaceMixer(r["heads"], r["vdim"], r["state"], r["groups"], r["norm_groups"], vec(p + "mix.right.conv"),
                                        vec(p + "mix.right.conv.b"), vec(p + "mix.right.dt_bias"), vec(p + "mix.right.A_log"),
                                        vec(p + "mix.right.D"), vec(p + "mix.right.norm"), cfg.eps)
                w_out = torch.cat([tensors[p + "mix.left.o"], tensors[p + "mix.right.o"]], dim=1).to(device=device, dtype=dtype).contiguous()
                w_in = mat(p + "mix.left.q", p + "mix.left.k", p + "mix.left.v", p + "mix.right.in")
                if w_in.shape[0] % 8:       # zero rows: the projection's rows then start on 16-byte boundaries
                    w_in = torch.cat([w_in, w_in.new_zeros(8 - w_in.shape[0] % 8, w_in.shape[1])]).contiguous()
                lay.mixer = M.ParallelMixer(attn, ssm, w_in, w_out, float(m["left_scale"]), float(m["right_scale"]), page_size)
            mlp = L.get("mlp")
            lay.mlp = None
            if mlp is not None:
                lay.norm2 = vec(p + "norm2")
                lay.hc2 = M.StreamResidual(vec(p + "hc2.in"), vec(p + "hc2.out"), vec(p + "hc2.mix"))
                if mlp["kind"] == "dense":
                    lay.mlp = M.DenseGLU(mat(p + "mlp.gate", p + "mlp.up"), mat(p + "mlp.down"), K.ACT_GELU_TANH)
                else:
                    r = mlp["router"]
                    E = r["experts"]
                    gu = torch.stack([mat(p + f"mlp.e{e}.gate", p + f"mlp.e{e}.up") for e in range(E)]).contiguous()
                    dn = torch.stack([mat(p + f"mlp.e{e}.down") for e in range(E)]).contiguous()
                    grp = r.get("groups") or {"count": 1, "keep": 1}                      # no grouping: one group, kept
                    lay.mlp = M.RoutedExperts(vec(p + "mlp.router"), vec(p + "mlp.correction"), gu, dn, r["top"], grp["count"], grp["keep"],
                                              K.ACT_SILU)
            self.layers.append(lay)

    # ---- loading ------------------------------------------------------------------------------------
    @classmethod
    def from_dir(cls, path, device, dtype=torch.bfloat16, page_size=16):
        return cls(NisasunConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), device, dtype, page_size)

    @classmethod
    def random(cls, cfg: NisasunConfig, device, dtype=torch.bfloat16, seed=0, page_size=16):
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
        return [lay.mixer.alloc_cache(n_state_slots, n_token_slots, self.dtype, self.device) for lay in self.layers]

    def forward(self, batch, caches, after_layer=None):
        """Logits f32 [len(batch.rows), vocab] of one step's flat batch; advances `caches`.  after_layer(i, streams) is
        called with the f32 streams after every layer (inspection only)."""
        cfg, eps = self.cfg, self.cfg.eps
        xs = K.embed_streams(self.embed, batch.ids, cfg.streams)
        first = self.layers[0]
        h = K.streams_read_norm(xs, first.hc1.w_in, first.norm1, eps, 1.0, self.dtype)
        for i, lay in enumerate(self.layers):
            y = lay.mixer.forward(h, batch, caches[i])
            nxt = self.layers[i + 1] if i + 1 < len(self.layers) else None
            if lay.mlp is not None:
                h = K.streams_write(xs, lay.hc1.w_mix, lay.hc1.w_out, y, lay.hc2.w_in, lay.norm2, eps, 1.0)
                y = lay.mlp.forward(h)
                hc = lay.hc2
            else:
                hc = lay.hc1
            if nxt is not None:
                h = K.streams_write(xs, hc.w_mix, hc.w_out, y, nxt.hc1.w_in, nxt.norm1, eps, 1.0)
            else:
                K.streams_write(xs, hc.w_mix, hc.w_out, y)
            if after_layer is not None:
                after_layer(i, xs)
        hn = K.streams_read_norm(xs, None, self.final_norm, eps, 1.0, self.dtype, rows=batch.rows)
        return M.linear(hn, self.head).float()


def random_tensors(cfg: NisasunConfig, seed=0):
    """Random bf16-representable weights with activations of order one (throughput runs and tests)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        leaf = name.split(".")[-1]
        if name.endswith(("hc1.in", "hc2.in")):
            t = torch.full(shape, 1.0 / shape[0]) + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(("hc1.out", "hc2.out")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(("hc1.mix", "hc2.mix")):
            t = torch.eye(shape[0]) + 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf == "norm" and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "dt_bias":
            t = torch.rand(shape, generator=g) * 2.0 - 3.0
        elif leaf == "A_log":
            t = torch.log(1.0 + 3.0 * torch.rand(shape, generator=g))
        elif leaf == "D":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name in ("embed",):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out
