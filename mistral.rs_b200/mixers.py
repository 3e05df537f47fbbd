"""Layer mechanisms built on the sequence-mixer kernels (`seq_ops`), each with its constants as parameters so any
model definition can compose them: multi-stream residuals, linear attention with per-head decay, windowed attention
with query/key norm over a paged cache, a Mamba-2 style state-space mixer, two mixers side by side, dense GLU and
routed-expert feed-forwards.

A mechanism owns its device weights and declares the per-layer cache it needs (`alloc_cache`): token-indexed pages
(sized by the engine's block pool) and / or per-request state slots (sized by the engine's slot pool).  `forward`
takes the activation rows of one step's flat batch (`engine.StepBatch`) — prompt portions and single decoded tokens
side by side — and advances that cache.  Dense matrix products are plain library GEMMs (`torch.nn.functional.linear`,
cuBLAS); everything between them is this package's CUDA."""
import torch
import torch.nn.functional as F

from . import seq_ops as K


def linear(x, w):
    return F.linear(x, w)


class StreamResidual:
    """Hyper-connections: `n_streams` f32 copies of the residual; a sublayer reads sum_s w_in[s] x_s and writes
    x_r <- sum_s w_mix[s, r] x_s + w_out[r] y."""

    def __init__(self, w_in, w_out, w_mix):
        self.w_in, self.w_out, self.w_mix = w_in, w_out, w_mix


class LinearAttentionMixer:
    """q, k, v = act(W h) per head; S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t; RMS norm over the concatenated
    heads, output gate sigmoid(W_g h), output projection."""

    def __init__(self, w_qkvg, w_o, norm_w, decay, heads, dk, dv, eps, act=K.ACT_SILU):
        self.w_qkvg, self.w_o, self.norm_w, self.decay = w_qkvg, w_o, norm_w, decay
        self.heads, self.dk, self.dv, self.eps, self.act = heads, dk, dv, eps, act

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"state": torch.zeros(n_slots, self.heads, self.dk, self.dv, dtype=torch.float32, device=device)}

    def forward(self, h, batch, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        y = linear(h, self.w_qkvg)                                         # [T, 2 H dk + 2 H dv]: q | k | v | g
        K.activate_cols(y, 0, 2 * H * dk + H * dv, self.act)                # once, not once per state tile inside the scan
        o = K.linear_scan(y, 0, y, H * dk, y, 2 * H * dk, H, H, dk, dv, cache["state"], batch, decay_head=self.decay)
        on = torch.empty(h.shape[0], H * dv, dtype=h.dtype, device=h.device)
        K.gated_group_norm(o, y, 2 * H * dk + H * dv, self.norm_w, 1, self.eps, K.ACT_SIGMOID, False, on)
        return linear(on, self.w_o)


class WindowAttention:
    """Grouped-query softmax attention without positional rotation: per-head RMS norm of q and k, scores scaled by a
    given constant, a sliding window of `window` positions (0: full causal), keys and values in pages."""

    def __init__(self, heads, kv_heads, dk, dv, scale, window, q_norm_w, k_norm_w, eps):
        self.heads, self.kv_heads, self.dk, self.dv = heads, kv_heads, dk, dv
        self.scale, self.window, self.q_norm_w, self.k_norm_w, self.eps = scale, window, q_norm_w, k_norm_w, eps

    @property
    def proj_cols(self):
        return self.heads * self.dk + self.kv_heads * (self.dk + self.dv)

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"k": torch.zeros(n_token_slots, self.kv_heads, self.dk, dtype=dtype, device=device),
                "v": torch.zeros(n_token_slots, self.kv_heads, self.dv, dtype=dtype, device=device)}

    def attend(self, y, col0, batch, cache, page_size, out, out_col=0, out_scale=1.0):
        """y holds q | k | v from column col0; writes heads * dv columns of `out` from out_col.  Keys and values of the new
        tokens are normed and stored first.  A sequence that starts in this step with a long enough portion (batch.fresh)
        runs on the package's prompt-attention kernels over its fresh q / k / v when they fit it (bf16, equal head sizes
        of 64 or 128, 16-byte aligned rows); every other token — portions that continue a sequence, decoded tokens, other
        head sizes, f32 — reads its keys from the pages."""
        kc, vc = col0 + self.heads * self.dk, col0 + self.heads * self.dk + self.kv_heads * self.dk
        K.qk_norm_store(y, col0, kc, vc, self.q_norm_w, self.k_norm_w, self.eps, self.heads, self.kv_heads, self.dk, self.dv,
                        cache["k"], cache["v"], batch.slot_of_tok)
        tok_index = None
        aligned = all(v % 8 == 0 for v in (y.stride(0), col0, out.stride(0), out_col))
        if batch.fresh and y.dtype == torch.bfloat16 and self.dk == self.dv and self.dk in (64, 128) and aligned:
            for row0, rows in batch.fresh:
                K.fresh_prompt_attention(y, row0, rows, col0, kc, vc, self.heads, self.kv_heads, self.dk, self.scale, self.window, out, out_col)
                if out_scale != 1.0:
                    K.scale_rows(out, row0, rows, out_col, self.heads * self.dv, out_scale)
            tok_index = batch.paged_tok
            if tok_index.numel() == 0:
                return
        K.window_attention(y, col0, cache["k"], cache["v"], self.heads, self.kv_heads, self.dk, self.dv, self.scale, self.window,
                           batch, page_size, out, out_col, out_scale, tok_index)


class StateSpaceMixer:
    """Mamba-2 (state-space duality) core: the input projection's columns are z | x | B | C | dt; x, B, C pass a short
    causal convolution and silu; dt = softplus(dt + bias); per head S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D x_t; y * silu(z) is RMS-normed in `norm_groups` parts."""

    def __init__(self, heads, dv, n_state, groups, norm_groups, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps):
        self.heads, self.dv, self.n_state, self.groups, self.norm_groups = heads, dv, n_state, groups, norm_groups
        self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w, self.eps = conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps
        self.inner = heads * dv
        self.conv_channels = self.inner + 2 * groups * n_state

    @property
    def proj_cols(self):
        return 2 * self.inner + 2 * self.groups * self.n_state + self.heads

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        taps = self.conv_w.shape[1]
        return {"state": torch.zeros(n_slots, self.heads, self.n_state, self.dv, dtype=torch.float32, device=device),
                "conv": torch.zeros(n_slots, max(taps - 1, 1), self.conv_channels, dtype=torch.float32, device=device)}

    def mix(self, y, col0, batch, cache, out, out_col=0, out_scale=1.0):
        """y holds z | xBC | dt from column col0; writes `inner` columns of `out` from out_col."""
        inner, GN = self.inner, self.groups * self.n_state
        xbc = K.causal_conv(y, col0 + inner, self.conv_channels, self.conv_w, self.conv_b, K.ACT_SILU, cache["conv"], batch)
        step, decay = K.ssm_steps(y, col0 + 2 * inner + 2 * GN, self.dt_bias, self.a_log)
        o = K.linear_scan(xbc, inner + GN, xbc, inner, xbc, 0, self.heads, self.groups, self.n_state, self.dv, cache["state"], batch,
                          decay_tok=decay, scale_tok=step, skip=self.d_skip)
        K.gated_group_norm(o, y, col0, self.norm_w, self.norm_groups, self.eps, K.ACT_SILU, True, out, out_col, out_scale)


class ParallelMixer:
    """Windowed attention and a state-space mixer reading the same input; result = left_scale * attention branch +
    right_scale * state-space branch.  One input GEMM feeds both; the scaled branch outputs sit side by side so one
    output GEMM over [W_o_left | W_o_right] sums them in its f32 accumulator."""

    def __init__(self, attn: WindowAttention, ssm: StateSpaceMixer, w_in, w_out, left_scale, right_scale, page_size):
        self.attn, self.ssm, self.w_in, self.w_out = attn, ssm, w_in, w_out
        self.left_scale, self.right_scale, self.page_size = left_scale, right_scale, page_size

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        c = self.attn.alloc_cache(n_slots, n_token_slots, dtype, device)
        c.update(self.ssm.alloc_cache(n_slots, n_token_slots, dtype, device))
        return c

    def forward(self, h, batch, cache):
        y = linear(h, self.w_in)                                          # q | k | v | z | xBC | dt
        a_cols = self.attn.heads * self.attn.dv
        both = torch.empty(h.shape[0], a_cols + self.ssm.inner, dtype=h.dtype, device=h.device)
        self.attn.attend(y, 0, batch, cache, self.page_size, both, 0, self.left_scale)
        self.ssm.mix(y, self.attn.proj_cols, batch, cache, both, a_cols, self.right_scale)
        return linear(both, self.w_out)


class DenseGLU:
    """down(act(gate h) * up h) with gate and up as one GEMM."""

    def __init__(self, w_gate_up, w_down, act):
        self.w_gate_up, self.w_down, self.act = w_gate_up, w_down, act

    def forward(self, h):
        return linear(K.glu_split(linear(h, self.w_gate_up), self.act), self.w_down)


class RoutedExperts:
    """Softmax router in f32 with a choice-only bias and group-limited top-k; experts are GLU feed-forwards.  Few
    (token, expert) pairs: two weight-streaming kernels.  Many: rows sorted by expert, one GEMM pair per expert that
    has rows (the per-expert row counts cross to the host once per layer), weighted combine in f32."""

    # Up to this many (token, expert) pairs per expert the weights are simply streamed once per pair: 4 while an expert is
    # small enough that repeated reads hit L2, 2 above that.
    SMALL_EXPERT_BYTES = 32 << 20

    def __init__(self, w_router, correction, w_gate_up, w_down, top, n_groups, keep_groups, act, renorm=False):
        self.w_router, self.correction, self.w_gate_up, self.w_down = w_router, correction, w_gate_up, w_down
        self.top, self.n_groups, self.keep_groups, self.act, self.renorm = top, n_groups, keep_groups, act, renorm
        self.n_experts = w_gate_up.shape[0]

    def streams_weights(self, n_tok):
        expert_bytes = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        per_expert = 4 if expert_bytes <= self.SMALL_EXPERT_BYTES else 2
        return n_tok * self.top <= per_expert * self.n_experts

    def route(self, h):
        logits = F.linear(h.float(), self.w_router)
        return K.moe_route(logits, self.correction, self.n_groups, self.keep_groups, self.top, self.renorm)

    def forward(self, h):
        experts, weights = self.route(h)
        if self.streams_weights(h.shape[0]):
            return K.moe_small(h, self.w_gate_up, self.w_down, experts, weights, self.act)
        counts, order = K.moe_sort(experts, self.n_experts)
        xs = K.moe_gather(h, order, self.top)
        ys = torch.empty_like(xs)
        at = 0
        for e, n in enumerate(counts.tolist()):
            if n:
                hid = K.glu_split(linear(xs[at:at + n], self.w_gate_up[e]), self.act)
                torch.mm(hid, self.w_down[e].t(), out=ys[at:at + n])
                at += n
        return K.moe_combine(ys, order, weights)
