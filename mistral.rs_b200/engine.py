"""Serving engine for models built from `mixers`: requests, a scheduler with chunked prefill and continuous
batching, the step function, and the two cache managers it drives — the paged KV manager (`kv_index.KVCacheManager`,
C++ host/kv_cache_manager.hpp) for token-indexed caches and the state-slot pool (host/state_slots.hpp) for
constant-size recurrent states.

One step = one flat batch: for every scheduled request its next tokens (a prompt portion of any length, or the one
token decoded last), concatenated; `StepBatch` carries the integer description the kernels read (token offsets per
sequence, tokens already cached, state slot, page table, cache slot and position of every token).  `Engine.execute`
runs such a batch on the model and returns logits for the asked rows; `Engine.step` = scheduler plan -> execute ->
sample (the package's device top-k / top-1 kernels + host tail) -> append.  REF for the division of labour:
mistralrs-core/src/scheduler (which sequences run), mistralrs-core/src/paged_attention (who owns blocks),
mistralrs-core/src/sampler.rs (what happens to the logits)."""
import ctypes
from collections import deque
from dataclasses import dataclass, field

import numpy as np
import torch

from . import kv_index, seq_ops


@dataclass
class SamplingParams:
    temperature: float = None          # None: greedy
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    max_new_tokens: int = 16
    stop_token: int = None
    seed: int = 0


@dataclass
class Request:
    rid: int
    tokens: list                         # prompt + generated so far
    n_prompt: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    n_computed: int = 0                  # tokens already in the caches
    generated: list = field(default_factory=list)
    finished: bool = False
    admitted: bool = False
    slot: int = -1                       # state slot once admitted


class StateSlots:
    """Python handle of the C++ state-slot pool."""

    def __init__(self, n_slots):
        self._L = seq_ops.ensure_host_lib()
        self._h = ctypes.c_void_p(self._L.mrs_state_slots_new(ctypes.c_int64(n_slots)))
        if not self._h:
            raise ValueError("a state-slot pool needs at least one slot")

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                self._L.mrs_state_slots_free(self._h)
            except Exception:
                pass
            self._h = None

    def capacity(self):
        return int(self._L.mrs_state_slots_capacity(self._h))

    def num_free(self):
        return int(self._L.mrs_state_slots_num_free(self._h))

    def acquire(self, rid):
        return int(self._L.mrs_state_slots_acquire(self._h, ctypes.c_uint64(rid)))

    def slot_of(self, rid):
        return int(self._L.mrs_state_slots_slot_of(self._h, ctypes.c_uint64(rid)))

    def release(self, rid):
        return bool(self._L.mrs_state_slots_release(self._h, ctypes.c_uint64(rid)))


class StepBatch:
    """Device-side integer description of one step.  Built on the host into one pinned buffer, copied once."""

    FRESH_MIN = 32     # a portion of at least this many tokens may take the prompt-attention kernels

    def __init__(self, device, ids, counts, pasts, slots, tables, slot_of_tok, rows, pages_ld=None):
        self.device, self._pages_ld = device, pages_ld
        host, layout = self._pack(ids, counts, pasts, slots, tables, slot_of_tok, rows)
        self._host, self._dev = host, host.to(device, non_blocking=True)
        self._bind(layout)

    def _pack(self, ids, counts, pasts, slots, tables, slot_of_tok, rows):
        n_seq, n_tok = len(counts), int(sum(counts))
        pages_ld = self._pages_ld or max(1, max(len(t) for t in tables))
        cu = np.zeros(n_seq + 1, dtype=np.int32)
        cu[1:] = np.cumsum(counts)
        seq_of = np.repeat(np.arange(n_seq, dtype=np.int32), counts)
        pos_of = np.concatenate([np.arange(p, p + c, dtype=np.int32) for p, c in zip(pasts, counts)]) if n_tok else np.zeros(0, np.int32)
        pages = np.zeros((n_seq, pages_ld), dtype=np.int32)
        for b, t in enumerate(tables):
            pages[b, :len(t)] = t
        is_fresh = [p == 0 and c >= self.FRESH_MIN for p, c in zip(pasts, counts)]
        self.fresh = [(int(cu[b]), int(counts[b])) for b in range(n_seq) if is_fresh[b]]      # (first row, rows) per such sequence
        paged = np.concatenate([np.arange(cu[b], cu[b + 1], dtype=np.int32) for b in range(n_seq) if not is_fresh[b]] + [np.zeros(0, np.int32)])
        # long portions, fresh or continued: (first row, rows, tokens cached before, sequence) for kernels that tile a portion's rows
        is_long = [c >= self.FRESH_MIN for c in counts]
        self.long = [(int(cu[b]), int(counts[b]), int(pasts[b]), b) for b in range(n_seq) if is_long[b]]
        long_rows = np.asarray(self.long, dtype=np.int32).reshape(-1)
        short = np.concatenate([np.arange(cu[b], cu[b + 1], dtype=np.int32) for b in range(n_seq) if not is_long[b]] + [np.zeros(0, np.int32)])
        parts = [np.asarray(ids, dtype=np.int32), cu, np.asarray(pasts, dtype=np.int32), np.asarray(slots, dtype=np.int32), seq_of, pos_of,
                 pages.reshape(-1), np.asarray(rows, dtype=np.int32), paged, long_rows, short]
        sizes = [p.size for p in parts]
        pad = sum(sizes) % 2                                       # keep the int64 tail 8-byte aligned
        total = sum(sizes) + pad + 2 * n_tok
        host = torch.empty(total, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else torch.empty(total, dtype=torch.int32)
        hv = host.numpy()
        at = 0
        for p in parts:
            hv[at:at + p.size] = p
            at += p.size
        at += pad
        hv[at:at + 2 * n_tok] = np.asarray(slot_of_tok, dtype=np.int64).view(np.int32)
        self.n_seq, self.n_tok, self.h2d_bytes = n_seq, n_tok, total * 4
        self.longest = int(max(counts)) if n_seq else 0            # host-side facts the mixers plan with
        return host, (tuple(sizes), pad, n_seq, n_tok, pages_ld)

    def _bind(self, layout):
        sizes, pad, n_seq, n_tok, pages_ld = layout
        self._layout, dev = layout, self._dev
        o = np.concatenate([[0], np.cumsum(sizes)])
        cut = lambda i: dev[int(o[i]):int(o[i + 1])]
        self.ids, self.cu_tok, self.past, self.slot, self.seq_of_tok, self.pos_of_tok = (cut(i) for i in range(6))
        self.pages = cut(6).view(n_seq, pages_ld)
        self.rows = cut(7)
        self.paged_tok = cut(8)                                    # tokens of the sequences not in `fresh`
        self.long_rows = cut(9)                                    # 4 integers per entry of `long`
        self.short_tok = cut(10)                                   # tokens of the sequences not in `long`
        at = int(o[-1]) + pad
        self.slot_of_tok = dev[at:at + 2 * n_tok].view(torch.int64)


class DecodeGraph:
    """One captured CUDA graph of the model's step for `n` sequences that each bring one decoded token.  The integer
    description lives in fixed device memory and is staged in one fixed pinned buffer: token ids, positions and state
    slots are written as arrays, block tables and cache slots by the KV manager's batched `decode_step` (one native
    call for the whole batch, straight into the staging memory); then one copy and one graph launch.  The page table
    is as wide as the longest request the pool can hold; logits come out for every row."""

    def __init__(self, engine, n):
        self.engine, self.n, P = engine, n, engine.max_pages_per_request
        shape = ([0] * n, [1] * n, [1] * n, [0] * n, [[0]] * n, np.zeros(n, dtype=np.int64))
        self.batch = StepBatch(engine.device, *shape, rows=list(range(n)), pages_ld=P)
        sizes, pad = self.batch._layout[0], self.batch._layout[1]
        self.host = self.batch._host                       # pinned; the constant parts (offsets, row lists) stay as packed
        hv, o = self.host.numpy(), np.concatenate([[0], np.cumsum(sizes)])
        self.h_ids, self.h_past, self.h_slot, self.h_pos = hv[o[0]:o[1]], hv[o[2]:o[3]], hv[o[3]:o[4]], hv[o[5]:o[6]]
        self.h_pages = hv[o[6]:o[7]].reshape(n, P)
        at = int(o[-1]) + pad
        self.h_slot_of_tok = hv[at:at + 2 * n].view(np.int64)
        self.copied = torch.cuda.Event()
        self.copied.record()
        torch.cuda.synchronize(engine.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = engine.model.forward(self.batch, engine.caches)

    def run(self, reqs):
        self.copied.synchronize()                          # the staging memory is free again
        pasts = [r.n_computed for r in reqs]
        self.h_ids[:] = [r.tokens[r.n_computed] for r in reqs]
        self.h_past[:] = pasts
        self.h_pos[:] = pasts
        self.h_slot[:] = [r.slot for r in reqs]
        self.engine.pages.decode_step([r.rid for r in reqs], [p + 1 for p in pasts], self.h_pages.shape[1], tables=self.h_pages,
                                      slots=self.h_slot_of_tok)
        self.batch._dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        self.graph.replay()
        return self.logits


class Scheduler:
    """Which requests run in the next step, and how many tokens of each: running requests first (their one decoded
    token, or the next portion of a prompt that is still being read), then waiting requests while a state slot, pages
    and the step's token budget last.  A prompt longer than what is left of the budget is read in portions."""

    def __init__(self, max_step_tokens=2048):
        self.max_step_tokens = max_step_tokens
        self.waiting, self.running = deque(), []

    def add(self, req):
        self.waiting.append(req)

    def plan(self, engine):
        budget, plan = self.max_step_tokens, []
        slots_left, pages_left = engine.free_slots(), engine.free_pages()      # what this plan has not yet promised
        for r in self.running:
            n = min(len(r.tokens) - r.n_computed, budget)
            need = engine.pages_needed(r, n) if n > 0 else 0
            if n > 0 and need <= pages_left:
                plan.append((r, n))
                budget -= n
                pages_left -= need
        while self.waiting and budget > 0 and slots_left > 0:
            r = self.waiting[0]
            n = min(len(r.tokens), budget)
            need = engine.pages_needed(r, n)
            if need > pages_left:
                break
            self.waiting.popleft()
            self.running.append(r)
            plan.append((r, n))
            budget -= n
            slots_left -= 1
            pages_left -= need
        return plan

    def retire(self, req):
        if req in self.running:
            self.running.remove(req)


class Engine:
    """Owns the model's caches and runs steps.  max_tokens: tokens the page pool holds at once (every request rounded up
    to whole pages); max_seqs: state slots, i.e. the most requests alive at once."""

    def __init__(self, model, max_tokens, max_seqs=4, max_step_tokens=2048, decode_graphs=True):
        self.model, self.device, self.page_size = model, model.device, model.page_size
        self.decode_graphs, self._graphs, self._decode_seen = decode_graphs, {}, {}
        seq_ops.ensure_host_lib()
        n_pages = -(-int(max_tokens) // self.page_size)
        self.max_pages_per_request = n_pages
        self.pages = kv_index.KVCacheManager(n_pages + 1, self.page_size, enable_caching=False)      # + the null block
        self.slots = StateSlots(max_seqs)
        self.caches = model.alloc_caches(max_seqs, (n_pages + 1) * self.page_size)
        self.scheduler = Scheduler(max_step_tokens)
        self.requests = {}
        self._next_rid = 1
        self._rng = {}
        if model.dtype == torch.float32:       # true 32-bit products: no reduced-precision matrix mode
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")

    # ---- capacity -------------------------------------------------------------------------------------
    def pages_needed(self, req, n_new):
        have = self.pages.num_blocks_for_request(req.rid) if self.pages.has_request(req.rid) else 0
        return max(0, -(-(req.n_computed + n_new) // self.page_size) - have)

    def free_pages(self):
        return self.pages.num_free_blocks()

    def free_slots(self):
        return self.slots.num_free()

    # ---- requests -------------------------------------------------------------------------------------
    def new_request(self, prompt, sampling=None):
        req = Request(self._next_rid, list(prompt), len(prompt), sampling or SamplingParams())
        self._next_rid += 1
        self.requests[req.rid] = req
        return req

    def add_request(self, prompt, sampling=None):
        req = self.new_request(prompt, sampling)
        self.scheduler.add(req)
        return req

    def finish(self, req):
        """Give back the request's pages and state slot."""
        req.finished, req.slot = True, -1
        self.pages.free(req.rid)
        self.slots.release(req.rid)
        self.scheduler.retire(req)
        self.requests.pop(req.rid, None)
        self._rng.pop(req.rid, None)

    # ---- the step -------------------------------------------------------------------------------------
    def execute(self, plan, want=None, after_layer=None):
        """plan: [(request, n_new)] — the next n_new tokens of request.tokens past n_computed.  want: per entry the
        offsets inside its portion whose logits are asked for (default: the last one).  Returns f32 logits
        [asked rows, vocab] in plan order, or None when nothing is asked."""
        if after_layer is None and self.decode_graphs and all(n == 1 and r.n_computed > 0 and r.slot >= 0 for r, n in plan):
            out = self._decode_by_graph(plan, want)
            if out is not NotImplemented:
                return out
        ids, counts, pasts, slots, tables, slot_map, rows = [], [], [], [], [], [], []
        base = 0
        for e, (req, n) in enumerate(plan):
            if n <= 0 or req.n_computed + n > len(req.tokens):
                raise ValueError("a step entry must bring 1..remaining tokens of its request")
            slot = self.slots.acquire(req.rid)
            if slot < 0:
                raise MemoryError("no state slot is free")
            if self.pages.allocate_slots(req.rid, req.n_computed + n) is None:
                raise MemoryError("the page pool cannot hold this step")
            req.admitted, req.slot = True, slot
            ids += req.tokens[req.n_computed:req.n_computed + n]
            counts.append(n)
            pasts.append(req.n_computed)
            slots.append(slot)
            tables.append(self.pages.get_block_ids(req.rid))
            slot_map.append(self.pages.get_slot_mapping(req.rid, req.n_computed, n))
            w = [n - 1] if want is None else want[e]
            rows += [base + int(i) for i in w]
            base += n
        batch = StepBatch(self.device, ids, counts, pasts, slots, tables, np.concatenate(slot_map), rows)
        self.last_batch = batch
        logits = self.model.forward(batch, self.caches, after_layer=after_layer)     # the caches advance also when no row is asked
        for req, n in plan:
            req.n_computed += n
        return logits if rows else None

    def _decode_by_graph(self, plan, want):
        """Steps in which every request brings exactly one token after its first run as a captured graph, from the
        second such step of a given batch size on (the first runs eagerly and warms every kernel up)."""
        n = len(plan)
        if any(req.n_computed + 1 > len(req.tokens) for req, _ in plan):
            raise ValueError("a step entry must bring 1..remaining tokens of its request")
        if not getattr(self.model, "capturable", lambda n_tok: False)(n):
            return NotImplemented
        g = self._graphs.get(n)
        if g is None:
            self._decode_seen[n] = self._decode_seen.get(n, 0) + 1
            if self._decode_seen[n] < 2:
                return NotImplemented
            try:
                g = self._graphs[n] = DecodeGraph(self, n)
            except RuntimeError:             # a step that cannot be captured on this system: stay eager for good
                self.decode_graphs = False
                return NotImplemented
        out = g.run([req for req, _ in plan])
        rows = list(range(n)) if want is None else [e for e, w in enumerate(want) if len(w)]
        for req, _ in plan:
            req.n_computed += 1
        if not rows:
            return None
        return out.clone() if len(rows) == n else out[rows]

    def step(self):
        """One scheduler-planned step; returns [(request, new token)] for the requests that produced one."""
        plan = self.scheduler.plan(self)
        if not plan:
            if self.scheduler.waiting or self.scheduler.running:
                raise MemoryError("no live or waiting request can take its next step: the pools are too small")
            return []
        logits = self.execute(plan)
        out = []
        samplers = [(i, r) for i, (r, n) in enumerate(plan) if r.n_computed == len(r.tokens)]
        if samplers:
            toks = self.sample(logits[[i for i, _ in samplers]], [r for _, r in samplers])
            for (_, r), t in zip(samplers, toks):
                r.tokens.append(int(t))
                r.generated.append(int(t))
                out.append((r, int(t)))
                sp = r.sampling
                if len(r.generated) >= sp.max_new_tokens or (sp.stop_token is not None and int(t) == sp.stop_token):
                    self.finish(r)
        return out

    def sample(self, logits, reqs):
        """Device top-1 / top-k kernels + the host tail (top-p / min-p / weighted draw), one row per request."""
        from . import ops, sampler
        toks = [None] * len(reqs)
        greedy = [i for i, r in enumerate(reqs) if r.sampling.temperature is None]
        if greedy:
            t1 = ops.cuda_top1_logits_f32(logits[greedy].contiguous()).reshape(-1).tolist()
            for i, t in zip(greedy, t1):
                toks[i] = int(t)
        for i, r in enumerate(reqs):
            if toks[i] is not None:
                continue
            sp = r.sampling
            k = sp.top_k if 0 < sp.top_k <= sampler.CUDA_TOPK_MAX_K else sampler.CUDA_TOPK_MAX_K
            vals, idx, denom, gmax = ops.cuda_topk_logits_f32_packed(logits[i:i + 1].contiguous(), k, sp.temperature)
            packed = torch.cat([vals.reshape(-1), idx.reshape(-1).float(), denom.reshape(-1), gmax.reshape(-1)]).cpu().numpy()
            rng = self._rng.setdefault(r.rid, np.random.default_rng(sp.seed))
            kk = min(k, logits.shape[1])
            toks[i], _ = sampler.sample_topk_packed_row(packed, kk, kk, 1.0 / sp.temperature, sp.top_p, sp.min_p, float(rng.random()))
        return toks

    def generate(self, prompts, sampling=None):
        """Run the given prompts to completion through the scheduler; returns the generated tokens per prompt."""
        reqs = [self.add_request(p, sampling) for p in prompts]
        while any(not r.finished for r in reqs):
            self.step()
        return [r.generated for r in reqs]
