"""The attention mixer: grouped-query attention over a paged cache.

Per token: q, k, v projections without bias (`rustml/nn/main/src/core/attention.rs:372-374`),
position encoding on q and k (`:394-398`), the new key and value rows go to the cache
(`:401`), scores times `score_scale`, soft-cap, causal and window mask, softmax, P.V
(`:413-446`), output projection (`:448`).  Head counts, head size, score scale, soft-cap,
window and the position encoding are parameters; the mixer does not know the model.

Interface of a mixer:
  needs() -> (KVRequirement | None, StateRequirement | None)  what it keeps per sequence
  forward(x [rows, hidden] normed, batch: StepBatch, cache: RunCache, run: int) -> [rows, hidden]
`cache.owns_kv` False means this run reads the keys and values another run wrote.

Optional parameters, for designs that have them (the reference's attention has none of these):
  qk_norm_eps  after rotation every query and key head is divided by its root mean square (no weight), in float
  proj_norm_eps  BEFORE rotation a token's whole query projection, all heads at once, is divided by its root mean square
               and multiplied by a learned weight per column, and its whole key projection likewise (tensor roles
               "q_norm" [n_heads * head_dim] and "k_norm" [n_kv_heads * head_dim]), in float
  sinks        a learned logit per query head without key or value: exp(sink_h) joins the softmax's denominator once
  gate         "sigmoid": the concatenated heads are multiplied element by element by sigmoid(W_g x) before W_o
  value_dim    values of another size than keys
  score_bias   no softmax: the weight of a visible key is sigmoid(score + score_bias[h]), a learned number per query head,
               and the weights are not normalised over the keys
  cache_window the keys the cache keeps per sequence where later runs that read this run's keys look further back than
               this run's own window (default: the window; "all": every key)
A run that reads another run's keys and values is built without wk and wv.
With any of them the mixer makes q, k, v and the gate's logits in one product and takes `ops.rope_norm_cache`
(rotation, head norm and cache write in one pass, rounded once) in place of `ops.rope_cache`.  Keys and values of
different sizes share the attention kernels by zero padding: the heads of q, k, v and of the gate are all laid out
with max(head_dim, value_dim) values, the padding made by zero rows of the product's matrix (and zero columns of
W_o), so that scores and outputs are unchanged and no kernel needs to know.
Optional offers for the split form of the norms around few-row products (`parts/norm.py`):
`takes_deferred_rows` (x may be `ops.DeferredRows`) and `delivers_branch` (forward takes `sink`).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.cache import KVRequirement, RunCache
from ..kernels import ops
from .registry import BuildContext, build_part, register_part
from .spec import PartSpec


class Attention:
    # the step's batch description lists its prompts cut into tiles of this many query rows (the prefill kernels' tiling)
    query_tile_rows = ops.PREFILL_QUERY_TILE

    def __init__(self, *, hidden_size, n_heads, n_kv_heads, head_dim, score_scale, softcap, window, position,
                 wq, wk, wv, wo, value_dim=None, qk_norm_eps=None, sinks=None, gate=None, wg=None, score_bias=None,
                 cache_window=None, proj_norm_eps=None, q_norm=None, k_norm=None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} key/value heads")
        value_dim = head_dim if value_dim is None else value_dim
        if window is None or cache_window == "all":
            self.cache_window = None
        else:
            self.cache_window = window if cache_window is None else int(cache_window)
            if self.cache_window < window:
                raise ValueError(f"attention: the cache keeps {self.cache_window} keys, the window spans {window}")
        if (proj_norm_eps is None) != (q_norm is None) or (q_norm is None) != (k_norm is None):
            raise ValueError("attention: the norm over the projections comes with its eps and both weights")
        if proj_norm_eps is not None and qk_norm_eps is not None:
            raise ValueError("attention: a norm over the whole projections and a norm of every head exclude each other")
        if score_bias is not None and (sinks is not None or qk_norm_eps is not None or gate is not None or proj_norm_eps is not None):
            raise ValueError("attention: sigmoid weights come without sinks, head norms or an output gate")
        if score_bias is not None and score_bias.numel() != n_heads:
            raise ValueError(f"attention: {score_bias.numel()} score biases for {n_heads} heads")
        self.score_bias = score_bias.to(torch.float32).contiguous() if score_bias is not None else None
        self.extended = (qk_norm_eps is not None or sinks is not None or gate is not None or proj_norm_eps is not None
                         or (value_dim != head_dim and score_bias is None))
        if self.extended:
            self._init_extended(hidden_size, n_heads, n_kv_heads, head_dim, value_dim, score_scale, softcap, window, position,
                                wq, wk, wv, wo, qk_norm_eps, sinks, gate, wg)
            self.proj_norm = None
            if proj_norm_eps is not None:
                if q_norm.numel() != n_heads * head_dim or k_norm.numel() != n_kv_heads * head_dim:
                    raise ValueError(f"attention: the projections' norms need {n_heads * head_dim} and {n_kv_heads * head_dim} weights")
                D = self.head_dim

                def columns(w, n):       # float32, laid out like the heads (zeros under their padding)
                    out = torch.zeros((n, D), dtype=torch.float32, device=w.device)
                    out[:, :head_dim] = w.to(torch.float32).view(n, head_dim)
                    return out.view(n * D).contiguous()

                self.proj_norm = (columns(q_norm, n_heads), columns(k_norm, n_kv_heads), float(proj_norm_eps),
                                  n_heads * head_dim, n_kv_heads * head_dim)
            return
        if (wk is None) != (wv is None):
            raise ValueError("attention: keys and values come together or not at all")
        if value_dim != head_dim:
            # keys and values of different sizes share the kernels by zero padding: every head is laid out with
            # max(head_dim, value_dim) values (zero rows of the products' matrices, zero columns of W_o)
            D = max(head_dim, value_dim)
            wq = _pad_heads(wq, n_heads, head_dim, D)
            if wk is not None:
                wk, wv = _pad_heads(wk, n_kv_heads, head_dim, D), _pad_heads(wv, n_kv_heads, value_dim, D)
            if value_dim != D:
                w = torch.zeros((wo.shape[0], n_heads, D), dtype=wo.dtype, device=wo.device)
                w[:, :, :value_dim] = wo.view(wo.shape[0], n_heads, value_dim)
                wo = w.view(wo.shape[0], n_heads * D).contiguous()
            head_dim = D
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.score_scale, self.softcap, self.window = float(score_scale), softcap, window
        self.position = position
        # one product for q, k and v: rows of the three matrices one after another
        self.w_qkv = torch.cat([wq, wk, wv], dim=0).contiguous() if wk is not None else wq.contiguous()
        self.w_q = self.w_qkv[: n_heads * head_dim]       # view, for runs that read another run's cache
        self.has_kv = wk is not None
        self.w_o = wo
        self.q_width = n_heads * head_dim
        self.kv_width = n_kv_heads * head_dim

    def _init_extended(self, hidden_size, n_heads, n_kv_heads, head_dim, value_dim, score_scale, softcap, window, position,
                       wq, wk, wv, wo, qk_norm_eps, sinks, gate, wg):
        if gate not in (None, "sigmoid", "silu") or (gate is None) != (wg is None):
            raise ValueError("attention: gate is None, 'sigmoid' or 'silu' and comes with its matrix")
        if sinks is not None and sinks.numel() != n_heads:
            raise ValueError(f"attention: {sinks.numel()} sinks for {n_heads} heads")
        D = max(head_dim, value_dim)          # the size all heads are laid out with

        def heads(w, n, d):                   # [n * d, in] -> [n * D, in], every head's rows padded with zero rows
            if d == D:
                return w
            out = torch.zeros((n, D, w.shape[1]), dtype=w.dtype, device=w.device)
            out[:, :d] = w.view(n, d, w.shape[1])
            return out.view(n * D, w.shape[1])

        parts = [heads(wq, n_heads, head_dim), heads(wk, n_kv_heads, head_dim), heads(wv, n_kv_heads, value_dim)]
        if wg is not None:
            parts.append(heads(wg, n_heads, value_dim))
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        if value_dim == D:
            self.w_o = wo
        else:                                 # zero columns under the padding of every head's output
            w = torch.zeros((wo.shape[0], n_heads, D), dtype=wo.dtype, device=wo.device)
            w[:, :, :value_dim] = wo.view(wo.shape[0], n_heads, value_dim)
            self.w_o = w.view(wo.shape[0], n_heads * D).contiguous()
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.head_dim, self.true_head_dim, self.value_dim = D, head_dim, value_dim
        self.score_scale, self.softcap, self.window, self.position = float(score_scale), softcap, window, position
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps is not None else 0.0
        self.sinks = sinks.to(torch.float32).contiguous() if sinks is not None else None
        self.gate = gate
        self.q_width, self.kv_width = n_heads * D, n_kv_heads * D
        self.g_col = self.q_width + 2 * self.kv_width
        self.takes_deferred_rows = False      # the rows are rotated and normed in place: a tensor is needed
        self.delivers_branch = False

    def _prepare_rows(self, rows, nh, nkv, hd, pages, prep):
        """Norm, rotation and cache write of a step's packed rows, in one pass."""
        if self.proj_norm is None:
            return ops.rope_norm_cache(rows, nh, nkv, hd, pages=pages, norm_eps=self.qk_norm_eps, norm_dim=self.true_head_dim, **prep)
        wq, wk, eps, q_count, k_count = self.proj_norm
        return ops.rope_projnorm_cache(rows, nh, nkv, hd, pages=pages, wq=wq, wk=wk, eps=eps, q_count=q_count, k_count=k_count, **prep)

    def _forward_extended(self, x, batch, cache: RunCache):
        """q, k, v and the gate in one product; the norms, rotation and cache write in one pass; attention with the
        sinks; the gate; the output product."""
        if not cache.owns_kv:
            raise ValueError("attention: a run with head norms, sinks or an output gate keeps keys and values of its own")
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        pages = self._pages(batch, cache)
        fast = x.dtype is torch.bfloat16 and hd % 16 == 0 and hd <= 256
        fast_decode = fast and nh // nkv <= 8 and cache.page_size % 16 == 0 and cache.page_size <= 64
        common = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, score_scale=self.score_scale, softcap=self.softcap,
                      window=self.window, sinks=self.sinks, status=batch.status)
        tables, rotary_dim = self._rotary_tables()
        if self.position is not None and tables is None:
            raise ValueError("attention: with head norms the position part must offer tables()")
        prep = dict(tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, cos=tables[0] if tables else None,
                    sin=tables[1] if tables else None, rotary_dim=rotary_dim, seq_end=batch.seq_end)
        rows = ops.linear(x, self.w_qkv)
        if batch.is_decode:
            self._prepare_rows(rows, nh, nkv, hd, pages, prep)
            ab = batch.attention_batch("all", self.window)
            ctx = ops.attention(rows, ab, pages, kind="decode" if fast_decode else "plain",
                                scratch=lambda n: batch.scratch_buffer("decode", n), **common)
        else:
            # in a ring the write may overwrite rows of earlier steps that this step's early queries still need
            write_first = pages is not None and (not cache.is_ring or not batch.has_past)
            self._prepare_rows(rows, nh, nkv, hd, pages if write_first else None, prep)
            ab = batch.attention_batch("past", self.window)
            if fast and batch.n_tiles:
                kind = "prefill_tc" if (hd % 64 == 0 and not batch.has_past) else "prefill"
            else:
                kind = "plain"
            ctx = ops.attention(rows, ab, pages, new_kv=(rows, self.q_width, self.q_width + self.kv_width), kind=kind, **common)
            if not write_first and pages is not None:
                ops.rope_norm_cache(rows, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, pages=pages, seq_end=batch.seq_end)
        if self.gate is not None:
            ctx = ops.gate_mul(ctx, rows[:, self.g_col:self.g_col + self.q_width], self.gate)
        return ops.linear(ctx, self.w_o)

    def needs(self):
        return KVRequirement(self.n_kv_heads, self.head_dim, self.cache_window), None

    def _pages(self, batch, cache: RunCache) -> Optional[ops.KVPages]:
        if cache.k is None:
            return None
        return ops.KVPages(cache.k, cache.v, batch.tables[cache.kv_group], cache.page_size, cache.ring_pages)

    def _rotary_tables(self):
        pos = self.position
        if pos is not None and hasattr(pos, "tables") and hasattr(pos, "rotary_dim"):
            return pos.tables(), pos.rotary_dim
        return None, 0

    takes_deferred_rows = True     # x goes into the q/k/v (or q) product and nowhere else
    delivers_branch = True         # the output projection may deliver the result through a stream's sink

    def forward(self, x, batch, cache: RunCache, run: int, sink=None):
        if self.extended:
            return self._forward_extended(x, batch, cache)
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        pages = self._pages(batch, cache)
        fast = x.dtype is torch.bfloat16 and hd % 16 == 0 and hd <= 256
        fast_decode = fast and nh // nkv <= 8 and cache.page_size % 16 == 0 and cache.page_size <= 64
        common = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, score_scale=self.score_scale,
                      softcap=self.softcap, window=self.window)
        if self.score_bias is not None:
            common["sigmoid_bias"] = self.score_bias
        tables, rotary_dim = self._rotary_tables()
        if cache.owns_kv and not self.has_kv:
            raise ValueError("attention: a run without key and value projections must read another run's cache")

        if not cache.owns_kv:
            # queries only; keys and values are those of another run of this step
            q = ops.linear(x, self.w_q)
            if self.position is not None:
                if tables is not None:
                    ops.rope_cache(q, nh, 0, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                                   cos=tables[0], sin=tables[1], rotary_dim=rotary_dim)
                else:
                    self.position.rotate(q, nh, 0, hd, batch)
            owner = batch.new_kv.get(cache_owner(batch, run))
            if batch.is_decode or owner is None:
                ab = batch.attention_batch("all", self.window)
                kind = "decode" if (fast_decode and batch.is_decode) else ("prefill" if fast and batch.n_tiles else "plain")
                ctx = ops.attention(q, ab, pages, kind=kind, scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
            else:
                rows, k_col, v_col = owner
                ab = batch.attention_batch("past", self.window)
                ctx = ops.attention(q, ab, pages, new_kv=(rows, k_col, v_col),
                                    kind="prefill" if fast and batch.n_tiles else "plain", **common)
            return ops.linear_branch(ctx, self.w_o, sink)

        qkv = ops.linear(x, self.w_qkv)
        if batch.is_decode and fast_decode and pages is not None and (tables is not None or self.position is None) \
                and rotary_dim % 16 == 0:
            # one kernel rotates, writes the new rows and attends over the cache
            ab = batch.attention_batch("all", self.window)
            ctx = ops.attention(qkv, ab, pages, new_kv=(qkv, self.q_width, self.q_width + self.kv_width), kind="decode",
                                rotate_and_write=(tables[0], tables[1], rotary_dim) if tables is not None else (None, None, 0),
                                scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
        elif batch.is_decode:
            # rotate, write the new row, then read everything from the cache
            if tables is not None or self.position is None:
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                               cos=tables[0] if tables else None, sin=tables[1] if tables else None,
                               rotary_dim=rotary_dim, pages=pages, seq_end=batch.seq_end)
            else:
                self.position.rotate(qkv, nh, nkv, hd, batch)
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, pages=pages,
                               seq_end=batch.seq_end)
            ab = batch.attention_batch("all", self.window)
            ctx = ops.attention(qkv, ab, pages, kind="decode" if fast_decode else "plain",
                                scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
        else:
            # rotate; attend over the cache (earlier steps) and the packed rows (this step); write.
            # In a ring the write may overwrite rows of earlier steps that this step's early queries still
            # need, so there it comes last; otherwise it rides along with the rotation.
            write_first = pages is not None and (not cache.is_ring or not batch.has_past)
            if tables is not None:
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                               cos=tables[0], sin=tables[1], rotary_dim=rotary_dim,
                               pages=pages if write_first else None, seq_end=batch.seq_end)
            else:
                if self.position is not None:
                    self.position.rotate(qkv, nh, nkv, hd, batch)
                write_first = False
            ab = batch.attention_batch("past", self.window)
            if fast and batch.n_tiles:
                # prompts that start at position 0 read nothing from the cache: the tcgen05 kernel takes them
                # (sigmoid weights: the mma.sync kernel, which has them; the tcgen05 kernel's softmax runs a thread per row)
                kind = "prefill_tc" if (hd % 64 == 0 and not batch.has_past and self.score_bias is None) else "prefill"
            else:
                kind = "plain"
            ctx = ops.attention(qkv, ab, pages, new_kv=(qkv, self.q_width, self.q_width + self.kv_width), kind=kind,
                                status=batch.status, **common)
            if run in batch.shared_runs:
                batch.new_kv[run] = (qkv, self.q_width, self.q_width + self.kv_width)
            if not write_first and pages is not None:
                def write(qkv=qkv, pages=pages):
                    ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, pages=pages,
                                   seq_end=batch.seq_end)
                if run in batch.shared_runs and cache.is_ring and batch.has_past:
                    # later runs of this step read this run's rows of earlier steps from the ring: write after them
                    batch.deferred_writes[run] = write
                else:
                    write()
        return ops.linear_branch(ctx, self.w_o, sink)


def _pad_heads(w, n, d, D):
    """[n * d, in] -> [n * D, in]: every head's rows followed by zero rows."""
    if d == D:
        return w
    out = torch.zeros((n, D, w.shape[1]), dtype=w.dtype, device=w.device)
    out[:, :d] = w.view(n, d, w.shape[1])
    return out.view(n * D, w.shape[1])


def cache_owner(batch, run: int) -> int:
    return batch.cache_owner_of[run]


def _build_attention(spec: PartSpec, ctx: BuildContext) -> Attention:
    p, t = spec.params, spec.tensors
    position = build_part("position", p["position"], ctx) if p.get("position") is not None else None
    return Attention(hidden_size=p["hidden_size"], n_heads=p["n_heads"], n_kv_heads=p["n_kv_heads"],
                     head_dim=p["head_dim"], score_scale=p["score_scale"], softcap=p.get("softcap"),
                     window=p.get("window"), position=position,
                     wq=ctx.tensor(t["q"]), wk=ctx.tensor(t["k"]) if "k" in t else None,
                     wv=ctx.tensor(t["v"]) if "v" in t else None, wo=ctx.tensor(t["o"]),
                     score_bias=ctx.tensor(t["score_bias"]) if "score_bias" in t else None, cache_window=p.get("cache_window"),
                     value_dim=p.get("value_dim"), qk_norm_eps=p.get("qk_norm_eps"),
                     sinks=ctx.tensor(t["sinks"]) if "sinks" in t else None, gate=p.get("gate"),
                     wg=ctx.tensor(t["g"]) if "g" in t else None, proj_norm_eps=p.get("proj_norm_eps"),
                     q_norm=ctx.tensor(t["q_norm"]) if "q_norm" in t else None,
                     k_norm=ctx.tensor(t["k_norm"]) if "k_norm" in t else None)


register_part("mixer", "attention", _build_attention, replace=True)
