"""The latent-attention mixer: keys and values of all heads compressed into one latent row per token.

Per token, with h the mixer's input, H heads, per head `dim` unrotated and `rot_dim` rotated query/key
dimensions, values of `vdim`, a latent of `kv_rank`:
    q          = W_q h                          heads laid out [dim | rot_dim]
    [l | kr0]  = W_dkv h                        kv_rank + rot_dim values
    c          = rms_norm(l; w_c, eps)          float statistics
    kr         = R_p(kr0),  q_rot <- R_p(q_rot) rotation by the position encoding (not on values)
    score_hj   = (q_un[h] . (W_uk[h] c_j) + q_rot[h] . kr_j) * score_scale      keys j inside the window
    o_h        = sum_j softmax_j(score_h) (W_uv[h] c_j)
    out        = W_o concat_h(o_h * sigmoid(W_g h)_h)
Only [c | kr] is cached: one row of kv_rank + rot_dim values per token for all heads
(`KVRequirement(1, kv_rank + rot_dim, window, value_dim=0)`: the values are read out of the key rows).
A layer may read the cached rows of an earlier layer instead of making its own (it then has no W_dkv;
`ScheduleEntry.reads_cache_of`), with its own W_uk, W_uv, queries, window and everything else.

Two ways of computing the same thing (`csrc/latent.cu`):
  * expanded - whole prompts in bfloat16: k_un and v of every head by one product c [W_uk; W_uv]^T, rows
    [Q | K | V] with heads padded to a common size, the ordinary prefill attention kernels, the gate;
  * absorbed - single tokens, prompts that continue a cached sequence, and the 32-bit path:
    q'[h] = [W_uk[h]^T q_un[h] | q_rot[h]] attends over the cached rows as keys and as values with one
    key/value head; head h's output is W_uv[h] applied to the first kv_rank values of the result.
Every size, the score scale, the window and the position encoding are parameters.  Two more, for designs that have them:
  sinks           a learned logit per head without key or value: exp(sink_h) joins the softmax's denominator once, unscaled
                  (tensor role "sinks")
  gate_per_value  the output gate has a row of W_g for every value of every head, out = W_o (concat_h(o_h) * sigmoid(W_g h)),
                  instead of one per head
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..cache.cache import KVRequirement, RunCache
from ..kernels import ops
from .attention import cache_owner
from .registry import BuildContext, build_part, register_part
from .spec import PartSpec


# "own": single-token steps use the decode kernel written for one cached row per token; "generic": the ordinary decode
# kernel with one key/value head where its sizes allow (for comparison; set RDL_LATENT_DECODE=generic)
LATENT_DECODE = os.environ.get("RDL_LATENT_DECODE", "own")


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class LatentAttention:
    query_tile_rows = ops.PREFILL_QUERY_TILE
    takes_deferred_rows = True     # x goes into the input projection and nowhere else
    delivers_branch = True         # the output projection may deliver the result through a stream's sink

    def __init__(self, *, hidden_size, n_heads, dim, rot_dim, vdim, kv_rank, score_scale, window, cache_window, eps,
                 position, wq, wdkv, dkv_norm, wuk, wuv, wg, wo, sinks=None, gate_per_value=False):
        H, d, rd, vd, r = n_heads, dim, rot_dim, vdim, kv_rank
        self.hidden_size, self.n_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = hidden_size, H, d, rd, vd, r
        self.score_scale, self.window, self.cache_window, self.eps = float(score_scale), window, cache_window, float(eps)
        self.position = position
        self.gate_per_value = bool(gate_per_value)
        self.gate_width = H * vd if self.gate_per_value else H
        if wg.shape[0] != self.gate_width:
            raise ValueError(f"latent attention: the gate's matrix has {wg.shape[0]} rows, {self.gate_width} are needed")
        if sinks is not None and sinks.numel() != H:
            raise ValueError(f"latent attention: {sinks.numel()} sinks for {H} heads")
        self.sinks = sinks.to(torch.float32).contiguous() if sinks is not None else None
        if not (hasattr(position, "tables") and hasattr(position, "rotary_dim")) or position.rotary_dim > rd:
            raise ValueError("latent attention needs a position encoding with tables over at most rot_dim dimensions")
        self.owns_latent = wdkv is not None
        # one product for q, the latent (where the layer has one) and the gate: rows of the matrices one after another
        self.w_in = torch.cat([wq] + ([wdkv] if self.owns_latent else []) + [wg], dim=0).contiguous()
        self.latent_col = H * (d + rd) if self.owns_latent else None
        self.gate_col = H * (d + rd) + ((r + rd) if self.owns_latent else 0)
        self.latent_norm = ops.NormParams(dkv_norm, self.eps, 0.0) if self.owns_latent else None
        # expanded form: [W_uk; W_uv] over the cached row [c | kr] (zero columns under kr, so that the row is used as it lies)
        w_ukv = torch.cat([wuk, wuv], dim=0)
        self.w_ukv = torch.cat([w_ukv, torch.zeros((w_ukv.shape[0], rd), dtype=w_ukv.dtype, device=w_ukv.device)], dim=1).contiguous()
        # absorbed form: per head W_uk[h]^T as [kv_rank, dim] and W_uv[h] as [vdim, kv_rank]
        self.w_uk_t = wuk.view(H, d, r).transpose(1, 2).contiguous()
        self.w_uk_b = wuk.view(H, d, r)      # the same matrices as a batched product's second operand
        self.w_uv_h = wuv.view(H, vd, r).contiguous()
        self.w_o = wo
        # the size heads are padded to for the ordinary prefill kernels: their fast forms take multiples of 64 (tensor
        # memory) or 16 (mma) up to 256
        need = max(d + rd, vd)
        self.pad = _round_up(need, 64) if _round_up(need, 64) <= 256 else _round_up(need, 16)

    def needs(self):
        return KVRequirement(1, self.kv_rank + self.rot_dim, self.cache_window, value_dim=0), None

    def _pages(self, batch, cache: RunCache) -> Optional[ops.KVPages]:
        if cache.k is None:
            return None
        return ops.KVPages(cache.k, cache.k, batch.tables[cache.kv_group], cache.page_size, cache.ring_pages)

    def forward(self, x, batch, cache: RunCache, run: int, sink=None):
        H, d, rd, vd, r = self.n_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        width = r + rd
        rows = ops.linear(x, self.w_in)
        pages = self._pages(batch, cache)
        cos, sin = self.position.tables()
        prep = dict(q_col=0, n_heads=H, dim=d, rot_dim=rd, latent_col=self.latent_col if cache.owns_kv else None, kv_rank=r,
                    norm=self.latent_norm, cos=cos, sin=sin, rot_n=self.position.rotary_dim,
                    interleaved=getattr(self.position, "interleaved", False), tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                    pages=pages, seq_end=batch.seq_end)
        gate = rows[:, self.gate_col:self.gate_col + self.gate_width]
        per_value = self.gate_per_value
        bf16 = rows.dtype is torch.bfloat16
        owner_rows = None if cache.owns_kv else batch.new_kv.get(cache_owner(batch, run))
        whole_prompts = not batch.is_decode and not batch.has_past and (cache.owns_kv or owner_rows is not None)

        if bf16 and whole_prompts and batch.n_tiles and self.pad <= 256:
            # ---- expanded: nothing is read from the cache, so the write rides along with the preparation ----
            latent = ops.latent_prepare(rows, write=True, **prep)
            if cache.owns_kv:
                if run in batch.shared_runs:
                    batch.new_kv[run] = (latent, 0, 0)
            else:
                latent = owner_rows[0]
            kv = ops.linear(latent, self.w_ukv)
            packed = ops.latent_assemble(rows, 0, kv, latent, n_heads=H, dim=d, rot_dim=rd, vdim=vd, kv_rank=r, pad=self.pad)
            ab = batch.attention_batch("past", self.window)
            ctx = ops.attention(packed, ab, None, n_heads=H, n_kv_heads=H, head_dim=self.pad, score_scale=self.score_scale,
                                softcap=None, window=self.window, new_kv=(packed, H * self.pad, 2 * H * self.pad),
                                kind="prefill_tc" if self.pad % 64 == 0 else "prefill", status=batch.status, sinks=self.sinks)
            return ops.linear_branch(ops.gate_heads(ctx, self.pad, gate, H, vd, per_value=per_value), self.w_o, sink)

        # ---- absorbed ----
        qp = torch.empty((rows.shape[0], H * width), dtype=rows.dtype, device=rows.device)
        # In a ring the write may overwrite rows of earlier steps that this step's early queries still need, so there
        # it comes after the attention (and after the runs that read this run's rows, if any).
        write_first = pages is not None and (batch.is_decode or not cache.is_ring or not batch.has_past)
        latent = ops.latent_prepare(rows, q_rot_out=qp, q_rot_col=r, q_rot_head=width, write=write_first, **prep)
        # the per-head products: the library's own kernel for few rows and in 32-bit; a batched library product where the
        # bfloat16 products of that many rows go to the library too (`ops.SKINNY_MAX_ROWS`)
        batched = bf16 and rows.shape[0] > ops.SKINNY_MAX_ROWS
        T = rows.shape[0]
        if batched:
            q_un = rows.as_strided((H, T, d), (d + rd, rows.stride(0), 1))
            qp.view(T, H, width)[:, :, :r].copy_(torch.bmm(q_un, self.w_uk_b).transpose(0, 1))
        else:
            ops.heads_linear(rows, 0, d + rd, self.w_uk_t, out=qp, out_col=0, out_head=width)
        common = dict(n_heads=H, n_kv_heads=1, head_dim=width, score_scale=self.score_scale, softcap=None, window=self.window,
                      sinks=self.sinks)
        if batch.is_decode or (not cache.owns_kv and owner_rows is None):
            ab = batch.attention_batch("all", self.window)
            generic = bf16 and batch.is_decode and H <= 8 and width % 16 == 0 and width <= 256 \
                and cache.page_size % 16 == 0 and cache.page_size <= 64
            if batch.is_decode and LATENT_DECODE == "own" and ops.latent_decode_ok(rows.dtype, width, r, cache.page_size):
                # all heads of a token share the cached rows a block has brought in
                ctx = ops.latent_decode(qp, ab, pages, n_heads=H, kv_rank=r, score_scale=self.score_scale, window=self.window,
                                        scratch=lambda n: batch.scratch_buffer("latent_decode", n), sinks=self.sinks)
            else:
                ctx = ops.attention(qp, ab, pages, kind="decode" if generic else "plain",
                                    scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
        else:
            if cache.owns_kv:
                if run in batch.shared_runs:
                    batch.new_kv[run] = (latent, 0, 0)
            else:
                latent = owner_rows[0]
            ab = batch.attention_batch("past", self.window)
            ctx = ops.attention(qp, ab, pages, new_kv=(latent, 0, 0), kind="plain", status=batch.status, **common)
            if cache.owns_kv and not write_first and pages is not None:
                def write(latent=latent, pages=pages):
                    ops.latent_write(latent, r, pages, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, seq_end=batch.seq_end)
                if run in batch.shared_runs and cache.is_ring and batch.has_past:
                    batch.deferred_writes[run] = write
                else:
                    write()
        if batched:
            per_head = torch.bmm(ctx.as_strided((H, T, r), (width, ctx.stride(0), 1)), self.w_uv_h.transpose(1, 2))     # [H, T, vdim]
            o = ops.gate_heads(per_head, T * vd, gate, H, vd, row_stride=vd, n_rows=T, per_value=per_value)
        else:
            o = ops.heads_linear(ctx, 0, width, self.w_uv_h, gate=gate, gate_per_value=per_value)
        return ops.linear_branch(o, self.w_o, sink)


def _build_latent_attention(spec: PartSpec, ctx: BuildContext) -> LatentAttention:
    p, t = spec.params, spec.tensors
    position = build_part("position", p["position"], ctx)
    get = lambda role: ctx.tensor(t[role]) if role in t else None
    return LatentAttention(hidden_size=p["hidden_size"], n_heads=p["n_heads"], dim=p["dim"], rot_dim=p["rot_dim"], vdim=p["vdim"],
                           kv_rank=p["kv_rank"], score_scale=p["score_scale"], window=p.get("window"),
                           cache_window=p.get("cache_window", p.get("window")), eps=p["eps"], position=position,
                           wq=get("q"), wdkv=get("dkv"), dkv_norm=get("dkv_norm"), wuk=get("uk"), wuv=get("uv"), wg=get("g"),
                           wo=get("o"), sinks=get("sinks"), gate_per_value=p.get("gate_per_value", False))


register_part("mixer", "latent_attention", _build_latent_attention, replace=True)
