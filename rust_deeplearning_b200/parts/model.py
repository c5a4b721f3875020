"""Embedding, output head, the arrangement of a block, and the model that runs a schedule.

Embedding: x[t] = E[id_t] * scale (`rustml/nn/main/src/core/embedding.rs:50-76`,
`rustml/nlp/main/src/core/model.rs:896-900`).  Head: z = n E^T for tied weights
(`model.rs:829-834, :936`) and cap * tanh(z / cap), which the architecture has and the
reference lacks.  Sandwich block: h = x + post(mixer(pre(x))); y = h + post'(ff(pre'(h)))
(`rustml/nn/main/src/core/transformer_block.rs:324-355`); which norms exist is data.

The model runs its schedule: a list of (layer, whose cache it reads).  A layer named
twice runs twice, each run with cache storage of its own.  Logits are formed only at the
rows the step wants (`model.rs:936` forms them at every position).

Post-norm block: x <- norm(alpha x + mixer(x)); x <- norm'(alpha x + ff(x)), for designs that
norm after the sum; alpha is `LayerSpec.params["alpha"]`.

Interface of a block: `forward(stream: ResidualStream, batch, cache: RunCache, run: int)`;
it adds its branches to the stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.cache import RunNeeds, StateRequirement
from ..kernels import ops
from .norm import ResidualStream
from .registry import BuildContext, build_part, register_part
from .spec import LayerSpec, ModelSpec


class ScaledEmbedding:
    def __init__(self, table: torch.Tensor, scale: float):
        self.table, self.scale = table, float(scale)
        self.vocab_size, self.hidden_size = table.shape

    def forward(self, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.embed_rows(self.table, tokens, self.scale, status)


register_part("embedding", "scaled_embedding",
              lambda spec, ctx: ScaledEmbedding(ctx.tensor(spec.tensors["table"]), spec.params.get("scale", 1.0)),
              replace=True)


class LinearHead:
    """float32 logits = soft-cap(pre_scale * n W^T) * scale: `pre_scale` multiplies the products before any soft-cap,
    `scale` the float32 result after it.  cap tanh(p z / cap) = p (cap / p) tanh(z / (cap / p)), so a pre_scale p runs as a
    soft-cap of cap / p in the product's epilogue followed by the scale p (times `scale`)."""

    def __init__(self, weight: torch.Tensor, softcap: Optional[float], scale: float = 1.0, pre_scale: float = 1.0):
        pre_scale = float(pre_scale)
        if pre_scale <= 0.0:
            raise ValueError(f"linear_head: pre_scale must be positive, got {pre_scale}")
        self.weight = weight
        self.softcap = float(softcap) / pre_scale if softcap is not None else None
        self.scale = float(scale) * pre_scale

    takes_deferred_rows = True      # n goes into one product and nowhere else

    def forward(self, n) -> torch.Tensor:
        z = ops.linear(n, self.weight, out_dtype=torch.float32, softcap=self.softcap)
        return ops.scale_(z, self.scale) if self.scale != 1.0 else z


register_part("head", "linear_head",
              lambda spec, ctx: LinearHead(ctx.tensor(spec.tensors["weight"]), spec.params.get("softcap"),
                                           spec.params.get("scale", 1.0), spec.params.get("pre_scale", 1.0)),
              replace=True)


class SandwichBlock:
    """pre-norm -> mixer -> optional post-norm -> add; pre-norm -> feed-forward -> optional post-norm -> add.
    A layer without a feed-forward (`LayerSpec.feed_forward` None) ends after the mixer's branch."""

    def __init__(self, mixer, feed_forward, norms: Dict[str, object], act_dtype: torch.dtype):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer = norms["pre_mixer"]
        self.post_mixer = norms.get("post_mixer")
        self.pre_ff = norms["pre_feed_forward"] if feed_forward is not None else None
        self.post_ff = norms.get("post_feed_forward")
        self.act_dtype = act_dtype

    @property
    def first_norm(self):
        """The norm this block asks the stream for first, if its mixer's first product takes the rows in the
        split form (`ops.DeferredRows`); the model tells the block before, so that its last product can prepare them."""
        return self.pre_mixer if getattr(self.mixer, "takes_deferred_rows", False) else None

    def forward(self, stream: ResidualStream, batch, cache, run: int):
        # Parts say what they can do with the split form of the norms (few rows; see ResidualStream):
        # takes_deferred_rows - x goes into ops.linear / ops.linear_gated only; delivers_branch - forward takes
        # `sink` and ends in ops.linear_branch.  Everything else runs through the norm kernels.
        mixer, ff = self.mixer, self.feed_forward
        m_in, m_out = getattr(mixer, "takes_deferred_rows", False), getattr(mixer, "delivers_branch", False)
        f_in, f_out = getattr(ff, "takes_deferred_rows", False), getattr(ff, "delivers_branch", False)
        after, stream.norm_after_block = stream.norm_after_block, None
        if ff is None:
            x = stream.normed(self.pre_mixer, self.act_dtype, deferred_ok=m_in, upcoming=after if m_out else None)
            sink = stream.branch_sink(self.post_mixer, after) if (m_out and after is not None) else None
            a = mixer.forward(x, batch, cache, run, sink=sink) if sink is not None else mixer.forward(x, batch, cache, run)
            stream.add(a, self.post_mixer)
            return
        x = stream.normed(self.pre_mixer, self.act_dtype, deferred_ok=m_in, upcoming=self.pre_ff if (m_out and f_in) else None)
        sink = stream.branch_sink(self.post_mixer, self.pre_ff) if (m_out and f_in) else None
        a = mixer.forward(x, batch, cache, run, sink=sink) if sink is not None else mixer.forward(x, batch, cache, run)
        stream.add(a, self.post_mixer)
        x = stream.normed(self.pre_ff, self.act_dtype, deferred_ok=f_in, upcoming=after if f_out else None)
        sink = stream.branch_sink(self.post_ff, after) if (f_out and after is not None) else None
        f = ff.forward(x, sink=sink) if sink is not None else ff.forward(x)
        stream.add(f, self.post_ff)


def _build_sandwich(layer: LayerSpec, ctx: BuildContext) -> SandwichBlock:
    mixer = build_part("mixer", layer.mixer, ctx)
    ff = build_part("feed_forward", layer.feed_forward, ctx) if layer.feed_forward is not None else None
    norms = {role: build_part("norm", s, ctx) for role, s in layer.norms.items()}
    return SandwichBlock(mixer, ff, norms, ctx.dtype)


register_part("block", "sandwich", _build_sandwich, replace=True)


class PostNormBlock:
    """Norm after the sum: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)).  The sublayers read the
    stream itself (in the activations' dtype), the sum and the norm run in float32 on the stream
    (`ResidualStream.renorm`); alpha is a parameter of the arrangement.  A layer without a feed-forward ends
    after the first sublayer."""

    def __init__(self, mixer, feed_forward, norms: Dict[str, object], act_dtype: torch.dtype, alpha: float):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.post_mixer = norms["post_mixer"]
        self.post_ff = norms["post_feed_forward"] if feed_forward is not None else None
        self.act_dtype, self.alpha = act_dtype, float(alpha)

    first_norm = None       # it asks the stream for its rows, not for a norm of them

    def forward(self, stream: ResidualStream, batch, cache, run: int):
        stream.norm_after_block = None
        a = self.mixer.forward(stream.rows(self.act_dtype), batch, cache, run)
        stream.renorm(a, self.post_mixer, self.alpha, self.act_dtype)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(stream.rows(self.act_dtype))
            stream.renorm(f, self.post_ff, self.alpha, self.act_dtype)


def _build_postnorm(layer: LayerSpec, ctx: BuildContext) -> PostNormBlock:
    mixer = build_part("mixer", layer.mixer, ctx)
    ff = build_part("feed_forward", layer.feed_forward, ctx) if layer.feed_forward is not None else None
    norms = {role: build_part("norm", s, ctx) for role, s in layer.norms.items()}
    return PostNormBlock(mixer, ff, norms, ctx.dtype, layer.params.get("alpha", 1.0))


register_part("block", "postnorm", _build_postnorm, replace=True)


class ParallelBlock:
    """One norm whose output both sublayers read, and one sum:
        n = norm(x);   x <- x + c1 * mixer(m) + c2 * ff(n)
    with two optional mechanisms, each a parameter of the arrangement (`LayerSpec.params`):
      token_shift      m_t = n_t + (n_(t-1) - n_t) * shift, element by element, n_(-1) = 0: the mixer reads every row moved
                       towards the row before it along its sequence (the feed-forward reads n as it is).  The sequence's
                       last n is state the block keeps per slot, beside the mixer's own (`needs()`); tensor role "shift".
      gated_residual   c1 = sigmoid(R1 n + b1), c2 = sigmoid(R2 n + b2), element by element (c = 1 without it); tensor
                       roles "gate_mixer", "gate_mixer_bias", "gate_ff", "gate_ff_bias".  Both gates are one product.
      branch_scale     x <- x + s * (mixer(n) + ff(n)) with a constant s (1 without it; not together with gated_residual).
    The norm, the shift, the gates' sigmoids and the sum run in float32 on the stream (one kernel before the sublayers,
    one after).  A feed-forward that keeps parts of its result apart (`forward_parts`) has them added in that last kernel.
    A layer without a feed-forward has the mixer's branch only.  Without shift and gates the block leaves its sum to
    the stream (`ResidualStream.add_sum`), which forms it together with the norm the next part asks for, in one kernel."""

    def __init__(self, mixer, feed_forward, norm, act_dtype: torch.dtype, hidden_size: int, shift, gates, branch_scale: float = 1.0):
        self.mixer, self.feed_forward, self.norm, self.act_dtype, self.hidden_size = mixer, feed_forward, norm, act_dtype, hidden_size
        self.branch_scale = float(branch_scale)
        if gates is not None and self.branch_scale != 1.0:
            raise ValueError("parallel block: a constant on the branches and gates on them exclude each other")
        if not callable(getattr(norm, "fused_params", None)) or norm.fused_params().offset != 0.0:
            raise ValueError("parallel block: the norm must be a scale-only root-mean-square norm without an offset")
        self.shift = shift
        self.w_gates = self.b_mixer = self.b_ff = None
        if gates is not None:
            w1, b1, w2, b2 = gates
            self.w_gates = torch.cat([w1, w2], dim=0).contiguous() if feed_forward is not None else w1.contiguous()
            self.b_mixer, self.b_ff = b1.contiguous(), (b2.contiguous() if feed_forward is not None else None)
        kv, state = mixer.needs()
        self._mixer_state = state
        own = (StateRequirement((hidden_size,), "float32"),) if shift is not None else ()
        mixer_states = () if state is None else (tuple(state) if isinstance(state, (tuple, list)) else (state,))
        self._needs = (kv, own + mixer_states if (own or mixer_states) else None)

    first_norm = None       # the norm is part of a kernel of the block's own

    def needs(self):
        return self._needs

    def _mixer_cache(self, cache):
        """The run's cache as the mixer declared it: its own state tensors without the block's."""
        if self._mixer_state is None:
            return cache._replace(state=None)
        rest = cache.state[1 if self.shift is not None else 0:]
        return cache._replace(state=rest if isinstance(self._mixer_state, (tuple, list)) else rest[0])

    def _feed_forward_parts(self, n):
        if self.feed_forward is None:
            return None, None
        if hasattr(self.feed_forward, "forward_parts"):
            return self.feed_forward.forward_parts(n)
        return self.feed_forward.forward(n), None

    def forward(self, stream: ResidualStream, batch, cache, run: int):
        stream.norm_after_block = None
        if self.shift is None and self.w_gates is None:
            n = stream.normed(self.norm, self.act_dtype)
            a = self.mixer.forward(n, batch, self._mixer_cache(cache), run)
            f1, f2 = self._feed_forward_parts(n)
            stream.add_sum((a, f1, f2), self.branch_scale)
            return
        x = stream.writable()
        p = self.norm.fused_params()
        if self.shift is not None:
            n, m = ops.norm_shift(x, p.weight, p.eps, self.shift, cache.state[0], tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                                  seq_start=batch.seq_start, slots=batch.slots, out_dtype=self.act_dtype)
        else:
            n = m = self.norm.apply(x, self.act_dtype)
        a = self.mixer.forward(m, batch, self._mixer_cache(cache), run)
        f1, f2 = self._feed_forward_parts(n)
        if self.w_gates is not None:
            ops.gated_residual_add_(x, ops.linear(n, self.w_gates), self.b_mixer, a, self.b_ff, f1, f2)
        else:
            ops.add_branches_norm_(x, (a, f1, f2), self.branch_scale)


def _build_parallel(layer: LayerSpec, ctx: BuildContext) -> ParallelBlock:
    mixer = build_part("mixer", layer.mixer, ctx)
    ff = build_part("feed_forward", layer.feed_forward, ctx) if layer.feed_forward is not None else None
    norm = build_part("norm", layer.norms["pre"], ctx)
    t = layer.tensors
    shift = ctx.tensor(t["shift"]) if layer.params.get("token_shift") else None
    gates = None
    if layer.params.get("gated_residual"):
        gates = (ctx.tensor(t["gate_mixer"]), ctx.tensor(t["gate_mixer_bias"]),
                 ctx.tensor(t["gate_ff"]) if ff is not None else None, ctx.tensor(t["gate_ff_bias"]) if ff is not None else None)
    return ParallelBlock(mixer, ff, norm, ctx.dtype, layer.params["hidden_size"], shift, gates, layer.params.get("branch_scale", 1.0))


register_part("block", "parallel", _build_parallel, replace=True)


class Model:
    """A model built from a ModelSpec and loaded tensors.  Nothing here names an architecture."""

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        ctx = BuildContext(weights, dtype, self.device)
        self.embedding = build_part("embedding", spec.embedding, ctx)
        keep = {t.name for p in (spec.embedding, spec.final_norm, spec.head) for t in p.tensors.values()}
        self.layers = []
        for layer in spec.layers:
            self.layers.append(build_block(layer, ctx))
            # parts hold what they need (fused copies or the tensors themselves)
            for p in (q for top in (layer.mixer, layer.feed_forward, *layer.norms.values()) if top is not None for q in top.walk()):
                for t in p.tensors.values():
                    if t.name not in keep:
                        weights.pop(t.name, None)
            for t in layer.tensors.values():
                if t.name not in keep:
                    weights.pop(t.name, None)
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)
        self.schedule = list(spec.schedule)
        self.cache_owner_of = {e: (s.reads_cache_of if s.reads_cache_of is not None else e)
                               for e, s in enumerate(self.schedule)}
        self.shared_runs = frozenset(s.reads_cache_of for s in self.schedule if s.reads_cache_of is not None)
        # the last run that reads each shared run's keys and values: a cache write that the owner puts off
        # (a ring whose rows this step's readers still need) is done after it
        self.last_reader = {}
        for e, s in enumerate(self.schedule):
            if s.reads_cache_of is not None:
                self.last_reader[s.reads_cache_of] = e
        self.vocab_size, self.hidden_size = spec.vocab_size, spec.hidden_size
        self.max_positions = spec.max_positions
        # Mixers may ask the step for its many-token sequences cut into query tiles of so many rows (a kernel's
        # tiling); the step's batch description then carries the tile lists.  One size per model.
        sizes = {getattr(layer.mixer, "query_tile_rows", 0) or 0 for layer in self.layers if hasattr(layer, "mixer")} - {0}
        if len(sizes) > 1:
            raise ValueError(f"the model's mixers ask for query tiles of different sizes: {sorted(sizes)}")
        self.query_tile_rows = sizes.pop() if sizes else 0

    def needs(self) -> List[RunNeeds]:
        """What each schedule entry needs of the cache."""
        out = []
        for s in self.schedule:
            block = self.layers[s.layer]
            # a block that keeps state of its own beside its mixer's says so itself
            kv, state = block.needs() if callable(getattr(block, "needs", None)) else block.mixer.needs()
            out.append(RunNeeds(kv, state, s.reads_cache_of))
        return out

    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the batch's tokens through the schedule; float32 logits [wanted rows, vocab]."""
        batch.cache_owner_of, batch.shared_runs = self.cache_owner_of, self.shared_runs
        batch.new_kv.clear()
        stream = ResidualStream(self.embedding.forward(batch.tokens))
        batch.deferred_writes.clear()
        lazy_head = getattr(self.head, "takes_deferred_rows", False)
        for run, entry in enumerate(self.schedule):
            # what the stream will be asked for after this block, where the asker's first product takes the split form
            if run + 1 < len(self.schedule):
                stream.norm_after_block = getattr(self.layers[self.schedule[run + 1].layer], "first_norm", None)
            else:
                stream.norm_after_block = self.final_norm if (lazy_head and batch.n_want) else None
            self.layers[entry.layer].forward(stream, batch, cache.run_cache(run), run)
            stream.norm_after_block = None
            for owner in [o for o in batch.deferred_writes if self.last_reader.get(o, o) <= run]:
                batch.deferred_writes.pop(owner)()
        for write in batch.deferred_writes.values():
            write()
        batch.deferred_writes.clear()
        batch.new_kv.clear()
        if batch.n_want == 0:
            stream.value()
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        n = stream.normed_rows(self.final_norm, batch.want_rows, self.dtype, deferred_ok=lazy_head)
        return self.head.forward(n)


def build_block(layer: LayerSpec, ctx: BuildContext):
    from .registry import _REGISTRY, PartError, registered_parts
    try:
        factory = _REGISTRY["block"][layer.block]
    except KeyError:
        raise PartError(f"no block of kind '{layer.block}'; registered: {registered_parts('block')}") from None
    return factory(layer, ctx)
