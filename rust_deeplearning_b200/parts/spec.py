"""The description of a model as data.

An architecture turns its typed configuration into a `ModelSpec`: which mixer,
feed-forward and norms each layer has (with every size and constant as a
parameter), which tensors of the weight file each part reads, and the order in
which layers run.  The parts are built from it through the registries in
`parts.registry`; nothing below this description knows which architecture it
came from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part reads from the weight file.

    kind: "matrix"  - kept in the compute dtype (bfloat16 on the fast path, float32 on the 32-bit path)
          "vector"  - small parameter; a tensor stored in 32 bits stays 32-bit, otherwise it follows
                      the compute dtype
          "int"     - integer table, kept as int32
    init_std, init_mean: standard deviation and mean used by the random-weights mode.
    A size of None in `shape` is one that only the file gives (a low rank the configuration does not name): any
    size passes the checks there, and the random-weights mode, which needs a number, refuses the tensor.
    """
    name: str
    shape: Tuple[Optional[int], ...]
    kind: str = "matrix"
    init_std: float = 0.02
    init_mean: float = 0.0


def shape_fits(got, want) -> bool:
    """Whether a tensor's shape is the described one (None in the description: any size)."""
    return len(got) == len(want) and all(w is None or int(g) == int(w) for g, w in zip(got, want))


@dataclass(frozen=True)
class PartSpec:
    """A part to build: registry key, its sizes and constants, and its tensors by role."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)

    def walk(self):
        """This part and the parts named in its parameters (a position encoding, the two halves of a pair), depth first."""
        yield self
        for v in self.params.values():
            if isinstance(v, PartSpec):
                yield from v.walk()


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (`block`) and the parts it arranges."""
    block: str
    mixer: PartSpec
    feed_forward: Optional[PartSpec]      # None: the layer has a mixer only
    norms: Dict[str, PartSpec]
    params: Dict[str, Any] = field(default_factory=dict)     # constants of the arrangement itself (a post-norm block's alpha)
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)   # tensors of the arrangement itself, by role (gates on its branches)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers` (a layer may be named twice:
    each run has cache storage of its own).  `reads_cache_of` names an earlier schedule entry
    whose keys and values this run reads instead of writing its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # tensors a checkpoint of this architecture may carry that the model does not read (buffers such as
    # rotary frequencies, a copy of tied weights): names or shell-style patterns; they are skipped silently
    ignored_tensors: Tuple[str, ...] = ()

    def part_specs(self):
        yield self.embedding
        for layer in self.layers:
            yield from layer.mixer.walk()
            if layer.feed_forward is not None:
                yield from layer.feed_forward.walk()
            for n in layer.norms.values():
                yield n
            if layer.tensors:
                yield PartSpec("block_tensors", {}, layer.tensors)
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Every tensor the model reads, by file name.  A name used by two parts (tied
        weights) must be described identically by both."""
        out: Dict[str, TensorSpec] = {}
        for part in self.part_specs():
            for t in part.tensors.values():
                prev = out.get(t.name)
                if prev is not None and (prev.shape != t.shape or prev.kind != t.kind):
                    raise ValueError(f"tensor '{t.name}' is described twice with different shapes or kinds")
                out[t.name] = t
        return out

    def validate(self):
        for e, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {e} names layer {entry.layer}, model has {len(self.layers)}")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < e:
                raise ValueError(f"schedule entry {e} reads the cache of entry {entry.reads_cache_of}, "
                                 f"which does not run before it")
