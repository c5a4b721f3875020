"""Typed entry points of the CUDA kernels, over torch tensors.

Each function checks devices, dtypes, shapes and contiguity, launches on torch's
current stream and returns torch tensors.  There is no other implementation
behind these names: on a machine without the library or without a GPU they
raise.  Parts call them as `ops.<name>` (attribute lookup at call time).
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import NamedTuple, Optional, Tuple

import torch

from . import library
from .library import AttentionArgs, KernelError, SamplingArgs

# Names of gated activations -> the codes of `csrc/api.h` (RDL_ACT_*).  The functions themselves are in
# `csrc/activations.cuh`, the one place every kernel with a gated epilogue takes them from.
ACTIVATIONS = {"gelu_pytorch_tanh": 0, "gelu_tanh": 0, "silu": 1}

# The status word of the step that is running: every kernel that can report a fault (a token id
# outside the table, a bounded wait that ran out) gets it unless the caller passes one of its own.
# The engine sets it around a step; parts need not know about it.
_step_status: Optional[torch.Tensor] = None


class step_status:
    """`with ops.step_status(word): ...` - kernels launched inside report their faults to `word` (int32[1])."""

    def __init__(self, word: Optional[torch.Tensor]):
        self.word = word

    def __enter__(self):
        global _step_status
        self.before, _step_status = _step_status, self.word
        return self.word

    def __exit__(self, *exc):
        global _step_status
        _step_status = self.before
        return False


def _status(status: Optional[torch.Tensor]):
    status = status if status is not None else _step_status
    return ctypes.c_void_p(status.data_ptr()) if status is not None else None


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype is torch.float32:
        return 0
    if t.dtype is torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _stream(t: torch.Tensor):
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; there is no CPU path")
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _dense(t, name):
    _need(t.is_contiguous(), f"{name} must be contiguous")
    return t


def _int32(t, name, n=None):
    _need(t.dtype is torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")
    if n is not None:
        _need(t.numel() >= n, f"{name} holds {t.numel()} entries, {n} are needed")
    return t


# ------------------------------------------------------------------------------------------
# row-wise kernels
# ------------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, scale: float, status: Optional[torch.Tensor] = None):
    """float32 rows `table[ids] * scale`.  An id outside the table poisons its row with NaN and
    sets `status[0]` (int32) if given."""
    _dense(table, "embedding table")
    _int32(ids, "ids")
    V, H = table.shape
    T = ids.numel()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    library.check(library.load().rdl_embed_rows(_ptr(out), _ptr(table), _dtype_code(table), _ptr(ids), float(scale),
                                                T, H, V, _status(status), _stream(table)))
    return out


class NormParams(NamedTuple):
    weight: torch.Tensor
    eps: float
    offset: float


def norm_residual_norm(x: torch.Tensor, *, first: Optional[NormParams] = None, residual: Optional[torch.Tensor] = None,
                       second: Optional[NormParams] = None, out_dtype: Optional[torch.dtype] = None,
                       row_index: Optional[torch.Tensor] = None, want_output: bool = True):
    """t = first ? rms_norm(x; first) : x;  h = residual + t (written back to `residual`, float32)
    or t;  returns second ? rms_norm(h; second) : h in `out_dtype`, or None if not wanted.
    rms_norm(v; w, eps, off) = v / sqrt(mean(v^2) + eps) * (w + off), statistics in float32."""
    _dense(x, "x")
    _need(x.dim() == 2, "x must be [rows, hidden]")
    H = x.shape[1]
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if row_index is not None:
        _int32(row_index, "row_index")
    for p, name in ((first, "first"), (second, "second")):
        if p is not None:
            _need(p.weight.is_contiguous() and p.weight.numel() == H, f"{name} norm weight must hold {H} values")
    if residual is not None:
        _need(residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, H),
              "residual must be a contiguous float32 [rows, hidden] tensor")
    y = torch.empty((rows, H), dtype=out_dtype or x.dtype, device=x.device) if want_output else None
    _need(y is not None or residual is not None, "norm_residual_norm: nothing to write")
    library.check(library.load().rdl_norm_residual_norm(
        _ptr(x), _dtype_code(x), _ptr(row_index),
        _ptr(first.weight) if first else None, _dtype_code(first.weight) if first else 0,
        float(first.eps) if first else 0.0, float(first.offset) if first else 0.0,
        _ptr(residual),
        _ptr(second.weight) if second else None, _dtype_code(second.weight) if second else 0,
        float(second.eps) if second else 0.0, float(second.offset) if second else 0.0,
        _ptr(y), _dtype_code(y) if y is not None else 0, rows, H, _stream(x)))
    return y


def gated_activation(gate_up: torch.Tensor, activation: str):
    """[rows, 2I] -> [rows, I]: act(gate_up[:, :I]) * gate_up[:, I:], computed in float32."""
    _dense(gate_up, "gate_up")
    _need(activation in ACTIVATIONS, f"unknown activation '{activation}', known: {sorted(ACTIVATIONS)}")
    rows, two_i = gate_up.shape
    _need(two_i % 2 == 0, "gate_up must have an even width")
    out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    library.check(library.load().rdl_gated_activation(_ptr(out), _ptr(gate_up), _dtype_code(gate_up),
                                                      ACTIVATIONS[activation], rows, two_i // 2, _stream(gate_up)))
    return out


def softcap_(z: torch.Tensor, cap: float):
    """In place on float32: cap * tanh(z / cap)."""
    _need(z.dtype is torch.float32 and z.is_contiguous(), "softcap_ takes a contiguous float32 tensor")
    library.check(library.load().rdl_softcap_inplace(_ptr(z), z.numel(), float(cap), _stream(z)))
    return z


def scale_(z: torch.Tensor, scale: float):
    """In place on float32: z * scale."""
    _need(z.dtype is torch.float32 and z.is_contiguous(), "scale_ takes a contiguous float32 tensor")
    library.check(library.load().rdl_scale_inplace(_ptr(z), z.numel(), float(scale), _stream(z)))
    return z


def residual_add_(residual: torch.Tensor, x: torch.Tensor):
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and x.is_contiguous()
          and residual.shape == x.shape, "residual_add_ takes a float32 residual and an addend of the same shape")
    library.check(library.load().rdl_residual_add(_ptr(residual), _ptr(x), _dtype_code(x), residual.numel(), _stream(x)))
    return residual


def convert_rows(x: torch.Tensor, out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None):
    """Rows of x (all, or those `row_index` names) converted to `out_dtype`."""
    _dense(x, "x")
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if row_index is not None:
        _int32(row_index, "row_index")
    out = torch.empty((rows, x.shape[1]), dtype=out_dtype, device=x.device)
    library.check(library.load().rdl_convert_rows(_ptr(out), _dtype_code(out), _ptr(x), _dtype_code(x), _ptr(row_index),
                                                  rows, x.shape[1], _stream(x)))
    return out


def postnorm_(residual: torch.Tensor, branch: torch.Tensor, norm: NormParams, alpha: float,
              out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """Norm after the sum, in place on the float32 stream: residual <- rms_norm(alpha * residual + branch; norm).
    With out_dtype the new rows are also returned in that type (the next part's input)."""
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and residual.dim() == 2,
          "postnorm_: the stream is a contiguous float32 [rows, width] tensor")
    _need(branch.is_contiguous() and branch.shape == residual.shape, "postnorm_: the branch must have the stream's shape")
    rows, width = residual.shape
    _need(norm.weight.is_contiguous() and norm.weight.numel() == width, f"postnorm_: the norm's weight must hold {width} values")
    y = torch.empty((rows, width), dtype=out_dtype, device=residual.device) if out_dtype is not None else None
    library.check(library.load().rdl_postnorm(_ptr(residual), _ptr(branch), _dtype_code(branch), float(alpha), _ptr(norm.weight),
                                              _dtype_code(norm.weight), float(norm.eps), float(norm.offset), _ptr(y),
                                              _dtype_code(y) if y is not None else 0, rows, width, _stream(residual)))
    return y


def add_branches_norm_(residual: torch.Tensor, branches, scale: float, norm: Optional[NormParams] = None,
                       out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """The sum of a block whose sublayers read one norm, in place on the float32 stream:
    residual <- residual + scale * (b0 + b1 + b2) for one to three branches of one dtype (added up in float, in that
    order); with `norm`, also returns rms_norm(residual; norm) in out_dtype, from the same pass over the rows."""
    branches = [b for b in branches if b is not None]
    _need(1 <= len(branches) <= 3, "add_branches_norm_: one to three branches")
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and residual.dim() == 2,
          "add_branches_norm_: the stream is a contiguous float32 [rows, width] tensor")
    for b in branches:
        _need(b.is_contiguous() and b.shape == residual.shape and b.dtype is branches[0].dtype,
              "add_branches_norm_: the branches must have the stream's shape and one dtype")
    rows, width = residual.shape
    y = None
    if norm is not None:
        _need(norm.weight.is_contiguous() and norm.weight.numel() == width, f"add_branches_norm_: the norm's weight must hold {width} values")
        y = torch.empty((rows, width), dtype=out_dtype or branches[0].dtype, device=residual.device)
    b = branches + [None, None]
    library.check(library.load().rdl_add_branches_norm(
        _ptr(residual), _ptr(b[0]), _ptr(b[1]), _ptr(b[2]), _dtype_code(b[0]), float(scale),
        _ptr(norm.weight) if norm is not None else None, _dtype_code(norm.weight) if norm is not None else 0,
        float(norm.eps) if norm is not None else 0.0, float(norm.offset) if norm is not None else 0.0,
        _ptr(y), _dtype_code(y) if y is not None else 0, rows, width, _stream(residual)))
    return y


def norm_pair(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, factor: float) -> torch.Tensor:
    """float32 factor * (rms_norm(a; wa) + rms_norm(b; wb)), both norms with plain weights."""
    _need(a.dim() == 2 and a.shape == b.shape and a.dtype is b.dtype and a.is_contiguous() and b.is_contiguous(),
          "norm_pair: two contiguous tensors of one shape and type")
    rows, width = a.shape
    _need(wa.dtype is wb.dtype and wa.is_contiguous() and wb.is_contiguous() and wa.numel() == width and wb.numel() == width,
          f"norm_pair: two weights of {width} values and one type")
    out = torch.empty((rows, width), dtype=torch.float32, device=a.device)
    library.check(library.load().rdl_norm_pair(_ptr(out), _ptr(a), _ptr(b), _dtype_code(a), _ptr(wa), _ptr(wb), _dtype_code(wa),
                                               float(eps), float(factor), rows, width, _stream(a)))
    return out


GATES = {"sigmoid": 0, "silu": 1}     # element-wise output gates (`csrc/api.h`, RDL_GATE_*)


def gate_mul(x: torch.Tensor, gate: torch.Tensor, kind: str) -> torch.Tensor:
    """x * gate_fn(gate), element by element, in float; x and gate may be column slices of wider rows."""
    _need(kind in GATES, f"unknown gate '{kind}', known: {sorted(GATES)}")
    _need(x.dim() == 2 and gate.shape == x.shape and gate.dtype is x.dtype and x.stride(1) == 1 and gate.stride(1) == 1,
          "gate_mul: rows and gates of one shape and type")
    out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    library.check(library.load().rdl_gate_mul(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0),
                                              _dtype_code(x), GATES[kind], x.shape[0], x.shape[1], _stream(x)))
    return out


def group_norm_gate(x: torch.Tensor, groups: int, *, eps: float, weight: Optional[torch.Tensor] = None,
                    gate: Optional[torch.Tensor] = None, gate_kind: str = "sigmoid",
                    out_dtype: torch.dtype = torch.float32, gate_first: bool = False) -> torch.Tensor:
    """float32 rows [rows, groups * n] normed group by group (v / sqrt(mean(v^2) + eps)), times weight[column] if
    given, times gate_fn(gate[row, column]) if given (gate may be a column slice of wider rows); result in out_dtype.
    gate_first: the gate multiplies the values before the norm, so that the root mean square is that of the gated values."""
    _need(x.dtype is torch.float32 and x.dim() == 2 and x.is_contiguous() and x.shape[1] % groups == 0,
          "group_norm_gate: contiguous float32 rows whose width the groups divide")
    _need(gate_kind in GATES, f"unknown gate '{gate_kind}', known: {sorted(GATES)}")
    rows, width = x.shape
    if weight is not None:
        _need(weight.is_contiguous() and weight.numel() == width, f"group_norm_gate: the weight must hold {width} values")
    if gate is not None:
        _need(gate.dim() == 2 and tuple(gate.shape) == (rows, width) and gate.stride(1) == 1, "group_norm_gate: bad gate rows")
    out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    library.check(library.load().rdl_group_norm_gate(
        _ptr(out), _dtype_code(out), _ptr(x), rows, groups, width // groups, _ptr(weight),
        _dtype_code(weight) if weight is not None else 0, float(eps), _ptr(gate), gate.stride(0) if gate is not None else 0,
        _dtype_code(gate) if gate is not None else 0, GATES[gate_kind], int(bool(gate_first)), _stream(x)))
    return out


# ------------------------------------------------------------------------------------------
# matrix products
# ------------------------------------------------------------------------------------------

SKINNY_MAX_ROWS = 16     # up to this many rows the weight-streaming kernel runs; above, the tcgen05 kernel
# "tcgen05": the library's own TMA + tcgen05 kernel for products with many rows; "cublas": the library
# product through torch (kept for comparison; set RDL_PREFILL_GEMM=cublas)
PREFILL_GEMM = os.environ.get("RDL_PREFILL_GEMM", "tcgen05")


def _bf16_ok(x, weight):
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _skinny_ok(x, weight):
    return _bf16_ok(x, weight) and x.shape[0] <= SKINNY_MAX_ROWS


TC_MIN_ROWS = 128        # a tcgen05 tile holds 128 rows; between 17 and 127 rows a library product stands


def _own_bf16_kernel(x, weight):
    """Few rows: the weight-streaming kernel.  A tile's worth of rows or more: the tcgen05 kernel.
    In between a 128-row tile would be mostly empty and too few blocks would stream the weights,
    so the library product (cuBLAS through torch) takes those."""
    if not _bf16_ok(x, weight):
        return False
    rows = x.shape[0]
    return rows <= SKINNY_MAX_ROWS or (rows >= TC_MIN_ROWS and PREFILL_GEMM == "tcgen05")


def _gemm_bf16(x, weight, n_out, out_dtype, gated, activation, softcap, status):
    """The library's own bfloat16 products: weight streaming for few rows, tcgen05 for many."""
    out = torch.empty((x.shape[0], n_out), dtype=out_dtype, device=x.device)
    lib = library.load()
    if x.shape[0] <= SKINNY_MAX_ROWS:
        library.check(lib.rdl_gemm_skinny(_ptr(out), _dtype_code(out), _ptr(x), _ptr(weight), x.shape[0], n_out, x.shape[1],
                                          int(gated), activation, float(softcap or 0.0), _status(status), _stream(x)))
    else:
        library.check(lib.rdl_gemm_tc(_ptr(out), _dtype_code(out), _ptr(x), _ptr(weight), x.shape[0], n_out, x.shape[1],
                                      int(gated), activation, float(softcap or 0.0), _status(status), _stream(x)))
    return out


# ------------------------------------------------------------------------------------------
# deferred norms: "norm the branch, add it to the stream, norm the sum" without a kernel of its own
# ------------------------------------------------------------------------------------------
# With up to DEFERRED_MAX_ROWS rows (decode) the two norms between the last product of a branch (P) and the
# first product after them (C) cost more than the products: a kernel that waits for whole rows twice.  The
# norms are scalings by one number a row and one number a column, so they can be split (the algebra stands in
# csrc/api.h at DeferredNormArgs): P's epilogue applies the column factors and writes partial sums of squares,
# C multiplies an operand of 2 x 8 rows (the stream's rows and the branch's rows, both with the second norm's
# column factors) and applies the row factors in its epilogue.  Three small types carry this through the parts.

DEFERRED_MAX_ROWS = 8
# A very wide product (the output head) runs for most of its time in its steady state, where multiplying 16 rows
# instead of 8 costs more than the two small kernels it saves (256,000 outputs: 230 against 165 us): its rows are
# made into a tensor first.
DEFERRED_MAX_OUTPUTS = 65536
DEFERRED_NORMS = os.environ.get("RDL_DEFERRED_NORMS", "1") != "0"     # 0: the norm kernels everywhere, for comparison


class BranchSink(NamedTuple):
    """What the last product of a branch is given so that it can deliver its result in the split form."""
    residual: torch.Tensor     # float32 [rows, width]: the stream the branch will be added to
    post: NormParams           # the norm of the branch before the sum
    then: NormParams           # the norm the sum is asked for next
    operand: torch.Tensor      # bfloat16 [16, width]: its first rows are (by the time the product runs) residual * (then.weight + then.offset)


class Branch:
    """A branch delivered through a BranchSink: a' = y (post.weight + post.offset) [rows, width] in bfloat16,
    the partial sums [units, 8, 4] and, in the operand's second half (`second_half_row`), a' (then.weight + then.offset)."""

    def __init__(self, sink: BranchSink, values: torch.Tensor, sums: torch.Tensor):
        self.sink, self.values, self.sums = sink, values, sums
        self.shape, self.dtype, self.device = values.shape, values.dtype, values.device


class DeferredRows:
    """Stands for then(residual + post(branch)) [rows, width], or for `row_index`'s rows of it, in the act dtype.
    `linear` and `linear_gated` take it in place of a tensor; `materialise()` gives the tensor.  Its first
    use also writes the updated stream to `residual_out` and, if `next_norm` is given, the first half of
    `next_operand` (the rows of the updated stream times that norm's column factors)."""

    def __init__(self, branch: Branch, residual_out: torch.Tensor, next_norm: Optional[NormParams] = None,
                 next_operand: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None):
        self.branch, self.residual_out = branch, residual_out
        self.next_norm, self.next_operand, self.row_index = next_norm, next_operand, row_index
        rows = row_index.numel() if row_index is not None else branch.shape[0]
        self.shape, self.dtype, self.device = (rows, branch.shape[1]), branch.dtype, branch.device
        self.consumed = False

    def _args(self) -> "library.DeferredNormArgs":
        b, k = self.branch, self.branch.sink
        d = library.DeferredNormArgs()
        d.mode = library.NORM_DEFERRED
        d.sums, d.n_sums = b.sums.data_ptr(), b.sums.shape[0]
        d.eps1, d.eps2 = float(k.post.eps), float(k.then.eps)
        d.n_out = self.shape[0]
        if self.row_index is not None:
            d.row_index = self.row_index.data_ptr()
        if not self.consumed:
            d.branch_in, d.residual_in, d.residual_out = b.values.data_ptr(), k.residual.data_ptr(), self.residual_out.data_ptr()
            if self.next_norm is not None:
                w = self.next_norm.weight
                d.w_next, d.w_next_dtype, d.off_next = w.data_ptr(), _dtype_code(w), float(self.next_norm.offset)
                d.scaled_next = self.next_operand.data_ptr()
        return d

    def materialise(self) -> torch.Tensor:
        b, k = self.branch, self.branch.sink
        rows, width = b.shape
        if not self.consumed:
            n = self.next_norm
            library.check(library.load().rdl_stream_rows(
                _ptr(b.sums), b.sums.shape[0], float(k.post.eps), _ptr(b.values), _ptr(k.residual), _ptr(self.residual_out),
                _ptr(n.weight) if n else None, _dtype_code(n.weight) if n else 0, float(n.offset) if n else 0.0,
                _ptr(self.next_operand) if n else None, rows, width, _stream(b.values)))
            self.consumed = True
        return norm_residual_norm(self.residual_out, second=k.then, out_dtype=self.dtype, row_index=self.row_index)


def add_branch_(branch: Branch) -> torch.Tensor:
    """residual += s1 * a' in place: a split branch that no product takes further."""
    k = branch.sink
    rows, width = branch.shape
    library.check(library.load().rdl_stream_rows(_ptr(branch.sums), branch.sums.shape[0], float(k.post.eps), _ptr(branch.values),
                                                 _ptr(k.residual), _ptr(k.residual), None, 0, 0.0, None, rows, width,
                                                 _stream(branch.values)))
    return k.residual


def scaled_rows(residual: torch.Tensor, norm: NormParams, operand: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The first half of a deferred product's operand, made by a kernel of its own (the first link of a chain):
    rows 0.. of a bfloat16 [16, width] buffer = residual * (norm.weight + norm.offset)."""
    rows, width = residual.shape
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and rows <= DEFERRED_MAX_ROWS, "scaled_rows: up to 8 contiguous float32 rows")
    if operand is None:
        operand = torch.empty((2 * DEFERRED_MAX_ROWS, width), dtype=torch.bfloat16, device=residual.device)
    library.check(library.load().rdl_stream_rows(None, 0, 0.0, None, _ptr(residual), None, _ptr(norm.weight), _dtype_code(norm.weight),
                                                 float(norm.offset), _ptr(operand), rows, width, _stream(residual)))
    return operand


def second_half_row(rows: int) -> int:
    """The operand's row at which the branch's half starts: 8, or 4 with up to 4 rows (the two halves then share one
    8-row fragment of the tensor-core product and cost what 8 plain rows cost)."""
    return 4 if rows <= 4 else DEFERRED_MAX_ROWS


def deferred_ok(rows: int, width: int, dtype: torch.dtype) -> bool:
    """Whether rows of this many and this width can take the split form at all."""
    return DEFERRED_NORMS and dtype is torch.bfloat16 and 0 < rows <= DEFERRED_MAX_ROWS and width % 8 == 0


def linear_branch(x: torch.Tensor, weight: torch.Tensor, sink: Optional[BranchSink], status: Optional[torch.Tensor] = None):
    """x W^T as a branch of a residual stream: a `Branch` where the split form applies, else the plain result."""
    if sink is None or not (_skinny_ok(x, weight) and deferred_ok(x.shape[0], weight.shape[0], x.dtype)
                            and tuple(sink.residual.shape) == (x.shape[0], weight.shape[0])):
        return linear(x, weight, status=status)
    rows, width = x.shape[0], weight.shape[0]
    for p in (sink.post, sink.then):
        _need(p.weight.is_contiguous() and p.weight.numel() == width, f"a norm's weight must hold {width} values")
    _need(sink.operand.dtype is torch.bfloat16 and tuple(sink.operand.shape) == (2 * DEFERRED_MAX_ROWS, width)
          and sink.operand.is_contiguous(), "the sink's operand must be bfloat16 [16, width]")
    values = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device)
    sums = torch.empty(((width + 15) // 16, 8, 4), dtype=torch.float32, device=x.device)
    d = library.DeferredNormArgs()
    d.mode = library.NORM_BRANCH
    d.sums = sums.data_ptr()
    d.residual = sink.residual.data_ptr()
    d.w1, d.w1_dtype, d.off1 = sink.post.weight.data_ptr(), _dtype_code(sink.post.weight), float(sink.post.offset)
    d.w2, d.w2_dtype, d.off2 = sink.then.weight.data_ptr(), _dtype_code(sink.then.weight), float(sink.then.offset)
    d.branch, d.scaled = values.data_ptr(), sink.operand.data_ptr() + second_half_row(rows) * width * 2
    library.check(library.load().rdl_gemm_skinny_norm(None, 0, _ptr(x), _ptr(weight), rows, width, x.shape[1], 0, 0, 0.0,
                                                      ctypes.byref(d), _status(status), _stream(x)))
    return Branch(sink, values, sums)


def _linear_deferred(x: DeferredRows, weight: torch.Tensor, n_out: int, out_dtype, gated: bool, activation: int, softcap, status):
    """The product after a deferred norm, or None if this weight cannot take it."""
    width = x.branch.shape[1]
    if not (weight.dtype is torch.bfloat16 and weight.is_contiguous() and weight.data_ptr() % 16 == 0 and weight.shape[1] == width):
        return None
    if n_out > DEFERRED_MAX_OUTPUTS:
        return None
    out = torch.empty((x.shape[0], n_out), dtype=out_dtype, device=weight.device)
    d = x._args()
    library.check(library.load().rdl_gemm_skinny_norm(_ptr(out), _dtype_code(out), _ptr(x.branch.sink.operand), _ptr(weight),
                                                      x.branch.shape[0], n_out, width, int(gated), activation, float(softcap or 0.0),
                                                      ctypes.byref(d), _status(status), _stream(out)))
    x.consumed = True
    return out


def activation_(x: torch.Tensor, kind: str) -> torch.Tensor:
    """An element-wise activation of `UNARY_FORMS` on a dense tensor, in place (float arithmetic)."""
    _need(kind in UNARY_FORMS, f"unknown activation '{kind}', known: {sorted(UNARY_FORMS)}")
    _need(x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16), "activation_: a dense float32 or bfloat16 tensor")
    library.check(library.load().rdl_activation_inplace(_ptr(x), _dtype_code(x), x.numel(), UNARY_FORMS[kind], _stream(x)))
    return x


def linear(x, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           softcap: Optional[float] = None, status: Optional[torch.Tensor] = None, activation: Optional[str] = None):
    """x [rows, in] times weight [out, in] transposed; optionally cap * tanh(. / cap) on the result.
    x may be `DeferredRows` (the rows after a deferred norm).  activation: an element-wise form of `UNARY_FORMS`
    on the result (the product's epilogue in the library's own bfloat16 kernels, a kernel of its own elsewhere).

    float32: the library's own FMA kernel (no tensor cores, no reduced-precision mode).
    bfloat16: up to 16 rows (decode) the weight-streaming tensor-core kernels, from 128 rows the TMA +
    tcgen05 kernels, all with float accumulation and the soft-cap in their epilogue.  17 to 127 rows, and
    operands that do not meet the alignment rules, go to a library product (cuBLAS through torch), which
    is what the reference's engine uses for all its products."""
    _need(activation is None or (activation in UNARY_FORMS and softcap is None),
          f"linear: activation '{activation}' is not one of {sorted(UNARY_FORMS)} (and comes without a soft-cap)")
    if isinstance(x, DeferredRows):
        _need(softcap is None or out_dtype is torch.float32, "linear: the soft-cap is applied to float32 results")
        out = _linear_deferred(x, weight, weight.shape[0], out_dtype or x.dtype, False, 0, softcap, status) if activation is None else None
        if out is not None:
            return out
        x = x.materialise()
    _need(x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1],
          f"linear: shapes {tuple(x.shape)} and {tuple(weight.shape)} do not fit")
    _need(x.dtype is weight.dtype, f"linear: input is {x.dtype}, weight is {weight.dtype}")
    out_dtype = out_dtype or x.dtype
    _need(softcap is None or out_dtype is torch.float32, "linear: the soft-cap is applied to float32 results")
    if x.dtype is torch.float32:
        _need(out_dtype is torch.float32, "linear: the 32-bit path writes float32")
        _dense(x, "x"); _dense(weight, "weight")
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        library.check(library.load().rdl_gemm_f32(_ptr(out), _ptr(x), _ptr(weight), x.shape[0], weight.shape[0],
                                                  x.shape[1], _stream(x)))
    elif _own_bf16_kernel(x, weight):
        return _gemm_bf16(x, weight, weight.shape[0], out_dtype, False, UNARY_FORMS[activation] if activation else 0, softcap, status)
    else:
        _need(x.is_cuda, "kernels run on CUDA tensors only; there is no CPU path")
        out = torch.mm(x, weight.t(), out_dtype=torch.float32) if out_dtype is torch.float32 else torch.mm(x, weight.t())
    if softcap is not None:
        softcap_(out, softcap)
    if activation is not None:
        activation_(out, activation)
    return out


def linear_gated(x, weight_gate_up: torch.Tensor, activation: str, status: Optional[torch.Tensor] = None):
    """act(x Wg^T) * (x Wu^T) for the row-concatenated matrix [Wg; Wu] ([2I, in]) -> [rows, I].
    In bfloat16 this is one kernel (the activation is the product's epilogue); otherwise a product
    and the gated activation kernel."""
    _need(activation in ACTIVATIONS, f"unknown activation '{activation}', known: {sorted(ACTIVATIONS)}")
    _need(weight_gate_up.shape[0] % 2 == 0, "linear_gated: the weight must hold gate rows and as many up rows")
    if isinstance(x, DeferredRows):
        out = _linear_deferred(x, weight_gate_up, weight_gate_up.shape[0] // 2, x.dtype, True, ACTIVATIONS[activation], None, status)
        if out is not None:
            return out
        x = x.materialise()
    if _own_bf16_kernel(x, weight_gate_up):
        return _gemm_bf16(x, weight_gate_up, weight_gate_up.shape[0] // 2, x.dtype, True, ACTIVATIONS[activation], None, status)
    return gated_activation(linear(x, weight_gate_up), activation)


# ------------------------------------------------------------------------------------------
# position encoding, cache write, attention
# ------------------------------------------------------------------------------------------

class KVPages(NamedTuple):
    """One schedule entry's key/value storage and the page lists of the step's sequences."""
    k: torch.Tensor            # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    tables: torch.Tensor       # int32 [n_seqs, table_width]
    page_size: int
    ring_pages: int            # entries of a page list used as a ring (= table width when all keys are kept)


def rope_cache(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, *, tok_seq, tok_pos,
               cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rotary_dim: int = 0,
               pages: Optional[KVPages] = None, seq_end: Optional[torch.Tensor] = None):
    """In place on packed rows [tokens, (n_heads + 2 n_kv_heads) * head_dim]: rotate query and key heads by
    the tables (if given), then write key and value rows to the cache (if `pages` is given)."""
    _dense(qkv, "qkv")
    T = qkv.shape[0]
    _need(qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "qkv width does not match the head counts")
    _int32(tok_pos, "tok_pos", T)
    _int32(tok_seq, "tok_seq", T)
    do_rope = cos is not None
    if do_rope:
        _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
    do_write = pages is not None and n_kv_heads > 0
    if do_write:
        _need(pages.k.dtype is qkv.dtype and pages.v.dtype is qkv.dtype, "cache dtype differs from the activations'")
        _need(tuple(pages.k.shape[1:]) == (n_kv_heads, pages.page_size, head_dim) and pages.k.is_contiguous()
              and pages.v.is_contiguous() and pages.v.shape == pages.k.shape, "cache storage has the wrong shape")
        _int32(pages.tables, "page tables")
        _int32(seq_end, "seq_end")
    library.check(library.load().rdl_rope_cache(
        _ptr(qkv), _dtype_code(qkv), T, n_heads, n_kv_heads, head_dim, rotary_dim,
        _ptr(cos), _ptr(sin), _ptr(tok_seq), _ptr(tok_pos), int(do_rope), int(do_write),
        _ptr(pages.k) if do_write else None, _ptr(pages.v) if do_write else None,
        _ptr(pages.tables) if do_write else None, pages.tables.shape[1] if do_write else 0,
        pages.page_size if do_write else 0, pages.ring_pages if do_write else 0,
        _ptr(seq_end) if do_write else None, _stream(qkv)))
    return qkv


def rope_norm_cache(rows: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, *, tok_seq, tok_pos,
                    cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                    norm_eps: float = 0.0, norm_dim: Optional[int] = None, pages: Optional[KVPages] = None,
                    seq_end: Optional[torch.Tensor] = None):
    """In place on packed rows [tokens, >= (n_heads + 2 n_kv_heads) * head_dim] (the row stride may exceed the heads):
    every query and key head is rotated by the tables (if given) and, with norm_eps > 0, divided by
    sqrt(sum of squares / norm_dim + norm_eps), all in float and rounded once; key and value rows then go to the
    cache (if `pages` is given).  norm_dim: the head's size without zero padding (default head_dim)."""
    _need(rows.dim() == 2 and rows.stride(1) == 1 and rows.shape[1] >= (n_heads + 2 * n_kv_heads) * head_dim,
          "rope_norm_cache: packed rows narrower than the heads")
    T = rows.shape[0]
    _int32(tok_pos, "tok_pos", T)
    _int32(tok_seq, "tok_seq", T)
    do_rope = cos is not None
    if do_rope:
        _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
    do_write = pages is not None and n_kv_heads > 0
    if do_write:
        _need(pages.k.dtype is rows.dtype and pages.v.dtype is rows.dtype, "cache dtype differs from the activations'")
        _need(tuple(pages.k.shape[1:]) == (n_kv_heads, pages.page_size, head_dim) and pages.k.is_contiguous()
              and pages.v.is_contiguous() and pages.v.shape == pages.k.shape, "cache storage has the wrong shape")
        _int32(pages.tables, "page tables")
        _int32(seq_end, "seq_end")
    library.check(library.load().rdl_rope_norm_cache(
        _ptr(rows), rows.stride(0), _dtype_code(rows), T, n_heads, n_kv_heads, head_dim, rotary_dim if do_rope else 0,
        _ptr(cos), _ptr(sin), _ptr(tok_seq), _ptr(tok_pos), int(do_rope), float(norm_eps), int(norm_dim or head_dim),
        int(do_write), _ptr(pages.k) if do_write else None, _ptr(pages.v) if do_write else None,
        _ptr(pages.tables) if do_write else None, pages.tables.shape[1] if do_write else 0,
        pages.page_size if do_write else 0, pages.ring_pages if do_write else 0,
        _ptr(seq_end) if do_write else None, _stream(rows)))
    return rows


def rope_projnorm_cache(rows: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, *, tok_seq, tok_pos, wq: torch.Tensor,
                        wk: Optional[torch.Tensor], eps: float, q_count: int, k_count: int, cos: Optional[torch.Tensor] = None,
                        sin: Optional[torch.Tensor] = None, rotary_dim: int = 0, pages: Optional[KVPages] = None,
                        seq_end: Optional[torch.Tensor] = None):
    """In place on packed rows [tokens, >= (n_heads + 2 n_kv_heads) * head_dim]: a root-mean-square norm over a token's
    WHOLE query projection and over its WHOLE key projection (all heads at once; float32 weights wq [n_heads * head_dim],
    wk [n_kv_heads * head_dim], one per column), then the rotation of every query and key head by the tables (if given),
    all in float and rounded once; key and value rows then go to the cache (if `pages` is given).
    q_count, k_count: the projections' sizes without any zero padding of their heads (what the mean divides by)."""
    _need(rows.dim() == 2 and rows.stride(1) == 1 and rows.shape[1] >= (n_heads + 2 * n_kv_heads) * head_dim,
          "rope_projnorm_cache: packed rows narrower than the heads")
    T = rows.shape[0]
    _int32(tok_pos, "tok_pos", T)
    _int32(tok_seq, "tok_seq", T)
    _need(wq.dtype is torch.float32 and wq.is_contiguous() and wq.numel() == n_heads * head_dim,
          "rope_projnorm_cache: the query norm's weight must be float32 [n_heads * head_dim]")
    _need(n_kv_heads == 0 or (wk is not None and wk.dtype is torch.float32 and wk.is_contiguous() and wk.numel() == n_kv_heads * head_dim),
          "rope_projnorm_cache: the key norm's weight must be float32 [n_kv_heads * head_dim]")
    do_rope = cos is not None
    if do_rope:
        _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
    do_write = pages is not None and n_kv_heads > 0
    if do_write:
        _need(pages.k.dtype is rows.dtype and pages.v.dtype is rows.dtype, "cache dtype differs from the activations'")
        _need(tuple(pages.k.shape[1:]) == (n_kv_heads, pages.page_size, head_dim) and pages.k.is_contiguous()
              and pages.v.is_contiguous() and pages.v.shape == pages.k.shape, "cache storage has the wrong shape")
        _int32(pages.tables, "page tables")
        _int32(seq_end, "seq_end")
    library.check(library.load().rdl_rope_projnorm_cache(
        _ptr(rows), rows.stride(0), _dtype_code(rows), T, n_heads, n_kv_heads, head_dim, rotary_dim if do_rope else 0,
        _ptr(cos), _ptr(sin), _ptr(tok_seq), _ptr(tok_pos), int(do_rope), _ptr(wq), _ptr(wk), float(eps), int(q_count), int(k_count),
        int(do_write), _ptr(pages.k) if do_write else None, _ptr(pages.v) if do_write else None,
        _ptr(pages.tables) if do_write else None, pages.tables.shape[1] if do_write else 0,
        pages.page_size if do_write else 0, pages.ring_pages if do_write else 0,
        _ptr(seq_end) if do_write else None, _stream(rows)))
    return rows


PREFILL_QUERY_TILE = 64    # query rows of a tile in the lists the prefill attention kernels take


class AttentionBatch(NamedTuple):
    """The step's sequences as the attention kernels see them (device int32 tensors)."""
    n_tokens: int
    n_seqs: int
    tok_seq: torch.Tensor      # [tokens]
    tok_pos: torch.Tensor      # [tokens], -1 marks a padding row
    seq_start: torch.Tensor    # [seqs + 1]
    seq_past: torch.Tensor     # [seqs]
    seq_cached: torch.Tensor   # [seqs] keys below this position are read from the cache
    tile_seq: Optional[torch.Tensor] = None   # prefill: query tiles of PREFILL_QUERY_TILE rows
    tile_q0: Optional[torch.Tensor] = None
    n_tiles: int = 0
    max_keys: int = 0          # decode: longest key run any token of the batch reads (window applied)


def _attention_args(q, q_stride, k_new, v_new, kv_stride, out, b: AttentionBatch, pages: Optional[KVPages],
                    n_heads, n_kv_heads, head_dim, score_scale, softcap, window):
    a = AttentionArgs()
    a.dtype = _dtype_code(out)
    a.n_tokens, a.n_seqs = b.n_tokens, b.n_seqs
    a.n_heads, a.n_kv_heads, a.head_dim = n_heads, n_kv_heads, head_dim
    a.score_scale = float(score_scale)
    a.softcap = float(softcap or 0.0)
    a.window = int(window or 0)
    a.q, a.q_stride = q, q_stride
    a.k_new, a.v_new, a.kv_stride = k_new, v_new, kv_stride
    a.out, a.out_stride = out.data_ptr(), out.stride(0)
    a.tok_seq, a.tok_pos = b.tok_seq.data_ptr(), b.tok_pos.data_ptr()
    a.seq_start, a.seq_past, a.seq_cached = b.seq_start.data_ptr(), b.seq_past.data_ptr(), b.seq_cached.data_ptr()
    if pages is not None:
        a.k_cache, a.v_cache = pages.k.data_ptr(), pages.v.data_ptr()
        a.tables, a.table_width = pages.tables.data_ptr(), pages.tables.shape[1]
        a.page_size, a.ring_pages = pages.page_size, pages.ring_pages
    return a


@functools.lru_cache(maxsize=None)
def sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def choose_keys_per_split(n_tokens: int, n_kv_heads: int, max_keys: int, page_size: int, sms: int = 148) -> int:
    """Keys per block of the decode kernel: runs of four pages (a block then streams its pages one after
    the other, and fewer partial results are merged), shorter ones while that leaves the GPU with
    fewer than about one and a half blocks per multiprocessor (`sms` of them)."""
    blocks = lambda pages: n_tokens * n_kv_heads * ((max_keys + pages * page_size - 1) // (pages * page_size))
    for pages in (4, 2):
        if 2 * blocks(pages) >= 3 * sms:
            return pages * page_size
    return page_size


def attention(q: torch.Tensor, b: AttentionBatch, pages: Optional[KVPages], *, n_heads: int, n_kv_heads: int,
              head_dim: int, score_scale: float, softcap: Optional[float], window: Optional[int],
              new_kv: Optional[Tuple[torch.Tensor, int, int]] = None, kind: str = "auto",
              scratch=None, keys_per_split: Optional[int] = None, status: Optional[torch.Tensor] = None,
              rotate_and_write: Optional[Tuple[Optional[torch.Tensor], Optional[torch.Tensor], int]] = None,
              sinks: Optional[torch.Tensor] = None, sigmoid_bias: Optional[torch.Tensor] = None):
    """Attention of the step's tokens over cache and new rows.

    q: [tokens, >= n_heads * head_dim] rows whose first n_heads * head_dim values are the (rotated)
    query heads; the row stride may be larger (packed q/k/v rows).
    new_kv: (rows, k_col, v_col) - this step's packed rows and the columns at which the rotated
    keys and the values start; needed when `b.seq_cached` says that new keys are not in the cache.
    kind: "plain" (float arithmetic, any dtype), "prefill" (bfloat16, mma.sync tensor cores, keys from
    cache and packed rows), "prefill_tc" (bfloat16, TMA + tcgen05, for sequences that start at position 0
    with head_dim a multiple of 64), "decode" (bfloat16, split keys; reads the cache only), or "auto".
    scratch: callable(nbytes) -> zero-initialised float32 tensor that only this kernel writes, for
    the decode kernel's counters and partial results.  status: int32 tensor that a kernel sets
    non-zero when it gives up on a bounded wait.
    rotate_and_write (kind "decode", one token per sequence, `b` describing all keys as cached):
    (cos, sin, rotary_dim) - q and new_kv are the rows as the projection left them; the kernel rotates
    the query and key heads by the float32 tables [positions, rotary_dim / 2] (None, None, 0: no
    rotation), writes the new key and value rows into the cache and attends over the cache including
    them.  The packed rows themselves stay as they are.
    sinks: float32 [n_heads] - a logit per head without key or value whose exponential joins the softmax's
    denominator once (neither scaled nor capped).
    sigmoid_bias: float32 [n_heads] - no softmax: the weight of a visible key is sigmoid(score + sigmoid_bias[h]) and the
    weights are not normalised over the keys.
    Returns [tokens, n_heads * head_dim] in the dtype of q."""
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= n_heads * head_dim, "attention: bad query rows")
    T = q.shape[0]
    _need(T >= b.n_tokens, "attention: fewer rows than tokens")
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    es = q.element_size()
    k_new = v_new = None
    kv_stride = 0
    if new_kv is not None:
        rows, k_col, v_col = new_kv
        _need(rows.dtype is q.dtype and rows.dim() == 2 and rows.stride(1) == 1 and
              rows.shape[1] >= max(k_col, v_col) + n_kv_heads * head_dim, "attention: bad new key/value rows")
        k_new, v_new, kv_stride = rows.data_ptr() + k_col * es, rows.data_ptr() + v_col * es, rows.stride(0)
    a = _attention_args(q.data_ptr(), q.stride(0), k_new, v_new, kv_stride, out, b, pages, n_heads, n_kv_heads,
                        head_dim, score_scale, softcap, window)
    if pages is not None:
        _need(pages.k.dtype is q.dtype, "attention: cache dtype differs from the activations'")
    if sinks is not None:
        _need(sinks.dtype is torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads and sinks.device == q.device,
              "attention: sinks must be float32 [n_heads]")
        a.sinks = sinks.data_ptr()
    if sigmoid_bias is not None:
        _need(sigmoid_bias.dtype is torch.float32 and sigmoid_bias.is_contiguous() and sigmoid_bias.numel() == n_heads
              and sigmoid_bias.device == q.device, "attention: sigmoid_bias must be float32 [n_heads]")
        _need(sinks is None, "attention: sigmoid weights have no denominator for sinks to join")
        a.sigmoid_bias = sigmoid_bias.data_ptr()
    fast_ok = q.dtype is torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
    if kind == "auto":
        kind = "prefill" if fast_ok and b.n_tiles > 0 else "plain"
    lib = library.load()
    if kind == "plain":
        library.check(lib.rdl_attention_plain(ctypes.byref(a), _stream(q)))
    elif kind in ("prefill", "prefill_tc"):
        _need(b.tile_seq is not None and b.tile_q0 is not None, "attention: prefill needs query tiles")
        a.tile_seq, a.tile_q0, a.n_tiles = b.tile_seq.data_ptr(), b.tile_q0.data_ptr(), b.n_tiles
        if kind == "prefill_tc":
            # sequences that start at position 0, packed q/k/v rows, head_dim a multiple of 64
            _need(new_kv is not None and new_kv[0] is q, "attention: the tcgen05 prefill kernel reads packed q/k/v rows")
            a.status = _status(status)
            library.check(lib.rdl_attention_prefill_tc(ctypes.byref(a), q.stride(0), _stream(q)))
        else:
            library.check(lib.rdl_attention_prefill(ctypes.byref(a), _stream(q)))
    elif kind == "decode":
        _need(pages is not None, "attention: decode reads the cache")
        ks = keys_per_split or choose_keys_per_split(b.n_tokens, n_kv_heads, b.max_keys, pages.page_size,
                                                     sm_count(q.device.index or 0))
        a.keys_per_split = ks
        # a run of max_keys positions can straddle one more split than its length suggests
        a.max_splits = (max(b.max_keys, 1) + ks - 1) // ks + 1
        need = lib.rdl_attention_decode_scratch_bytes(b.n_tokens, n_heads, n_kv_heads, head_dim, a.max_splits)
        # the counters at the start of the scratch must be zero before a launch; the kernel leaves them so
        buf = scratch(need) if scratch is not None else torch.zeros(-(-need // 4), dtype=torch.float32, device=q.device)
        _need(buf.dtype is torch.float32 and buf.numel() * 4 >= need, "attention: decode scratch too small")
        a.scratch, a.scratch_bytes = buf.data_ptr(), buf.numel() * 4
        a.counter_bytes = lib.rdl_attention_decode_counter_bytes(b.n_tokens, n_kv_heads)
        a.status = _status(status)
        if rotate_and_write is not None:
            cos, sin, rotary_dim = rotate_and_write
            _need(new_kv is not None, "attention: rotate_and_write needs the step's key and value rows")
            if rotary_dim:
                _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
                      and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
                a.rope_cos, a.rope_sin = cos.data_ptr(), sin.data_ptr()
            a.rotary_dim, a.new_rows = int(rotary_dim), 1
        library.check(lib.rdl_attention_decode(ctypes.byref(a), _stream(q)))
    else:
        raise KernelError(f"attention: unknown kind '{kind}'")
    return out


# ------------------------------------------------------------------------------------------
# random weights
# ------------------------------------------------------------------------------------------

def random_normal(shape, key: int, std: float, dtype: torch.dtype, device) -> torch.Tensor:
    """N(0, std) values of the tensor with 64-bit `key`, made on the device: element j depends only on
    (key, j) and equals, bit for bit in float32, what `weights.counter_random.normal` makes on the host."""
    out = torch.empty(shape, dtype=dtype, device=device)
    library.check(library.load().rdl_random_normal(_ptr(out), _dtype_code(out), out.numel(), int(key) & (2**64 - 1),
                                                   float(std), _stream(out)))
    return out


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------

def sample(logits: torch.Tensor, *, temperature: float, top_k: Optional[int] = None, top_p: Optional[float] = None,
           repetition_penalty: Optional[float] = None, seed: int = 0, row_stream: Optional[torch.Tensor] = None,
           row_step: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_start: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           host_out: Optional[torch.Tensor] = None):
    """One token per row of float32 logits [rows, vocab] -> int32 [rows].  host_out: pinned int32 host memory of
    at least `rows` values that the kernel writes the tokens to as well (readable once the kernel has ended)."""
    _need(logits.dtype is torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "sample takes contiguous float32 logits [rows, vocab]")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    prm = SamplingArgs(float(temperature), int(top_k or 0), float(top_p if top_p is not None else 1.0),
                       float(repetition_penalty if repetition_penalty is not None else 1.0), int(seed) & (2**64 - 1))
    work = None
    if temperature >= 1e-7:
        work = torch.empty_like(logits)
        if row_stream is not None:
            _need(row_stream.dtype is torch.int64 and row_stream.numel() >= rows, "row_stream must be int64 [rows]")
        if row_step is not None:
            _int32(row_step, "row_step", rows)
        if history is not None:
            _int32(history, "history")
            _int32(history_start, "history_start", rows + 1)
    if host_out is not None:
        _need(host_out.dtype is torch.int32 and host_out.is_pinned() and host_out.is_contiguous() and host_out.numel() >= rows,
              "sample: host_out must be pinned int32 host memory with a value per row")
    library.check(library.load().rdl_sample(_ptr(out), host_out.data_ptr() if host_out is not None else None, _ptr(logits), rows, vocab,
                                            ctypes.byref(prm), _ptr(row_stream),
                                            _ptr(row_step), _ptr(history), _ptr(history_start), _ptr(work), _stream(logits)))
    return out


def upload_batch(dst: torch.Tensor, src_pinned: torch.Tensor, n_ints: int, fed: Optional[Tuple[torch.Tensor, int, int, int]] = None):
    """A step's int32 batch description from pinned host memory to the device by a kernel (no copy engine between the
    kernels of two steps).  fed = (sampled ids on the device, where the description lists their rows, where its
    tokens lie, how many): those tokens are taken from `sampled` on the way."""
    _need(dst.dtype is torch.int32 and dst.is_cuda and src_pinned.dtype is torch.int32 and src_pinned.is_pinned()
          and dst.numel() >= n_ints and src_pinned.numel() >= n_ints, "upload_batch: int32 device buffer and pinned int32 host buffer")
    sampled, src_at, tok_at, n_fed = fed if fed is not None else (None, 0, 0, 0)
    if sampled is not None:
        _int32(sampled, "sampled")
    library.check(library.load().rdl_upload_batch(_ptr(dst), src_pinned.data_ptr(), n_ints, _ptr(sampled), src_at, tok_at, n_fed,
                                                  _stream(dst)))


# ------------------------------------------------------------------------------------------
# latent attention
# ------------------------------------------------------------------------------------------

def latent_prepare(rows: torch.Tensor, *, q_col: int, n_heads: int, dim: int, rot_dim: int, latent_col: Optional[int],
                   kv_rank: int, norm: Optional[NormParams], cos: torch.Tensor, sin: torch.Tensor, rot_n: int,
                   interleaved: bool, tok_seq: torch.Tensor, tok_pos: torch.Tensor, q_rot_out: Optional[torch.Tensor] = None,
                   q_rot_col: int = 0, q_rot_head: int = 0, pages: Optional[KVPages] = None,
                   seq_end: Optional[torch.Tensor] = None, write: bool = True) -> Optional[torch.Tensor]:
    """The latent-attention step between the input projection and attention, on the projection's packed rows
    [tokens, ...]: rotates the rotated part ([.., dim:dim + rot_dim] of each of the n_heads query heads from column
    q_col) by the position's angles, in place or into `q_rot_out[t, q_rot_col + h * q_rot_head ...]`; and, if the layer
    has a latent of its own (latent_col), norms its kv_rank values in float (norm: weight, eps; offset 0), rotates the
    rot_dim values after them and returns the rows [c | kr] ([tokens, kv_rank + rot_dim]), which it also writes into the
    cache (`pages.k`, rows of one head and that width) when `write`.  cos / sin: float32 [positions, rot_n / 2]."""
    _need(rows.dim() == 2 and rows.stride(1) == 1, "latent_prepare: packed rows [tokens, width]")
    T = rows.shape[0]
    a = library.LatentPrepareArgs()
    a.dtype, a.n_tokens = _dtype_code(rows), T
    a.rows, a.row_stride = rows.data_ptr(), rows.stride(0)
    a.q_col, a.n_heads, a.dim, a.rot_dim = q_col, n_heads, dim, rot_dim
    a.kv_rank = kv_rank
    _need(rot_n % 2 == 0 and 0 <= rot_n <= rot_dim, "latent_prepare: the rotated dimensions must be even and fit the rotated part")
    _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
          and cos.shape == sin.shape and cos.shape[1] * 2 == rot_n, "rotary tables must be float32 [positions, rot_n / 2]")
    a.cos_t, a.sin_t, a.rot_n, a.interleaved = cos.data_ptr(), sin.data_ptr(), rot_n, int(interleaved)
    _int32(tok_pos, "tok_pos", T)
    _int32(tok_seq, "tok_seq", T)
    a.tok_seq, a.tok_pos = tok_seq.data_ptr(), tok_pos.data_ptr()
    _need(rows.shape[1] >= q_col + n_heads * (dim + rot_dim), "latent_prepare: the rows are narrower than the query heads")
    if q_rot_out is not None:
        _need(q_rot_out.dtype is rows.dtype and q_rot_out.dim() == 2 and q_rot_out.stride(1) == 1 and q_rot_out.shape[0] >= T
              and q_rot_out.shape[1] >= q_rot_col + (n_heads - 1) * q_rot_head + rot_dim, "latent_prepare: bad q_rot_out")
        a.q_rot_out = q_rot_out.data_ptr() + q_rot_col * rows.element_size()
        a.q_rot_stride, a.q_rot_head = q_rot_out.stride(0), q_rot_head
    latent = None
    a.latent_col = -1
    if latent_col is not None:
        _need(rows.shape[1] >= latent_col + kv_rank + rot_dim, "latent_prepare: the rows are narrower than the latent")
        _need(norm is not None and norm.weight.is_contiguous() and norm.weight.numel() == kv_rank and norm.offset == 0.0,
              "latent_prepare: the latent's norm needs a plain weight of kv_rank values")
        a.latent_col = latent_col
        a.norm_w, a.norm_w_dtype, a.eps = norm.weight.data_ptr(), _dtype_code(norm.weight), float(norm.eps)
        latent = torch.empty((T, kv_rank + rot_dim), dtype=rows.dtype, device=rows.device)
        a.latent_out = latent.data_ptr()
        if write and pages is not None:
            _latent_cache_args(a, pages, seq_end, rows.dtype, kv_rank + rot_dim)
    library.check(library.load().rdl_latent_prepare(ctypes.byref(a), _stream(rows)))
    return latent


def _latent_cache_args(a, pages: KVPages, seq_end, dtype, width):
    _need(pages.k.dtype is dtype and pages.k.is_contiguous() and tuple(pages.k.shape[1:]) == (1, pages.page_size, width),
          "latent cache storage must be [pages, 1, page_size, kv_rank + rot_dim] in the activations' dtype")
    _int32(pages.tables, "page tables")
    _int32(seq_end, "seq_end")
    a.do_write = 1
    a.cache, a.tables, a.table_width = pages.k.data_ptr(), pages.tables.data_ptr(), pages.tables.shape[1]
    a.page_size, a.ring_pages, a.seq_end = pages.page_size, pages.ring_pages, seq_end.data_ptr()


def latent_write(latent: torch.Tensor, kv_rank: int, pages: KVPages, *, tok_seq, tok_pos, seq_end):
    """The rows [c | kr] of a step into the cache, as a call of its own."""
    _dense(latent, "latent rows")
    a = library.LatentPrepareArgs()
    a.dtype, a.n_tokens = _dtype_code(latent), latent.shape[0]
    a.kv_rank, a.rot_dim = kv_rank, latent.shape[1] - kv_rank
    a.latent_out = latent.data_ptr()
    _int32(tok_pos, "tok_pos", latent.shape[0])
    _int32(tok_seq, "tok_seq", latent.shape[0])
    a.tok_seq, a.tok_pos = tok_seq.data_ptr(), tok_pos.data_ptr()
    _latent_cache_args(a, pages, seq_end, latent.dtype, latent.shape[1])
    library.check(library.load().rdl_latent_write(ctypes.byref(a), _stream(latent)))


def latent_assemble(rows: torch.Tensor, q_col: int, kv: torch.Tensor, latent: torch.Tensor, *, n_heads: int, dim: int,
                    rot_dim: int, vdim: int, kv_rank: int, pad: int) -> torch.Tensor:
    """Packed rows [Q | K | V], [tokens, 3 * n_heads * pad], heads zero-padded to `pad` values: Q[h] = the projection's
    query head (its rotated part already rotated), K[h] = [k_un[h] | kr], V[h] = v[h]; kv = c [W_uk; W_uv]^T."""
    _need(rows.dim() == 2 and rows.stride(1) == 1, "latent_assemble: packed rows")
    _dense(kv, "kv"); _dense(latent, "latent rows")
    T = rows.shape[0]
    _need(kv.dtype is rows.dtype and latent.dtype is rows.dtype and tuple(kv.shape) == (T, n_heads * (dim + vdim))
          and tuple(latent.shape) == (T, kv_rank + rot_dim), "latent_assemble: shapes do not fit")
    out = torch.empty((T, 3 * n_heads * pad), dtype=rows.dtype, device=rows.device)
    library.check(library.load().rdl_latent_assemble(_ptr(out), _dtype_code(out), _ptr(rows), rows.stride(0), q_col, _ptr(kv), _ptr(latent),
                                                     T, n_heads, dim, rot_dim, vdim, kv_rank, pad, _stream(rows)))
    return out


def gate_heads(x: torch.Tensor, head_stride: int, gate: torch.Tensor, n_heads: int, vdim: int,
               row_stride: Optional[int] = None, n_rows: Optional[int] = None, per_value: bool = False) -> torch.Tensor:
    """[tokens, n_heads * vdim] = x[t * row_stride + h * head_stride + i] * sigmoid(gate[t, h]) for i < vdim; `gate` may be
    a column slice of wider rows.  per_value: a gate for every value, sigmoid(gate[t, h * vdim + i]).  By default x is
    [tokens, ...] and row_stride its row stride; with row_stride and n_rows
    given x is any dense tensor addressed by the two strides (head-major results of a batched product, say)."""
    _need(gate.dim() == 2 and gate.stride(1) == 1 and gate.dtype is x.dtype and gate.shape[1] >= n_heads * (vdim if per_value else 1),
          "gate_heads: bad gate")
    if row_stride is None:
        _need(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= (n_heads - 1) * head_stride + vdim, "gate_heads: shapes do not fit")
        T, row_stride = x.shape[0], x.stride(0)
    else:
        _need(x.is_contiguous() and n_rows is not None and x.numel() >= (n_rows - 1) * row_stride + (n_heads - 1) * head_stride + vdim,
              "gate_heads: the strides reach beyond the tensor")
        T = n_rows
    out = torch.empty((T, n_heads * vdim), dtype=x.dtype, device=x.device)
    library.check(library.load().rdl_gate_heads(_ptr(out), _dtype_code(out), _ptr(x), row_stride, head_stride, _ptr(gate), gate.stride(0),
                                                T, n_heads, vdim, int(bool(per_value)), _stream(x)))
    return out


def heads_linear(x: torch.Tensor, x_col: int, x_head: int, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_col: int = 0,
                 out_head: Optional[int] = None, gate: Optional[torch.Tensor] = None, gate_per_value: bool = False) -> torch.Tensor:
    """A product per head: out[t, out_col + h * out_head + j] = sum_k w[h, j, k] * x[t, x_col + h * x_head + k], optionally
    times sigmoid(gate[t, h]) (gate_per_value: of gate[t, h * n_out + j]).  w: [heads, n_out, k].  Without `out` the
    result is dense [tokens, heads * n_out]."""
    _need(x.dim() == 2 and x.stride(1) == 1 and w.dim() == 3 and w.is_contiguous() and w.dtype is x.dtype, "heads_linear: bad operands")
    H, n_out, k = w.shape
    T = x.shape[0]
    _need(x.shape[1] >= x_col + (H - 1) * x_head + k, "heads_linear: the rows are narrower than the heads")
    if out is None:
        out = torch.empty((T, H * n_out), dtype=x.dtype, device=x.device)
        out_head = n_out
    _need(out.dtype is x.dtype and out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= T
          and out.shape[1] >= out_col + (H - 1) * out_head + n_out, "heads_linear: bad output rows")
    a = library.HeadsLinearArgs()
    a.dtype, a.n_tokens, a.n_heads, a.n_out, a.k = _dtype_code(x), T, H, n_out, k
    es = x.element_size()
    a.x, a.x_stride, a.x_head = x.data_ptr() + x_col * es, x.stride(0), x_head
    a.w = w.data_ptr()
    a.out, a.out_stride, a.out_head = out.data_ptr() + out_col * es, out.stride(0), out_head
    if gate is not None:
        _need(gate.dtype is x.dtype and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape[1] >= H * (n_out if gate_per_value else 1),
              "heads_linear: bad gate")
        a.gate, a.gate_stride, a.gate_elem = gate.data_ptr(), gate.stride(0), int(bool(gate_per_value))
    library.check(library.load().rdl_heads_linear(ctypes.byref(a), _stream(x)))
    return out


def latent_decode_ok(dtype, width: int, kv_rank: int, page_size: int) -> bool:
    """Whether the tensor-core decode kernel of the absorbed form takes these sizes."""
    return (dtype is torch.bfloat16 and width % 16 == 0 and width <= 640 and kv_rank % 16 == 0 and 0 < kv_rank <= min(512, width)
            and page_size % 8 == 0)


def latent_decode(q: torch.Tensor, b: AttentionBatch, pages: KVPages, *, n_heads: int, kv_rank: int, score_scale: float,
                  window: Optional[int], scratch=None, n_splits: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-token attention of the absorbed form: q [tokens, n_heads * width] (width = kv_rank + rot_dim) over the
    cached rows `pages.k` [pages, 1, page_size, width], which are keys and, in their first kv_rank values, values.
    Returns [tokens, n_heads * width] whose first kv_rank values per head hold the result (the rest is not written).
    scratch: callable(nbytes) -> float32 tensor for the partial results when a token's keys are shared between blocks.
    sinks: float32 [n_heads] - a logit per head without key or value whose exponential joins the denominator once."""
    _dense(q, "q")
    if sinks is not None:
        _need(sinks.dtype is torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads and sinks.device == q.device,
              "latent_decode: sinks must be float32 [n_heads]")
    T = q.shape[0]
    width = pages.k.shape[3]
    _need(q.dtype is torch.bfloat16 and pages.k.dtype is torch.bfloat16 and q.shape[1] == n_heads * width
          and tuple(pages.k.shape[1:3]) == (1, pages.page_size) and pages.k.is_contiguous(), "latent_decode: shapes do not fit")
    out = torch.empty_like(q)
    groups = (n_heads + 15) // 16
    tiles = (max(b.max_keys, 1) + 63) // 64 + 1
    # one wave of two blocks a multiprocessor (two blocks of the widest rows fit its shared memory), a block per 64 keys at most
    splits = max(1, min(tiles, 64, (2 * sm_count(q.device.index or 0)) // max(1, b.n_tokens * groups)))
    splits = min(splits, max(1, (tiles + 1) // 2))      # two tiles a block at least: the merge costs as much as a tile
    if n_splits is not None:
        splits = max(1, min(tiles, 64, n_splits))
    lib = library.load()
    need = lib.rdl_latent_decode_scratch_bytes(b.n_tokens, n_heads, kv_rank, splits)
    buf = None
    if need:
        buf = scratch(need) if scratch is not None else torch.empty(-(-need // 4), dtype=torch.float32, device=q.device)
    library.check(lib.rdl_latent_decode(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(pages.k), _ptr(pages.tables), pages.tables.shape[1],
                                        pages.page_size, pages.ring_pages, _ptr(b.tok_seq), _ptr(b.tok_pos), b.n_tokens, n_heads, width,
                                        kv_rank, float(score_scale), int(window or 0), max(b.max_keys, 1), splits, _ptr(buf),
                                        buf.numel() * 4 if buf is not None else 0, _ptr(sinks), _stream(q)), 2 if splits > 1 else 1)
    return out


# ------------------------------------------------------------------------------------------
# routed feed-forward
# ------------------------------------------------------------------------------------------

# gated forms with a parameter (`csrc/activations.cuh`): name -> code
GATED_FORMS = dict(ACTIVATIONS, swish_limit=2)
# element-wise activations of a product that is not gated (`csrc/api.h`, RDL_UNARY_*): experts of two matrices,
# y = W_down act(W_up x), take these as their `form`
UNARY_FORMS = {"relu2": 16, "silu_plain": 17}
EXPERT_FORMS = dict(GATED_FORMS, **UNARY_FORMS)


ROUTE_SCORING = {"softmax": 0, "sigmoid": 1, "softmax_chosen": 2}     # `csrc/api.h`, RDL_ROUTE_*


def moe_route(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], top: int, scoring: str = "softmax",
              bias: Optional[torch.Tensor] = None):
    """Per row: scores of all experts from the float32 logits W_r x + bias (softmax over the experts, or sigmoid expert by
    expert); the `top` experts with the largest score + correction (int32 [rows, top]) and their scores without it
    (float32 [rows, top]).  scoring "softmax_chosen": the choice is by the logits themselves and the weights are the
    softmax over the chosen logits only."""
    _need(scoring in ROUTE_SCORING, f"moe_route: unknown scoring '{scoring}', known: {sorted(ROUTE_SCORING)}")
    _dense(x, "x")
    _need(w_router.dtype is torch.float32 and w_router.is_contiguous() and w_router.shape[1] == x.shape[1], "moe_route: float32 router [experts, width]")
    E = w_router.shape[0]
    if correction is not None:
        _need(correction.dtype is torch.float32 and correction.is_contiguous() and correction.numel() == E, "moe_route: float32 correction [experts]")
    if bias is not None:
        _need(bias.dtype is torch.float32 and bias.is_contiguous() and bias.numel() == E, "moe_route: float32 bias [experts]")
    sel = torch.empty((x.shape[0], top), dtype=torch.int32, device=x.device)
    sel_w = torch.empty((x.shape[0], top), dtype=torch.float32, device=x.device)
    logits = torch.empty((x.shape[0], E), dtype=torch.float32, device=x.device)
    library.check(library.load().rdl_moe_route(_ptr(x), _dtype_code(x), _ptr(w_router), _ptr(bias), _ptr(correction), x.shape[0], E, x.shape[1], top,
                                               ROUTE_SCORING[scoring], _ptr(sel), _ptr(sel_w), _ptr(logits), _stream(x)), 2)
    return sel, sel_w


MOE_PAIR_ROWS = 4096     # rows of one launch of the per-pair expert kernels (their grids hold rows x top <= 65,535)


def moe_experts_few(x: torch.Tensor, sel: torch.Tensor, sel_w: torch.Tensor, w_gate_up: Optional[torch.Tensor],
                    w_down: Optional[torch.Tensor], n_real: int, form: str, param: float,
                    weights_on_input: bool = False) -> torch.Tensor:
    """The routed experts with every (row, choice) pair streaming its expert's matrices: out[t] = sum_k sel_w[t, k] y_k,
    y_k = W_down[e] gated(W_gate[e] x_t, W_up[e] x_t) for e = sel[t, k] < n_real, else x_t (an identity expert).
    w_gate_up: [n_real, 2 ff, width] (an expert's gate rows, then its up rows); w_down: [n_real, width, ff].
    form in UNARY_FORMS: experts of two matrices, y_k = W_down[e] act(W_up[e] x_t), with w_gate_up [n_real, ff, width].
    weights_on_input: y_k = expert(sel_w[t, k] x_t) and out[t] = sum_k y_k."""
    _dense(x, "x")
    T, width = x.shape
    top = sel.shape[1]
    _need(form in EXPERT_FORMS, f"unknown expert form '{form}', known: {sorted(EXPERT_FORMS)}")
    per = 1 if form in UNARY_FORMS else 2
    ff = 0
    if n_real:
        _need(w_gate_up.dtype is x.dtype and w_down.dtype is x.dtype and w_gate_up.is_contiguous() and w_down.is_contiguous()
              and w_gate_up.dim() == 3 and w_gate_up.shape[0] == n_real and w_gate_up.shape[2] == width and w_gate_up.shape[1] % per == 0
              and tuple(w_down.shape) == (n_real, width, w_gate_up.shape[1] // per), "moe_experts_few: expert matrices do not fit")
        ff = w_gate_up.shape[1] // per
    out = torch.empty_like(x)
    lib = library.load()
    step = max(1, min(MOE_PAIR_ROWS, 65535 // top))
    for r0 in range(0, T, step):
        n = min(step, T - r0)
        xs, ss, sw, os_ = x[r0:r0 + n], sel[r0:r0 + n], sel_w[r0:r0 + n], out[r0:r0 + n]
        mid = None
        if n_real:
            mid = torch.empty((n * top, ff), dtype=x.dtype, device=x.device)
            library.check(lib.rdl_moe_gate_up(_ptr(mid), _dtype_code(x), _ptr(xs), _ptr(w_gate_up), _ptr(ss),
                                              _ptr(sw) if weights_on_input else None, n, top, n_real, ff, width,
                                              EXPERT_FORMS[form], float(param), _stream(x)))
        library.check(lib.rdl_moe_down_combine(_ptr(os_), _dtype_code(x), _ptr(mid), _ptr(xs), _ptr(w_down), _ptr(ss),
                                               None if weights_on_input else _ptr(sw), n, top,
                                               n_real, max(ff, 1), width, _stream(x)))
    return out


MOE_TILE = 128               # rows of a tile of the grouped product: one expert per tile
MOE_GROUPED_MIN_PAIRS = 128  # from this many (row, choice) pairs on the rows are sorted by expert


def moe_experts_grouped(x, sel, sel_w, w_gate_up, w_down, n_real: int, form: str, param: float,
                        status: Optional[torch.Tensor] = None, weights_on_input: bool = False) -> torch.Tensor:
    """The routed experts for many rows in bfloat16: pairs sorted by expert into tiles of 128 rows, both products on the
    tcgen05 kernel with one expert per row tile, then the weighted sum per row.  No step of it needs the host to
    know the counts: the buffers are sized for the worst case and tiles no expert uses are skipped."""
    T, width = x.shape
    top = sel.shape[1]
    unary = form in UNARY_FORMS
    ff = w_gate_up.shape[1] // (1 if unary else 2)
    pairs = T * top
    max_tiles = (pairs + n_real * (MOE_TILE - 1) + MOE_TILE - 1) // MOE_TILE
    dev = x.device
    pair_slot = torch.empty(pairs, dtype=torch.int32, device=dev)
    slot_pair = torch.empty(max_tiles * MOE_TILE, dtype=torch.int32, device=dev)
    tile_group = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    lib = library.load()
    st = _stream(x)
    library.check(lib.rdl_moe_align(_ptr(sel), pairs, n_real, max_tiles, _ptr(pair_slot), _ptr(slot_pair), _ptr(tile_group), st))
    xs = torch.empty((max_tiles * MOE_TILE, width), dtype=x.dtype, device=dev)
    library.check(lib.rdl_moe_gather(_ptr(xs), _ptr(x), _ptr(slot_pair), _ptr(tile_group), _ptr(sel_w) if weights_on_input else None,
                                     max_tiles, top, width, st))
    mid = torch.empty((max_tiles * MOE_TILE, ff), dtype=x.dtype, device=dev)
    library.check(lib.rdl_gemm_tc_grouped(_ptr(mid), _dtype_code(mid), _ptr(xs), _ptr(w_gate_up), max_tiles * MOE_TILE, ff, width, n_real,
                                          _ptr(tile_group), 0 if unary else 1, EXPERT_FORMS[form], float(param), _status(status), st))
    y = torch.empty((max_tiles * MOE_TILE, width), dtype=x.dtype, device=dev)
    library.check(lib.rdl_gemm_tc_grouped(_ptr(y), _dtype_code(y), _ptr(mid), _ptr(w_down), max_tiles * MOE_TILE, width, ff, n_real,
                                          _ptr(tile_group), 0, 0, 0.0, _status(status), st))
    out = torch.empty_like(x)
    library.check(lib.rdl_moe_combine(_ptr(out), _ptr(y), _ptr(x), _ptr(pair_slot), None if weights_on_input else _ptr(sel_w), T, top,
                                      width, st))
    return out


def moe_experts(x, sel, sel_w, w_gate_up, w_down, n_real: int, form: str, param: float, weights_on_input: bool = False) -> torch.Tensor:
    """The routed experts' weighted sum for every row (see `moe_experts_few` for the meaning of the arguments): with
    few pairs each streams its expert's matrices; with many, in bfloat16, the rows are sorted by expert and multiplied
    tile by tile (`moe_experts_grouped`)."""
    T, width = x.shape
    if (n_real and x.dtype is torch.bfloat16 and T * sel.shape[1] >= MOE_GROUPED_MIN_PAIRS and width % 8 == 0
            and (w_gate_up.shape[1] // (1 if form in UNARY_FORMS else 2)) % 8 == 0 and w_gate_up.shape[1] % 16 == 0
            and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return moe_experts_grouped(x, sel, sel_w, w_gate_up, w_down, n_real, form, param, weights_on_input=weights_on_input)
    return moe_experts_few(x, sel, sel_w, w_gate_up, w_down, n_real, form, param, weights_on_input)


# ------------------------------------------------------------------------------------------
# linear attention with a fixed decay per head
# ------------------------------------------------------------------------------------------

DECAY_CHUNKED_MIN_TOKENS = 64    # from this many rows on a bfloat16 step takes the chunked tensor-core kernel
DECAY_CHUNKED_MIN_PER_SEQUENCE = 8    # ... and this many rows a sequence on average
DECAY_CHUNKED = os.environ.get("RDL_DECAY_ATTENTION", "chunked") != "scan"     # "scan": token by token everywhere, for comparison


def decay_attention_chunked_ok(dtype, dim: int, vdim: int) -> bool:
    """Whether the chunked kernel takes these head sizes."""
    return dtype is torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128


def decay_attention(rows: torch.Tensor, *, q_col: int, k_col: int, v_col: int, n_heads: int, dim: int, vdim: int,
                    decay: torch.Tensor, state: torch.Tensor, tok_pos: torch.Tensor, seq_start: torch.Tensor,
                    slots: torch.Tensor, n_seqs: int, silu: bool = False, k_scale: float = 1.0,
                    cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rot_n: int = 0,
                    kind: str = "auto") -> torch.Tensor:
    """Per sequence and head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over the step's packed rows, from and
    into `state` (float32 [slots, n_heads, dim, vdim], the row of a sequence given by `slots`).  q, k and v are read
    from `rows` at the given columns (heads one after another); on the way into the recurrence q and k are rotated
    (the first rot_n values, half-split pairs, float32 tables [positions, rot_n / 2]), q, k and v go through SiLU
    (silu) and k is multiplied by k_scale, all in float.  Returns float32 [tokens, n_heads * vdim].
    kind: "scan" (token by token, float), "chunked" (bfloat16 rows, tensor cores), "auto"."""
    _need(rows.dim() == 2 and rows.stride(1) == 1, "decay_attention: packed rows")
    T = rows.shape[0]
    _need(rows.shape[1] >= max(q_col + n_heads * dim, k_col + n_heads * dim, v_col + n_heads * vdim),
          "decay_attention: the rows are narrower than the heads")
    _need(decay.dtype is torch.float32 and decay.is_contiguous() and decay.numel() == n_heads, "decay_attention: float32 decay [heads]")
    _need(state.dtype is torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (n_heads, dim, vdim),
          "decay_attention: the state must be float32 [slots, heads, dim, vdim]")
    _int32(tok_pos, "tok_pos", T)
    _int32(seq_start, "seq_start", n_seqs + 1)
    _int32(slots, "slots", n_seqs)
    if rot_n:
        _need(cos is not None and cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous()
              and sin.is_contiguous() and cos.shape == sin.shape and cos.shape[1] * 2 == rot_n,
              "rotary tables must be float32 [positions, rot_n / 2]")
    out = torch.empty((T, n_heads * vdim), dtype=torch.float32, device=rows.device)
    a = library.DecayAttentionArgs()
    a.dtype, a.n_tokens, a.n_seqs, a.n_heads, a.dim, a.vdim = _dtype_code(rows), T, n_seqs, n_heads, dim, vdim
    a.rows, a.row_stride = rows.data_ptr(), rows.stride(0)
    a.q_col, a.k_col, a.v_col = q_col, k_col, v_col
    a.silu, a.k_scale = int(silu), float(k_scale)
    if rot_n:
        a.cos_t, a.sin_t, a.rot_n = cos.data_ptr(), sin.data_ptr(), rot_n
    a.decay, a.tok_pos, a.seq_start, a.slots = decay.data_ptr(), tok_pos.data_ptr(), seq_start.data_ptr(), slots.data_ptr()
    a.state, a.out = state.data_ptr(), out.data_ptr()
    if kind == "auto":
        # chunks pay when sequences bring many tokens each; a step of single tokens (any batch) reads and writes each state once
        many = T >= DECAY_CHUNKED_MIN_TOKENS and T >= DECAY_CHUNKED_MIN_PER_SEQUENCE * n_seqs
        kind = "chunked" if (DECAY_CHUNKED and many and decay_attention_chunked_ok(rows.dtype, dim, vdim)) else "scan"
    lib = library.load()
    if kind == "scan":
        library.check(lib.rdl_decay_attention_scan(ctypes.byref(a), _stream(rows)))
    elif kind == "chunked":
        _need(decay_attention_chunked_ok(rows.dtype, dim, vdim), "decay_attention: the chunked kernel takes bfloat16 heads of 16..128 values in steps of 16")
        chunks = lib.rdl_decay_attention_chunks(T, n_seqs)
        work = torch.empty((chunks, n_heads, dim, vdim), dtype=torch.float32, device=rows.device)     # a state per chunk and head
        library.check(lib.rdl_decay_attention_chunked(ctypes.byref(a), _ptr(work), work.numel() * 4, _stream(rows)), 3)
    else:
        raise KernelError(f"decay_attention: unknown kind '{kind}'")
    return out


# ------------------------------------------------------------------------------------------
# rows that look back along their sequence, and recurrences whose decay depends on the token
# ------------------------------------------------------------------------------------------

def norm_shift(x: torch.Tensor, weight: torch.Tensor, eps: float, shift: torch.Tensor, state: torch.Tensor, *, tok_seq, tok_pos,
               seq_start, slots, out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """n_t = x_t / sqrt(mean(x_t^2) + eps) * weight and m_t = n_t + (n_(t-1) - n_t) * shift along each sequence, in float;
    the row before a sequence's first row of the step comes from `state` (float32 [slots, width]; zeros at position 0),
    which is left holding the sequence's last n.  x: float32 [rows, width].  Returns (n, m) in out_dtype."""
    _need(x.dtype is torch.float32 and x.dim() == 2 and x.is_contiguous(), "norm_shift: contiguous float32 rows")
    T, width = x.shape
    _need(weight.is_contiguous() and weight.numel() == width and shift.is_contiguous() and shift.numel() == width,
          f"norm_shift: the weight and the shift must hold {width} values")
    _need(state.dtype is torch.float32 and state.is_contiguous() and state.dim() == 2 and state.shape[1] == width,
          "norm_shift: the state must be float32 [slots, width]")
    _int32(tok_seq, "tok_seq", T); _int32(tok_pos, "tok_pos", T); _int32(seq_start, "seq_start"); _int32(slots, "slots")
    normed = torch.empty((T, width), dtype=out_dtype, device=x.device)
    mixed = torch.empty((T, width), dtype=out_dtype, device=x.device)
    library.check(library.load().rdl_norm_shift(_ptr(x), _ptr(weight), _dtype_code(weight), float(eps), _ptr(shift), _dtype_code(shift),
                                                _ptr(state), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_start), _ptr(slots), _ptr(normed),
                                                _ptr(mixed), _dtype_code(normed), T, width, _stream(x)))
    return normed, mixed


SHORT_CONV_MAX_TAPS = 8


def short_conv(rows: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], *, tok_seq,
               tok_pos, seq_start, slots, silu: bool = True) -> torch.Tensor:
    """Causal convolution over time per channel along each sequence, then SiLU if asked:
    out[t, c] = act(bias[c] + sum_j weight[c, j] rows[t - (taps - 1 - j), c]), inputs before a sequence's start being zero and
    inputs of earlier steps coming from `state` (float32 [slots, taps - 1, channels]), which is left holding the sequence's
    last taps - 1 inputs.  rows may be a column slice of wider rows.  Returns dense [rows, channels] in the rows' dtype."""
    _need(rows.dim() == 2 and rows.stride(1) == 1, "short_conv: rows (or a column slice of rows)")
    T, C = rows.shape
    _need(weight.dim() == 2 and weight.shape[0] == C and weight.is_contiguous(), f"short_conv: the weight must be [{C}, taps]")
    taps = weight.shape[1]
    _need(1 <= taps <= SHORT_CONV_MAX_TAPS, f"short_conv: {taps} taps, the kernel takes 1 to {SHORT_CONV_MAX_TAPS}")
    if bias is not None:
        _need(bias.is_contiguous() and bias.numel() == C and bias.dtype is weight.dtype, "short_conv: the bias must match the weight")
    if taps > 1:
        _need(state is not None and state.dtype is torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, C),
              "short_conv: the state must be float32 [slots, taps - 1, channels]")
    _int32(tok_seq, "tok_seq", T); _int32(tok_pos, "tok_pos", T); _int32(seq_start, "seq_start"); _int32(slots, "slots")
    out = torch.empty((T, C), dtype=rows.dtype, device=rows.device)
    library.check(library.load().rdl_short_conv(_ptr(rows), rows.stride(0), _dtype_code(rows), C, taps, _ptr(weight), _dtype_code(weight),
                                                _ptr(bias), int(bool(silu)), _ptr(state) if taps > 1 else None, _ptr(tok_seq),
                                                _ptr(tok_pos), _ptr(seq_start), _ptr(slots), _ptr(out), T, _stream(rows)))
    return out


def gated_residual_add_(residual: torch.Tensor, gates: torch.Tensor, bias_a: torch.Tensor, a: torch.Tensor,
                        bias_b: Optional[torch.Tensor] = None, b1: Optional[torch.Tensor] = None,
                        b2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual[t, i] += sigmoid(gates[t, i] + bias_a[i]) a[t, i] + sigmoid(gates[t, width + i] + bias_b[i]) (b1[t, i] + b2[t, i]),
    in float, in place (residual float32).  Without b1 the first term only; b2 is optional.  gates may be a column slice."""
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and residual.dim() == 2, "gated_residual_add_: float32 stream")
    T, width = residual.shape
    _need(gates.dim() == 2 and gates.stride(1) == 1 and gates.shape[0] == T and gates.shape[1] >= (2 if b1 is not None else 1) * width,
          "gated_residual_add_: the gates' rows are narrower than the branches")
    for t in (a, b1, b2):
        if t is not None:
            _need(tuple(t.shape) == (T, width) and t.is_contiguous() and t.dtype is gates.dtype, "gated_residual_add_: branches like the stream")
    _need(bias_a.numel() == width and bias_a.is_contiguous(), "gated_residual_add_: a bias per column")
    if b1 is not None:
        _need(bias_b is not None and bias_b.numel() == width and bias_b.dtype is bias_a.dtype and bias_b.is_contiguous(),
              "gated_residual_add_: a bias per column for the second branch")
    _need(b2 is None or b1 is not None, "gated_residual_add_: b2 comes with b1")
    library.check(library.load().rdl_gated_residual_add(_ptr(residual), _ptr(gates), gates.stride(0), _ptr(bias_a), _ptr(bias_b),
                                                        _dtype_code(bias_a), _ptr(a), _ptr(b1), _ptr(b2), _dtype_code(gates), T, width,
                                                        _stream(residual)))
    return residual


def _recurrence_common(a, rows, state, n_heads, n_key_heads, dim, vdim, tok_pos, seq_start, slots, n_seqs):
    T = rows.shape[0]
    _need(rows.dim() == 2 and rows.stride(1) == 1, "recurrence: packed rows")
    _need(n_heads % n_key_heads == 0, f"recurrence: {n_heads} heads cannot share {n_key_heads} key heads")
    _need(state.dtype is torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (n_heads, dim, vdim),
          "recurrence: the state must be float32 [slots, heads, dim, vdim]")
    _int32(tok_pos, "tok_pos", T); _int32(seq_start, "seq_start", n_seqs + 1); _int32(slots, "slots", n_seqs)
    a.dtype, a.n_tokens, a.n_seqs, a.n_heads, a.n_key_heads, a.dim, a.vdim = _dtype_code(rows), T, n_seqs, n_heads, n_key_heads, dim, vdim
    a.rows, a.row_stride = rows.data_ptr(), rows.stride(0)
    a.tok_pos, a.seq_start, a.slots, a.state = tok_pos.data_ptr(), seq_start.data_ptr(), slots.data_ptr(), state.data_ptr()
    # rows of padding sequences are not written by the kernel: they start as zeros, so that what follows sees finite numbers
    out = torch.zeros((T, n_heads * vdim), dtype=torch.float32, device=rows.device)
    a.out = out.data_ptr()
    return out


def _f32_vec(t, n, name):
    _need(t is not None and t.dtype is torch.float32 and t.is_contiguous() and t.numel() == n, f"recurrence: {name} must be float32 [{n}]")
    return t.data_ptr()


def state_space_chunked_ok(rows: torch.Tensor, x_col: int, b_col: int, c_col: int, state_dim: int, vdim: int) -> bool:
    """Whether the chunked kernels take these rows and sizes."""
    return (rows.dtype is torch.bfloat16 and state_dim % 16 == 0 and 16 <= state_dim <= 128 and vdim % 16 == 0 and vdim >= 16
            and rows.data_ptr() % 16 == 0 and rows.stride(0) % 8 == 0 and x_col % 8 == 0 and b_col % 8 == 0 and c_col % 8 == 0)


def state_space_scan(rows: torch.Tensor, dt_rows: torch.Tensor, *, x_col: int, b_col: int, c_col: int, n_heads: int, n_groups: int,
                     state_dim: int, vdim: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: Optional[torch.Tensor],
                     state: torch.Tensor, tok_pos, seq_start, slots, n_seqs: int, kind: str = "auto") -> torch.Tensor:
    """A selective state space in float: per head h of group g,
    dt_t = softplus(dt_rows[t, h] + dt_bias[h]);  S_t = exp(-exp(a_log[h]) dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + d_skip[h] x_t,
    with x [vdim] of head h from column x_col, B and C [state_dim] of group g from b_col and c_col of `rows`, S float32
    [slots, heads, state_dim, vdim] read from and left in `state`.  Returns float32 [tokens, heads * vdim].
    kind: "scan" (token by token), "chunked" (bfloat16 rows, chunks of 64 tokens on tensor cores, three launches), "auto"
    (chunks where sequences bring many tokens each)."""
    a = library.RecurrenceArgs()
    out = _recurrence_common(a, rows, state, n_heads, n_groups, state_dim, vdim, tok_pos, seq_start, slots, n_seqs)
    T = rows.shape[0]
    _need(rows.shape[1] >= max(x_col + n_heads * vdim, b_col + n_groups * state_dim, c_col + n_groups * state_dim),
          "state_space_scan: the rows are narrower than the heads")
    _need(dt_rows.dim() == 2 and dt_rows.stride(1) == 1 and tuple(dt_rows.shape) == (T, n_heads) and dt_rows.dtype is rows.dtype,
          "state_space_scan: step sizes [tokens, heads] in the rows' dtype")
    a.mode, a.q_col, a.k_col, a.v_col = library.REC_SSM, c_col, b_col, x_col
    a.dt_rows, a.dt_stride = dt_rows.data_ptr(), dt_rows.stride(0)
    a.dt_bias, a.a_log = _f32_vec(dt_bias, n_heads, "dt_bias"), _f32_vec(a_log, n_heads, "a_log")
    a.d_skip = _f32_vec(d_skip, n_heads, "d_skip") if d_skip is not None else None
    if kind == "auto":
        many = T >= DECAY_CHUNKED_MIN_TOKENS and T >= DECAY_CHUNKED_MIN_PER_SEQUENCE * n_seqs
        kind = "chunked" if (DECAY_CHUNKED and many and state_space_chunked_ok(rows, x_col, b_col, c_col, state_dim, vdim)) else "scan"
    lib = library.load()
    if kind == "scan":
        library.check(lib.rdl_recurrence_scan(ctypes.byref(a), _stream(rows)))
    elif kind == "chunked":
        _need(state_space_chunked_ok(rows, x_col, b_col, c_col, state_dim, vdim),
              "state_space_scan: the chunked kernels take bfloat16 rows, sizes in steps of 16 (state up to 128) and columns on 16-byte boundaries")
        nbytes = lib.rdl_state_space_chunked_work_bytes(T, n_seqs, n_heads, state_dim, vdim)
        work = torch.empty((nbytes // 4,), dtype=torch.float32, device=rows.device)
        library.check(lib.rdl_state_space_chunked(ctypes.byref(a), _ptr(work), nbytes, _stream(rows)), 3)
    else:
        raise KernelError(f"state_space_scan: unknown kind '{kind}'")
    return out


DELTA_CHUNKED_MAX_DIM = 128


def delta_prepare(rows: torch.Tensor, *, q_col: int, k_col: int, n_heads: int, n_key_heads: int, dim: int, decay_rows: torch.Tensor,
                  beta_rows: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, q_scale: float, unit_eps: float):
    """What enters a delta-rule recurrence, in float32: q and k of every key head as unit vectors, v / sqrt(sum(v^2) + unit_eps)
    (q times q_scale) [tokens, key heads * dim]; decays exp(-exp(a_log[h]) softplus(decay_rows[t, h, i] + dt_bias[h, i]))
    [tokens, heads * dim]; betas sigmoid(beta_rows[t, h]) [tokens, heads]."""
    _need(rows.dim() == 2 and rows.stride(1) == 1 and rows.shape[1] >= max(q_col, k_col) + n_key_heads * dim, "delta_prepare: bad rows")
    T = rows.shape[0]
    for t, n, name in ((decay_rows, n_heads * dim, "decay rows"), (beta_rows, n_heads, "beta rows")):
        _need(t.dim() == 2 and t.stride(1) == 1 and tuple(t.shape) == (T, n) and t.dtype is rows.dtype, f"delta_prepare: bad {name}")
    _need(dt_bias.is_contiguous() and dt_bias.numel() == n_heads * dim, "delta_prepare: a bias per head and key channel")
    dev = rows.device
    q_f = torch.empty((T, n_key_heads * dim), dtype=torch.float32, device=dev)
    k_f = torch.empty((T, n_key_heads * dim), dtype=torch.float32, device=dev)
    g_f = torch.empty((T, n_heads * dim), dtype=torch.float32, device=dev)
    beta_f = torch.empty((T, n_heads), dtype=torch.float32, device=dev)
    a = library.DeltaPrepareArgs()
    a.dtype, a.bias_dtype, a.n_tokens, a.n_heads, a.n_key_heads, a.dim = _dtype_code(rows), _dtype_code(dt_bias), T, n_heads, n_key_heads, dim
    a.rows, a.row_stride, a.q_col, a.k_col = rows.data_ptr(), rows.stride(0), q_col, k_col
    a.decay_rows, a.decay_stride = decay_rows.data_ptr(), decay_rows.stride(0)
    a.beta_rows, a.beta_stride = beta_rows.data_ptr(), beta_rows.stride(0)
    a.dt_bias, a.a_log = dt_bias.data_ptr(), _f32_vec(a_log, n_heads, "a_log")
    a.q_scale, a.unit_eps = float(q_scale), float(unit_eps)
    a.q_f, a.k_f, a.g_f, a.beta_f = q_f.data_ptr(), k_f.data_ptr(), g_f.data_ptr(), beta_f.data_ptr()
    library.check(library.load().rdl_delta_prepare(ctypes.byref(a), _stream(rows)))
    return q_f, k_f, g_f, beta_f


def delta_rule_scan(rows: torch.Tensor, *, v_col: int, q_f, k_f, g_f, beta_f, n_heads: int, n_key_heads: int, dim: int, vdim: int,
                    state: torch.Tensor, tok_pos, seq_start, slots, n_seqs: int, kind: str = "auto") -> torch.Tensor:
    """The delta rule with a decay per key channel, in float: per head h with key head j(h),
    S <- g_t (.) S (row i times g_t[i]);  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t,
    v [vdim] of head h from column v_col of `rows`, the rest as `delta_prepare` made it; S float32 [slots, heads, dim, vdim]
    read from and left in `state`.  Returns float32 [tokens, heads * vdim].
    kind: "scan" (token by token), "chunked" (eight tokens at a time: what depends on no state is made for all groups at
    once, the state takes a group's writes in one pass; heads of up to 128 key channels), "auto" (groups where sequences
    bring many bfloat16 tokens each)."""
    a = library.RecurrenceArgs()
    out = _recurrence_common(a, rows, state, n_heads, n_key_heads, dim, vdim, tok_pos, seq_start, slots, n_seqs)
    T = rows.shape[0]
    _need(rows.shape[1] >= v_col + n_heads * vdim, "delta_rule_scan: the rows are narrower than the heads")
    for t, n, name in ((q_f, n_key_heads * dim, "q"), (k_f, n_key_heads * dim, "k"), (g_f, n_heads * dim, "decays"), (beta_f, n_heads, "betas")):
        _need(t.dtype is torch.float32 and t.is_contiguous() and tuple(t.shape) == (T, n), f"delta_rule_scan: {name} must be float32 [{T}, {n}]")
    a.mode, a.v_col = library.REC_DELTA, v_col
    a.q_f, a.k_f, a.g_f, a.beta_f = q_f.data_ptr(), k_f.data_ptr(), g_f.data_ptr(), beta_f.data_ptr()
    if kind == "auto":
        many = T >= DECAY_CHUNKED_MIN_TOKENS and T >= DECAY_CHUNKED_MIN_PER_SEQUENCE * n_seqs
        # float32 rows stay token by token: there a step's cut leaves the same bits
        kind = "chunked" if (DECAY_CHUNKED and many and rows.dtype is torch.bfloat16 and dim <= DELTA_CHUNKED_MAX_DIM) else "scan"
    lib = library.load()
    if kind == "scan":
        library.check(lib.rdl_recurrence_scan(ctypes.byref(a), _stream(rows)))
    elif kind == "chunked":
        _need(dim <= DELTA_CHUNKED_MAX_DIM, f"delta_rule_scan: the chunked kernels take heads of up to {DELTA_CHUNKED_MAX_DIM} key channels")
        nbytes = lib.rdl_delta_rule_chunked_work_bytes(T, n_seqs, n_heads, dim, vdim)
        work = torch.empty((nbytes // 4,), dtype=torch.float32, device=rows.device)
        library.check(lib.rdl_delta_rule_chunked(ctypes.byref(a), _ptr(work), nbytes, _stream(rows)), 2)
    else:
        raise KernelError(f"delta_rule_scan: unknown kind '{kind}'")
    return out
