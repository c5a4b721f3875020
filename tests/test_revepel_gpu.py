"""Revepel on the GPU: each new kernel alone against the plain functions of `plain_revepel.py` in float64, then the engine
against the plain model: whole prompts, token by token, portions, unequal batches on reused slots and pages, long
decoding, a token far back, generation, the command line and the trace replay."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs as ref
import plain_revepel as plain
import revepel_helpers as rh
from rust_deeplearning_b200.kernels import ops
from test_kernels_gpu import Case, assert_close, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["RA", "RB", "RC"]
F64 = torch.float64


def _dev(a):
    return torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)


def _np(t):
    return t.detach().cpu().to(F64).numpy()


class Rows:
    """Sequences of a step as the engine packs them: lens new rows each after `past` earlier ones, on slots in another
    order than the sequences."""

    def __init__(self, lens, past):
        self.lens, self.past, self.n, self.T = lens, past, len(lens), sum(lens)
        self.starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        self.slot_ids = (np.arange(self.n, dtype=np.int32)[::-1] * 2 + 1).copy()
        self.n_slots = 2 * self.n + 2
        self.tok_seq = _dev(np.concatenate([np.full(L, i) for i, L in enumerate(lens)]))
        self.tok_pos = _dev(np.concatenate([np.arange(p, p + L) for p, L in zip(past, lens)]))
        self.seq_start, self.slots = _dev(self.starts), _dev(self.slot_ids)

    def where(self):
        return dict(tok_pos=self.tok_pos, seq_start=self.seq_start, slots=self.slots)

    def one(self, s, t):
        """Row t of sequence s as a step of its own."""
        r = Rows([1], [self.past[s] + t - int(self.starts[s])])
        r.slots = self.slots[s:s + 1].contiguous()
        return r


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,lens,past", [(64, [5, 1, 2], [0, 7, 0]), (72, [1], [0]), (1000, [3, 40], [9, 0]), (4608, [2, 2], [1, 0])])
def test_norm_and_token_shift(dtype, width, lens, past):
    r = Rows(lens, past)
    x = rnd((r.T, width), torch.float32, 1, 3.0)
    w, shift = rnd((width,), dtype, 2, 0.3) + 1.0, rnd((width,), dtype, 3, 0.4)
    state = rnd((r.n_slots, width), torch.float32, 4)
    before = state.clone()
    n_want = plain.rms_rows(_np(x), 1e-5) * _np(w)
    m_want = np.zeros_like(n_want)
    for s in range(r.n):
        a, b = r.starts[s], r.starts[s + 1]
        prev = np.zeros(width) if past[s] == 0 else _np(before[int(r.slot_ids[s])])
        seq = np.vstack([prev[None], n_want[a:b]])
        m_want[a:b] = seq[1:] + (seq[:-1] - seq[1:]) * _np(shift)
    n, m = ops.norm_shift(x, w, 1e-5, shift, state, tok_seq=r.tok_seq, out_dtype=dtype, **r.where())
    assert_close(n, torch.from_numpy(n_want).to(dtype).to(DEV), dtype, what="normed rows")
    assert_close(m, torch.from_numpy(m_want).to(dtype).to(DEV), dtype, what="shifted rows")
    for s in range(r.n):
        assert_close(state[int(r.slot_ids[s])], torch.from_numpy(n_want[r.starts[s + 1] - 1]).float().to(DEV), torch.float32, what="kept row")
    untouched = [i for i in range(r.n_slots) if i not in r.slot_ids.tolist()]
    assert torch.equal(state[untouched], before[untouched])
    # the same bits when the rows come one by one
    st2 = before.clone()
    for s in range(r.n):
        for t in range(r.starts[s], r.starts[s + 1]):
            o = r.one(s, t)
            n1, m1 = ops.norm_shift(x[t:t + 1].contiguous(), w, 1e-5, shift, st2, tok_seq=o.tok_seq, out_dtype=dtype, **o.where())
            assert torch.equal(n1[0], n[t]) and torch.equal(m1[0], m[t])
    assert torch.equal(st2, state)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,channels,lens,past,bias", [(4, 40, [9, 1, 2, 1], [0, 5, 0, 0], True), (2, 130, [3, 30], [1, 0], False),
                                                          (1, 24, [4], [2], True), (3, 300, [1, 2, 70], [1, 1, 2], False), (8, 16, [3, 20], [0, 4], True)])
def test_short_convolution_with_carried_inputs(dtype, taps, channels, lens, past, bias):
    """Sequences shorter than the taps, a first token, carried inputs (also fewer than taps - 1 of them), rows that are a
    column slice of wider rows; and the same bits one row a step."""
    r = Rows(lens, past)
    wide = rnd((r.T, channels + 24), dtype, 11)
    rows = wide[:, 8:8 + channels]
    w, b = rnd((channels, taps), dtype, 12, 0.5), (rnd((channels,), dtype, 13, 0.3) if bias else None)
    keep = taps - 1
    state = rnd((r.n_slots, max(keep, 1), channels), torch.float32, 14) if keep else None
    before = state.clone() if keep else None
    want = np.zeros((r.T, channels))
    want_state = {}
    for s in range(r.n):
        a, e = r.starts[s], r.starts[s + 1]
        old = np.zeros((keep, channels))
        if keep and past[s] > 0:
            old = _np(before[int(r.slot_ids[s])]).copy()
            old[:max(0, keep - past[s])] = 0.0            # positions before the sequence's start
        seq = np.vstack([old, _np(rows[a:e])])
        out = plain.short_conv(seq, _np(w), _np(b) if bias else None)[keep:]
        want[a:e] = plain.silu(out)
        want_state[s] = seq[len(seq) - keep:] if keep else None
    got = ops.short_conv(rows, w, b, state, tok_seq=r.tok_seq, silu=True, **r.where())
    assert_close(got, torch.from_numpy(want).to(dtype).to(DEV), dtype, what="convolution")
    for s in range(r.n):
        if keep:
            assert_close(state[int(r.slot_ids[s])], torch.from_numpy(want_state[s]).float().to(DEV), torch.float32, what="kept inputs")
    if keep:
        st2 = before.clone()
        for s in range(r.n):
            if past[s] > 0:
                st2[int(r.slot_ids[s]), :max(0, keep - past[s])] = 0.0
        ref_state = st2.clone()
        got2 = ops.short_conv(rows, w, b, ref_state, tok_seq=r.tok_seq, silu=True, **r.where())
        for s in range(r.n):
            for t in range(r.starts[s], r.starts[s + 1]):
                o = r.one(s, t)
                g1 = ops.short_conv(rows[t:t + 1], w, b, st2, tok_seq=o.tok_seq, silu=True, **o.where())
                assert torch.equal(g1[0], got2[t])
        assert torch.equal(st2, ref_state)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_sum_group_norm_with_the_gate_first_and_activations(dtype):
    T, W = 7, 72
    res = rnd((T, W), torch.float32, 21, 2.0)
    gates = rnd((T, 2 * W + 8), dtype, 22, 2.0)[:, 8:]
    a, b1, b2 = rnd((T, W), dtype, 23), rnd((T, W), dtype, 24), rnd((T, W), dtype, 25)
    ba, bb = rnd((W,), dtype, 26), rnd((W,), dtype, 27)
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    g = _np(gates)
    want = _np(res) + sig(g[:, :W] + _np(ba)) * _np(a) + sig(g[:, W:2 * W] + _np(bb)) * (_np(b1) + _np(b2))
    got = ops.gated_residual_add_(res.clone(), gates, ba, a, bb, b1, b2)
    assert_close(got, torch.from_numpy(want).float().to(DEV), torch.float32, what="both branches")
    want = _np(res) + sig(g[:, :W] + _np(ba)) * _np(a)
    assert_close(ops.gated_residual_add_(res.clone(), gates, ba, a), torch.from_numpy(want).float().to(DEV), torch.float32, what="one branch")

    for rows, groups, group in ((5, 3, 20), (70, 2, 128), (2, 1, 96)):
        x = rnd((rows, groups * group), torch.float32, 28, 4.0)
        gate = rnd((rows, groups * group + 8), dtype, 29)[:, 8:]
        wn = rnd((groups * group,), dtype, 30) + 1.0
        y = _np(x) * plain.silu(_np(gate))
        want = plain.rms_rows(y.reshape(rows, groups, group), 1e-5).reshape(rows, -1) * _np(wn)
        got = ops.group_norm_gate(x, groups, eps=1e-5, weight=wn, gate=gate, gate_kind="silu", out_dtype=dtype, gate_first=True)
        assert_close(got, torch.from_numpy(want).to(dtype).to(DEV), dtype, what="gate before the norm")

    for m, n, k in ((3, 40, 64), (60, 24, 72), (200, 256, 128)):
        x, w = rnd((m, k), dtype, 31), rnd((n, k), dtype, 32, 0.2)
        want = plain.relu2(_np(x) @ _np(w).T)
        assert_close(ops.linear(x, w, activation="relu2"), torch.from_numpy(want).to(dtype).to(DEV), dtype, what=f"relu2 after a product of {m} rows")


def _ssm_case(H, G, N, P, lens, past, dtype, seed, lead=4):
    r = Rows(lens, past)
    inner = H * P
    rows = rnd((r.T, inner + 2 * G * N + lead), dtype, seed, 0.8)[:, lead:]
    dt_rows = rnd((r.T, H + 3), dtype, seed + 1)[:, 3:]
    dt_bias, a_log, d_skip = rnd((H,), torch.float32, seed + 2, 0.5), rnd((H,), torch.float32, seed + 3, 0.7), rnd((H,), torch.float32, seed + 4)
    a_log[0] = -9.0                                       # a head that forgets nothing
    state = rnd((r.n_slots, H, N, P), torch.float32, seed + 5, 0.5)
    for s in range(r.n):
        if past[s] == 0:
            state[int(r.slot_ids[s])] = 0
    R, DT = _np(rows), _np(dt_rows)
    want = np.zeros((r.T, inner))
    want_state = _np(state).copy()
    for s in range(r.n):
        a, e = r.starts[s], r.starts[s + 1]
        for h in range(H):
            g = h // (H // G)
            S = want_state[int(r.slot_ids[s]), h]
            dt = plain.softplus(DT[a:e, h] + float(dt_bias[h]))
            for t in range(a, e):       # the plain recurrence from the given state
                S = math.exp(-math.exp(float(a_log[h])) * dt[t - a]) * S + dt[t - a] * np.outer(R[t, inner + g * N:inner + (g + 1) * N], R[t, h * P:(h + 1) * P])
                want[t, h * P:(h + 1) * P] = S.T @ R[t, inner + G * N + g * N:inner + G * N + (g + 1) * N] + float(d_skip[h]) * R[t, h * P:(h + 1) * P]
            want_state[int(r.slot_ids[s]), h] = S
    kw = dict(x_col=0, b_col=inner, c_col=inner + G * N, n_heads=H, n_groups=G, state_dim=N, vdim=P, dt_bias=dt_bias, a_log=a_log, d_skip=d_skip)
    return r, rows, dt_rows, state, kw, want, want_state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [dict(H=4, G=2, N=8, P=16, lens=[33, 1, 2], past=[0, 7, 0]), dict(H=3, G=3, N=12, P=20, lens=[5, 70], past=[3, 0]),
                                   dict(H=2, G=1, N=64, P=64, lens=[9, 1], past=[0, 0]), dict(H=1, G=1, N=300, P=33, lens=[6], past=[2])])
def test_state_space_scan(dtype, sizes):
    """The scan against the plain recurrence from a carried state: heads that share B and C, sizes that are no multiples
    of anything, a head that never decays; untouched slots stay; one token a step gives the same bits."""
    r, rows, dt_rows, state, kw, want, want_state = _ssm_case(dtype=dtype, seed=40, **sizes)
    st = state.clone()
    got = ops.state_space_scan(rows, dt_rows, state=st, n_seqs=r.n, **r.where(), **kw)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(_np(got) - want).max() <= 3e-5 * scale
    assert np.abs(_np(st) - want_state).max() <= 3e-5 * max(1.0, float(np.abs(want_state).max()))
    untouched = [i for i in range(r.n_slots) if i not in r.slot_ids.tolist()]
    assert torch.equal(st[untouched], state[untouched])
    st2 = state.clone()
    for s in range(r.n):
        for t in range(r.starts[s], r.starts[s + 1]):
            o = r.one(s, t)
            g1 = ops.state_space_scan(rows[t:t + 1], dt_rows[t:t + 1], state=st2, n_seqs=1, **o.where(), **kw)
            assert torch.equal(g1[0], got[t])
    assert torch.equal(st2, st)


@pytest.mark.parametrize("sizes", [dict(H=4, G=2, N=16, P=16, lens=[130, 64, 1, 65], past=[0, 9, 3, 0]), dict(H=2, G=1, N=128, P=64, lens=[200], past=[0]),
                                   dict(H=3, G=1, N=48, P=80, lens=[63, 129], past=[5, 0]), dict(H=2, G=2, N=32, P=144, lens=[2, 320], past=[0, 64])])
def test_state_space_in_chunks(sizes):
    """The chunked kernels against the plain recurrence and against the scan: chunks that end early, sequences of one and two
    tokens beside long ones, carried states, a head that never decays, head sizes that need a second block of columns; and the
    state they leave carries on, token by token, as the scan's does."""
    r, rows, dt_rows, state, kw, want, want_state = _ssm_case(dtype=torch.bfloat16, seed=44, lead=8, **sizes)
    assert ops.state_space_chunked_ok(rows, kw["x_col"], kw["b_col"], kw["c_col"], kw["state_dim"], kw["vdim"])
    st, st_scan = state.clone(), state.clone()
    got = ops.state_space_scan(rows, dt_rows, state=st, n_seqs=r.n, kind="chunked", **r.where(), **kw)
    ref = ops.state_space_scan(rows, dt_rows, state=st_scan, n_seqs=r.n, kind="scan", **r.where(), **kw)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(_np(got) - want).max() <= 1e-4 * scale
    assert np.abs(_np(got) - _np(ref)).max() <= 1e-4 * scale
    assert np.abs(_np(st) - want_state).max() <= 1e-4 * max(1.0, float(np.abs(want_state).max()))
    untouched = [i for i in range(r.n_slots) if i not in r.slot_ids.tolist()]
    assert torch.equal(st[untouched], state[untouched])
    with pytest.raises(ops.KernelError):
        ops.state_space_scan(rows[:, 4:], dt_rows, state=st, n_seqs=r.n, kind="chunked", **r.where(), **{**kw, "b_col": kw["b_col"] - 4, "c_col": kw["c_col"] - 4})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [dict(H=4, J=2, d=16, e=24, lens=[33, 1, 2], past=[0, 7, 0]), dict(H=3, J=1, d=12, e=20, lens=[5, 70], past=[3, 0]),
                                   dict(H=2, J=2, d=64, e=64, lens=[40], past=[0]), dict(H=1, J=1, d=130, e=33, lens=[6, 1], past=[2, 0]),
                                   dict(H=2, J=1, d=128, e=48, lens=[17, 8, 1, 9], past=[0, 4, 2, 0]), dict(H=2, J=2, d=72, e=16, lens=[64, 7], past=[0, 0])])
def test_delta_rule_preparation_and_scan(dtype, sizes):
    """The prepared vectors and both forms of the recurrence against the plain one from a carried state: token by token
    (one token a step gives the same bits), and eight tokens at a time (groups that end early, sequences of one token
    beside long ones, head sizes that are no multiples of anything)."""
    H, J, d, e, lens, past = (sizes[k] for k in ("H", "J", "d", "e", "lens", "past"))
    r = Rows(lens, past)
    rows = rnd((r.T, 2 * J * d + H * e + 4), dtype, 50, 0.8)[:, 4:]
    decay_rows, beta_rows = rnd((r.T, H * d + 8), dtype, 51, 1.5)[:, 8:], rnd((r.T, H + 1), dtype, 52, 2.0)[:, 1:]
    dt_bias, a_log = rnd((H * d,), dtype, 53, 0.5), rnd((H,), torch.float32, 54, 0.7)
    a_log[0] = -9.0
    R = _np(rows)
    q = plain.unit(R[:, :J * d].reshape(r.T, J, d)) * d ** -0.5
    k = plain.unit(R[:, J * d:2 * J * d].reshape(r.T, J, d))
    step = plain.softplus(_np(decay_rows) + _np(dt_bias)).reshape(r.T, H, d)
    g = np.exp(-np.exp(_np(a_log))[None, :, None] * step)
    beta = plain.sigmoid(_np(beta_rows))
    q_f, k_f, g_f, beta_f = ops.delta_prepare(rows, q_col=0, k_col=J * d, n_heads=H, n_key_heads=J, dim=d, decay_rows=decay_rows,
                                              beta_rows=beta_rows, dt_bias=dt_bias, a_log=a_log, q_scale=d ** -0.5, unit_eps=1e-6)
    for got, want, what in ((q_f, q, "q"), (k_f, k, "k"), (g_f, g, "decays"), (beta_f, beta, "betas")):
        assert np.abs(_np(got) - want.reshape(r.T, -1)).max() <= 1e-5, what
    state = rnd((r.n_slots, H, d, e), torch.float32, 55, 0.5)
    for s in range(r.n):
        if past[s] == 0:
            state[int(r.slot_ids[s])] = 0
    want = np.zeros((r.T, H * e))
    want_state = _np(state).copy()
    for s in range(r.n):
        a, b = r.starts[s], r.starts[s + 1]
        for h in range(H):
            j = h // (H // J)
            S = want_state[int(r.slot_ids[s]), h]
            for t in range(a, b):
                S = g[t, h][:, None] * S
                u = beta[t, h] * (R[t, 2 * J * d + h * e:2 * J * d + (h + 1) * e] - S.T @ k[t, j])
                S = S + np.outer(k[t, j], u)
                want[t, h * e:(h + 1) * e] = S.T @ q[t, j]
            want_state[int(r.slot_ids[s]), h] = S
    kw = dict(v_col=2 * J * d, n_heads=H, n_key_heads=J, dim=d, vdim=e)
    st = state.clone()
    got = ops.delta_rule_scan(rows, q_f=q_f, k_f=k_f, g_f=g_f, beta_f=beta_f, state=st, n_seqs=r.n, kind="scan", **r.where(), **kw)
    assert np.abs(_np(got) - want).max() <= 3e-5 * max(1.0, float(np.abs(want).max()))
    assert np.abs(_np(st) - want_state).max() <= 3e-5 * max(1.0, float(np.abs(want_state).max()))
    untouched = [i for i in range(r.n_slots) if i not in r.slot_ids.tolist()]
    if d <= ops.DELTA_CHUNKED_MAX_DIM:
        st3 = state.clone()
        got3 = ops.delta_rule_scan(rows, q_f=q_f, k_f=k_f, g_f=g_f, beta_f=beta_f, state=st3, n_seqs=r.n, kind="chunked", **r.where(), **kw)
        assert np.abs(_np(got3) - want).max() <= 3e-5 * max(1.0, float(np.abs(want).max()))
        assert np.abs(_np(st3) - want_state).max() <= 3e-5 * max(1.0, float(np.abs(want_state).max()))
        assert torch.equal(st3[untouched], state[untouched])
    else:
        with pytest.raises(ops.KernelError):
            ops.delta_rule_scan(rows, q_f=q_f, k_f=k_f, g_f=g_f, beta_f=beta_f, state=state.clone(), n_seqs=r.n, kind="chunked", **r.where(), **kw)
    st2 = state.clone()
    for s in range(r.n):
        for t in range(r.starts[s], r.starts[s + 1]):
            o = r.one(s, t)
            sl = slice(t, t + 1)
            g1 = ops.delta_rule_scan(rows[sl], q_f=q_f[sl], k_f=k_f[sl], g_f=g_f[sl], beta_f=beta_f[sl], state=st2, n_seqs=1, kind="scan", **o.where(), **kw)
            assert torch.equal(g1[0], got[t])
    assert torch.equal(st2, st)


def _sigmoid_attention_ref(c, b, bias, new_kv, scale):
    """Key by key in float64, from the cache (through the page lists, rows unswizzled) or the step's packed rows."""
    hd, group = c.head_dim, c.n_heads // c.n_kv_heads
    out = torch.zeros((c.T, c.n_heads * hd), dtype=F64)
    q = c.qkv.cpu().to(F64)
    k_all, v_all, tables = c.pages.k.cpu(), c.pages.v.cpu(), c.pages.tables.cpu()
    for t in range(c.T):
        p, seq = int(b.tok_pos[t]), int(b.tok_seq[t])
        cached, row0 = int(b.seq_cached[seq]), int(b.seq_start[seq]) - int(b.seq_past[seq])
        for h in range(c.n_heads):
            g = h // group
            for j in range(max(0, p - c.window + 1) if c.window else 0, p + 1):
                if j < cached:
                    page, r = ref._cache_index(tables[seq], j, c.page_size, c.ring_pages)
                    kr, vr = ref.cache_load(k_all[page, g, r], r).to(F64), ref.cache_load(v_all[page, g, r], r).to(F64)
                else:
                    rows, k_col, v_col = new_kv
                    kr = rows[row0 + j, k_col + g * hd:k_col + (g + 1) * hd].cpu().to(F64)
                    vr = rows[row0 + j, v_col + g * hd:v_col + (g + 1) * hd].cpu().to(F64)
                z = float(q[t, h * hd:(h + 1) * hd] @ kr) * scale + float(bias[h])
                out[t, h * hd:(h + 1) * hd] += vr / (1.0 + math.exp(-z))
    return out


@pytest.mark.parametrize("dtype,head_dim,fast", [(torch.float32, 24, False), (torch.bfloat16, 40, False), (torch.bfloat16, 64, False),
                                                 (torch.bfloat16, 32, True), (torch.bfloat16, 64, True), (torch.bfloat16, 96, True),
                                                 (torch.bfloat16, 128, True)])
@pytest.mark.parametrize("window,decode", [(None, False), (None, True), (9, False), (9, True), (70, False), (70, True)])
def test_attention_with_sigmoid_weights(dtype, head_dim, fast, window, decode):
    """Weights sigmoid(score + bias per head), not normalised: against the key-by-key sum over cache pages in shuffled
    order (a ring under a window) and the step's own rows, for prompts on a cached prefix and for single tokens; the
    plain kernel and the tensor-core kernels (prompts: mma.sync tiles; single tokens: split keys merged in the kernel)."""
    past = [130, 63, 67] if decode else [70, 0, 5]
    new = [1, 1, 1] if decode else [9, 140, 66]
    c = Case(past=past, new=new, n_heads=6, n_kv_heads=2, head_dim=head_dim, page_size=16, window=window, dtype=dtype, seed=61)
    bias = torch.tensor([-4.0, -1.0, 0.0, 0.7, -2.0, 1.5], dtype=torch.float32, device=DEV)
    b = c.batch("all" if decode else "past")
    if decode:
        ref.rope_cache(c.qkv, 6, 2, head_dim, tok_seq=c.tok_seq, tok_pos=c.tok_pos, pages=c.pages, seq_end=c.seq_end)
    extra = {} if decode else dict(new_kv=c.new_kv())
    kind = "plain" if not fast else ("decode" if decode else "prefill")
    if kind == "decode":
        extra["keys_per_split"] = 32         # several runs of keys, merged by the last block
    got = ops.attention(c.qkv, b, c.pages, kind=kind, sigmoid_bias=bias, **extra, **c.kw())
    want = _sigmoid_attention_ref(c, b, bias.cpu(), None if decode else c.new_kv(), c.kw()["score_scale"])
    assert_close(got, want.to(dtype).to(DEV), dtype, rel=8.0, what=f"sigmoid weights, {kind}")
    if fast:      # two bfloat16 terms carry the weights: the tensor-core kernels stay close to the float kernel
        plain_out = ops.attention(c.qkv, b, c.pages, kind="plain", sigmoid_bias=bias, **({} if decode else dict(new_kv=c.new_kv())), **c.kw())
        assert_close(got, plain_out, dtype, rel=2.0, what=f"{kind} beside plain")
    with pytest.raises(Exception, match="sinks"):
        ops.attention(c.qkv, b, c.pages, kind="plain", sigmoid_bias=bias, sinks=bias, **extra, **c.kw())


@pytest.mark.parametrize("dtype,fast", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("distance", [0, 1, 15, 16, 39, 40, 41, 200])
def test_one_key_stands_out_inside_the_window_and_not_outside(dtype, fast, decode, distance):
    """A window of 40 on pages of 16: for the last query one key `distance` back is given a large score and every other
    weight is made tiny by the bias, so the output is that key's value while distance < 40 and next to nothing from 40
    on - in a prompt on a cached prefix, and for a single token over the ring."""
    W, hd, total = 40, 32, 260
    past, new = ([total - 1], [1]) if decode else ([total - 30], [30])
    c = Case(past=past, new=new, n_heads=2, n_kv_heads=1, head_dim=hd, page_size=16, window=W, dtype=dtype, seed=70, max_context=total)
    j = total - 1 - distance
    qv = torch.zeros(hd)
    qv[3] = 10.0
    kv = torch.zeros(hd)
    kv[3] = 10.0
    c.qkv[-1, :2 * hd] = torch.cat([qv, qv]).to(dtype)
    value = torch.arange(1, hd + 1, dtype=torch.float32) / hd
    row = j - past[0]                                       # among the step's rows if >= 0
    if row >= 0:
        c.qkv[row, 2 * hd:3 * hd], c.qkv[row, 3 * hd:4 * hd] = kv.to(dtype), value.to(dtype)
    if decode:
        ref.rope_cache(c.qkv, 2, 1, hd, tok_seq=c.tok_seq, tok_pos=c.tok_pos, pages=c.pages, seq_end=c.seq_end)
    if row < 0 and distance < W + 40:                       # rows further back have left the ring
        page, r = ref._cache_index(c.pages.tables[0].cpu(), j, c.page_size, c.ring_pages)
        ref.cache_store(c.pages.k[page, 0, r], kv.to(dtype).to(DEV), r)
        ref.cache_store(c.pages.v[page, 0, r], value.to(dtype).to(DEV), r)
    bias = torch.tensor([-80.0, -80.0], dtype=torch.float32, device=DEV)     # the chosen key: 100 - 80; any other: below 50 - 80
    b = c.batch("all" if decode else "past")
    extra = {} if decode else dict(new_kv=c.new_kv())
    kind = "plain" if not fast else ("decode" if decode else "prefill")
    got = ops.attention(c.qkv, b, c.pages, kind=kind, sigmoid_bias=bias, **extra, **c.kw(scale=1.0))[-1].float().cpu()
    for h in range(2):
        o = got[h * hd:(h + 1) * hd]
        if distance < W:
            assert torch.allclose(o, value.to(dtype).float(), atol=2e-2 if dtype is torch.bfloat16 else 1e-5), (distance, o[:4])
        else:
            assert float(o.abs().max()) < 1e-6, (distance, o[:4])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,E,top,ff,width", [(5, 5, 2, 24, 64), (3, 3, 3, 20, 72), (300, 8, 2, 32, 128), (140, 1, 1, 64, 64)])
def test_experts_of_two_matrices_with_weights_on_their_inputs(dtype, rows, E, top, ff, width):
    """Sigmoid scores, the largest chosen (where the plain choice is no close call), the score on the expert's input; few
    rows (a warp per output) and many (sorted by expert onto the tensor cores)."""
    x = rnd((rows, width), dtype, 80)
    w_router = rnd((E, width), torch.float32, 81, 0.2)
    ups, downs = rnd((E, ff, width), dtype, 82, 0.15), rnd((E, width, ff), dtype, 83, 0.15)
    sel, sel_w = ops.moe_route(x, w_router, None, top, "sigmoid")
    s = plain.sigmoid(_np(x) @ _np(w_router).T)
    order = np.argsort(-s, axis=1, kind="stable")
    gap = np.full(rows, np.inf) if top == E else s[np.arange(rows), order[:, top - 1]] - s[np.arange(rows), order[:, top]]
    inner_gap = np.min(-np.diff(np.take_along_axis(s, order[:, :top], 1), axis=1), axis=1) if top > 1 else np.full(rows, np.inf)
    safe = (gap > 1e-5) & (inner_gap > 1e-5)
    assert safe.sum() >= rows * 0.9
    assert np.array_equal(sel.cpu().numpy()[safe], order[safe, :top])
    assert np.abs(_np(sel_w)[safe] - np.take_along_axis(s, order[:, :top], 1)[safe]).max() < 1e-5
    got = ops.moe_experts(x, sel, sel_w, ups, downs, E, "relu2", 0.0, weights_on_input=True)
    X, U, D = _np(x), _np(ups), _np(downs)
    chosen, weights = sel.cpu().numpy(), _np(sel_w)
    want = np.zeros((rows, width))
    for t in range(rows):
        for kk in range(top):
            e_ = int(chosen[t, kk])
            want[t] += plain.relu2((weights[t, kk] * X[t]) @ U[e_].T) @ D[e_].T
    assert_close(got, torch.from_numpy(want).to(dtype).to(DEV), dtype, rel=8.0, what="experts")


# ------------------------------------------------------------------------------------------
# the model through the engine
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(name, dtype):
    name = rh.name_for(name, dtype)
    eng = rh.engine(name, dtype)
    for seed, n in ((1, 1), (2, 2), (3, 63), (4, 64), (5, 65), (6, 200)):
        ids = rh.prompt(name, seed, n)
        slot = eng.new_sequence()
        rh.assert_logits(eng.step([slot], [ids], "all"), rh.plain_logits(name, ids), dtype, f"{name} whole {n}")
        eng.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first_and_after_a_prompt(name, dtype):
    """From position 0 one token a step; and a prompt of 100 tokens, then 40 single tokens past page and window edges
    (pages of 16), another sequence alive meanwhile on other pages and other state rows."""
    name = rh.name_for(name, dtype)
    eng = rh.engine(name, dtype, page_size=16)
    ids = rh.prompt(name, 7, 140)
    want = rh.plain_logits(name, ids)
    slot = eng.new_sequence()
    for t in range(20):
        rh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")
    other = eng.new_sequence()
    eng.step([other], [ids[:20]], [[]])
    slot2 = eng.new_sequence()
    rh.assert_logits(eng.step([slot2], [ids[:100]], "all"), want[:100], dtype, "prefix")
    for t in range(100, 140):
        rh.assert_logits(eng.step([slot2], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype):
    """A prompt in portions of 1 to 70 tokens on what earlier portions left in cache and state (pages of 8): portions
    shorter than the convolutions' taps, and starts that fall inside a window and on page borders."""
    name = rh.name_for(name, dtype)
    eng = rh.engine(name, dtype, page_size=8)
    ids = rh.prompt(name, 8, 171)
    want = rh.plain_logits(name, ids)
    slot, at = eng.new_sequence(), 0
    for n in (5, 2, 70, 2, 1, 3, 64, 16, 8):
        rh.assert_logits(eng.step([slot], [ids[at:at + n]], "all"), want[at:at + n], dtype, f"{name} portion at {at}")
        at += n
    assert at == 171


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Batches one after another on a cache with 4 slots and few pages: prompts of unequal lengths in one step, then one
    token each; shorter requests end earlier; later batches land on the slots, pages and state rows earlier ones gave
    back (every state must start from zero again).  Each request's logits equal those it gives alone."""
    name = rh.name_for(name, dtype)
    eng = rh.engine(name, dtype, max_tokens=14 * 16, max_seqs=4, page_size=16)
    shapes = [([5, 11, 17], [8, 8, 8]), ([1, 9, 70, 30], [12, 3, 7, 1]), ([90, 2, 20], [2, 22, 5])]
    for b, (lens, extra) in enumerate(shapes):
        seqs = [rh.prompt(name, 100 + 10 * b + i, n + e) for i, (n, e) in enumerate(zip(lens, extra))]
        want = [rh.plain_logits(name, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        rh.assert_logits(got, np.concatenate([w[:n] for w, n in zip(want, lens)]), dtype, f"batch {b} prompts")
        pos, live = list(lens), list(range(len(seqs)))
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            rh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), dtype, f"batch {b} decode at {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert eng.cache.n_free_slots == 4
    if dtype == "bfloat16":
        assert eng.graph_replays > 0


def test_float32_logits_do_not_depend_on_the_cut():
    """In 32-bit the same bits whole, in portions and token by token, alone and in a batch."""
    name = "RB"
    ids, other = rh.prompt(name, 9, 90), rh.prompt(name, 10, 33)
    eng = rh.engine(name, "float32", page_size=16)
    a = eng.new_sequence()
    whole = eng.step([a], [ids], "all").clone()
    b, c = eng.new_sequence(), eng.new_sequence()
    first = eng.step([c, b], [other, ids[:50]], "all")[33:].clone()
    rest = torch.cat([eng.step([b, c], [[ids[t]], [other[0]]], "all")[:1].clone() for t in range(50, 70)]
                     + [eng.step([b], [ids[70:]], "all").clone()])
    assert torch.equal(torch.cat([first, rest]), whole)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["RA", "RB"])
def test_a_token_far_back_shows_at_the_end_of_a_long_prompt(name, dtype):
    """Heads that never decay carry the first token to the end of a long prompt, through a prompt step and through
    single-token steps; with the first token changed the logits at the end differ, and the engine follows the plain
    implementation in both."""
    name = rh.name_for(name, dtype)
    eng = rh.engine(name, dtype)
    ids = rh.prompt(name, 12, 330)
    changed = None
    for k in range(1, 40):          # a changed first token whose prompt also routes without close calls
        cand = [(ids[0] + k) % rh.vocab(name)] + ids[1:]
        if name.endswith("x") or rh._run_plain(name, cand)[1] > rh.MARGIN:
            changed = cand
            break
    want, want_changed = rh.plain_logits(name, ids), rh.plain_logits(name, changed)
    effect = np.abs(want[-10:] - want_changed[-10:]).max()
    assert effect > 50 * 2e-5 * max(1.0, np.abs(want).max())

    def check(got, t, mine, other, what):
        rh.assert_logits(got, mine[t:t + 1], dtype, what)
        g = got.detach().float().cpu().double().numpy()[0]       # in bfloat16 too the logits side with their own first token
        assert np.linalg.norm(g - mine[t]) < np.linalg.norm(g - other[t]), what

    for seq, mine, other in ((ids, want, want_changed), (changed, want_changed, want)):
        slot = eng.new_sequence()
        got = eng.step([slot], [seq[:320]], [[300, 319]])
        check(got[:1], 300, mine, other, "prompt at 300")
        check(got[1:], 319, mine, other, "prompt at 319")
        for t in range(320, 330):
            check(eng.step([slot], [[seq[t]]], "last"), t, mine, other, f"position {t}")
        eng.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """400 single-token steps: windows slide over decoded tokens, rings wrap, and every state is updated 400 times in place."""
    name = rh.name_for("RC", dtype)
    eng = rh.engine(name, dtype)
    ids = rh.prompt(name, 11, 400)
    want = rh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:3]], [[]])
    for t in range(3, 400):
        got = eng.step([slot], [[ids[t]]], "last")
        if t % 9 == 0 or t > 385:
            rh.assert_logits(got, want[t:t + 1], dtype, f"position {t}")


def test_greedy_generation_through_the_entry_point():
    from rust_deeplearning_b200 import Generator
    name = "RA"
    cfg, w = rh.plain_model(name)
    prompts = [rh.prompt(name, 300 + i, n) for i, n in enumerate((1, 9, 70))]
    gen = Generator(rh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    got = gen.generate_batch(prompts, 10)
    for p, g in zip(prompts, got):
        assert g[:len(p)] == p and len(g) == len(p) + 10
        ids = list(p)
        for tok in g[len(p):]:      # the plain loop, while neither its best two tokens nor a routed choice is a close call
            margins = []
            row = np.sort(plain.forward(cfg, w, ids, None, margins)[-1])
            if row[-1] - row[-2] < 1e-3 or min(float(m.min()) for m in margins) < rh.MARGIN:
                break
            assert tok == int(np.argmax(plain.forward(cfg, w, ids)[-1]))
            ids.append(tok)
        assert len(ids) > len(p)
        assert gen.generate(p, 10) == g
    # bfloat16 through the same entry point, with sampling: it runs, and the same seed gives the same tokens
    gen16 = Generator(rh.loaded_model(name, "bfloat16"), max_batch=4, max_context=128).with_temperature(0.8).with_top_k(20).with_seed(5)
    assert gen16.generate_batch(prompts, 8) == gen16.generate_batch(prompts, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype, tmp_path):
    """bin/trace_run on a Revepel folder: two requests as one batch, then one token each, the shorter one ending first."""
    name = rh.name_for("RB", dtype)
    a, b = rh.prompt(name, 40, 30), rh.prompt(name, 41, 21)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:26], "want": [0, 25]}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[26]], "want": [0]}, {"id": "b", "tokens": [b[19]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[27]], "want": [0]}, {"id": "b", "tokens": [b[20]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[28]], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[29]], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", rh.model_folder(name), "--dtype", dtype,
                             "--out", str(tmp_path), "--max-tokens", "128"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    wa, wb = rh.plain_logits(name, a), rh.plain_logits(name, b)
    V = rh.vocab(name)
    read = lambda n: torch.tensor(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
    rh.assert_logits(read(0), np.stack([wa[0], wa[25], wb[18]]), dtype, "step 0")
    rh.assert_logits(read(1), wa[26:27], dtype, "step 1")
    rh.assert_logits(read(2), np.stack([wa[27], wb[20]]), dtype, "step 2")
    rh.assert_logits(read(3), wa[28:29], dtype, "step 3")
    rh.assert_logits(read(4), wa[29:30], dtype, "step 4")


def test_command_line_generates_with_a_revepel_folder(capsys):
    """The command line picks the architecture by config.json; its greedy tokens are the entry point's."""
    import io
    from rust_deeplearning_b200 import Generator, cli
    name = "RC"
    p = rh.prompt(name, 50, 12)
    out = io.StringIO()
    code = cli.main([rh.model_folder(name), "--prompt-ids", " ".join(map(str, p)), "--max-tokens", "6", "--temperature", "0",
                     "--dtype", "float32", "--max-context", "64"], stdout=out)
    assert code == 0
    assert "arch=Revepel" in capsys.readouterr().err
    gen = Generator(rh.loaded_model(name, "float32"), max_batch=1, max_context=64).with_temperature(0.0)
    assert [int(t) for t in out.getvalue().split()] == gen.generate(p, 6)[len(p):]
