"""Gasetar on a GPU against the plain implementation, in 32-bit and in bfloat16: each new mechanism's kernels alone,
whole prompts, single tokens through the cache, portions, unequal batches on reused slots and pages, window edges and
far keys under a sharp softmax, long decoding, greedy generation, the trace replay and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gasetar_helpers as gh
import plain_gasetar as plain
import tiny_gasetar

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["GA", "GB"]
DEV = "cuda:0"


def _t(a, dtype):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(DEV).to(getattr(torch, dtype))


def _back(t):
    return t.float().cpu().double().numpy()


def _close(got, want, dtype, what, bf16=2e-2):
    got = _back(got.detach())
    tol = (1e-5 if dtype == "float32" else bf16) * max(1.0, float(np.abs(want).max()))
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), what
    assert np.abs(got - want).max() <= tol, f"{what}: {np.abs(got - want).max():.3e} > {tol:.3e}"


def _ti(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


# ---- each mechanism alone ----

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(3, 1, 12, 6, 0, 12), (6, 2, 16, 8, 5, 16), (4, 4, 64, 32, 0, 64), (5, 5, 24, 12, 3, 20), (2, 1, 8, 0, 0, 8),
                                   (40, 8, 256, 64, 0, 256), (20, 4, 256, 128, 0, 256), (16, 8, 128, 64, 0, 128), (24, 8, 128, 32, 0, 128),
                                   (10, 2, 128, 64, 0, 128)])
def test_projection_norm_rotation_and_cache_write(dtype, sizes):
    """The kernel between the q/k/v product and attention against the plain norm over the whole projections and the plain
    rotation: sizes that are whole numbers of 16-byte pieces and sizes that are not, rows wider than their heads, heads
    laid out with zero padding (the mean divides by the unpadded size), no rotation at all; the cache rows are read back
    through a shuffled page list, and in a ring only the last writer of a row writes."""
    from rust_deeplearning_b200.kernels import ops
    from rust_deeplearning_b200.parts.position import Rotary
    H, G, D, rot_n, extra, true_d = sizes
    rng = np.random.default_rng(sum(sizes))
    T, page, eps = 11, 4, 1e-3
    rot = {"base": 80.0, "dims": rot_n, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 24}} if rot_n else None
    rows = rng.normal(size=(T, (H + 2 * G) * D + extra))
    wq, wk = rng.normal(size=(H, D)) + 1.0, rng.normal(size=(G, D)) + 1.0
    if true_d < D:      # padded heads: zeros beyond the true size, as the products' zero rows leave them
        rows[:, :(H + G) * D].reshape(T, H + G, D)[:, :, true_d:] = 0.0
        wq[:, true_d:] = 0.0
        wk[:, true_d:] = 0.0
    pos = np.arange(3, 3 + T, dtype=np.int32)
    x = _t(rows, dtype)
    rows = _back(x)
    part = Rotary(rot["base"], D, rot_n, 64, DEV, pairing="half", scaling=dict(rot["scaling"], kind="llama3")) if rot else None
    k_cache = torch.zeros((6, G, page, D), dtype=x.dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    tables = _ti([[5, 2, 0, 1, 3, 4]])
    pages = ops.KVPages(k_cache, v_cache, tables, page, 6)
    ops.rope_projnorm_cache(x, H, G, D, tok_seq=_ti([0] * T), tok_pos=_ti(pos), wq=_t(wq.reshape(-1), "float32"),
                            wk=_t(wk.reshape(-1), "float32"), eps=eps, q_count=H * true_d, k_count=G * true_d,
                            cos=part.cos if part else None, sin=part.sin if part else None, rotary_dim=rot_n, pages=pages,
                            seq_end=_ti([3 + T]))
    got = _back(x)
    wq32, wk32 = wq.astype(np.float32).astype(np.float64), wk.astype(np.float32).astype(np.float64)
    table = [5, 2, 0, 1, 3, 4]
    for t in range(T):
        q = rows[t, :H * D].reshape(H, D)[:, :true_d]
        k = rows[t, H * D:(H + G) * D].reshape(G, D)[:, :true_d]
        qn = plain.rms_norm(q.reshape(-1), wq32[:, :true_d].reshape(-1), eps).reshape(H, true_d)
        kn = plain.rms_norm(k.reshape(-1), wk32[:, :true_d].reshape(-1), eps).reshape(G, true_d)
        for h in range(H):
            _close(torch.tensor(got[t, h * D:h * D + true_d]), plain.rotate(qn[h], int(pos[t]), rot), dtype, f"query head {h} of token {t}")
        p, r = table[int(pos[t]) // page], int(pos[t]) % page
        for g in range(G):
            want_k = plain.rotate(kn[g], int(pos[t]), rot)
            _close(torch.tensor(got[t, (H + g) * D:(H + g) * D + true_d]), want_k, dtype, f"key head {g} of token {t}")
            stored_k, stored_v = _back(k_cache[p, g, r]), _back(v_cache[p, g, r])
            es = 2 if dtype == "bfloat16" else 4
            if (D * es) % 16 == 0:      # the stored row has its 16-byte pieces swizzled by its place in the page
                n = 16 // es
                un = lambda row: np.concatenate([row[((c ^ (r & 7)) if (c | 7) < D // n else c) * n:][:n] for c in range(D // n)])
                stored_k, stored_v = un(stored_k), un(stored_v)
            assert np.array_equal(stored_k, got[t, (H + g) * D:(H + g + 1) * D]) and np.array_equal(stored_v, rows[t, (H + G + g) * D:(H + G + g + 1) * D])
        assert np.array_equal(got[t, (H + G) * D:], rows[t, (H + G) * D:])      # values and whatever lies beyond the heads stay
    # a ring of two pages: positions 3..13 fall on 8 rows, and every row holds its last writer
    k_ring, v_ring = torch.zeros((2, G, page, D), dtype=x.dtype, device=DEV), torch.zeros((2, G, page, D), dtype=x.dtype, device=DEV)
    y = _t(rows, dtype)
    ops.rope_projnorm_cache(y, H, G, D, tok_seq=_ti([0] * T), tok_pos=_ti(pos), wq=_t(wq.reshape(-1), "float32"),
                            wk=_t(wk.reshape(-1), "float32"), eps=eps, q_count=H * true_d, k_count=G * true_d,
                            cos=part.cos if part else None, sin=part.sin if part else None, rotary_dim=rot_n,
                            pages=ops.KVPages(k_ring, v_ring, _ti([[1, 0]]), page, 2), seq_end=_ti([3 + T]))
    assert torch.equal(y, x)
    for t in range(T):
        p, r = [1, 0][(int(pos[t]) // page) % 2], int(pos[t]) % page
        last = max(u for u in range(T) if (int(pos[u]) - int(pos[t])) % (2 * page) == 0)
        pl, rl = table[int(pos[last]) // page], int(pos[last]) % page
        assert torch.equal(k_ring[p, :, r], k_cache[pl, :, rl]) or r != rl
        if r == rl and (r & 7) == (rl & 7):
            assert torch.equal(v_ring[p, :, r], v_cache[pl, :, rl])


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_norm_with_many_tokens(dtype):
    """Steps of many tokens take smaller blocks in bfloat16: 300 tokens at once against the same tokens eleven at a time and
    against the plain norm and rotation; in 32-bit a token's values do not depend on the step's row count."""
    from rust_deeplearning_b200.kernels import ops
    from rust_deeplearning_b200.parts.position import Rotary
    H, G, D, rot_n, T, eps = 6, 2, 64, 32, 300, 1e-4
    rng = np.random.default_rng(7)
    rows = _t(rng.normal(size=(T, (H + 2 * G) * D)), dtype)
    wq, wk = _t(rng.normal(size=H * D) + 1.0, "float32"), _t(rng.normal(size=G * D) + 1.0, "float32")
    part = Rotary(900.0, D, rot_n, 512, DEV, pairing="half")
    pos = np.arange(5, 5 + T, dtype=np.int32)
    kw = dict(wq=wq, wk=wk, eps=eps, q_count=H * D, k_count=G * D, cos=part.cos, sin=part.sin, rotary_dim=rot_n)
    whole = rows.clone()
    ops.rope_projnorm_cache(whole, H, G, D, tok_seq=_ti([0] * T), tok_pos=_ti(pos), **kw)
    pieces = rows.clone()
    for t0 in range(0, T, 11):
        piece = pieces[t0:t0 + 11]
        ops.rope_projnorm_cache(piece, H, G, D, tok_seq=_ti([0] * len(piece)), tok_pos=_ti(pos[t0:t0 + 11]), **kw)
    if dtype == "float32":
        assert torch.equal(whole, pieces)
    else:
        _close(whole, _back(pieces), dtype, "many tokens against few")
    x, wq64, wk64 = _back(rows), _back(wq), _back(wk)
    rot = {"base": 900.0, "dims": rot_n}
    for t in (0, 137, 299):
        qn = plain.rms_norm(x[t, :H * D], wq64, eps).reshape(H, D)
        kn = plain.rms_norm(x[t, H * D:(H + G) * D], wk64, eps).reshape(G, D)
        want = np.concatenate([plain.rotate(v, int(pos[t]), rot) for v in list(qn) + list(kn)] + [x[t, (H + G) * D:]])
        _close(whole[t], want, dtype, f"token {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 75, 1000, 2304, 9000])
def test_sum_of_branches_with_the_next_norm(dtype, width):
    """x <- x + s (a + b + c) and the norm of the sum in one kernel, for one to three branches, with and without the norm;
    in 32-bit a row's result does not depend on how many rows the step has."""
    from rust_deeplearning_b200.kernels import ops
    rng = np.random.default_rng(width)
    rows = 7
    x = rng.normal(size=(rows, width))
    br = [rng.normal(size=(rows, width)) for _ in range(3)]
    w = rng.normal(size=width) + 1.0
    bt = [_t(b, dtype) for b in br]
    br = [_back(b) for b in bt]
    wt = _t(w, dtype)
    for n in (1, 2, 3):
        xt = _t(x, "float32")
        want = _back(xt) + 0.7 * sum(br[:n])
        y = ops.add_branches_norm_(xt, bt[:n], 0.7, ops.NormParams(wt, 1e-5, 0.0), getattr(torch, dtype))
        _close(xt, want, "float32", f"sum of {n}")
        _close(y, plain.rms_norm(want, _back(wt), 1e-5), dtype, f"norm of the sum of {n}")
        x2 = _t(x, "float32")
        assert ops.add_branches_norm_(x2, (bt[0], None, bt[2]) if n == 2 else bt[:n], 0.7) is None
        if n != 2:
            assert torch.equal(x2, xt)
    if dtype == "float32":
        one = _t(x[3:4], "float32")
        y1 = ops.add_branches_norm_(one, [b[3:4].contiguous() for b in bt], 0.7, ops.NormParams(wt, 1e-5, 0.0))
        allx = _t(x, "float32")
        y = ops.add_branches_norm_(allx, bt, 0.7, ops.NormParams(wt, 1e-5, 0.0))
        assert torch.equal(y[3:4], y1) and torch.equal(allx[3:4], one)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 5, 200])
@pytest.mark.parametrize("shape", [(5, 2, True), (3, 1, False), (40, 6, True), (2, 2, False)])
def test_router_by_logit_and_experts(dtype, rows, shape):
    """Router (logits with a bias, the largest chosen, softmax over the chosen alone) and experts with a shared one
    against the plain ones: one expert of several, every expert, both expert kernels' forms."""
    from rust_deeplearning_b200.parts.routed_experts import RoutedExperts
    from rust_deeplearning_b200.kernels import ops
    n_exp, top, shared = shape
    rng = np.random.default_rng(3 + n_exp)
    W, ff = 48, 24
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n_exp, "top": top}, **({"shared": {"ff": 16}} if shared else {})}
    w = {"router": rng.normal(size=(n_exp, W)) * 0.5, "router.b": rng.normal(size=n_exp)}
    names = [f"e{e}." for e in range(n_exp)] + (["shared."] if shared else [])
    for p in names:
        n = 16 if p == "shared." else ff
        w[p + "gate"], w[p + "up"], w[p + "down"] = (rng.normal(size=s) * 0.3 for s in ((n, W), (n, W), (W, n)))
    wt = {k: _t(v, dtype) for k, v in w.items()}
    w = {k: _back(v) for k, v in wt.items()}
    xt = _t(rng.normal(size=(rows, W)), dtype)
    x = _back(xt)
    chosen, weight, margin = plain.router(x, w, "", f)
    sel, sel_w = ops.moe_route(xt, wt["router"].float(), None, top, "softmax_chosen", bias=wt["router.b"].float())
    safe = margin > 1e-5
    assert np.array_equal(sel.cpu().numpy()[safe], chosen[safe])        # in the order of the logits
    _close(sel_w[torch.tensor(safe, device=DEV)], weight[safe], "float32", "weights")
    assert torch.allclose(sel_w.sum(dim=1), torch.ones(rows, device=DEV), atol=1e-6)
    part = RoutedExperts(hidden_size=W, expert_size=ff, n_experts=n_exp, n_identity=0, top=top, form="silu", form_param=0.0,
                         w_router=wt["router"], correction=None, gates=[wt[f"e{e}.gate"] for e in range(n_exp)],
                         ups=[wt[f"e{e}.up"] for e in range(n_exp)], downs=[wt[f"e{e}.down"] for e in range(n_exp)],
                         scoring="softmax_chosen", router_bias=wt["router.b"],
                         shared=(wt["shared.gate"], wt["shared.up"], wt["shared.down"]) if shared else None)
    want = plain.feed_forward(x, w, "", f)
    _close(part.forward(xt)[torch.tensor(safe, device=DEV)], want[safe], dtype, "routed experts", bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_for_every_value(dtype):
    from rust_deeplearning_b200.kernels import ops
    rng = np.random.default_rng(5)
    for T, H, n, k, head in ((7, 3, 4, 9, 9), (20, 4, 16, 24, 32)):
        x, wgt, g = rng.normal(size=(T, 2 + H * head)), rng.normal(size=(H, n, k)), rng.normal(size=(T, 1 + H * n))
        xt, wt, gt = _t(x, dtype), _t(wgt, dtype), _t(g, dtype)
        x, wgt, g = _back(xt), _back(wt), _back(gt)
        sig = 1 / (1 + np.exp(-g[:, 1:].reshape(T, H, n)))
        want = np.einsum("hjk,thk->thj", wgt, x[:, 2:].reshape(T, H, head)[:, :, :k]) * sig
        _close(ops.heads_linear(xt, 2, head, wt, gate=gt[:, 1:], gate_per_value=True), want.reshape(T, H * n), dtype, "heads_linear, a gate per value")
        want = x[:, 2:].reshape(T, H, head)[:, :, :n] * sig
        _close(ops.gate_heads(xt[:, 2:], head, gt[:, 1:], H, n, per_value=True), want.reshape(T, H * n), dtype, "gate_heads, a gate per value")
        aligned = gt[:, 1:].contiguous()
        _close(ops.gate_heads(xt[:, 2:].contiguous(), head, aligned, H, n, per_value=True), want.reshape(T, H * n), dtype, "gate_heads, aligned")


@pytest.mark.parametrize("case", [
    # heads, kv_rank, rot_dim, page, splits
    (6, 32, 16, 16, 1), (6, 32, 16, 16, 3), (16, 96, 32, 64, None), (20, 48, 16, 8, 2), (3, 448, 64, 64, None), (17, 256, 64, 32, 5)])
def test_latent_decode_kernel_with_sinks(case):
    """The tensor-core decode kernel of the absorbed form against the float kernel, both with a sink per head (one of them
    large enough to take most of the weight): pages in random order, sequences of unequal lengths, a padding row, one split
    and several, no window.  In every sequence one key is made to dominate: the very first key (hundreds of keys back),
    the newest key, a key at a page's edge, in turn."""
    from rust_deeplearning_b200.kernels import ops
    H, r, rd, page, splits = case
    width = r + rd
    rng = np.random.default_rng(sum(case[:4]))
    lens = [1, 5, page, page + 1, 150, 333, 64, 65, 700]
    T = len(lens) + 1
    n_pages = sum(-(-n // page) for n in lens) + 2
    cache = torch.tensor(rng.normal(size=(n_pages, 1, page, width)) * 0.5, dtype=torch.float32).to(DEV).to(torch.bfloat16)
    order = rng.permutation(n_pages)
    tw = max(-(-n // page) for n in lens)
    tables = np.zeros((T, tw), dtype=np.int32)
    at = 0
    for i, n in enumerate(lens):
        k = -(-n // page)
        tables[i, :k] = order[at:at + k]
        at += k
    q = torch.tensor(rng.normal(size=(T, H * width)) * 0.5, dtype=torch.float32).to(DEV).to(torch.bfloat16)
    for i, n in enumerate(lens):
        p = n - 1
        target = [0, p, (p // page) * page, max(0, (p // page) * page - 1)][i % 4]
        row = q[i, :width].float() * 6.0
        pg, rr = tables[i, target // page], target % page
        sw = torch.empty(width, dtype=torch.float32, device=DEV)
        for c in range(width // 8):      # the stored row has its 16-byte chunks swizzled by its place in the page
            cc = (c ^ (rr & 7)) if (c | 7) < width // 8 else c
            sw[cc * 8:cc * 8 + 8] = row[c * 8:c * 8 + 8]
        cache[pg, 0, rr] = sw.to(torch.bfloat16)
    sinks = torch.tensor(rng.normal(size=H), dtype=torch.float32, device=DEV)
    sinks[H // 2] = 9.0
    pos = [n - 1 for n in lens] + [-1]
    ab = ops.AttentionBatch(T, T, _ti(list(range(T))), _ti(pos), _ti(list(range(T + 1))), _ti(pos[:-1] + [0]), _ti(lens + [0]),
                            max_keys=max(lens))
    pages = ops.KVPages(cache, cache, _ti(tables), page, tw)
    common = dict(n_heads=H, n_kv_heads=1, head_dim=width, score_scale=0.3, softcap=None, window=None, kind="plain")
    want = ops.attention(q, ab, pages, sinks=sinks, **common)
    bare = ops.attention(q, ab, pages, **common)
    got = ops.latent_decode(q, ab, pages, n_heads=H, kv_rank=r, score_scale=0.3, window=None, n_splits=splits, sinks=sinks)
    w = want.float().view(T, H, width)[:-1, :, :r]
    g = got.float().view(T, H, width)[:-1, :, :r]
    assert torch.isfinite(g).all()
    assert (bare.float().view(T, H, width)[:-1, :, :r] - w).abs().max().item() > 0.1      # the sinks show
    assert (g - w).abs().max().item() <= 0.02 * max(1.0, w.abs().max().item()), (g - w).abs().max().item()


# ---- the model ----

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_first_tokens(name, dtype):
    eng = gh.engine(name, dtype, page_size=16)
    for seed, n in ((1, 1), (2, 2), (3, 37), (4, 70)):
        ids = gh.prompt(name, seed, n, dtype)
        slot = eng.new_sequence()
        gh.assert_logits(eng.step([slot], [ids], "all"), gh.plain_logits(name, ids), dtype, f"{name} whole n={n}")
        eng.release(slot)
    ids = gh.prompt(name, 5, 6, dtype)
    slot = eng.new_sequence()
    for t in range(6):      # positions 0, 1, 2, ... each as a step of its own
        gh.assert_logits(eng.step([slot], [[ids[t]]], "all"), gh.plain_logits(name, ids)[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_stream_after_every_layer(dtype):
    """The stream after each layer against the plain one (the model cut after 1, 2, ... layers gives it as its last)."""
    from rust_deeplearning_b200.parts.norm import ResidualStream
    name = "GA"
    model = gh.loaded_model(name, dtype)
    eng = gh.engine(name, dtype, page_size=16)
    ids = gh.prompt(name, 8, 21, dtype)
    cfg, w = gh.plain_model(name)
    streams = []
    plain.forward(cfg, w, ids, streams=streams)
    seen = []
    for i, block in enumerate(model.layers):
        inner = block.forward

        def spy(stream, batch, cache, run, inner=inner):
            inner(stream, batch, cache, run)
            seen.append(stream.value().clone())
        block.forward = spy
    try:
        slot = eng.new_sequence()
        eng.step([slot], [ids], "last")
    finally:
        for block in model.layers:
            del block.forward
    assert len(seen) == len(streams) and isinstance(ResidualStream, type)
    for i, (got, want) in enumerate(zip(seen, streams)):
        _close(got, want, dtype, f"stream after layer {i}", bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype):
    """The last 45 tokens one by one: the windows (5, 9 and 33 keys) pass wholly over decoded tokens, pages of 16 positions
    are crossed and the rings wrap."""
    eng = gh.engine(name, dtype, page_size=16)
    ids = gh.prompt(name, 6, 80, dtype)
    want = gh.plain_logits(name, ids)
    other = eng.new_sequence()
    eng.step([other], [ids[:20]], [[]])          # shifts which pages the next sequence gets
    slot = eng.new_sequence()
    gh.assert_logits(eng.step([slot], [ids[:35]], "all"), want[:35], dtype, "prefix")
    for t in range(35, 80):
        gh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype):
    """A prompt cut into portions of 2 to 19 tokens on a cached prefix (pages of 8: rings wrap inside a portion)."""
    eng = gh.engine(name, dtype, page_size=8)
    ids = gh.prompt(name, 7, 66, dtype)
    want = gh.plain_logits(name, ids)
    slot = eng.new_sequence()
    at = 0
    for n in (5, 2, 19, 2, 3, 16, 11, 8):
        gh.assert_logits(eng.step([slot], [ids[at:at + n]], "all"), want[at:at + n], dtype, f"{name} portion at {at}")
        at += n
    assert at == 66


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Batches one after another on a cache with 4 slots and few pages: prompts of unequal lengths in one step, then one
    token each; shorter requests end earlier; later batches land on what earlier ones gave back.  Each request's logits
    equal those it gives alone (the plain implementation runs it alone)."""
    eng = gh.engine(name, dtype, max_tokens=10 * 16, max_seqs=4, page_size=16)
    shapes = [([5, 11, 17], [8, 8, 8]), ([1, 9, 23, 30], [12, 3, 7, 1]), ([40, 2, 20], [2, 22, 5])]
    for b, (lens, extra) in enumerate(shapes):
        seqs = [gh.prompt(name, 100 + 10 * b + i, n + e, dtype) for i, (n, e) in enumerate(zip(lens, extra))]
        want = [gh.plain_logits(name, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        gh.assert_logits(got, np.concatenate([w[:n] for w, n in zip(want, lens)]), dtype, f"batch {b} prompts")
        pos, live = list(lens), list(range(len(seqs)))
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            gh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), dtype, f"batch {b} decode at {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert eng.cache.n_free_slots == 4
    if dtype == "bfloat16":
        assert eng.graph_replays > 0


def test_window_edges_and_far_keys_under_a_sharp_softmax():
    """With scores multiplied by 10 (and the caps lifted) nearly all weight lies on one key per query and head; over 90
    positions that key is often the first or the last one a window keeps, would be the one just outside it, or, in the
    layers without a window, lies far back.  32-bit, whole and token by token, pages of 16, windows of 5 and 9 keys."""
    from rust_deeplearning_b200 import Engine, load_model, write_random_model
    cfg, seed = tiny_gasetar.config("GA")
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] *= 10.0      # (every sharp layer multiplies the rounding of the layers before it by as much)
        if "softcap" in layer["mixer"]:
            layer["mixer"]["softcap"] *= 20.0
    folder = os.path.join(gh.mh.tmp_root(), "tiny_GA_sharp")
    write_random_model(folder, cfg, seed, "bfloat16")
    pcfg, w = plain.load_folder(folder)
    ids = [int(v) for v in np.random.default_rng(9).integers(0, cfg["vocab"], size=90)]
    margins = []
    want = plain.forward(pcfg, w, ids, margins)
    safe = np.minimum.reduce(margins) > 1e-4
    first_unsafe = int(np.argmin(safe)) if not safe.all() else len(ids)      # logits after a close call are another computation
    assert first_unsafe > 50
    # one key more or one key less changes the plain logits by far more than the tolerance: the test can see an edge
    for i in (1, 2):
        moved = json.loads(json.dumps(pcfg))
        moved["layers"][i]["mixer"]["mask"]["size"] += 1
        assert np.abs(plain.forward(moved, w, ids)[:first_unsafe] - want[:first_unsafe]).max() > 1e-2
    no_sink = dict(w, **{"l0.mix.sink": np.full(3, -1e9)})
    assert np.abs(plain.forward(pcfg, no_sink, ids)[:first_unsafe] - want[:first_unsafe]).max() > 1e-2
    eng = Engine(load_model(folder, "float32", DEV), max_tokens=1024, page_size=16)
    slot = eng.new_sequence()
    gh.assert_logits(eng.step([slot], [ids[:first_unsafe]], "all"), want[:first_unsafe], "float32", "whole")
    slot = eng.new_sequence()
    n0 = min(30, first_unsafe)
    gh.assert_logits(eng.step([slot], [ids[:n0]], "all"), want[:n0], "float32", "prefix")
    for t in range(n0, first_unsafe):
        gh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], "float32", f"position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sinks_weigh_in_the_logits(dtype):
    """A model whose sinks are large differs from the same model with small ones by far more than the tolerance, and
    the engine follows the plain implementation in both: a sink left out would show."""
    from rust_deeplearning_b200 import Engine, load_model, write_random_model
    from rust_deeplearning_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg, seed = tiny_gasetar.config("GC")
    folder = os.path.join(gh.mh.tmp_root(), "tiny_GC_sinks")
    write_random_model(folder, cfg, seed, "bfloat16")
    file = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: file.tensor(n).clone() for n in file.names()}
    del file
    tensors["l1.mix.sink"] = torch.full_like(tensors["l1.mix.sink"], 4.0)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    pcfg, w = plain.load_folder(folder)
    ids = gh.mh.prompt(12, 40, cfg["vocab"])
    want = plain.forward(pcfg, w, ids)
    assert np.abs(want - gh.plain_logits("GC", ids)).max() > 0.05
    eng = Engine(load_model(folder, dtype, DEV), max_tokens=256, page_size=16)
    slot = eng.new_sequence()
    gh.assert_logits(eng.step([slot], [ids[:25]], "all"), want[:25], dtype, "prompt")
    for t in range(25, 40):
        gh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """300 single-token steps with every expert chosen: crosses pages, wraps the window's ring several times."""
    name = "GC"
    eng = gh.engine(name, dtype)
    ids = gh.mh.prompt(11, 300, gh.vocab(name))
    want = gh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:3]], [[]])
    for t in range(3, 300):
        got = eng.step([slot], [[ids[t]]], "last")
        if t % 7 == 0 or t > 280:
            gh.assert_logits(got, want[t:t + 1], dtype, f"position {t}")


def test_greedy_generation_through_the_entry_point():
    from rust_deeplearning_b200 import Generator
    name = "GB"
    cfg, w = gh.plain_model(name)
    prompts = [gh.prompt(name, 300 + i, n, "float32") for i, n in enumerate((1, 9, 23))]
    gen = Generator(gh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    got = gen.generate_batch(prompts, 10)
    for p, g in zip(prompts, got):
        assert g[:len(p)] == p
        # the plain loop, as long as its own margin between the best and the second best token is not a close call
        ids = list(p)
        for tok in g[len(p):]:
            row = np.sort(plain.forward(cfg, w, ids)[-1])
            if row[-1] - row[-2] < 1e-3 or plain.min_margin(cfg, w, ids) < 1e-4:
                break
            assert tok == int(np.argmax(plain.forward(cfg, w, ids)[-1]))
            ids.append(tok)
        assert gen.generate(p, 10) == g


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype, tmp_path):
    """bin/trace_run on a Gasetar folder: two requests as one batch, then one token each, the shorter one ending first."""
    name = "GA"
    a, b = gh.prompt(name, 40, 30, dtype), gh.prompt(name, 41, 21, dtype)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:26], "want": [0, 25]}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[26]], "want": [0]}, {"id": "b", "tokens": [b[19]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[27]], "want": [0]}, {"id": "b", "tokens": [b[20]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[28]], "want": [0]}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[29]], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", gh.model_folder(name), "--dtype", dtype,
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
    wa, wb = gh.plain_logits(name, a), gh.plain_logits(name, b)
    V = gh.vocab(name)
    read = lambda n: torch.tensor(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
    gh.assert_logits(read(0), np.stack([wa[0], wa[25], wb[18]]), dtype, "step 0")
    gh.assert_logits(read(1), wa[26:27], dtype, "step 1")
    gh.assert_logits(read(2), np.stack([wa[27], wb[20]]), dtype, "step 2")
    gh.assert_logits(read(3), wa[28:29], dtype, "step 3")
    gh.assert_logits(read(4), wa[29:30], dtype, "step 4")


def test_trace_replay_with_the_promise_counted_in_tokens(tmp_path):
    """Seven short requests in one batch, then two tokens each, with --max-tokens set to the tokens they hold, padding not
    counted (far fewer than seven pages' worth): the replay's cache has a slot and a page's slack for each of them."""
    name, dtype = "GA", "float32"
    seqs = [gh.prompt(name, 60 + i, n + 2, dtype) for i, n in enumerate((3, 1, 9, 20, 2, 5, 14))]
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": s[:-2], "want": [len(s) - 3]} for i, s in enumerate(seqs)], "end": []},
             {"step": 1, "entries": [{"id": f"r{i}", "tokens": [s[-2]], "want": [0]} for i, s in enumerate(seqs)], "end": []},
             {"step": 2, "entries": [{"id": f"r{i}", "tokens": [s[-1]], "want": [0]} for i, s in enumerate(seqs)], "end": [f"r{i}" for i in range(7)]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", gh.model_folder(name), "--dtype", dtype,
                        "--out", str(tmp_path), "--max-tokens", str(sum(len(s) for s in seqs))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.split() == ["done", "0", "done", "1", "done", "2"], (r.stdout, r.stderr)
    V = gh.vocab(name)
    want = [gh.plain_logits(name, s) for s in seqs]
    for n, at in ((0, -3), (1, -2), (2, -1)):
        got = torch.tensor(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
        gh.assert_logits(got, np.stack([w[at] for w in want]), dtype, f"step {n}")


def test_command_line_generates_with_a_gasetar_folder(capsys):
    """The command line picks the architecture by config.json; its greedy tokens are the entry point's."""
    import io
    from rust_deeplearning_b200 import Generator, cli
    name = "GB"
    p = gh.prompt(name, 50, 12, "float32")
    out = io.StringIO()
    code = cli.main([gh.model_folder(name), "--prompt-ids", " ".join(map(str, p)), "--max-tokens", "6", "--temperature", "0",
                     "--dtype", "float32", "--max-context", "64"], stdout=out)
    assert code == 0
    assert "arch=Gasetar" in capsys.readouterr().err
    gen = Generator(gh.loaded_model(name, "float32"), max_batch=1, max_context=64).with_temperature(0.0)
    assert [int(t) for t in out.getvalue().split()] == gen.generate(p, 6)[len(p):]
