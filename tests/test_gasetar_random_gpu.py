"""Gasetar configurations drawn at random (seeded): one to three layers in any order of the two mixers, head sizes and ranks
that are and are not multiples of 8 and 16, one to three key heads with one to nine query heads each, values narrower and wider
than keys, rotation on all or a part of a head with and without slowed-down wavelengths, windows from 5 keys to none, caps on
and off, dense, routed (one expert to all of them, with and without a shared one) and no feed-forward, any constants, pages of 16,
32 and 64 rows.  Each case runs one to four sequences of unequal length through the engine in both dtypes - whole, as a prefix
with single tokens after it, and as chunks of 1 to 29 tokens a step that mix with one another - and compares the logits with the
plain implementation up to each sequence's first token whose routing is a close call (the routers' matrices are made six times
as large, so that close calls are few); in float32 the three ways of cutting also
have to give the same bits."""
import tempfile

import numpy as np
import pytest
import torch

import model_helpers as mh
import plain_gasetar as plain

pytestmark = pytest.mark.gpu
MARGIN = {"float32": 1e-4, "bfloat16": 5e-2}


def _rot(rng, limit):
    dims = int(rng.choice([d for d in (limit, limit // 2, 8, 6) if d % 2 == 0 and 2 <= d <= limit]))
    rot = {"base": float(rng.choice([100.0, 10000.0, 250000.0])), "dims": dims}
    if rng.integers(0, 2):
        rot["scaling"] = {"factor": float(rng.choice([2.0, 8.0])), "low": 1.0, "high": float(rng.choice([4.0, 16.0])),
                          "original": int(rng.choice([16, 64, 1024]))}
    return rot


def _mlp(rng):
    kind = int(rng.integers(0, 5))
    if kind == 0:
        return None
    if kind == 1:
        return {"kind": "dense", "ff": int(rng.choice([40, 64, 96, 52]))}
    experts = int(rng.choice([1, 2, 4, 8]))
    top = experts if kind == 2 else int(rng.integers(1, experts + 1))
    f = {"kind": "moe", "expert": {"ff": int(rng.choice([16, 24, 64, 20]))}, "router": {"experts": experts, "top": top}}
    if rng.integers(0, 2):
        f["shared"] = {"ff": int(rng.choice([16, 40]))}
    return f


def draw(case: int):
    rng = np.random.default_rng(100 + case)
    layers = []
    for _ in range(int(rng.integers(1, 4))):
        if rng.integers(0, 3) < 2:
            dim = int(rng.choice([16, 24, 32, 64, 40, 128]))
            kv = int(rng.choice([1, 2, 3]))
            m = {"heads": kv * int(rng.choice([1, 2, 3, 5, 9])), "kv_heads": kv, "dim": dim, "vdim": int(rng.choice([dim, dim, 16, 48])),
                 "scale": float(rng.choice([dim ** -0.5, 0.3, 1.0])), "rot": _rot(rng, dim)}
            if rng.integers(0, 3):
                m["softcap"] = float(rng.choice([5.0, 30.0]))
            window = int(rng.choice([0, 5, 17, 40, 70]))
            if window:
                m["mask"] = {"size": window}
            layers.append({"type": "attention", "mixer": m, "mlp": _mlp(rng)})
        else:
            rd = int(rng.choice([8, 16, 32, 6]))
            m = {"heads": int(rng.choice([1, 3, 6, 17])), "dim": int(rng.choice([8, 16, 32, 20])), "rot_dim": rd,
                 "vdim": int(rng.choice([8, 16, 24, 32])), "kv_rank": int(rng.choice([16, 24, 48, 56, 64])),
                 "scale": float(rng.choice([0.15, 0.3])), "rot": dict(_rot(rng, rd), dims=rd)}
            layers.append({"type": "latent_attention", "mixer": m, "mlp": _mlp(rng)})
    cfg = {"architecture": "Gasetar", "width": int(rng.choice([48, 64, 72, 88, 136, 50])), "vocab": int(rng.integers(90, 400)),
           "norm": {"eps": float(rng.choice([1e-6, 1e-5, 1e-3]))}, "embedding": {"scale": float(rng.choice([1.0, 4.0, 9.5]))},
           "residual_mult": float(rng.choice([1.0, 0.8, 0.25])), "logit_scale": float(rng.choice([1.0, 0.4, 1.7])),
           "max_positions": 512, "layers": layers}
    if rng.integers(0, 2):
        cfg["logit_softcap"] = float(rng.choice([10.0, 25.0]))
    page = int(rng.choice([16, 32, 64]))
    lengths = [int(v) for v in rng.integers(1, 90, size=int(rng.integers(1, 5)))]
    return rng, cfg, page, lengths


@pytest.mark.parametrize("case", range(16))
def test_a_configuration_drawn_at_random(case):
    from rust_deeplearning_b200 import Engine, load_model, write_random_model
    from rust_deeplearning_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    rng, cfg, page, lengths = draw(case)
    what = f"case {case}: width {cfg['width']}, " + "; ".join(
        f"{l['type']} {sorted((k, v) for k, v in l['mixer'].items() if k not in ('rot', 'scale'))} mlp {l['mlp']}" for l in cfg["layers"]) + \
        f", page {page}, lengths {lengths}"
    with tempfile.TemporaryDirectory(prefix="rdl_random_") as folder:
        write_random_model(folder, cfg, case, "bfloat16")
        # routers six times as large: fewer close calls, so that bfloat16 is compared over most of every sequence
        path = f"{folder}/model.safetensors"
        file = SafetensorsFile(path)
        tensors = {n: file.tensor(n).clone() for n in file.names()}
        del file
        write_safetensors(path, {n: (t.float() * 6.0).to(t.dtype) if n.endswith(".mlp.router") else t for n, t in tensors.items()})
        pcfg, pw = plain.load_folder(folder)
        seqs = [mh.prompt(2000 + 10 * case + i, n, cfg["vocab"]) for i, n in enumerate(lengths)]
        want, least = [], []
        for s in seqs:
            margins = []
            want.append(plain.forward(pcfg, pw, s, margins))
            least.append(np.minimum.reduce(margins) if margins else np.full(len(s), np.inf))
        for dtype in ("float32", "bfloat16"):
            # rows up to a sequence's first close call of the router; what follows one is another computation
            safe = [int(np.argmax(m <= MARGIN[dtype])) if (m <= MARGIN[dtype]).any() else len(m) for m in least]
            eng = Engine(load_model(folder, dtype, "cuda:0"), max_tokens=2048, max_seqs=8, page_size=page)
            # one tolerance for the whole case, from the largest logit of all its sequences (a step's few rows may hold small
            # logits only, while the rounding of a bfloat16 model is that of its largest values)
            largest = max(float(np.abs(w).max()) for w in want)
            tol = 2e-5 * max(1.0, largest) if dtype == "float32" else 0.035 * largest + 1e-3

            def compare(got, rows, label):
                """rows: (sequence, position) of each row of got"""
                keep = [r for r, (i, p) in enumerate(rows) if p < safe[i]]
                if keep:
                    g = got[torch.tensor(keep, device=got.device)].float().cpu().double().numpy()
                    w = np.stack([want[rows[r][0]][rows[r][1]] for r in keep])
                    assert np.isfinite(g).all(), f"{dtype}, {label}: non-finite logits; {what}"
                    worst = float(np.abs(g - w).max())
                    assert worst <= tol, f"{dtype}, {label}: max error {worst:.3e} > {tol:.3e} (row {int(np.abs(g - w).max(axis=1).argmax())} of {len(keep)}); {what}"

            slots = [eng.new_sequence() for _ in seqs]
            whole = eng.step(slots, seqs, "all").clone()
            compare(whole, [(i, p) for i, s in enumerate(seqs) for p in range(len(s))], "whole")
            first_row = np.concatenate([[0], np.cumsum(lengths)])
            exact = dtype == "float32"
            for s in slots:
                eng.release(s)
            k = int(rng.integers(1, 12))
            cut = [max(1, len(s) - k) for s in seqs]
            slots = [eng.new_sequence() for _ in seqs]
            eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [[] for _ in seqs])
            for j in range(k):
                live = [i for i, (s, c) in enumerate(zip(seqs, cut)) if c + j < len(s)]
                if not live:
                    break
                got = eng.step([slots[i] for i in live], [[seqs[i][cut[i] + j]] for i in live], "last")
                compare(got, [(i, cut[i] + j) for i in live], f"single tokens, step {j}")
                for r, i in enumerate(live):
                    assert not exact or torch.equal(got[r], whole[first_row[i] + cut[i] + j]), \
                        f"float32 bits of position {cut[i] + j} of sequence {i} differ between a single-token step and the whole prompt; {what}"
            for s in slots:
                eng.release(s)
            slots = [eng.new_sequence() for _ in seqs]
            pos = [0] * len(seqs)
            while True:
                live = [i for i in range(len(seqs)) if pos[i] < len(seqs[i])]
                if not live:
                    break
                toks = [seqs[i][pos[i]:pos[i] + int(rng.integers(1, 30))] for i in live]
                got = eng.step([slots[i] for i in live], toks, "all")
                compare(got, [(i, pos[i] + p) for i, t in zip(live, toks) for p in range(len(t))], f"chunks from {pos}")
                r = 0
                for i, t in zip(live, toks):
                    at = first_row[i] + pos[i]
                    assert not exact or torch.equal(got[r:r + len(t)], whole[at:at + len(t)]), \
                        f"float32 bits of a chunk of {len(t)} at position {pos[i]} of sequence {i} differ from the whole prompt; {what}"
                    r += len(t)
                    pos[i] += len(t)
            for s in slots:
                eng.release(s)
            eng.check_status()
