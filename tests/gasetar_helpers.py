"""Shared by the Gasetar tests: tiny model folders, engines on them, the plain logits, prompts whose routing
does not hang on a close call."""
import functools
import os

import numpy as np

import model_helpers as mh
import plain_gasetar as plain
import tiny_gasetar

assert_logits = mh.assert_logits


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from rust_deeplearning_b200 import write_random_model
    cfg, seed = tiny_gasetar.config(name)
    folder = os.path.join(mh.tmp_root(), f"tiny_{name}")
    write_random_model(folder, cfg, seed, "bfloat16")
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return plain.load_folder(model_folder(name))


@functools.lru_cache(maxsize=None)
def loaded_model(name: str, dtype: str):
    from rust_deeplearning_b200 import load_model
    return load_model(model_folder(name), dtype, "cuda:0")


def engine(name: str, dtype: str, **kw):
    from rust_deeplearning_b200 import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine(loaded_model(name, dtype), **kw)


def vocab(name):
    return tiny_gasetar.config(name)[0]["vocab"]


_LOGITS = {}


def plain_logits(name: str, ids):
    key = (name, tuple(ids))
    if key not in _LOGITS:
        cfg, w = plain_model(name)
        _LOGITS[key] = plain.forward(cfg, w, list(ids))
    return _LOGITS[key]


# A router's choice may flip between number formats where two choice scores nearly tie; what follows the flip is
# another computation, not a rounding of the same one.  Prompts for comparisons are therefore built so that, in the
# plain implementation, every routed layer's margin at every token exceeds what rounding can move.
MARGIN = {"float32": 1e-4, "bfloat16": 5e-2}


@functools.lru_cache(maxsize=None)
def prompt(name: str, seed: int, n: int, dtype: str = "bfloat16"):
    """n token ids, built eight at a time: a piece is drawn again until the margins of its tokens suffice
    (a token's margin depends on the tokens before it only)."""
    cfg, w = plain_model(name)
    rng = np.random.default_rng(seed)
    ids = []
    while len(ids) < n:
        k = min(8, n - len(ids))
        for _ in range(200):
            piece = [int(v) for v in rng.integers(0, cfg["vocab"], size=k)]
            margins = []
            plain.forward(cfg, w, ids + piece, margins)
            if all(float(m[len(ids):].min()) > MARGIN[dtype] for m in margins):
                break
        else:
            raise AssertionError("no piece with a safe routing margin found")
        ids += piece
    return ids
