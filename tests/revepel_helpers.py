"""Shared by the Revepel tests: tiny model folders, engines on them, the plain logits."""
import functools
import os

import torch

import model_helpers as mh
import plain_revepel as plain
import tiny_revepel

# bfloat16 tolerance: 5 % of the largest logit.  The tiny models are 64 to 128 wide, so that few terms average the
# roundings out, and the design squares what it rounds (the experts' activation, scores that scale their inputs) and
# feeds it to recurrences; observed over these tests: up to 2.8 %, about the same whole, in portions and token by token.
BF16_FRACTION = 0.05


def assert_logits(got, want, dtype, what="", bf16_fraction=BF16_FRACTION):
    mh.assert_logits(got, want, dtype, what, bf16_fraction)


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from rust_deeplearning_b200 import write_random_model
    from rust_deeplearning_b200.weights.safetensors_io import WeightFiles, write_safetensors
    cfg, seed = tiny_revepel.config(name)
    folder = os.path.join(mh.tmp_root(), f"tiny_{name}")
    write_random_model(folder, cfg, seed, "bfloat16")
    files = WeightFiles(folder)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    for tensor, index, value in tiny_revepel.ADJUST.get(name.rstrip("x"), ()):
        tensors[tensor].view(-1)[index] = value
    del files
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
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
    return tiny_revepel.config(name)[0]["vocab"]


# A router's choice may flip between number formats where two scores nearly tie; what follows the flip is another
# computation, not a rounding of the same one.  Comparisons in float32 use prompts whose every routed choice, in the
# plain implementation, has a margin rounding cannot move; comparisons in bfloat16 use the configurations in which every
# expert is chosen (names with an x at their end: the same weights).
MARGIN = 1e-4
_LOGITS = {}


def _run_plain(name: str, ids):
    key = (name, tuple(ids))
    if key not in _LOGITS:
        cfg, w = plain_model(name)
        margins = []
        logits = plain.forward(cfg, w, list(ids), None, margins)
        _LOGITS[key] = (logits, min((float(m.min()) for m in margins), default=float("inf")))
    return _LOGITS[key]


def plain_logits(name: str, ids):
    return _run_plain(name, ids)[0]


def name_for(name: str, dtype: str) -> str:
    """The configuration a comparison in `dtype` runs on."""
    return name if dtype == "float32" else name + "x"


@functools.lru_cache(maxsize=None)
def prompt(name, seed, n):
    """n token ids from the seed; drawn again (seed + 1000, ...) while a routed choice of the plain implementation is a
    close call."""
    for attempt in range(12):
        ids = mh.prompt(seed + 1000 * attempt, n, vocab(name))
        if name.endswith("x") or _run_plain(name, ids)[1] > MARGIN:
            return ids
    raise AssertionError("no prompt with safe routing margins found")
