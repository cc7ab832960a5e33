"""Random Zanelorn configurations (sizes, order of layers, windows, kept tokens, routers, constants
drawn from a seed): the engine against the plain implementation, whole prompts, a batch of two,
the last tokens one by one and portions of a random size, in both precisions."""
import random

import pytest
import torch

import plain_zanelorn as P
from helpers import random_ids
from test_zanelorn_engine_gpu import LEAST_MARGIN, Plain
from test_zanelorn_engine_gpu import _close as _close_rows
from zanelorn_cases import make_folder

pytestmark = pytest.mark.gpu


def _close(got, want, dtype):
    """The bounds of the engine tests, wider where the drawn sizes make the design's output norms
    touchier than any real model's: a retention head of 8 keys or values, a state of one number a
    channel or a window of one position leave a sum or a norm a handful of numbers, and a token whose
    handful nearly cancels has its float32 rounding scaled up several times (seen over 130 seeds: up to
    1e-4 of the largest logit with heads of 8 and wider, 4e-4 with heads of 4, against 2e-5)."""
    _close_rows(got, want, dtype, float32_bound=1e-4, few=0.2)


def divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def make(rng):
    """A configuration drawn from ``rng``: 1 to 6 layers of either kind in any order, sizes that are
    multiples of nothing, with or without every optional key."""
    width = rng.choice([40, 48, 64, 96, 100, 128, 160, 192, 256, 320])
    layers = []
    for _ in range(rng.randint(1, 6)):
        if rng.random() < 0.5:
            heads = rng.randint(1, 5)
            dim = rng.choice([8, 10, 16, 32, 48, 64, 96, 128, 132])
            m = {"heads": heads, "dim": dim, "vdim": rng.choice([dim, 8, 9, 16, 40, 64, 128]),
                 "decay": [rng.choice([1.0, 0.999, 0.99, 0.95, 0.8, 0.5]) for _ in range(heads)]}
            if rng.random() < 0.8:
                m["rot"] = {"base": rng.choice([1e4, 5e5, 2e6]), "dims": rng.choice([dim, 2 * rng.randint(1, dim // 2)])}
            layer = {"type": "retention", "mixer": m}
        else:
            heads = rng.choice([1, 2, 3, 4, 6, 8])
            dim = rng.choice([8, 10, 16, 24, 32, 48, 64, 64, 128, 128])
            left = {"heads": heads, "kv_heads": rng.choice(divisors(heads)), "dim": dim,
                    "vdim": rng.choice([dim, dim, dim, 8, 12, 32, 64]),
                    "scale": rng.choice([dim ** -0.5, 0.125, 0.3]),
                    "rot": {"base": rng.choice([1e4, 3e5]), "dims": rng.choice([dim, 2 * rng.randint(1, dim // 2)])}}
            if rng.random() < 0.6:
                left["rot"]["scaling"] = {"factor": rng.choice([1.0, 2.0, 2.5, 8.0])}
            if rng.random() < 0.15:
                del left["rot"]                     # no rotation at all
            if rng.random() < 0.15:
                left["vdim"] = dim
                del left["vdim"]                    # values as wide as keys
            if rng.random() < 0.15:
                left["kv_heads"] = heads
                del left["kv_heads"]                # a key/value head for every head
            if rng.random() < 0.85:
                left["mask"] = {"size": rng.choice([1, 2, 7, 63, 64, 65, 100, 140, 200, 300])}
                if rng.random() < 0.7:
                    left["mask"]["keep_first"] = rng.choice([0, 1, 2, 5, 8, 33, 64, 70])
            right = {"inner": rng.choice([8, 20, 48, 64, 100, 192, 384]), "state": rng.choice([1, 4, 5, 8, 16, 24, 64]),
                     "dt_rank": rng.choice([1, 3, 4, 8, 12, 16]), "conv": rng.randint(1, 5)}
            m = {"left": left, "right": right}
            if rng.random() < 0.8:
                m["left_scale"], m["right_scale"] = rng.choice([0.5, 0.8, 1.0, 1.3]), rng.choice([0.6, 0.9, 1.0])
            layer = {"type": "parallel", "mixer": m}
        kind = rng.choice(["none", "dense", "dense", "moe", "moe"])
        if kind == "none":
            layer["mlp"] = None
        elif kind == "dense":
            layer["mlp"] = {"kind": "dense", "ff": rng.choice([8, 24, 40, 64, 136, 320])}
        else:
            experts, identity = rng.randint(1, 12), rng.choice([0, 0, 1, 2, 3])
            layer["mlp"] = {"kind": "moe", "expert": {"ff": rng.choice([8, 16, 24, 64, 96]), "limit": rng.choice([0.7, 1.5, 4.0])},
                            "router": {"experts": experts, "identity": identity,
                                       "top": rng.randint(1, min(8, experts + identity))},
                            "shared": rng.choice([None, {"ff": rng.choice([8, 40, 128]), "limit": rng.choice([0.9, 2.0])}])}
        layers.append(layer)
    cfg = {"architecture": "Zanelorn", "vocab": rng.randint(50, 700), "width": width,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.8:
        cfg["residual_mult"] = rng.choice([0.4, 0.7, 1.0, 1.4])
    if rng.random() < 0.8:
        cfg["embedding"] = {"scale": rng.choice([1.0, 4.0, 11.0, 20.0])}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": rng.choice([1, 4, 8, 16, 24])}
    return cfg


@pytest.mark.parametrize("seed", [2, 5, 11, 23, 27, 31, 34, 47])
def test_random_configuration(seed):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    rng = random.Random(seed)
    cfg = make(rng)
    folder = make_folder("r", "bfloat16", cfg, seed)
    c, w = P.load_folder(folder)
    n = rng.choice([1, 5, 37, 70, 130, 210])
    ids = random_ids(n, cfg["vocab"], seed)
    ids2 = random_ids(rng.randint(1, 60), cfg["vocab"], seed + 1000)
    cut = max(1, n - rng.randint(1, 24))
    portion = rng.choice([2, 3, 50, 64, 170])
    for dtype in ("float32", "bfloat16"):
        want = Plain(*P.forward_marked(c, w, ids, LEAST_MARGIN[dtype]))
        want2 = Plain(*P.forward_marked(c, w, ids2, LEAST_MARGIN[dtype]))
        eng = Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=2048)
        s = eng.acquire()
        got = eng.step([s], [ids], [list(range(n))])
        eng.release(s)
        _close(got, want, dtype)
        a, b = eng.acquire(), eng.acquire()
        out = eng.step([a, b], [ids[:cut], ids2], [list(range(cut)), list(range(len(ids2)))])
        _close(out[cut:], want2, dtype)
        eng.release(b)
        rows = [out[:cut]] + [eng.step([a], [[ids[t]]], [[0]]) for t in range(cut, n)]
        eng.release(a)
        _close(torch.cat(rows), want, dtype)
        s = eng.acquire()
        rows = []
        for lo in range(0, n, portion):
            part = ids[lo:lo + portion]
            rows.append(eng.step([s], [part], [list(range(len(part)))]))
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
        eng.check_status()
        eng.cache.check_canaries()
