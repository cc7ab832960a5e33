"""Small Zanelorn configurations of the tests, each with sizes of its own, and their folders."""
from __future__ import annotations

import os
import tempfile

import torch


def _retention(heads, dim, vdim, decay, rot_dims, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "retention", "mixer": m}


def _parallel(heads, kv, dim, vdim, scale, window, keep, rot_dims, factor, inner, state, rank, conv,
              ls, rs, base=50000.0):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": rot_dims}}
    if factor is not None:
        left["rot"]["scaling"] = {"factor": factor}
    if window is not None:
        left["mask"] = {"size": window, "keep_first": keep}
    return {"type": "parallel",
            "mixer": {"left": left, "right": {"inner": inner, "state": state, "dt_rank": rank, "conv": conv},
                      "left_scale": ls, "right_scale": rs}}


def _dense(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff})


def _moe(layer, experts, identity, top, ff, limit, shared):
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
           "router": {"experts": experts, "identity": identity, "top": top},
           "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}
    return dict(layer, mlp=mlp)


def _bare(layer):
    return dict(layer, mlp=None)


# every mixer and feed-forward once; odd sizes everywhere; a window shorter than a page with kept
# first tokens; a rotation of the whole retention head and of half an attention head
ZAN_A = {
    "architecture": "Zanelorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "residual_mult": 0.6, "embedding": {"scale": 3.0}, "token_side": {"dim": 8},
    "layers": [_dense(_parallel(4, 2, 16, 24, 0.3, 20, 3, 8, 2.0, 48, 8, 5, 3, 0.7, 1.2), 48),
               _moe(_retention(3, 12, 20, [0.9, 0.97, 0.995], 12), 5, 1, 2, 24, 1.2, (40, 0.9)),
               _bare(_retention(2, 16, 8, [0.5, 0.999], 6)),
               _moe(_parallel(3, 3, 12, 12, 0.5, 65, 1, 12, None, 40, 24, 3, 2, 1.0, 0.5), 4, 2, 3, 16, 0.8, None)],
}
# no token input, no embedding scale, no residual factor; a width the tensor-core product does not
# take; attention without a mask and with a window that keeps nothing (a ring); retention without a
# rotation; a router without identity or shared experts that picks one expert; one tap; more kept
# tokens than the window is long
ZAN_B = {
    "architecture": "Zanelorn", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
    "layers": [_moe(_retention(5, 10, 14, [0.8, 0.9, 0.95, 0.99, 1.0], None), 3, 0, 1, 28, 2.0, None),
               _dense(_parallel(2, 1, 20, 12, 0.4, None, 0, 10, 3.0, 36, 5, 7, 1, 0.9, 0.8), 36),
               _bare(_parallel(5, 5, 12, 16, 0.3, 64, 0, 4, None, 52, 40, 2, 4, 1.1, 1.0)),
               _dense(_parallel(3, 1, 8, 8, 0.6, 9, 30, 8, 1.5, 24, 12, 4, 5, 0.5, 0.5), 20)],
}
# sizes the tensor-core kernels take: keys and values of 64; a window longer than a page that is
# no multiple of one, with kept first tokens; retention keys of 64 with values of 128
ZAN_C = {
    "architecture": "Zanelorn", "vocab": 211, "width": 256, "norm": {"eps": 1e-5},
    "residual_mult": 0.8, "embedding": {"scale": 8.0}, "token_side": {"dim": 16},
    "layers": [_moe(_parallel(4, 1, 64, 64, 0.11, 100, 5, 32, 2.5, 128, 16, 8, 4, 0.9, 0.7, 300000.0),
                    8, 2, 3, 64, 1.5, (128, 1.0)),
               _dense(_retention(2, 64, 128, [0.96875, 0.998], 64, 2000000.0), 384),
               _dense(_parallel(8, 4, 64, 64, 0.14, 130, 0, 64, None, 96, 8, 4, 2, 1.0, 1.0), 192)],
}
# keys and values of 128 (the tensor-memory kernel's other size), kept tokens beyond the first
# page, two retention layers in a row, a state of 64 per channel
ZAN_D = {
    "architecture": "Zanelorn", "vocab": 173, "width": 128, "norm": {"eps": 1e-6},
    "residual_mult": 1.3, "token_side": {"dim": 4},
    "layers": [_dense(_retention(1, 128, 64, [0.99], 32), 160),
               _bare(_retention(4, 32, 32, [0.7, 0.9, 0.97, 0.99], 32)),
               _dense(_parallel(2, 1, 128, 128, 0.09, 40, 70, 128, 8.0, 64, 64, 6, 4, 0.8, 0.9, 500000.0), 96)],
}
CASES = {"A": (ZAN_A, 41), "B": (ZAN_B, 42), "C": (ZAN_C, 43), "D": (ZAN_D, 44)}


def loud_weights(folder: str, seed: int) -> None:
    """Rewrites the small learned tensors of a folder so that every one of them matters: routers
    that decide clearly, corrections that change some choices, biases, decays from slow to fast,
    step sizes of several magnitudes, head norms away from 1."""
    from minfer_b200.weights.safetensors_io import load_all, save_file
    w = load_all(folder)
    gen = torch.Generator().manual_seed(seed)

    def rnd(shape, mean, std):
        return torch.randn(shape, generator=gen) * std + mean

    for name in sorted(w):
        t = w[name]
        if name.endswith("mlp.router"):
            new = rnd(t.shape, 0.0, 2.0)
        elif name.endswith("mlp.correction"):
            new = rnd(t.shape, 0.0, 0.05)
        elif name.endswith("shared.sg"):
            new = rnd(t.shape, 0.0, 0.3)
        elif name.endswith((".q.b", ".k.b", ".v.b", "conv.b")):
            new = rnd(t.shape, 0.0, 0.3)
        elif name.endswith((".q.norm", ".k.norm")):
            new = rnd(t.shape, 1.0, 0.2)
        elif name.endswith("A_log"):
            new = rnd(t.shape, -0.5, 1.0)
        elif name.endswith("dt.b"):
            new = rnd(t.shape, -1.5, 1.0)
        elif name.endswith("right.dt"):
            new = rnd(t.shape, 0.0, 0.4)
        elif name.endswith("right.conv"):
            new = rnd(t.shape, 0.3, 0.5)
        elif name.endswith("right.D"):
            new = rnd(t.shape, 1.0, 0.3)
        else:
            continue
        w[name] = new.to(t.dtype)
    save_file(w, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})


def make_folder(name: str, store: str = "bfloat16", cfg=None, seed=None) -> str:
    """A folder with seeded weights: matrices N(0, 0.08), norm weights 1 + N(0, 0.05), the small
    learned tensors loud (``loud_weights``)."""
    from minfer_b200.model import write_random_model
    if cfg is None:
        cfg, seed = CASES[name]
    folder = tempfile.mkdtemp(prefix=f"minfer_b200_zan{name}_")
    write_random_model(folder, cfg, seed, store, norm_std=0.05, weight_std=0.08)
    loud_weights(folder, seed)
    return folder
