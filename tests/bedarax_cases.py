"""Small Bedarax configurations of the tests, each with sizes of its own, and their folders."""
from __future__ import annotations

import json
import os
import tempfile

import torch


def attention(heads, kv, dim, vdim, scale, window, v_mix):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                      "mask": {"size": window}, "v_mix": v_mix}}


def delta(heads, kv, dim, vdim, conv):
    return {"type": "delta",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def channel_delta(heads, kv, dim, vdim, conv, a_rank, g_rank):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                      "a_rank": a_rank, "g_rank": g_rank}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp=None):
    out = dict(mixer)
    out["mlp"] = mlp
    return out


# a delta layer first; grouped query/key heads in every mixer; windows shorter than a page; three
# layers in the blend of values and one outside it; a layer without a feed-forward; one expert a
# token; ranks that differ
BED_A = {
    "architecture": "Bedarax", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "layers": [layer(delta(4, 2, 16, 24, 4), moe(6, 3, 40)),
               layer(attention(4, 2, 16, 24, 0.3, 20, True), dense(48)),
               layer(channel_delta(2, 1, 24, 8, 2, 5, 7)),
               layer(attention(4, 2, 8, 24, 0.4, 7, True), moe(3, 1, 56)),
               layer(attention(3, 3, 8, 8, 0.5, 33, False), dense(72)),
               layer(attention(2, 2, 12, 24, 0.35, 11, True), moe(5, 2, 24))],
}
# a width the tensor-core product does not take; sizes that are multiples of nothing; one head (a
# 1 x 1 mix of scores); windows of exactly a page and of a page and one; a convolution of one tap
# (no convolution state); every expert chosen; one layer in the blend only
BED_B = {
    "architecture": "Bedarax", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
    "layers": [layer(attention(1, 1, 12, 20, 0.4, 64, False), dense(36)),
               layer(channel_delta(3, 3, 10, 14, 1, 3, 9), moe(4, 4, 28)),
               layer(delta(5, 1, 12, 6, 3), moe(7, 2, 20)),
               layer(attention(6, 2, 10, 14, 0.5, 65, True)),
               layer(delta(2, 2, 20, 10, 2), dense(44))],
}
# sizes the tensor-core kernels take; a window longer than a page that is no multiple of one;
# keys of 128 and 256 in the recurrent layers
BED_C = {
    "architecture": "Bedarax", "vocab": 211, "width": 256, "norm": {"eps": 1e-5},
    "layers": [layer(attention(8, 2, 64, 64, 0.125, 100, True), moe(8, 2, 128)),
               layer(delta(4, 2, 64, 128, 4), dense(384)),
               layer(channel_delta(4, 4, 128, 64, 3, 16, 24), moe(8, 2, 128)),
               layer(attention(8, 2, 32, 64, 0.2, 130, True), dense(256)),
               layer(delta(2, 1, 256, 32, 4), moe(16, 4, 64))],
}
# a window that nothing reaches; keys wider than values and the other way round; a model that ends
# in a recurrent layer without a feed-forward
BED_D = {
    "architecture": "Bedarax", "vocab": 173, "width": 128, "norm": {"eps": 1e-6},
    "layers": [layer(channel_delta(2, 2, 48, 40, 4, 8, 8), dense(192)),
               layer(attention(2, 1, 128, 32, 0.09, 1000, True), moe(4, 2, 96)),
               layer(attention(2, 1, 16, 32, 0.25, 150, True), moe(4, 3, 96)),
               layer(channel_delta(4, 1, 32, 32, 2, 12, 4))],
}
CASES = {"A": (BED_A, 21), "B": (BED_B, 22), "C": (BED_C, 23), "D": (BED_D, 24)}


def loud_weights(folder: str, seed: int) -> None:
    """Rewrites the small learned tensors of a folder so that every one of them matters: depth
    weights of both signs and unequal sizes, a score mix far from the identity, blend factors away
    from 0 and 1, decay rates from slow to fast, PolyNorm numbers that differ, a router bias that
    favours some experts."""
    from minfer_b200.weights.safetensors_io import load_all, save_file
    w = load_all(folder)
    gen = torch.Generator().manual_seed(seed)

    def rnd(shape, mean, std):
        return torch.randn(shape, generator=gen) * std + mean

    for name in sorted(w):
        t = w[name]
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "dwa":
            new = rnd(t.shape, 1.0 / t.numel(), 0.5)
        elif leaf == "talk":
            new = torch.eye(t.shape[0]) * 0.7 + rnd(t.shape, 0.0, 0.5)
        elif leaf == "vmix":
            new = rnd(t.shape, 0.45, 0.1)
        elif leaf == "A_log":
            new = rnd(t.shape, -1.0, 1.2)
        elif leaf == "dt_bias":
            new = rnd(t.shape, -1.5, 1.0)
        elif leaf == "act":
            new = rnd(t.shape, 0.5, 0.3)
        elif name.endswith("router.b"):
            new = rnd(t.shape, 0.0, 1.0)
        elif leaf == "conv":
            new = rnd(t.shape, 0.3, 0.5)
        elif name.endswith("mix.norm"):
            new = rnd(t.shape, 0.9, 0.2)
        else:
            continue
        w[name] = new.to(t.dtype)
    save_file(w, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})


def make_folder(name: str, store_dtype: str = "bfloat16", config=None, seed=None) -> str:
    """A folder with seeded weights: matrices N(0, 0.08), norm weights 1 + N(0, 0.05), the small
    learned tensors loud (``loud_weights``)."""
    from minfer_b200.model import write_random_model
    if config is None:
        config, seed = CASES[name]
    folder = tempfile.mkdtemp(prefix=f"minfer_b200_bed{name}_")
    write_random_model(folder, config, seed, store_dtype, norm_std=0.05, weight_std=0.08)
    loud_weights(folder, seed)
    return folder


def drop_ranks(folder: str) -> None:
    """Takes the ranks of the low-rank pairs out of a folder's config.json: the tensors' shapes
    give them."""
    path = os.path.join(folder, "config.json")
    with open(path) as f:
        cfg = json.load(f)
    for entry in cfg["layers"]:
        entry["mixer"].pop("a_rank", None)
        entry["mixer"].pop("g_rank", None)
    with open(path, "w") as f:
        json.dump(cfg, f)
