"""A plain, slow implementation of the Zanelorn decoder, written from its equations: one function
per mechanism, tensors in, tensors out, no kernels, no cache manager, no code shared with the
library.  Everything runs in the dtype of the weights it is given (float64 in the tests), on the
CPU, over a whole sequence at once (position p counts from 0, T tokens, W the width).

    rms(x) = x / sqrt(mean(x^2) + eps);  norm(x, w) = rms(x) * w
    embedding     x_p = c_e E[t_p]
    layer i       x += m norm(mixer(x), w1);  x += m norm(ff(x), w2)  (ff optional);
                  token input: e = Es[t_p][i d : (i+1) d];  y = Wp (gelu_tanh(Wa x) * e);
                  x += m norm(y, ws)
    retention     q, k, v, g = Wq x, Wk x, Wv x, Wg x;  the first R dims of each head of q, k rotated
                  (pairs (i, i + R/2), angle p base^(-2i/R));  k <- k D^(-1/2);
                  S_p = a_h S_(p-1) + k_p v_p^T;  o_p = S_p^T q_p;  o <- rms(o) per head;
                  out = Wo (o * silu(g))
    windowed      q, k, v = Wq x + bq, ..;  q, k <- norm over each head with one weight;  rotation as
    attention     above with every frequency divided by f;  s_ij = (q_i . k_j) c;  j visible from i
                  iff j <= i and (i - j < window or j < first);  softmax;
                  out = Wo (concat_h(o_h) * sigmoid(Wg x))
    selective     [u | z] = Wi x;  u <- silu(causal conv(u) + b);  [r | B | C] = Wx u;
    scan          dt = softplus(Wd r + bd);  A = -exp(A_log);  per channel c, state n:
                  S <- exp(dt_c A[c, n]) S + dt_c u_c B_n;  y_c = sum_n S[c, n] C_n + D_c u_c;
                  out = Wo (y * silu(z))
    parallel      a * windowed_attention(x) + b * selective_scan(x)
    dense ff      Wd gelu(Wu x)  (the erf form)
    routed ff     z = Wr x;  s = softmax(z) over all outputs;  chosen = the `top` largest of s + corr;
                  expert e: Wd_e y,  y = g sigmoid(1.702 g) (u + 1),  g = min(Wg_e x, L),
                  u = clamp(Wu_e x, -L, L);  the last `identity` outputs stand for experts that return
                  x itself;  out = sum_chosen s_e expert_e(x) + sigmoid(Ws x) shared(x)
    output        logits = H norm(x, wf)
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


# ---- rotation ----------------------------------------------------------------------------------
def rotate_half(x: torch.Tensor, dims: int, base: float, divide: float = 1.0) -> torch.Tensor:
    """x [T, heads, D]: the first ``dims`` of every head rotated, pair (i, i + dims/2) at position
    p by the angle p * base^(-2i/dims) / divide."""
    if dims == 0:
        return x
    T = x.shape[0]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) / divide for i in range(half)], dtype=x.dtype)
    ang = torch.arange(T, dtype=x.dtype)[:, None] * freq[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---- mixers ------------------------------------------------------------------------------------
def retention(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, D, Dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = (x @ w[p + "q"].T).view(T, H, D)
    k = (x @ w[p + "k"].T).view(T, H, D)
    v = (x @ w[p + "v"].T).view(T, H, Dv)
    g = x @ w[p + "g"].T
    q = rotate_half(q, rot["dims"], rot["base"])
    k = rotate_half(k, rot["dims"], rot["base"]) * D ** -0.5
    out = torch.zeros(T, H, Dv, dtype=x.dtype)
    for h in range(H):
        S = torch.zeros(D, Dv, dtype=x.dtype)
        for t in range(T):
            S = m["decay"][h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    out = rms_unit(out, eps).reshape(T, H * Dv)
    return (out * silu(g)) @ w[p + "o"].T


def visible(T: int, window: int, first: int) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < window) | (j < first))


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int,
                     first: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence -> [T, H, Dv]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    see = visible(T, window, first)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        kv = h // (H // G)
        s = (q[:, h] @ k[:, kv].T) * scale
        s = s.masked_fill(~see, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, kv]
    return out


def windowed_attention(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping,
                       eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, G, D = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    Dv = m.get("vdim", D)
    q = (x @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (x @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = (x @ w[p + "v"].T + w[p + "v.b"]).view(T, G, Dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    divide = (rot.get("scaling") or {}).get("factor", 1.0)
    q = rotate_half(q, rot["dims"], rot["base"], divide)
    k = rotate_half(k, rot["dims"], rot["base"], divide)
    mask = m.get("mask") or {}
    out = masked_attention(q, k, v, m["scale"], mask.get("size", T + 1), mask.get("keep_first", 0))
    gate = torch.sigmoid(x @ w[p + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ w[p + "o"].T


def selective_scan(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping) -> torch.Tensor:
    T = x.shape[0]
    C, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    uz = x @ w[p + "in"].T
    u, z = uz[:, :C], uz[:, C:]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), u], dim=0)
    conv = torch.zeros(T, C, dtype=x.dtype)
    for j in range(taps):                      # the last column multiplies the current token
        conv = conv + padded[j:j + T] * w[p + "conv"][:, j]
    u = silu(conv + w[p + "conv.b"])
    rbc = u @ w[p + "x"].T
    r, B, Cm = rbc[:, :R], rbc[:, R:R + N], rbc[:, R + N:R + 2 * N]
    dt = softplus(r @ w[p + "dt"].T + w[p + "dt.b"])             # [T, C]
    A = -torch.exp(w[p + "A_log"])                                 # [C, N]
    S = torch.zeros(C, N, dtype=x.dtype)
    y = torch.zeros(T, C, dtype=x.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + w[p + "D"] * u[t]
    return (y * silu(z)) @ w[p + "o"].T


def parallel(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    left = windowed_attention(x, w, p + "left.", m["left"], eps)
    right = selective_scan(x, w, p + "right.", m["right"])
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


# ---- feed-forwards -----------------------------------------------------------------------------
def dense_ff(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_erf(x @ w[p + "up"].T) @ w[p + "down"].T


def clamped_expert(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(x @ w[p + "gate"].T, max=limit)
    u = torch.clamp(x @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, top: int):
    """(chosen [T, top], their weights [T, top], the margin between the last chosen and the first
    left out as a fraction of their scores, per token)."""
    s = torch.softmax(x @ w[p + "router"].T, dim=-1)
    pick = s + w[p + "correction"]
    order = torch.argsort(pick, dim=-1, descending=True, stable=True)
    chosen = order[:, :top]
    ranked = torch.gather(pick, 1, order)
    if ranked.shape[1] > top:
        # relative to the two scores it separates: rounding moves a score by a fraction of itself
        near = torch.gather(s, 1, order[:, top - 1:top + 1]).sum(dim=-1) / 2
        # (small scores count too: the feed-forward's output is normed, and an expert without
        # weights returns the token's whole input, so a weight of a thousandth can be most of it)
        margin = (ranked[:, top - 1] - ranked[:, top]) / near.clamp(min=1e-30)
    else:
        margin = torch.full((x.shape[0],), float("inf"), dtype=x.dtype)
    return chosen, torch.gather(s, 1, chosen), margin


def routed_ff(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping,
              margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    r = mlp["router"]
    n_real = r["experts"]
    chosen, weight, margin = route(x, w, p, r["top"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t]):
            if e >= n_real:
                out[t] += s * x[t]
            else:
                out[t] += s * clamped_expert(x[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(x @ w[p + "shared.sg"].T)                       # [T, 1]
        out = out + gate * clamped_expert(x, w, p + "shared.", mlp["shared"]["limit"])
    return out


def token_side(x: torch.Tensor, tokens: torch.Tensor, w: Mapping[str, torch.Tensor], i: int, dim: int,
               eps: float) -> torch.Tensor:
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e) @ w[f"l{i}.side.proj"].T
    return rms_norm(y, w[f"l{i}.side.norm"], eps)


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens, streams: Optional[List] = None,
            margins: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``streams`` collects x after every layer, ``margins`` the
    routers' margins (a small one means a router's choice is a close call)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "retention":
            y = retention(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel(x, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(y, w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, w, p + "mlp.", mlp, margins)
            x = x + mult * rms_norm(y, w[p + "norm2"], eps)
        if side is not None:
            x = x + mult * token_side(x, tokens, w, i, side["dim"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def forward_sure(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens, least_margin: float) -> torch.Tensor:
    """``forward`` with NaN in the rows of every token for which some router's choice hangs on less
    than ``least_margin``: an implementation that rounds its activations may choose otherwise there,
    rightly, so a comparison leaves those rows out."""
    margins: List[torch.Tensor] = []
    logits = forward(cfg, w, tokens, None, margins).clone()
    for m in margins:
        logits[m < least_margin] = float("nan")
    return logits


def forward_marked(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens, least_margin: float):
    """(logits, sure): ``sure[t]`` is False where some router's choice at token t is a close call."""
    margins: List[torch.Tensor] = []
    logits = forward(cfg, w, tokens, None, margins)
    sure = torch.ones(logits.shape[0], dtype=torch.bool)
    for m in margins:
        sure &= m >= least_margin
    return logits, sure


def generate_greedy(cfg: Mapping, w: Mapping[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, w, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out


def load_folder(folder: str, dtype: torch.dtype = torch.float64):
    """(config.json as a dict, every tensor of model.safetensors in ``dtype``)."""
    import json
    import os
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            weights[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, weights


def load_weights(model, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    """The weights of a library model by name, on the CPU, as ``dtype``."""
    return {n: t.detach().to("cpu").to(dtype) if t.is_floating_point() else t.detach().cpu()
            for n, t in model.export_state_dict().items()}
