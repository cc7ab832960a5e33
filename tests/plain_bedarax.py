"""A plain, slow implementation of the Bedarax decoder, written from its equations: one function
per mechanism, tensors in, tensors out, no kernels, no cache manager, no code shared with the
library.  Everything runs in the dtype of the weights it is given (float64 in the tests), on the
CPU, over a whole sequence at once (position p counts from 0).

    norm               rms(x) = x / sqrt(mean(x^2) + eps);  norm(x, w) = rms(x) * w
    embedding          X_0 = norm(E[t_p], w_e)
    layer i            y = a_i + mixer(norm(a_i, w1));  X_{i+1} = y + ff(norm(y, w2))   (ff optional)
    depth average      a_{i+1} = sum_{j <= i+1} c_i[j] X_j        (a_0 = X_0; a_L feeds the output)
    short convolution  y_t[c] = silu(sum_j K[c][j] x_{t - (T-1-j)}[c]), zeros before the start
    delta rule         per head, S (D x Dv) from zero:  S <- diag(g_t) S  (g_t a number per head, or
                       one per key channel);  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;
                       o_t = S^T q_t;  q, k unit vectors per head, q times D^(-1/2)
    delta mixer        g = exp(-exp(A_h) softplus(Wa u + b));  gate silu(Wg u)
    channel form       g = exp(-exp(A_h) softplus(Wa2 Wa1 u + b)) per key channel; gate
                       sigmoid(Wg2 Wg1 u)
    attention          s^g_ij = (q^g_i . k_j) * scale;  s'^h = sum_g T[h][g] s^g;  j visible from i
                       iff 0 <= i - j < window;  softmax;  v <- (1 - lam) v + lam v_first in every
                       value-mixing layer after the first;  head h's output times sigmoid(Wg u)_h
    PolyNorm           a rms(z) + b rms(z^2) + c rms(z^3) + e over a token's feed-forward values
    routed experts     z = Wr u + br;  the `top` largest; weights softmax over the chosen;
                       expert Wd (silu(Wg u) * (Wu u))
    output             logits = H norm(a_L, wf)
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def unit_vector(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


# ---- short convolution ---------------------------------------------------------------------------
def causal_conv_silu(x: torch.Tensor, kernel: torch.Tensor) -> torch.Tensor:
    """``x`` [n, channels], ``kernel`` [channels, taps]; the last column multiplies the current
    token, the one before it the previous token, and so on; nothing before the first token."""
    n, taps = x.shape[0], kernel.shape[1]
    out = torch.zeros_like(x)
    for t in range(n):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                out[t] += kernel[:, j] * x[s]
    return silu(out)


# ---- the delta rule ------------------------------------------------------------------------------
def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor,
               decay: torch.Tensor) -> torch.Tensor:
    """One head.  q, k [n, D]; v [n, Dv]; beta [n]; decay [n] (a number a token) or [n, D] (a number
    per key channel).  Token by token: decay, correct what the state holds for k towards v, read."""
    n, D = k.shape
    S = torch.zeros((D, v.shape[1]), dtype=q.dtype)
    out = torch.zeros_like(v)
    for t in range(n):
        g = decay[t]
        S = S * (g.reshape(-1, 1) if g.dim() else g)
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(u: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float,
                channel: bool) -> torch.Tensor:
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = u.shape[0]
    q = causal_conv_silu(u @ w[p + "q"].T, w[p + "q.conv"]).reshape(n, G, D)
    k = causal_conv_silu(u @ w[p + "k"].T, w[p + "k.conv"]).reshape(n, G, D)
    v = causal_conv_silu(u @ w[p + "v"].T, w[p + "v.conv"]).reshape(n, H, Dv)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(u @ w[p + "b"].T)                              # [n, H]
    rate = torch.exp(w[p + "A_log"])                                   # [H]
    if channel:
        raw = (u @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]    # [n, H * D]
        decay = torch.exp(-rate.reshape(1, H, 1) * softplus(raw).reshape(n, H, D))
        gate = torch.sigmoid((u @ w[p + "g1"].T) @ w[p + "g2"].T)
    else:
        raw = u @ w[p + "a"].T + w[p + "dt_bias"]                       # [n, H]
        decay = torch.exp(-rate * softplus(raw))
        gate = silu(u @ w[p + "g"].T)
    o = torch.zeros((n, H, Dv), dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        o[:, h] = delta_rule(q[:, g], k[:, g], v[:, h], beta[:, h], decay[:, h])
    o = rms_unit(o, eps) * w[p + "norm"]
    return (o.reshape(n, H * Dv) * gate) @ w[p + "o"].T


# ---- attention with mixed scores -----------------------------------------------------------------
def talking_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, talk: torch.Tensor,
                      q_pos: List[int], scale: float, window: int) -> torch.Tensor:
    """q [nq, H, D]; k [nk, G, D]; v [nk, G, Dv]; key j is at position j, query a at q_pos[a].  All
    heads' scores of a (query, key) pair are mixed by ``talk`` [H, H] before the softmax."""
    nq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((nq, H, v.shape[-1]), dtype=q.dtype)
    for a in range(nq):
        i = q_pos[a]
        lo = max(0, i - window + 1) if window > 0 else 0
        raw = torch.stack([(k[lo:i + 1, h // (H // G)] @ q[a, h]) * scale for h in range(H)])
        mixed = talk @ raw                                              # [H, keys]
        wts = torch.softmax(mixed, dim=-1)
        for h in range(H):
            out[a, h] = wts[h] @ v[lo:i + 1, h // (H // G)]
    return out


def attention_values(u, w, p, m, v_first: Optional[torch.Tensor]) -> torch.Tensor:
    """The values a layer caches: its own, or blended with the first value-mixing layer's."""
    v = u @ w[p + "v"].T
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    return v


def attention_mixer(u, w, p, m, v_first: Optional[torch.Tensor]):
    """Returns (output, the values it used)."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = u.shape[0]
    q = (u @ w[p + "q"].T).reshape(n, H, D)
    k = (u @ w[p + "k"].T).reshape(n, G, D)
    v = attention_values(u, w, p, m, v_first)
    window = (m.get("mask") or {}).get("size", 0)
    o = talking_attention(q, k, v.reshape(n, G, Dv), w[p + "talk"], list(range(n)),
                          float(m["scale"]), window)
    o = o * torch.sigmoid(u @ w[p + "g"].T).reshape(n, H, 1)
    return o.reshape(n, H * Dv) @ w[p + "o"].T, v


# ---- feed-forwards -------------------------------------------------------------------------------
def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    return (coef[0] * rms_unit(z, eps) + coef[1] * rms_unit(z * z, eps)
            + coef[2] * rms_unit(z * z * z, eps) + coef[3])


def dense_ff(y, w, p, eps):
    return poly_norm(y @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def route(y: torch.Tensor, w_router: torch.Tensor, b_router: torch.Tensor, top: int):
    """(indices [n, top], weights [n, top]): the largest logits, softmax over the chosen only."""
    z = y @ w_router.T + b_router
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def route_margin(y: torch.Tensor, w_router: torch.Tensor, b_router: torch.Tensor, top: int):
    """Per token, by how much the last chosen logit leads the first one left out (inf when every
    expert is chosen): a rounding error of that size in the logits changes the choice."""
    z = y @ w_router.T + b_router
    if top >= z.shape[-1]:
        return torch.full((z.shape[0],), float("inf"), dtype=z.dtype)
    ranked, _ = torch.sort(z, dim=-1, descending=True)
    return ranked[:, top - 1] - ranked[:, top]


def routed_ff(y, w, p, spec, margins: Optional[List[torch.Tensor]] = None):
    idx, wts = route(y, w[p + "router"], w[p + "router.b"], spec["router"]["top"])
    if margins is not None:
        margins.append(route_margin(y, w[p + "router"], w[p + "router.b"], spec["router"]["top"]))
    out = torch.zeros((y.shape[0], w[p + "e0.down"].shape[0]), dtype=y.dtype)
    for t in range(y.shape[0]):
        for j in range(idx.shape[1]):
            e = f"{p}e{int(idx[t, j])}."
            hidden = silu(w[e + "gate"] @ y[t]) * (w[e + "up"] @ y[t])
            out[t] += wts[t, j] * (w[e + "down"] @ hidden)
    return out


# ---- the model -----------------------------------------------------------------------------------
def forward(config: Mapping, w: Mapping[str, torch.Tensor], ids: List[int],
            taps: Optional[List[torch.Tensor]] = None,
            margins: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence.  ``taps`` collects the stream after every layer (after
    the depth average), ``margins`` every router's margin per token (``route_margin``)."""
    eps = float(config["norm"]["eps"])
    x = rms_norm(w["embed"][torch.tensor(ids, dtype=torch.long)], w["embed.norm"], eps)
    history = [x]
    v_first = None
    for i, spec in enumerate(config["layers"]):
        p = f"l{i}."
        m = spec["mixer"]
        u = rms_norm(x, w[p + "norm1"], eps)
        if spec["type"] == "attention":
            mixed, v = attention_mixer(u, w, p + "mix.", m, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        else:
            mixed = delta_mixer(u, w, p + "mix.", m, eps, spec["type"] == "channel_delta")
        y = x + mixed
        mlp = spec.get("mlp")
        if mlp is not None:
            u2 = rms_norm(y, w[p + "norm2"], eps)
            y = y + (dense_ff(u2, w, p + "mlp.", eps) if mlp["kind"] == "dense"
                     else routed_ff(u2, w, p + "mlp.", mlp, margins))
        history.append(y)
        c = w[p + "dwa"]
        x = sum(c[j] * history[j] for j in range(i + 2))
        if taps is not None:
            taps.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def forward_sure(config: Mapping, w: Mapping[str, torch.Tensor], ids: List[int],
                 least_margin: float) -> torch.Tensor:
    """``forward`` with NaN in the rows of every token for which some router's choice hangs on
    less than ``least_margin``: an implementation that rounds its activations may choose otherwise
    there, rightly, so a comparison leaves those rows out."""
    margins: List[torch.Tensor] = []
    logits = forward(config, w, ids, None, margins).clone()
    for m in margins:
        logits[m < least_margin] = float("nan")
    return logits


def generate_greedy(config: Mapping, w: Mapping[str, torch.Tensor], prompt: List[int],
                    n_new: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(config, w, ids)[-1]))
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
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights
