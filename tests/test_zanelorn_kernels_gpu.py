"""The kernels of the Zanelorn mechanisms, each alone against its plain function
(``tests/plain_zanelorn.py``): heads normed and rotated one by one; the retention recurrence and
the selective scan over cuts of every size with the state carried in slots; the output-norm add;
the activations; the scored router with ties and a correction; experts with the clamped
activation and experts without weights; and attention with a window that keeps the first tokens,
with marked keys just inside and just outside the window, among the kept tokens and just beyond
them, far back and at page borders, in prompts and over the paged cache."""
import math

import pytest
import torch

import plain_zanelorn as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err < tol, err


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ---- heads prepared one by one -------------------------------------------------------------------
@pytest.mark.parametrize("nh,nk,qw,vw,rot,norm", [(3, 3, 12, 20, 12, False), (4, 2, 16, 24, 8, True),
                                                  (8, 2, 64, 64, 32, True), (2, 2, 10, 6, 0, True),
                                                  (1, 1, 128, 128, 128, False)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_head_prepare(nh, nk, qw, vw, rot, norm, dt):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(nh * 100 + qw)
    n, pad = 37, 5
    width = pad + nh * qw + nk * qw + nk * vw + 3
    proj = torch.randn(n, width, generator=g)
    pos = torch.randint(0, 5000, (n,), generator=g)
    qn, kn = (torch.rand(qw, generator=g) + 0.5, torch.rand(qw, generator=g) + 0.5) if norm else (None, None)
    base, divide, eps = 12345.0, 2.5, 1e-5
    inv = torch.tensor([base ** (-2.0 * i / rot) / divide for i in range(rot // 2)], dtype=torch.float64) if rot else None
    q = torch.empty(n, nh, qw, dtype=dt, device=DEV)
    k = torch.empty(n, nk, qw, dtype=dt, device=DEV)
    v = torch.empty(n, nk, vw, dtype=dt, device=DEV)
    q_off, k_off, v_off = pad, pad + nh * qw, pad + (nh + nk) * qw
    K.head_prepare(proj.to(DEV), _i32(pos.tolist()), _i32([0] * n), _i32([0]), q, k, v, None, None, None, 0, 0,
                   q_off=q_off, n_heads=nh, q_width=qw, k_off=k_off, n_kv=nk, k_width=qw, v_off=v_off,
                   v_width=vw, q_norm=None if qn is None else qn.to(DEV), k_norm=None if kn is None else kn.to(DEV),
                   eps=eps, inv_freq=None if inv is None else inv.to(DEV), rot_dims=rot, rot_style=0,
                   rot_magnitude=1.0, q_mul=1.0, k_mul=0.37, status=_status())
    p64 = proj.double()

    def plain(seg, heads, w, mul):
        x = seg.reshape(n, heads, qw)
        if w is not None:
            x = P.rms_norm(x, w.double(), eps)
        out = torch.empty_like(x)
        for t in range(n):              # the plain rotation counts positions from 0: one token at a time
            many = x[t:t + 1].repeat(int(pos[t]) + 1, 1, 1)
            out[t] = P.rotate_half(many, rot, base, divide)[-1] if rot else x[t]
        return out * mul

    tol = 2e-6 if dt == torch.float32 else 6e-3
    small = pos.clone()
    _close(q, plain(p64[:, q_off:k_off], nh, qn, 1.0), tol)
    _close(k, plain(p64[:, k_off:v_off], nk, kn, 0.37), tol)
    _close(v, p64[:, v_off:v_off + nk * vw].reshape(n, nk, vw), tol)


# ---- the retention recurrence ------------------------------------------------------------------------
def _plain_retention(q, k, v, decay, S):
    """q, k [T, H, D], v [T, H, Dv], S [H, D, Dv] (changed in place) -> o [T, H, Dv]."""
    T, H = q.shape[0], q.shape[1]
    o = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o


@pytest.mark.parametrize("H,D,Dv", [(3, 12, 20), (2, 64, 128), (1, 128, 33), (5, 7, 5), (2, 256, 40)])
def test_retention_scan_over_cuts_and_slots(H, D, Dv):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(D + Dv)
    decay = [1.0, 0.5, 0.97, 0.999, 0.9][:H]
    lens = [53, 1, 20]
    slots = [4, 0, 2]
    state = torch.randn(6, H, Dv, D, generator=g).to(DEV)             # stale values in every slot
    state[slots] = 0.0
    seqs = [(torch.randn(n, H, D, generator=g), torch.randn(n, H, D, generator=g) * D ** -0.5,
             torch.randn(n, H, Dv, generator=g)) for n in lens]
    want = [_plain_retention(q.double(), k.double(), v.double(), decay, torch.zeros(H, D, Dv, dtype=torch.float64))
            for q, k, v in seqs]
    got = [[] for _ in lens]
    at = [0] * len(lens)
    cuts = [1, 2, 17, 16, 3, 15, 40]                                   # tokens a row brings per step
    for cut in cuts:
        rows = [b for b in range(len(lens)) if at[b] < lens[b]]
        if not rows:
            break
        take = [min(cut, lens[b] - at[b]) for b in rows]
        q = torch.cat([seqs[b][0][at[b]:at[b] + t] for b, t in zip(rows, take)]).to(DEV)
        k = torch.cat([seqs[b][1][at[b]:at[b] + t] for b, t in zip(rows, take)]).to(DEV)
        v = torch.cat([seqs[b][2][at[b]:at[b] + t] for b, t in zip(rows, take)])
        n = q.shape[0]
        proj = torch.randn(n, 9 + H * Dv, generator=g)                 # v sits behind 9 other columns
        proj[:, 9:] = v.reshape(n, H * Dv)
        cu = [0]
        for t in take:
            cu.append(cu[-1] + t)
        out = torch.empty(n, H * Dv, device=DEV)
        K.retention_scan(q.contiguous(), k.contiguous(), proj.to(DEV), 9,
                         torch.tensor(decay, dtype=torch.float32, device=DEV), state, _i32(cu),
                         _i32([slots[b] for b in rows]), out, len(rows))
        for i, (b, t) in enumerate(zip(rows, take)):
            got[b].append(out[cu[i]:cu[i + 1]].reshape(t, H, Dv).cpu())
            at[b] += t
    for b in range(len(lens)):
        _close(torch.cat(got[b]), want[b], 2e-5)
    assert float(state[1].abs().max()) > 0                              # slots not in use keep their values


# ---- the selective scan ----------------------------------------------------------------------------
def _plain_scan(u, dt_raw, B, Cm, z, a_log, d_skip, S):
    T = u.shape[0]
    y = torch.zeros_like(u)
    A = -torch.exp(a_log)
    for t in range(T):
        dt = P.softplus(dt_raw[t])
        S.copy_(torch.exp(dt[:, None] * A) * S + (dt * u[t])[:, None] * B[t][None, :])
        y[t] = S @ Cm[t] + d_skip * u[t]
    return y * P.silu(z)


@pytest.mark.parametrize("C,N", [(48, 8), (40, 20), (33, 5), (128, 16), (20, 64), (8, 200)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_selective_scan_over_cuts_and_slots(C, N, dt):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(C + N)
    lens, slots = [45, 2, 19], [1, 3, 0]
    a_log = torch.randn(C, N, generator=g) * 0.5
    d_skip = torch.randn(C, generator=g)
    state = torch.randn(5, C, N, generator=g).to(DEV)
    state[slots] = 0.0
    R = 3
    seqs = []
    for n in lens:
        seqs.append({"u": torch.randn(n, C, generator=g), "dt": torch.randn(n, C, generator=g),
                     "bc": torch.randn(n, R + 2 * N, generator=g), "z": torch.randn(n, 2 * C, generator=g)})
    want = [_plain_scan(s["u"].double(), s["dt"].double(), s["bc"][:, R:R + N].double(),
                        s["bc"][:, R + N:].double(), s["z"][:, C:].double(), a_log.double(), d_skip.double(),
                        torch.zeros(C, N, dtype=torch.float64)) * 0.75 for s in seqs]
    got = [[] for _ in lens]
    at = [0] * len(lens)
    for cut in [1, 2, 15, 16, 17, 1, 40]:
        rows = [b for b in range(len(lens)) if at[b] < lens[b]]
        if not rows:
            break
        take = [min(cut, lens[b] - at[b]) for b in rows]
        cat = {key: torch.cat([seqs[b][key][at[b]:at[b] + t] for b, t in zip(rows, take)]).contiguous().to(DEV)
               for key in ("u", "dt", "bc", "z")}
        cu = [0]
        for t in take:
            cu.append(cu[-1] + t)
        out = torch.empty(cu[-1], C, dtype=dt, device=DEV)
        K.selective_scan(cat["u"], cat["dt"], cat["bc"], R, R + N, cat["z"], C, a_log.to(DEV), d_skip.to(DEV),
                         state, _i32(cu), _i32([slots[b] for b in rows]), out, len(rows), mul=0.75)
        for i, (b, t) in enumerate(zip(rows, take)):
            got[b].append(out[cu[i]:cu[i + 1]].float().cpu())
            at[b] += t
    for b in range(len(lens)):
        _close(torch.cat(got[b]), want[b], 3e-5 if dt == torch.float32 else 6e-3)


# ---- row-wise kernels ---------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [64, 100, 257])
def test_norm_add_plain_and_from_partial_sums(width):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(width)
    n = 13
    h, y, w = torch.randn(n, width, generator=g), torch.randn(n, width, generator=g) * 3, torch.rand(width, generator=g) + 0.5
    want = h.double() + 0.7 * P.rms_norm(y.double(), w.double(), 1e-6)
    hd = h.clone().to(DEV)
    K.norm_add(hd, y.to(DEV), w.to(DEV), 1e-6, 0.7)
    _close(hd, want, 2e-6)
    parts = torch.randn(3, n, width, generator=g)
    bias = torch.randn(width, generator=g)
    want = h.double() + 1.3 * P.rms_norm(parts.double().sum(0) + bias.double(), w.double(), 1e-5)
    hd = h.clone().to(DEV)
    K.norm_add(hd, parts.to(DEV), w.to(DEV), 1e-5, 1.3, bias=bias.to(DEV))
    _close(hd, want, 2e-6)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_activations_and_gates(dt):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(5)
    tol = 2e-6 if dt == torch.float32 else 6e-3
    n, ff = 19, 37
    z = torch.randn(n, ff, generator=g) * 3
    out = torch.empty(n, ff, dtype=dt, device=DEV)
    K.unary_act(z.to(DEV), out, "gelu")
    _close(out, P.gelu_erf(z.double()), tol)
    gu = torch.randn(n, 2 * ff, generator=g) * 2
    rg = torch.randn(n, 5, generator=g)
    K.gated_act(gu.to(DEV), out, "clamped_swish", 1.1, 1.702, row_gate=rg.to(DEV)[:, 3])
    gg = torch.clamp(gu[:, :ff].double(), max=1.1)
    uu = torch.clamp(gu[:, ff:].double(), -1.1, 1.1)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1) * torch.sigmoid(rg[:, 3:4].double())
    _close(out, want, tol)
    assert float(gu[:, :ff].max()) > 1.1 and float(gu[:, ff:].min()) < -1.1     # the clamps did work
    K.gated_act(gu.to(DEV), out, "clamped_swish", 0.4, 1.702)
    gg, uu = torch.clamp(gu[:, :ff].double(), max=0.4), torch.clamp(gu[:, ff:].double(), -0.4, 0.4)
    _close(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1), tol)
    # the output gate of attention, with a constant
    o = torch.randn(n, ff, generator=g).to(dt)
    gate = torch.randn(n, ff + 9, generator=g)
    od = o.clone().to(DEV)
    K.gate_mul(od, gate.to(DEV), 9, 0.8)
    _close(od, o.double() * torch.sigmoid(gate[:, 9:].double()) * 0.8, tol)
    # per-head unit norm times silu of a gate
    H, Dv = 3, 20
    oo = torch.randn(n, H * Dv, generator=g) * 5
    gt = torch.randn(n, 4 + H * Dv, generator=g)
    res = torch.empty(n, H * Dv, dtype=dt, device=DEV)
    K.unit_norm_gate(oo.to(DEV), gt.to(DEV), 4, res, H, 1e-6, "silu", 1.25)
    want = P.rms_unit(oo.double().reshape(n, H, Dv), 1e-6).reshape(n, H * Dv) * P.silu(gt[:, 4:].double()) * 1.25
    _close(res, want, tol)
    # a per-token input looked up by token id, all rows and only some
    table = torch.randn(50, 24, generator=g).to(dt)
    ids = torch.randint(0, 50, (n,), generator=g)
    a = torch.randn(n, 8, generator=g)
    res = torch.empty(n, 8, dtype=dt, device=DEV)
    st = _status()
    K.table_gate(a.to(DEV), table.to(DEV), 16, _i32(ids.tolist()), None, res, st)
    _close(res, P.gelu_tanh(a.double()) * table.double()[ids][:, 16:24], tol)
    rows = [7, 0, 18]
    res3 = torch.empty(3, 8, dtype=dt, device=DEV)
    K.table_gate(a[:3].contiguous().to(DEV), table.to(DEV), 8, _i32(ids.tolist()), _i32(rows), res3, st)
    _close(res3, P.gelu_tanh(a[:3].double()) * table.double()[ids[rows]][:, 8:16], tol)
    assert int(st.item()) == 0


# ---- the router and the experts ----------------------------------------------------------------------
@pytest.mark.parametrize("outputs,top", [(6, 2), (20, 5), (3, 1), (40, 8), (5, 5)])
def test_scored_router(outputs, top):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(outputs)
    n = 64
    z = torch.randn(n, outputs + 1, generator=g) * 2               # one more column rides along
    z[0, :outputs] = 0.0                                           # all tied: the lowest indices win
    z[1, :outputs] = torch.arange(outputs).float() * 1e-3          # nearly tied: the correction decides
    corr = torch.randn(outputs, generator=g) * 0.05
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, device=DEV)
    K.moe_route_scored(z.to(DEV), corr.to(DEV), idx, wts, top, outputs)
    w = {"router": torch.eye(outputs).double(), "correction": corr.double()}
    chosen, weight, margin = P.route(z[:, :outputs].double(), w, "", top)
    sure = margin > 1e-4
    sure[0] = False
    assert int(sure.sum()) > n // 2
    assert torch.equal(idx.cpu().long()[sure], chosen[sure])
    _close(wts.cpu()[sure], weight[sure], 1e-5)
    zero = torch.zeros(outputs, device=DEV)
    K.moe_route_scored(z.to(DEV), zero, idx, wts, top, outputs)
    assert idx[0].tolist() == list(range(top))
    assert abs(float(wts[0, 0]) - 1.0 / outputs) < 1e-6
    K.moe_route_scored(z.to(DEV), None, idx, wts, top, outputs)
    assert idx[0].tolist() == list(range(top))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_experts_with_the_clamped_activation_and_experts_without_weights(dt):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(9)
    n, width, ff, experts, identity, top = 11, 48, 24, 4, 2, 3
    x = torch.randn(n, width, generator=g).to(dt)
    wg = (torch.randn(experts, ff, width, generator=g) * 0.3).to(dt)
    wu = (torch.randn(experts, ff, width, generator=g) * 0.3).to(dt)
    wd = (torch.randn(experts, width, ff, generator=g) * 0.3).to(dt)
    idx = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(n)]).int()
    wts = torch.rand(n, top, generator=g)
    h = torch.randn(n, width, generator=g)
    hd = h.clone().to(DEV)
    hidden = torch.empty(n, top, ff, dtype=dt, device=DEV)
    K.moe_experts(x.to(DEV), wg.to(DEV), wu.to(DEV), wd.to(DEV), idx.to(DEV), wts.to(DEV), hidden, hd,
                  "clamped_swish", 0.9, 1.702)
    want = h.double().clone()
    for t in range(n):
        for k in range(top):
            e = int(idx[t, k])
            if e >= experts:
                want[t] += float(wts[t, k]) * x[t].double()
            else:
                w = {"gate": wg[e].double(), "up": wu[e].double(), "down": wd[e].double()}
                want[t] += float(wts[t, k]) * P.clamped_expert(x[t:t + 1].double(), w, "", 0.9)[0]
    assert int((idx >= experts).sum()) > 0
    _close(hd, want, 1e-5 if dt == torch.float32 else 1e-2)


# ---- attention with a window that keeps the first tokens ------------------------------------------
DIM, BIG = 3, 30.0


def _marked(n, nh, nk, hd, vd, marks, g, dt):
    """Queries of head 0 and the keys at ``marks`` point along DIM: a marked key's score stands out,
    so a query's output is the value of the marked key it sees (the latest one)."""
    q = torch.randn(n, nh, hd, generator=g)
    k = torch.randn(n, nk, hd, generator=g)
    v = torch.randn(n, nk, vd, generator=g)
    q[:, 0] = 0.0
    q[:, 0, DIM] = BIG
    for rank, j in enumerate(marks):
        k[j, 0] = 0.0
        k[j, 0, DIM] = BIG * (1.0 + 0.2 * rank)          # a later mark outshines an earlier one
    return q.to(dt), k.to(dt), v.to(dt)


@pytest.mark.parametrize("hd,vd,nh,nk,window,keep", [(16, 24, 4, 2, 20, 3), (64, 64, 8, 2, 100, 7),
                                                     (12, 12, 3, 3, 65, 1), (8, 8, 3, 1, 9, 30),
                                                     (128, 128, 2, 1, 40, 70), (64, 64, 2, 2, 64, 64)])
@pytest.mark.parametrize("dt,kernel", [(torch.float32, "any"), (torch.bfloat16, "any"),
                                       (torch.bfloat16, "mma"), (torch.bfloat16, "generic")])
def test_kept_first_tokens_and_the_window_edge(hd, vd, nh, nk, window, keep, dt, kernel, monkeypatch):
    """Marks: the last kept token (keep - 1), the first one not kept (keep), and one in the middle.
    Far queries see mark keep - 1 for ever; mark keep is seen for exactly ``window`` queries; the
    middle one is seen up to its window's edge and not one query longer.  Whole prompts over
    packed keys, then the last 200 queries as one step over the paged cache with scattered pages,
    then single queries at the edges."""
    from minfer_b200.kernels import api as K
    from minfer_b200.parts.sink_attention import ScoreSpec, scored_attention
    from minfer_b200.parts import sink_attention
    from minfer_b200.parts.base import CacheView, StepContext
    # bfloat16: the tensor-memory kernel where the sizes allow (keys and values of 64 or 128), the
    # mma.sync kernels otherwise and when asked for, the generic kernel for the rest and when asked for
    if kernel == "mma":
        monkeypatch.setattr(sink_attention, "PROMPT_KERNEL", "mma")
    if kernel == "generic":
        monkeypatch.setattr(sink_attention, "FORCE_GENERIC", True)
    g = torch.Generator().manual_seed(hd + window + keep)
    n = 400
    mid = 2 * window + keep + 77
    marks = [keep - 1, keep, mid]
    q, k, v = _marked(n, nh, nk, hd, vd, marks, g, dt)
    scale = 0.1
    want = P.masked_attention(q.double(), k.double(), v.double(), scale, window, keep)
    spec = ScoreSpec(n_heads=nh, n_kv_heads=nk, head_dim=hd, value_dim=vd, scale=scale, window=window,
                     keep_first=keep)

    def ctx(from_start, rows_tokens, positions, seq_end):
        cu = [0]
        for t in rows_tokens:
            cu.append(cu[-1] + t)
        token_row = [b for b, t in enumerate(rows_tokens) for _ in range(t)]
        return StepContext(device=torch.device(DEV), act_dtype=dt, n_tokens=cu[-1], n_rows=len(rows_tokens),
                           token_ids=_i32([0] * cu[-1]), positions=_i32(positions), token_row=_i32(token_row),
                           cu_seqlens=_i32(cu), seq_end=_i32(seq_end), slots=_i32(list(range(len(rows_tokens)))),
                           from_start=from_start, single_token=all(t == 1 for t in rows_tokens),
                           max_row_tokens=max(rows_tokens), max_end=max(seq_end), status=_status())

    def check(got):
        got = got.reshape(-1, nh, vd)
        tol = 1e-5 if dt == torch.float32 else 2e-2
        _close(got, want[-got.shape[0]:], tol)
        far = got[-1, 0].float().cpu()                     # the last query is far beyond every window
        assert torch.allclose(far, v[keep - 1, 0].float(), atol=3e-2)
        for j in (keep, mid):
            last = j + window - 1                          # the last query that sees key j
            at = last - (n - got.shape[0])
            if at >= 0:
                assert torch.allclose(got[at, 0].float().cpu(), v[j, 0].float(), atol=3e-2), j
                assert not torch.allclose(got[at + 1, 0].float().cpu(), v[j, 0].float(), atol=0.3), j

    # whole prompt, packed keys (two sequences in the step: the other one is short)
    q2 = torch.cat([q[:5], q]).to(DEV)
    k2 = torch.cat([k[:5], k]).to(DEV)
    v2 = torch.cat([v[:5], v]).to(DEV)
    c = ctx(True, [5, n], list(range(5)) + list(range(n)), [5, n])
    o = torch.empty(n + 5, nh * vd, dtype=dt, device=DEV)
    scored_attention(spec, q2, k2, v2, None, c, o)
    check(o[5:])
    # over the paged cache: pages scattered, stale values elsewhere; the last 200 queries in a step
    # of several tokens, then each of them alone as a step of one token a row
    n_pages = (n + 63) // 64
    kc = torch.randn(n_pages + 5, nk, 64, hd, generator=g).to(dt).to(DEV)
    vc = torch.randn(n_pages + 5, nk, 64, vd, generator=g).to(dt).to(DEV)
    order = torch.randperm(n_pages + 5, generator=g)[:n_pages].tolist()
    for p in range(n):
        kc[order[p // 64], :, p % 64] = k[p].to(DEV)
        vc[order[p // 64], :, p % 64] = v[p].to(DEV)
    cache = CacheView(k=kc, v=vc, page_table=_i32([order]), table_stride=n_pages, ring=0)
    tail = 200
    c = ctx(False, [tail], list(range(n - tail, n)), [n])
    o = torch.empty(tail, nh * vd, dtype=dt, device=DEV)
    scored_attention(spec, q[n - tail:].contiguous().to(DEV), None, None, cache, c, o)
    check(o)
    singles = [keep + window - 1, keep + window, mid + window - 1, mid + window, n - 1]
    for p in singles:
        c = ctx(False, [1], [p], [p + 1])
        o1 = torch.empty(1, nh * vd, dtype=dt, device=DEV)
        scored_attention(spec, q[p:p + 1].contiguous().to(DEV), None, None, cache, c, o1)
        _close(o1.reshape(nh, vd), want[p], 1e-5 if dt == torch.float32 else 2e-2)
