"""The kernels of the Bedarax mixers and feed-forwards alone against plain functions, on inputs
made so that a fault shows: one key whose score stands out placed just inside and just outside a
window, at page borders and far back, through a score mix far from the identity; a recurrent state
that must keep what it was told hundreds of tokens ago; state carried over cuts of every size;
routers with ties; PolyNorm numbers that all differ."""
import pytest
import torch

import plain_bedarax as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _paged(k, v, dtype, ring=0):
    """One sequence's keys and values written into pages in a scrambled order."""
    n, g, d = k.shape
    dv = v.shape[-1]
    n_pages = (n + 63) // 64 if not ring else ring // 64
    order = list(reversed(range(n_pages)))
    kc = torch.zeros((n_pages + 1, g, 64, d), dtype=dtype, device=DEV)
    vc = torch.zeros((n_pages + 1, g, 64, dv), dtype=dtype, device=DEV)
    lo = max(0, n - ring) if ring else 0
    for j in range(lo, n):
        p_eff = j % ring if ring else j
        page = order[p_eff // 64]
        kc[page, :, p_eff % 64] = k[j].to(dtype)
        vc[page, :, p_eff % 64] = v[j].to(dtype)
    return kc, vc, _i32(order)


def _standout(n, H, G, D, Dv, window, standout, dtype, seed):
    """Random q, k, v of one sequence in which, for the last query, the oldest key the window
    admits (plus ``standout``) scores far above the others, and so does the key one further back
    (outside the window) with another value."""
    torch.manual_seed(seed)
    q = torch.randn(n, H, D, dtype=torch.float64) * 0.5
    k = torch.randn(n, G, D, dtype=torch.float64) * 0.5
    v = torch.randn(n, G, Dv, dtype=torch.float64)
    last = n - 1
    inside = (last - window + 1 + standout) if 0 < window <= n else standout
    marked = [inside] + ([inside - 1] if 0 < window <= n and standout == 0 and inside >= 1 else [])
    for g in range(G):
        for j in marked:
            k[j, g] = q[last, g * (H // G)] * 3.0
    for j in marked:
        v[j] = 10.0 * (1 + marked.index(j))
    return tuple(t.to(dtype).to(torch.float64) for t in (q, k, v))


WINDOWS = [(0, 3), (70, 0), (70, 1), (64, 0), (64, 1), (65, 0), (1, 0), (136, 0), (136, 1),
           (200, 150), (1000, 2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, standout", WINDOWS)
@pytest.mark.parametrize("H, G, D, Dv", [(4, 2, 24, 40), (3, 3, 10, 6), (1, 1, 96, 32)])
def test_talking_attention_over_a_prompt(dtype, window, standout, H, G, D, Dv):
    """600 keys of one prompt; queries at the end, at a page's border and at the start."""
    from minfer_b200.kernels import api as K
    n = 600
    q, k, v = _standout(n, H, G, D, Dv, window, standout, dtype, window * 7 + standout + H)
    talk = torch.eye(H, dtype=torch.float64) * 0.6 + torch.randn(H, H, dtype=torch.float64) * 0.5
    talk = talk.to(torch.float32).to(torch.float64)
    rows = [n - 1, n - 2, 64, 63, 0]
    gate = torch.randn(len(rows), H + 3, dtype=torch.float32)
    want = P.talking_attention(q[rows], k, v, talk, rows, 0.4, window)
    want = want * torch.sigmoid(gate[:, 3:].to(torch.float64)).unsqueeze(-1)
    out = torch.empty((len(rows), H * Dv), dtype=dtype, device=DEV)
    K.talk_attention(q[rows].to(dtype).to(DEV).contiguous(), k.to(dtype).to(DEV), v.to(dtype).to(DEV),
                     _i32([0] * len(rows)), _i32(rows), _i32([0, n]), None, 0, 0,
                     talk.to(torch.float32).to(DEV), gate.to(DEV), 3, out, H, G, D, Dv, window, 0.4)
    err = float((out.cpu().to(torch.float64).view(len(rows), H, Dv) - want).abs().max())
    assert err < _tol(dtype) * float(want.abs().max()), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, standout", WINDOWS)
@pytest.mark.parametrize("ring", [0, 1])
def test_talking_attention_over_the_cache(dtype, window, standout, ring):
    """The same over pages (in a scrambled order; as a ring that has wrapped): one query (a decode
    step, its keys cut into stretches over several blocks) and several at once."""
    from minfer_b200.kernels import api as K
    n, H, G, D, Dv = 600, 4, 2, 24, 40
    if ring and not window:
        pytest.skip("a ring belongs to a window")
    q, k, v = _standout(n, H, G, D, Dv, window, standout, dtype, window * 5 + standout)
    ring_len = ((window + 19 + 63) // 64) * 64 if ring else 0
    if ring_len >= n:
        ring_len = 0
    kc, vc, table = _paged(k, v, dtype, ring_len)
    talk = (torch.eye(H) * 0.6 + torch.randn(H, H) * 0.5).to(torch.float64)
    for rows in ([n - 1], [n - 1, n - 2, n - 5, n - 19]):
        want = P.talking_attention(q[rows], k, v, talk, rows, 0.4, window)
        out = torch.empty((len(rows), H * Dv), dtype=dtype, device=DEV)
        reach = min(window, n) if window else n
        K.talk_attention(q[rows].to(dtype).to(DEV).contiguous(), kc, vc, _i32([0] * len(rows)),
                         _i32(rows), None, table.view(1, -1), table.numel(), ring_len,
                         talk.to(torch.float32).to(DEV), None, 0, out, H, G, D, Dv, window, 0.4,
                         reach_keys=reach)
        err = float((out.cpu().to(torch.float64).view(len(rows), H, Dv) - want).abs().max())
        assert err < _tol(dtype) * float(want.abs().max()), (rows, err)


TILE_SHAPES = [(4, 2, 32, 40), (8, 2, 16, 24), (16, 8, 16, 16), (32, 4, 16, 8), (6, 3, 48, 16),
               (2, 1, 16, 8), (12, 4, 32, 32), (8, 2, 128, 128)]


@pytest.mark.parametrize("window, standout", [(0, 3), (70, 0), (70, 1), (64, 0), (33, 0), (32, 1),
                                              (1, 0), (136, 1), (200, 150)])
@pytest.mark.parametrize("H, G, D, Dv", TILE_SHAPES)
def test_talking_attention_tiles_of_queries_over_a_prompt(window, standout, H, G, D, Dv):
    """Every query of a 300-token prompt and of a 21-token prompt beside it through the tiled
    kernel: clusters of 1 to 8 blocks, heads a block that are fewer, as many and more than a
    key/value head serves."""
    from minfer_b200.kernels import api as K
    dtype = torch.bfloat16
    assert K.talk_tile_cluster(H, G, D, Dv) > 0
    n, m = 300, 21
    q, k, v = _standout(n, H, G, D, Dv, window, standout, dtype, window * 3 + standout + H)
    q2, k2, v2 = _standout(m, H, G, D, Dv, min(window, m), 0, dtype, 11)
    talk = torch.eye(H, dtype=torch.float64) * 0.6 + torch.randn(H, H, dtype=torch.float64) * 0.5
    talk = talk.to(torch.float32).to(torch.float64)
    gate = torch.randn(n + m, H + 2, dtype=torch.float32)
    want = torch.cat([P.talking_attention(q, k, v, talk, list(range(n)), 0.4, window),
                      P.talking_attention(q2, k2, v2, talk, list(range(m)), 0.4, window)])
    want = want * torch.sigmoid(gate[:, 2:].to(torch.float64)).unsqueeze(-1)
    out = torch.empty((n + m, H * Dv), dtype=dtype, device=DEV)
    cu = _i32([0, n, n + m])
    K.talk_attention(torch.cat([q, q2]).to(dtype).to(DEV), torch.cat([k, k2]).to(dtype).to(DEV),
                     torch.cat([v, v2]).to(dtype).to(DEV), _i32([0] * n + [1] * m),
                     _i32(list(range(n)) + list(range(m))), cu, None, 0, 0,
                     talk.to(torch.float32).to(DEV), gate.to(DEV), 2, out, H, G, D, Dv, window, 0.4,
                     q_cu_seqlens=cu, n_seq=2, max_row_tokens=n)
    got = out.cpu().to(torch.float64).view(n + m, H, Dv)
    err = (got - want).abs().amax(dim=(1, 2))
    assert float(err.max()) < _tol(dtype) * float(want.abs().max()), (int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("window, standout", [(0, 3), (70, 0), (70, 1), (64, 0), (65, 0), (136, 1)])
@pytest.mark.parametrize("ring", [0, 1])
@pytest.mark.parametrize("H, G, D, Dv", [(4, 2, 32, 40), (16, 4, 16, 16)])
def test_talking_attention_tiles_of_queries_over_the_cache(window, standout, ring, H, G, D, Dv):
    """A portion of a prompt over pages (scrambled; a ring that has wrapped): the last 1, 2, 17 and
    51 positions of 600 as one row's queries, beside a row that brings one token; the key tiles
    dealt to several clusters and merged."""
    from minfer_b200.kernels import api as K
    dtype = torch.bfloat16
    n = 600
    if ring and not window:
        pytest.skip("a ring belongs to a window")
    q, k, v = _standout(n, H, G, D, Dv, window, standout, dtype, window * 5 + standout)
    talk = (torch.eye(H) * 0.6 + torch.randn(H, H) * 0.5).to(torch.float64)
    for portion in (1, 2, 17, 51):
        ring_len = ((window + portion + 63) // 64) * 64 if ring else 0
        if ring_len >= n:
            ring_len = 0
        kc, vc, table = _paged(k, v, dtype, ring_len)
        rows = list(range(n - portion, n))
        other = n - 7                       # a second row: the same sequence seen at one position
        want = P.talking_attention(q[[other] + rows], k, v, talk, [other] + rows, 0.4, window)
        if ring_len and other - window + 1 < n - ring_len:
            want[0] = float("nan")          # the ring has dropped keys this position would see
        out = torch.empty((portion + 1, H * Dv), dtype=dtype, device=DEV)
        cu = _i32([0, 1, portion + 1])
        tables = torch.stack([table, table])
        K.talk_attention(q[[other] + rows].to(dtype).to(DEV).contiguous(), kc, vc,
                         _i32([0] + [1] * portion), _i32([other] + rows), None, tables,
                         table.numel(), ring_len, talk.to(torch.float32).to(DEV), None, 0, out,
                         H, G, D, Dv, window, 0.4, reach_keys=min(window, n) if window else n,
                         q_cu_seqlens=cu, n_seq=2, max_row_tokens=portion)
        got = out.cpu().to(torch.float64).view(portion + 1, H, Dv)
        keep = ~torch.isnan(want[:, 0, 0])
        err = float((got[keep] - want[keep]).abs().max())
        assert err < _tol(dtype) * float(want[keep].abs().max()), (portion, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_talking_attention_two_sequences_and_an_identity_mix(dtype):
    """Two packed prompts of unequal length: a query never sees the other prompt's keys; with the
    identity as the mix the result is ordinary attention, head by head."""
    from minfer_b200.kernels import api as K
    torch.manual_seed(5)
    H, G, D, Dv, window = 6, 2, 16, 16, 40
    lens = [75, 130]
    q = (torch.randn(sum(lens), H, D, dtype=torch.float64)).to(dtype).to(torch.float64)
    k = (torch.randn(sum(lens), G, D, dtype=torch.float64)).to(dtype).to(torch.float64)
    v = (torch.randn(sum(lens), G, Dv, dtype=torch.float64)).to(dtype).to(torch.float64)
    eye = torch.eye(H, dtype=torch.float64)
    want = torch.cat([
        P.talking_attention(q[:75], k[:75], v[:75], eye, list(range(75)), 0.25, window),
        P.talking_attention(q[75:], k[75:], v[75:], eye, list(range(130)), 0.25, window)])
    plain = torch.zeros_like(want)
    for a in range(sum(lens)):
        base, i = (0, a) if a < 75 else (75, a - 75)
        lo = max(0, i - window + 1)
        for h in range(H):
            s = (k[base + lo:base + i + 1, h // 3] @ q[a, h]) * 0.25
            plain[a, h] = torch.softmax(s, 0) @ v[base + lo:base + i + 1, h // 3]
    assert float((plain - want).abs().max()) < 1e-9
    out = torch.empty((sum(lens), H * Dv), dtype=dtype, device=DEV)
    K.talk_attention(q.to(dtype).to(DEV), k.to(dtype).to(DEV), v.to(dtype).to(DEV),
                     _i32([0] * 75 + [1] * 130), _i32(list(range(75)) + list(range(130))),
                     _i32([0, 75, 205]), None, 0, 0, eye.to(torch.float32).to(DEV), None, 0, out,
                     H, G, D, Dv, window, 0.25)
    err = float((out.cpu().to(torch.float64).view(-1, H, Dv) - want).abs().max())
    assert err < _tol(dtype) * float(want.abs().max()), err


def test_value_blend():
    from minfer_b200.kernels import api as K
    torch.manual_seed(2)
    own = torch.randn(37, 50, device=DEV)
    first = torch.randn(37, 70, device=DEV)
    lam = torch.tensor(0.37, device=DEV)
    want = own.clone()
    want[:, 11:31] = (1 - 0.37) * own[:, 11:31] + 0.37 * first[:, 40:60]
    K.value_mix(own, 11, first, 40, lam, 20)
    assert float((own - want).abs().max()) < 1e-6
