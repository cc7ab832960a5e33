"""Bedarax through the engine against the plain implementation, in float32 and bfloat16: whole
prompts and the stream after every layer; the last tokens one by one; every token a step from the
first; prompts in portions down to two tokens; batches of unequal requests against each alone, one
batch after another so that slots, pages and state are used again; a mixed step; decoding far past
a window's ring; greedy generation through the generator, the command line and the trace replay."""
import copy
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_bedarax as P
from bedarax_cases import BED_A, BED_B, CASES, drop_ranks, loud_weights, make_folder
from helpers import logits_err, random_ids

pytestmark = pytest.mark.gpu

LENGTHS = [37, 5, 131, 64, 1, 65, 11]


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def case(request):
    folder = make_folder(request.param)
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab"], 700 + i) for i, n in enumerate(LENGTHS)]
    plain = [_plain(cfg, w, ids) for ids in prompts]
    return {"name": request.param, "folder": folder, "cfg": cfg, "w": w, "prompts": prompts,
            "plain": plain}


def _engine(folder, dtype, max_tokens=4096, **kw):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    return Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=max_tokens, **kw)


# a router's choice that hangs on less than this is left out of a comparison: rounding the
# activations to bfloat16 moves the router's logits by up to a few thousandths
LEAST_MARGIN = 0.03


def _plain(cfg, w, ids):
    """The plain logits, NaN where a router's choice is a close call."""
    return P.forward_sure(cfg, w, ids, LEAST_MARGIN)


def _close(got, want, dtype):
    """Compares the rows whose plain logits are sure; nearly all are."""
    sure = ~torch.isnan(want).any(dim=-1)
    if want.shape[0] >= 20:
        assert int(sure.sum()) * 10 >= 7 * want.shape[0]
    if not bool(sure.any()):
        return
    err, bound = logits_err(got[sure.to(got.device)], want[sure], dtype)
    assert err < bound, (err, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_every_layer(case, dtype):
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"], case["plain"]):
        s = eng.acquire()
        got = eng.step([s], [ids], [list(range(len(ids)))])
        eng.release(s)
        assert got.shape == want.shape
        _close(got, want, dtype)
    # the stream that goes on after every layer (after the depth average)
    ids = case["prompts"][2]
    taps, seen = [], []
    P.forward(case["cfg"], case["w"], ids, taps)
    eng.layer_tap = lambda i, h: seen.append(h.detach().cpu().to(torch.float64))
    s = eng.acquire()
    eng.step([s], [ids], [list(range(len(ids)))])
    eng.release(s)
    eng.layer_tap = None
    assert len(seen) == len(taps)
    for got, want in zip(seen, taps):
        tol = 3e-5 if dtype == "float32" else 4e-2
        assert float((got - want).abs().max()) < tol * float(want.abs().max())
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(case, dtype):
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"], case["plain"]):
        n = len(ids)
        head = max(1, n - 40)
        s = eng.acquire()
        rows = [eng.step([s], [ids[:head]], [list(range(head))])]
        for t in range(head, n):
            rows.append(eng.step([s], [[ids[t]]], [[0]]))
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_by_token_from_the_first(case, dtype):
    """Every token a step of its own, from position 0: the first tokens see the zeros before the
    sequence in the convolutions, an empty recurrent state, and nothing but themselves in
    attention."""
    eng = _engine(case["folder"], dtype)
    ids, want = case["prompts"][0], case["plain"][0]
    s = eng.acquire()
    rows = [eng.step([s], [[t]], [[0]]) for t in ids]
    eng.release(s)
    _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("portion", [2, 3, 7, 15, 16, 17, 63, 64, 65])
def test_prompts_in_portions(case, dtype, portion):
    """Portions around the recurrence's chunk of 16 tokens and around a page of 64 positions."""
    eng = _engine(case["folder"], dtype)
    for ids, want in zip(case["prompts"][:4], case["plain"][:4]):
        s = eng.acquire()
        rows = []
        for lo in range(0, len(ids), portion):
            part = ids[lo:lo + portion]
            rows.append(eng.step([s], [part], [list(range(len(part)))]))
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_slots_reused(case, dtype):
    """The prompts' first parts in one step, then one token each; a request that runs out of
    tokens leaves the batch; the next batch starts in the slots, pages and state the first one
    gave back.  Every request's logits equal those it has alone."""
    eng = _engine(case["folder"], dtype, max_tokens=1024, max_seqs=4)
    prompts, plain = case["prompts"], case["plain"]
    for batch in ([0, 1, 2], [3, 4, 5, 6], [2, 0], [6, 2, 4]):
        slots = {r: eng.acquire() for r in batch}
        heads = {r: max(1, len(prompts[r]) - 9) for r in batch}
        got = {r: [] for r in batch}
        out = eng.step([slots[r] for r in batch], [prompts[r][:heads[r]] for r in batch],
                       [list(range(heads[r])) for r in batch])
        at = 0
        for r in batch:
            got[r].append(out[at:at + heads[r]])
            at += heads[r]
        pos = dict(heads)
        live = [r for r in batch if pos[r] < len(prompts[r])]
        while live:
            out = eng.step([slots[r] for r in live], [[prompts[r][pos[r]]] for r in live],
                           [[0]] * len(live))
            for i, r in enumerate(live):
                got[r].append(out[i:i + 1])
                pos[r] += 1
            live = [r for r in live if pos[r] < len(prompts[r])]
        for r in batch:
            _close(torch.cat(got[r]), plain[r], dtype)
            eng.release(slots[r])
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_stale_slot_does_not_leak_into_the_next_request(case, dtype):
    """A long request fills a slot's recurrent state, convolution inputs and pages; the slot is
    given back and the next, short request in it must start from nothing."""
    eng = _engine(case["folder"], dtype, max_tokens=512, max_seqs=1)
    prompts, plain = case["prompts"], case["plain"]
    for r in (2, 1, 4, 0, 4):
        s = eng.acquire()
        got = eng.step([s], [prompts[r]], [list(range(len(prompts[r])))])
        eng.release(s)
        _close(got, plain[r], dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_step_a_new_portion_beside_single_tokens(case, dtype):
    """One request goes on by 20 tokens while two others go on by one, in the same step."""
    eng = _engine(case["folder"], dtype)
    prompts, plain = case["prompts"], case["plain"]
    a, b, c = 2, 0, 6
    sa, sb, sc = eng.acquire(), eng.acquire(), eng.acquire()
    eng.step([sa, sb, sc], [prompts[a][:100], prompts[b][:30], prompts[c][:10]], [[], [], []])
    out = eng.step([sb, sa, sc], [[prompts[b][30]], prompts[a][100:120], [prompts[c][10]]],
                   [[0], list(range(20)), [0]])
    _close(out[0:1], plain[b][30:31], dtype)
    _close(out[1:21], plain[a][100:120], dtype)
    _close(out[21:22], plain[c][10:11], dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_past_the_rings(name, dtype):
    """330 tokens: a prompt of 70, then one by one far past the windows' rings, with the recurrent
    layers' state carried all the way; the same in portions of 50 with a ring that has slack for
    one new position only."""
    folder = make_folder(name)
    cfg, w = P.load_folder(folder)
    ids = random_ids(330, cfg["vocab"], 91)
    want = _plain(cfg, w, ids)
    eng = _engine(folder, dtype, max_tokens=1024)
    assert any(g.ring and g.ring < 330 for g in eng.cache.groups)
    s = eng.acquire()
    rows = [eng.step([s], [ids[:70]], [list(range(70))])]
    for t in range(70, 330):
        rows.append(eng.step([s], [[ids[t]]], [[0]]))
    eng.release(s)
    _close(torch.cat(rows), want, dtype)
    eng2 = _engine(folder, dtype, max_tokens=1024, ring_step_tokens=1)
    s = eng2.acquire()
    rows = []
    for lo in range(0, 330, 50):
        part = ids[lo:lo + 50]
        rows.append(eng2.step([s], [part], [list(range(len(part)))]))
    _close(torch.cat(rows), want, dtype)
    eng.check_status()
    eng2.check_status()
    eng2.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_a_long_prompt_in_large_portions(name, dtype):
    """430 tokens in portions of 200, 220 and 10: the later portions attend over the cache's pages
    across the windows' edges, the experts take their grouped path; then the same prompt whole
    beside a short one."""
    folder = make_folder(name)
    cfg, w = P.load_folder(folder)
    ids = random_ids(430, cfg["vocab"], 17)
    want = _plain(cfg, w, ids)
    eng = _engine(folder, dtype, max_tokens=2048)
    s = eng.acquire()
    rows, at = [], 0
    for n in (200, 220, 10):
        rows.append(eng.step([s], [ids[at:at + n]], [list(range(n))]))
        at += n
    eng.release(s)
    _close(torch.cat(rows), want, dtype)
    short = random_ids(33, cfg["vocab"], 18)
    a, b = eng.acquire(), eng.acquire()
    out = eng.step([b, a], [short, ids], [[32], [429, 0, 215]])
    _close(out[0:1], _plain(cfg, w, short)[32:33], dtype)
    _close(out[1:4], want[[429, 0, 215]], dtype)
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_generator(case, dtype):
    from helpers import TOL
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = case["cfg"], case["w"]
    prompts = [case["prompts"][0], case["prompts"][1], case["prompts"][6]]
    gen = Generator(Model.from_folder(case["folder"], dtype, "cuda:0"), max_tokens=2048, max_batch=4)
    got = gen.generate(prompts, 8, SamplingParams.greedy(), stop_token_ids=[])
    for prompt, res in zip(prompts, got):
        assert len(res.tokens) == 8
        ids = list(prompt)
        for tok in res.tokens:             # each token on the prefix the engine itself produced
            logits = P.forward(cfg, w, ids)[-1]
            if dtype == "float32":
                assert tok == int(torch.argmax(logits))
            else:
                slack = 2 * TOL["bfloat16"] * float(logits.abs().max())
                assert float(logits[tok]) >= float(logits.max()) - slack
            ids.append(tok)


def test_command_line_generates(capsys):
    from minfer_b200 import cli
    folder = make_folder("B")
    cfg, w = P.load_folder(folder)
    rc = cli.main([folder, "5,17,3", "--greedy", "--repeat-penalty", "1.0", "-n", "6",
                   "--dtype", "float32", "--stop", "100000"])
    out = capsys.readouterr().out
    assert rc == 0
    want = P.generate_greedy(cfg, w, [5, 17, 3], 6)
    assert " ".join(str(t) for t in want) in out
    assert "Prefill: 3 tokens" in out and "Generated: 6 tokens" in out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_process(dtype):
    """``bin/trace_run`` on a Bedarax folder whose config.json leaves the low-rank pairs' ranks to
    the tensors' shapes: two prompts of unequal length in one step, then one request's last tokens
    one by one beside another that ends earlier; logits files against the plain implementation."""
    folder = make_folder("A")
    drop_ranks(folder)
    cfg, w = P.load_folder(folder)
    a, b = random_ids(70, cfg["vocab"], 1), random_ids(9, cfg["vocab"], 2)
    plain = {"a": _plain(cfg, w, a), "b": _plain(cfg, w, b)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []}]
    expect = {0: [("a", [0, 59]), ("b", [6])]}
    for i in range(10):
        entries = [{"id": "a", "tokens": [a[60 + i]], "want": [0] if i % 2 == 0 else []}]
        rows = [("a", [60 + i])] if i % 2 == 0 else []
        if i < 2:
            entries.append({"id": "b", "tokens": [b[7 + i]], "want": [0]})
            rows.append(("b", [7 + i]))
        end = (["b"] if i == 1 else []) + (["a"] if i == 9 else [])
        steps.append({"step": i + 1, "entries": entries, "end": end})
        expect[i + 1] = rows
    out = tempfile.mkdtemp()
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", out, "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    for step, rows in expect.items():
        path = os.path.join(out, f"{step}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, cfg["vocab"]))
        want = torch.cat([plain[r][places] for r, places in rows])
        _close(got, want, dtype)


def _folder_of(cfg, seed, store="bfloat16"):
    return make_folder("x", store, cfg, seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_recurrent_layers_only(dtype):
    """No attention anywhere: the cache has no page group at all, only state."""
    cfg = copy.deepcopy(BED_A)
    cfg["layers"] = [cfg["layers"][0], cfg["layers"][2], copy.deepcopy(BED_B["layers"][2])]
    folder = _folder_of(cfg, 31)
    cfg, w = P.load_folder(folder)
    ids = random_ids(90, cfg["vocab"], 4)
    want = _plain(cfg, w, ids)
    eng = _engine(folder, dtype, max_tokens=512)
    assert not eng.cache.groups
    s = eng.acquire()
    rows = [eng.step([s], [ids[:50]], [list(range(50))])]
    rows.append(eng.step([s], [ids[50:53]], [[0, 1, 2]]))
    for t in range(53, 90):
        rows.append(eng.step([s], [[ids[t]]], [[0]]))
    eng.release(s)
    _close(torch.cat(rows), want, dtype)
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_attention_layers_only_and_one_layer(dtype):
    """Attention only (no state at all), and a model of a single layer (a depth average of two)."""
    cfg = copy.deepcopy(BED_A)
    cfg["layers"] = [cfg["layers"][1], cfg["layers"][4], cfg["layers"][3]]
    one = copy.deepcopy(BED_B)
    one["layers"] = [one["layers"][2]]
    for c, seed in ((cfg, 33), (one, 34)):
        folder = _folder_of(c, seed)
        c, w = P.load_folder(folder)
        ids = random_ids(90, c["vocab"], 5)
        want = _plain(c, w, ids)
        eng = _engine(folder, dtype, max_tokens=512)
        s = eng.acquire()
        rows = [eng.step([s], [ids[:41]], [list(range(41))])]
        rows.append(eng.step([s], [ids[41:60]], [list(range(19))]))
        rows += [eng.step([s], [[t]], [[0]]) for t in ids[60:]]
        eng.release(s)
        _close(torch.cat(rows), want, dtype)
        eng.check_status()


def test_matrices_stored_in_32_bit_run_in_the_bfloat16_engine():
    """A checkpoint whose matrices are float32 keeps them so in the bfloat16 engine (FP32-pipe
    products, bfloat16 cache and attention): every mixer and feed-forward takes the mix."""
    folder = make_folder("A", "float32")
    cfg, w = P.load_folder(folder)
    ids = random_ids(75, cfg["vocab"], 8)
    want = _plain(cfg, w, ids)
    eng = _engine(folder, "bfloat16", max_tokens=512)
    s = eng.acquire()
    rows = [eng.step([s], [ids[:60]], [list(range(60))])]
    rows += [eng.step([s], [[t]], [[0]]) for t in ids[60:]]
    eng.release(s)
    _close(torch.cat(rows), want, "bfloat16")
    eng.check_status()
