"""Benchmark of the flagship serving step: decoding with the Qwen2.5-7B shape in bfloat16,
random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from 2,048-token
contexts, timed on the device with CUDA events over K decode steps (model step + greedy
sampling, token ids staying on the device).  ``e2e`` is the same through the Python entry
point (``Generator.generate``): host token ids in, host token ids out, every step.
``prefill`` is one 2,048-token prompt (median of 20); ``roofline`` is the decode step's bytes
(every weight it uses once, plus the cache of the live requests) over its time, against the
measured copy bandwidth; ``points`` are medians of per-step device times of the other
workloads: decoding at batch 1 and 64, the 0.5B shape with 64 ragged prompts, the 14B shape
at 8,192 positions, one sequence at 32,000 positions, each with its fraction of the roofline,
and the host's share of a step where the host could show.  ``points_clocks`` gives the median
SM clock inside each figure's own window.  ``reference_kernels`` times the reference's own
float32 CUDA kernels, compiled unchanged, beside this library's kernels for the same op.

The reference (yusiwen/minfer) is a Rust program; there is no Rust toolchain here, so
``--impl reference`` prints its ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the headline configuration (Qwen2.5-7B shape)
CONFIG_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 152064, "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "max_position_embeddings": 32768,
}
CONTEXT = 4096          # positions per sequence the cache is sized for
PROMPT = 2048           # tokens each sequence holds when decoding starts
BATCH = 8
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            found = 0

            def look(node):                       # the keys may sit at the top or one level down
                nonlocal found
                if isinstance(node, dict):
                    for k, v in node.items():
                        if k in out and isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                            out[k] = float(v)
                            found += 1
                        elif k in out and isinstance(v, dict) and isinstance(v.get("value"), (int, float)):
                            out[k] = float(v["value"])
                            found += 1
                        else:
                            look(v)
            look(d)
            if found:
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self, window=None):
        """Summary of the samples; with ``window`` (host times of the timed region's start and
        end) only of those taken inside it, if there are any."""
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        samples = list(self.samples)
        lines = [line for _, line in samples]
        if window is not None:
            inside = [line for t, line in samples if window[0] <= t <= window[1]]
            if inside:
                lines = inside
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_bytes(model, batch, context_tokens):
    """Bytes one decode step has to read: every weight it uses once (the embedding table is
    only touched at `batch` rows) and the cache of the live requests."""
    plan = model.plan
    weights = model.parameter_bytes()
    esz = 2 if str(model.dtype).endswith("bfloat16") else 4
    if model.head.weight.data_ptr() != model.embedding.data_ptr():
        weights -= model.embedding.numel() * model.embedding.element_size()
    kv = 0
    for call in plan.schedule:
        req = model.blocks[call.layer].mixer.cache_request()
        if req is not None and call.writes_cache:
            # keys and values may differ in width; a layer with a window or a chunk mask reads
            # at most that many positions back
            seen = min(context_tokens, req.window) if req.window else context_tokens
            kv += req.n_kv_heads * (req.head_dim + (req.value_dim or req.head_dim)) * esz * seen
        # fixed-size state per sequence (a recurrent mixer's): read and written once a step
        block = model.blocks[call.layer]
        for st in (block.state_request() if hasattr(block, "state_request") else ()):
            n = 1
            for d in st.shape:
                n *= d
            kv += 2 * n * 4
    return weights + batch * kv


def prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only) plus causal
    attention."""
    ne, nh, nk = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, nf, L, V = ne // nh, cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    per_token = 2 * ne * (nh + 2 * nk) * hd + 2 * ne * nh * hd + 2 * ne * 2 * nf + 2 * nf * ne
    linear = L * per_token * tokens + 2 * ne * V
    attention = L * nh * 4 * hd * tokens * (tokens + 1) / 2
    return linear + attention


SETTLE_S = 1.0


def time_decode(engine, torch, K, batch, steps, warmup, prompt_len, seed=0):
    """CUDA-event times of `steps` decode steps at `batch`, after `warmup` untimed ones: the
    mean (all steps between two events, the contract's figure), the median of the per-step
    times (an event after every step), and the kernels launched.  The sequences' caches come
    from a real prefill of `batch` random prompts of `prompt_len` tokens (one number, or a
    length for each row) in one step."""
    from minfer_b200.kernels import api
    plan = engine.model.plan
    slots = [engine.acquire() for _ in range(batch)]
    g = torch.Generator().manual_seed(seed)
    lens = list(prompt_len) if isinstance(prompt_len, (list, tuple)) else [prompt_len] * batch
    prompts = [torch.randint(0, plan.vocab_size, (n,), generator=g).tolist() for n in lens]
    logits = engine.step(slots, prompts)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    K.sample(logits, out, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
             frequency_penalty=0.0, presence_penalty=0.0, seed=0)
    tokens = out.clone()
    del logits, prompts
    # the prefill that built the caches is a burst at over 1 PFLOP/s; for some twenty steps
    # after it the GPU's power management holds the clocks down (3.9 ms, then 3.5, then the
    # steady 3.26 ms a step).  That belongs to the prefill, not to a decode step: let it pass.
    torch.cuda.synchronize()
    time.sleep(SETTLE_S)

    def one_step(tok):
        logits = engine.decode_on_device(slots, tok)
        K.sample(logits, out, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 frequency_penalty=0.0, presence_penalty=0.0, seed=0)
        return out

    for _ in range(warmup):
        tokens = one_step(tokens).clone()
    torch.cuda.synchronize()
    before = api.launches
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.time()
    marks[0].record()
    for i in range(steps):
        tokens = one_step(tokens)
        marks[i + 1].record()
    torch.cuda.synchronize()
    time_decode.window = (t0, time.time())
    ms = marks[0].elapsed_time(marks[steps])
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    time_decode.median_ms = statistics.median(per_step)
    launched = api.launches - before
    engine.check_status()
    for s in slots:
        engine.release(s)
    return ms / steps, launched


def time_prefill(engine, torch, ids, reps):
    """Median device time of `reps` whole-prompt steps of `ids` (one warm-up first), in ms."""
    times = []
    t0 = None
    for i in range(reps + 1):
        s = engine.acquire()
        torch.cuda.synchronize()
        if i == 1:
            t0 = time.time()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([s], [ids])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.release(s)
    time_prefill.window = (t0, time.time())
    time_prefill.times = times[1:]
    return statistics.median(times[1:])


CONFIG_05B = dict(CONFIG_7B, vocab_size=151936, hidden_size=896, num_hidden_layers=24,
                  num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                  tie_word_embeddings=True)
CONFIG_14B = dict(CONFIG_7B, hidden_size=5120, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5)


def _frac(step_bytes, ms, pk):
    return round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)


def point_05b(torch, K, pk, new_tokens=256):
    """Qwen2.5-0.5B shape, 64 sequences with prompt lengths uniform in [16, 1024], `new_tokens`
    decoded tokens each: the device's time of a step (graph replays fed from the device, an
    event after every step), and the same through Generator.generate (host ids in and out every
    step, the host's clock).  Their difference is what the Python host adds to a step."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg = dict(CONFIG_05B)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(16, 1025, (64,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    gen = Generator(model, max_tokens=64 * 1280, max_batch=64)
    time_decode(gen.engine, torch, K, 64, new_tokens, 3, lens, seed=3)
    ms_dev, window = time_decode.median_ms, time_decode.window
    gen.generate(prompts, 8, SamplingParams.greedy(), stop_token_ids=[])      # warm-up
    gen.stats.__init__()
    gen.generate(prompts, new_tokens, SamplingParams.greedy(), stop_token_ids=[])
    st = gen.stats
    ms_host = st.decode_seconds / max(st.steps - 1, 1) * 1e3
    step_bytes = decode_bytes(model, 64, sum(lens) / 64 + new_tokens / 2)
    out = {"decode_05b_ragged64_ms": round(ms_dev, 4),
           "decode_05b_ragged64_frac": _frac(step_bytes, ms_dev, pk),
           "decode_05b_ragged64_e2e_ms": round(ms_host, 4),
           "host_share_05b_ragged64": round(max(0.0, ms_host - ms_dev) / ms_host, 4)}
    return out, {"decode_05b_ragged64": (window, ms_dev)}


def point_14b(torch, K, pk, steps=96):
    """Qwen2.5-14B shape: prefill of one 8,192-token prompt, decode at batch 8 from 8,192-token
    contexts."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    cfg = dict(CONFIG_14B)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    gen = Generator(model, max_tokens=8 * (8192 + 256), max_batch=8)
    engine = gen.engine
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg["vocab_size"], (8192,), generator=g).tolist()
    ms_prefill = time_prefill(engine, torch, ids, 5)
    w_prefill = time_prefill.window
    time_decode(engine, torch, K, 8, steps, 3, 8192)
    ms_step = time_decode.median_ms
    step_bytes = decode_bytes(model, 8, 8192 + 3 + steps / 2)
    out = {"prefill_14b_8192_ms": round(ms_prefill, 2),
           "prefill_14b_8192_frac": round(prefill_flops(cfg, 8192) / (ms_prefill * 1e-3) /
                                          (pk["bf16_tflops"] * 1e12), 4),
           "decode_14b_b8_ctx8192_ms": round(ms_step, 4),
           "decode_14b_b8_ctx8192_frac": _frac(step_bytes, ms_step, pk)}
    return out, {"prefill_14b_8192": (w_prefill, ms_prefill),
                 "decode_14b_b8_ctx8192": (time_decode.window, ms_step)}


def point_long(engine, torch, K, pk, cfg, context=32000, steps=32):
    """The headline shape with one sequence at 32,000 positions: its prefill, then decoding."""
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, cfg["vocab_size"], (context,), generator=g).tolist()
    ms_prefill = time_prefill(engine, torch, ids, 2)
    w_prefill = time_prefill.window
    time_decode(engine, torch, K, 1, steps, 3, context, seed=6)
    ms_step = time_decode.median_ms
    step_bytes = decode_bytes(engine.model, 1, context + 3 + steps / 2)
    out = {"prefill_7b_32000_ms": round(ms_prefill, 2),
           "prefill_7b_32000_frac": round(prefill_flops(cfg, context) / (ms_prefill * 1e-3) /
                                          (pk["bf16_tflops"] * 1e12), 4),
           "decode_7b_b1_ctx32000_ms": round(ms_step, 4),
           "decode_7b_b1_ctx32000_frac": _frac(step_bytes, ms_step, pk)}
    return out, {"prefill_7b_32000": (w_prefill, ms_prefill),
                 "decode_7b_b1_ctx32000": (time_decode.window, ms_step)}


# ------------------------------------------------------------------------------------------
# --workload furitar: the Furitar design beside the Qwen2 decoder at equal sizes
# ------------------------------------------------------------------------------------------
def furitar_config(width, heads, kv, dim, vdim, ff, chunk, layers, vocab, positions):
    layer = {"type": "attention",
             "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim,
                       "scale": dim ** -0.5 * 8.0, "mask": {"size": chunk}},
             "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Furitar", "vocab": vocab, "width": width, "max_positions": positions,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
            "layers": [layer] * layers}


# (name, width, heads, kv heads, head size, Qwen2's intermediate size, chunk, layers): the dense
# feed-forward gets 1.5 x the gated one's inner width, so both have the same weights per layer
FURITAR_SIZES = [("w2048", 2048, 16, 4, 128, 5632, 1024, 8),
                 ("w4096", 4096, 32, 8, 128, 11264, 2048, 6)]
FURITAR_VOCAB = 32000


def furitar_prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only) plus the attention
    of the keys a chunk mask leaves visible."""
    w, flops = cfg["width"], 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        per_token = 2 * w * ((m["heads"] + m["kv_heads"]) * m["dim"] + m["kv_heads"] * m["vdim"])
        per_token += 2 * w * m["heads"] * m["vdim"]
        if layer["mlp"] is not None:
            per_token += 4 * w * layer["mlp"]["ff"]
        flops += per_token * tokens
        c = m["mask"]["size"]
        full, rest = divmod(tokens, c)
        pairs = full * c * (c + 1) / 2 + rest * (rest + 1) / 2
        flops += m["heads"] * 2 * (m["dim"] + m["vdim"]) * pairs
    return flops + 2 * w * cfg["vocab"]


def _median_ms(torch, fn, reps=20, flush=None):
    """Median device time of ``fn`` over ``reps`` runs after three warm-ups; L2 is flushed by a
    write of ``flush`` (a buffer larger than L2) before each."""
    times = []
    for i in range(reps + 3):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b))
    return statistics.median(times)


def furitar_attention_kernels(torch, K, pk, heads, kv, dim, chunk, tokens=2048, batch=8):
    """The attention kernels alone at one layer's sizes: a whole prompt of ``tokens`` and
    ``batch`` single queries at position ``tokens`` - 1, Furitar's beside Qwen2's, each with its
    share of its roofline (flops of the visible pairs over the measured product peak for a
    prompt; bytes of the visible keys and values over the measured copy bandwidth for single
    queries)."""
    from minfer_b200.parts.attention import decode_chunks
    dev, bf = "cuda:0", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(bf)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {}
    # a whole prompt
    q, k, v = rnd(tokens, heads, dim), rnd(tokens, kv, dim), rnd(tokens, kv, dim)
    o = torch.empty(tokens, heads * dim, dtype=bf, device=dev)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=dev)
    r1 = torch.full((heads,), 0.5, dtype=torch.float32, device=dev)
    r2 = torch.full((heads,), 0.5, dtype=torch.float32, device=dev)
    scale = dim ** -0.5
    ms_f = _median_ms(torch, lambda: K.sink_attention_mma(q, k, v, cu, None, None, 0, 0, o, r1, r2, 1,
                                                          tokens, heads, kv, dim, dim, 0, chunk, True,
                                                          scale), flush=flush)
    ms_f_mma = ms_f
    ms_f = _median_ms(torch, lambda: K.sink_attention_tc(q, k, v, cu, None, None, 0, 0, o, r1, r2, 1,
                                                         tokens, heads, kv, dim, 0, chunk, True, scale,
                                                         status), flush=flush)
    ms_q = _median_ms(torch, lambda: K.attention_prefill_tc(q, k, v, cu, o, 1, tokens, heads, kv, dim, 0,
                                                            scale, status), flush=flush)
    full, rest = divmod(tokens, chunk)
    pairs_f = full * chunk * (chunk + 1) / 2 + rest * (rest + 1) / 2
    pairs_q = tokens * (tokens + 1) / 2
    peak = pk["bf16_tflops"] * 1e12
    out["prompt"] = {
        "furitar_us": round(ms_f * 1e3, 1), "qwen2_us": round(ms_q * 1e3, 1),
        "furitar_mma_sync_us": round(ms_f_mma * 1e3, 1),
        "furitar_frac": round(heads * 4 * dim * pairs_f / (ms_f * 1e-3) / peak, 4),
        "qwen2_frac": round(heads * 4 * dim * pairs_q / (ms_q * 1e-3) / peak, 4)}
    # single queries over pages
    pages_per = tokens // 64
    n_pages = batch * pages_per
    kc, vc = rnd(n_pages, kv, 64, dim), rnd(n_pages, kv, 64, dim)
    table = torch.arange(n_pages, dtype=torch.int32, device=dev)
    rows = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), tokens - 1, dtype=torch.int32, device=dev)
    q1 = rnd(batch, heads, dim)
    o1 = torch.empty(batch, heads * dim, dtype=bf, device=dev)
    ms_f = _median_ms(torch, lambda: K.sink_attention_decode(q1, kc, vc, rows, pos, table, pages_per, 0,
                                                             o1, r1, r2, heads, kv, dim, dim, 0, chunk,
                                                             True, scale, chunk), flush=flush)
    ck, n_ck = decode_chunks(batch * kv, tokens)
    part = torch.empty(batch * heads * n_ck * (dim + 2), dtype=torch.float32, device=dev)
    ms_q = _median_ms(torch, lambda: K.attention_paged(q1, kc, vc, rows, pos, table, pages_per, 0, o1,
                                                       part, heads, kv, dim, 0, ck, n_ck, scale,
                                                       status=status, old_keys_final=True), flush=flush)
    seen_f = min(chunk, (tokens - 1) % chunk + 1)
    bw = pk["hbm_gbs"] * 1e9
    out["single"] = {
        "furitar_us": round(ms_f * 1e3, 1), "qwen2_us": round(ms_q * 1e3, 1),
        "furitar_keys": seen_f, "qwen2_keys": tokens,
        "furitar_frac": round(batch * kv * seen_f * 2 * dim * 2 / (ms_f * 1e-3) / bw, 4),
        "qwen2_frac": round(batch * kv * tokens * 2 * dim * 2 / (ms_q * 1e-3) / bw, 4)}
    return out


def workload_furitar(args) -> int:
    """Prefill of one 2,048-token prompt and decoding at batch 8 from 2,048-token contexts, for
    the Furitar design and for the Qwen2 decoder at equal width, heads, head size, layers and
    feed-forward weights, random weights, bfloat16; and the attention kernels of both alone."""
    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    pk, pk_kind = peaks()
    torch.cuda.set_device(0)
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler()
    clocks.start()
    t_all = time.time()
    sizes = []
    for name, width, heads, kv, dim, inter, chunk, layers in FURITAR_SIZES:
        cfg_f = furitar_config(width, heads, kv, dim, dim, inter * 3 // 2, chunk, layers,
                               FURITAR_VOCAB, CONTEXT)
        cfg_q = dict(CONFIG_7B, vocab_size=FURITAR_VOCAB, hidden_size=width, num_hidden_layers=layers,
                     num_attention_heads=heads, num_key_value_heads=kv, intermediate_size=inter,
                     max_position_embeddings=CONTEXT)
        entry = {"name": name, "width": width, "heads": heads, "kv_heads": kv, "head_size": dim,
                 "layers": layers, "chunk": chunk, "furitar_ff": inter * 3 // 2, "qwen2_intermediate": inter}
        for label, cfg in (("furitar", cfg_f), ("qwen2", cfg_q)):
            model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
            gen = Generator(model, max_tokens=BATCH * CONTEXT, max_batch=BATCH)
            engine = gen.engine
            g = torch.Generator().manual_seed(2)
            ids = torch.randint(0, FURITAR_VOCAB, (PROMPT,), generator=g).tolist()
            ms_prefill = time_prefill(engine, torch, ids, 10)
            flops = furitar_prefill_flops(cfg, PROMPT) if label == "furitar" else prefill_flops(cfg, PROMPT)
            ms_step, launched = time_decode(engine, torch, K, BATCH, steps, max(3, args.warmup), PROMPT)
            ms_med = time_decode.median_ms
            step_bytes = decode_bytes(model, BATCH, PROMPT + 3 + steps / 2)
            entry[label] = {
                "weights_gb": round(model.parameter_bytes() / 1e9, 3),
                "prefill_tokens_per_s": round(PROMPT * 1e3 / ms_prefill, 1),
                "prefill_ms": round(ms_prefill, 3),
                "prefill_frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(BATCH * 1e3 / ms_med, 1),
                "decode_ms_per_step": round(ms_med, 4), "decode_frac": _frac(step_bytes, ms_med, pk),
                "decode_launches_per_step": round(launched / steps, 1)}
            del gen, engine, model
            torch.cuda.empty_cache()
        entry["attention_kernels"] = furitar_attention_kernels(torch, K, pk, heads, kv, dim, chunk)
        sizes.append(entry)
    summary = clocks.summary((t_all, time.time()))
    clocks.stop()
    print(json.dumps({
        "workload": "furitar", "impl": "ours", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
        "metric": "prefill tokens/s of one 2048-token prompt and decode tokens/s at batch 8 from "
                  "2048-token contexts, Furitar beside Qwen2 at equal sizes",
        "unit": "tokens/s", "steps": steps, "prompt_len": PROMPT, "batch": BATCH,
        "fractions": f"prefill: flops over the {pk_kind} bf16 product peak; decode: bytes of the "
                     f"weights and of the visible cache over the {pk_kind} copy bandwidth",
        "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed before each run",
        "clocks": summary, "sizes": sizes}))
    return 0


# ------------------------------------------------------------------------------------------
# --workload budanex: the Budanex design beside the Qwen2 decoder at equal width and layer runs
# ------------------------------------------------------------------------------------------
# (name, width, attention heads, kv heads, head size, feed-forward width, state-space heads,
#  latent heads, window): six layers [state-space, latent attention + ff, attention + ff] x 2,
# the last three run twice (nine layer runs); Qwen2 beside it with nine layers
BUDANEX_SIZES = [("w2048", 2048, 16, 4, 128, 5632, 64, 16, 1024),
                 ("w4096", 4096, 32, 8, 128, 11264, 128, 32, 2048)]
BUDANEX_RUNS = 9


def budanex_config(width, heads, kv, dim, ff, ssm_heads, lat_heads, window, vocab):
    mamba = {"type": "mamba2", "mlp": None,
             "mixer": {"heads": ssm_heads, "vdim": 64, "state": 128, "groups": 1, "conv": 4,
                       "norm_groups": 1}}
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
              "mixer": {"heads": lat_heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 96,
                        "scale": 96 ** -0.5, "mask": {"size": window},
                        "rot": {"base": 500000.0, "dims": 32,
                                "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                           "scale": dim ** -0.5, "softcap": 50.0,
                           "rot": {"base": 1000000.0, "dims": dim // 2}}}
    return {"architecture": "Budanex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "logit_softcap": 30.0, "loop": {"start": 3, "stop": 6, "times": 2},
            "layers": [mamba, latent, attention, mamba, latent, attention]}


def budanex_prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only), the attention of the
    visible keys (latent attention in the form it is computed in: one shared key of kv_rank +
    rot_dim, values of kv_rank, and the two per-head products), and the recurrence."""
    w, n = cfg["width"], tokens
    lo, hi, times = cfg["loop"]["start"], cfg["loop"]["stop"], cfg["loop"]["times"]
    flops = 0.0
    for i, layer in enumerate(cfg["layers"]):
        runs = times if lo <= i < hi else 1
        m = layer["mixer"]
        if layer["type"] == "mamba2":
            inner = m["heads"] * m["vdim"]
            per_token = 2 * w * (2 * inner + 2 * m["groups"] * m["state"] + m["heads"]) + 2 * w * inner
            per_token += 6 * inner * m["state"]
            pairs = 0.0
        elif layer["type"] == "attention":
            per_token = 2 * w * ((m["heads"] + m["kv_heads"]) * m["dim"] + m["kv_heads"] * m["vdim"])
            per_token += 2 * w * m["heads"] * m["vdim"]
            pairs = m["heads"] * 2 * (m["dim"] + m["vdim"]) * n * (n + 1) / 2
        else:
            h, rank, rd = m["heads"], m["kv_rank"], m["rot_dim"]
            per_token = 2 * w * (h * (m["dim"] + rd) + rank + rd + h * m["vdim"]) + 2 * w * h * m["vdim"]
            per_token += 2 * h * rank * (m["dim"] + m["vdim"])
            c = m["mask"]["size"]
            seen = n * (n + 1) / 2 if n <= c else c * (c + 1) / 2 + (n - c) * c
            pairs = h * 2 * (2 * rank + rd) * seen
        if layer["mlp"] is not None:
            per_token += 6 * w * layer["mlp"]["ff"]
        flops += runs * (per_token * n + pairs)
    return flops + 2 * w * cfg["vocab"]


def budanex_kernels(torch, K, pk, width, heads, kv, dim, ssm_heads, lat_heads, window, tokens=2048,
                    batch=8):
    """The design's own kernels alone (median of 20, L2 flushed before each): device time and
    the fraction of the copy bandwidth their algorithmic bytes reach; for the attention kernels,
    the same kernel without the design's score modifiers beside it."""
    dev = "cuda:0"
    bw = pk["hbm_gbs"] * 1e9
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}

    def timed(name, fn, nbytes):
        ms = _median_ms(torch, fn, 20, flush)
        out[name] = {"us": round(ms * 1e3, 1), "frac_of_copy": round(nbytes / (ms * 1e-3) / bw, 4)}

    for label, n, rows in (("prompt", tokens, 1), ("decode", batch, batch)):
        per = n // rows
        P_, N = 64, 128
        inner, ch = ssm_heads * P_, ssm_heads * P_ + 2 * N
        in_w = 2 * inner + 2 * N + ssm_heads
        proj = torch.randn(n, in_w, device=dev)
        conv_w, conv_b = torch.randn(ch, 4, device=dev) * 0.3, torch.zeros(ch, device=dev)
        conv_state = torch.zeros(rows + 1, ch, 3, device=dev)
        ssm_state = torch.zeros(rows + 1, ssm_heads, P_, N, device=dev)
        token_row = torch.arange(rows, dtype=torch.int32, device=dev).repeat_interleave(per)
        cu = torch.arange(rows + 1, dtype=torch.int32, device=dev) * per
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
        u = torch.empty(n, ch, device=dev)
        y = torch.empty(n, inner, device=dev)
        g = torch.empty(n, inner, dtype=bf, device=dev)
        vec = {k_: torch.zeros(ssm_heads, device=dev) for k_ in ("dt", "a", "d")}
        nw = torch.ones(inner, device=dev)
        timed(f"conv_silu_{label}", lambda: K.conv_silu(proj, inner, ch, conv_w, conv_b, conv_state,
                                                         token_row, cu, slots, u, rows, single=(per == 1)),
              n * ch * 8 + (rows * ch * 3 * 8 if per == 1 else 0))
        timed(f"ssm_scan_{label}", lambda: K.ssm_scan(u, proj, inner + ch, vec["dt"], vec["a"], vec["d"],
                                                       ssm_state, cu, slots, y, rows, ssm_heads, P_, N, 1),
              n * (ch + inner + ssm_heads) * 4 + rows * ssm_heads * P_ * N * 8)
        timed(f"gated_group_norm_{label}", lambda: K.gated_group_norm(y, proj, 0, nw, g, 1, 1e-5),
              n * inner * (4 + 4 + 2))
        # latent attention: prepare, the two per-head products
        lw = lat_heads * 96 + 128 + lat_heads * 64
        lproj = torch.randn(n, lw, device=dev)
        q = torch.empty(n, lat_heads * 96, dtype=bf, device=dev)
        qa = torch.empty(n, lat_heads * 128, dtype=bf, device=dev)
        uk = (torch.randn(lat_heads, 96, 64, device=dev) * 0.1).to(bf)
        uv = (torch.randn(lat_heads, 64, 96, device=dev) * 0.1).to(bf)
        ol = torch.randn(n, lat_heads * 128, device=dev).to(bf)
        o = torch.empty(n, lat_heads * 64, dtype=bf, device=dev)
        timed(f"head_linear_uk_{label}", lambda: K.head_linear(q, uk, qa, x_head=96, x_off=0, y_head=128,
                                                               tail=32, x_tail_off=64),
              n * lat_heads * (96 + 128) * 2 + uk.numel() * 2)
        timed(f"head_linear_uv_gate_{label}", lambda: K.head_linear(ol, uv, o, x_head=128, x_off=0, y_head=64,
                                                                    gate=lproj, gate_off=lat_heads * 96 + 128),
              n * lat_heads * (96 * 2 + 64 * 2 + 64 * 4) + uv.numel() * 2)
    # attention kernels with and without the design's modifiers, over packed keys (a prompt) ...
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    cu1 = torch.tensor([0, tokens], dtype=torch.int32, device=dev)
    peak = pk["bf16_tflops"] * 1e12
    for name, nh, nk, hd, vd, win, cap, with_sink in (("attention", heads, kv, dim, dim, 0, 50.0, False),
                                                       ("latent", lat_heads, 1, 128, 128, window, 0.0, True)):
        qq = (torch.randn(tokens, nh, hd, device=dev) * 0.5).to(bf)
        kk = (torch.randn(tokens, nk, hd, device=dev) * 0.5).to(bf)
        vv = torch.randn(tokens, nk, vd, device=dev).to(bf)
        oo = torch.empty(tokens, nh * vd, dtype=bf, device=dev)
        sink = torch.zeros(nh, device=dev) if with_sink else None
        pairs = tokens * (tokens + 1) / 2 if not win or tokens <= win else win * (win + 1) / 2 + (tokens - win) * win
        fl = nh * 2 * (hd + vd) * pairs
        for tag, c, sk in (("", cap, sink), ("_plain_scores", 0.0, None)):
            ms = _median_ms(torch, lambda: K.sink_attention_mma(
                qq, kk, vv, cu1, None, None, 0, 0, oo, None, None, 1, tokens, nh, nk, hd, vd, win, 0,
                with_sink, hd ** -0.5, sink_logit=sk, softcap=c), 20, flush)
            out[f"{name}_prompt_mma{tag}"] = {"us": round(ms * 1e3, 1),
                                              "frac_of_product_peak": round(fl / (ms * 1e-3) / peak, 4)}
        if hd == vd:
            for tag, c, sk in (("", cap, sink), ("_plain_scores", 0.0, None)):
                ms = _median_ms(torch, lambda: K.sink_attention_tc(
                    qq, kk, vv, cu1, None, None, 0, 0, oo, None, None, 1, tokens, nh, nk, hd, win, 0,
                    with_sink, hd ** -0.5, status, sink_logit=sk, softcap=c), 20, flush)
                out[f"{name}_prompt_tcgen05{tag}"] = {"us": round(ms * 1e3, 1),
                                                      "frac_of_product_peak": round(fl / (ms * 1e-3) / peak, 4)}
            ms = _median_ms(torch, lambda: K.attention_prefill_tc(qq, kk, vv, cu1, oo, 1, tokens, nh, nk, hd,
                                                                  win, hd ** -0.5, status), 20, flush)
            out[f"{name}_prompt_qwen2_tcgen05"] = {"us": round(ms * 1e3, 1),
                                                   "frac_of_product_peak": round(fl / (ms * 1e-3) / peak, 4)}
        # ... and single queries over the cache
        pages = batch * (tokens // 64)
        kc = (torch.randn(pages, nk, 64, hd, device=dev) * 0.5).to(bf)
        vc = torch.randn(pages, nk, 64, vd, device=dev).to(bf)
        table = torch.arange(pages, dtype=torch.int32, device=dev)
        rows_i = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), tokens - 1, dtype=torch.int32, device=dev)
        q1 = (torch.randn(batch, nh, hd, device=dev) * 0.5).to(bf)
        o1 = torch.empty(batch, nh * vd, dtype=bf, device=dev)
        seen = min(tokens, win) if win else tokens
        nbytes = batch * nk * seen * (hd + vd) * 2
        for tag, c, sk in (("", cap, sink), ("_plain_scores", 0.0, None)):
            ms = _median_ms(torch, lambda: K.sink_attention_decode(
                q1, kc, vc, rows_i, pos, table, tokens // 64, 0, o1, None, None, nh, nk, hd, vd, win, 0,
                with_sink, hd ** -0.5, seen, sink_logit=sk, softcap=c), 20, flush)
            out[f"{name}_decode_mma{tag}"] = {"us": round(ms * 1e3, 1), "keys": seen,
                                              "frac_of_copy": round(nbytes / (ms * 1e-3) / bw, 4)}
    return out


def workload_budanex(args) -> int:
    """Prefill of one 2,048-token prompt and decoding at batch 8 from 2,048-token contexts, for
    the Budanex design (state-space, latent-attention and attention layers, three of them run
    twice) and for the Qwen2 decoder at equal width, feed-forward width and layer runs, random
    weights, bfloat16; and the design's kernels alone."""
    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    pk, pk_kind = peaks()
    torch.cuda.set_device(0)
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler()
    clocks.start()
    t_all = time.time()
    sizes = []
    for name, width, heads, kv, dim, ff, ssm_heads, lat_heads, window in BUDANEX_SIZES:
        cfg_b = budanex_config(width, heads, kv, dim, ff, ssm_heads, lat_heads, window, FURITAR_VOCAB)
        cfg_q = dict(CONFIG_7B, vocab_size=FURITAR_VOCAB, hidden_size=width,
                     num_hidden_layers=BUDANEX_RUNS, num_attention_heads=heads,
                     num_key_value_heads=kv, intermediate_size=ff, max_position_embeddings=CONTEXT)
        entry = {"name": name, "width": width, "heads": heads, "kv_heads": kv, "head_size": dim,
                 "feed_forward": ff, "state_space_heads": ssm_heads, "latent_heads": lat_heads,
                 "window": window, "layer_runs": BUDANEX_RUNS}
        for label, cfg in (("budanex", cfg_b), ("qwen2", cfg_q)):
            model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
            gen = Generator(model, max_tokens=BATCH * CONTEXT, max_batch=BATCH)
            engine = gen.engine
            g = torch.Generator().manual_seed(2)
            ids = torch.randint(0, FURITAR_VOCAB, (PROMPT,), generator=g).tolist()
            ms_prefill = time_prefill(engine, torch, ids, 10)
            flops = budanex_prefill_flops(cfg, PROMPT) if label == "budanex" else prefill_flops(cfg, PROMPT)
            ms_step, launched = time_decode(engine, torch, K, BATCH, steps, max(3, args.warmup), PROMPT)
            ms_med = time_decode.median_ms
            step_bytes = decode_bytes(model, BATCH, PROMPT + 3 + steps / 2)
            entry[label] = {
                "weights_gb": round(model.parameter_bytes() / 1e9, 3),
                "prefill_tokens_per_s": round(PROMPT * 1e3 / ms_prefill, 1),
                "prefill_ms": round(ms_prefill, 3),
                "prefill_frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(BATCH * 1e3 / ms_med, 1),
                "decode_ms_per_step": round(ms_med, 4), "decode_frac": _frac(step_bytes, ms_med, pk),
                "decode_launches_per_step": round(launched / steps, 1)}
            del gen, engine, model
            torch.cuda.empty_cache()
        entry["kernels"] = budanex_kernels(torch, K, pk, width, heads, kv, dim, ssm_heads, lat_heads, window)
        sizes.append(entry)
    summary = clocks.summary((t_all, time.time()))
    clocks.stop()
    print(json.dumps({
        "workload": "budanex", "impl": "ours", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
        "metric": "prefill tokens/s of one 2048-token prompt and decode tokens/s at batch 8 from "
                  "2048-token contexts, Budanex beside Qwen2 at equal width and layer runs",
        "unit": "tokens/s", "steps": steps, "prompt_len": PROMPT, "batch": BATCH,
        "fractions": f"prefill: flops over the {pk_kind} bf16 product peak; decode: bytes of the "
                     f"weights, the visible cache and the recurrent state over the {pk_kind} copy "
                     f"bandwidth",
        "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed before each run",
        "clocks": summary, "sizes": sizes}))
    return 0


# --workload bedarax: the Bedarax design beside the Qwen2 decoder at equal width and layers
# ------------------------------------------------------------------------------------------
# (name, width, attention heads, kv heads, head size, feed-forward width, recurrent heads, their
#  query/key heads, window, experts, experts a token): six layers [delta rule + routed experts,
# talking attention + dense PolyNorm feed-forward, channel-wise delta rule + routed experts] x 2;
# an expert is half as wide as the dense feed-forward, so two of them make its width
BEDARAX_SIZES = [("w2048", 2048, 16, 4, 128, 5632, 16, 8, 1024, 8, 2),
                 ("w4096", 4096, 32, 8, 128, 11264, 32, 16, 2048, 8, 2)]
BEDARAX_LAYERS = 6


def bedarax_config(width, heads, kv, dim, ff, rec_heads, rec_kv, window, experts, top, vocab):
    moe = {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": experts, "top": top}}
    delta = {"type": "delta", "mlp": moe,
             "mixer": {"heads": rec_heads, "kv_heads": rec_kv, "dim": 128, "vdim": 128, "conv": 4}}
    channel = {"type": "channel_delta", "mlp": moe,
               "mixer": {"heads": rec_heads, "kv_heads": rec_kv, "dim": 128, "vdim": 128, "conv": 4,
                         "a_rank": 64, "g_rank": 64}}
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                           "scale": dim ** -0.5, "mask": {"size": window}, "v_mix": True}}
    return {"architecture": "Bedarax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [delta, attention, channel, delta, attention, channel]}


def bedarax_prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only; the experts a token
    uses, not all), the attention of the visible keys with the mix of the heads' scores, and the
    recurrence (decay, two products with the state and the rank-one update per token)."""
    w, n = cfg["width"], tokens
    flops = 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        pairs = 0.0
        if layer["type"] == "attention":
            per_token = 2 * w * (h * d + g * d + g * dv + h) + 2 * w * h * dv
            c = m["mask"]["size"]
            seen = n * (n + 1) / 2 if n <= c else c * (c + 1) / 2 + (n - c) * c
            pairs = (h * 2 * (d + dv) + 2 * h * h) * seen
        else:
            a_in = m.get("a_rank", 0) or h
            g_in = m.get("g_rank", 0) or h * dv
            per_token = 2 * w * (2 * g * d + h * dv + h + a_in + g_in) + 2 * w * h * dv
            if layer["type"] == "channel_delta":
                per_token += 2 * m["a_rank"] * h * d + 2 * m["g_rank"] * h * dv
            per_token += 8 * h * d * dv
        mlp = layer["mlp"]
        if mlp is not None and mlp["kind"] == "dense":
            per_token += 4 * w * mlp["ff"]
        elif mlp is not None:
            per_token += mlp["router"]["top"] * 6 * w * mlp["expert"]["ff"] + 2 * w * mlp["router"]["experts"]
        flops += per_token * n + pairs
    return flops + 2 * w * cfg["vocab"]


def bedarax_decode_bytes(model, cfg, batch, context_tokens):
    """``decode_bytes`` with the experts a step can touch at most (batch x top of each layer's)
    in place of all of them."""
    total = decode_bytes(model, batch, context_tokens)
    for layer in cfg["layers"]:
        mlp = layer["mlp"]
        if mlp is not None and mlp["kind"] == "moe":
            experts, top = mlp["router"]["experts"], mlp["router"]["top"]
            idle = max(0, experts - batch * top)
            total -= idle * 3 * cfg["width"] * mlp["expert"]["ff"] * 2
    return total


def bedarax_kernels(torch, K, pk, width, heads, kv, dim, ff, rec_heads, rec_kv, window, experts, top,
                    tokens=2048, batch=8):
    """The design's own kernels alone (median of 20, L2 flushed before each): device time and the
    fraction of the copy bandwidth (or of the product peak) their algorithmic bytes (flops) reach,
    each beside the like kernel of another design at equal sizes."""
    dev = "cuda:0"
    bw = pk["hbm_gbs"] * 1e9
    peak = pk["bf16_tflops"] * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}

    def timed(name, fn, nbytes):
        ms = _median_ms(torch, fn, 20, flush)
        out[name] = {"us": round(ms * 1e3, 1), "frac_of_copy": round(nbytes / (ms * 1e-3) / bw, 4)}

    D = Dv = 128
    for label, n, rows in (("prompt", tokens, 1), ("decode", batch, batch)):
        per = n // rows
        qk, vw = rec_kv * D, rec_heads * Dv
        ch = 2 * qk + vw
        token_row = torch.arange(rows, dtype=torch.int32, device=dev).repeat_interleave(per)
        cu = torch.arange(rows + 1, dtype=torch.int32, device=dev) * per
        slots = torch.arange(rows, dtype=torch.int32, device=dev)
        for kind, n_decay in (("head", rec_heads), ("channel", rec_heads * D)):
            proj = torch.randn(n, ch + rec_heads, device=dev)
            decay = torch.randn(n, n_decay, device=dev)
            gate = torch.randn(n, vw, device=dev)
            u = torch.randn(n, ch, device=dev) * 0.5
            state = torch.zeros(rows + 1, rec_heads, Dv, D, device=dev)
            dt_bias = torch.full((n_decay,), -1.0, device=dev)
            a_log = torch.zeros(rec_heads, device=dev)
            o = torch.empty(n, vw, device=dev)
            timed(f"delta_scan_{kind}_{label}",
                  lambda: K.delta_scan(u, 0, qk, 2 * qk, proj, ch, decay, 0, dt_bias, a_log, state, cu,
                                       slots, o, rows, per, rec_heads, rec_kv, D, Dv, kind == "channel"),
                  n * (ch + rec_heads + n_decay + vw) * 4 + rows * rec_heads * D * Dv * 8)
            out[f"delta_scan_{kind}_{label}"]["frac_of_fp32_fma"] = round(
                n * rec_heads * D * Dv * 4 / (out[f"delta_scan_{kind}_{label}"]["us"] * 1e-6)
                / (148 * 128 * 1.9e9), 4)
        g16 = torch.empty(n, vw, dtype=bf, device=dev)
        nw = torch.ones(Dv, device=dev)
        timed(f"head_norm_gate_{label}", lambda: K.head_norm_gate(o, gate, 0, nw, g16, rec_heads, Dv,
                                                                   1e-5, "silu"),
              n * vw * (4 + 4 + 2))
        conv_w = torch.randn(ch, 4, device=dev) * 0.3
        conv_state = torch.zeros(rows + 1, ch, 3, device=dev)
        praw = torch.randn(n, ch, device=dev)
        timed(f"conv_silu_{label}", lambda: K.conv_silu(praw, 0, ch, conv_w, None, conv_state, token_row,
                                                         cu, slots, u, rows, single=(per == 1)),
              n * ch * 8 + (rows * ch * 3 * 8 if per == 1 else 0))
        # the state-space scan of the Budanex design at an equal state (heads x 64 x 128 floats)
        sh, P_, N = rec_heads * 2, 64, 128
        inner, sch = sh * P_, sh * P_ + 2 * N
        sproj = torch.randn(n, 2 * inner + 2 * N + sh, device=dev)
        su = torch.randn(n, sch, device=dev) * 0.5
        sstate = torch.zeros(rows + 1, sh, P_, N, device=dev)
        sy = torch.empty(n, inner, device=dev)
        zero = torch.zeros(sh, device=dev)
        timed(f"budanex_ssm_scan_{label}", lambda: K.ssm_scan(su, sproj, inner + sch, zero, zero, zero,
                                                               sstate, cu, slots, sy, rows, sh, P_, N, 1),
              n * (sch + inner + sh) * 4 + rows * sh * P_ * N * 8)
        out[f"budanex_ssm_scan_{label}"]["frac_of_fp32_fma"] = round(
            n * sh * P_ * N * 3 / (out[f"budanex_ssm_scan_{label}"]["us"] * 1e-6) / (148 * 128 * 1.9e9), 4)
        # the stream's row-wise kernels
        z = torch.randn(n, ff, device=dev)
        zo = torch.empty(n, ff, dtype=bf, device=dev)
        coef = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
        timed(f"poly_norm_{label}", lambda: K.poly_norm(z, coef, zo, 1e-5), n * ff * 6)
        hist = torch.randn(BEDARAX_LAYERS + 1, n, width, device=dev)
        last = torch.randn(n, width, device=dev)
        wts = torch.randn(BEDARAX_LAYERS + 1, device=dev)
        timed(f"depth_mix_{label}", lambda: K.depth_mix(hist, BEDARAX_LAYERS, None, last, wts, last),
              (BEDARAX_LAYERS + 2) * n * width * 4)
        nv = kv * dim
        aproj = torch.randn(n, heads * dim + 2 * nv + heads, device=dev)
        first = torch.randn(n, heads * dim + 2 * nv + heads, device=dev)
        lam = torch.tensor(0.4, device=dev)
        timed(f"value_mix_{label}", lambda: K.value_mix(aproj, heads * dim + nv, first, heads * dim + nv,
                                                        lam, nv), n * nv * 12)
    # routed experts, the per-token kernels of a decode step: every chosen expert's matrices once
    x8 = torch.randn(batch, width, device=dev).to(bf)
    eff = ff // 2
    wg = (torch.randn(experts, 2 * eff, width, device=dev) * 0.02).to(bf)
    pairs = wg.view(experts, eff, 2, width)
    wd = (torch.randn(experts, width, eff, device=dev) * 0.02).to(bf)
    logits = torch.randn(batch, experts, device=dev)
    idx = torch.empty(batch, top, dtype=torch.int32, device=dev)
    rw = torch.empty(batch, top, device=dev)
    hidden = torch.empty(batch, top, eff, dtype=bf, device=dev)
    res = torch.zeros(batch, width, device=dev)
    timed("moe_route_decode", lambda: K.moe_route(logits, idx, rw, top), batch * experts * 4)
    K.moe_route(logits, idx, rw, top)
    timed("moe_experts_decode", lambda: K.moe_experts(x8, pairs[:, :, 0], pairs[:, :, 1], wd, idx, rw,
                                                      hidden, res),
          batch * top * 3 * eff * width * 2)
    # attention: the talking kernel beside the plain-score kernels at equal sizes
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    cu1 = torch.tensor([0, tokens], dtype=torch.int32, device=dev)
    qq = (torch.randn(tokens, heads, dim, device=dev) * 0.5).to(bf)
    kk = (torch.randn(tokens, kv, dim, device=dev) * 0.5).to(bf)
    vv = torch.randn(tokens, kv, dim, device=dev).to(bf)
    oo = torch.empty(tokens, heads * dim, dtype=bf, device=dev)
    talk = torch.eye(heads, device=dev) + torch.randn(heads, heads, device=dev) * 0.1
    gate = torch.randn(tokens, heads, device=dev)
    row_seq = torch.zeros(tokens, dtype=torch.int32, device=dev)
    row_pos = torch.arange(tokens, dtype=torch.int32, device=dev)
    seen = tokens * (tokens + 1) / 2 if tokens <= window else window * (window + 1) / 2 + (tokens - window) * window
    fl = heads * 2 * (dim + dim) * seen

    def product_frac(name, fn):
        ms = _median_ms(torch, fn, 10, flush)
        out[name] = {"us": round(ms * 1e3, 1), "frac_of_product_peak": round(fl / (ms * 1e-3) / peak, 4)}

    product_frac("talk_attention_prompt", lambda: K.talk_attention(
        qq, kk, vv, row_seq, row_pos, cu1, None, 0, 0, talk, gate, 0, oo, heads, kv, dim, dim, window,
        dim ** -0.5, q_cu_seqlens=cu1, n_seq=1, max_row_tokens=tokens))
    product_frac("talk_attention_prompt_a_query_a_block", lambda: K.talk_attention(
        qq, kk, vv, row_seq, row_pos, cu1, None, 0, 0, talk, gate, 0, oo, heads, kv, dim, dim, window,
        dim ** -0.5))
    product_frac("plain_attention_prompt_mma", lambda: K.sink_attention_mma(
        qq, kk, vv, cu1, None, None, 0, 0, oo, None, None, 1, tokens, heads, kv, dim, dim, window, 0,
        False, dim ** -0.5))
    product_frac("plain_attention_prompt_tcgen05", lambda: K.attention_prefill_tc(
        qq, kk, vv, cu1, oo, 1, tokens, heads, kv, dim, window, dim ** -0.5, status))
    n_pages = batch * (tokens // 64)
    kc = (torch.randn(n_pages, kv, 64, dim, device=dev) * 0.5).to(bf)
    vc = torch.randn(n_pages, kv, 64, dim, device=dev).to(bf)
    table = torch.arange(n_pages, dtype=torch.int32, device=dev)
    rows_i = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), tokens - 1, dtype=torch.int32, device=dev)
    q1 = (torch.randn(batch, heads, dim, device=dev) * 0.5).to(bf)
    o1 = torch.empty(batch, heads * dim, dtype=bf, device=dev)
    reach = min(tokens, window)
    nbytes = batch * kv * reach * 2 * dim * 2
    cu_b = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    timed("talk_attention_decode", lambda: K.talk_attention(
        q1, kc, vc, rows_i, pos, None, table, tokens // 64, 0, talk, gate, 0, o1, heads, kv, dim, dim,
        window, dim ** -0.5, reach_keys=reach, q_cu_seqlens=cu_b, n_seq=batch, max_row_tokens=1), nbytes)
    timed("talk_attention_decode_a_query_a_block", lambda: K.talk_attention(
        q1, kc, vc, rows_i, pos, None, table, tokens // 64, 0, talk, gate, 0, o1, heads, kv, dim, dim,
        window, dim ** -0.5, reach_keys=reach), nbytes)
    timed("plain_attention_decode_mma", lambda: K.sink_attention_decode(
        q1, kc, vc, rows_i, pos, table, tokens // 64, 0, o1, None, None, heads, kv, dim, dim, window, 0,
        False, dim ** -0.5, reach), nbytes)
    return out


def workload_bedarax(args) -> int:
    """Prefill of one 2,048-token prompt and decoding at batch 8 from 2,048-token contexts, for
    the Bedarax design (delta-rule, talking-attention and channel-wise delta-rule layers with
    routed and dense feed-forwards) and for the Qwen2 decoder at equal width, heads, feed-forward
    width and layers, random weights, bfloat16; and the design's kernels alone."""
    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    pk, pk_kind = peaks()
    torch.cuda.set_device(0)
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler()
    clocks.start()
    t_all = time.time()
    sizes = []
    for name, width, heads, kv, dim, ff, rec_heads, rec_kv, window, experts, top in BEDARAX_SIZES:
        cfg_b = bedarax_config(width, heads, kv, dim, ff, rec_heads, rec_kv, window, experts, top,
                               FURITAR_VOCAB)
        cfg_q = dict(CONFIG_7B, vocab_size=FURITAR_VOCAB, hidden_size=width,
                     num_hidden_layers=BEDARAX_LAYERS, num_attention_heads=heads,
                     num_key_value_heads=kv, intermediate_size=ff, max_position_embeddings=CONTEXT)
        entry = {"name": name, "width": width, "heads": heads, "kv_heads": kv, "head_size": dim,
                 "feed_forward": ff, "recurrent_heads": rec_heads, "recurrent_qk_heads": rec_kv,
                 "window": window, "experts": experts, "experts_a_token": top,
                 "layers": BEDARAX_LAYERS}
        for label, cfg in (("bedarax", cfg_b), ("qwen2", cfg_q)):
            model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
            gen = Generator(model, max_tokens=BATCH * CONTEXT, max_batch=BATCH)
            engine = gen.engine
            g = torch.Generator().manual_seed(2)
            ids = torch.randint(0, FURITAR_VOCAB, (PROMPT,), generator=g).tolist()
            ms_prefill = time_prefill(engine, torch, ids, 10)
            flops = bedarax_prefill_flops(cfg, PROMPT) if label == "bedarax" else prefill_flops(cfg, PROMPT)
            ms_step, launched = time_decode(engine, torch, K, BATCH, steps, max(3, args.warmup), PROMPT)
            ms_med = time_decode.median_ms
            context = PROMPT + 3 + steps / 2
            step_bytes = (bedarax_decode_bytes(model, cfg, BATCH, context) if label == "bedarax"
                          else decode_bytes(model, BATCH, context))
            entry[label] = {
                "weights_gb": round(model.parameter_bytes() / 1e9, 3),
                "prefill_tokens_per_s": round(PROMPT * 1e3 / ms_prefill, 1),
                "prefill_ms": round(ms_prefill, 3),
                "prefill_frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(BATCH * 1e3 / ms_med, 1),
                "decode_ms_per_step": round(ms_med, 4), "decode_frac": _frac(step_bytes, ms_med, pk),
                "decode_launches_per_step": round(launched / steps, 1)}
            del gen, engine, model
            torch.cuda.empty_cache()
        entry["kernels"] = bedarax_kernels(torch, K, pk, width, heads, kv, dim, ff, rec_heads, rec_kv,
                                           window, experts, top)
        sizes.append(entry)
    summary = clocks.summary((t_all, time.time()))
    clocks.stop()
    print(json.dumps({
        "workload": "bedarax", "impl": "ours", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
        "metric": "prefill tokens/s of one 2048-token prompt and decode tokens/s at batch 8 from "
                  "2048-token contexts, Bedarax beside Qwen2 at equal width and layers",
        "unit": "tokens/s", "steps": steps, "prompt_len": PROMPT, "batch": BATCH,
        "fractions": f"prefill: flops over the {pk_kind} bf16 product peak; decode: bytes of the "
                     f"weights a step can touch, the visible cache and the recurrent state over "
                     f"the {pk_kind} copy bandwidth",
        "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed before each run",
        "clocks": summary, "sizes": sizes}))
    return 0


# ------------------------------------------------------------------------------------------
# --workload zanelorn: the Zanelorn design beside the Qwen2 decoder at equal width and layers
# ------------------------------------------------------------------------------------------
# (name, width, attention heads, kv heads, head size, feed-forward width, retention heads, window,
#  experts, experts a token): six layers, retention and parallel (attention + selective scan) in
# turn, with routed and dense feed-forwards in turn; an expert is half as wide as the dense
# feed-forward; retention keys of 128 with values of 256; the scan as wide as the model, 16 state
# numbers a channel, a step-size rank of width / 16
ZANELORN_SIZES = [("w2048", 2048, 16, 4, 128, 5632, 8, 1024, 8, 2),
                  ("w4096", 4096, 32, 8, 128, 11264, 16, 2048, 8, 2)]
ZANELORN_LAYERS = 6
ZANELORN_KEEP = 4


def zanelorn_config(width, heads, kv, dim, ff, ret_heads, window, experts, top, vocab):
    moe = {"kind": "moe", "expert": {"ff": ff // 2, "limit": 7.0},
           "router": {"experts": experts, "identity": 1, "top": top},
           "shared": {"ff": ff // 2, "limit": 7.0}}
    dense = {"kind": "dense", "ff": ff}
    retention = {"type": "retention",
                 "mixer": {"heads": ret_heads, "dim": 128, "vdim": 256,
                           "decay": [1.0 - 0.03 / (1 + i % 4) for i in range(ret_heads)],
                           "rot": {"base": 500000.0, "dims": 64}}}
    parallel = {"type": "parallel",
                "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                                   "scale": dim ** -0.5, "mask": {"size": window, "keep_first": ZANELORN_KEEP},
                                   "rot": {"base": 100000.0, "dims": 64, "scaling": {"factor": 8.0}}},
                          "right": {"inner": width, "state": 16, "dt_rank": width // 16, "conv": 4},
                          "left_scale": 1.0, "right_scale": 0.75}}
    layers = []
    for i in range(ZANELORN_LAYERS):
        layers.append(dict(retention if i % 2 == 0 else parallel, mlp=moe if i % 3 == 0 else dense))
    return {"architecture": "Zanelorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "embedding": {"scale": 12.0}, "token_side": {"dim": 64},
            "layers": layers}


def zanelorn_prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only; the experts a token
    uses, not all), the attention of the visible keys, and the recurrences (per token and state
    element: decay, update and read-out)."""
    w, n = cfg["width"], tokens
    side = (cfg.get("token_side") or {}).get("dim", 0)
    flops = 0.0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        pairs = 0.0
        if layer["type"] == "retention":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            per_token = 2 * w * (2 * h * d + 2 * h * dv) + 2 * w * h * dv + 4 * h * d * dv
        else:
            a, r = m["left"], m["right"]
            h, g, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            per_token = 2 * w * (h * d + g * d + g * dv + h * dv) + 2 * w * h * dv
            c = a["mask"]["size"]
            seen = n * (n + 1) / 2 if n <= c else c * (c + 1) / 2 + (n - c) * c
            pairs = h * 2 * (d + dv) * seen
            ci, ns, rk = r["inner"], r["state"], r["dt_rank"]
            per_token += 2 * w * 2 * ci + 2 * ci * (rk + 2 * ns) + 2 * rk * ci + 2 * w * ci + 6 * ci * ns
        mlp = layer["mlp"]
        if mlp is not None and mlp["kind"] == "dense":
            per_token += 4 * w * mlp["ff"]
        elif mlp is not None:
            per_token += mlp["router"]["top"] * 6 * w * mlp["expert"]["ff"] + 2 * w * (mlp["router"]["experts"] + 2)
            if mlp.get("shared"):
                per_token += 6 * w * mlp["shared"]["ff"]
        per_token += 4 * w * side
        flops += per_token * n + pairs
    return flops + 2 * w * cfg["vocab"]


def zanelorn_decode_bytes(model, cfg, batch, context_tokens):
    """Bytes a decode step must read: the weights it can touch (at most batch x top of each
    layer's experts, one row of each table per sequence), the visible keys and values and the
    recurrent states (read and written)."""
    total = model.parameter_bytes()
    w = cfg["width"]
    total -= cfg["vocab"] * w * 2                                     # the embedding: rows, not the table
    side = (cfg.get("token_side") or {}).get("dim", 0)
    total -= cfg["vocab"] * side * len(cfg["layers"]) * 2
    for layer in cfg["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        if mlp is not None and mlp["kind"] == "moe":
            idle = max(0, mlp["router"]["experts"] - batch * mlp["router"]["top"])
            total -= idle * 3 * w * mlp["expert"]["ff"] * 2
        if layer["type"] == "retention":
            total += batch * 2 * m["heads"] * m["dim"] * m["vdim"] * 4
        else:
            a, r = m["left"], m["right"]
            seen = min(context_tokens, a["mask"]["size"] + a["mask"].get("keep_first", 0))
            total += batch * seen * a["kv_heads"] * (a["dim"] + a["vdim"]) * 2
            total += batch * 2 * r["inner"] * r["state"] * 4
    return total


def zanelorn_kernels(torch, K, pk, width, heads, kv, dim, ret_heads, window, tokens=2048, batch=8):
    """The design's own kernels alone (median of 20, L2 flushed before each): device time and the
    fraction of the copy bandwidth (or of the product peak) their algorithmic bytes (flops) reach,
    each beside the like kernel of another design at equal sizes."""
    from minfer_b200.parts.base import CacheView, StepContext
    from minfer_b200.parts.sink_attention import ScoreSpec, scored_attention
    dev = "cuda:0"
    bw = pk["hbm_gbs"] * 1e9
    peak = pk["bf16_tflops"] * 1e12
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {}

    def timed(name, fn, nbytes=None, flops=None):
        ms = _median_ms(torch, fn, 20, flush)
        out[name] = {"us": round(ms * 1e3, 1)}
        if nbytes is not None:
            out[name]["frac_of_copy"] = round(nbytes / (ms * 1e-3) / bw, 4)
        if flops is not None:
            out[name]["frac_of_product_peak"] = round(flops / (ms * 1e-3) / peak, 4)

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    D, Dv, N = 128, 256, 16
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for label, n, rows in (("prompt", tokens, 1), ("decode", batch, batch)):
        per = n // rows
        cu, slots = i32([per * b for b in range(rows + 1)]), i32(list(range(rows)))
        positions = i32([tokens + (t % per) if label == "decode" else t for t in range(n)])
        token_row = i32([t // per for t in range(n)])
        # ---- retention: prepare, scan, norm and gate --------------------------------------------
        H = ret_heads
        proj = torch.randn(n, 2 * H * D + 2 * H * Dv, device=dev)
        q = torch.empty(n, H, D, device=dev)
        k = torch.empty(n, H, D, device=dev)
        inv = torch.tensor([5e5 ** (-2.0 * i / 64) for i in range(32)], dtype=torch.float64, device=dev)
        decay = torch.full((H,), 0.97, device=dev)
        state = torch.zeros(rows, H, Dv, D, device=dev)
        o = torch.empty(n, H * Dv, device=dev)
        gated = torch.empty(n, H * Dv, dtype=bf, device=dev)
        timed(f"head_prepare_retention_{label}", lambda: K.head_prepare(
            proj, positions, token_row, cu[1:], q, k, None, None, None, None, 0, 0, q_off=0, n_heads=H,
            q_width=D, k_off=H * D, n_kv=H, k_width=D, v_off=2 * H * D, v_width=Dv, q_norm=None, k_norm=None,
            eps=1e-6, inv_freq=inv, rot_dims=64, rot_style=0, rot_magnitude=1.0, q_mul=1.0, k_mul=D ** -0.5,
            status=status), nbytes=n * 2 * H * D * 8)
        scan_bytes = n * (2 * H * D + 2 * H * Dv) * 4 + rows * 2 * H * D * Dv * 4
        timed(f"retention_scan_{label}", lambda: K.retention_scan(q, k, proj, 2 * H * D, decay, state, cu,
                                                                  slots, o, rows),
              nbytes=scan_bytes, flops=None)
        out[f"retention_scan_{label}"]["frac_of_fp32_pipe"] = round(
            4.0 * n * H * D * Dv / (out[f"retention_scan_{label}"]["us"] * 1e-6) / 80e12, 4)
        timed(f"unit_norm_gate_{label}", lambda: K.unit_norm_gate(o, proj, 2 * H * D + H * Dv, gated, H, 1e-6,
                                                                  "silu", 1.0), nbytes=n * H * Dv * 10)
        # ---- the selective scan, beside the scalar-decay scan of the Mamba-2 form -------------------
        C = width
        u = torch.randn(n, C, device=dev)
        dt_raw = torch.randn(n, C, device=dev)
        bc = torch.randn(n, 2 * N, device=dev)
        z = torch.randn(n, 2 * C, device=dev)
        a_log, d_skip = torch.randn(C, N, device=dev) * 0.5, torch.ones(C, device=dev)
        sstate = torch.zeros(rows, C, N, device=dev)
        y = torch.empty(n, C, dtype=bf, device=dev)
        timed(f"selective_scan_{label}", lambda: K.selective_scan(u, dt_raw, bc, 0, N, z, C, a_log, d_skip,
                                                                  sstate, cu, slots, y, rows, 0.75),
              nbytes=n * C * 14 + n * 2 * N * 4 + rows * 2 * C * N * 4)
        P_, N2 = 64, 128
        heads2 = C // P_
        u2 = torch.randn(n, C + 2 * N2, device=dev)
        proj2 = torch.randn(n, heads2, device=dev)
        st2 = torch.zeros(rows, heads2, P_, N2, device=dev)
        y2 = torch.empty(n, C, device=dev)
        ones = torch.ones(heads2, device=dev)
        timed(f"like:ssm_scan_{label}", lambda: K.ssm_scan(u2, proj2, 0, ones, ones, ones, st2, cu, slots,
                                                          y2, rows, heads2, P_, N2, 1),
              nbytes=n * (2 * C + 2 * N2) * 4 + rows * 2 * C * N2 * 4)
        # ---- the output-norm add and the per-token input ---------------------------------------------
        h = torch.randn(n, width, device=dev)
        yv = torch.randn(n, width, device=dev)
        wv = torch.ones(width, device=dev)
        timed(f"norm_add_{label}", lambda: K.norm_add(h, yv, wv, 1e-6, 0.5), nbytes=n * width * 12)
        xo = torch.empty(n, width, dtype=bf, device=dev)
        timed(f"like:rmsnorm_{label}", lambda: K.rmsnorm(h, wv, 1e-6, xo), nbytes=n * width * 6)
        # ---- attention with a window that keeps the first tokens, beside the same without them ---------
        qa = torch.randn(n, heads, dim, device=dev).to(bf)
        o2 = torch.empty(n, heads * dim, dtype=bf, device=dev)
        if label == "prompt":
            ka = torch.randn(n, kv, dim, device=dev).to(bf)
            va = torch.randn(n, kv, dim, device=dev).to(bf)
            ctx = StepContext(device=torch.device(dev), act_dtype=bf, n_tokens=n, n_rows=1, token_ids=positions,
                              positions=positions, token_row=token_row, cu_seqlens=cu, seq_end=cu[1:], slots=slots,
                              from_start=True, single_token=False, max_row_tokens=n, max_end=n, status=status)
            seen = window * (window + 1) / 2 + (n - window) * window if n > window else n * (n + 1) / 2
            fl = heads * 4 * dim * seen
            for name, keep in (("attention_kept_first_prompt", ZANELORN_KEEP), ("like:attention_window_prompt", 0)):
                spec = ScoreSpec(n_heads=heads, n_kv_heads=kv, head_dim=dim, value_dim=dim, scale=dim ** -0.5,
                                 window=window, keep_first=keep)
                timed(name, lambda: scored_attention(spec, qa, ka, va, None, ctx, o2), flops=fl)
        else:
            ctx_len = tokens
            pages = (ctx_len + 64) // 64 + 1
            kc = torch.randn(rows * pages, kv, 64, dim, device=dev).to(bf)
            vc = torch.randn(rows * pages, kv, 64, dim, device=dev).to(bf)
            table = i32([[b * pages + p for p in range(pages)] for b in range(rows)])
            cache = CacheView(k=kc, v=vc, page_table=table, table_stride=pages, ring=0)
            pos1 = i32([ctx_len] * rows)
            ctx = StepContext(device=torch.device(dev), act_dtype=bf, n_tokens=rows, n_rows=rows, token_ids=pos1,
                              positions=pos1, token_row=slots, cu_seqlens=cu, seq_end=i32([ctx_len + 1] * rows),
                              slots=slots, from_start=False, single_token=True, max_row_tokens=1,
                              max_end=ctx_len + 1, status=status)
            nb = rows * (window + ZANELORN_KEEP) * kv * 2 * dim * 2
            for name, keep in (("attention_kept_first_decode", ZANELORN_KEEP), ("like:attention_window_decode", 0)):
                spec = ScoreSpec(n_heads=heads, n_kv_heads=kv, head_dim=dim, value_dim=dim, scale=dim ** -0.5,
                                 window=window, keep_first=keep)
                timed(name, lambda: scored_attention(spec, qa, None, None, cache, ctx, o2), nbytes=nb)
    return out


def workload_zanelorn(args) -> int:
    """Prefill of one 2,048-token prompt and decoding at batch 8 from 2,048-token contexts, for
    the Zanelorn design (retention and attention-plus-selective-scan layers with routed and dense
    feed-forwards) and for the Qwen2 decoder at equal width, heads, feed-forward width and layers,
    random weights, bfloat16; and the design's kernels alone."""
    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    pk, pk_kind = peaks()
    torch.cuda.set_device(0)
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler()
    clocks.start()
    t_all = time.time()
    sizes = []
    for name, width, heads, kv, dim, ff, ret_heads, window, experts, top in ZANELORN_SIZES:
        cfg_z = zanelorn_config(width, heads, kv, dim, ff, ret_heads, window, experts, top, FURITAR_VOCAB)
        cfg_q = dict(CONFIG_7B, vocab_size=FURITAR_VOCAB, hidden_size=width,
                     num_hidden_layers=ZANELORN_LAYERS, num_attention_heads=heads,
                     num_key_value_heads=kv, intermediate_size=ff, max_position_embeddings=CONTEXT)
        entry = {"name": name, "width": width, "heads": heads, "kv_heads": kv, "head_size": dim,
                 "feed_forward": ff, "retention_heads": ret_heads, "window": window,
                 "kept_first": ZANELORN_KEEP, "experts": experts, "experts_a_token": top,
                 "layers": ZANELORN_LAYERS}
        for label, cfg in (("zanelorn", cfg_z), ("qwen2", cfg_q)):
            model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
            gen = Generator(model, max_tokens=BATCH * CONTEXT, max_batch=BATCH)
            engine = gen.engine
            g = torch.Generator().manual_seed(2)
            ids = torch.randint(0, FURITAR_VOCAB, (PROMPT,), generator=g).tolist()
            ms_prefill = time_prefill(engine, torch, ids, 10)
            flops = zanelorn_prefill_flops(cfg, PROMPT) if label == "zanelorn" else prefill_flops(cfg, PROMPT)
            ms_step, launched = time_decode(engine, torch, K, BATCH, steps, max(3, args.warmup), PROMPT)
            ms_med = time_decode.median_ms
            context = PROMPT + 3 + steps / 2
            step_bytes = (zanelorn_decode_bytes(model, cfg, BATCH, context) if label == "zanelorn"
                          else decode_bytes(model, BATCH, context))
            entry[label] = {
                "weights_gb": round(model.parameter_bytes() / 1e9, 3),
                "prefill_tokens_per_s": round(PROMPT * 1e3 / ms_prefill, 1),
                "prefill_ms": round(ms_prefill, 3),
                "prefill_frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(BATCH * 1e3 / ms_med, 1),
                "decode_ms_per_step": round(ms_med, 4), "decode_frac": _frac(step_bytes, ms_med, pk),
                "decode_launches_per_step": round(launched / steps, 1)}
            del gen, engine, model
            torch.cuda.empty_cache()
        entry["kernels"] = zanelorn_kernels(torch, K, pk, width, heads, kv, dim, ret_heads, window)
        sizes.append(entry)
    summary = clocks.summary((t_all, time.time()))
    clocks.stop()
    print(json.dumps({
        "workload": "zanelorn", "impl": "ours", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
        "metric": "prefill tokens/s of one 2048-token prompt and decode tokens/s at batch 8 from "
                  "2048-token contexts, Zanelorn beside Qwen2 at equal width and layers",
        "unit": "tokens/s", "steps": steps, "prompt_len": PROMPT, "batch": BATCH,
        "fractions": f"prefill: flops over the {pk_kind} bf16 product peak; decode: bytes of the "
                     f"weights a step can touch, the visible cache and the recurrent state over "
                     f"the {pk_kind} copy bandwidth",
        "l2": "weights larger than L2 are read every step; kernels alone: L2 flushed before each run",
        "clocks": summary, "sizes": sizes}))
    return 0


REF_KERNELS = os.path.join(ROOT, "baseline", "_ref", "libref_kernels.so")
# the reference's checkout, if it sits beside this repository (or where MINFER_REFERENCE_DIR says)
REF_SOURCE = os.path.join(os.environ.get("MINFER_REFERENCE_DIR",
                                         os.path.join(os.path.dirname(ROOT), "reference")),
                          "src", "cuda_kernels.cu")


def reference_kernel_times(torch, K):
    """The reference's own float32 CUDA kernels (src/cuda_kernels.cu of yusiwen/minfer, compiled
    as they are into baseline/_ref/, driven through its stock launchers at its stock launch
    shapes) timed beside this library's kernels for the same op and sizes: median of 10 runs,
    CUDA events, L2 flushed between runs.  A kernel-level comparison, not a model-level one:
    the reference's model path cannot be built here."""
    import ctypes
    import math
    if not os.path.exists(REF_KERNELS) and os.path.exists(REF_SOURCE):
        os.makedirs(os.path.dirname(REF_KERNELS), exist_ok=True)
        subprocess.run(["nvcc", "-shared", "-Xcompiler", "-fPIC", "-gencode",
                        "arch=compute_100a,code=sm_100a", "-O2", "-o", REF_KERNELS, REF_SOURCE],
                       check=False, capture_output=True)
    if not os.path.exists(REF_KERNELS):
        return {"unavailable": "baseline/_ref/libref_kernels.so is not there and the reference's "
                               "source is not on this machine"}
    lib = ctypes.CDLL(REF_KERNELS)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.launch_rms_norm_f32.argtypes = [vp, vp, vp, ci, cf, ci, vp]
    lib.launch_rope_f32.argtypes = [vp, ci, ci, ci, cf, cf, vp, vp]
    lib.launch_swiglu_f32.argtypes = [vp, vp, vp, ci, vp]
    lib.launch_store_kv_f32.argtypes = [vp, vp, ci, ci, vp, vp]
    lib.launch_gqa_attn_f32.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, cf, ci, vp]
    dev = "cuda:0"
    stream = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def med_us(fn, reps=10):
        fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return round(statistics.median(times), 1)

    nh, nk, hd, ne, nf, T, ctx = 28, 4, 128, 3584, 18944, 2048, 2048
    scale = 1.0 / math.sqrt(hd)
    g = torch.Generator(device=dev).manual_seed(1)
    out = {}
    st = torch.zeros(1, dtype=torch.int32, device=dev)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, device=dev)

    # ---- attention, one new token over 2,048 cached positions --------------------------------
    kc, vc = rnd(ctx, nk * hd), rnd(ctx, nk * hd)
    q1, o1 = rnd(1, nh, hd), torch.empty(1, nh, hd, device=dev)
    pos1 = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
    out["attn_decode_ctx2048_ref_us"] = med_us(lambda: lib.launch_gqa_attn_f32(
        q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), o1.data_ptr(), pos1.data_ptr(), nh, nk, hd,
        scale, 1, stream))
    pages = ctx // 64
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    row0 = torch.zeros(1, dtype=torch.int32, device=dev)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        kp = kc.view(pages, 64, nk, hd).transpose(1, 2).contiguous().to(dt)
        vp_ = vc.view(pages, 64, nk, hd).transpose(1, 2).contiguous().to(dt)
        qd = q1.to(dt)
        od = torch.empty(1, nh * hd, dtype=dt, device=dev)
        n_chunks = ctx // 256
        part = torch.empty(nh * n_chunks * (hd + 2), device=dev)
        out[f"attn_decode_ctx2048_ours_{name}_us"] = med_us(lambda: K.attention_paged(
            qd, kp, vp_, row0, pos1, table, pages, 0, od, part, nh, nk, hd, 0, 256, n_chunks, scale,
            status=st, old_keys_final=True))
    # ---- attention, a whole prompt of 2,048 tokens --------------------------------------------
    qT, kT, vT = rnd(T, nh, hd), rnd(T, nk, hd), rnd(T, nk, hd)
    oT = torch.empty(T, nh, hd, device=dev)
    posT = torch.arange(T, dtype=torch.int32, device=dev)
    kT2, vT2 = kT.reshape(T, nk * hd), vT.reshape(T, nk * hd)
    out["attn_prefill_2048_ref_us"] = med_us(lambda: lib.launch_gqa_attn_f32(
        qT.data_ptr(), kT2.data_ptr(), vT2.data_ptr(), oT.data_ptr(), posT.data_ptr(), nh, nk, hd,
        scale, T, stream), reps=3)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    rowT = torch.zeros(T, dtype=torch.int32, device=dev)
    of = torch.empty(T, nh * hd, device=dev)
    out["attn_prefill_2048_ours_f32_us"] = med_us(lambda: K.attention_packed(
        qT, kT, vT, rowT, posT, cu, of, nh, nk, hd, 0, scale), reps=3)
    qb, kb, vb = qT.bfloat16(), kT.bfloat16(), vT.bfloat16()
    ob = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=dev)
    out["attn_prefill_2048_ours_bf16_us"] = med_us(lambda: K.attention_prefill_tc(
        qb, kb, vb, cu, ob, 1, T, nh, nk, hd, 0, scale, st))
    # ---- RMSNorm of 2,048 rows of 3,584 ----------------------------------------------------------
    x, w = rnd(T, ne), rnd(ne)
    y = torch.empty(T, ne, device=dev)
    out["rmsnorm_2048x3584_ref_us"] = med_us(lambda: lib.launch_rms_norm_f32(
        x.data_ptr(), w.data_ptr(), y.data_ptr(), ne, 1e-6, T, stream))
    out["rmsnorm_2048x3584_ours_f32_us"] = med_us(lambda: K.rmsnorm(x, w, 1e-6, y))
    yb = torch.empty(T, ne, dtype=torch.bfloat16, device=dev)
    out["rmsnorm_2048x3584_ours_bf16_us"] = med_us(lambda: K.rmsnorm(x, w, 1e-6, yb))
    # ---- rotation of q and k plus the cache write, 2,048 tokens ----------------------------------
    qkv = rnd(T, (nh + 2 * nk) * hd)
    qr, kr = rnd(T, nh, hd), rnd(T, nk, hd)
    vr = rnd(T, nk * hd)
    kcache, vcache = torch.zeros(T, nk * hd, device=dev), torch.zeros(T, nk * hd, device=dev)

    def ref_rope_store():
        lib.launch_rope_f32(qr.data_ptr(), nh, hd, T, 1e6, 1.0, posT.data_ptr(), stream)
        lib.launch_rope_f32(kr.data_ptr(), nk, hd, T, 1e6, 1.0, posT.data_ptr(), stream)
        lib.launch_store_kv_f32(kr.data_ptr(), kcache.data_ptr(), nk * hd, T, posT.data_ptr(), stream)
        lib.launch_store_kv_f32(vr.data_ptr(), vcache.data_ptr(), nk * hd, T, posT.data_ptr(), stream)
    out["rope_store_2048_ref_us"] = med_us(ref_rope_store)
    inv = (1e6 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)).to(dev)
    seq_end = torch.tensor([T], dtype=torch.int32, device=dev)
    tableT = torch.arange(T // 64, dtype=torch.int32, device=dev).reshape(1, T // 64)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        qo = torch.empty(T, nh, hd, dtype=dt, device=dev)
        ko, vo = torch.empty(T, nk, hd, dtype=dt, device=dev), torch.empty(T, nk, hd, dtype=dt, device=dev)
        kpg = torch.zeros(T // 64, nk, 64, hd, dtype=dt, device=dev)
        vpg = torch.zeros_like(kpg)
        out[f"rope_store_2048_ours_{name}_us"] = med_us(lambda: K.rope_kvstore(
            qkv, posT, rowT, seq_end, inv, qo, ko, vo, kpg, vpg, tableT, T // 64, 0, nh, nk, hd, hd, 0, st))
    # ---- SwiGLU, 2,048 rows of 18,944 -------------------------------------------------------------
    gate, up = rnd(T, nf), rnd(T, nf)
    dst = torch.empty(T, nf, device=dev)
    out["swiglu_2048x18944_ref_us"] = med_us(lambda: lib.launch_swiglu_f32(
        gate.data_ptr(), up.data_ptr(), dst.data_ptr(), T * nf, stream))
    gu = torch.cat([gate, up], dim=1).contiguous()
    out["swiglu_2048x18944_ours_f32_us"] = med_us(lambda: K.swiglu(gu, dst))
    gub, dstb = gu.bfloat16(), torch.empty(T, nf, dtype=torch.bfloat16, device=dev)
    out["swiglu_2048x18944_ours_bf16_us"] = med_us(lambda: K.swiglu(gub, dstb))
    torch.cuda.synchronize()
    if int(st.item()) != 0:
        out["status"] = int(st.item())
    # reference time over ours, per op: float32 against float32, and against the bfloat16 kernel
    # that the product path runs
    for op in ("attn_decode_ctx2048", "attn_prefill_2048", "rmsnorm_2048x3584", "rope_store_2048",
               "swiglu_2048x18944"):
        for name in ("f32", "bf16"):
            out[f"{op}_ref_over_ours_{name}"] = round(out[f"{op}_ref_us"] / out[f"{op}_ours_{name}_us"], 2)
    out["note"] = ("the reference's float32 kernels, unchanged, through its own launchers; in the "
                   "bfloat16 engine SwiGLU runs inside the product's epilogue, not as this kernel")
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--workload", default="qwen2-7b", choices=["qwen2-7b", "furitar", "budanex", "bedarax", "zanelorn"],
                    help="qwen2-7b (the default): the headline figure and its points; furitar: "
                         "the Furitar design beside Qwen2 at equal sizes, prefill and decode")
    ap.add_argument("--skip-points", action="store_true",
                    help="only the headline figure and its end-to-end twin")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "yusiwen/minfer is a Rust program that loads GGUF files; there is no "
                          "Rust toolchain (cargo/rustc) in this image, pip cannot build it, and "
                          "its CUDA forward path is dead code at this commit"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    if args.workload == "furitar":
        return workload_furitar(args)
    if args.workload == "budanex":
        return workload_budanex(args)
    if args.workload == "bedarax":
        return workload_bedarax(args)
    if args.workload == "zanelorn":
        return workload_zanelorn(args)

    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams

    warmup = max(3, args.warmup)
    steps = max(1, min(args.steps, CONTEXT - PROMPT - warmup - 2))     # the context is 4,096
    cfg = dict(CONFIG_7B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_kind = peaks()

    torch.cuda.set_device(0)
    t_build = time.time()
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t_build:.1f} s, "
          f"{model.parameter_bytes() / 1e9:.2f} GB of weights", file=sys.stderr, flush=True)

    max_batch = BATCH if args.skip_points else 64
    gen = Generator(model, max_tokens=max_batch * CONTEXT, max_batch=max_batch)
    engine = gen.engine
    clocks = ClockSampler()
    clocks.start()
    ms_step, launched = time_decode(engine, torch, K, BATCH, steps, warmup, PROMPT)
    clock_summary = clocks.summary(time_decode.window)
    value = BATCH * 1000.0 / ms_step

    # roofline of the decode step, mean context over the timed steps
    ctx_tokens = PROMPT + warmup + steps / 2
    step_bytes = decode_bytes(model, BATCH, ctx_tokens)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_kind}

    # end to end through the Python entry point: host ids in, host ids out every step
    def end_to_end(batch, new_tokens):
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
                   for _ in range(batch)]
        gen.stats.__init__()
        engine.h2d_bytes = engine.d2h_bytes = 0
        gen.generate(prompts, new_tokens, SamplingParams.greedy(), stop_token_ids=[])
        return gen.stats

    # long enough that the clock dip which follows the prompt's burst (about 30 steps: 3.9 ms,
    # then 3.5 ms, then the steady 3.3 ms a step) does not dominate
    st = end_to_end(BATCH, max(steps, 128) + 1)
    e2e_value = st.decode_tokens / max(st.decode_seconds, 1e-9)
    prompt_bytes = 4 * BATCH * PROMPT
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int((engine.h2d_bytes - prompt_bytes) / max(st.steps, 1)),
           "d2h_bytes_per_step": int(engine.d2h_bytes / max(st.steps, 1)), "steps": st.steps - 1,
           "device_value": round(st.decode_tokens / max(st.decode_device_seconds, 1e-9), 1)}

    out = {
        "metric": "decode tokens/s, Qwen2.5-7B shape, batch 8, 2048-token contexts",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "Qwen2.5-7B shape, random weights", "global_batch": BATCH,
            "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_config": full_layers,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"],
            "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
            "l2": "inputs larger than L2 (weights read every step)",
            "cache": "decode starts from a real prefill of batch x 2048 random tokens",
            "settle_s": SETTLE_S,
        },
        "clocks": clock_summary, "e2e": e2e, "gpu_launches": launched, "roofline": roofline,
        "ms_per_step_median": round(time_decode.median_ms, 4),
    }

    if not args.skip_points:
        points, windows = {}, {}
        # prefill of one 2,048-token prompt: median of 20
        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
        ms_prefill = time_prefill(engine, torch, ids, 20)
        windows["prefill"] = (time_prefill.window, ms_prefill)
        flops = prefill_flops(cfg, PROMPT)
        out["prefill"] = {"value": round(PROMPT * 1000.0 / ms_prefill, 1), "tokens": PROMPT,
                          "ms": round(ms_prefill, 3),
                          "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "of": pk_kind, "runs": 20, "statistic": "median",
                          # the first timed prompt runs before the power cap pulls the clock down,
                          # as one prompt that arrives alone does: its time against the burst peak
                          "ms_first": round(time_prefill.times[0], 3),
                          "frac_first": round(flops / (time_prefill.times[0] * 1e-3) /
                                              (pk["bf16_tflops"] * 1e12), 4),
                          # twenty prompts back to back run under the power cap, as the
                          # library's seconds-long product does: the fraction of that peak too
                          "frac_sustained": round(flops / (ms_prefill * 1e-3) /
                                                  (pk["bf16_tflops_sustained"] * 1e12), 4)}
        n_point = max(64, min(steps, 128))
        for b in (1, 64):
            time_decode(engine, torch, K, b, n_point, 3, PROMPT)
            ms_b = time_decode.median_ms
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
            points[f"decode_b{b}_frac"] = _frac(decode_bytes(model, b, PROMPT + 3 + n_point / 2), ms_b, pk)
            windows[f"decode_b{b}"] = (time_decode.window, ms_b)
        # the host's share at batch 64: the same loop the user calls, device marks beside the host's clock
        st64 = end_to_end(64, 129)
        host_ms = st64.decode_seconds / max(st64.steps - 1, 1) * 1e3
        dev_ms = windows["decode_b64"][1]
        points["decode_b64_e2e"] = round(64e3 / host_ms, 1)
        points["host_share_7b_b64"] = round(max(0.0, host_ms - dev_ms) / host_ms, 4)
        more, win = point_long(engine, torch, K, pk, cfg)
        points.update(more)
        windows.update(win)
        out["reference_kernels"] = reference_kernel_times(torch, K)
        # the other shapes need the memory: the headline model goes first
        del gen, engine, model
        torch.cuda.empty_cache()
        for fn, fn_args in ((point_05b, (torch, K, pk)), (point_14b, (torch, K, pk))):
            more, win = fn(*fn_args)
            points.update(more)
            windows.update(win)
            torch.cuda.empty_cache()
        out["points"] = points
        out["points_note"] = ("medians of per-step device times (CUDA events); *_frac is the step's "
                              "bytes or flops over its time over the measured peak")
        pc = {}
        for name, (window, ms) in windows.items():
            c = clocks.summary(window)
            pc[name] = {"sm_mhz": c["sm_mhz"], "reasons": c["reasons"], "samples": c["samples"],
                        "ms_x_mhz": round(ms * c["sm_mhz"], 1) if c["sm_mhz"] else None}
        out["points_clocks"] = pc
    clocks.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
