"""Decode and prefill throughput of the Llama-3-8B shape on one B200, random weights, bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L] [--model NAME]
                    [--dtype bf16|fp32] [--points default|main|long]

Prints ONE JSON line.  ``value``: decoded tokens a second at batch 8 (prompt lengths uniform in
[128, 2048]); after W warm-up steps, ``regions`` (5) regions of K decode steps each are timed on the device
with CUDA events and the median region counts; a step is one decode step, the next token chosen greedily on
the device.  ``e2e``: the same through the Python entry point ``generate`` with host token lists in and out (a
pinned host-to-device copy of every step's tokens and a device-to-host read of every step's result inside the
timed region), again the median of 5 regions of K steps.  ``prefill``: one prompt of 2,048 tokens.
``roofline``: the bytes a decode step has to read (every weight it uses once, and the cache of the live
requests) over its time, against the measured copy bandwidth.  ``points``: tokens a second of decode at batch
1, 16, 32, 64 and 128, of a batch of 64 of which one sequence ends every third step (down to 16; by the clock, host
tokens in, the live set changing under the captured graphs), of decode at batch 8 with 7,000 to 8,000 cached tokens a request, of prefills of 512 and 8,192
tokens, and of the benchmark's further configurations (decode at batch 8 and a prefill of 2,048 tokens for the
Llama-2-7B and Llama-2-13B shapes, decode at batch 8 in float32); ``points_frac``: each point's fraction of its
roofline (copy bandwidth for decode, the dtype's arithmetic peak for prefill).  Weights (15 GB a step) are
larger than L2, so no flush is needed between steps.

``--dtype fp32`` measures the true 32-bit path (FFMA products, float32 cache) in the same line format.
``--points main`` leaves the further configurations out; ``--points long`` adds decode at batch 64 with
7,000 to 8,000 cached tokens a request (a prefill of half a million tokens comes before it).
``--only decode_b<N>`` or ``--only prefill`` prints that part alone (for profilers); ``--only gemm_rows``,
``attention_prefill`` and ``attention_decode`` time single kernels at the model's layer sizes over a range of rows,
tokens or contexts, one JSON line a size.  The default warm-up of 24 steps covers the 80 ms or so that the GPU's
clocks take to come back up after the prefill's power-capped run.

``--model llama-2-7b`` or ``llama-2-13b`` measures the benchmark's further shapes (32 and 40 kv heads: eight and
ten times the keys and values a token) with their own prompt lengths instead of the default.
``--impl reference`` runs the unmodified reference (baseline/_ref) through its own get_model/generate.
For more than one GPU the program says that it has no such path and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The benchmark's shapes (the default is the first) with their registry variants and prompt lengths.
MODELS = {
    "llama-3-8b": dict(name="llama-3-8b", variant="3-8b", label="Llama-3-8B", nlayers=32, emb_dim=4096, nheads=32, kvheads=8,
                       head_dim=128, ffn_hidden=14336, vocab=128256, context=8192, prompts=(128, 2048)),
    "llama-2-7b": dict(name="llama-2-7b", variant="7b", label="Llama-2-7B", nlayers=32, emb_dim=4096, nheads=32, kvheads=32,
                       head_dim=128, ffn_hidden=11008, vocab=32000, context=4096, prompts=(64, 2048)),
    "llama-2-13b": dict(name="llama-2-13b", variant="13b", label="Llama-2-13B", nlayers=40, emb_dim=5120, nheads=40,
                        kvheads=40, head_dim=128, ffn_hidden=13824, vocab=32000, context=4096, prompts=(1024, 1024)),
}
MODEL = MODELS["llama-3-8b"]
PROMPT_MIN, PROMPT_MAX, PREFILL_TOKENS, BATCH = 128, 2048, 2048, 8


def choose_model(name):
    global MODEL, PROMPT_MIN, PROMPT_MAX
    MODEL = MODELS[name]
    PROMPT_MIN, PROMPT_MAX = MODEL["prompts"]


# float32 on the CUDA cores: 148 multiprocessors x 128 lanes x 2 flops x 1.965 GHz (nominal; nobody measured it here)
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12
REGIONS = 5  # timed regions of --steps steps each; the median counts


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def prompt_lengths(batch, seed=0):
    import numpy as np

    rng = np.random.default_rng(seed + batch)
    return [int(x) for x in rng.integers(PROMPT_MIN, PROMPT_MAX + 1, size=batch)]


def random_prompts(lengths, vocab, seed=0):
    import numpy as np

    rng = np.random.default_rng(1000 + seed)
    return [[int(t) for t in rng.integers(0, vocab, size=n)] for n in lengths]


def decode_bytes(nlayers, batch_context_tokens, m=None, itemsize=2):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    m = m or MODEL
    d, hd, h, kv, f, v = m["emb_dim"], m["head_dim"], m["nheads"], m["kvheads"], m["ffn_hidden"], m["vocab"]
    per_layer = ((h + 2 * kv) * hd * d + h * hd * d + 2 * f * d + f * d + 2 * d) * itemsize
    weights = nlayers * per_layer + d * itemsize + v * d * itemsize
    cache = batch_context_tokens * nlayers * 2 * kv * hd * itemsize
    return weights + cache


def prefill_flops(nlayers, tokens, m=None):
    m = m or MODEL
    d, hd, h, kv, f, v = m["emb_dim"], m["head_dim"], m["nheads"], m["kvheads"], m["ffn_hidden"], m["vocab"]
    gemm = 2 * tokens * ((h + 2 * kv) * hd * d + h * hd * d + 3 * f * d) * nlayers
    attention = 2 * tokens * tokens * hd * h * nlayers  # causal half of 4 T^2 hd per head
    return gemm + attention + 2 * v * d


# --------------------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------------------
def run_kernels(args):
    """--only gemm_rows / attention_prefill / attention_decode: single kernels at the model's layer sizes over a
    range of rows, tokens or contexts, timed alone with CUDA events (L2 flushed before every launch), the products
    beside the library's.  One JSON line a size."""
    import torch

    from fms_b200.cache import Cache, KVRequest
    from fms_b200.engine.batch import Batch
    from fms_b200.kernels import ops

    m = MODEL
    d, hd, h, kv, f = m["emb_dim"], m["head_dim"], m["nheads"], m["kvheads"], m["ffn_hidden"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, repeats=10):
        for _ in range(3):
            fn()
        us = []
        for _ in range(repeats):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3)
        return round(statistics.median(us), 1)

    bf16 = torch.bfloat16
    if args.only == "gemm_rows":
        # every own kernel that takes the size, called directly (whatever the step would choose), beside the library
        shapes = {"qkv": ((h + 2 * kv) * hd, d), "dense": (d, h * hd), "down": (d, f)}
        ws = {k: (torch.randn(n, kk, device="cuda") * 0.02).to(bf16) for k, (n, kk) in shapes.items()}
        wg = (torch.randn(2 * f, d, device="cuda") * 0.02).to(bf16)
        ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS = True, ["linear", "glu", "qkv"], 256
        for rows in (1, 8, 16, 64, 256, 512, 1024, 2048, 4096):
            xs = {d: torch.randn(rows, d, device="cuda").to(bf16), f: torch.randn(rows, f, device="cuda").to(bf16)}
            line = {"only": "gemm_rows", "rows": rows, "us": "weight-streaming (<= 8 rows: mma.sync; 9-256: tcgen05, "
                    "weights on the rows), tcgen05 with the tokens on the rows (>= 128), library"}
            small, large = rows <= 256, rows >= 128
            for name, (n, kk) in shapes.items():
                line[name] = [timed(lambda: ops.linear(xs[kk], ws[name])) if small else None,
                              timed(lambda: ops.linear_tensor_core(xs[kk], ws[name])) if large else None,
                              timed(lambda: torch.nn.functional.linear(xs[kk], ws[name]))]
            line["glu"] = [timed(lambda: ops.gated_linear(xs[d], wg, None, 0)) if small else None,
                           timed(lambda: ops.gated_linear_tensor_core(xs[d], wg, None, 0)) if large else None,
                           timed(lambda: ops.gated_activation(torch.nn.functional.linear(xs[d], wg), 0))]
            print(json.dumps(line), flush=True)
    else:
        cases = [(1, n) for n in (512, 1024, 2048, 4096, 8192)] if args.only == "attention_prefill" else \
            [(b, n) for b, n in ((1, 1024), (1, 8192), (8, 1155), (8, 8192), (64, 1155), (64, 4096))]
        for b, n in cases:
            decode = args.only == "attention_decode"
            cache = Cache([KVRequest(kv, hd, 0)], max_tokens=b * (n + 128), max_positions=n + 128, dtype=bf16, device="cuda")
            slots = cache.begin(b)
            if decode:
                cache.prepare(slots, [n] * b)
                cache.commit(slots, [n] * b)
            new = 1 if decode else n
            cache.prepare(slots, [new] * b)
            view = cache.layer_view(0)
            view.keys.normal_()
            view.values.normal_()
            batch = Batch.from_lists(slots, [n if decode else 0] * b, [[0] * new] * b, [[]] * b, "cuda")
            q = torch.randn(b * new, h * hd, device="cuda").to(bf16)
            us = timed(lambda: ops.attention(q, batch, view, h, kv, hd, hd ** -0.5, 0), repeats=20)
            line = {"only": args.only, "sequences": b, "tokens": n, "us": us}
            if decode:
                line["kv_GBs"] = round(b * n * kv * hd * 2 * 2 / us / 1e3, 1)
            else:
                line["tflops"] = round(4.0 * n * n / 2 * hd * h / us / 1e6, 1)
            print(json.dumps(line), flush=True)
            del cache, view
    ops.check_error_flag("cuda")


class Measured:
    """One model on the device with an engine, and the measurements taken on it."""

    def __init__(self, model_info, dtype, nlayers, room, max_prompt, slots=64, long_requests=0):
        """``room``: decode steps a request goes through; ``long_requests``: how many requests of up to the model's
        whole context the cache has to hold beside ``slots`` requests of ``max_prompt`` tokens."""
        import torch

        from fms_b200.models import get_model

        self.m, self.dtype, self.nlayers = model_info, dtype, nlayers
        self.itemsize = 2 if dtype == "bf16" else 4
        self.model = get_model("llama", model_info["variant"], device_type="cuda", data_type=dtype, seed=0, nlayers=nlayers)
        cfg = self.model.config
        assert (cfg.emb_dim, cfg.nheads, cfg.n_kvheads, cfg.ffn_hidden, cfg.src_vocab_size, cfg.max_expected_seq_len) == (
            model_info["emb_dim"], model_info["nheads"], model_info["kvheads"], model_info["ffn_hidden"], model_info["vocab"],
            model_info["context"])
        self.engine = self.model.new_engine(max_tokens=max(slots * (max_prompt + 2 * room + 128),
                                                           long_requests * model_info["context"]), max_slots=slots)
        self.torch = torch

    def close(self):
        self.engine = self.model = None
        self.torch.cuda.empty_cache()

    def device_decode(self, batch, steps, warmup, lengths=None, regions=REGIONS):
        """(tokens a second, ms a step, mean context, own kernels launched, ms a step of every region): after the
        prompts and ``warmup`` decode steps, ``regions`` regions of ``steps`` decode steps, each between two CUDA events;
        the median region counts."""
        from fms_b200.kernels import ops

        torch, engine = self.torch, self.engine
        lengths = lengths or prompt_lengths(batch)
        prompts = random_prompts(lengths, self.m["vocab"])
        slots = engine.begin(batch)
        try:
            warmup = max(3, warmup)
            horizon = max(lengths) + warmup + regions * steps + 1
            if sum(lengths) > 100_000:  # many long prompts: eight requests a step
                for i in range(0, batch, 8):
                    last = engine.step(slots[i:i + 8], prompts[i:i + 8])
                    logits = last if i == 0 else torch.cat([logits, last])
            else:
                logits = engine.step(slots, prompts)
            tokens = ops.argmax(logits)
            for _ in range(warmup):
                tokens = ops.argmax(engine.decode(slots, tokens_device=tokens, horizon=horizon))
            torch.cuda.synchronize()
            context = sum(engine.length(s) for s in slots) + batch * (regions * steps + 1) / 2.0
            launches0, graphs0 = ops.launches, engine.graph_launches
            events = [torch.cuda.Event(enable_timing=True) for _ in range(regions + 1)]
            events[0].record()
            for r in range(regions):
                for _ in range(steps):
                    tokens = ops.argmax(engine.decode(slots, tokens_device=tokens, horizon=horizon))
                events[r + 1].record()
            torch.cuda.synchronize()
            per_region = [events[r].elapsed_time(events[r + 1]) / steps for r in range(regions)]
            ms = statistics.median(per_region)
            launched = ((ops.launches - launches0) + (engine.graph_launches - graphs0) * engine.kernels_per_graph) // regions
            engine.check()
        finally:
            engine.release(slots)
        return batch / (ms / 1e3), ms, context, launched, per_region

    def ending_decode(self, batch=64, every=3, until=16):
        """Tokens a second of a batch whose sequences end one by one (one every ``every`` steps, down to ``until``):
        host tokens in and out as a generation loop has them, timed by the clock from the first decode step to the
        last, the second of two passes (the first leaves the graphs of the sizes captured, as a running engine has them)."""
        import random as _random
        import time as _time

        torch, engine = self.torch, self.engine
        lengths = prompt_lengths(batch)
        prompts = random_prompts(lengths, self.m["vocab"])
        value = 0.0
        for _ in range(2):
            rng = _random.Random(3)
            slots = engine.begin(batch)
            live = list(slots)
            try:
                engine.step(slots, prompts)
                horizon = max(lengths) + every * batch
                torch.cuda.synchronize()
                start, done, step = _time.perf_counter(), 0, 0
                while len(live) > until:
                    step += 1
                    if step % every == 0:
                        engine.release([live.pop(rng.randrange(len(live)))])
                    engine.decode(live, [1] * len(live), horizon=horizon)
                    done += len(live)
                torch.cuda.synchronize()
                value = done / (_time.perf_counter() - start)
                engine.check()
            finally:
                engine.release(live)
        return value

    def host_decode(self, batch, steps, warmup, regions=REGIONS):
        """The same through generate(): host token lists in, host tokens out, every step."""
        from fms_b200.utils.generation import generate

        torch, engine = self.torch, self.engine
        lengths = prompt_lengths(batch)
        prompts = [torch.tensor(p) for p in random_prompts(lengths, self.m["vocab"])]
        h2d0 = engine.h2d_bytes
        _, times = generate(engine, prompts, max_new_tokens=1 + max(3, warmup) + regions * steps, do_sample=False,
                            timing="per-token")
        timed = times[-regions * steps:]
        per_region = [sum(timed[r * steps:(r + 1) * steps]) for r in range(regions)]
        h2d_decode = 4 * batch  # each decode step copies its tokens from a pinned host array
        assert engine.h2d_bytes - h2d0 >= h2d_decode * regions * steps
        return batch * steps / statistics.median(per_region), h2d_decode, 4 * batch

    def prefill(self, tokens, repeats=5):
        torch, engine = self.torch, self.engine
        prompt = random_prompts([tokens], self.m["vocab"], seed=7)
        ms = []
        for i in range(3 + repeats):  # three warm-up runs, then the timed ones
            (slot,) = engine.begin(1)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([slot], prompt)
            end.record()
            torch.cuda.synchronize()
            engine.release([slot])
            if i >= 3:
                ms.append(start.elapsed_time(end))
        return statistics.median(ms)

    def decode_frac(self, ms_step, context, pk):
        return decode_bytes(self.nlayers, context, self.m, self.itemsize) / (ms_step / 1e3) / 1e9 / pk["hbm_gbs"]

    def prefill_frac(self, ms, tokens, pk):
        peak = pk["bf16_tflops"] if self.dtype == "bf16" else FP32_TFLOPS_NOMINAL
        return prefill_flops(self.nlayers, tokens, self.m) / (ms / 1e3) / (peak * 1e12)


def run_ours(args):
    import numpy as np

    pk = peaks()
    dtype = args.dtype
    nlayers = args.layers or MODEL["nlayers"]
    room = max(3, args.warmup) + REGIONS * args.steps + 8
    long_context = args.points != "main" and not args.only and MODEL["context"] >= 8192
    # 128 slots (for the point at batch 128) where their cache stays well inside the memory: the 8B shape in bfloat16
    # holds 128 KB a token, the shapes with as many kv heads as heads four times that
    token_bytes = 2 * nlayers * MODEL["kvheads"] * MODEL["head_dim"] * (2 if dtype == "bf16" else 4)
    roomy = 128 * (PROMPT_MAX + 2 * room + 128) * token_bytes < 60e9
    slots = max(64, int(args.only.split("_b")[1])) if args.only.startswith("decode_b") else (128 if roomy else 64)
    run = Measured(MODEL, dtype, nlayers, room, PROMPT_MAX, slots=slots,
                   long_requests=(64 if args.points == "long" else 8) if long_context else 0)

    if args.only:  # a short run of one part, for profilers: prints that part's figures only
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "tokens": args.prefill_tokens,
                              "ms": round(run.prefill(args.prefill_tokens, repeats=args.steps), 3)}))
        else:
            batch = int(args.only.split("_b")[1])
            v, ms, _, _, _ = run.device_decode(batch, args.steps, args.warmup, regions=1)
            e2e, _, _ = run.host_decode(batch, args.steps, args.warmup, regions=1)
            print(json.dumps({"only": args.only, "value": round(v, 1), "ms_per_step": round(ms, 4), "e2e": round(e2e, 1)}))
        return
    sampler = ClockSampler()
    sampler.start()
    value, ms_step, context, launched, per_region = run.device_decode(BATCH, args.steps, args.warmup)
    e2e, h2d, d2h = run.host_decode(BATCH, args.steps, args.warmup)
    sampler.stop()
    points, fracs = {}, {}

    def decode_point(name, r, batch, steps, lengths=None, regions=3):
        v, ms, ctx, _, _ = r.device_decode(batch, steps, args.warmup, lengths, regions)
        points[name], fracs[name] = round(v, 1), round(r.decode_frac(ms, ctx, pk), 4)

    def prefill_point(name, r, tokens, repeats=3):
        ms = r.prefill(tokens, repeats)
        points[name], fracs[name] = round(tokens / (ms / 1e3), 1), round(r.prefill_frac(ms, tokens, pk), 4)

    side = max(32, args.steps // 2)
    for b in (1, 16, 32, 64) + ((128,) if slots >= 128 else ()):
        decode_point(f"decode_b{b}", run, b, side)
    points["decode_b64_ending_one_by_one"] = round(run.ending_decode(), 1)
    pf_ms = run.prefill(PREFILL_TOKENS)
    prefill_point("prefill_512", run, 512)
    if long_context:
        rng = np.random.default_rng(5)
        prefill_point("prefill_8192", run, 8192)
        decode_point("decode_b8_ctx8192", run, 8, side, [int(x) for x in rng.integers(7000, 8000 - 3 * side - 32, size=8)])
        if args.points == "long":
            decode_point("decode_b64_ctx8192", run, 64, side, [int(x) for x in rng.integers(7000, 8000 - 3 * side - 32, size=64)])
    gbs = decode_bytes(nlayers, context, MODEL, run.itemsize) / (ms_step / 1e3) / 1e9
    pf_frac = run.prefill_frac(pf_ms, PREFILL_TOKENS, pk)
    run.close()
    if args.points != "main" and args.model == "llama-3-8b" and not args.layers:
        # the benchmark's further configurations, each on a model of its own: decode at batch 8 and one prefill
        others = [("l2_7b", MODELS["llama-2-7b"], "bf16"), ("l2_13b", MODELS["llama-2-13b"], "bf16")]
        others.append(("fp32", MODELS["llama-3-8b"], "fp32") if dtype == "bf16" else ("bf16", MODELS["llama-3-8b"], "bf16"))
        for tag, info, dt in others:
            lo, hi = info["prompts"]
            rng = np.random.default_rng(8)
            lengths = [int(x) for x in rng.integers(lo, hi + 1, size=BATCH)]
            steps = side if dt == "bf16" else 8
            other = Measured(info, dt, info["nlayers"], max(3, args.warmup) + 3 * steps + 8, PROMPT_MAX, slots=BATCH)
            decode_point(f"{tag}_decode_b8", other, BATCH, steps, lengths)
            prefill_point(f"{tag}_prefill_2048", other, PREFILL_TOKENS, 3 if dt == "bf16" else 1)
            other.close()
    out = {
        "metric": f"decode tok/s at batch 8 ({MODEL['label']} shape, random weights)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic", "impl": "ours",
        "config": {
            "model": MODEL["name"], "layers": nlayers, "layers_of_model": MODEL["nlayers"], "emb_dim": MODEL["emb_dim"],
            "nheads": MODEL["nheads"], "kvheads": MODEL["kvheads"], "head_dim": MODEL["head_dim"],
            "ffn_hidden": MODEL["ffn_hidden"], "vocab": MODEL["vocab"], "context": MODEL["context"],
            "global_batch": BATCH, "seq_len": f"prompts uniform in [{PROMPT_MIN},{PROMPT_MAX}]",
            "mean_context": round(context / BATCH, 1), "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 gpu",
            "weights": "random N(0,0.02), seed 0",
            "l2": f"weights read per step ({decode_bytes(nlayers, 0, MODEL, run.itemsize) / 1e9:.0f} GB) exceed L2; no flush",
            "timed": f"median of {REGIONS} regions of {args.steps} steps", "cache_block_tokens": 64,
            "peaks": pk["source"] + ("" if dtype == "bf16" else f"; fp32 arithmetic {FP32_TFLOPS_NOMINAL:.1f} TFLOP/s nominal"),
        },
        "clocks": sampler.summary(),
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launched),
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                    "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4)},
        "regions": {"count": REGIONS, "ms_per_step": [round(x, 4) for x in per_region]},
        "points": points, "points_frac": fracs,
    }
    print(json.dumps(out))


# --------------------------------------------------------------------------------------------------
# the reference, unmodified, through its own public API
# --------------------------------------------------------------------------------------------------
def run_reference(args):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "fms")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference"}))
        return
    sys.path.insert(0, ref)
    try:
        import torch
        from fms.models import get_model
        from fms.utils.generation import generate, pad_input_ids
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:200]}))
        return

    nlayers = args.layers or MODEL["nlayers"]
    torch.manual_seed(0)
    model = get_model("llama", MODEL["variant"], device_type="cuda", data_type=torch.bfloat16, nlayers=nlayers)
    model.eval()
    torch.set_grad_enabled(False)
    warmup = max(3, args.warmup)

    def decode(batch, steps):
        lengths = prompt_lengths(batch)
        prompts = [torch.tensor(p, dtype=torch.long, device="cuda") for p in random_prompts(lengths, MODEL["vocab"])]
        ids, extra = pad_input_ids(prompts)
        extra["last_n_tokens"] = 1
        events = []

        def hook(i, logits, next_val, kwargs):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            events.append(ev)
            return next_val, kwargs

        _, times = generate(model, ids, max_new_tokens=1 + warmup + steps, use_cache=True, do_sample=False,
                            timing="per-token", post_iteration_hook=hook, extra_kwargs=extra)
        torch.cuda.synchronize()
        ms = events[-steps - 1].elapsed_time(events[-1])
        context = sum(lengths) + batch * (1 + warmup + steps / 2.0)
        return batch * steps / (ms / 1e3), ms / steps, batch * steps / sum(times[-steps:]), context

    sampler = ClockSampler()
    sampler.start()
    value, ms_step, e2e, context = decode(BATCH, args.steps)
    sampler.stop()
    side = max(32, args.steps // 2)
    b1 = decode(1, side)[0]
    b64 = decode(64, side)[0]
    ids = torch.tensor(random_prompts([PREFILL_TOKENS], MODEL["vocab"], seed=7), dtype=torch.long, device="cuda")
    ms = []
    for i in range(8):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        model(ids, use_cache=True, last_n_tokens=1)
        end.record()
        torch.cuda.synchronize()
        if i >= 3:
            ms.append(start.elapsed_time(end))
    pf_ms = statistics.median(ms)
    pk = peaks()
    gbs = decode_bytes(nlayers, context) / (ms_step / 1e3) / 1e9
    print(json.dumps({
        "metric": f"decode tok/s at batch 8 ({MODEL['label']} shape, random weights)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {"model": MODEL["name"], "layers": nlayers, "layers_of_model": MODEL["nlayers"], "global_batch": BATCH,
                   "seq_len": f"prompts uniform in [{PROMPT_MIN},{PROMPT_MAX}], left-padded", "parallelism": "1 gpu",
                   "path": "fms get_model + generate, eager, sdpa, use_cache", "prefill_tokens": PREFILL_TOKENS},
        "clocks": sampler.summary(),
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                    "frac": round(prefill_flops(nlayers, PREFILL_TOKENS) / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)},
    }))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=64)
    # the default covers the 20 or so steps (80 ms) that the GPU's clocks take to come back up after the prefill
    ap.add_argument("--warmup", type=int, default=24)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--only", default="", help="decode_b<batch> or prefill: run and print that part only; gemm_rows, "
                    "attention_prefill, attention_decode: single kernels over a range of sizes")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--model", choices=sorted(MODELS), default="llama-3-8b",
                    help="the shape to measure; the default is the benchmark's, the others are its further configurations")
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="fp32: the true 32-bit path")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --only prefill: the prompt's length")
    ap.add_argument("--points", choices=["default", "main", "long"], default="default",
                    help="main: without the further configurations; long: also decode at batch 64 with 8k contexts")
    args = ap.parse_args()
    choose_model(args.model)
    if args.gpus != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        sys.exit(2)
    if args.impl == "reference":
        run_reference(args)
    elif args.only in ("gemm_rows", "attention_prefill", "attention_decode"):
        run_kernels(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
