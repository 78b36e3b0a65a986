"""Decode and prefill throughput of the Llama-3-8B shape on one B200, random weights, bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L] [--model NAME]

Prints ONE JSON line.  ``value``: decoded tokens a second at batch 8 (prompt lengths uniform in
[128, 2048]), K decode steps timed on the device with CUDA events after W warm-up steps; a step is one
decode step, the next token chosen greedily on the device.  ``e2e``: the same through the Python entry
point ``generate`` with host token lists in and out (a pinned host-to-device copy of every step's tokens
and a device-to-host read of every step's result inside the timed region).  ``prefill``: one prompt of
2,048 tokens.  ``roofline``: the bytes a decode step has to read (every weight it uses once, and the
cache of the live requests) over its time, against the measured copy bandwidth.  ``points``: decode at
batch 1 and 64.  Weights (15 GB a step) are larger than L2, so no flush is needed between steps.

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


def decode_bytes(nlayers, batch_context_tokens, m=None):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    m = m or MODEL
    d, hd, h, kv, f, v = m["emb_dim"], m["head_dim"], m["nheads"], m["kvheads"], m["ffn_hidden"], m["vocab"]
    per_layer = ((h + 2 * kv) * hd * d + h * hd * d + 2 * f * d + f * d + 2 * d) * 2
    weights = nlayers * per_layer + d * 2 + v * d * 2
    cache = batch_context_tokens * nlayers * 2 * kv * hd * 2
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
        shapes = {"qkv": ((h + 2 * kv) * hd, d), "dense": (d, h * hd), "down": (d, f)}
        ws = {k: (torch.randn(n, kk, device="cuda") * 0.02).to(bf16) for k, (n, kk) in shapes.items()}
        wg = (torch.randn(2 * f, d, device="cuda") * 0.02).to(bf16)
        for rows in (1, 8, 16, 64, 256, 512, 1024, 2048, 4096):
            xs = {d: torch.randn(rows, d, device="cuda").to(bf16), f: torch.randn(rows, f, device="cuda").to(bf16)}
            line = {"only": "gemm_rows", "rows": rows, "us": "own, library"}
            for name, (n, kk) in shapes.items():
                line[name] = [timed(lambda: ops.linear(xs[kk], ws[name])),
                              timed(lambda: torch.nn.functional.linear(xs[kk], ws[name]))]
            line["glu"] = [timed(lambda: ops.gated_linear(xs[d], wg, None, 0)),
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


def run_ours(args):
    import torch

    from fms_b200.kernels import ops
    from fms_b200.models import get_model
    from fms_b200.utils.generation import generate

    pk = peaks()
    nlayers = args.layers or MODEL["nlayers"]
    model = get_model("llama", MODEL["variant"], device_type="cuda", data_type="bf16", seed=0, nlayers=nlayers)
    cfg = model.config
    assert (cfg.emb_dim, cfg.nheads, cfg.n_kvheads, cfg.ffn_hidden, cfg.src_vocab_size, cfg.max_expected_seq_len) == (
        MODEL["emb_dim"], MODEL["nheads"], MODEL["kvheads"], MODEL["ffn_hidden"], MODEL["vocab"], MODEL["context"])
    room = args.warmup + args.steps + 8
    engine = model.new_engine(max_tokens=64 * (PROMPT_MAX + 2 * room + 128), max_slots=64)

    def device_decode(batch, steps, warmup):
        """(tokens a second, ms a step, mean context, own kernels launched) of `steps` decode steps."""
        lengths = prompt_lengths(batch)
        prompts = random_prompts(lengths, MODEL["vocab"])
        slots = engine.begin(batch)
        try:
            horizon = max(lengths) + max(3, warmup) + steps + 1
            logits = engine.step(slots, prompts)
            tokens = ops.argmax(logits)
            for _ in range(max(3, warmup)):
                tokens = ops.argmax(engine.decode(slots, tokens_device=tokens, horizon=horizon))
            torch.cuda.synchronize()
            context = sum(engine.length(s) for s in slots) + batch * (steps + 1) / 2.0
            launches0, graphs0 = ops.launches, engine.graph_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                tokens = ops.argmax(engine.decode(slots, tokens_device=tokens, horizon=horizon))
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            launched = (ops.launches - launches0) + (engine.graph_launches - graphs0) * engine.kernels_per_graph
            engine.check()
        finally:
            engine.release(slots)
        return batch * steps / (ms / 1e3), ms / steps, context, launched

    def host_decode(batch, steps, warmup):
        """The same through generate(): host token lists in, host tokens out, every step."""
        lengths = prompt_lengths(batch)
        prompts = [torch.tensor(p) for p in random_prompts(lengths, MODEL["vocab"])]
        h2d0 = engine.h2d_bytes
        _, times = generate(engine, prompts, max_new_tokens=1 + max(3, warmup) + steps, do_sample=False,
                            timing="per-token")
        timed = times[-steps:]
        h2d_decode = 4 * batch  # each decode step copies its tokens from a pinned host array
        assert engine.h2d_bytes - h2d0 >= h2d_decode * steps
        return batch * steps / sum(timed), h2d_decode, 4 * batch

    def prefill(tokens, repeats=5):
        prompt = random_prompts([tokens], MODEL["vocab"], seed=7)
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

    if args.only:  # a short run of one part, for profilers: prints that part's figures only
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "ms": round(prefill(PREFILL_TOKENS, repeats=args.steps), 3)}))
        else:
            batch = int(args.only.split("_b")[1])
            v, ms, _, _ = device_decode(batch, args.steps, args.warmup)
            print(json.dumps({"only": args.only, "value": round(v, 1), "ms_per_step": round(ms, 4)}))
        return
    sampler = ClockSampler()
    sampler.start()
    value, ms_step, context, launched = device_decode(BATCH, args.steps, args.warmup)
    e2e, h2d, d2h = host_decode(BATCH, args.steps, args.warmup)
    sampler.stop()
    side = max(8, args.steps // 4)
    b1 = device_decode(1, side, args.warmup)[0]
    b64 = device_decode(64, side, args.warmup)[0]
    pf_ms = prefill(PREFILL_TOKENS)
    pf_flops = prefill_flops(nlayers, PREFILL_TOKENS)
    gbs = decode_bytes(nlayers, context) / (ms_step / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch 8 ({MODEL['label']} shape, random weights)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": MODEL["name"], "layers": nlayers, "layers_of_model": MODEL["nlayers"], "emb_dim": MODEL["emb_dim"],
            "nheads": MODEL["nheads"], "kvheads": MODEL["kvheads"], "head_dim": MODEL["head_dim"],
            "ffn_hidden": MODEL["ffn_hidden"], "vocab": MODEL["vocab"], "context": MODEL["context"],
            "global_batch": BATCH, "seq_len": f"prompts uniform in [{PROMPT_MIN},{PROMPT_MAX}]",
            "mean_context": round(context / BATCH, 1), "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 gpu",
            "weights": "random N(0,0.02), seed 0", "l2": f"weights read per step ({decode_bytes(nlayers, 0) / 1e9:.0f} GB) exceed L2; no flush",
            "cache_block_tokens": 64, "peaks": pk["source"],
        },
        "clocks": sampler.summary(),
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launched),
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                    "frac": round(pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)},
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
    side = max(8, args.steps // 4)
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
