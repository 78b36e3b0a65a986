"""The engine on the GPU against the plain implementation, in float32 and in bfloat16: each request alone
and whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests end
earlier, one batch after another so that slots and blocks are used again; long decoding; the first
tokens of a sequence; generation through the entry point; the replay program."""
import io
import json
import os
import select
import subprocess
import sys

import pytest
import torch

import plain_llama as pl
from tiny_models import TINY, tiny_prompts

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["fp32", "bf16"]


def close(got, want, dtype):
    """float32: the engine's own rounding only.  bfloat16: activations are rounded to 8 bits of mantissa
    between kernels; 2% of the largest logit, fixed before the first run."""
    want = want.double()
    got = got.double().cpu()
    if dtype == "fp32":
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    else:
        torch.testing.assert_close(got, want, atol=0.02 * want.abs().max().item(), rtol=0.02)


@pytest.fixture(scope="module")
def oracles(tiny_folders):
    return {w: pl.PlainLlama(tiny_folders[w]) for w in tiny_folders}


@pytest.fixture(scope="module")
def models(tiny_folders):
    from fms_b200.models import get_model

    cache = {}

    def get(which, dtype):
        if (which, dtype) not in cache:
            cache[(which, dtype)] = get_model("hf_pretrained", model_path=tiny_folders[which], device_type="cuda",
                                              data_type=dtype)
        return cache[(which, dtype)]

    return get


def long_requests(which, n=5, seed=0):
    """Requests of unequal lengths, some longer than a cache block and than a decode split."""
    cfg = TINY[which][0]
    g = torch.Generator().manual_seed(50 + seed)
    top = cfg["max_position_embeddings"]
    lengths = [min(top, x) for x in ([33, 64, 65, 40, 128, 1] if top <= 128 else [33, 300, 65, 700, 129, 1])][:n]
    return [torch.randint(0, cfg["vocab_size"], (k,), generator=g).tolist() for k in lengths]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["a", "b", "c", "d", "e"])
def test_each_request_alone_and_whole(models, oracles, which, dtype):
    engine = models(which, dtype).new_engine(max_tokens=1024)
    for req in tiny_prompts(which) + long_requests(which, 4):
        (slot,) = engine.begin(1)
        got = engine.step([slot], [req], [list(range(len(req)))])
        engine.release([slot])
        close(got, oracles[which].logits(req), dtype)
    engine.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["a", "b", "c", "d", "e"])
def test_last_32_tokens_one_by_one(models, oracles, which, dtype):
    engine = models(which, dtype).new_engine(max_tokens=1024)
    for req in long_requests(which, 6):
        want = oracles[which].logits(req)
        cut = max(0, len(req) - 32)
        (slot,) = engine.begin(1)
        parts = []
        if cut:
            parts.append(engine.step([slot], [req[:cut]], [list(range(cut))]))
        for t in range(cut, len(req)):
            parts.append(engine.step([slot], [[req[t]]], [[0]]))
        engine.release([slot])
        close(torch.cat(parts), want, dtype)
    engine.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["a", "b", "c", "d", "e"])
def test_unequal_batches_one_after_another_with_reuse(models, oracles, which, dtype):
    """Three batches on a cache that holds only one of them: every slot and block is used again.  Freed
    blocks are filled with NaN, so anything stale that is read shows."""
    reqs = [long_requests(which, 5, seed=s) for s in range(3)]
    need = max(sum((len(r) + 63) // 64 * 64 for r in batch) for batch in reqs)
    engine = models(which, dtype).new_engine(max_tokens=need, max_slots=5)
    group = engine.cache.groups[0]
    for batch in reqs:
        want = [oracles[which].logits(r) for r in batch]
        prefill = [max(1, len(r) - 6 - i) for i, r in enumerate(batch)]  # unequal numbers of decoded tokens
        slots = engine.begin(len(batch))
        got = [[] for _ in batch]
        lg = engine.step(slots, [r[:k] for r, k in zip(batch, prefill)], [list(range(k)) for k in prefill])
        o = 0
        for i, k in enumerate(prefill):
            got[i].append(lg[o:o + k])
            o += k
        live = list(range(len(batch)))
        at = list(prefill)
        while live:
            # requests that have no tokens left end here, earlier than the others
            done = [i for i in live if at[i] >= len(batch[i])]
            for i in done:
                blocks = group.held_blocks(slots[i])
                engine.release([slots[i]])
                group.storage[:, :, blocks] = float("nan")
            live = [i for i in live if i not in done]
            if not live:
                break
            lg = engine.step([slots[i] for i in live], [[batch[i][at[i]]] for i in live])
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                at[i] += 1
        for i in range(len(batch)):
            close(torch.cat(got[i]), want[i], dtype)
        assert engine.cache.slots.n_held == 0 and group.pool.n_held == 0
    engine.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["c", "d"])
def test_long_decoding(models, oracles, which, dtype):
    """A short prompt, then hundreds of tokens one by one: across block edges and decode splits ("d": with
    attention that a few keys carry)."""
    g = torch.Generator().manual_seed(60)
    req = torch.randint(0, TINY[which][0]["vocab_size"], (600,), generator=g).tolist()
    want = oracles[which].logits(req)
    engine = models(which, dtype).new_engine(max_tokens=640)
    (slot,) = engine.begin(1)
    parts = [engine.step([slot], [req[:3]], [[0, 1, 2]])]
    for t in range(3, len(req)):
        parts.append(engine.step([slot], [[req[t]]]))
    engine.release([slot])
    close(torch.cat(parts), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["a", "b"])
def test_first_tokens_of_a_sequence(models, oracles, which, dtype):
    """Position 0 sees one key; a one-token prompt is a prefill of one token."""
    engine = models(which, dtype).new_engine(max_tokens=256)
    req = tiny_prompts(which)[-1][:6]
    want = oracles[which].logits(req)
    (slot,) = engine.begin(1)
    parts = [engine.step([slot], [[t]]) for t in req]
    engine.release([slot])
    close(torch.cat(parts), want, dtype)
    slots = engine.begin(2)
    lg = engine.step(slots, [req[:1], req[:2]], [[0], [0, 1]])
    engine.release(slots)
    close(lg, torch.cat([want[:1], want[:2]]), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["b", "c", "d", "e"])
def test_prompts_cut_into_steps_of_several_tokens(models, oracles, which, dtype):
    """Two requests whose tokens come in pieces of unequal sizes (several tokens onto what is already cached,
    across the edges of cache blocks, one request resting while the other goes on): the same logits as whole.
    The reference needs an explicit mask for this (fms/modules/attention.py:268-271); here a row sees the
    cached positions up to its own."""
    engine = models(which, dtype).new_engine(max_tokens=2048)
    reqs = long_requests(which, 5)[1:3]
    want = [oracles[which].logits(r) for r in reqs]
    slots = engine.begin(2)
    got = [[], []]
    at = [0, 0]
    pieces = [(7, 3), (1, 62), (57, 0), (0, 1), (10 ** 6, 10 ** 6)]  # (tokens of request 0, of request 1) a step
    for piece in pieces:
        who = [i for i in (0, 1) if piece[i] and at[i] < len(reqs[i])]
        if not who:
            continue
        toks = [reqs[i][at[i]:at[i] + piece[i]] for i in who]
        lg = engine.step([slots[i] for i in who], toks, [list(range(len(t))) for t in toks])
        o = 0
        for i, t in zip(who, toks):
            got[i].append(lg[o:o + len(t)])
            o += len(t)
            at[i] += len(t)
    engine.release(slots)
    engine.check()
    for i in (0, 1):
        assert at[i] == len(reqs[i])
        close(torch.cat(got[i]), want[i], dtype)


@pytest.mark.parametrize("which", ["a", "b"])
def test_greedy_generation_through_the_entry_point(models, oracles, which):
    from fms_b200.utils.generation import generate

    prompts = tiny_prompts(which)
    model = models(which, "fp32")
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=8, do_sample=False)
    for o, p in zip(out, prompts):
        assert o.tolist() == pl.plain_generate(oracles[which], p, 8)
    # one prompt alone gives the same tokens as in the batch
    alone = generate(model, torch.tensor(prompts[1]), max_new_tokens=8, do_sample=False)
    assert alone.tolist() == out[1].tolist()
    # model(x): logits of whole sequences, as the reference's forward without a cache
    one = model(torch.tensor(prompts[1]))
    close(one, oracles[which].logits(prompts[1]), "fp32")
    two = model(torch.tensor([prompts[1], prompts[1][::-1]]), last_n_tokens=2)
    assert two.shape == (2, 2, one.shape[-1])
    close(two[0], oracles[which].logits(prompts[1])[-2:], "fp32")
    close(two[1], oracles[which].logits(prompts[1][::-1])[-2:], "fp32")
    ragged = model(prompts)
    assert [r.shape[0] for r in ragged] == [len(p) for p in prompts]
    close(ragged[0], oracles[which].logits(prompts[0]), "fp32")
    with pytest.raises(NotImplementedError):
        model(torch.tensor(prompts[1]), use_cache=True)
    # the reference's way with unequal prompts, a padded rectangle: padding changes no token
    from fms_b200.utils.generation import pad_input_ids, trim_prefix

    pad = max(max(p) for p in prompts) + 1  # an id that no prompt starts with
    ids, extra = pad_input_ids([torch.tensor(p) for p in prompts], min_pad_length=max(map(len, prompts)) + 7,
                               pad_token_id=pad)
    padded = generate(model, ids, max_new_tokens=8, do_sample=False, extra_kwargs=extra)
    assert padded.shape == (len(prompts), ids.shape[1] + 8)
    assert [trim_prefix(r, pad).tolist() for r in padded] == [o.tolist() for o in out]


def test_sampled_generation_is_the_same_alone_and_in_batches(models, oracles):
    from fms_b200.utils.generation import generate

    prompts = tiny_prompts("b")
    model = models("b", "fp32")
    kw = dict(max_new_tokens=16, do_sample=True, temperature=0.8, top_k=0, seed=11)
    together = generate(model, [torch.tensor(p) for p in prompts], **kw)
    in_twos = generate(model, [torch.tensor(p) for p in prompts], batch_size=2, **kw)
    assert [t.tolist() for t in together] == [t.tolist() for t in in_twos]
    plain = [pl.plain_generate(oracles["b"], p, 16, do_sample=True, temperature=0.8, top_k=0, seed=11, request=i)
             for i, p in enumerate(prompts)]
    same = sum(a == b for t, w in zip(together, plain) for a, b in zip(t.tolist(), w))
    assert same >= sum(len(w) for w in plain) - 1  # float32 against float64 running sums


def test_bfloat16_greedy_generation(models, oracles):
    from fms_b200.utils.generation import generate

    prompts = tiny_prompts("a")
    logits = []
    out = generate(models("a", "bf16"), [torch.tensor(p) for p in prompts], max_new_tokens=8, do_sample=False,
                   post_iteration_hook=lambda it, lg, toks, reqs: logits.append((reqs, lg.float().cpu())))
    # every step's logits belong to the sequence generated so far
    for i, (o, p) in enumerate(zip(out, prompts)):
        want = oracles["a"].logits(o.tolist()[:-1])[len(p) - 1:]
        got = torch.stack([lg[reqs.index(i)] for reqs, lg in logits if i in reqs])
        close(got, want, "bf16")


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_that_ask_for_no_logits(models, oracles, dtype):
    """A prompt that comes in three pieces of which only the last asks for logits, beside a request that asks at every
    place; then a step in which nobody asks for anything (an empty result), then single tokens again."""
    engine = models("d", dtype).new_engine(max_tokens=1024)
    a, b = long_requests("d", 5)[1:3]  # 300 and 65 tokens
    want_a, want_b = oracles["d"].logits(a), oracles["d"].logits(b)
    slots = engine.begin(2)
    lg = engine.step(slots, [a[:100], b[:20]], [[], list(range(20))])
    assert lg.shape[0] == 20
    got_b = [lg]
    lg = engine.step(slots, [a[100:170], b[20:21]], [[], [0]])  # one of the two brings a single token
    got_b.append(lg)
    nothing = engine.step(slots, [a[170:250], b[21:40]], [[], []])
    assert tuple(nothing.shape) == (0, want_a.shape[1])
    lg = engine.step(slots, [a[250:298], b[40:]], [[47], list(range(25))])
    got_a = [lg[:1]]
    got_b.append(lg[1:])
    for t in (298, 299):
        got_a.append(engine.step([slots[0]], [[a[t]]]))
    engine.release(slots)
    engine.check()
    close(torch.cat(got_a), want_a[297:], dtype)
    close(torch.cat(got_b), torch.cat([want_b[:21], want_b[40:]]), dtype)


def test_a_batch_whose_requests_end_one_by_one_keeps_few_graphs(models, oracles):
    """Thirty-two requests that start together and end one at a time: decode steps of 32, 31, ... 1 sequences, each
    number for several steps.  More than eight sequences are filled up to 12, 16, 24 or 32 rows (the filler rows live in
    the cache's spare slot), so twelve sizes are captured instead of thirty-two.  The engine keeps at most
    ``max_graphs`` captures (and their logits buffers), all drawing from one pool: the logits stay right and a second
    pass over the same schedule holds no more memory than the first."""
    model = models("d", "bf16")
    engine = model.new_engine(max_tokens=64 * 2 * 32, max_slots=32, max_graphs=4)
    g = torch.Generator().manual_seed(90)
    reqs = [torch.randint(0, TINY["d"][0]["vocab_size"], (20 + 3 * i,), generator=g).tolist() for i in range(32)]
    want = [oracles["d"].logits(r) for r in reqs]
    prompt = 12

    def run():
        slots = engine.begin(32)
        got = [[] for _ in reqs]
        lg = engine.step(slots, [r[:prompt] for r in reqs])
        for i in range(32):
            got[i].append(lg[i:i + 1])
        at = [prompt] * 32
        live = list(range(32))
        while live:
            lg = engine.step([slots[i] for i in live], [[reqs[i][at[i]]] for i in live])
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                at[i] += 1
            for i in [i for i in live if at[i] == len(reqs[i])]:
                engine.release([slots[i]])
                live.remove(i)
        for i in range(32):
            close(torch.cat(got[i]), want[i][prompt - 1:], "bf16")

    run()
    torch.cuda.synchronize()
    first = torch.cuda.memory_allocated()
    captured = engine.graphs_captured
    assert sorted(engine._decode) == [1, 2, 3, 4, 5, 6, 7, 8, 12, 16, 24, 32]  # the sizes that steps were run at
    assert 12 <= captured <= 16 and len(engine._graphs) <= 4
    run()
    torch.cuda.synchronize()
    assert engine.graphs_captured > captured  # dropped captures are made again when their size comes back
    assert len(engine._graphs) <= 4
    assert torch.cuda.memory_allocated() <= first + (1 << 20)
    engine.check()


def test_generate_asks_for_no_more_cache_than_the_device_has_room_for(tiny_folders, oracles, monkeypatch):
    """Twelve requests whose cache would take twelve blocks, on a device that (the test says) has room for five: the
    model's own engine is made for what fits, the requests run in several batches, and the tokens are the plain loop's."""
    from fms_b200.models import get_model
    from fms_b200.utils.generation import generate

    model = get_model("hf_pretrained", model_path=tiny_folders["b"], device_type="cuda", data_type="fp32")
    per_token = model.cache_bytes_per_token()
    cfg = TINY["b"][0]
    assert per_token == 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * (cfg["hidden_size"] // cfg["num_attention_heads"]) * 4
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (int(5 * 64 * per_token / 0.8) + 1, 1 << 40))
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, cfg["vocab_size"], (int(k),), generator=g).tolist() for k in torch.randint(1, 50, (12,), generator=g)]
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=5, do_sample=False)
    engine = model.engine()
    assert engine.cache.n_blocks == 5 and engine.cache.max_slots <= 5 and engine.cache.slots.n_held == 0
    for o, p in zip(out, prompts):
        assert o.tolist() == pl.plain_generate(oracles["b"], p, 5)


def test_warm_up_captures_the_graphs_before_the_first_request(models, oracles):
    model = models("b", "fp32")
    engine = model.new_engine(max_tokens=64 * 2 * 12, max_slots=12)
    engine.warm_up([1, 3, 10, 11], horizon=100)  # ten and eleven sequences are both steps of twelve rows
    assert engine.graphs_captured == 3 and engine.cache.slots.n_held == 0 and sorted(engine._decode) == [1, 3, 12]
    assert all(g.pool.n_held == 0 for g in engine.cache.groups)
    reqs = long_requests("b", 3)
    slots = engine.begin(3)
    engine.step(slots, [r[:-2] for r in reqs], [[] for _ in reqs])
    launched = engine.graph_launches
    got = [engine.decode(slots, [r[-2 + t] for r in reqs], horizon=100).clone() for t in range(2)]
    assert engine.graph_launches == launched + 2 and engine.graphs_captured == 3  # replayed from the first step on
    engine.release(slots)
    for i, r in enumerate(reqs):
        close(torch.stack([got[0][i], got[1][i]]), oracles["b"].logits(r)[-2:], "fp32")
    engine.check()


def _trace_lines(reqs, prefill):
    """Steps of one batch: prompts together, then one token each; shorter requests end earlier."""
    lines, step = [], 0
    at = list(prefill)
    ids = [f"r{i}" for i in range(len(reqs))]
    entries = [{"id": ids[i], "tokens": reqs[i][:at[i]], "want": list(range(at[i]))} for i in range(len(reqs))]
    live = list(range(len(reqs)))
    while True:
        end = [ids[i] for i in live if at[i] >= len(reqs[i])]
        lines.append({"step": step, "entries": entries, "end": end})
        live = [i for i in live if at[i] < len(reqs[i])]
        if not live:
            break
        step += 1
        entries = [{"id": ids[i], "tokens": [reqs[i][at[i]]], "want": [0]} for i in live]
        for i in live:
            at[i] += 1
    return lines


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_folders, oracles, tmp_path, dtype):
    reqs = long_requests("b", 4)
    prefill = [max(1, len(r) - 5) for r in reqs]
    lines = _trace_lines(reqs, prefill)
    out = tmp_path / f"out_{dtype}"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_folders["b"], "--dtype", dtype, "--out",
         str(out), "--max-tokens", str(sum((len(r) + 63) // 64 * 64 for r in reqs))],
        input="\n".join(json.dumps(l) for l in lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for l in lines for x in ("done", str(l["step"]))]
    import numpy as np

    vocab = TINY["b"][0]["vocab_size"]
    got = {i: [] for i in range(len(reqs))}
    for l in lines:
        data = torch.from_numpy(np.fromfile(out / f"{l['step']}.f32", dtype="<f4").reshape(-1, vocab).copy())
        o = 0
        for e in l["entries"]:
            k = len(e["want"])
            got[int(e["id"][1:])].append(data[o:o + k])
            o += k
        assert o == data.shape[0]
    for i, r in enumerate(reqs):
        close(torch.cat(got[i]), oracles["b"].logits(r), "fp32" if dtype == "float32" else "bf16")


def test_trace_run_with_steps_that_want_nothing(tiny_folders, oracles, tmp_path):
    """A prompt cut into three steps of which only the last asks for logits (no file for the first two), and a
    step with an empty ``entries`` list."""
    import numpy as np

    req = long_requests("d", 5)[1]
    want = oracles["d"].logits(req)
    vocab = TINY["d"][0]["vocab_size"]
    lines = [{"step": 0, "entries": [{"id": "p", "tokens": req[:128], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": req[128:130]}], "end": []},
             {"step": 2, "entries": [], "end": []},
             {"step": 3, "entries": [{"id": "p", "tokens": req[130:], "want": [0, len(req) - 131]}], "end": ["p"]}]
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_folders["d"], "--dtype", "float32", "--out",
         str(tmp_path), "--max-tokens", "320"], input="\n".join(json.dumps(l) for l in lines) + "\n", capture_output=True,
        text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(tmp_path)) == ["3.f32"]
    got = torch.from_numpy(np.fromfile(tmp_path / "3.f32", dtype="<f4").reshape(-1, vocab).copy())
    close(got, want[[130, len(req) - 1]], "fp32")


def test_trace_run_answers_each_step_before_the_next_is_written(tiny_folders, oracles, tmp_path):
    """The caller writes a step only after ``done`` of the step before: the program must not wait for more
    input before it runs a line, and must have written the step's file when it says ``done``."""
    import numpy as np

    req = tiny_prompts("a")[2]
    vocab = TINY["a"][0]["vocab_size"]
    proc = subprocess.Popen(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_folders["a"], "--dtype", "float32",
         "--out", str(tmp_path), "--max-tokens", "64"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        want = oracles["a"].logits(req)
        cut = len(req) - 3
        steps = [{"step": 0, "entries": [{"id": "x", "tokens": req[:cut], "want": [cut - 1]}], "end": []}]
        steps += [{"step": k + 1, "entries": [{"id": "x", "tokens": [req[cut + k]], "want": [0]}],
                   "end": ["x"] if cut + k == len(req) - 1 else []} for k in range(3)]
        for k, step in enumerate(steps):
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            assert select.select([proc.stdout], [], [], 600)[0], f"no answer to step {k}"
            assert proc.stdout.readline().split() == ["done", str(k)]
            got = torch.from_numpy(np.fromfile(tmp_path / f"{k}.f32", dtype="<f4").reshape(-1, vocab).copy())
            close(got, want[cut - 1 + k][None], "fp32")
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


FURTHER_MODELS = {
    # biases on every projection, a tied head, eps 1e-3, a feed-forward width that is no multiple of 8
    "biases_tied_hd16": (dict(vocab=97, hidden=48, intermediate=100, layers=1, heads=3, kvheads=3, eps=1e-3, tied=True,
                              attention_bias=True, mlp_bias=True), [5, 70, 33]),
    # one kv head for five, an odd feed-forward width, the llama3 rescaling of the rotation's frequencies
    "mqa_f173_llama3": (dict(vocab=1000, hidden=160, intermediate=173, layers=2, heads=5, kvheads=1, theta=5e5, context=2048,
                             rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                           "high_freq_factor": 4.0, "original_max_position_embeddings": 64}),
                        [300, 65, 1]),
    # seven query heads a kv head (no whole tile of eight), head size 80
    "group7_hd80": (dict(vocab=129, hidden=560, intermediate=96, layers=1, heads=7, kvheads=1), [64, 65, 200]),
    # the largest head size, a feed-forward of 8
    "hd256_f8": (dict(vocab=50, hidden=512, intermediate=8, layers=1, heads=2, kvheads=1), [40]),
    # prompts of more than 1,024 rows (the tcgen05 product) with a k of 1,016 and biases in its epilogue
    "tc_k1016_biases": (dict(vocab=300, hidden=1024, intermediate=1016, layers=1, heads=16, kvheads=4, context=2048,
                             attention_bias=True, mlp_bias=True), [1030, 20]),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(FURTHER_MODELS))
def test_further_configurations_against_the_plain_implementation(tmp_path, monkeypatch, name, dtype):
    """Sizes and options that the tiny models do not have: the prompts in one step, then four tokens one by one."""
    from fms_b200.models import get_model
    from tiny_models import llama_config, tiny_tensors_with_biases, write_folder

    from fms_b200.kernels import ops

    if name.startswith("tc_"):  # send the long prompt's products through the own tcgen05 kernel, as smaller prompts do not by default
        monkeypatch.setattr(ops, "TENSOR_CORE_ROWS", 1024)
        monkeypatch.setattr(ops, "TENSOR_CORE_ROWS_GLU", 1024)
        monkeypatch.setattr(ops, "TENSOR_CORE_ROWS_QKV", 1024)
        monkeypatch.setattr(ops, "TENSOR_CORE_MAX_PADDING", 10.0)
    sizes, lengths = FURTHER_MODELS[name]
    cfg = llama_config(**sizes)
    folder = write_folder(str(tmp_path / name), cfg, tiny_tensors_with_biases(cfg, 7))
    oracle = pl.PlainLlama(folder)
    g = torch.Generator().manual_seed(3)
    reqs = [torch.randint(0, cfg["vocab_size"], (n + 4,), generator=g).tolist() for n in lengths]
    want = torch.cat([oracle.logits(r)[-5:] for r in reqs])
    engine = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype).new_engine(4096)
    slots = engine.begin(len(reqs))
    rows = [engine.step(slots, [r[:-4] for r in reqs]).cpu()]
    for t in range(4, 0, -1):
        rows.append(engine.step(slots, [[r[-t]] for r in reqs]).cpu())
    engine.release(slots)
    engine.check()
    close(torch.stack(rows, 1).reshape(-1, cfg["vocab_size"]), want, dtype)


def test_matrices_stored_in_32_bit_inside_a_bfloat16_model(tmp_path):
    """A checkpoint whose output projections, down projections and head are stored in float32 (with values that
    bfloat16 cannot hold), loaded with data_type="bf16": those matrices stay float32 and take the float32 product,
    everything else runs as in any bfloat16 model.  Prompts in one step, then single tokens."""
    from fms_b200.models import get_model
    from tiny_models import TINY_D, tiny_tensors_of, write_folder

    t = tiny_tensors_of("d")
    g = torch.Generator().manual_seed(5)
    for k in list(t):
        if "o_proj" in k or "down_proj" in k or k == "lm_head.weight":
            t[k] = t[k].float() * (1.0 + 0.003 * torch.rand(t[k].shape, generator=g))  # many mantissa bits
    folder = write_folder(str(tmp_path / "m"), TINY_D, t)
    oracle = pl.PlainLlama(folder)
    model = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type="bf16")
    sd = model.state_dict()
    assert sd["head.weight"].dtype == torch.float32 and sd["base_model.layers.1.attn.dense.weight"].dtype == torch.float32
    assert sd["base_model.layers.1.attn.in_proj.qkv_fused.weight"].dtype == torch.bfloat16
    reqs = long_requests("d", 4)
    engine = model.new_engine(max_tokens=2048)
    slots = engine.begin(len(reqs))
    cut = [max(1, len(r) - 4) for r in reqs]
    first = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)])
    rows = [engine.step(slots, [[r[c + i]] for r, c in zip(reqs, cut)]) for i in range(4)]
    engine.release(slots)
    engine.check()
    for i, (r, c) in enumerate(zip(reqs, cut)):
        close(torch.cat([first[i:i + 1]] + [x[i:i + 1] for x in rows]), oracle.logits(r)[c - 1:], "bf16")


def _peaked_model(tmp_path, qk_std, **sizes):
    """A model folder of the given sizes whose q and k projections are drawn wide enough for attention scores with a
    standard deviation between 1.5 and 2, and its oracle."""
    from tiny_models import llama_config, tiny_tensors, write_folder

    cfg = llama_config(**sizes)
    folder = write_folder(str(tmp_path / "m"), cfg, tiny_tensors(cfg, 5, torch.float32, qk_std=qk_std))
    return folder, pl.PlainLlama(folder)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_size_128_model(tmp_path, dtype):
    """A model with the head size, group size and widths (in small) of the benchmark's: prompts long enough for
    the tcgen05 product (1,024 rows and more in one step) and the tcgen05 attention, decode through the
    weight-streaming product and the CUDA graph."""
    from fms_b200.models import get_model

    folder, oracle = _peaked_model(tmp_path, 0.04, vocab=4099, hidden=1024, intermediate=2816, layers=2, heads=8, kvheads=2,
                                   theta=5e5, context=2048)
    g = torch.Generator().manual_seed(70)
    reqs = [torch.randint(0, 4099, (k,), generator=g).tolist() for k in (900, 300, 41)]
    engine = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype).new_engine(2048)
    slots = engine.begin(3)
    cut = [len(r) - 5 for r in reqs]
    places = [[0, c // 2, c - 1] for c in cut]
    first = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], places)
    rows = [engine.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)]) for t in range(5)]
    engine.release(slots)
    engine.check()
    for i, (r, c) in enumerate(zip(reqs, cut)):
        got = torch.cat([first[3 * i:3 * i + 3]] + [x[i:i + 1] for x in rows])
        close(got, oracle.logits(r, rows=places[i] + list(range(c, len(r)))), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_many_short_requests_in_one_batch(tmp_path, dtype):
    """Forty requests of 1 to 120 tokens in one batch (prompts in one step of more than a thousand rows, whose
    attention tiles span many sequences; then decode steps of forty rows), on the model shape of the test above."""
    from fms_b200.models import get_model

    folder, oracle = _peaked_model(tmp_path, 0.04, vocab=4099, hidden=1024, intermediate=2816, layers=2, heads=8, kvheads=2,
                                   theta=5e5, context=2048)
    g = torch.Generator().manual_seed(71)
    lens = [1, 2, 63, 64, 65, 120] + [int(v) for v in torch.randint(1, 121, (34,), generator=g)]
    reqs = [torch.randint(0, 4099, (k + 3,), generator=g).tolist() for k in lens]
    assert sum(lens) > 1024
    engine = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype).new_engine(64 * 120)
    slots = engine.begin(len(reqs))
    rows = [engine.step(slots, [r[:k] for r, k in zip(reqs, lens)], [[k - 1] for k in lens])]
    for t in range(3):
        rows.append(engine.step(slots, [[r[k + t]] for r, k in zip(reqs, lens)]))
    engine.release(slots)
    engine.check()
    got = torch.stack(rows, 1)
    for i, (r, k) in enumerate(zip(reqs, lens)):
        close(got[i], oracle.logits(r, rows=list(range(k - 1, k + 3))), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_of_many_long_sequences(tmp_path, dtype):
    """Sixty-four requests of 700 to 1,000 tokens: enough keys and values for decode attention to take its
    streaming kernel (persistent warps fed by TMA), first by plain launches, then inside the captured graph."""
    from fms_b200.kernels import ops
    from fms_b200.models import get_model

    folder, oracle = _peaked_model(tmp_path, 0.06, vocab=1031, hidden=512, intermediate=1024, layers=2, heads=8, kvheads=4,
                                   theta=5e5, context=2048)
    g = torch.Generator().manual_seed(71)
    reqs = [torch.randint(0, 1031, (int(k),), generator=g).tolist() for k in torch.randint(700, 1000, (64,), generator=g)]
    steps = 4
    engine = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype).new_engine(64 * 1024)
    before = ops.attention_stream_launches(64)
    slots = engine.begin(len(reqs))
    rows = [engine.step(slots, [r[:-steps] for r in reqs])]
    for t in range(steps, 0, -1):
        rows.append(engine.step(slots, [[r[-t]] for r in reqs]))
    engine.release(slots)
    engine.check()
    # 2 layers: the first decode step launches them plainly, the second captures them; replays launch nothing new
    assert ops.attention_stream_launches(64) - before == (4 if dtype == "bf16" else 0)
    got = torch.stack(rows, 1)
    for i, r in enumerate(reqs):
        close(got[i], oracle.logits(r, rows=list(range(len(r) - steps - 1, len(r)))), dtype)


def windowed_model(folder, dtype, window):
    """Llama's layers with a window on every mixer (``window``: one number, or one a layer with 0 for none): a
    test's variation, not a model of anyone's."""
    import dataclasses

    from fms_b200.models import get_model
    from fms_b200.models.llama import LLaMA
    from fms_b200.weights import FileSource

    class WindowedLLaMA(LLaMA):
        def decoder_spec(self):
            spec = super().decoder_spec()
            windows = window if isinstance(window, (list, tuple)) else [window] * len(spec.layers)
            layers = tuple(dataclasses.replace(b, mixer=dataclasses.replace(b.mixer, window=w))
                           for b, w in zip(spec.layers, windows))
            return dataclasses.replace(spec, layers=layers)

    base = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype)
    model = WindowedLLaMA(base.config)
    model.load(FileSource(folder), "hf", "cuda", base.dtype)
    return model


def plain_windowed_logits(plain, ids, window):
    x = pl.plain_embedding(torch.as_tensor(ids), plain.w["model.embed_tokens.weight"])
    windows = window if isinstance(window, (list, tuple)) else [window] * plain.c["nlayers"]
    for i in range(plain.c["nlayers"]):
        x = plain.block(i, x, torch.arange(len(ids)), window=windows[i])
    x = pl.plain_rmsnorm(x, plain.w["model.norm.weight"], plain.c["eps"])
    return x @ plain.w["lm_head.weight"].T


@pytest.mark.parametrize("which", ["c", "d"])
def test_window_attention_through_the_engine(tiny_folders, oracles, which):
    """A decoder whose mixers keep a window of 40 keys: the cache gives blocks back as they leave the window, and
    the logits equal the plain implementation's with the same window, whole and token by token."""
    g = torch.Generator().manual_seed(80)
    req = torch.randint(0, TINY[which][0]["vocab_size"], (300,), generator=g).tolist()
    want = plain_windowed_logits(oracles[which], req, 40)
    for dtype in ("fp32", "bf16"):
        model = windowed_model(tiny_folders[which], dtype, 40)
        engine = model.new_engine(max_tokens=64 * 4, max_slots=1)  # 4 blocks: the sequence of 300 needs 5 without a window
        (slot,) = engine.begin(1)
        parts = [engine.step([slot], [req[:130]], [list(range(130))])]
        parts.append(engine.step([slot], [req[130:200]], [list(range(70))]))
        for t in range(200, 300):
            parts.append(engine.step([slot], [[req[t]]]))
        assert len(engine.cache.groups[0].held_blocks(slot)) <= 2
        engine.release([slot])
        engine.check()
        close(torch.cat(parts), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layers_with_different_needs_have_storage_of_their_own(tiny_folders, oracles, dtype):
    """Layer 0 keeps a window of 40 keys, layer 1 all keys: two groups in the cache, each with its own blocks and
    table; the windowed group gives blocks back while the other keeps them.  Three requests of unequal lengths,
    prompts in one step and then single tokens, the shortest ending first."""
    windows = [40, 0]
    reqs = long_requests("d", 4)[:3]  # 33, 300, 65 tokens
    want = [plain_windowed_logits(oracles["d"], r, windows) for r in reqs]
    engine = windowed_model(tiny_folders["d"], dtype, windows).new_engine(max_tokens=64 * 8, max_slots=3)
    assert len(engine.cache.groups) == 2 and sorted(g.request.window for g in engine.cache.groups) == [0, 40]
    slots = engine.begin(3)
    cut = [20, 200, 60]
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], [list(range(c)) for c in cut])
    o = 0
    for i, c in enumerate(cut):
        got[i].append(lg[o:o + c])
        o += c
    at, live = list(cut), [0, 1, 2]
    while live:
        lg = engine.step([slots[i] for i in live], [[reqs[i][at[i]]] for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
            at[i] += 1
        if 1 in live and at[1] == 290:
            held = {g.request.window: len(g.held_blocks(slots[1])) for g in engine.cache.groups}
            assert held[0] == 5 and held[40] <= 2  # all 290 keys there, 40 of them here
        for i in [i for i in live if at[i] == len(reqs[i])]:
            engine.release([slots[i]])
            live.remove(i)
    engine.check()
    assert all(g.pool.n_held == 0 for g in engine.cache.groups)
    for i in range(3):
        close(torch.cat(got[i]), want[i], dtype)


@pytest.fixture(scope="module")
def planted(tmp_path_factory):
    from tiny_models import TINY_D, planted_tensors, write_folder

    folder = write_folder(str(tmp_path_factory.mktemp("planted")), TINY_D, planted_tensors())
    return folder, pl.PlainLlama(folder)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_key_that_carries_the_whole_attention(planted, dtype):
    """Five requests in one batch, in each a key that gets all the attention of certain queries: at position 0,
    on both sides of a cache block's edge (63, 64) and of a decode split's edge (255, 256).  The queries stand right
    behind the key, further on in the prompt, and among the last 32 tokens, which are fed one by one; the shorter
    requests end earlier.  A key that is dropped, read from a wrong place or counted twice changes these rows
    altogether."""
    from fms_b200.models import get_model
    from tiny_models import PLANT_KEYS, planted_request

    folder, oracle = planted
    places = [0, 63, 64, 255, 256]
    lengths = [300, 345, 322, 310, 333]
    reqs = [planted_request(n, at, PLANT_KEYS[i], [at + 1, n - 50, n - 20, n - 1], 40 + i)
            for i, (n, at) in enumerate(zip(lengths, places))]
    want = [oracle.logits(r) for r in reqs]
    # the rows that rest on the planted key differ from what they would be without it by far more than any tolerance
    for r, w, at in zip(reqs, want, places):
        other = list(r)
        other[at] = 1
        assert (oracle.logits(other)[-1] - w[-1]).abs().max() > 0.2 * w[-1].abs().max()
    engine = get_model("hf_pretrained", model_path=folder, device_type="cuda", data_type=dtype).new_engine(
        max_tokens=sum((n + 63) // 64 * 64 for n in lengths), max_slots=5)
    slots = engine.begin(5)
    cut = [n - 32 for n in lengths]
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], [list(range(c)) for c in cut])
    o = 0
    for i, c in enumerate(cut):
        got[i].append(lg[o:o + c])
        o += c
    for t in range(32):
        lg = engine.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)])
        for i in range(5):
            got[i].append(lg[i:i + 1])
    engine.release(slots)
    engine.check()
    for i in range(5):
        close(torch.cat(got[i]), want[i], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_at_the_edge_of_the_window(planted, dtype):
    """With a window of 40 the query at position p sees the keys p-39..p.  A key that carries all the attention is
    the oldest one in the window of one query token and just outside the window of the next; both stand in the
    prompt in one request and among the tokens fed one by one in another."""
    from tiny_models import PLANT_KEYS, planted_request

    folder, oracle = planted
    window = 40
    # (length, key at, queries at): the key leaves the window between the two queries
    cases = [(200, 100, [139, 140]), (200, 150, [189, 190]), (130, 63, [102, 103]), (150, 64, [103, 104])]
    reqs = [planted_request(n, at, PLANT_KEYS[i], q, 60 + i) for i, (n, at, q) in enumerate(cases)]
    want = [plain_windowed_logits(oracle, r, window) for r in reqs]
    for w, (_, _, q) in zip(want, cases):  # seeing the key or not makes all the difference
        assert (w[q[0]] - w[q[1]]).abs().max() > 0.2 * w[q[0]].abs().max()
    engine = windowed_model(folder, dtype, window).new_engine(max_tokens=64 * 16, max_slots=4)
    slots = engine.begin(4)
    cut = [160, 160, 90, 90]  # the queries of the first request lie in the prompt, the others' among the single tokens
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], [list(range(c)) for c in cut])
    o = 0
    for i, c in enumerate(cut):
        got[i].append(lg[o:o + c])
        o += c
    at = list(cut)
    live = [0, 1, 2, 3]
    while live:
        lg = engine.step([slots[i] for i in live], [[reqs[i][at[i]]] for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
            at[i] += 1
        for i in [i for i in live if at[i] == len(reqs[i])]:
            engine.release([slots[i]])
            live.remove(i)
    engine.check()
    for i in range(4):
        close(torch.cat(got[i]), want[i], dtype)


def test_command_line(tiny_folders):
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "fms_inference"), "--model_path", tiny_folders["a"], "--model_source", "hf",
         "--default_dtype", "fp32", "--prompt_ids", "5,17,3", "--prompt_ids", "9,8,7,6,5,4", "--batch_input",
         "--max_new_tokens", "6", "--deterministic"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    oracle = pl.PlainLlama(tiny_folders["a"])
    want = [pl.plain_generate(oracle, p, 6) for p in ([5, 17, 3], [9, 8, 7, 6, 5, 4])]
    assert [[int(x) for x in l.split(",")] for l in lines] == want
    # with the reference's --min_pad_length the prompts are padded to a rectangle first: the same tokens
    padded = subprocess.run(proc.args + ["--min_pad_length", "11"], capture_output=True, text=True, timeout=600)
    assert padded.returncode == 0, padded.stderr[-2000:]
    assert [[int(x) for x in l.split(",")] for l in padded.stdout.splitlines() if l.strip()] == want


def test_bench_line_has_the_keys_of_its_contract():
    """bench.py on two layers and a few steps: one JSON line with the figures and a flat config of at most 20 keys."""
    import json

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--layers", "2", "--steps", "4", "--warmup", "3"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [line for line in r.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "prefill", "roofline", "points"):
        assert key in out, key
    assert out["n_gpus"] == 1 and out["steps"] == 4 and out["value"] > 0 and out["gpu_launches"] > 0
    assert len(out["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in out["config"].values())
    assert out["config"]["layers"] == 2 and out["config"]["layers_of_model"] == 32
    assert set(out["prefill"]) >= {"value", "tokens", "ms", "frac"} and out["prefill"]["tokens"] == 2048
    assert set(out["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac"} and out["roofline"]["bound"] == "hbm"
    assert set(out["points"]) >= {"decode_b1", "decode_b64"}
    assert out["e2e"]["h2d_bytes_per_step"] > 0 and out["e2e"]["d2h_bytes_per_step"] > 0
