"""Schedules drawn at random (fixed seeds): batches of one to five requests of unequal lengths, each request cut
into pieces of its own (so that one step holds a request's first 40 tokens beside another's next single token),
requests that end while others go on, a cache with just enough blocks so that every batch takes over what the one
before gave back, and logits wanted at random places.  Every wanted row is compared with the plain implementation's
row for the whole request.  A hand-made schedule tests what its author thought of; these are there for the rest."""
import random

import pytest
import torch

import plain_llama as pl
from tiny_models import TINY

pytestmark = pytest.mark.gpu


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


def close(got, want, largest, dtype, what):
    """The rule of the other engine tests: float32 to the engine's own rounding; bfloat16 to 2% of the largest logit
    of the request (``largest``), not of the one row."""
    want, got = want.double(), got.double().cpu()
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "fp32" else dict(atol=0.02 * largest, rtol=0.02)
    torch.testing.assert_close(got, want, msg=lambda m: f"{what}: {m}", **tol)


def draw_batch(rng, vocab, top):
    """Requests (token lists) and, for each, the sizes of the pieces it is fed in."""
    n = rng.randint(1, 5)
    requests, pieces = [], []
    for _ in range(n):
        hi = min(top, 330)
        length = rng.choice([1, 2, rng.randint(3, min(70, hi)), rng.randint(min(60, hi), min(140, hi)), rng.randint(min(120, hi), hi)])
        requests.append([rng.randrange(vocab) for _ in range(length)])
        cut, left = [], length
        first = rng.randint(1, left)  # the prompt's first piece: anything from one token to the whole request
        cut.append(first)
        left -= first
        while left:
            piece = 1 if rng.random() < 0.6 else rng.randint(1, min(left, 70))
            cut.append(piece)
            left -= piece
        pieces.append(cut)
    return requests, pieces


def run_batches(rng, new_engine, plain_logits, vocab, top, dtype, label):
    """Three batches one after another through engines from ``new_engine(max_tokens)``; every wanted row against
    ``plain_logits(request)``."""
    engine = None
    for batch_number in range(3):
        requests, pieces = draw_batch(rng, vocab, top)
        need = sum((len(r) + 63) // 64 for r in requests) * 64
        if engine is None or engine.cache.n_blocks * 64 < need:
            # no more blocks than the largest batch so far needs: each batch reuses what the last one gave back
            engine = new_engine(need)
        want = [plain_logits(r) for r in requests]
        largest = [w.abs().max().item() for w in want]
        slots = engine.begin(len(requests))
        fed = [0] * len(requests)
        turn = [0] * len(requests)
        live = list(range(len(requests)))
        step = 0
        while live:
            tokens, wanted, rows = [], [], []
            for i in live:
                k = pieces[i][turn[i]]
                tokens.append(requests[i][fed[i]:fed[i] + k])
                mode = rng.random()
                places = list(range(k)) if mode < 0.4 else ([k - 1] if mode < 0.8 else sorted(rng.sample(range(k), rng.randint(0, min(k, 3)))))
                wanted.append(places)
                rows += [(i, fed[i] + p) for p in places]
            logits = engine.step([slots[i] for i in live], tokens, wanted)
            assert logits.shape[0] == len(rows)
            for row, (i, p) in enumerate(rows):
                close(logits[row], want[i][p], largest[i], dtype, f"{label} batch {batch_number} step {step} request {i} "
                                                                  f"(of {len(requests[i])} tokens) position {p}")
            done = []
            for i in live:
                fed[i] += pieces[i][turn[i]]
                turn[i] += 1
                if fed[i] == len(requests[i]):
                    done.append(i)
            if done:  # those that are through leave; the others go on
                engine.release([slots[i] for i in done])
                live = [i for i in live if i not in done]
            step += 1
        engine.check()
        assert engine.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(15))
def test_a_random_schedule_against_the_plain_implementation(models, oracles, seed, dtype):
    which = "abcde"[seed % 5]
    cfg = TINY[which][0]
    run_batches(random.Random(1000 + seed), lambda need: models(which, dtype).new_engine(max_tokens=need, max_slots=5),
                oracles[which].logits, cfg["vocab_size"], cfg["max_position_embeddings"], dtype, f"seed {seed} model {which}")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(6))
def test_a_random_schedule_with_windows_on_some_layers(tiny_folders, oracles, seed, dtype):
    """The same with layers that keep a window of keys (a test's variation of the model): the windowed group of the
    cache gives blocks back while a request runs and takes them again for the next, beside a group that keeps all."""
    from test_engine_gpu import plain_windowed_logits, windowed_model

    which = "cd"[seed % 2]
    cfg = TINY[which][0]
    layers = cfg["num_hidden_layers"]
    windows = [[40, 0], [0, 33], [70, 70]][seed % 3]
    windows = (windows * layers)[:layers]
    model = windowed_model(tiny_folders[which], dtype, windows)
    run_batches(random.Random(2000 + seed), lambda need: model.new_engine(max_tokens=need, max_slots=5),
                lambda r: plain_windowed_logits(oracles[which], r, windows), cfg["vocab_size"],
                cfg["max_position_embeddings"], dtype, f"seed {seed} model {which} windows {windows}")


@pytest.mark.parametrize("seed", range(4))
def test_random_requests_through_generate_with_stop_tokens_and_small_batches(models, oracles, seed, monkeypatch):
    """More requests than a batch holds, of unequal lengths, greedy; two stop tokens chosen so that some requests
    end early (the tokens that the plain implementation emits third for one request and sixth for another).  Each
    request's tokens equal the plain loop's, whatever batch it fell into."""
    from fms_b200.utils.generation import generate

    rng = random.Random(3000 + seed)
    which = "bcde"[seed % 4]
    cfg = TINY[which][0]
    top = min(cfg["max_position_embeddings"], 200) - 12
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.choice([1, 2, rng.randint(3, top)]))]
               for _ in range(rng.randint(3, 7))]
    free = [pl.plain_generate(oracles[which], p, 10) for p in prompts]
    stop = [free[0][len(prompts[0]) + 2], free[1][len(prompts[1]) + 5]]
    want = [pl.plain_generate(oracles[which], p, 10, eos=stop) for p in prompts]
    assert any(len(w) < len(p) + 10 for w, p in zip(want, prompts))  # some do end early
    model = models(which, "fp32")
    for batch_size in (None, rng.randint(1, 3)):
        out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=10, do_sample=False, eos_token_id=stop,
                       batch_size=batch_size)
        assert [o.tolist() for o in out] == want
    # the prompts of a batch in several steps, a few sequences at a time: the same tokens
    from fms_b200.engine import generation

    monkeypatch.setattr(generation, "PROMPT_TOKENS_PER_STEP", 60)
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=10, do_sample=False, eos_token_id=stop)
    assert [o.tolist() for o in out] == want
    engine = model.engine()
    assert engine.cache.slots.n_held == 0


def run_shrinking_batches(rng, engine, plain_logits, vocab, top, dtype, label):
    """Two batches of nine to twenty sequences: the prompts in one step, then one token each, the sequences leaving at
    random steps; every logit against ``plain_logits(request)``."""
    for batch_number in range(2):
        n = rng.randint(9, 20)
        requests = [[rng.randrange(vocab) for _ in range(rng.randint(2, top))] for _ in range(n)]
        prompt = [rng.randint(1, len(r) - 1) for r in requests]
        want = [plain_logits(r) for r in requests]
        largest = [w.abs().max().item() for w in want]
        slots = engine.begin(n)
        engine.step(slots, [r[:p] for r, p in zip(requests, prompt)], [[] for _ in requests])
        at = list(prompt)
        live = list(range(n))
        sizes = set()
        while live:
            logits = engine.step([slots[i] for i in live], [[requests[i][at[i]]] for i in live])
            sizes.add(len(live))
            for row, i in enumerate(live):
                close(logits[row], want[i][at[i]], largest[i], dtype, f"{label} batch {batch_number} request {i} "
                                                                     f"position {at[i]} among {len(live)}")
                at[i] += 1
            done = [i for i in live if at[i] == len(requests[i])]
            if done:
                engine.release([slots[i] for i in done])
                live = [i for i in live if i not in done]
        engine.check()
        assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups)
        assert max(sizes) > 8 and not set(engine._decode) - {1, 2, 3, 4, 5, 6, 7, 8, 12, 16, 24}


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("seed", range(4))
def test_random_batches_of_many_sequences_that_end_at_random_times(models, oracles, seed, dtype):
    """Nine to twenty sequences decode together and leave at random steps: their steps are filled up to 12, 16 or 24
    rows with rows in the cache's spare slot, and the live set changes under the captured graphs.  Two batches through
    the same engine; every logit against the plain implementation."""
    which = "bcde"[seed % 4]
    cfg = TINY[which][0]
    engine = models(which, dtype).new_engine(max_tokens=64 * 2 * 20, max_slots=20)
    run_shrinking_batches(random.Random(4000 + seed), engine, oracles[which].logits, cfg["vocab_size"],
                          min(cfg["max_position_embeddings"], 128), dtype, f"seed {seed} model {which}")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_many_sequences_that_end_at_random_times_with_windows_on_some_layers(tiny_folders, oracles, dtype):
    """The same where one layer keeps a window of 40 keys and the other all: the filler rows sit in the spare slot
    of both groups of the cache."""
    from test_engine_gpu import plain_windowed_logits, windowed_model

    cfg = TINY["d"][0]
    windows = [40, 0]
    engine = windowed_model(tiny_folders["d"], dtype, windows).new_engine(max_tokens=64 * 2 * 20, max_slots=20)
    assert len(engine.cache.groups) == 2
    run_shrinking_batches(random.Random(5000), engine, lambda r: plain_windowed_logits(oracles["d"], r, windows),
                          cfg["vocab_size"], 128, dtype, f"model d windows {windows}")
