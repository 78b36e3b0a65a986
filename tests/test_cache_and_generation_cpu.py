"""The cache's bookkeeping (no slot or block lost, held twice or freed twice), the generation loop's
decisions on a fake engine, the tokenizer and the command line's parser — all on the CPU."""
import random

import pytest
import torch


# ---- slots and blocks ---------------------------------------------------------------------------------
def test_slot_allocator_never_loses_or_doubles():
    from fms_b200.cache import CacheFull, SlotAllocator

    a = SlotAllocator(5)
    got = [a.alloc() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4] and a.n_free == 0
    with pytest.raises(CacheFull):
        a.alloc()
    a.free(3)
    with pytest.raises(ValueError):
        a.free(3)  # freed twice
    with pytest.raises(ValueError):
        a.free(7)  # never existed
    assert a.alloc() == 3  # used again
    rng = random.Random(0)
    held = set(got)
    for _ in range(2000):
        if held and rng.random() < 0.5:
            s = rng.choice(sorted(held))
            a.free(s)
            held.discard(s)
        elif a.n_free:
            s = a.alloc()
            assert s not in held  # never held twice
            held.add(s)
        assert a.n_held == len(held) and a.n_free + a.n_held == 5


def test_block_pool_never_loses_or_doubles():
    from fms_b200.cache import BlockPool, CacheFull

    p = BlockPool(10)
    a = p.alloc(4)
    b = p.alloc(6)
    assert sorted(a + b) == list(range(10))
    with pytest.raises(CacheFull):
        p.alloc(1)
    p.free(a)
    with pytest.raises(ValueError):
        p.free([a[0]])
    assert p.n_free == 4 and p.n_held == 6
    with pytest.raises(CacheFull):
        p.alloc(5)  # refused whole: nothing is taken
    assert p.n_free == 4
    assert sorted(p.alloc(4)) == sorted(a)


def test_cache_lengths_blocks_groups_and_reuse():
    from fms_b200.cache import Cache, CacheFull, KVRequest, StateRequest

    reqs = [KVRequest(2, 16), KVRequest(2, 16), KVRequest(2, 16, window=70), None, StateRequest((3, 4), torch.float32)]
    c = Cache(reqs, max_tokens=64 * 6, max_positions=512, dtype=torch.float32, device="cpu", max_slots=3)
    assert len(c.groups) == 3  # layers 0 and 1 share a group; the windowed layer and the state have their own
    full, win, state = c.groups
    assert full.layers == [0, 1] and win.layers == [2] and state.layers == [4]
    # one block and one slot more than are handed out: the spare slot with its block, for a step's filler rows
    assert full.storage.shape == (2, 2, 7, 2, 64, 16) and state.storage.shape == (1, 4, 3, 4)
    assert c.layer_view(3) is None and c.layer_view(0).keys.shape == (7, 2, 64, 16)
    assert c.spare_slot == 3 and full.table_host[3].tolist()[:2] == [6, -1] and full.pool.n_blocks == 6
    s0, s1 = c.begin(2)
    state.storage[0, s0] = 1.0
    assert c.prepare([s0, s1], [100, 5]) == [0, 0]
    c.commit([s0, s1], [100, 5])
    assert (c.length[s0], c.length[s1]) == (100, 5)
    assert full.pool.n_held == 3 and len(full.held_blocks(s0)) == 2
    # the device table says where each position lies; unheld entries are -1
    assert full.table[s0, :2].tolist() == full.held_blocks(s0) and full.table[s0, 2].item() == -1
    for _ in range(100):
        c.prepare_decode([s0, s1])
        c.commit([s0, s1], [1, 1])
    assert c.length[s0] == 200 and len(full.held_blocks(s0)) == 4
    # the window of 70 keeps positions 130..199: blocks 2 and 3 only; earlier ones went back to the pool
    assert win.table_host[s0].tolist()[:5] == [-1, -1] + win.held_blocks(s0) + [-1]
    assert len(win.held_blocks(s0)) == 2
    # a step that does not fit is refused before anything is taken
    held = full.pool.n_held
    with pytest.raises(CacheFull):
        c.prepare([s1], [64 * 3])
    assert full.pool.n_held == held and c.length[s1] == 105
    with pytest.raises(CacheFull):
        c.prepare([s0], [400])  # beyond the model's positions
    c.release([s0])
    with pytest.raises(ValueError):
        c.release([s0])
    assert full.pool.n_held == 2 and full.table_host[s0].max().item() == -1
    (again,) = c.begin(1)
    assert again == s0 and c.length[again] == 0
    assert state.storage[0, again].abs().sum().item() == 0  # state starts at zero for the new sequence
    c.release([again, s1])
    assert c.slots.n_held == 0 and full.pool.n_held == 0 and win.pool.n_held == 0
    with pytest.raises(CacheFull):
        c.begin(4)


def test_cache_random_walk_keeps_its_books():
    from fms_b200.cache import Cache, CacheFull, KVRequest

    c = Cache([KVRequest(1, 16), KVRequest(1, 16, window=100)], max_tokens=64 * 12, max_positions=640,
              dtype=torch.float32, device="cpu", max_slots=4)
    rng = random.Random(1)
    live = {}
    for _ in range(600):
        r = rng.random()
        try:
            if r < 0.15 and c.slots.n_free:
                (s,) = c.begin(1)
                assert s not in live
                live[s] = 0
            elif r < 0.25 and live:
                s = rng.choice(sorted(live))
                c.release([s])
                del live[s]
            elif live:
                s = rng.choice(sorted(live))
                n = rng.choice([1, 1, 1, 7, 64, 130])
                c.prepare([s], [n])
                c.commit([s], [n])
                live[s] += n
        except CacheFull:
            pass
        for g in c.groups:
            owned = [b for s in range(4) for b in g.held_blocks(s)]
            assert len(owned) == len(set(owned)) == g.pool.n_held  # no block held twice, none lost
            assert g.pool.n_held + g.pool.n_free == g.pool.n_blocks
        for s, n in live.items():
            assert c.length[s] == n
            full = c.groups[0]
            assert len(full.held_blocks(s)) == (n + 63) // 64
        assert c.slots.n_held == len(live)


# ---- the generation loop on a fake engine --------------------------------------------------------------
class CountingEngine:
    """next token = (last token + 1) % vocab, as the reference's ModelMock (tests/utils/test_generate.py:15-30);
    keeps the books of slots so that the loop's decisions can be checked."""

    def __init__(self, vocab=20, max_slots=3):
        self.vocab, self.device = vocab, torch.device("cpu")
        self.free = list(range(max_slots))
        self.last = {}
        self.steps = []  # (kind, number of sequences)
        self.released = []

    def begin(self, n, first_positions=None):
        assert n <= len(self.free)
        self.first_positions = first_positions
        out = [self.free.pop(0) for _ in range(n)]
        return out

    def release(self, slots):
        for s in slots:
            assert s not in self.free
            self.free.append(s)
            self.released.append(s)

    def _logits(self, slots):
        lg = torch.zeros(len(slots), self.vocab)
        for i, s in enumerate(slots):
            lg[i, (self.last[s] + 1) % self.vocab] = 5.0
        return lg

    def step(self, slots, tokens, want=None):
        self.steps.append(("step", len(slots), [len(t) for t in tokens]))
        for s, t in zip(slots, tokens):
            self.last[s] = t[-1]
        return self._logits(slots)

    def decode(self, slots, tokens, horizon=0):
        self.steps.append(("decode", len(slots), horizon))
        for s, t in zip(slots, tokens):
            self.last[s] = t
        return self._logits(slots)


@pytest.fixture
def greedy_on_cpu(monkeypatch):
    from fms_b200.kernels import ops

    monkeypatch.setattr(ops, "argmax", lambda logits, out=None: torch.argmax(logits, -1).to(torch.int32))


def test_generate_stops_each_sequence_at_its_stop_token(greedy_on_cpu):
    from fms_b200.utils.generation import generate

    e = CountingEngine()
    out = generate(e, [[5], [1, 2], [9, 6]], max_new_tokens=8, do_sample=False, eos_token_id=7)
    assert [o.tolist() for o in out] == [[5, 6, 7], [1, 2, 3, 4, 5, 6, 7], [9, 6, 7]]
    # the prompts in one step, then one token each; the batch shrinks as sequences end (the reference would
    # end everything at the first stop token, fms/utils/generation.py:338-341)
    assert e.steps[0] == ("step", 3, [1, 2, 2])
    assert [s[:2] for s in e.steps[1:]] == [("decode", 2), ("decode", 1), ("decode", 1), ("decode", 1)]
    assert all(s[2] == 2 + 8 for s in e.steps[1:])  # the horizon: longest prompt + max_new_tokens
    assert sorted(e.released) == [0, 1, 2] and sorted(e.free) == [0, 1, 2]  # every slot given back once


def test_generate_runs_batches_one_after_another_and_keeps_the_order(greedy_on_cpu):
    from fms_b200.utils.generation import generate

    e = CountingEngine(max_slots=2)
    prompts = [[i] for i in range(5)]
    out = generate(e, prompts, max_new_tokens=3, do_sample=False, batch_size=2)
    assert [o.tolist() for o in out] == [[i, i + 1, i + 2, i + 3] for i in range(5)]
    assert [s[1] for s in e.steps if s[0] == "step"] == [2, 2, 1]  # three batches
    assert len(e.released) == 5 and sorted(e.free) == [0, 1]  # slots were used again
    # a 1-D prompt gives a 1-D result; a rectangle gives a rectangle, padded after early stops
    assert generate(e, torch.tensor([3]), max_new_tokens=2, do_sample=False).tolist() == [3, 4, 5]
    rect = generate(e, torch.tensor([[3], [5]]), max_new_tokens=4, do_sample=False, eos_token_id=7, pad_token_id=0)
    assert rect.tolist() == [[3, 4, 5, 6, 7], [5, 6, 7, 0, 0]]


def test_prompts_of_many_tokens_run_a_few_sequences_at_a_time(greedy_on_cpu, monkeypatch):
    """A batch's prompts go through one step up to a number of tokens; beyond it, consecutive sequences are packed
    into steps of at most that many (a longer prompt alone), and the tokens are the same."""
    from fms_b200.engine import generation
    from fms_b200.utils.generation import generate

    assert generation.prompt_groups([5, 5, 5], 100) == [[0, 1, 2]]
    assert generation.prompt_groups([5, 5, 5], 10) == [[0, 1], [2]]
    assert generation.prompt_groups([50, 5, 5, 7], 10) == [[0], [1, 2], [3]]
    prompts = [[1] * 6, [2] * 3, [3] * 3, [4] * 9, [5]]
    whole = generate(CountingEngine(max_slots=5), prompts, max_new_tokens=3, do_sample=False)
    monkeypatch.setattr(generation, "PROMPT_TOKENS_PER_STEP", 8)
    e = CountingEngine(max_slots=5)
    cut = generate(e, prompts, max_new_tokens=3, do_sample=False)
    assert [o.tolist() for o in cut] == [o.tolist() for o in whole]
    assert [s[2] for s in e.steps if s[0] == "step"] == [[6], [3, 3], [9], [1]]
    assert [s[:2] for s in e.steps if s[0] == "decode"] == [("decode", 5)] * 2


def test_generate_argument_checks_and_release_on_error(greedy_on_cpu):
    from fms_b200.utils.generation import generate

    e = CountingEngine()
    with pytest.raises(NotImplementedError):
        generate(e, [[1]], num_beams=2)
    with pytest.raises(ValueError):
        generate(e, [[]])
    with pytest.raises(ValueError):
        generate(e, [[1]], timing="sometimes")
    with pytest.raises(ValueError):
        generate(e, [[1]], do_sample=True, temperature=0.0)
    # the reference's remaining parameters are accepted where they mean nothing here and refused where they would
    assert generate(e, [[1]], max_new_tokens=1, do_sample=False, contiguous_cache=True, extra_kwargs={})[0].tolist() == [1, 2]
    with pytest.raises(NotImplementedError):
        generate(e, [[1]], prepare_model_inputs_hook=lambda *a: a)
    with pytest.raises(NotImplementedError):
        generate(e, [[1]], extra_kwargs={"attn_name": "sdpa_causal"})

    def boom(*a, **k):
        raise RuntimeError("hook failed")

    with pytest.raises(RuntimeError):
        generate(e, [[1], [2]], max_new_tokens=3, do_sample=False, post_iteration_hook=boom)
    assert sorted(e.free) == [0, 1, 2]  # the slots came back although the loop ended in an error
    out, times = generate(e, [[1]], max_new_tokens=3, do_sample=False, timing="per-token")
    assert len(times) == 3 and out[0].tolist() == [1, 2, 3, 4]
    out, times = generate(e, [[1, 2, 3, 4]], max_new_tokens=2, do_sample=False, timing="e2e", max_seq_len=2)
    assert len(times) == 1 and out[0].tolist() == [3, 4, 5, 6]  # the prompt was cut to its last 2 tokens


def test_padded_rectangle_runs_without_its_padding_and_comes_back_with_it(greedy_on_cpu):
    """The reference's way with unequal prompts (fms/utils/generation.py:16-109, scripts/inference.py:205-218):
    pad_input_ids, then generate with what it returned as extra_kwargs."""
    from fms_b200.utils.generation import generate, pad_input_ids, trim_prefix, truncate_after_eos

    prompts = [torch.tensor([4]), torch.tensor([1, 2, 3]), torch.tensor([9, 10])]
    ids, extra = pad_input_ids(prompts, min_pad_length=5)
    assert ids.tolist() == [[0, 0, 0, 0, 4], [0, 0, 1, 2, 3], [0, 0, 0, 9, 10]]
    assert extra["position_ids"].tolist() == [[0, 0, 0, 0, 0], [0, 0, 0, 1, 2], [0, 0, 0, 0, 1]]
    m = extra["mask"]
    assert m.shape == (3, 5, 5) and m.dtype == torch.float32
    # row 1: its tokens (places 2..4) look at tokens up to themselves, its padding at padding up to itself
    assert (m[1] == 0).tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                                    [False, False, True, False, False], [False, False, True, True, False],
                                    [False, False, True, True, True]]
    assert torch.isinf(m[1][~(m[1] == 0)]).all()

    e = CountingEngine()
    out = generate(e, ids, max_new_tokens=4, do_sample=False, eos_token_id=12, extra_kwargs=extra)
    assert e.steps[0] == ("step", 3, [1, 3, 2])  # only the tokens ran: padding can change no result
    assert out.tolist() == [[0, 0, 0, 0, 4, 5, 6, 7, 8], [0, 0, 1, 2, 3, 4, 5, 6, 7], [0, 0, 0, 9, 10, 11, 12, 12, 12]]
    assert truncate_after_eos(trim_prefix(out[2]), 12).tolist() == [9, 10, 11, 12]
    # the same tokens as from the list of prompts
    plain = generate(CountingEngine(), prompts, max_new_tokens=4, do_sample=False, eos_token_id=12)
    assert [trim_prefix(r).tolist()[:len(p)] for r, p in zip(out, plain)] == [p.tolist() for p in plain]

    # padding on the right, an offset, another pad token
    ids, extra = pad_input_ids(prompts, padding_side="right", position_ids_offset=2, pad_token_id=7, is_causal_mask=False)
    assert ids.tolist() == [[4, 7, 7], [1, 2, 3], [9, 10, 7]]
    assert extra["position_ids"].tolist() == [[2, 2, 2], [2, 3, 4], [2, 3, 2]]
    assert (extra["mask"][2] == 0).tolist() == [[True, True, False], [True, True, False], [False, False, True]]
    e = CountingEngine()
    out = generate(e, ids[1:], max_new_tokens=2, do_sample=False, extra_kwargs={k: v[1:] for k, v in extra.items()})
    assert out.tolist() == [[1, 2, 3, 4, 5], [9, 10, 7, 11, 12]]
    assert e.first_positions == [2, 2]  # the sequences start at the offset

    with pytest.raises(ValueError):  # the mapping belongs to the rectangle it was made with
        generate(CountingEngine(), prompts, max_new_tokens=1, do_sample=False, extra_kwargs=extra)
    with pytest.raises(ValueError):
        generate(CountingEngine(), ids, max_new_tokens=1, do_sample=False,
                 extra_kwargs={"position_ids": torch.tensor([[0, 5, 1], [0, 1, 2], [0, 1, 0]])})


def test_plan_batches_respects_cache_and_slots():
    from fms_b200.utils.generation import plan_batches

    # each request needs ceil((len + new) / 64) blocks of the cache
    assert plan_batches([10, 10, 10], 10, None, 64 * 3, 8) == [[0, 1, 2]]
    assert plan_batches([10, 60, 10], 30, None, 64 * 3, 8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, 10, 2, 64 * 100, 8) == [[0, 1], [2, 3], [4]]
    assert plan_batches([10] * 5, 10, None, 64 * 100, 3) == [[0, 1, 2], [3, 4]]
    with pytest.raises(ValueError):
        plan_batches([200], 10, None, 128, 8)


def test_helpers_and_tokenizer_and_parser():
    from fms_b200.cli.inference import build_parser
    from fms_b200.utils.generation import trim_prefix, truncate_after_eos
    from fms_b200.utils.tokenizers import CharTokenizer, get_tokenizer

    assert truncate_after_eos(torch.tensor([5, 6, 3, 9, 3]), 3).tolist() == [5, 6, 3]
    assert truncate_after_eos(torch.tensor([5, 6]), 3).tolist() == [5, 6]
    assert trim_prefix(torch.tensor([0, 0, 4, 0, 5]), 0).tolist() == [4, 0, 5]
    t = get_tokenizer("char_tokenizer")
    assert isinstance(t, CharTokenizer) and t.vocab_size() == 256 and (t.bos_token_id, t.eos_token_id) == (2, 3)
    ids = t.encode("héllo", add_special_tokens=True)
    assert ids == [2, 104, 233, 108, 108, 111] and t.decode(ids + [3]) == "héllo"
    # the older calls that the reference's scripts use (scripts/inference.py:178-186, :232-236)
    tokens = t.tokenize("héllo")
    assert tokens == list("héllo") and t.convert_tokens_to_ids(tokens) == ids[1:] and t.convert_tokens_to_ids("h") == 104
    assert t.convert_tokens_to_ids(["ab", "\u4e2d"]) == [0, 0]  # what is no single character below 256 becomes 0
    assert t.convert_tokens_to_string(t.convert_ids_to_tokens(torch.tensor(ids[1:]))) == "héllo"
    with pytest.raises(ValueError):
        get_tokenizer("/no/such/tokenizer")
    args = build_parser().parse_args(["--variant", "micro", "--prompt", "a", "--prompt", "b", "--batch_input",
                                      "--default_dtype", "fp32", "--max_new_tokens", "7"])
    assert args.prompt == ["a", "b"] and args.batch_input and args.default_dtype == "fp32" and args.max_new_tokens == 7
    assert args.device_type == "cuda" and args.architecture == "llama" and args.top_k == 10 and args.min_pad_length == 0


def test_tokenizer_json_folder(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    from fms_b200.utils.tokenizers import JsonTokenizer, get_tokenizer

    vocab = {"<s>": 0, "</s>": 1, "<unk>": 2, "a": 3, "cat": 4, "sat": 5}
    tok = tokenizers.Tokenizer(WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(tmp_path / "tokenizer.json"))
    t = get_tokenizer(str(tmp_path))
    assert isinstance(t, JsonTokenizer) and t.vocab_size() == 6 and (t.bos_token_id, t.eos_token_id) == (0, 1)
    assert t.encode("a cat sat") == [3, 4, 5] and t.encode("a dog", add_special_tokens=True) == [0, 3, 2]
    assert t.tokenize("cat sat") == ["cat", "sat"] and t.convert_tokens_to_ids(["cat", "sat"]) == [4, 5]
    assert t.convert_ids_to_tokens([5, 3]) == ["sat", "a"] and t.convert_tokens_to_ids("a") == 3
    assert t.decode([3, 4]).split() == ["a", "cat"]


def test_sampler_arguments():
    from fms_b200.sampling import Sampler

    with pytest.raises(ValueError):
        Sampler(do_sample=True, temperature=0.0)
    with pytest.raises(ValueError):
        Sampler(do_sample=True, top_k=-1)
    Sampler(do_sample=False, temperature=0.0)  # greedy ignores the temperature


def test_bench_says_that_it_measures_one_gpu_only():
    """For more than one GPU bench.py prints one line that says so and exits with 2 (no GPU is needed for that)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 2
    lines = [line for line in r.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_bench_counts_the_bytes_and_flops_of_its_shapes():
    """The denominators of the roofline figures: what a decode step has to read (every weight once, and the
    cache of the live tokens) and what a prefill has to compute, for the benchmark's three shapes."""
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    want = {  # GB of weights a step, bytes of cache a token, TFLOP of a 2,048-token prefill
        "llama-3-8b": (15.01, 131072, 29.69), "llama-2-7b": (13.21, 524288, 27.63), "llama-2-13b": (25.70, 819200, 53.69)}
    for name, (gb, per_token, tflop) in want.items():
        bench.choose_model(name)
        layers = bench.MODEL["nlayers"]
        assert abs(bench.decode_bytes(layers, 0) / 1e9 - gb) < 0.01
        assert bench.decode_bytes(layers, 1) - bench.decode_bytes(layers, 0) == per_token
        assert abs(bench.prefill_flops(layers, 2048) / 1e12 - tflop) < 0.01
        assert (bench.PROMPT_MIN, bench.PROMPT_MAX) == bench.MODEL["prompts"]
    bench.choose_model("llama-3-8b")


def test_a_window_group_with_a_full_pool_takes_a_step_that_frees_as_much_as_it_needs():
    """Two sequences in a pool without a free block: the step needs a new block for each, and gives one back for each
    (it has left the window).  Everything that is given back is given back before anything is taken."""
    from fms_b200.cache import Cache, CacheFull, KVRequest

    cache = Cache([KVRequest(1, 16, window=64)], max_tokens=64 * 4, max_positions=1024, dtype=torch.float32, device="cpu",
                  max_slots=2)
    a, b = cache.begin(2)
    cache.prepare([a, b], [128, 128])
    cache.commit([a, b], [128, 128])
    pool = cache.groups[0].pool
    assert pool.n_free == 0
    # position 128 sees keys 65..128: block 0 (0..63) has left the window, block 2 is needed
    cache.prepare([a, b], [1, 1])
    cache.commit([a, b], [1, 1])
    assert pool.n_free == 0 and all(len(cache.groups[0].held_blocks(s)) == 2 for s in (a, b))
    # a step that does not fit raises before anything is taken or given back
    held = [cache.groups[0].held_blocks(s) for s in (a, b)]
    with pytest.raises(CacheFull):
        cache.prepare([a, b], [64, 64])  # keeps blocks 1.. of each (the first query still sees them) and needs one more each
    assert [cache.groups[0].held_blocks(s) for s in (a, b)] == held and pool.n_free == 0
    cache.release([a, b])
    assert pool.n_held == 0


def test_sequences_that_start_at_other_positions_keep_length_and_position_apart():
    from fms_b200.cache import Cache, CacheFull, KVRequest

    cache = Cache([KVRequest(1, 16)], max_tokens=256, max_positions=100, dtype=torch.float32, device="cpu")
    a, b = cache.begin(2, [0, 40])
    cache.prepare([a, b], [10, 10])
    cache.commit([a, b], [10, 10])
    assert (cache.length[a], cache.position[a], cache.offset(a)) == (10, 10, 0)
    assert (cache.length[b], cache.position[b], cache.offset(b)) == (10, 50, 40)
    with pytest.raises(CacheFull, match="positions"):
        cache.prepare([b], [51])  # position 50 + 51 exceeds the model's 100 positions although the cache has room
    cache.prepare([b], [50])
    cache.release([a, b])
    (c,) = cache.begin(1)
    assert cache.offset(c) == 0  # nothing of the old offset is left in a slot that is used again
    with pytest.raises(ValueError):
        cache.begin(1, [-1])


def test_sentencepiece_model_file(tmp_path):
    sentencepiece = pytest.importorskip("sentencepiece")
    from fms_b200.utils.tokenizers import get_tokenizer

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog", "a small whole engine for one gpu",
                                 "keys and values in blocks of sixty four tokens"] * 20))
    sentencepiece.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "tokenizer"), vocab_size=60,
                                             model_type="bpe", bos_id=1, eos_id=2, unk_id=0)
    for where in (str(tmp_path / "tokenizer.model"), str(tmp_path)):
        tok = get_tokenizer(where)
        assert (tok.bos_token_id, tok.eos_token_id) == (1, 2) and tok.vocab_size() == 60
        ids = tok.encode("the lazy fox", add_special_tokens=True)
        assert ids[0] == 1 and tok.decode(ids[1:]) == "the lazy fox"
        pieces = tok.tokenize("the lazy fox")
        assert tok.convert_tokens_to_ids(pieces) == ids[1:] and tok.convert_tokens_to_string(pieces) == "the lazy fox"
        assert tok.convert_ids_to_tokens(ids[1:]) == pieces
