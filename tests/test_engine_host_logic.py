"""The library's host logic on the CPU: loader, adapter, cache, batching and the step function, with the
CUDA kernels replaced by their plain restatements (tests/plain_ops.py).  Every way of cutting the work
must give the plain implementation's logits."""
import pytest
import torch

import plain_llama as pl
from plain_ops import use_plain_ops
from tiny_models import tiny_prompts


def _model(folder, dtype="fp32"):
    from fms_b200.models import get_model

    return get_model("llama", model_path=folder, source="hf", device_type="cpu", data_type=dtype)


@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_whole_prompts_alone(tiny_folders, which):
    oracle = pl.PlainLlama(tiny_folders[which])
    with use_plain_ops():
        model = _model(tiny_folders[which])
        engine = model.new_engine(max_tokens=512)
        for prompt in tiny_prompts(which):
            (slot,) = engine.begin(1)
            got = engine.step([slot], [prompt], [list(range(len(prompt)))])
            engine.release([slot])
            torch.testing.assert_close(got.double(), oracle.logits(prompt), atol=2e-5, rtol=1e-4)
        assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("which", ["a", "b"])
def test_unequal_batch_then_one_token_each(tiny_folders, which):
    oracle = pl.PlainLlama(tiny_folders[which])
    prompts = tiny_prompts(which)
    full = [p + [(7 * i + 3) % 200 for i in range(6)] for p in prompts]
    with use_plain_ops():
        model = _model(tiny_folders[which])
        engine = model.new_engine(max_tokens=64 * 2 * len(prompts))
        slots = engine.begin(len(prompts))
        got = {i: [] for i in range(len(prompts))}
        lg = engine.step(slots, prompts)  # last place of every prompt
        for i in range(len(prompts)):
            got[i].append(lg[i])
        for t in range(6):
            lg = engine.step(slots, [[f[len(p) + t]] for f, p in zip(full, prompts)])
            for i in range(len(prompts)):
                got[i].append(lg[i])
        engine.release(slots)
    for i, (f, p) in enumerate(zip(full, prompts)):
        want = oracle.logits(f)[len(p) - 1:]
        torch.testing.assert_close(torch.stack(got[i]).double(), want, atol=2e-5, rtol=1e-4)


def test_continuation_of_several_tokens_onto_a_cached_prefix(tiny_folders):
    """The reference needs an explicit mask here (fms/modules/attention.py:268-271); position-based
    causality does not."""
    oracle = pl.PlainLlama(tiny_folders["a"])
    prompt = tiny_prompts("a")[2]
    with use_plain_ops():
        engine = _model(tiny_folders["a"]).new_engine(max_tokens=128)
        (slot,) = engine.begin(1)
        a = engine.step([slot], [prompt[:7]], [list(range(7))])
        b = engine.step([slot], [prompt[7:12]], [list(range(5))])
        c = engine.step([slot], [prompt[12:]], [list(range(len(prompt) - 12))])
        engine.release([slot])
    torch.testing.assert_close(torch.cat([a, b, c]).double(), oracle.logits(prompt), atol=2e-5, rtol=1e-4)


def test_step_refuses_what_does_not_fit(tiny_folders):
    from fms_b200.cache import CacheFull

    with use_plain_ops():
        engine = _model(tiny_folders["a"]).new_engine(max_tokens=64, max_slots=2)
        (slot,) = engine.begin(1)
        with pytest.raises(ValueError, match="outside the vocabulary"):
            engine.step([slot], [[1, 256]])
        with pytest.raises(CacheFull):
            engine.step([slot], [[1] * 65])  # the model's 64 positions
        engine.step([slot], [[1] * 60])
        (other,) = engine.begin(1)
        with pytest.raises(CacheFull):
            engine.step([other], [[1, 2]])  # the only block is held
        assert engine.length(other) == 0
        with pytest.raises(ValueError, match="twice"):
            engine.step([slot, slot], [[1], [2]])
        engine.release([slot, other])
        with pytest.raises(ValueError, match="not held"):
            engine.step([slot], [[1]])


def test_model_called_on_whole_sequences(tiny_folders):
    """model(x), the reference's forward without a cache (fms/models/llama.py:425-450): a sequence, a rectangle with
    last_n_tokens, sequences of unequal lengths; the engine it makes for itself grows when it has to and holds
    nothing afterwards."""
    oracle = pl.PlainLlama(tiny_folders["a"])
    prompts = tiny_prompts("a")
    with use_plain_ops():
        model = _model(tiny_folders["a"])
        one = model(torch.tensor(prompts[0]))
        torch.testing.assert_close(one.double(), oracle.logits(prompts[0]), atol=2e-5, rtol=1e-4)
        rect = model(torch.tensor([prompts[1], prompts[1][::-1]]), last_n_tokens=3)
        assert rect.shape == (2, 3, one.shape[-1])
        torch.testing.assert_close(rect[1].double(), oracle.logits(prompts[1][::-1])[-3:], atol=2e-5, rtol=1e-4)
        ragged = model(prompts)  # more sequences and tokens than the first call's engine had room for
        for got, p in zip(ragged, prompts):
            torch.testing.assert_close(got.double(), oracle.logits(p), atol=2e-5, rtol=1e-4)
        engine = model.engine()
        assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups)
        with pytest.raises(NotImplementedError):
            model(torch.tensor(prompts[0]), use_cache=True)
        with pytest.raises(ValueError):
            model([[]])


def test_a_sequence_that_starts_at_another_position(tiny_folders):
    """Tiny E has the llama3 rescaling, so not even the rotation is a plain function of position differences in float32
    rounding; the logits must be the plain implementation's with the same first position, prompt and single tokens."""
    oracle = pl.PlainLlama(tiny_folders["e"])
    prompt = tiny_prompts("e")[1]
    with use_plain_ops():
        engine = _model(tiny_folders["e"]).new_engine(max_tokens=256)
        slots = engine.begin(2, first_positions=[0, 77])
        got = [engine.step(slots, [prompt[:30], prompt[:30]], [list(range(30))] * 2)]
        for t in range(30, len(prompt)):
            got.append(engine.step(slots, [[prompt[t]], [prompt[t]]]))
        engine.release(slots)
    rows = torch.cat([got[0].view(2, 30, -1)] + [g.view(2, 1, -1) for g in got[1:]], 1).double()
    torch.testing.assert_close(rows[0], oracle.logits(prompt), atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(rows[1], oracle.logits(prompt, first_position=77), atol=2e-5, rtol=1e-4)


def test_generate_honours_the_offset_of_padded_position_ids(tiny_folders):
    """``pad_input_ids(..., position_ids_offset=k)`` makes every prompt start at position k
    (fms/utils/generation.py:16-109); the engine starts the sequences there."""
    from fms_b200.utils.generation import generate, pad_input_ids, trim_prefix

    oracle = pl.PlainLlama(tiny_folders["e"])
    prompts = [p for p in tiny_prompts("e")[:2]]
    with use_plain_ops():
        model = _model(tiny_folders["e"])
        ids, extra = pad_input_ids([torch.tensor(p) for p in prompts], position_ids_offset=9, pad_token_id=172)
        out = generate(model.new_engine(max_tokens=512), ids, max_new_tokens=4, do_sample=False, extra_kwargs=extra)
    for row, p in zip(out, prompts):
        got = row.tolist()[ids.shape[1] - len(p):]
        assert got == pl.plain_generate(oracle, p, 4, first_position=9)


def test_decode_steps_filled_up_to_a_captured_size_change_no_result(tiny_folders):
    """Eleven sequences decode as twelve rows, nine as twelve, then (two ended) seven as seven: the filler row lives in
    the cache's spare slot and its block; the live sequences' logits are those of the plain implementation, no block
    of the pool is taken for the filler, and the arrays on the device are brought anew when the live set changes."""
    from fms_b200.engine.step import decode_rows

    assert [decode_rows(n) for n in (1, 8, 9, 12, 13, 17, 33, 49, 64, 65, 100, 129)] == [1, 8, 12, 12, 16, 24, 48, 64, 64, 96, 128, 192]
    oracle = pl.PlainLlama(tiny_folders["b"])
    g = torch.Generator().manual_seed(4)
    reqs = [torch.randint(0, 384, (int(k) + 8,), generator=g).tolist() for k in torch.randint(1, 40, (11,), generator=g)]
    with use_plain_ops():
        engine = _model(tiny_folders["b"]).new_engine(max_tokens=64 * 11, max_slots=11)
        engine.fill_rows = True  # as on a GPU, where a size means a captured graph
        slots = engine.begin(11)
        engine.step(slots, [r[:-8] for r in reqs])
        live = list(range(11))
        got = {i: [] for i in live}
        for t in range(8):
            if t == 3:
                engine.release([slots[2], slots[9]])
                live = [i for i in live if i not in (2, 9)]
            if t == 6:
                engine.release([slots[0], slots[5]])
                live = [i for i in live if i not in (0, 5)]
            lg = engine.decode([slots[i] for i in live], [reqs[i][len(reqs[i]) - 8 + t] for i in live])
            assert lg.shape[0] == len(live)
            for row, i in enumerate(live):
                got[i].append(lg[row].clone())
            assert all(gr.pool.n_held == sum((engine.cache.length[slots[i]] + 63) // 64 for i in live)
                       for gr in engine.cache.groups)
        assert sorted(engine._decode) == [7, 12]
        engine.release([slots[i] for i in live])
        assert engine.cache.slots.n_held == 0 and all(gr.pool.n_held == 0 for gr in engine.cache.groups)
    for i, r in enumerate(reqs):
        want = oracle.logits(r)[len(r) - 8:][: len(got[i])]
        torch.testing.assert_close(torch.stack(got[i]).double(), want, atol=2e-5, rtol=1e-4)
