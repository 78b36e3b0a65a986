"""The plain implementation against the stored outputs of the reference's own model code
(tests/golden/make_golden.py), and its parts against hand calculations."""
import math
import os

import pytest
import torch

import plain_llama as pl
from tiny_models import TINY, tiny_prompts, tiny_tensors_of

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_logits.safetensors")


@pytest.fixture(scope="module")
def golden():
    from safetensors.torch import load_file

    return load_file(GOLDEN)


def test_pad_input_ids_returns_what_the_reference_returns():
    """Not the plain implementation but the library's own helper: it has the reference's signature, so it
    is held against the reference's stored results (tests/golden/make_golden.py, PADDING_CASES)."""
    import importlib.util
    from safetensors.torch import load_file

    from fms_b200.utils.generation import pad_input_ids

    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(GOLDEN), "make_golden.py"))
    made = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(made)
    stored = load_file(os.path.join(os.path.dirname(GOLDEN), "reference_padding.safetensors"))
    for name, kwargs in made.PADDING_CASES.items():
        ids, extra = pad_input_ids([torch.tensor(p) for p in made.PADDING_PROMPTS], **kwargs)
        assert ids.dtype == torch.long and extra["position_ids"].dtype == torch.long
        assert torch.equal(ids.to(torch.int32), stored[f"{name}.ids"]), name
        assert torch.equal(extra["position_ids"].to(torch.int32), stored[f"{name}.position_ids"]), name
        zero = extra["mask"] == 0
        assert torch.equal(zero.to(torch.uint8), stored[f"{name}.mask_is_zero"]), name
        assert torch.isinf(extra["mask"][~zero]).all() and (extra["mask"][~zero] < 0).all()


@pytest.mark.parametrize("which", sorted(TINY))
def test_weights_are_the_ones_the_golden_was_made_with(golden, which):
    tensors = tiny_tensors_of(which)
    total = torch.stack([t.float().abs().sum() for _, t in sorted(tensors.items())]).sum().double()
    assert abs(total.item() - golden[f"{which}.weight_abs_sum"].item()) < 1e-6 * total.item()


@pytest.mark.parametrize("which", sorted(TINY))
def test_plain_logits_equal_reference(golden, tiny_folders, which):
    model = pl.PlainLlama(tiny_folders[which], dtype=torch.float64)
    for n, prompt in enumerate(tiny_prompts(which)):
        assert golden[f"{which}.{n}.ids"].tolist() == prompt
        sel = golden[f"{which}.{n}.positions"].long()
        ours = model.logits(prompt)[sel]
        ref = golden[f"{which}.{n}.logits"].double()
        # the reference ran in float32: its own rounding is the only difference
        torch.testing.assert_close(ours, ref, atol=2e-5, rtol=1e-4)


def test_rope_rotates_adjacent_pairs():
    inv = pl.plain_rope_inv_freq(8, 10000.0)
    assert torch.allclose(inv, 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8)))
    x = torch.randn(5, 1, 8, dtype=torch.float64)
    out = pl.plain_rope(x, torch.arange(5), inv)
    for p in range(5):
        for i in range(4):
            a = float(torch.tensor(float(p)) * inv[i])
            c, s = math.cos(a), math.sin(a)
            assert abs(out[p, 0, 2 * i] - (c * x[p, 0, 2 * i] - s * x[p, 0, 2 * i + 1])) < 1e-6
            assert abs(out[p, 0, 2 * i + 1] - (s * x[p, 0, 2 * i] + c * x[p, 0, 2 * i + 1])) < 1e-6


def test_attention_window_and_groups():
    torch.manual_seed(0)
    q = torch.randn(6, 4, 8, dtype=torch.float64)
    k = torch.randn(6, 2, 8, dtype=torch.float64)
    v = torch.randn(6, 2, 8, dtype=torch.float64)
    full = pl.plain_attention(q, k, v)
    # position 0 sees only key 0
    assert torch.allclose(full[0, 3], v[0, 1])
    # a window of 1 sees only the own key everywhere
    w1 = pl.plain_attention(q, k, v, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0]) and torch.allclose(w1[:, 2], v[:, 1])
    # a window as long as the sequence changes nothing
    assert torch.allclose(pl.plain_attention(q, k, v, window=6), full)
    # by hand for one head, one position, window 3
    p, h = 5, 1
    s = (k[3:6, 0] @ q[p, h]) / math.sqrt(8)
    expect = torch.softmax(s, 0) @ v[3:6, 0]
    assert torch.allclose(pl.plain_attention(q, k, v, window=3)[p, h], expect)


def test_rmsnorm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    g = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = pl.plain_rmsnorm(x, g, 0.5)
    r = 1.0 / math.sqrt((9 + 16) / 2 + 0.5)
    assert torch.allclose(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))
    wg = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    wu = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[2.0], [1.0]], dtype=torch.float64)
    out = pl.plain_swiglu_ffn(x, wg, wu, wd)
    m = 3.0 / (1 + math.exp(-3.0)) * 4.0
    assert torch.allclose(out, torch.tensor([[2 * m, m]], dtype=torch.float64))


def test_sampling_rules():
    lg = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert pl.plain_greedy(lg) == 1  # lowest index among equals
    # top_k = 1 is greedy whatever the draw
    assert pl.plain_sample(lg, 0.7, 1, 0.0) in (1, 2)
    # inverse CDF: u just below the first probability picks index 0
    p = torch.softmax(lg.double() / 0.5, 0)
    assert pl.plain_sample(lg, 0.5, 0, float(p[0]) * 0.999) == 0
    assert pl.plain_sample(lg, 0.5, 0, float(p[0]) * 1.001) == 1
    assert pl.plain_sample(lg, 0.5, 0, 0.999999) == 3
    u = [pl.plain_uniform(7, r, s) for r in range(4) for s in range(50)]
    assert all(0.0 <= x < 1.0 for x in u) and len(set(u)) > 190
    assert 0.35 < sum(u) / len(u) < 0.65


def test_llama3_rope_scaling_formula():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    base = pl.plain_rope_inv_freq(128, 500000.0)
    scaled = pl.plain_rope_inv_freq(128, 500000.0, sc)
    wavelen = 2 * math.pi / base
    assert torch.equal(scaled[wavelen < 8192 / 4.0], base[wavelen < 8192 / 4.0])
    assert torch.allclose(scaled[wavelen > 8192], base[wavelen > 8192] / 8.0)
