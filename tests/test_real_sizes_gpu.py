"""The engine at the real layer sizes against the plain implementation: two layers of the Llama-3-8B shape
(width 4,096, 32 query heads over 8 key/value heads, head size 128, feed-forward 14,336, vocabulary 128,256) and
two layers of the Llama-2-7B shape (32 key/value heads, feed-forward 11,008, vocabulary 32,000), random weights,
in float32 and in bfloat16.

At these sizes the step takes the kernels that the benchmark's numbers come from: the tcgen05 products and
the tcgen05 attention (a prompt of more than 1,024 tokens in one step), the weight-streaming product with the
rotation and cache write in its epilogue and the 128,256-row head (one token a step, also inside the captured
graph), and the products of 9 to 1,023 rows (a batch of sixteen, prompts of a few hundred tokens).

The oracle runs in float32 on the CPU (float64 would need 12 GB and twice the time); the reference's own
comparisons at model level are in true float32 too (fms/testing/comparison.py:88-102).  Its weights are
drawn on the GPU with torch's generator and written by the tests' own writer, so that the library's
random-weights mode is not part of what is compared.  With matrices ~ N(0, 0.02) at width 4,096 the
attention scores have a standard deviation of about 1.6: no near-uniform softmax hides a wrong key here.
"""
import json
import os

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu

SHAPES = {
    # config.json keys of two layers of the benchmark's shapes
    "llama3_8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=8192),
    "llama2_7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=32, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=4096),
}


def write_big_folder(path, cfg, seed):
    """config.json + model.safetensors with HF names; matrices ~ N(0, 0.02) in bfloat16, gains 1 + U(-0.1, 0.1)
    in float32, drawn on the GPU (a CPU generator needs minutes for 1.5e9 values)."""
    from safetensors.torch import save_file

    cfg = dict({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "tie_word_embeddings": False,
                "hidden_act": "silu", "attention_bias": False, "mlp_bias": False}, **cfg)
    g = torch.Generator(device="cuda").manual_seed(seed)
    d, h, kv, f, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                      cfg["intermediate_size"], cfg["vocab_size"])
    hd = d // h

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=g, device="cuda") * 0.02).to(torch.bfloat16).cpu()

    def gain(n):
        return (1.0 + (torch.rand(n, generator=g, device="cuda") * 0.2 - 0.1)).cpu()

    t = {"model.embed_tokens.weight": mat(v, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = gain(d)
        t[p + "self_attn.q_proj.weight"] = mat(h * hd, d)
        t[p + "self_attn.k_proj.weight"] = mat(kv * hd, d)
        t[p + "self_attn.v_proj.weight"] = mat(kv * hd, d)
        t[p + "self_attn.o_proj.weight"] = mat(d, h * hd)
        t[p + "post_attention_layernorm.weight"] = gain(d)
        t[p + "mlp.gate_proj.weight"] = mat(f, d)
        t[p + "mlp.up_proj.weight"] = mat(f, d)
        t[p + "mlp.down_proj.weight"] = mat(d, f)
    t["model.norm.weight"] = gain(d)
    t["lm_head.weight"] = mat(v, d)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    save_file(t, os.path.join(path, "model.safetensors"))
    return path


def requests_of(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


class Case:
    """A model folder, its oracle and the oracle's logits for the requests of the tests (computed once)."""

    def __init__(self, folder, shape):
        self.folder = folder
        self.vocab = SHAPES[shape]["vocab_size"]
        self.oracle = pl.PlainLlama(folder, dtype=torch.float32)
        self._want = {}
        self._models = {}

    def want(self, req, rows):
        key = (tuple(req), tuple(rows))
        if key not in self._want:
            self._want[key] = self.oracle.logits(req, rows=rows)
        return self._want[key]

    def engine(self, dtype, max_tokens, max_slots=None):
        from fms_b200.models import get_model

        if dtype not in self._models:
            self._models[dtype] = get_model("hf_pretrained", model_path=self.folder, device_type="cuda", data_type=dtype)
        return self._models[dtype].new_engine(max_tokens=max_tokens, max_slots=max_slots)


@pytest.fixture(scope="module")
def llama3(tmp_path_factory):
    return Case(write_big_folder(str(tmp_path_factory.mktemp("llama3_8b_2layers")), SHAPES["llama3_8b"], 11), "llama3_8b")


@pytest.fixture(scope="module")
def llama2(tmp_path_factory):
    return Case(write_big_folder(str(tmp_path_factory.mktemp("llama2_7b_2layers")), SHAPES["llama2_7b"], 12), "llama2_7b")


def close(got, want, dtype):
    """float32: 2e-3 of the logits' standard deviation (both sides sum in float32, in different orders, over up to
    14,336 terms).  bfloat16: 2% of the largest logit, as everywhere in these tests."""
    got, want = got.double().cpu(), want.double()
    assert got.shape == want.shape
    if dtype == "fp32":
        torch.testing.assert_close(got, want, atol=2e-3 * want.std().item(), rtol=0)
    else:
        torch.testing.assert_close(got, want, atol=0.02 * want.abs().max().item(), rtol=0.02)


LONG = 1100
PLACES = [0, 1, 63, 64, 511, 1023, 1024, LONG - 1]


@pytest.fixture(params=["default_products", "own_plain_products"])
def products_of_many_rows(request):
    """bfloat16 products of a prompt of 1,100 tokens: by default the library's; with the row limits at 1,024 and no
    limit on padding the own tcgen05 kernel for all of them (plain, gated, and the projection with the rotation and
    the cache write in its epilogue), which by default waits for more rows and for tiles that fit."""
    from fms_b200.kernels import ops

    saved = ops.TENSOR_CORE_ROWS, ops.TENSOR_CORE_ROWS_GLU, ops.TENSOR_CORE_ROWS_QKV, ops.TENSOR_CORE_MAX_PADDING
    if request.param == "own_plain_products":
        ops.TENSOR_CORE_ROWS = ops.TENSOR_CORE_ROWS_GLU = ops.TENSOR_CORE_ROWS_QKV = 1024
        ops.TENSOR_CORE_MAX_PADDING = 10.0
    yield request.param
    ops.TENSOR_CORE_ROWS, ops.TENSOR_CORE_ROWS_GLU, ops.TENSOR_CORE_ROWS_QKV, ops.TENSOR_CORE_MAX_PADDING = saved


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_one_long_prompt_whole(llama3, dtype, products_of_many_rows):
    """1,100 tokens in one step: in bfloat16 the tcgen05 products (pairs of blocks, GLU epilogue) and the tcgen05
    attention; logits at a handful of places (the first, block and tile edges, the last)."""
    if dtype == "fp32" and products_of_many_rows == "own_plain_products":
        pytest.skip("the float32 path has one product")
    (req,) = requests_of(llama3.vocab, [LONG], 1)
    engine = llama3.engine(dtype, max_tokens=1152)
    (slot,) = engine.begin(1)
    got = engine.step([slot], [req], [PLACES])
    engine.release([slot])
    engine.check()
    close(got, llama3.want(req, PLACES), dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_the_long_prompt_with_its_last_32_tokens_one_by_one(llama3, dtype):
    """All but 32 tokens in one step, then one token a step: the weight-streaming products (projection, rotation and
    cache write in one kernel; the head of 128,256 rows), split-key decode attention over 1,068 to 1,099 keys, plain
    launches at the first decode step and the captured graph from the second on."""
    (req,) = requests_of(llama3.vocab, [LONG], 1)
    cut = LONG - 32
    engine = llama3.engine(dtype, max_tokens=1152)
    (slot,) = engine.begin(1)
    parts = [engine.step([slot], [req[:cut]], [[cut - 1]])]
    for t in range(cut, LONG):
        parts.append(engine.step([slot], [[req[t]]], [[0]]))
    engine.release([slot])
    engine.check()
    if dtype == "bf16":
        assert engine.graph_launches >= 30
    close(torch.cat(parts), llama3.want(req, list(range(cut - 1, LONG))), dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_three_unequal_prompts_then_one_token_each(llama3, dtype):
    """Prompts of 700, 257 and 40 tokens in one step (997 rows: the products between 9 and 1,023 rows), then
    decode steps of three rows; the shortest request ends after two of them, the next after four."""
    reqs = requests_of(llama3.vocab, [706, 261, 42], 2)
    prompt = [700, 257, 40]
    engine = llama3.engine(dtype, max_tokens=64 * 18, max_slots=3)
    slots = engine.begin(3)
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:k] for r, k in zip(reqs, prompt)], [[0, k - 1] for k in prompt])
    for i in range(3):
        got[i].append(lg[2 * i:2 * i + 2])
    at = list(prompt)
    live = [0, 1, 2]
    while live:
        lg = engine.step([slots[i] for i in live], [[reqs[i][at[i]]] for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
            at[i] += 1
        for i in [i for i in live if at[i] == len(reqs[i])]:
            engine.release([slots[i]])
            live.remove(i)
    engine.check()
    for i, (r, k) in enumerate(zip(reqs, prompt)):
        close(torch.cat(got[i]), llama3.want(r, [0] + list(range(k - 1, len(r)))), dtype)


@pytest.fixture(params=["library_product", "own_product"])
def product_for_some_rows(request):
    """Products of 9 to 256 bfloat16 rows: all by the library's product, or all by this library's own tcgen05 kernel
    with its fused epilogues (the default is in between: the gated feed-forward product by the own kernel)."""
    from fms_b200.kernels import ops

    saved = ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS
    if request.param == "own_product":
        ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS = True, ["linear", "glu", "qkv"], 256
    else:
        ops.USE_MID_GEMM = False
    yield request.param
    ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS = saved


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_sixteen_requests_in_one_batch(llama3, dtype, product_for_some_rows):
    """Sixteen prompts of 3 to 90 tokens, then four decode steps of sixteen rows (more rows than the
    weight-streaming product takes)."""
    if dtype == "fp32" and product_for_some_rows == "own_product":
        pytest.skip("the float32 path has one product")
    lengths = [3, 64, 65, 90] + [7 + 5 * i for i in range(12)]
    reqs = requests_of(llama3.vocab, [n + 4 for n in lengths], 3)
    engine = llama3.engine(dtype, max_tokens=64 * 2 * 16, max_slots=16)
    slots = engine.begin(16)
    rows = [engine.step(slots, [r[:n] for r, n in zip(reqs, lengths)])]
    for t in range(4):
        rows.append(engine.step(slots, [[r[n + t]] for r, n in zip(reqs, lengths)]))
    engine.release(slots)
    engine.check()
    got = torch.stack(rows, 1)  # [request, step, vocab]
    for i, (r, n) in enumerate(zip(reqs, lengths)):
        close(got[i], llama3.want(r, list(range(n - 1, n + 4))), dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_full_multi_head_layout_of_llama_2_7b(llama2, dtype):
    """32 key/value heads (one query head each, eight times the keys and values a token): a prompt of 1,100 tokens
    whole, its last 8 tokens one by one, and beside it in the same batch a request of 300 tokens."""
    reqs = requests_of(llama2.vocab, [LONG, 300], 4)
    cut = [LONG - 8, 300 - 8]
    engine = llama2.engine(dtype, max_tokens=64 * 23, max_slots=2)
    slots = engine.begin(2)
    got = [[], []]
    places = [[0, 64, 1023, 1024, cut[0] - 1], [0, cut[1] - 1]]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], places)
    got[0].append(lg[:5])
    got[1].append(lg[5:])
    for t in range(8):
        lg = engine.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)])
        got[0].append(lg[0:1])
        got[1].append(lg[1:2])
    engine.release(slots)
    engine.check()
    for i in (0, 1):
        close(torch.cat(got[i]), llama2.want(reqs[i], places[i] + list(range(cut[i], len(reqs[i])))), dtype)
