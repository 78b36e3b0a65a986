"""The tiny Llama configurations of the tests and a writer of model folders with random weights.

The writer belongs to the tests (it does not use the library's own random-weights mode), so that the plain
implementation and the stored reference outputs do not depend on the code under test.  The
configurations differ in every size and option: head counts and groups, head size, widths that are no
power of two, number of layers, vocabulary, eps, rope theta, tied or untied head, context length and the
dtype in which the norm gains are stored.
"""
from __future__ import annotations

import json
import os

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 176,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 64,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 256,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "max_position_embeddings": 128,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
}

# A third shape for long sequences: head size 48 (a multiple of 16 that is no power of two), 5 query
# heads over 5 key/value heads, an odd vocabulary, a context of 1024.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 331,
    "hidden_size": 240,
    "intermediate_size": 328,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
}

# A fourth whose attention is peaked: the q and k projections are drawn with a standard deviation of 0.125
# instead of 0.02, so that scores have a standard deviation of about 2 and a softmax row is carried by a few
# keys.  With N(0, 0.02) everywhere a tiny model's scores stay within +-0.4 and every row is close to a plain
# average, in which a dropped or misplaced key hardly shows.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 211,
    "hidden_size": 128,
    "intermediate_size": 200,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "mlp_bias": False,
}

# A fifth with what the others lack: biases on every projection (~ N(0, 0.1)) and the llama3 rescaling of the
# rotation's frequencies (five query heads over one key/value head, head size 16).
TINY_E = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 173,
    "hidden_size": 80,
    "intermediate_size": 120,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 1,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 512,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": True,
    "mlp_bias": True,
}

TINY = {"a": (TINY_A, 0, torch.bfloat16), "b": (TINY_B, 1, torch.float32), "c": (TINY_C, 2, torch.bfloat16),
        "d": (TINY_D, 3, torch.float32), "e": (TINY_E, 4, torch.float32)}
# how a configuration's tensors are drawn, where not as tiny_tensors' defaults have it
TINY_OPTIONS = {"d": {"qk_std": 0.125}, "e": {"biases": True}}


def tiny_tensors(cfg: dict, seed: int, gain_dtype: torch.dtype = torch.bfloat16, matrix_std: float = 0.02,
                 qk_std: float = None, biases: bool = False):
    """Linear and embedding weights ~ N(0, 0.02) rounded to bfloat16, norm gains 1 + U(-0.1, 0.1), drawn
    in a fixed order from a CPU generator.  ``qk_std``: another standard deviation for the q and k
    projections; ``biases``: also the biases that the configuration asks for."""
    if biases:
        return tiny_tensors_with_biases(cfg, seed)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    d = cfg["hidden_size"]
    h = cfg["num_attention_heads"]
    kv = cfg["num_key_value_heads"]
    hd = d // h
    f = cfg["intermediate_size"]
    v = cfg["vocab_size"]

    def mat(rows, cols, std=matrix_std):
        return (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)

    def gain(n):
        return (1.0 + (torch.rand(n, generator=g) * 0.2 - 0.1)).to(gain_dtype)

    t = {"model.embed_tokens.weight": mat(v, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = gain(d)
        t[p + "self_attn.q_proj.weight"] = mat(h * hd, d, qk_std or matrix_std)
        t[p + "self_attn.k_proj.weight"] = mat(kv * hd, d, qk_std or matrix_std)
        t[p + "self_attn.v_proj.weight"] = mat(kv * hd, d)
        t[p + "self_attn.o_proj.weight"] = mat(d, h * hd)
        t[p + "post_attention_layernorm.weight"] = gain(d)
        t[p + "mlp.gate_proj.weight"] = mat(f, d)
        t[p + "mlp.up_proj.weight"] = mat(f, d)
        t[p + "mlp.down_proj.weight"] = mat(d, f)
    t["model.norm.weight"] = gain(d)
    if not cfg["tie_word_embeddings"]:
        t["lm_head.weight"] = mat(v, d)
    return t


def tiny_tensors_of(which: str):
    """The tensors of one of the named tiny configurations."""
    cfg, seed, gain_dtype = TINY[which]
    return tiny_tensors(cfg, seed, gain_dtype, **TINY_OPTIONS.get(which, {}))


def llama_config(vocab, hidden, intermediate, layers, heads, kvheads, eps=1e-5, theta=1e4, context=512, tied=False,
                 attention_bias=False, mlp_bias=False, rope_scaling=None) -> dict:
    """A config.json of further sizes and options, for tests that make their own model."""
    cfg = dict(TINY_A, vocab_size=vocab, hidden_size=hidden, intermediate_size=intermediate, num_hidden_layers=layers,
               num_attention_heads=heads, num_key_value_heads=kvheads, rms_norm_eps=eps, rope_theta=theta,
               max_position_embeddings=context, tie_word_embeddings=tied, attention_bias=attention_bias,
               mlp_bias=mlp_bias)
    if rope_scaling:
        cfg["rope_scaling"] = rope_scaling
    return cfg


def tiny_tensors_with_biases(cfg: dict, seed: int) -> dict:
    """``tiny_tensors`` and, where the configuration asks for them, biases ~ N(0, 0.1) of the projections."""
    t = tiny_tensors(cfg, seed, torch.float32)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed + 99)
    d, h, kv, f = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    hd = d // h
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if cfg.get("attention_bias"):
            for name, rows in (("q_proj", h * hd), ("k_proj", kv * hd), ("v_proj", kv * hd), ("o_proj", d)):
                t[p + f"self_attn.{name}.bias"] = (torch.randn(rows, generator=g) * 0.1).to(torch.bfloat16)
        if cfg.get("mlp_bias"):
            for name, rows in (("gate_proj", f), ("up_proj", f), ("down_proj", d)):
                t[p + f"mlp.{name}.bias"] = (torch.randn(rows, generator=g) * 0.1).to(torch.bfloat16)
    return t


def write_folder(path: str, cfg: dict, tensors: dict) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(path, "model.safetensors"))
    return path


def write_tiny(path: str, which: str) -> str:
    return write_folder(path, TINY[which][0], tiny_tensors_of(which))


def tiny_prompts(which: str):
    """Seeded prompts of unequal lengths with token ids uniform in [0, vocab).  No prompt is as long as its model
    has key/value heads (unless both are 1): scored whole and without a cache, the reference takes keys of shape
    [batch, tokens, kv heads, head size] for already transposed when tokens == kv heads
    (fms/modules/attention.py:228-230) and mixes tokens with heads, which its stored outputs would then hold."""
    cfg, seed, _ = TINY[which]
    lengths = {"a": [5, 11, 17], "b": [1, 7, 30, 64], "c": [3, 70, 200], "d": [3, 65, 300], "e": [1, 40, 130]}[which]
    g = torch.Generator(device="cpu")
    g.manual_seed(1000 + seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


# ---- a model in which one key carries a query's whole attention --------------------------------------------------
PLANT_QUERY, PLANT_KEYS, PLANT_ORDINARY = 199, (200, 201, 202, 203, 204, 205), 190


def planted_tensors():
    """Tiny D's tensors with layer 0 changed so that the query of token ``PLANT_QUERY`` gives nearly all of its
    attention, in every head, to the key of a token of ``PLANT_KEYS`` wherever in the sequence that token stands;
    tokens below ``PLANT_ORDINARY`` are ordinary.  How: the planted tokens' embeddings lie along one direction of
    the stream (plus a direction of their own, so that their values differ), the query token's along another; row
    15 of every head of k_proj reads the first direction and row 15 of q_proj the second.  In the HF layout rows
    15 and 31 of a head are the rotation's slowest pair (angle 1.8e-4 a position), so the product keeps its size
    over hundreds of positions.  A kernel that drops, misplaces or double-counts that one key changes the layer's
    output beyond any tolerance, where among near-equal weights it would change it by a few hundredths."""
    cfg = TINY_D
    t = tiny_tensors_of("d")
    d, h, kv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = d // h
    emb = t["model.embed_tokens.weight"].float()
    key_dir, query_dir = 5, 6
    for n, tok in enumerate(PLANT_KEYS):
        emb[tok] = 0.0
        emb[tok, key_dir] = 1.0
        emb[tok, 10 + n] = 0.5
    emb[PLANT_QUERY] = 0.0
    emb[PLANT_QUERY, query_dir] = 1.0
    emb[PLANT_QUERY, 30] = 0.5
    t["model.embed_tokens.weight"] = emb.to(torch.bfloat16)
    t["model.layers.0.input_layernorm.weight"] = torch.ones(d)
    wq = t["model.layers.0.self_attn.q_proj.weight"].float()
    wk = t["model.layers.0.self_attn.k_proj.weight"].float()
    for head in range(h):
        wq[head * hd + hd // 2 - 1] = 0.0
        wq[head * hd + hd // 2 - 1, query_dir] = 1.5
    for head in range(kv):
        wk[head * hd + hd // 2 - 1] = 0.0
        wk[head * hd + hd // 2 - 1, key_dir] = 1.5
    t["model.layers.0.self_attn.q_proj.weight"] = wq.to(torch.bfloat16)
    t["model.layers.0.self_attn.k_proj.weight"] = wk.to(torch.bfloat16)
    return t


def planted_request(length: int, key_at: int, key_token: int, queries_at, seed: int):
    """``length`` ordinary tokens with ``key_token`` at ``key_at`` and the query token at ``queries_at``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    ids = torch.randint(0, PLANT_ORDINARY, (length,), generator=g).tolist()
    ids[key_at] = key_token
    for p in queries_at:
        assert p != key_at
        ids[p] = PLANT_QUERY
    return ids
