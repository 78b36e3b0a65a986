"""Plain, slow Llama: the oracle of every test.

Whole sequences, no cache, one function for each part, torch ops on the CPU only.  It shares no code
with the library under test: it reads ``config.json`` and ``model.safetensors`` itself and is written
from the formulas of the reference (Foundation Model Stack), each cited as ``file:line`` of that project.
``tests/golden/make_golden.py`` compared it once with the reference's own model code on tiny random
models; ``tests/test_plain_vs_golden.py`` repeats that comparison from the stored outputs.

All functions take a ``dtype`` (float64 by default) in which the whole computation runs, so that the
oracle's own rounding is far below any tolerance a test uses.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

MASK64 = (1 << 64) - 1


# --------------------------------------------------------------------------------------------------
# reading a model folder
# --------------------------------------------------------------------------------------------------

def read_model_folder(path: str):
    """Returns (config dict, {HF tensor name: tensor}) of a folder with config.json + model.safetensors."""
    from safetensors import safe_open

    with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


def config_values(cfg: dict) -> dict:
    """config.json keys -> the sizes and constants of the architecture
    (fms/models/hf/config_utils/param_builders.py:37-58 and :512-546)."""
    rope_theta = cfg.get("rope_theta")
    rope_scaling = cfg.get("rope_scaling")
    if cfg.get("rope_parameters") is not None:  # param_builders.py:18-34
        rope_theta = cfg["rope_parameters"]["rope_theta"]
        rope_scaling = cfg["rope_parameters"].get("rope_scaling")
    d = cfg["hidden_size"]
    h = cfg["num_attention_heads"]
    kv = cfg.get("num_key_value_heads", h) or h  # kvheads 0 means nheads, fms/models/llama.py:69-70
    return dict(
        vocab=cfg["vocab_size"],
        dim=d,
        nheads=h,
        kvheads=kv,
        head_dim=d // h,  # fms/models/llama.py:67-68
        nlayers=cfg["num_hidden_layers"],
        hidden=cfg["intermediate_size"],
        eps=cfg["rms_norm_eps"],
        theta=10000.0 if rope_theta is None else float(rope_theta),
        rope_scaling=rope_scaling or {},
        max_pos=cfg.get("max_position_embeddings", 4096),
        tied=bool(cfg.get("tie_word_embeddings", False)),
        attn_bias=bool(cfg.get("attention_bias", False)),
        mlp_bias=bool(cfg.get("mlp_bias", False)),
    )


def hf_rows_to_interleaved(w: torch.Tensor, head_dim: int) -> torch.Tensor:
    """HF checkpoints keep each head's rotary pairs as two halves; the reference's RoPE rotates adjacent
    pairs, so its loader permutes the rows of the q and k projections (fms/models/llama.py:730-736)."""
    rows = w.shape[0]
    n = rows // head_dim
    if w.dim() == 2:
        return w.view(n, 2, head_dim // 2, w.shape[1]).transpose(1, 2).reshape(rows, w.shape[1])
    return w.view(n, 2, head_dim // 2).transpose(1, 2).reshape(rows)


# --------------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------------

def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x0[s, :] = E[ids[s], :]  (fms/models/llama.py:332)."""
    return table[ids.long()]


def plain_rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * gain, eps inside the root, no mean subtraction, no bias
    (fms/modules/layernorm.py:56-69 with use_mean=False, elementwise_shift=False)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain.to(x.dtype)


def plain_rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """inv_f[i] = 1 / theta^(2i/head_dim), in float32 as the reference builds it
    (fms/modules/positions.py:124-132); the llama3 rescaling of fms/modules/positions.py:171-196."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    scaling = scaling or {}
    kind = scaling.get("rope_type", scaling.get("type", "regular"))
    if kind in ("regular", "default", None):
        return inv
    if kind == "llama3":
        factor = scaling["factor"]
        low = scaling["low_freq_factor"]
        high = scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > old / low, inv / factor, inv)
        smooth = (old / wavelen - low) / (high - low)
        smoothed = (1 - smooth) * scaled / factor + smooth * scaled
        medium = ~(wavelen < old / high) * ~(wavelen > old / low)
        return torch.where(medium, smoothed, scaled)
    raise ValueError(f"plain implementation has no rope scaling {kind!r}")


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotates adjacent pairs of the last dimension: o[2i] = cos*x[2i] - sin*x[2i+1],
    o[2i+1] = sin*x[2i] + cos*x[2i+1], angle = position * inv_f[i] as a float32 product
    (fms/modules/positions.py:311-355 for the table, :438-456 for the rotation).
    x: [S, heads, head_dim]; positions: [S]."""
    ang = torch.outer(positions.float(), inv_freq.float())  # float32, as the reference's table
    cos = ang.cos().to(x.dtype)[:, None, :]
    sin = ang.sin().to(x.dtype)[:, None, :]
    x0 = x[..., 0::2]
    x1 = x[..., 1::2]
    out = torch.stack([cos * x0 - sin * x1, sin * x0 + cos * x1], dim=-1)
    return out.flatten(-2)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
                    scale: Optional[float] = None) -> torch.Tensor:
    """softmax(q k^T * scale + causal mask) v with grouped key/value heads: query head h uses key/value
    head h // (H/KV); scale 1/sqrt(head_dim) (fms/modules/attention.py:215-294).  A window W keeps, for
    the query at position p, the keys p-W+1..p (the trimming of fms/modules/attention.py:197-204).
    q: [S, H, hd]; k, v: [S, KV, hd]; returns [S, H, hd]."""
    s, h, hd = q.shape
    kvh = k.shape[1]
    group = h // kvh
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    kk = k.repeat_interleave(group, dim=1)  # attention.py:244-250 expands the kv heads
    vv = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("shd,thd->hst", q, kk) * scale
    pos = torch.arange(s)
    visible = pos[None, :] <= pos[:, None]
    if window:
        visible &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hst,thd->shd", p, vv)


def plain_swiglu_ffn(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                     b_gate=None, b_up=None, b_down=None) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (fms/modules/feedforward.py:288-297, activation "swish" = SiLU,
    fms/utils/activation.py:21-22)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    if b_gate is not None:
        g = g + b_gate
        u = u + b_up
    y = (torch.nn.functional.silu(g) * u) @ w_down.T
    if b_down is not None:
        y = y + b_down
    return y


# --------------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------------

class PlainLlama:
    """Holds a folder's tensors under their HF names, converted once to ``dtype``."""

    def __init__(self, path: str, dtype: torch.dtype = torch.float64):
        cfg, tensors = read_model_folder(path)
        self.raw_config = cfg
        self.c = config_values(cfg)
        self.dtype = dtype
        self.w: Dict[str, torch.Tensor] = {k: t.to(dtype) for k, t in tensors.items()}
        hd = self.c["head_dim"]
        for i in range(self.c["nlayers"]):
            for proj in ("q_proj", "k_proj"):
                for kind in ("weight", "bias"):
                    name = f"model.layers.{i}.self_attn.{proj}.{kind}"
                    if name in self.w:
                        self.w[name] = hf_rows_to_interleaved(self.w[name], hd)
        self.inv_freq = plain_rope_inv_freq(hd, self.c["theta"], self.c["rope_scaling"])

    def block(self, i: int, x: torch.Tensor, positions: torch.Tensor, window: int = 0) -> torch.Tensor:
        """Pre-norm attention and pre-norm feed-forward, each added to the residual stream
        (fms/models/llama.py:118-167)."""
        c, w = self.c, self.w
        p = f"model.layers.{i}."
        s = x.shape[0]
        h = plain_rmsnorm(x, w[p + "input_layernorm.weight"], c["eps"])
        q = h @ w[p + "self_attn.q_proj.weight"].T
        k = h @ w[p + "self_attn.k_proj.weight"].T
        v = h @ w[p + "self_attn.v_proj.weight"].T
        if c["attn_bias"]:
            q = q + w[p + "self_attn.q_proj.bias"]
            k = k + w[p + "self_attn.k_proj.bias"]
            v = v + w[p + "self_attn.v_proj.bias"]
        q = plain_rope(q.view(s, c["nheads"], c["head_dim"]), positions, self.inv_freq)
        k = plain_rope(k.view(s, c["kvheads"], c["head_dim"]), positions, self.inv_freq)
        v = v.view(s, c["kvheads"], c["head_dim"])
        a = plain_attention(q, k, v, window=window).reshape(s, -1)
        a = a @ w[p + "self_attn.o_proj.weight"].T
        if c["attn_bias"]:
            a = a + w[p + "self_attn.o_proj.bias"]
        x = x + a
        h = plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        f = plain_swiglu_ffn(
            h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"],
            w.get(p + "mlp.gate_proj.bias"), w.get(p + "mlp.up_proj.bias"), w.get(p + "mlp.down_proj.bias"),
        )
        return x + f

    def logits(self, ids: Sequence[int], rows: Optional[Sequence[int]] = None, first_position: int = 0) -> torch.Tensor:
        """Logits at every position of one whole sequence: [S, vocab]
        (fms/models/llama.py:318-357 and :425-450).  With ``rows`` the head is applied at those positions
        only (the layers still run the whole sequence): [len(rows), vocab].  ``first_position``: the position
        of the first token (the reference's position_ids, fms/models/llama.py:337-343; 0 by default)."""
        ids_t = torch.as_tensor(list(ids), dtype=torch.long)
        positions = torch.arange(ids_t.shape[0]) + int(first_position)
        x = plain_embedding(ids_t, self.w["model.embed_tokens.weight"])
        for i in range(self.c["nlayers"]):
            x = self.block(i, x, positions)
        if rows is not None:
            x = x[torch.as_tensor(list(rows), dtype=torch.long)]
        x = plain_rmsnorm(x, self.w["model.norm.weight"], self.c["eps"])
        head = self.w["model.embed_tokens.weight"] if self.c["tied"] else self.w["lm_head.weight"]
        return x @ head.T


# --------------------------------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------------------------------

def plain_uniform(seed: int, request: int, step: int) -> float:
    """The uniform number in [0, 1) that the library draws for one request at one decoding step: a
    splitmix64 hash of (seed, request, step), top 24 bits.  This is the library's own definition (the
    reference draws from torch's global generator, fms/utils/generation.py:318-326), restated here with
    Python integers."""
    def mix(z: int) -> int:
        z = (z + 0x9E3779B97F4A7C15) & MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    z = mix(seed & MASK64)
    z = mix(z ^ (request & MASK64))
    z = mix(z ^ (step & MASK64))
    return (z >> 40) / float(1 << 24)


def plain_greedy(logits: torch.Tensor) -> int:
    """argmax, the lowest index among equals (fms/utils/generation.py:328)."""
    return int(torch.argmax(logits).item())


def plain_sample(logits: torch.Tensor, temperature: float, top_k: int, u: float) -> int:
    """logits / temperature; with top_k, everything below the k-th largest value becomes -inf; softmax;
    one draw (fms/utils/generation.py:318-326).  The draw is the inverse CDF at ``u``: the first index
    whose running sum of probabilities exceeds u * total."""
    x = logits.to(torch.float64) / temperature
    if top_k:
        kth = torch.topk(x, min(top_k, x.numel())).values[-1]
        x = torch.where(x < kth, torch.full_like(x, float("-inf")), x)
    p = torch.exp(x - x.max())
    c = torch.cumsum(p, 0)
    target = u * c[-1]
    idx = int(torch.searchsorted(c, target, right=True).item())
    return min(idx, x.numel() - 1)


def plain_generate(model: PlainLlama, prompt: Sequence[int], max_new_tokens: int, do_sample: bool = False,
                   temperature: float = 1.0, top_k: int = 0, seed: int = 0, request: int = 0,
                   eos: Optional[Sequence[int]] = None, logits_out: Optional[List[torch.Tensor]] = None,
                   first_position: int = 0) -> List[int]:
    """Recomputes the whole sequence for every new token (the reference's loop without a cache,
    fms/utils/generation.py:287-346); stops after a stop token."""
    ids = list(prompt)
    for step in range(max_new_tokens):
        lg = model.logits(ids, first_position=first_position)[-1]
        if logits_out is not None:
            logits_out.append(lg)
        if do_sample:
            nxt = plain_sample(lg, temperature, top_k, plain_uniform(seed, request, step))
        else:
            nxt = plain_greedy(lg)
        ids.append(nxt)
        if eos and nxt in eos:
            break
    return ids
