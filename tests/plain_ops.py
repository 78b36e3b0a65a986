"""Plain torch restatements of the library's kernels, one function per kernel with the kernel's own
signature (``fms_b200.kernels.ops``).  Two uses: on the GPU each kernel is compared with its
restatement; on the CPU ``use_plain_ops`` puts them in the kernels' place so that the library's host
logic (loader, cache, batching, schedule, generation) can be tested without a device.  They are test
code: the library never imports them and has no CPU path of its own.
"""
from __future__ import annotations

import contextlib
import math

import torch

from plain_llama import plain_uniform


def embed(table, tokens, scale=1.0):
    return table[tokens.long()].float() * scale


def add_rmsnorm(residual, delta, gain, eps, out_dtype, rows=None):
    if rows is None:
        if delta is not None:
            residual += delta.float()
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain.float()
    return y.to(out_dtype)


def linear(x, weight, bias=None, out_dtype=None):
    out_dtype = out_dtype or x.dtype
    y = x.double() @ weight.double().T
    if bias is not None:
        y = y + bias.double()
    return y.to(out_dtype)


def gated_activation(gate_up, activation):
    hidden = gate_up.shape[1] // 2
    g, u = gate_up[:, :hidden].float(), gate_up[:, hidden:].float()
    act = {0: torch.nn.functional.silu, 1: torch.nn.functional.gelu,
           2: lambda t: torch.nn.functional.gelu(t, approximate="tanh"), 3: torch.relu}[activation]
    return (act(g) * u).to(gate_up.dtype)


def gated_linear(x, weight, bias, activation):
    return gated_activation(linear(x, weight, bias), activation)


def rope_store(qkv, inv_freq, batch, view, nheads, kvheads, head_dim, writes_cache=True):
    n = qkv.shape[0]
    x = qkv.float().view(n, nheads + 2 * kvheads, head_dim)
    pos = batch.positions.long()  # the place in the cache
    ids = getattr(batch, "position_ids", None)  # what the rotation sees, where that differs
    if inv_freq is not None:
        ang = torch.outer((pos if ids is None else ids.long()).float(), inv_freq.float().cpu().to(qkv.device))
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        rot = x[:, : nheads + kvheads]
        x0, x1 = rot[..., 0::2], rot[..., 1::2]
        rot = torch.stack([cos * x0 - sin * x1, sin * x0 + cos * x1], -1).flatten(-2)
        x = torch.cat([rot, x[:, nheads + kvheads:]], 1)
    q = x[:, :nheads].reshape(n, nheads * head_dim).to(qkv.dtype)
    if writes_cache:
        slots = batch.slots.long()[batch.token_seq.long()]
        blocks = view.table[slots, pos // view.block_tokens].long()
        assert (blocks >= 0).all(), "a token's position has no cache block"
        rows = pos % view.block_tokens
        view.keys[blocks, :, rows] = x[:, nheads: nheads + kvheads].to(view.keys.dtype)
        view.values[blocks, :, rows] = x[:, nheads + kvheads:].to(view.values.dtype)
    return q


def qkv_rope_store(x, weight, bias, inv_freq, batch, view, nheads, kvheads, head_dim, writes_cache=True):
    return rope_store(linear(x, weight, bias), inv_freq, batch, view, nheads, kvheads, head_dim, writes_cache)


def gather_cache(view, slot, lo, hi):
    """Keys and values [hi - lo, kvheads, head_dim] of positions lo..hi-1 of the sequence in ``slot``."""
    pos = torch.arange(lo, hi, device=view.keys.device)
    blocks = view.table[slot, pos // view.block_tokens].long()
    assert (blocks >= 0).all(), "a visible position has no cache block"
    rows = pos % view.block_tokens
    return view.keys[blocks, :, rows].float(), view.values[blocks, :, rows].float()


def attention(q, batch, view, nheads, kvheads, head_dim, scale, window):
    out = torch.zeros_like(q)
    first = batch.first_row.tolist()
    lens = batch.len_after.tolist()
    slots = batch.slots.tolist()
    group = nheads // kvheads
    for i in range(batch.n_seqs):
        n_new = first[i + 1] - first[i]
        for j in range(n_new):
            p = lens[i] - n_new + j
            lo = max(0, p - window + 1) if window else 0
            k, v = gather_cache(view, slots[i], lo, p + 1)
            qq = q[first[i] + j].float().view(nheads, head_dim)
            kk = k.repeat_interleave(group, dim=1)
            vv = v.repeat_interleave(group, dim=1)
            s = torch.einsum("hd,thd->ht", qq, kk) * scale
            pr = torch.softmax(s, -1)
            out[first[i] + j] = torch.einsum("ht,thd->hd", pr, vv).reshape(-1).to(q.dtype)
    return out


def decode_advance(positions, lengths, offsets=None, position_ids=None, slots=None, spare_slot=-1):
    if slots is not None:
        lengths.masked_fill_(slots == spare_slot, 0)
    positions.copy_(lengths)
    if offsets is not None:
        position_ids.copy_(lengths + offsets)
    lengths += 1


def argmax(logits, out=None):
    r = torch.argmax(logits, dim=-1).to(torch.int32)
    if out is not None:
        out.copy_(r)
        return out
    return r


def sample(logits, temperature, top_k, seed, requests, step, out=None):
    from plain_llama import plain_sample

    res = [plain_sample(logits[i].cpu(), temperature, top_k, plain_uniform(seed, int(requests[i]), step))
           for i in range(logits.shape[0])]
    r = torch.tensor(res, dtype=torch.int32, device=logits.device)
    if out is not None:
        out.copy_(r)
        return out
    return r


def error_flag(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_error_flag(device):
    return None


PLAIN = dict(embed=embed, add_rmsnorm=add_rmsnorm, linear=linear, gated_activation=gated_activation, gated_linear=gated_linear,
             rope_store=rope_store, qkv_rope_store=qkv_rope_store, attention=attention, decode_advance=decode_advance, argmax=argmax, sample=sample, error_flag=error_flag,
             check_error_flag=check_error_flag)


@contextlib.contextmanager
def use_plain_ops():
    """Within the block the library's kernel entry points are the functions above, and the engine accepts
    the CPU as its device."""
    from fms_b200.engine import step as step_module
    from fms_b200.kernels import ops

    saved = {k: getattr(ops, k) for k in PLAIN}
    for k, f in PLAIN.items():
        setattr(ops, k, f)
    saved_flag = getattr(step_module, "_REQUIRE_CUDA", True)
    step_module._REQUIRE_CUDA = False
    try:
        yield
    finally:
        for k, f in saved.items():
            setattr(ops, k, f)
        step_module._REQUIRE_CUDA = saved_flag
