"""Each part of a layer alone against the plain implementation, and the generality of the assembly: a toy
mixer with state of its own, a toy feed-forward with routing and a decoder whose schedule names a layer
twice are defined HERE, registered, built and stepped without a change to the library's files."""
import math

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu


def close(got, want, dtype):
    want = want.double().cpu()
    got = got.double().cpu()
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    else:
        torch.testing.assert_close(got, want, atol=0.02 * want.abs().max().item(), rtol=0.02)


def fill(part, dtype, seed, scale=0.05):
    """Random tensors for everything a part declares; returns them by qualified name (float64 copies)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, owner, local, decl in part.named_decls():
        if decl.role == "vector":
            t = 1 + 0.1 * torch.randn(decl.shape, generator=g)
        else:
            t = torch.randn(decl.shape, generator=g) * scale
        t = t.to(dtype)
        owner.set_tensor(local, t.cuda())
        out[name] = t.double()
    part.finalize(torch.device("cuda"), dtype)
    return out


def one_sequence_batch(n_new, len_before, cache, slot):
    from fms_b200.engine.batch import Batch

    cache.prepare([slot], [n_new])
    b = Batch.from_lists([slot], [len_before], [[0] * n_new], [[]], "cuda")
    return b


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from fms_b200.config import NormSpec
    from fms_b200.parts import build_norm

    norm = build_norm(NormSpec("rmsnorm", 240, 1e-6))
    w = fill(norm, dtype, 0)
    g = torch.Generator().manual_seed(1)
    res = torch.randn(9, 240, generator=g).cuda()
    delta = torch.randn(9, 240, generator=g).to(dtype).cuda()
    want = pl.plain_rmsnorm(res.double().cpu() + delta.double().cpu(), w["weight"], 1e-6)
    got = norm.apply(res, delta, dtype)
    close(got, want, dtype)
    with pytest.raises(KeyError):
        build_norm(NormSpec("no_such_norm", 8, 1e-5))


def test_rotary_part_frequencies():
    from fms_b200.config import PositionSpec
    from fms_b200.parts import build_position

    for theta, scaling in ((10000.0, {}), (500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                       "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})):
        part = build_position(PositionSpec("rope", head_dim=64, theta=theta, scaling=tuple(sorted(scaling.items()))))
        part.finalize(torch.device("cuda"), torch.float32)
        torch.testing.assert_close(part.rotary_frequencies().cpu(), pl.plain_rope_inv_freq(64, theta, scaling), rtol=1e-6,
                                   atol=0)
    from fms_b200.parts import PositionEncoding

    assert type(build_position(PositionSpec("none"))) is PositionEncoding  # the base: encodes nothing
    with pytest.raises(ValueError):
        build_position(PositionSpec("rope", head_dim=64, scaling=(("rope_type", "yarn"),)))


def plain_mixer(w, x, nheads, kvheads, hd, theta, window, positions):
    s = x.shape[0]
    qkv = x @ w["in_proj.qkv_fused.weight"].T
    q, k, v = qkv.split([nheads * hd, kvheads * hd, kvheads * hd], -1)
    inv = pl.plain_rope_inv_freq(hd, theta)
    q = pl.plain_rope(q.view(s, nheads, hd), positions, inv)
    k = pl.plain_rope(k.view(s, kvheads, hd), positions, inv)
    a = pl.plain_attention(q, k, v.view(s, kvheads, hd), window=window).reshape(s, -1)
    return a @ w["dense.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nheads,kvheads,hd,window", [(4, 2, 16, 0), (6, 1, 32, 0), (3, 3, 48, 40)])
def test_attention_part_alone(dtype, nheads, kvheads, hd, window):
    """The mixer with a cache of its own: a whole sequence, then the same sequence cut in three."""
    from fms_b200.cache import Cache
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import build_mixer

    dim, theta, n = nheads * hd, 10000.0, 150
    spec = MixerSpec("attention", dim=dim, nheads=nheads, kvheads=kvheads, head_dim=hd, window=window,
                     position=PositionSpec("rope", head_dim=hd, theta=theta))
    mixer = build_mixer(spec)
    w = fill(mixer, dtype, 2, scale=0.08)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(n, dim, generator=g).to(dtype)
    want = plain_mixer(w, x.double(), nheads, kvheads, hd, theta, window, torch.arange(n))
    cache = Cache([mixer.cache_request()], max_tokens=512, max_positions=512, dtype=dtype, device="cuda")
    for cuts in ([n], [70, 1, 79]):
        (slot,) = cache.begin(1)
        outs, at = [], 0
        for k in cuts:
            batch = one_sequence_batch(k, at, cache, slot)
            outs.append(mixer.forward(x[at:at + k].cuda().contiguous(), batch, cache.layer_view(0), True))
            cache.commit([slot], [k])
            at += k
        cache.release([slot])
        close(torch.cat(outs), want, dtype)


def _run_mixer_in_three_steps(mixer, x, dtype, first_position=0):
    from fms_b200.cache import Cache
    from fms_b200.engine.batch import Batch

    cache = Cache([mixer.cache_request()], max_tokens=256, max_positions=512, dtype=dtype, device="cuda")
    (slot,) = cache.begin(1, [first_position])
    outs, at = [], 0
    for k_new in (60, 1, x.shape[0] - 61):
        cache.prepare([slot], [k_new])
        batch = Batch.from_lists([slot], [at], [[0] * k_new], [[]], "cuda", [cache.offset(slot)])
        outs.append(mixer.forward(x[at:at + k_new].to(dtype).cuda().contiguous(), batch, cache.layer_view(0), True))
        cache.commit([slot], [k_new])
        at += k_new
    return torch.cat(outs)


def wave(positions, head_dim):
    """[n, head_dim] float64: what the toy encoding ``toy_added_wave`` adds to every q and k head at a position."""
    d = torch.arange(head_dim, dtype=torch.float64, device=positions.device)
    return 0.3 * torch.sin(positions.double()[:, None] * 0.05 * (d[None, :] + 1.0))


def register_toy_encodings():
    from fms_b200.kernels import ops
    from fms_b200.parts import PositionEncoding, register_position, registered

    class LinearFrequencies(PositionEncoding):
        def __init__(self, spec):
            super().__init__(spec)
            self.half, self.top = spec.head_dim // 2, spec.theta
            self._f = None

        def frequencies(self):
            return (self.top * (1.0 - torch.arange(self.half).float() / self.half)).float()

        def finalize(self, device, dtype):
            self._f = self.frequencies().to(device).contiguous()

        def project(self, x, linear, batch, cache_view, nheads, kvheads, head_dim, writes_cache=True):
            return ops.qkv_rope_store(x, linear.tensor("weight"), linear.tensor("bias"), self._f, batch, cache_view, nheads,
                                      kvheads, head_dim, writes_cache)

    class AddedWave(PositionEncoding):
        def project(self, x, linear, batch, cache_view, nheads, kvheads, head_dim, writes_cache=True):
            qkv = ops.linear(x, linear.tensor("weight"), linear.tensor("bias"))
            pos = batch.positions if batch.position_ids is None else batch.position_ids
            rows = qkv.float().view(qkv.shape[0], nheads + 2 * kvheads, head_dim)  # no host synchronisation: capturable
            rows[:, : nheads + kvheads] += wave(pos, head_dim).float()[:, None, :]
            qkv = rows.view(qkv.shape).to(qkv.dtype)
            return ops.rope_store(qkv, None, batch, cache_view, nheads, kvheads, head_dim, writes_cache)  # stores as it is

    if "toy_linear_frequencies" not in registered("position"):
        register_position("toy_linear_frequencies", LinearFrequencies)
        register_position("toy_added_wave", AddedWave)


def test_toy_position_encodings_are_registered_and_used_by_the_mixer():
    """Two other position encodings, defined here, registered under names of their own and chosen by the mixer's
    spec; the attention part and its kernels take them without a change.  The first rotates pairs with frequencies
    that fall linearly instead of geometrically (it keeps the rotary kernels).  The second is no rotation at all: it
    adds a vector that depends on the position to every head of q and k (written with torch operations: a test's
    toy), and leaves the write into the cache to the library's kernel.  Its result depends on the positions
    themselves, not on their differences: the case that starts at position 17 shows that the encoding sees 17 + i."""
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import build_mixer

    register_toy_encodings()
    nheads, kvheads, hd, n, dtype = 4, 2, 32, 90, torch.float32
    x = torch.randn(n, nheads * hd, generator=torch.Generator().manual_seed(13))
    for kind, first in (("toy_linear_frequencies", 0), ("toy_added_wave", 0), ("toy_added_wave", 17)):
        spec = MixerSpec("attention", dim=nheads * hd, nheads=nheads, kvheads=kvheads, head_dim=hd,
                         position=PositionSpec(kind, head_dim=hd, theta=0.3))
        mixer = build_mixer(spec)
        assert type(mixer.position).__name__ == {"toy_linear_frequencies": "LinearFrequencies", "toy_added_wave": "AddedWave"}[kind]
        w = fill(mixer, dtype, 12, scale=0.08)
        qkv = x.double() @ w["in_proj.qkv_fused.weight"].T
        q, k, v = qkv.split([nheads * hd, kvheads * hd, kvheads * hd], -1)
        pos = torch.arange(n) + first
        if kind == "toy_linear_frequencies":
            inv = mixer.position.frequencies().double()
            q, k = pl.plain_rope(q.view(n, nheads, hd), pos, inv), pl.plain_rope(k.view(n, kvheads, hd), pos, inv)
            # the toy's frequencies are not the ordinary ones, so the agreement below is not an accident
            assert not torch.allclose(inv.float(), pl.plain_rope_inv_freq(hd, 10000.0).float())
        else:
            q, k = q.view(n, nheads, hd) + wave(pos, hd)[:, None], k.view(n, kvheads, hd) + wave(pos, hd)[:, None]
        want = pl.plain_attention(q, k, v.view(n, kvheads, hd)).reshape(n, -1) @ w["dense.weight"].T
        close(_run_mixer_in_three_steps(mixer, x, dtype, first), want, dtype)
        if first:  # and from position 0 the rows would have been others
            q0, k0 = q - wave(pos, hd)[:, None] + wave(pos - first, hd)[:, None], k - wave(pos, hd)[:, None] + wave(pos - first, hd)[:, None]
            other = pl.plain_attention(q0, k0, v.view(n, kvheads, hd)).reshape(n, -1) @ w["dense.weight"].T
            assert (other - want).abs().max() > 100 * 2e-5


def test_an_encoding_that_adds_to_the_scores_is_refused_by_the_built_in_mixer():
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import PositionEncoding, build_mixer, register_position, registered

    class Slopes(PositionEncoding):
        def score_bias(self):
            return torch.ones(4)

    if "toy_slopes" not in registered("position"):
        register_position("toy_slopes", Slopes)
    with pytest.raises(ValueError, match="adds to the attention scores"):
        build_mixer(MixerSpec("attention", dim=64, nheads=4, kvheads=2, head_dim=16, position=PositionSpec("toy_slopes")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_attention_of_a_sequence_that_starts_at_another_position(dtype):
    """The rotation sees position 300 + i while the cache holds the tokens from its place 0 on.  (Rotary scores
    depend on differences of positions only, so this shows no more than that q and k are turned by the same
    positions and stored at the right places; the toy encoding above shows the positions themselves.)"""
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import build_mixer

    nheads, kvheads, hd, n, theta = 4, 2, 32, 90, 10000.0
    mixer = build_mixer(MixerSpec("attention", dim=nheads * hd, nheads=nheads, kvheads=kvheads, head_dim=hd,
                                  position=PositionSpec("rope", head_dim=hd, theta=theta)))
    w = fill(mixer, dtype, 21, scale=0.2)
    x = torch.randn(n, nheads * hd, generator=torch.Generator().manual_seed(22)).to(dtype)
    want = plain_mixer(w, x.double(), nheads, kvheads, hd, theta, 0, torch.arange(n) + 300)
    close(_run_mixer_in_three_steps(mixer, x, dtype, 300), want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 40])
def test_feed_forward_part_alone(dtype, rows):
    from fms_b200.config import FeedForwardSpec
    from fms_b200.parts import build_feed_forward

    ff = build_feed_forward(FeedForwardSpec("glu", dim=96, hidden=328, activation="swish"))
    w = fill(ff, dtype, 4, scale=0.1)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, 96, generator=g).to(dtype)
    gate, up = w["wg1_fused.weight"][:328], w["wg1_fused.weight"][328:]
    want = pl.plain_swiglu_ffn(x.double(), gate, up, w["w2.weight"])
    close(ff.forward(x.cuda()), want, dtype)
    with pytest.raises(ValueError):
        build_feed_forward(FeedForwardSpec("glu", dim=8, hidden=8, activation="mish"))


# ---------------------------------------------------------------------------------------------------
# toy parts, defined in this test only
# ---------------------------------------------------------------------------------------------------
def register_toys():
    from fms_b200.cache import StateRequest
    from fms_b200.parts import Linear, Part, register_feed_forward, register_mixer, registered

    class DecayMixer(Part):
        """y_t = W s_t with s_t = decay * s_{t-1} + x_t: a mixer whose only memory is a state vector per
        sequence.  Written with torch operations: it is a test's toy, not a kernel."""

        def __init__(self, spec):
            super().__init__()
            self.dim = spec.dim
            self.decay = dict(spec.options)["decay"]
            self.out = self.add("out", Linear(spec.dim, spec.dim))

        def cache_request(self):
            return StateRequest((self.dim,), torch.float32, name="decay_state")

        def forward(self, x, batch, view, writes_cache=True):
            slots = batch.slots.long()
            if batch.decode:  # one token per sequence; no host synchronisation, so that it can be captured
                s = view.state[slots] * self.decay + x.float()
                if writes_cache:
                    view.state[slots] = s
                return self.out.forward(s.to(x.dtype))
            rows, at = [], 0
            for i, n in enumerate(batch.num_new):
                s = view.state[slots[i]].clone()
                for t in range(n):
                    s = s * self.decay + x[at + t].float()
                    rows.append(s)
                at += n
                if writes_cache:
                    view.state[slots[i]] = s
            return self.out.forward(torch.stack(rows).to(x.dtype))

    class TopOneExperts(Part):
        """A feed-forward with routing: each token goes to the expert with the largest router logit (router
        logits in float32) and is scaled by the softmax weight of that expert."""

        def __init__(self, spec):
            super().__init__()
            self.n = dict(spec.options)["experts"]
            self.router = self.add("router", Linear(spec.dim, self.n))
            self.experts = [self.add(f"expert{i}", Linear(spec.dim, spec.dim)) for i in range(self.n)]

        def forward(self, x):
            logits = x.float() @ self.router.tensor("weight").float().T
            weight, choice = torch.softmax(logits, -1).max(-1)
            out = torch.zeros_like(x)
            for i, e in enumerate(self.experts):
                out = out + torch.where((choice == i)[:, None], e.forward(x), torch.zeros_like(x))
            return (out.float() * weight[:, None]).to(x.dtype)

    if "toy_decay" not in registered("mixer"):
        register_mixer("toy_decay", DecayMixer)
        register_feed_forward("toy_experts", TopOneExperts)


def toy_model(dtype, seed=7):
    """A two-layer decoder: layer 0 is Llama's attention + SwiGLU, layer 1 the toy mixer + the toy experts;
    the schedule runs layer 0, layer 1, and layer 0 again, the second time reading the cache of the first."""
    from fms_b200.config import (BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec)
    from fms_b200.models.base import Model
    from fms_b200.weights import RandomSource, TensorLayout

    register_toys()
    dim, vocab = 64, 97
    norm = NormSpec("rmsnorm", dim, 1e-5)
    attn = BlockSpec(
        MixerSpec("attention", dim=dim, nheads=4, kvheads=2, head_dim=16, position=PositionSpec("rope", head_dim=16)),
        FeedForwardSpec("glu", dim=dim, hidden=96), norm, norm)
    toy = BlockSpec(MixerSpec("toy_decay", dim=dim, options=(("decay", 0.5),)),
                    FeedForwardSpec("toy_experts", dim=dim, hidden=0, options=(("experts", 3),)), norm, norm)
    spec = DecoderSpec(vocab_size=vocab, dim=dim, layers=(attn, toy),
                       schedule=(LayerCall(0), LayerCall(1), LayerCall(0, cache_of=0, writes_cache=False)),
                       final_norm=norm, tie_head=True, max_positions=256)

    class Toy(Model):
        architecture = "toy_architecture_of_a_test"
        default_source = "native"

        def decoder_spec(self):
            return spec

    from fms_b200.engine.decoder import Decoder

    layout = [TensorLayout(n, d.shape, "gain" if d.role == "vector" else "matrix")
              for n, _, _, d in Decoder(spec, dtype).named_decls()]
    model = Toy(config=None)
    model.load(RandomSource(layout, seed, dtype=torch.bfloat16, device="cpu", std=0.08), "native", "cuda", dtype)
    return model, spec


def plain_toy(model, ids):
    """The toy decoder restated in float64 from the model's own tensors."""
    w = {k: v.double().cpu() for k, v in model.state_dict().items()}
    n = len(ids)
    x = w["base_model.embedding.weight"][torch.tensor(ids)]
    pos = torch.arange(n)

    def attn_block(x, kv=None):
        """Layer 0; with ``kv`` the keys and values of an earlier call are read instead of its own."""
        p = "base_model.layers.0."
        h = pl.plain_rmsnorm(x, w[p + "ln.weight"], 1e-5)
        qkv = h @ w[p + "attn.in_proj.qkv_fused.weight"].T
        q, k, v = qkv.split([64, 32, 32], -1)
        inv = pl.plain_rope_inv_freq(16, 10000.0)
        q = pl.plain_rope(q.view(n, 4, 16), pos, inv)
        if kv is None:
            kv = (pl.plain_rope(k.view(n, 2, 16), pos, inv), v.view(n, 2, 16))
        a = pl.plain_attention(q, kv[0], kv[1]).reshape(n, -1) @ w[p + "attn.dense.weight"].T
        x = x + a
        h = pl.plain_rmsnorm(x, w[p + "ff_ln.weight"], 1e-5)
        gu = w[p + "ff_sub_layer.wg1_fused.weight"]
        return x + pl.plain_swiglu_ffn(h, gu[:96], gu[96:], w[p + "ff_sub_layer.w2.weight"]), kv

    def toy_block(x):
        p = "base_model.layers.1."
        h = pl.plain_rmsnorm(x, w[p + "ln.weight"], 1e-5)
        s, rows = torch.zeros(64, dtype=torch.float64), []
        for t in range(n):
            s = 0.5 * s + h[t]
            rows.append(s)
        x = x + torch.stack(rows) @ w[p + "attn.out.weight"].T
        h = pl.plain_rmsnorm(x, w[p + "ff_ln.weight"], 1e-5)
        weight, choice = torch.softmax(h @ w[p + "ff_sub_layer.router.weight"].T, -1).max(-1)
        out = torch.stack([h[t] @ w[p + f"ff_sub_layer.expert{int(choice[t])}.weight"].T for t in range(n)])
        return x + out * weight[:, None]

    x, kv = attn_block(x)
    x, _ = attn_block(toy_block(x), kv)  # the schedule's third call reads the first call's cache
    x = pl.plain_rmsnorm(x, w["base_model.dec_norm.weight"], 1e-5)
    return x @ w["base_model.embedding.weight"].T


def test_toy_mixer_with_state_and_routed_feed_forward_are_registered_built_and_stepped():
    """float32 only: the toy's torch products are not the point, the assembly is."""
    torch.backends.cuda.matmul.allow_tf32 = False
    model, spec = toy_model(torch.float32)
    engine = model.new_engine(max_tokens=512, max_slots=3)
    kinds = [type(g).__name__ for g in engine.cache.groups]
    assert kinds == ["KVGroup", "StateGroup"]  # the toy's state got storage of its own
    g = torch.Generator().manual_seed(8)
    reqs = [torch.randint(0, 97, (k,), generator=g).tolist() for k in (40, 9, 70)]
    want = [plain_toy(model, r) for r in reqs]
    # whole and alone
    for r, w in zip(reqs, want):
        (slot,) = engine.begin(1)
        close(engine.step([slot], [r], [list(range(len(r)))]), w, torch.float32)
        engine.release([slot])
    # as a batch of unequal lengths: prompts, then one token each (the decode path, captured as a graph from
    # its second step on); slots are used again, so the state must have been zeroed
    cut = [len(r) - 6 for r in reqs]
    slots = engine.begin(3)
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], [list(range(c)) for c in cut])
    o = 0
    for i, c in enumerate(cut):
        got[i].append(lg[o:o + c])
        o += c
    for t in range(6):
        lg = engine.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)])
        for i in range(3):
            got[i].append(lg[i:i + 1])
    engine.release(slots)
    for i in range(3):
        close(torch.cat(got[i]), want[i], torch.float32)
    assert engine.graph_launches > 0


def test_toy_parts_in_decode_steps_that_are_filled_up_with_rows_in_the_spare_slot():
    """Ten sequences decode as twelve rows: the two filler rows go through the toy mixer too, where they find a row
    of state of their own (the spare slot's) and touch no sequence's; then seven of the ten go on."""
    torch.backends.cuda.matmul.allow_tf32 = False
    model, spec = toy_model(torch.float32)
    engine = model.new_engine(max_tokens=64 * 10, max_slots=10)
    g = torch.Generator().manual_seed(9)
    reqs = [torch.randint(0, 97, (int(k),), generator=g).tolist() for k in torch.randint(9, 40, (10,), generator=g)]
    want = [plain_toy(model, r) for r in reqs]
    slots = engine.begin(10)
    engine.step(slots, [r[:-8] for r in reqs], [[] for _ in reqs])
    live = list(range(10))
    for t in range(8):
        if t == 5:
            engine.release([slots[i] for i in (1, 4, 8)])
            live = [i for i in live if i not in (1, 4, 8)]
        lg = engine.step([slots[i] for i in live], [[reqs[i][len(reqs[i]) - 8 + t]] for i in live])
        for row, i in enumerate(live):
            close(lg[row:row + 1], want[i][len(reqs[i]) - 8 + t][None], torch.float32)
    assert sorted(engine._decode) == [7, 12] and engine.graph_launches > 0
    engine.release([slots[i] for i in live])
    engine.check()


# ---------------------------------------------------------------------------------------------------
# another arrangement of a layer, scales at both ends of the decoder, sequences that start at other positions
# ---------------------------------------------------------------------------------------------------
def register_toy_arrangement():
    from fms_b200.parts import Part, build_feed_forward, build_mixer, build_norm, register_block, registered

    class ParallelBlock(Part):
        """x += r * (mixer(norm(x)) + feed_forward(norm(x))): one norm, both sublayers beside one another, and a
        multiplier r on what they add (``BlockSpec.options``)."""

        def __init__(self, spec):
            super().__init__()
            self.norm = self.add("norm", build_norm(spec.mixer_norm))
            self.mixer = self.add("mixer", build_mixer(spec.mixer))
            self.feed_forward = self.add("ff", build_feed_forward(spec.feed_forward))
            self.multiplier = dict(spec.options)["residual_multiplier"]

        def cache_request(self):
            return self.mixer.cache_request()

        def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
            h = self.norm.apply(residual, pending, dtype)
            both = self.mixer.forward(h, batch, cache_view, writes_cache).float() + self.feed_forward.forward(h).float()
            return (both * self.multiplier).to(dtype)

    if "toy_parallel" not in registered("block"):
        register_block("toy_parallel", ParallelBlock)


def parallel_toy_model(dtype, seed=9):
    from fms_b200.config import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec
    from fms_b200.engine.decoder import Decoder
    from fms_b200.models.base import Model
    from fms_b200.weights import RandomSource, TensorLayout

    register_toy_encodings()
    register_toy_arrangement()
    dim, vocab = 64, 89
    norm = NormSpec("rmsnorm", dim, 1e-5)
    block = BlockSpec(MixerSpec("attention", dim=dim, nheads=4, kvheads=2, head_dim=16,
                                position=PositionSpec("toy_added_wave", head_dim=16)),
                      FeedForwardSpec("glu", dim=dim, hidden=80), norm, norm, arrangement="toy_parallel",
                      options=(("residual_multiplier", 0.7),))
    spec = DecoderSpec(vocab_size=vocab, dim=dim, layers=(block, block), schedule=(LayerCall(0), LayerCall(1)),
                       final_norm=norm, tie_head=False, max_positions=512, embedding_scale=3.0, logit_scale=0.25)

    class ParallelToy(Model):
        architecture = "toy_parallel_architecture_of_a_test"
        default_source = "native"

        def decoder_spec(self):
            return spec

    layout = [TensorLayout(n, d.shape, "gain" if d.role == "vector" else "matrix")
              for n, _, _, d in Decoder(spec, dtype).named_decls()]
    model = ParallelToy(config=None)
    model.load(RandomSource(layout, seed, dtype=torch.bfloat16, device="cpu", std=0.1), "native", "cuda", dtype)
    return model


def plain_parallel_toy(model, ids, first_position):
    w = {k: v.double().cpu() for k, v in model.state_dict().items()}
    n = len(ids)
    pos = torch.arange(n) + first_position
    x = 3.0 * w["base_model.embedding.weight"][torch.tensor(ids)]
    for layer in (0, 1):
        p = f"base_model.layers.{layer}."
        h = pl.plain_rmsnorm(x, w[p + "norm.weight"], 1e-5)
        q, k, v = (h @ w[p + "mixer.in_proj.qkv_fused.weight"].T).split([64, 32, 32], -1)
        q, k = q.view(n, 4, 16) + wave(pos, 16)[:, None], k.view(n, 2, 16) + wave(pos, 16)[:, None]
        a = pl.plain_attention(q, k, v.view(n, 2, 16)).reshape(n, -1) @ w[p + "mixer.dense.weight"].T
        gu = w[p + "ff.wg1_fused.weight"]
        x = x + 0.7 * (a + pl.plain_swiglu_ffn(h, gu[:80], gu[80:], w[p + "ff.w2.weight"]))
    x = pl.plain_rmsnorm(x, w["base_model.dec_norm.weight"], 1e-5)
    return 0.25 * (x @ w["head.weight"].T)


def test_another_arrangement_scales_and_sequences_that_start_at_other_positions():
    """A decoder defined here: both layers in a parallel arrangement registered by this test (one norm, mixer and
    feed-forward beside one another, a residual multiplier), a position encoding that shows absolute positions, a
    scale on the embedding and one on the logits.  Three sequences start at positions 0, 5 and 130; prompts in one
    step, then one token each (the decode arrays and the captured graph carry the positions too)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    model = parallel_toy_model(torch.float32)
    engine = model.new_engine(max_tokens=512, max_slots=3)
    g = torch.Generator().manual_seed(8)
    reqs = [torch.randint(0, 89, (k,), generator=g).tolist() for k in (40, 9, 70)]
    firsts = [0, 5, 130]
    want = [plain_parallel_toy(model, r, f) for r, f in zip(reqs, firsts)]
    assert (plain_parallel_toy(model, reqs[2], 0) - want[2]).abs().max() > 1e-2  # the start does matter
    cut = [len(r) - 6 for r in reqs]
    slots = engine.begin(3, first_positions=firsts)
    got = [[] for _ in reqs]
    lg = engine.step(slots, [r[:c] for r, c in zip(reqs, cut)], [list(range(c)) for c in cut])
    o = 0
    for i, c in enumerate(cut):
        got[i].append(lg[o:o + c])
        o += c
    for t in range(6):
        lg = engine.step(slots, [[r[c + t]] for r, c in zip(reqs, cut)])
        for i in range(3):
            got[i].append(lg[i:i + 1])
    engine.release(slots)
    engine.check()
    assert engine.graph_launches > 0
    for i in range(3):
        close(torch.cat(got[i]), want[i], torch.float32)
    # the same slots again, from position 0: nothing of the offsets is left
    slots = engine.begin(1)
    close(engine.step(slots, [reqs[2]], [list(range(70))]), plain_parallel_toy(model, reqs[2], 0), torch.float32)
    engine.release(slots)
