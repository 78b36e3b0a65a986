"""A whole architecture that only this file knows.  It has config.json keys of its own, checkpoint names of its own
(separate q, k, v and gate, up matrices that its adapter fuses), layers that differ from one another (feed-forward
sizes, a window on one of them), a tied head and a scale on the embedding.  The test registers it, writes a folder of
random weights, finds the model class again through the folder's config.json, and replays a trace through the trace
program's own loop and through ``generate``.  No file of the framework is changed for it: the registries are its only
way in."""
import dataclasses
import io
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu

ARCHITECTURE = "toy_stack_of_a_test"
CONFIG_JSON = {
    "architectures": ["ToyStackForTests"], "width": 48, "heads": 3, "groups": 1, "head_width": 16,
    "inner": [72, 40, 56], "windows": [0, 20, 0], "vocabulary": 61, "epsilon": 1e-4, "theta": 5000.0,
    "reach": 512, "embedding_multiplier": 2.0,
}


def register_toy_architecture():
    from fms_b200 import models
    from fms_b200.config import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec
    from fms_b200.models.base import Model
    from fms_b200.weights import TensorLayout, register_adapter, register_adapter_step

    if ARCHITECTURE in models.list_models():
        return

    @dataclasses.dataclass
    class ToyConfig:
        width: int
        heads: int
        groups: int
        head_width: int
        inner: tuple
        windows: tuple
        vocabulary: int
        epsilon: float
        theta: float
        reach: int
        embedding_multiplier: float

    class ToyStack(Model):
        architecture = ARCHITECTURE
        default_source = "toy"

        @classmethod
        def config_from_json(cls, values):
            keys = [f.name for f in dataclasses.fields(ToyConfig)]
            missing = [k for k in keys if k not in values]
            if missing:
                raise ValueError(f"config.json lacks {missing}")
            c = ToyConfig(**{k: values[k] for k in keys})
            c.inner, c.windows = tuple(c.inner), tuple(c.windows)
            if len(c.inner) != len(c.windows):
                raise ValueError("config.json: `inner` and `windows` name one value a layer")
            return c

        def config_json(self):
            return {"architectures": ["ToyStackForTests"], **dataclasses.asdict(self.config)}

        def decoder_spec(self):
            c = self.config
            norm = NormSpec("rmsnorm", c.width, c.epsilon)
            position = PositionSpec("rope", head_dim=c.head_width, theta=c.theta, max_positions=c.reach)
            layers = tuple(
                BlockSpec(MixerSpec("attention", dim=c.width, nheads=c.heads, kvheads=c.groups, head_dim=c.head_width,
                                    window=w, position=position),
                          FeedForwardSpec("glu", dim=c.width, hidden=f), norm, norm)
                for f, w in zip(c.inner, c.windows))
            return DecoderSpec(vocab_size=c.vocabulary, dim=c.width, layers=layers,
                               schedule=tuple(LayerCall(i) for i in range(len(layers))), final_norm=norm, tie_head=True,
                               max_positions=c.reach, embedding_scale=c.embedding_multiplier)

        def checkpoint_layout(self):
            c = self.config
            q, kv = c.heads * c.head_width, c.groups * c.head_width
            out = [TensorLayout("tok.weight", (c.vocabulary, c.width), "embedding"),
                   TensorLayout("last.gain", (c.width,), "gain")]
            for i, f in enumerate(c.inner):
                p = f"stack.{i}."
                out += [TensorLayout(p + "mix.q", (q, c.width), "matrix"), TensorLayout(p + "mix.k", (kv, c.width), "matrix"),
                        TensorLayout(p + "mix.v", (kv, c.width), "matrix"), TensorLayout(p + "mix.o", (c.width, q), "matrix"),
                        TensorLayout(p + "ffn.gate", (f, c.width), "matrix"), TensorLayout(p + "ffn.up", (f, c.width), "matrix"),
                        TensorLayout(p + "ffn.down", (c.width, f), "matrix"),
                        TensorLayout(p + "gain_a", (c.width,), "gain"), TensorLayout(p + "gain_b", (c.width,), "gain")]
            return out

    def to_engine_names(tensors, **kwargs):
        """Its checkpoints' names to the decoder's; q, k, v and gate, up become the fused matrices.  (The rotary pairs
        are adjacent dimensions in this architecture's checkpoints, as in the kernels: no rows are moved.)"""
        out = {}
        for name, t in tensors.items():
            if name == "tok.weight":
                out["base_model.embedding.weight"] = t
            elif name == "last.gain":
                out["base_model.dec_norm.weight"] = t
            elif not name.startswith("stack."):
                out[name] = t  # not a name of this architecture: the loader will say so
            elif name.endswith((".mix.k", ".mix.v", ".ffn.up")):
                continue  # taken with their partner below
            else:
                i = name.split(".")[1]
                p, e = f"stack.{i}.", f"base_model.layers.{i}."
                if name == p + "mix.q":
                    out[e + "attn.in_proj.qkv_fused.weight"] = torch.cat([t, tensors[p + "mix.k"], tensors[p + "mix.v"]])
                elif name == p + "ffn.gate":
                    out[e + "ff_sub_layer.wg1_fused.weight"] = torch.cat([t, tensors[p + "ffn.up"]])
                else:
                    out[e + {"mix.o": "attn.dense.weight", "ffn.down": "ff_sub_layer.w2.weight", "gain_a": "ln.weight",
                             "gain_b": "ff_ln.weight"}[name[len(p):]]] = t
        return out

    models.register_architecture(ARCHITECTURE, ToyStack, config_json_names=("ToyStackForTests",))
    models.register_model(ARCHITECTURE, "small", lambda **kw: ToyStack(ToyStack.config_from_json({**CONFIG_JSON, **kw})))
    register_adapter_step(ARCHITECTURE, "toy_names_and_fusion", to_engine_names)
    register_adapter(ARCHITECTURE, "toy", ["toy_names_and_fusion"])


def plain_toy_logits(folder, ids):
    """The same architecture from its folder, whole sequences in float64, with the plain parts of tests/plain_llama.py."""
    c, tensors = pl.read_model_folder(folder)
    w = {k: v.double() for k, v in tensors.items()}
    n, h, g, hd = len(ids), c["heads"], c["groups"], c["head_width"]
    positions = torch.arange(n)
    inv_freq = pl.plain_rope_inv_freq(hd, c["theta"])
    x = c["embedding_multiplier"] * pl.plain_embedding(torch.as_tensor(ids), w["tok.weight"])
    for i, window in enumerate(c["windows"]):
        p = f"stack.{i}."
        y = pl.plain_rmsnorm(x, w[p + "gain_a"], c["epsilon"])
        q = (y @ w[p + "mix.q"].T).view(n, h, hd)
        k = (y @ w[p + "mix.k"].T).view(n, g, hd)
        v = (y @ w[p + "mix.v"].T).view(n, g, hd)
        q, k = pl.plain_rope(q, positions, inv_freq), pl.plain_rope(k, positions, inv_freq)
        x = x + pl.plain_attention(q, k, v, window=window).reshape(n, -1) @ w[p + "mix.o"].T
        y = pl.plain_rmsnorm(x, w[p + "gain_b"], c["epsilon"])
        x = x + pl.plain_swiglu_ffn(y, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
    return pl.plain_rmsnorm(x, w["last.gain"], c["epsilon"]) @ w["tok.weight"].T


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from fms_b200.models import get_model
    from fms_b200.weights.random_init import write_random_model

    register_toy_architecture()
    model = get_model(ARCHITECTURE, "small", device_type="cuda", data_type="fp32", seed=3)  # random weights, no folder
    assert model.config.inner == (72, 40, 56)
    folder = str(tmp_path_factory.mktemp("toy") / "model")
    return write_random_model(folder, model.config_json(), model.checkpoint_layout(), seed=11, std=0.08)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_architecture_from_its_folder_through_the_trace_loop(toy_folder, tmp_path, dtype):
    from fms_b200.engine.trace import replay
    from fms_b200.models import get_model

    model = get_model("hf_pretrained", model_path=toy_folder, device_type="cuda", data_type=dtype)
    assert type(model).__name__ == "ToyStack" and model.architecture == ARCHITECTURE
    engine = model.new_engine(max_tokens=64 * 6, sampling=False)
    assert sorted(g.request.window for g in engine.cache.groups) == [0, 20]  # two groups of layers in the cache
    g = torch.Generator().manual_seed(5)
    reqs = {"a": torch.randint(0, 61, (90,), generator=g).tolist(), "b": torch.randint(0, 61, (37,), generator=g).tolist()}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:80], "want": list(range(80))},
                                      {"id": "b", "tokens": reqs["b"][:30], "want": [0, 29]}], "end": []}]
    for t in range(10):
        live = [("a", 80 + t)] + ([("b", 30 + t)] if 30 + t < 37 else [])
        steps.append({"step": t + 1, "entries": [{"id": r, "tokens": [reqs[r][p]], "want": [0]} for r, p in live],
                      "end": ["b"] if 30 + t == 36 else []})
    steps[-1]["end"] = ["a"]
    log = io.StringIO()
    replay(engine, io.StringIO("\n".join(json.dumps(s) for s in steps)), str(tmp_path), log)
    assert log.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    assert engine.cache.slots.n_held == 0
    want = {r: plain_toy_logits(toy_folder, ids) for r, ids in reqs.items()}
    tol = dict(atol=2e-4, rtol=1e-4) if dtype == "float32" else dict(atol=0.02 * want["a"].abs().max().item(), rtol=0.02)

    def written(step):
        return torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{step}.f32"), dtype="<f4").reshape(-1, 61).copy())

    first = written(0)
    torch.testing.assert_close(first[:80].double(), want["a"][:80], **tol)
    torch.testing.assert_close(first[80:].double(), want["b"][[0, 29]], **tol)
    for t in range(10):
        got = written(t + 1)
        torch.testing.assert_close(got[0].double(), want["a"][80 + t], **tol)
        if 30 + t < 37:
            torch.testing.assert_close(got[1].double(), want["b"][30 + t], **tol)


def test_a_toy_architecture_generates_through_the_entry_point(toy_folder):
    from fms_b200.engine.generation import generate
    from fms_b200.models import get_model

    model = get_model(ARCHITECTURE, model_path=toy_folder, device_type="cuda", data_type="fp32")
    prompt = [7, 3, 50, 21, 9]
    out = generate(model, torch.tensor(prompt), max_new_tokens=6, do_sample=False)
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(plain_toy_logits(toy_folder, ids)[-1].argmax()))
    assert out.tolist() == ids


def test_a_checkpoint_of_the_toy_architecture_with_a_missing_and_a_misshapen_tensor_is_refused(toy_folder, tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError
    from fms_b200.weights.safetensors_io import write_safetensors

    _, tensors = pl.read_model_folder(toy_folder)
    del tensors["stack.1.gain_b"]
    tensors["stack.2.ffn.down"] = tensors["stack.2.ffn.down"][:, :-1].contiguous()
    tensors["stray"] = torch.zeros(3)
    os.makedirs(tmp_path / "broken")
    with open(os.path.join(toy_folder, "config.json")) as f, open(tmp_path / "broken" / "config.json", "w") as out:
        out.write(f.read())
    write_safetensors(str(tmp_path / "broken" / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=str(tmp_path / "broken"), device_type="cuda", data_type="fp32")
    text = str(e.value)
    assert "base_model.layers.1.ff_ln.weight" in text and "stray" in text and "base_model.layers.2.ff_sub_layer.w2.weight" in text


def test_the_trace_program_finds_the_toy_architecture_through_a_plugin_module(toy_folder, tmp_path):
    """bin/trace_run is a process of its own: it knows the architecture because FMS_B200_PLUGINS names a module that
    registers it (here a two-line module that calls this file's registration)."""
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    (tmp_path / "toy_plugin_of_a_test.py").write_text(
        "import test_toy_architecture_gpu as t\nt.register_toy_architecture()\n")
    ids = [3, 60, 17, 17, 42, 8, 0, 25]
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": ids[:5], "want": [0, 4]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": ids[5:6], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": ids[6:], "want": [1]}], "end": ["r"]}]
    env = dict(os.environ, FMS_B200_PLUGINS="toy_plugin_of_a_test",
               PYTHONPATH=os.pathsep.join([str(tmp_path), here, os.environ.get("PYTHONPATH", "")]))
    proc = subprocess.run(
        [sys.executable, os.path.join(os.path.dirname(here), "bin", "trace_run"), "--model", toy_folder, "--dtype", "float32",
         "--out", str(tmp_path / "out"), "--max-tokens", "64"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    want = plain_toy_logits(toy_folder, ids)
    got = torch.cat([torch.from_numpy(np.fromfile(tmp_path / "out" / f"{s}.f32", dtype="<f4").reshape(-1, 61).copy())
                     for s in range(3)])
    torch.testing.assert_close(got.double(), want[[0, 4, 5, 7]], atol=2e-4, rtol=1e-4)
    # without the plugin the program says which architectures it knows
    env.pop("FMS_B200_PLUGINS")
    proc = subprocess.run(
        [sys.executable, os.path.join(os.path.dirname(here), "bin", "trace_run"), "--model", toy_folder, "--dtype", "float32",
         "--out", str(tmp_path / "out2"), "--max-tokens", "64"], input="", capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode != 0 and "ToyStackForTests" in proc.stderr and "LlamaForCausalLM" in proc.stderr
