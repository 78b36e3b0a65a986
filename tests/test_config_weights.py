"""Configuration, registry, checkpoint reading and its errors (CPU)."""
import json
import os
import struct

import pytest
import torch

from tiny_models import TINY, TINY_A, TINY_B, tiny_tensors, write_folder


def test_config_from_config_json_keys():
    from fms_b200.models.llama import LLaMA

    c = LLaMA.config_from_json(TINY_B)
    assert (c.src_vocab_size, c.emb_dim, c.nheads, c.kvheads, c.nlayers) == (384, 96, 3, 1, 3)
    assert (c.ffn_hidden, c.norm_eps, c.rope_theta, c.max_expected_seq_len, c.tie_heads) == (256, 1e-6, 500000.0, 128, True)
    assert c.head_dim == 32 and c.n_kvheads == 1
    # transformers 5 folds rope keys into rope_parameters (param_builders.py:18-34)
    c2 = LLaMA.config_from_json({**TINY_A, "rope_theta": None, "rope_parameters": {"rope_theta": 123.0}})
    assert c2.rope_theta == 123.0
    for bad in ({"architectures": ["MistralForCausalLM"]}, {"head_dim": 99}, {"hidden_act": "gelu"}):
        with pytest.raises(ValueError):
            LLaMA.config_from_json({**TINY_A, **bad})
    with pytest.raises(ValueError, match="lacks"):
        LLaMA.config_from_json({k: v for k, v in TINY_A.items() if k != "rms_norm_eps"})


def test_config_defaults_and_reference_rounding_of_hidden_size():
    from fms_b200.models.llama import LLaMAConfig

    assert LLaMAConfig().ffn_hidden == 11008  # 7B: 8/3 * 4096 rounded up to 256
    assert LLaMAConfig(emb_dim=5120, nheads=40).ffn_hidden == 13824
    assert LLaMAConfig(hidden_grow_factor=3.5, multiple_of=1024).ffn_hidden == 14336
    with pytest.raises(ValueError):
        LLaMAConfig(emb_dim=100, nheads=3)
    with pytest.raises(ValueError):
        LLaMAConfig(nheads=32, kvheads=5)


def test_config_json_round_trip_and_updated(tmp_path):
    from fms_b200.models.llama import LLaMAConfig

    c = LLaMAConfig(src_vocab_size=331, emb_dim=240, nheads=5, nlayers=2, rope_scaling={"rope_type": "llama3"})
    c.save(tmp_path / "c.json")
    assert LLaMAConfig.load(tmp_path / "c.json") == c
    d = c.updated(nlayers=7, not_a_field=1)
    assert d.nlayers == 7 and c.nlayers == 2
    d.rope_scaling["x"] = 1
    assert "x" not in c.rope_scaling  # a deep copy
    # unknown keys of a JSON file are ignored
    with open(tmp_path / "d.json", "w") as f:
        json.dump({**c.as_dict(), "something_else": 3}, f)
    assert LLaMAConfig.load(tmp_path / "d.json") == c


def test_registry():
    from fms_b200 import models

    assert "llama" in models.list_models()
    assert {"micro", "7b", "13b", "70b", "3-8b"} <= set(models.list_variants("llama"))
    with pytest.raises(KeyError):
        models.list_variants("no_such_architecture")
    with pytest.raises(KeyError):
        models.register_model("llama", "micro", lambda: None)
    with pytest.raises(KeyError):
        models.get_model("llama", "no_such_variant", device_type="cpu")
    with pytest.raises(KeyError):
        models.get_model("no_such_architecture", "x", device_type="cpu")
    m = models.get_model("llama", "micro", device_type="cpu", data_type="fp32", nlayers=1)
    assert m.config.nlayers == 1 and m.config.emb_dim == 192
    with pytest.raises(NotImplementedError):  # the reference's parameters for several devices: one GPU here
        models.get_model("llama", "micro", device_type="cpu", distributed_strategy="tp")
    # a head size that the kernels do not take is refused when the model is built, in words
    with pytest.raises(ValueError, match="head size 24 is not supported: a multiple of 16 up to 256"):
        models.get_model("llama", "micro", device_type="cpu", data_type="fp32", nlayers=1, emb_dim=72, nheads=3)
    with pytest.raises(ValueError, match="head size 512"):
        models.get_model("llama", "micro", device_type="cpu", data_type="fp32", nlayers=1, emb_dim=1024, nheads=2)


def test_state_dict_names_are_the_references(tmp_path):
    """The names the reference's Llama has (tests/resources/expectations/models.test_llama.TestLlama2
    .test_model_weight_keys lists them): fused qkv and gate/up."""
    from fms_b200.models import get_model

    m = get_model("llama", "micro", device_type="cpu", data_type="fp32", nlayers=1)
    assert sorted(m.state_dict()) == sorted([
        "base_model.embedding.weight", "base_model.dec_norm.weight", "head.weight",
        "base_model.layers.0.ln.weight", "base_model.layers.0.ff_ln.weight",
        "base_model.layers.0.attn.in_proj.qkv_fused.weight", "base_model.layers.0.attn.dense.weight",
        "base_model.layers.0.ff_sub_layer.wg1_fused.weight", "base_model.layers.0.ff_sub_layer.w2.weight"])


def test_loading_a_folder_adapts_names_rows_and_fusion(tiny_folders):
    from fms_b200.models import get_model

    cfg, seed, gain_dtype = TINY["b"]
    hf = tiny_tensors(cfg, seed, gain_dtype)
    m = get_model("hf_pretrained", model_path=tiny_folders["b"], device_type="cpu", data_type="bf16")
    sd = m.state_dict()
    assert "head.weight" not in sd and m.decoder.head_weight() is sd["base_model.embedding.weight"]  # tied
    hd, h, kv = 32, 3, 1
    qkv = sd["base_model.layers.1.attn.in_proj.qkv_fused.weight"]
    q_hf = hf["model.layers.1.self_attn.q_proj.weight"]
    # row 2i of a head is HF's row i, row 2i+1 is HF's row hd/2 + i (fms/models/llama.py:730-736)
    assert torch.equal(qkv[0], q_hf[0]) and torch.equal(qkv[1], q_hf[hd // 2]) and torch.equal(qkv[2], q_hf[1])
    assert torch.equal(qkv[(h + kv) * hd:], hf["model.layers.1.self_attn.v_proj.weight"])  # v untouched, last
    gu = sd["base_model.layers.2.ff_sub_layer.wg1_fused.weight"]
    assert torch.equal(gu[:256], hf["model.layers.2.mlp.gate_proj.weight"])  # gate first
    assert torch.equal(gu[256:], hf["model.layers.2.mlp.up_proj.weight"])
    # dtypes: matrices stay bfloat16; the gains of this folder are stored in 32-bit and stay so
    assert qkv.dtype == torch.bfloat16 and sd["base_model.layers.0.ln.weight"].dtype == torch.float32
    m32 = get_model("hf_pretrained", model_path=tiny_folders["b"], device_type="cpu", data_type="fp32")
    assert all(t.dtype == torch.float32 for t in m32.state_dict().values())
    ma = get_model("hf_pretrained", model_path=tiny_folders["a"], device_type="cpu", data_type="bf16")
    assert ma.state_dict()["base_model.layers.0.ln.weight"].dtype == torch.bfloat16  # stored in bfloat16
    assert "head.weight" in ma.state_dict()


def test_kept_dtype_rule():
    from fms_b200.weights import kept_dtype

    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert kept_dtype("matrix", bf, bf) == bf and kept_dtype("matrix", f16, bf) == bf
    assert kept_dtype("matrix", f32, bf) == f32 and kept_dtype("vector", f32, bf) == f32
    assert kept_dtype("matrix", bf, f32) == f32
    assert kept_dtype("table", torch.int64, bf) == torch.int32 and kept_dtype("vector", torch.int64, f32) == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    t = tiny_tensors(TINY_A, 0)
    del t["model.layers.1.mlp.down_proj.weight"]                      # missing
    del t["model.layers.0.self_attn.k_proj.weight"]                   # breaks the qkv fusion of layer 0
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # known and ignored
    t["model.extra.weight"] = torch.zeros(3)                           # unexpected
    t["model.norm.weight"] = torch.zeros(65)                           # wrong shape
    folder = write_folder(str(tmp_path / "broken"), TINY_A, t)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    err = e.value
    assert "base_model.layers.1.ff_sub_layer.w2.weight" in err.missing
    assert "base_model.layers.0.attn.in_proj.qkv_fused.weight" in err.missing
    assert "model.extra.weight" in err.unexpected
    assert "base_model.layers.0.attn.in_proj.query.weight" in err.unexpected
    assert not any("inv_freq" in n for n in err.unexpected)
    assert [w[0] for w in err.wrong_shapes] == ["base_model.dec_norm.weight"]
    text = str(err)
    assert "missing tensors (2)" in text and "unexpected tensors" in text and "checkpoint (65,), model (64,)" in text


def test_untied_model_without_head_is_an_error_and_tied_with_head_is_fine(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    t = tiny_tensors(TINY_A, 0)
    del t["lm_head.weight"]
    with pytest.raises(WeightError, match="head.weight"):
        get_model("hf_pretrained", model_path=write_folder(str(tmp_path / "a"), TINY_A, t), device_type="cpu")
    t = tiny_tensors(TINY_B, 1)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    get_model("hf_pretrained", model_path=write_folder(str(tmp_path / "b"), TINY_B, t), device_type="cpu")


def test_safetensors_reader_and_writer(tmp_path):
    from fms_b200.weights import SafetensorsError, SafetensorsFile, find_checkpoint_files, write_safetensors
    from safetensors.torch import load_file, save_file

    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(2, 2, 2), "empty": torch.zeros(0, 4)}
    ours = str(tmp_path / "ours.safetensors")
    write_safetensors(ours, tensors)
    back = load_file(ours)  # the package reads what we write
    assert all(torch.equal(back[k], v) for k, v in tensors.items())
    theirs = str(tmp_path / "theirs.safetensors")
    save_file(tensors, theirs)
    f = SafetensorsFile(theirs)  # and we read what the package writes
    assert sorted(f.keys()) == sorted(tensors)
    assert all(torch.equal(f.get(k), v) and f.spec(k) == (v.dtype, tuple(v.shape)) for k, v in tensors.items())
    # broken files
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(bad))
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(bad))
    bad.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(bad))
    with pytest.raises(FileNotFoundError, match="Can't find the requested checkpoint"):
        find_checkpoint_files(str(tmp_path / "nothing_here"))
    os.makedirs(tmp_path / "dir")
    with pytest.raises(FileNotFoundError):
        find_checkpoint_files(str(tmp_path / "dir"))


def test_sharded_checkpoint(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import write_safetensors

    t = tiny_tensors(TINY_A, 0)
    names = sorted(t)
    folder = tmp_path / "sharded"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as f:
        json.dump(TINY_A, f)
    for i in range(0, len(names), 5):
        write_safetensors(str(folder / f"model-{i:03d}.safetensors"), {k: t[k] for k in names[i:i + 5]})
    one = get_model("hf_pretrained", model_path=write_folder(str(tmp_path / "one"), TINY_A, t), device_type="cpu")
    many = get_model("hf_pretrained", model_path=str(folder), device_type="cpu")
    assert all(torch.equal(v, many.state_dict()[k]) for k, v in one.state_dict().items())


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.models.llama import LLaMA, LLaMAConfig
    from fms_b200.weights import SafetensorsFile, write_random_model

    arch = LLaMA(LLaMAConfig(src_vocab_size=331, emb_dim=96, nheads=6, kvheads=2, nlayers=2, hidden_dim=200,
                             max_expected_seq_len=128, tie_heads=True))
    a = write_random_model(str(tmp_path / "a"), arch.config_json(), arch.checkpoint_layout(), seed=3)
    b = write_random_model(str(tmp_path / "b"), arch.config_json(), arch.checkpoint_layout(), seed=3)
    c = write_random_model(str(tmp_path / "c"), arch.config_json(), arch.checkpoint_layout(), seed=4,
                           gain_dtype=torch.float32)
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert sorted(fa.keys()) == sorted(t.name for t in arch.checkpoint_layout())
    assert all(torch.equal(fa.get(k), fb.get(k)) for k in fa.keys())  # same seed, same weights
    assert not torch.equal(fa.get("model.embed_tokens.weight"), fc.get("model.embed_tokens.weight"))
    w = fa.get("model.layers.0.mlp.up_proj.weight").float()
    assert w.dtype == torch.float32 and abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    gain = fc.get("model.norm.weight")
    assert gain.dtype == torch.float32 and 0.9 <= gain.min() and gain.max() <= 1.1 and gain.std() > 0.02
    m = get_model("hf_pretrained", model_path=a, device_type="cpu")  # the folder is a model like any other
    assert m.config.ffn_hidden == 200 and m.config.tie_heads
    # no model_path: random weights straight into the model, through the same adapter
    r1 = get_model("llama", "micro", device_type="cpu", seed=9, nlayers=1)
    r2 = get_model("llama", "micro", device_type="cpu", seed=9, nlayers=1)
    assert all(torch.equal(v, r2.state_dict()[k]) for k, v in r1.state_dict().items())


def test_adapter_registry():
    from fms_b200.weights import get_adapted, list_sources, register_adapter, register_adapter_step

    assert {"hf", "fms"} <= set(list_sources("llama"))
    register_adapter_step("toy_arch", "double", lambda t, **kw: {k + k: v for k, v in t.items()})
    register_adapter("toy_arch", "src", ["double"])
    assert list(get_adapted("toy_arch", "src", {"a": torch.zeros(1)})) == ["aa"]
    assert list(get_adapted("toy_arch", "unknown_source", {"a": torch.zeros(1)})) == ["a"]  # identity
    with pytest.raises(KeyError):
        register_adapter_step("toy_arch", "double", lambda t: t)
    with pytest.raises(KeyError):
        register_adapter("toy_arch", "src", ["double"])
    with pytest.raises(KeyError):
        register_adapter("toy_arch", "other", ["no_such_step"])
    # the engine's own names load through the "fms" source (fusion only)
    fused = get_adapted("llama", "fms", {"x.ff_sub_layer.wg.weight": torch.ones(2, 3), "x.ff_sub_layer.w1.weight": torch.zeros(2, 3)})
    assert list(fused) == ["x.ff_sub_layer.wg1_fused.weight"] and fused["x.ff_sub_layer.wg1_fused.weight"][0, 0] == 1


def test_the_references_serialization_import_path(tiny_folders):
    """fms.utils.serialization's names (fms/utils/serialization.py:27-160, :292-316, :339-450) under the same path."""
    from fms_b200.utils.serialization import get_adapted, list_sources, load_state_dict

    assert "hf" in list_sources("llama")
    sd = load_state_dict(tiny_folders["a"])
    assert "model.embed_tokens.weight" in sd.keys() and sd.spec("model.norm.weight") == (torch.bfloat16, (64,))
    assert sd.get("model.norm.weight").shape == (64,)
    with pytest.raises(FileNotFoundError):
        load_state_dict("/no/such/checkpoint")
    assert callable(get_adapted)


def test_extend_adapter():
    """fms/utils/serialization.py:104-148: steps appended to a source that exists; the others stay."""
    from fms_b200.utils.serialization import extend_adapter, get_adapted, list_sources, register_adapter, register_adapter_step

    register_adapter_step("toy_arch2", "double", lambda t, **kw: {k + k: v for k, v in t.items()})
    register_adapter_step("toy_arch2", "upper", lambda t, **kw: {k.upper(): v for k, v in t.items()})
    register_adapter("toy_arch2", "src", ["double"])
    register_adapter("toy_arch2", "other", ["upper"])
    extend_adapter("toy_arch2", "src", ["upper"])
    assert list(get_adapted("toy_arch2", "src", {"a": torch.zeros(1)})) == ["AA"]
    assert list(get_adapted("toy_arch2", "other", {"a": torch.zeros(1)})) == ["A"]  # untouched, still there
    assert set(list_sources("toy_arch2")) == {"src", "other"}
    with pytest.raises(KeyError, match="must already be registered"):
        extend_adapter("toy_arch2", "no_such_source", ["upper"])
    with pytest.raises(KeyError, match="is not registered"):
        extend_adapter("toy_arch2", "src", ["no_such_step"])


def test_compute_dtype_without_data_type_is_the_checkpoints(tmp_path):
    """The matrix of fms tests/models/test_getmodel_datatype.py:17-85 for this library's two dtypes: no data_type means
    the dtype the checkpoint's matrices are stored in (fms/utils/serialization.py:679-687), a data_type is obeyed, and
    a checkpoint in float16 (or mixed) asks for one instead of being cast in silence."""
    from fms_b200.models import get_model

    base = tiny_tensors(TINY_A, 0, torch.float32)  # gains in float32, matrices in bfloat16

    def folder(name, cast):
        return write_folder(str(tmp_path / name), TINY_A, {k: (cast(k, v)) for k, v in base.items()})

    as_bf16 = folder("bf16", lambda k, v: v)
    as_fp32 = folder("fp32", lambda k, v: v.float())
    as_fp16 = folder("fp16", lambda k, v: v.half())
    mixed = folder("mixed", lambda k, v: v.float() if "o_proj" in k else v)

    def dtypes(model):
        sd = model.state_dict()
        return model.dtype, sd["base_model.layers.0.attn.dense.weight"].dtype, sd["base_model.dec_norm.weight"].dtype

    bf, f32 = torch.bfloat16, torch.float32
    assert dtypes(get_model("hf_pretrained", model_path=as_bf16, device_type="cpu")) == (bf, bf, f32)
    assert dtypes(get_model("hf_pretrained", model_path=as_fp32, device_type="cpu")) == (f32, f32, f32)
    assert dtypes(get_model("hf_pretrained", model_path=as_bf16, device_type="cpu", data_type="fp32")) == (f32, f32, f32)
    assert dtypes(get_model("hf_pretrained", model_path=as_fp16, device_type="cpu", data_type="bf16")) == (bf, bf, bf)
    assert dtypes(get_model("hf_pretrained", model_path=as_fp16, device_type="cpu", data_type="fp32")) == (f32, f32, f32)
    # a tensor stored in 32-bit stays so inside a bfloat16 model
    assert dtypes(get_model("hf_pretrained", model_path=mixed, device_type="cpu", data_type="bf16")) == (bf, f32, f32)
    for path in (as_fp16, mixed):
        with pytest.raises(ValueError, match="pass data_type"):
            get_model("hf_pretrained", model_path=path, device_type="cpu")
    # random weights: bfloat16 unless told otherwise
    assert get_model("llama", "tiny-a", device_type="cpu").dtype == bf
    assert get_model("llama", "tiny-a", device_type="cpu", data_type=torch.float32).dtype == f32


def test_the_references_own_initialisation():
    from fms_b200.models import get_model

    m = get_model("llama", "micro", device_type="cpu", data_type="fp32", init="fms", nlayers=1, seed=2)
    sd = m.state_dict()
    d, v = 192, 256
    assert torch.equal(sd["base_model.dec_norm.weight"], torch.ones(d))
    assert abs(sd["base_model.layers.0.attn.dense.weight"].std().item() - 0.02) < 0.002
    assert abs(sd["base_model.embedding.weight"].std().item() - d ** -0.5) < 0.1 * d ** -0.5
    assert abs(sd["head.weight"].std().item() - (d * v) ** -0.25) < 0.1 * (d * v) ** -0.25
    with pytest.raises(ValueError):
        get_model("llama", "micro", device_type="cpu", init="no_such_init")


def test_meta_named_checkpoint_loads_like_the_hf_one(tmp_path, tiny_folders):
    """fms/models/llama.py:618-645: Meta's own names (tok_embeddings, layers.N.attention.wq, feed_forward.w1/w3/w2,
    attention_norm, ffn_norm, norm, output); their q and k rows are adjacent rotary pairs already."""
    import plain_llama as pl
    from fms_b200.models import get_model
    from fms_b200.weights import list_sources

    assert "meta" in list_sources("llama")
    cfg, seed, gain_dtype = TINY["a"]
    hf = tiny_tensors(cfg, seed, gain_dtype)
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    meta = {"tok_embeddings.weight": hf["model.embed_tokens.weight"], "norm.weight": hf["model.norm.weight"],
            "output.weight": hf["lm_head.weight"], "rope.freqs": torch.zeros(hd // 2)}
    names = {"self_attn.q_proj": "attention.wq", "self_attn.k_proj": "attention.wk", "self_attn.v_proj": "attention.wv",
             "self_attn.o_proj": "attention.wo", "mlp.gate_proj": "feed_forward.w1", "mlp.up_proj": "feed_forward.w3",
             "mlp.down_proj": "feed_forward.w2", "input_layernorm": "attention_norm", "post_attention_layernorm": "ffn_norm"}
    for i in range(cfg["num_hidden_layers"]):
        for h_name, m_name in names.items():
            t = hf[f"model.layers.{i}.{h_name}.weight"]
            if h_name in ("self_attn.q_proj", "self_attn.k_proj"):
                t = pl.hf_rows_to_interleaved(t, hd)  # the layout Meta's checkpoints have
            meta[f"layers.{i}.{m_name}.weight"] = t
    folder = write_folder(str(tmp_path / "meta"), cfg, meta)
    a = get_model("llama", model_path=tiny_folders["a"], source="hf", device_type="cpu", data_type="bf16").state_dict()
    b = get_model("llama", model_path=folder, source="meta", device_type="cpu", data_type="bf16").state_dict()
    assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a)


def test_a_plugin_module_that_cannot_be_imported_is_named_in_the_error(tmp_path):
    """FMS_B200_PLUGINS: modules that register architectures or parts from outside the library."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    (tmp_path / "a_plugin_of_a_test.py").write_text(
        "from fms_b200 import models\nmodels.register_model('llama', 'from_a_plugin', lambda **kw: None)\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), root]), FMS_B200_PLUGINS="a_plugin_of_a_test")
    code = "from fms_b200 import models; print('from_a_plugin' in models.list_variants('llama'))"
    ok = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert ok.returncode == 0 and ok.stdout.strip() == "True", ok.stderr[-1000:]
    env["FMS_B200_PLUGINS"] = "a_plugin_of_a_test, no_such_module_anywhere"
    bad = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert bad.returncode != 0 and "no_such_module_anywhere" in bad.stderr and "FMS_B200_PLUGINS" in bad.stderr
