"""Writes tests/golden/reference_logits.safetensors: the logits of the reference's own Llama
(fms.models.llama.LLaMA, loaded through its ``get_model(..., source="hf")`` path, float32, CPU) on the
tiny random models of tests/tiny_models.py, for whole prompts and for prompt + cached one-token steps.

Run once where the reference's sources are present:

    python tests/golden/make_golden.py /path/to/foundation-model-stack

The reference is not pip-installed there, and its ``fms/__init__.py`` asks importlib.metadata for the
version of "ibm-fms"; only that lookup is patched.  Nothing of the reference is modified or copied.
tests/test_plain_vs_golden.py compares the plain implementation with the stored file.

Also writes tests/golden/reference_padding.safetensors: what the reference's ``pad_input_ids``
(fms/utils/generation.py:16-109) returns for the prompts and settings of ``PADDING_CASES``, which
``fms_b200.utils.generation.pad_input_ids`` has to return too.
"""
import importlib.metadata as md
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


PADDING_PROMPTS = [[4], [1, 2, 3], [9, 10], [7, 7, 7, 7, 7, 7]]
# keyword arguments of pad_input_ids, by case
PADDING_CASES = {
    "default": {},
    "min_pad_length": {"min_pad_length": 9},
    "right": {"padding_side": "right", "pad_token_id": 3},
    "offset_not_causal": {"position_ids_offset": 2, "is_causal_mask": False, "pad_token_id": 11},
}


def padding_golden():
    from fms.utils.generation import pad_input_ids

    out = {}
    for name, kwargs in PADDING_CASES.items():
        ids, extra = pad_input_ids([torch.tensor(p) for p in PADDING_PROMPTS], **kwargs)
        out[f"{name}.ids"] = ids.to(torch.int32).contiguous()
        out[f"{name}.position_ids"] = extra["position_ids"].to(torch.int32).contiguous()
        mask = extra["mask"]
        assert ((mask == 0) | (mask == float("-inf"))).all()
        out[f"{name}.mask_is_zero"] = (mask == 0).to(torch.uint8).contiguous()
    return out


def main(reference_root: str):
    os.environ["HF_HUB_OFFLINE"] = "1"
    os.environ["TRANSFORMERS_OFFLINE"] = "1"
    orig = md.version
    md.version = lambda n: "0.0.0+ref" if n == "ibm-fms" else orig(n)
    sys.path.insert(0, reference_root)
    from fms.models import get_model
    from safetensors.torch import save_file

    from tiny_models import TINY, tiny_prompts, tiny_tensors_of, write_tiny

    out = {}
    for which in sorted(TINY):
        folder = write_tiny(tempfile.mkdtemp(), which)
        cfg = TINY[which][0]
        if cfg.get("rope_scaling"):
            # With transformers 5 the reference's "hf_pretrained" route finds config.json's rope_scaling folded into
            # rope_parameters, where it does not look for it (fms/models/hf/config_utils/param_builders.py:17-34),
            # and builds the model without the rescaling.  Its other route takes the configuration as keyword
            # arguments, the rescaling among them.
            model = get_model(
                "llama", "micro", model_path=folder, source="hf", data_type=torch.float32, device_type="cpu",
                src_vocab_size=cfg["vocab_size"], emb_dim=cfg["hidden_size"], nheads=cfg["num_attention_heads"],
                kvheads=cfg["num_key_value_heads"], nlayers=cfg["num_hidden_layers"],
                hidden_grow_factor=cfg["intermediate_size"] / cfg["hidden_size"], multiple_of=1,
                norm_eps=cfg["rms_norm_eps"], max_expected_seq_len=cfg["max_position_embeddings"],
                attn_bias=cfg["attention_bias"], mlp_bias=cfg["mlp_bias"], tie_heads=cfg["tie_word_embeddings"],
                rope_theta=cfg["rope_theta"], rope_scaling=cfg["rope_scaling"])
            assert type(model.base_model.rot_emb.rope_scaling).__name__ == "RopeLlama3ScalingImpl"
        else:
            model = get_model("hf_pretrained", model_path=folder, data_type=torch.float32, device_type="cpu")
        model.eval()
        tensors = tiny_tensors_of(which)
        out[f"{which}.weight_abs_sum"] = torch.stack(
            [t.float().abs().sum() for _, t in sorted(tensors.items())]
        ).sum().reshape(1).double()
        for n, prompt in enumerate(tiny_prompts(which)):
            ids = torch.tensor([prompt])
            with torch.no_grad():
                whole = model(ids)[0]
                # the same prompt: all but the last 4 tokens at once, then one token per call from the cache
                cut = max(1, len(prompt) - 4)
                lg, cache = model(ids[:, :cut], use_cache=True)
                parts = [lg[0]]
                for t in range(cut, len(prompt)):
                    lg, cache = model(ids[:, t : t + 1], past_key_value_states=cache, use_cache=True)
                    parts.append(lg[0])
                stepped = torch.cat(parts, 0)
            assert (whole - stepped).abs().max() < 1e-4, (which, n, (whole - stepped).abs().max())
            # stored: the first 4 and the last 12 positions (the file stays small)
            sel = sorted(set(range(min(len(prompt), 4))) | set(range(max(0, len(prompt) - 12), len(prompt))))
            out[f"{which}.{n}.ids"] = torch.tensor(prompt, dtype=torch.int32)
            out[f"{which}.{n}.positions"] = torch.tensor(sel, dtype=torch.int32)
            out[f"{which}.{n}.logits"] = whole[sel].float().contiguous()
            print(which, n, len(prompt), "max|whole - stepped| =", (whole - stepped).abs().max().item())
    save_file(out, os.path.join(HERE, "reference_logits.safetensors"))
    print("wrote", os.path.join(HERE, "reference_logits.safetensors"))
    save_file(padding_golden(), os.path.join(HERE, "reference_padding.safetensors"))
    print("wrote", os.path.join(HERE, "reference_padding.safetensors"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of a checkout of foundation-model-stack>")
    main(sys.argv[1])
