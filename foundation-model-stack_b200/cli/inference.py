"""Command line in the manner of the reference's ``scripts/inference.py`` (flags :23-113): load a model,
turn prompts into ids, generate, print.

    bin/fms_inference --architecture llama --variant micro --tokenizer char_tokenizer --prompt "Hello"
    bin/fms_inference --model_path /folder --model_source hf --prompt_ids 1,5,9 --max_new_tokens 20

Kept from the reference: --device_type, --architecture, --variant, --model_path, --model_source,
--tokenizer, --default_dtype, --batch_input (run all prompts as one batch), --context_file, --deterministic
(here: greedy).  Added: --prompt (repeatable), --prompt_ids, --max_new_tokens, --do_sample, --temperature,
--top_k, --seed, --eos_token_id, --timing.  Dropped, with what they selected gone: --no_use_cache,
--unfuse_weights, --compile, --compile_mode, --distributed, --attn_name.  --min_pad_length is kept with its
meaning: the prompts go through ``pad_input_ids`` and come back out of their padding, which changes no token.
"""
from __future__ import annotations

import argparse
import sys


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Generate text with a model of this library")
    p.add_argument("--device_type", type=str, default="cuda")
    p.add_argument("--architecture", type=str, default="llama", help="The model architecture")
    p.add_argument("--variant", type=str, default=None, help="The model variant (configuration)")
    p.add_argument("--model_path", type=str, default=None,
                   help="Folder (or file, or glob) of safetensors; with a config.json the configuration is read "
                        "from it.  Without it the weights are random.")
    p.add_argument("--model_source", type=str, default=None, help="Naming of the checkpoint: hf, meta or fms")
    p.add_argument("--tokenizer", type=str, default=None,
                   help='"char_tokenizer" or a folder with a tokenizer.json; without one give --prompt_ids')
    p.add_argument("--default_dtype", type=str, default=None, choices=["bf16", "fp32"],
                   help="Compute dtype; fp32 uses no reduced-precision product")
    p.add_argument("--batch_input", action="store_true", help="Run all prompts as one batch")
    p.add_argument("--min_pad_length", type=int, default=0,
                   help="Pad inputs to a minimum length. If any prompt is longer, padding will be determined by "
                        "the largest prompt")
    p.add_argument("--context_file", type=str, default=None, help="File whose text is put before every prompt")
    p.add_argument("--deterministic", action="store_true", help="Greedy decoding (the kernels are deterministic)")
    p.add_argument("--prompt", action="append", default=[], help="A prompt; may be given several times")
    p.add_argument("--prompt_ids", action="append", default=[], help="A prompt as comma-separated token ids")
    p.add_argument("--max_new_tokens", type=int, default=100)
    p.add_argument("--do_sample", action="store_true")
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top_k", type=int, default=10)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--eos_token_id", type=int, default=None)
    p.add_argument("--timing", type=str, default="", choices=["", "per-token", "e2e"])
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from ..models import get_model
    from ..utils.generation import generate, pad_input_ids, truncate_after_eos
    from ..utils.tokenizers import get_tokenizer

    tokenizer = get_tokenizer(args.tokenizer) if args.tokenizer else None
    prompts = []
    context = ""
    if args.context_file:
        with open(args.context_file, "r", encoding="utf-8") as f:
            context = f.read()
    for text in args.prompt:
        if tokenizer is None:
            print("--prompt needs --tokenizer; use --prompt_ids otherwise", file=sys.stderr)
            return 2
        prompts.append(tokenizer.encode(context + text, add_special_tokens=True))
    for ids in args.prompt_ids:
        prompts.append([int(x) for x in ids.split(",") if x.strip()])
    if not prompts:
        if tokenizer is None:
            print("give --prompt (with --tokenizer) or --prompt_ids", file=sys.stderr)
            return 2
        template = ("Below is an instruction that describes a task. Write a response that appropriately completes "
                    "the request.\n\n### Instruction:\n{}\n\n### Response:")
        prompts = [tokenizer.encode(context + template.format(t), add_special_tokens=True)
                   for t in ("Provide a list of instructions for preparing chicken soup.",
                             "Explain some popular greetings in Spanish.")]

    if args.variant is None and args.model_path is None:
        args.variant = "micro"
    print("loading model", file=sys.stderr)
    model = get_model(args.architecture, args.variant, model_path=args.model_path, source=args.model_source,
                      device_type=args.device_type, data_type=args.default_dtype, seed=args.seed)
    eos = args.eos_token_id if args.eos_token_id is not None else (tokenizer.eos_token_id if tokenizer else None)
    do_sample = args.do_sample and not args.deterministic
    groups = [prompts] if args.batch_input else [[p] for p in prompts]
    for group in groups:
        ids, padding = [torch.tensor(p) for p in group], None
        if args.min_pad_length > 0:
            ids, padding = pad_input_ids(ids, min_pad_length=args.min_pad_length)
        out = generate(model, ids, max_new_tokens=args.max_new_tokens,
                       do_sample=do_sample, temperature=args.temperature, top_k=args.top_k, seed=args.seed,
                       eos_token_id=eos, timing=args.timing, extra_kwargs=padding)
        if args.timing:
            out, times = out
            print(f"timing ({args.timing}): {[round(t * 1e3, 3) for t in times]} ms", file=sys.stderr)
        if padding is not None:  # out of the rectangle again: no padding in front, nothing after a stop token
            width = ids.shape[1]
            out = [torch.cat((row[width - len(p):width], truncate_after_eos(row[width:], eos)))
                   for row, p in zip(out, group)]
        for ids in out:
            ids = ids.tolist()
            print(tokenizer.decode(ids) if tokenizer else ",".join(str(i) for i in ids))
            print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
