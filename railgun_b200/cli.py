"""The command line: ``railgun generate`` and ``railgun random-weights``.

``generate`` keeps the reference's options and meanings
(crates/vllm-cli/src/generate.rs:29-53): ``--model/-m DIR``, ``--max-tokens``
(default 128), ``--temperature`` (default 0.0 = greedy; honoured here, the
reference parses and ignores it), ``--cuda-device N``, ``--show-token-ids``.  ``--random-weights SEED`` runs a
folder's config.json with seeded random weights.  Log messages are filtered by
``RAILGUN_LOG`` (default info), as the reference filters by an environment
variable (crates/vllm-cli/src/main.rs:40-49).
Prompts are token ids (``--prompt-ids 1,2,3;4,5``), or, as in the reference,
text (``--prompt/-p TEXT``) when the model folder holds a ``tokenizer.json``
(read with the ``tokenizers`` library, the one the reference's
RailgunTokenizer wraps, crates/vllm-models/src/tokenizer.rs:29-52: encode with
special tokens, decode skipping them; the tokenizer's end-of-sequence id, or
the configuration's, ends generation, generate.rs:83-85; the prompt is printed
with the generated text after it, generate.rs:99).  The engine options of the
reference's ``serve`` (crates/vllm-cli/src/serve.rs:44-77) are accepted with
their names and defaults.  It prints the generated ids and a ``[stats]`` line
with tokens per second, as the reference does (generate.rs:99-111).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="railgun", description="a small B200 inference engine")
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens from prompt token ids")
    g.add_argument("-m", "--model", required=True, help="model folder (config.json + *.safetensors)")
    what = g.add_mutually_exclusive_group(required=True)
    what.add_argument("--prompt-ids",
                      help="prompt token ids, comma separated; several prompts separated by ';'")
    what.add_argument("-p", "--prompt", help="prompt text (the model folder must hold a tokenizer.json)")
    g.add_argument("--max-tokens", type=int, default=128, help="maximum number of new tokens")
    g.add_argument("--temperature", type=float, default=0.0, help="sampling temperature (0.0 = greedy)")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--seed", type=int, default=0, help="seed of the requests' random draws")
    g.add_argument("--stop-token-ids", default="", help="comma separated ids that end generation")
    g.add_argument("--cuda-device", type=int, default=0, help="CUDA device ordinal (there is no CPU path)")
    g.add_argument("--show-token-ids", action="store_true", help="print prompt ids beside the generated ids")
    g.add_argument("--dtype", default="bf16", choices=["bf16", "f32", "bfloat16", "float32"])
    g.add_argument("--max-num-seqs", type=int, default=256)
    g.add_argument("--max-num-batched-tokens", type=int, default=4096)
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--num-gpu-blocks", type=int, default=1000)
    g.add_argument("--max-model-len", type=int, default=4096)
    g.add_argument("--max-prefill-chunk", type=int, default=0)
    g.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="ignore the folder's weights: draw them from SEED for its config.json (into a temporary folder)")

    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True, help="folder to write config.json and model.safetensors into")
    r.add_argument("--std", type=float, default=0.02)
    return ap


def _ids(text: str) -> list:
    return [int(t) for t in text.replace(" ", "").split(",") if t != ""]


def load_tokenizer(model_dir):
    """``tokenizer.json`` of the model folder (crates/vllm-models/src/tokenizer.rs:29-31)."""
    import os
    path = os.path.join(str(model_dir), "tokenizer.json")
    if not os.path.isfile(path):
        raise OSError(f"{path} does not exist (use --prompt-ids for a model without a tokenizer)")
    from tokenizers import Tokenizer
    try:
        return Tokenizer.from_file(path)
    except Exception as e:                                  # the library raises its own exception type
        raise ValueError(f"cannot read {path}: {e}") from e


def run_generate(args) -> int:
    from .engine.engine import Engine
    from .engine.request import SamplingParams

    tokenizer, stop_ids = None, _ids(args.stop_token_ids)
    if args.prompt is not None:
        try:
            tokenizer = load_tokenizer(args.model)
        except (OSError, ImportError, ValueError) as e:
            print(f"error: --prompt needs a tokenizer: {e}", file=sys.stderr)
            return 2
        prompts = [tokenizer.encode(args.prompt, add_special_tokens=True).ids]
        # the end-of-sequence id: the first of these names that the tokenizer knows, else the configuration's
        # (crates/vllm-models/src/tokenizer.rs:73-83, crates/vllm-cli/src/generate.rs:83-85)
        eos = next((tokenizer.token_to_id(n) for n in ("<|eot_id|>", "<|end_of_text|>", "</s>")
                    if tokenizer.token_to_id(n) is not None), None)
        if eos is None:
            from .config.registry import load_config
            stop_ids += [t for t in (load_config(args.model)[1].to_dict().get("eos_token_id") or []) if t not in stop_ids]
        elif eos not in stop_ids:
            stop_ids.append(eos)
    else:
        prompts = [_ids(p) for p in args.prompt_ids.split(";") if p.strip()]
    if not prompts or any(not p for p in prompts):
        print("error: the prompt needs at least one token", file=sys.stderr)
        return 2
    model_dir, scratch = args.model, None
    if args.random_weights is not None:
        import os
        import shutil
        import tempfile
        from .config.registry import load_config
        from .weights.random_init import write_random_model
        scratch = tempfile.mkdtemp(prefix="railgun_random_")
        write_random_model(load_config(args.model)[1], args.random_weights, scratch)
        shutil.copyfile(os.path.join(str(args.model), "config.json"), os.path.join(scratch, "config.json"))
        model_dir = scratch
    t0 = time.time()
    engine = Engine(model_dir, dtype=args.dtype, cuda_device=args.cuda_device, block_size=args.block_size,
                    num_gpu_blocks=args.num_gpu_blocks, max_num_seqs=args.max_num_seqs,
                    max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len,
                    max_prefill_chunk=args.max_prefill_chunk)
    load_ms = (time.time() - t0) * 1e3
    params = [SamplingParams(max_new_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                             top_k=args.top_k, stop_token_ids=stop_ids, seed=args.seed + i)
              for i in range(len(prompts))]
    t0 = time.time()
    outs = engine.generate(prompts, params)
    dt = time.time() - t0
    for p, o in zip(prompts, outs):
        if args.show_token_ids:
            print(f"prompt ids: {p}")
        if tokenizer is not None:
            print(args.prompt + tokenizer.decode(o.token_ids, skip_special_tokens=True))
        if tokenizer is None or args.show_token_ids:
            print(",".join(str(t) for t in o.token_ids))
        if o.error:
            print(f"[error] request {o.request_id}: {o.error}", file=sys.stderr)
    if scratch is not None:
        import shutil
        shutil.rmtree(scratch, ignore_errors=True)
    n = sum(len(o.token_ids) for o in outs)
    print(f"[stats] {n} tokens in {dt * 1e3:.1f} ms = {n / dt:.1f} tok/s (load {load_ms:.0f} ms)")
    return 0


def run_random_weights(args) -> int:
    from .config.base import read_json
    from .config.registry import architecture_of
    from .weights.random_init import write_random_model

    data = read_json(args.config)
    archs = data.get("architectures") or []
    if not archs:
        print("error: the config has no 'architectures'", file=sys.stderr)
        return 2
    arch = architecture_of(archs[0])
    out = write_random_model(arch.config_from_dict(data, args.config), args.seed, args.out, std=args.std)
    print(json.dumps({"written": str(out)}))
    return 0


def main(argv=None) -> int:
    args = make_parser().parse_args(argv)
    if args.command == "generate":
        return run_generate(args)
    return run_random_weights(args)


if __name__ == "__main__":
    sys.exit(main())
