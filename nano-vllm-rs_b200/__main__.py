"""Command line of the package:

    python -m nano_vllm_rs_b200 architectures
    python -m nano_vllm_rs_b200 generate --model DIR [--dtype bfloat16|float32] --prompt-ids 5,17,3 [--prompt-ids ...]
                                         [--max-tokens N] [--temperature T] [--top-k K] [--top-p P]

`generate` loads the checkpoint in DIR (config.json picks the model class, *.safetensors the weights), runs the prompts
(token ids; the package has no tokenizer of its own) through LLMEngine.generate and prints one JSON line per prompt.
Replaying a recorded schedule step by step is bin/trace_run."""
import argparse
import json
import sys


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m nano_vllm_rs_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("architectures", help="model architectures the library can serve")
    g = sub.add_parser("generate", help="greedy or sampled generation from token-id prompts")
    g.add_argument("--model", required=True)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    g.add_argument("--max-tokens", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--block-size", type=int, default=None)
    a = ap.parse_args(argv)
    from .engine import LLMEngine, SamplingParams, lib
    if a.cmd == "architectures":
        print(lib().nvllm_registered_architectures().decode())
        return 0
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids]
    over = {"max_num_seqs": max(4, len(prompts)), "max_model_len": max(len(p) for p in prompts) + a.max_tokens + 1}
    if a.block_size:
        over["kvcache_block_size"] = a.block_size
    eng = LLMEngine.from_pretrained(a.model, dtype=a.dtype, **over)
    sp = SamplingParams(temperature=a.temperature, max_tokens=a.max_tokens, ignore_eos=True, top_k=a.top_k, top_p=a.top_p)
    for p, out in zip(prompts, eng.generate(prompts, sp)):
        print(json.dumps({"prompt_ids": p, "completion_ids": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
