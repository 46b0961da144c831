"""Command line in the manner of thanhauco/rust-inference's runner (src/bin/runner.rs:24-123):

    python -m rust_inference_b200.runner MODEL_DIR --prompt "5 17 3" [-n 600] [--temperature 0.8] ...
    bin/runner MODEL_DIR --prompt-file prompts.txt --ignore-eos

Options keep the reference's names and meanings where it has them (-p/--prompt,
-n/--max-new-tokens, --ignore-eos, --max-pages, --pages-per-seq, --profile,
--temperature, --top-k, --top-p, --repetition-penalty, --seed, --device).  The
tokenizer is not part of this library, so a prompt is a list of token ids
(separated by spaces or commas) and the output is token ids; several prompts
(-p given more than once, or one per line of --prompt-file) run as a batch.
Added: --dtype, --batch-size, --stop-ids, --random-prompt, and
--write-random-model, which makes a model folder from MODEL_DIR/config.json and
a seed.  Generated ids go to stdout, one line per prompt; timing lines go to
stderr as in the reference (prefill / decode tok/s).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="runner", description="Token-id generation with a Qwen3 checkpoint on one B200")
    ap.add_argument("model_dir", help="folder with config.json and *.safetensors")
    ap.add_argument("-p", "--prompt", action="append", help="prompt as token ids; may be given several times")
    ap.add_argument("--prompt-file", help="file with one prompt (token ids) per line")
    ap.add_argument("--random-prompt", type=int, metavar="LEN", help="a seeded random prompt of LEN tokens per batch entry")
    ap.add_argument("-n", "--max-new-tokens", type=int, default=600, help="number of tokens to generate")
    ap.add_argument("--ignore-eos", action="store_true", help="keep generating past end-of-sequence tokens")
    ap.add_argument("--stop-ids", help="stop token ids (default: eos_token_id of config.json)")
    ap.add_argument("--max-pages", type=int, default=256, help="KV cache pages per layer (32 tokens each)")
    ap.add_argument("--pages-per-seq", type=int, default=128, help="maximum KV pages per sequence")
    ap.add_argument("--batch-size", type=int, default=8, help="sequences that run together")
    ap.add_argument("--profile", action="store_true",
                    help="print the time per section (device time of eager steps: no CUDA graphs) and the launch count at the end")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature; 0 = greedy")
    ap.add_argument("--top-k", type=int, default=0, help="keep only the k most likely tokens (0 = off)")
    ap.add_argument("--top-p", type=float, default=1.0, help="nucleus sampling threshold (1.0 = off)")
    ap.add_argument("--repetition-penalty", type=float, default=1.0, help="penalty for tokens already in the context (1.0 = off)")
    ap.add_argument("--seed", type=lambda s: int(s, 0), default=0x5EED, help="sampling seed")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="only cuda is built")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--write-random-model", type=int, metavar="SEED",
                    help="write model.safetensors with random weights for MODEL_DIR/config.json and exit")
    ap.add_argument("--weights-dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="stored dtype of --write-random-model")
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.device != "cuda":
        print("error: this library has no CPU backend; use --device cuda", file=sys.stderr)
        return 1
    import rust_inference_b200 as ri
    try:
        if a.write_random_model is not None:
            with open(os.path.join(a.model_dir, "config.json")) as f:
                cfg = json.load(f)
            ri.write_random_model(cfg, a.write_random_model, a.model_dir, dtype=a.weights_dtype)
            print(f"wrote {os.path.join(a.model_dir, 'model.safetensors')}", file=sys.stderr)
            return 0
        prompts = [_ids(p) for p in (a.prompt or [])]
        if a.prompt_file:
            with open(a.prompt_file) as f:
                prompts += [_ids(line) for line in f if line.strip()]
        t0 = time.perf_counter()
        llm = ri.LLM(a.model_dir, dtype=a.dtype, max_pages=a.max_pages, pages_per_seq=a.pages_per_seq,
                     max_seqs=a.batch_size, use_graphs=not a.profile)
        if a.profile:
            from rust_inference_b200 import profiler
            profiler.reset()
            profiler.enable(True)          # as src/bin/runner.rs:207 switches the reference's timers on
        spec = llm.model.spec
        print(f"loaded {spec.architecture} ({len(spec.layers)} layers) in {time.perf_counter() - t0:.2f}s", file=sys.stderr)
        if a.random_prompt:
            import numpy as np
            rng = np.random.default_rng(a.seed)
            prompts += [[int(t) for t in rng.integers(0, spec.vocab_size, size=a.random_prompt)]
                        for _ in range(max(1, a.batch_size if not prompts else 1))]
        if not prompts:
            line = sys.stdin.readline()
            prompts = [_ids(line)]
        if any(not p for p in prompts):
            print("error: empty prompt", file=sys.stderr)
            return 1
        from rust_inference_b200 import ops
        n0 = ops.launch_count()
        res = llm.generate(prompts, max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_k=a.top_k,
                           top_p=a.top_p, repetition_penalty=a.repetition_penalty, seed=a.seed,
                           stop_ids=_ids(a.stop_ids) if a.stop_ids else None, ignore_eos=a.ignore_eos,
                           batch_size=a.batch_size, return_result=True)
    except (ri.ConfigError, ri.WeightsError, ValueError, RuntimeError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    for toks in res.tokens:
        print(" ".join(str(t) for t in toks))
    st = res.stats
    print(file=sys.stderr)
    print(f"prefill: {st.prefill_tokens} tokens in {st.prefill_s:.3f}s ({st.prefill_tokens / max(st.prefill_s, 1e-9):.1f} tok/s)",
          file=sys.stderr)
    if st.decode_steps:
        print(f"decode:  {st.decode_tokens} tokens in {st.decode_s:.3f}s ({st.decode_tokens / max(st.decode_s, 1e-9):.2f} tok/s)",
              file=sys.stderr)
    if a.profile:
        print("\n" + profiler.report(), file=sys.stderr, end="")
        print(f"kernel launches: {ops.launch_count() - n0} (graph replays: {llm.engine.graph_replays}, "
              f"batches: {st.batches}, decode steps: {st.decode_steps})", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
