"""The Python entry point: load a model folder, generate token ids.

It mirrors thanhauco/rust-inference's examples/generate.rs:18-43 (load, make a
cache, run the prompt, then one token at a time until a stop token or the
limit) for batches of token-id prompts; the tokenizer is not part of this
library, so prompts and results are token ids.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

from .cache import PAGE_SIZE
from .engine import Engine, GenerationResult, Model
from .engine.generate import generate as _generate
from .sampling import SamplingParams


class LLM:
    """A loaded model with a cache, ready to generate.

    ``max_pages`` (pages of 32 tokens per layer) and ``pages_per_seq`` have the
    meaning of the reference runner's ``--max-pages`` / ``--pages-per-seq``
    (src/bin/runner.rs:54-60); ``max_seqs`` is the number of sequences a batch
    may hold."""

    def __init__(self, model_dir: Optional[str] = None, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_pages: int = 256, pages_per_seq: int = 128, max_seqs: int = 8, use_graphs: bool = True,
                 model: Optional[Model] = None, engine: Optional[Engine] = None):
        if engine is not None:
            self.model, self.engine = engine.model, engine
            return
        if model is None:
            if model_dir is None:
                raise ValueError("give a model folder or a built model")
            model = Model.from_dir(model_dir, dtype=dtype, device=device)
        self.model = model
        self.engine = Engine(model, max_tokens=max_pages * PAGE_SIZE, max_seqs=max_seqs,
                             max_seq_len=pages_per_seq * PAGE_SIZE, use_graphs=use_graphs)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, repetition_penalty: float = 1.0, seed: int = 0x5EED,
                 stop_ids: Optional[Iterable[int]] = None, ignore_eos: bool = False,
                 batch_size: Optional[int] = None, return_result: bool = False):
        """New token ids for each prompt (lists of ints in, lists of ints out)."""
        params = SamplingParams(temperature, top_k, top_p, repetition_penalty, seed)
        res = _generate(self.engine, prompts, max_new_tokens, params, stop_ids, ignore_eos, batch_size)
        return res if return_result else res.tokens


def generate(model_dir: str, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, dtype: str = "bfloat16",
             **options) -> List[List[int]]:
    """One call: load ``model_dir`` and generate for ``prompts``.  Options as in
    :meth:`LLM.generate`; the cache is sized for these prompts."""
    llm_keys = ("device", "max_pages", "pages_per_seq", "max_seqs", "use_graphs")
    llm_opts = {k: options.pop(k) for k in llm_keys if k in options}
    longest = max((len(p) for p in prompts), default=1) + max_new_tokens
    llm_opts.setdefault("pages_per_seq", -(-longest // PAGE_SIZE))
    llm_opts.setdefault("max_seqs", max(1, min(len(prompts), 64)))
    llm_opts.setdefault("max_pages", llm_opts["pages_per_seq"] * llm_opts["max_seqs"])
    return LLM(model_dir, dtype=dtype, **llm_opts).generate(prompts, max_new_tokens, **options)
