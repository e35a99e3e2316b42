"""The Python entry point: load a model folder, generate from token-id prompts.

    from ghost_infer_b200 import LLM
    llm = LLM("model_dir", dtype="bfloat16", max_tokens=8 * 4096)
    results = llm.generate([[1, 5, 9], [4, 4]], max_new=16, temperature=0.0)

Option names and defaults are the reference's command line's (src/main.rs:55-65): max_new 256,
temperature 0.7 (0 = greedy), top_k 40 (0 = all), top_p 0.9, seed from the clock.  Prompts are token
ids: the tokenizer is not part of this library.
"""
from __future__ import annotations

from typing import List, Mapping, Optional, Sequence

from .engine.generate import GenerationLoop, GenerationResult, GenerationStats
from .engine.model import Model
from .engine.step import Engine
from .sampling import DeviceSampler, SamplingParams


class LLM:
    def __init__(self, model, dtype: str = "bfloat16", device: str = "cuda:0", max_tokens: int = 8 * 2048,
                 max_slots: Optional[int] = None, max_seq_len: Optional[int] = None, seed: int = 0,
                 beyond_trained_positions: bool = False):
        """`model`: a model folder (config.json, model.safetensors), or a config mapping, for which random
        weights are made on the device from `seed`.  `max_seq_len` above the model's own
        `max_position_embeddings` is lowered to it unless `beyond_trained_positions` is set."""
        if isinstance(model, Model):
            self.model = model
        elif isinstance(model, Mapping):
            self.model = Model.random(model, seed=seed, dtype=dtype, device=device)
        else:
            self.model = Model.from_pretrained(str(model), dtype=dtype, device=device)
        self.cache = self.model.new_cache(max_tokens=max_tokens, max_slots=max_slots, max_seq_len=max_seq_len,
                                          beyond_trained_positions=beyond_trained_positions)
        self.engine = Engine(self.model, self.cache)
        self.last_stats: Optional[GenerationStats] = None

    @property
    def stop_token_ids(self) -> Sequence[int]:
        return tuple(self.model.spec.stop_token_ids)

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 256, temperature: float = 0.7,
                 top_k: int = 40, top_p: float = 0.9, seed: Optional[int] = None,
                 stop_token_ids: Optional[Sequence[int]] = None, batch_size: int = 8,
                 on_token=None, max_step_tokens: Optional[int] = None,
                 time_steps_every: Optional[int] = None) -> List[GenerationResult]:
        """Generates for every prompt, `batch_size` at a time, one batch after another.  `max_step_tokens`
        bounds the prompt tokens a single step carries (long prompts are then read in several steps).
        `time_steps_every` = n records the device time of every stretch of n decode steps in `last_stats.step_ms`."""
        params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
        sampler = DeviceSampler(params, self.model.rt.device)
        stop = self.stop_token_ids if stop_token_ids is None else stop_token_ids
        loop = GenerationLoop(self.engine, sampler, stop_token_ids=stop, batch_size=batch_size, on_token=on_token,
                              max_step_tokens=max_step_tokens, time_steps_every=time_steps_every)
        results = loop.run(prompts, max_new)
        self.last_stats = loop.stats
        if self.model.rt.device.type == "cuda":
            from .kernels import ops
            ops.check_status()          # a kernel whose bounded wait ran out has said so: never hand out its tokens silently
        return results
