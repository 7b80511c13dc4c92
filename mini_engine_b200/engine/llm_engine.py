"""The Python entry point: requests in, generated tokens out.

Same surface as the reference (engine/llm_engine.py:11-64): ``LLM(model, **engine options)``,
``add_request``, ``step`` (schedule -> run -> postprocess), ``is_finished`` and ``generate``
returning ``[{"text", "token_ids"}]`` in the order of the prompts.  Prompts are lists of
token ids; strings are accepted when the model folder carries a tokenizer.
"""
from __future__ import annotations

import os
from dataclasses import fields
from time import perf_counter
from typing import Optional, Sequence as Seq

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from .model_runner import ModelRunner, StepItem
from .scheduler import Scheduler
from .sequence import Sequence


def _load_tokenizer(folder: str):
    if not any(os.path.isfile(os.path.join(folder, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
        return None
    from transformers import AutoTokenizer       # text <-> ids only; no model code
    return AutoTokenizer.from_pretrained(folder, use_fast=True)


class LLMEngine:
    def __init__(self, model: str, **kwargs):
        names = {f.name for f in fields(EngineConfig)}
        config = EngineConfig(model, **{k: v for k, v in kwargs.items() if k in names})
        self.config = config
        self.model_runner = ModelRunner(
            config.model, dtype=config.dtype, page_size=config.kvcache_block_size,
            num_pages=config.num_kvcache_blocks, max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens, max_model_len=config.max_model_len,
            gpu_memory_utilization=config.gpu_memory_utilization, use_cuda_graphs=config.use_cuda_graphs,
            model_config=config.model_config)
        config.num_kvcache_blocks = self.model_runner.num_pages
        self.tokenizer = _load_tokenizer(config.model)
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            config.eos = self.tokenizer.eos_token_id        # engine/llm_engine.py:19
        self.cache = self.model_runner.make_cache_manager(config.enable_prefix_caching)
        self.scheduler = Scheduler(config, self.cache)
        self._tokens_dev = torch.empty(config.max_num_seqs + 4, dtype=torch.int32, device=self.model_runner.device)
        self._tokens_pin = torch.empty(config.max_num_seqs + 4, dtype=torch.int32, pin_memory=True)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---- requests --------------------------------------------------------------------
    def add_request(self, prompt: str | Seq[int], sampling_params: SamplingParams, priority: int = 0) -> int:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("the model folder has no tokenizer: give prompts as lists of token ids")
            prompt = self.tokenizer.encode(prompt)
        seq = Sequence(prompt, sampling_params, priority)
        self.scheduler.add(seq)
        return seq.seq_id

    def _seed_of(self, seq: Sequence) -> int:
        s = seq.sampling_params.seed
        if s is None:
            s = self.config.seed * 1000003 + seq.seq_id
        return int(s) & 0x7FFFFFFF

    # ---- one step --------------------------------------------------------------------
    def step(self):
        seqs = self.scheduler.schedule()
        num_decode = sum(1 for s in seqs if s.num_scheduled_tokens == 1)
        num_prefill = sum(s.num_scheduled_tokens for s in seqs if s.num_scheduled_tokens > 1)
        items, samplers = [], []
        for s in seqs:
            a, n = s.num_computed_tokens, s.num_scheduled_tokens
            wants = s.samples_this_step
            items.append(StepItem(s, s.scheduled_tokens(), a, [n - 1] if wants else [],
                                  (s.sampling_params.temperature, self._seed_of(s)) if wants else None))
            if wants:
                samplers.append(s)
        # One copy to the device (the step's metadata, sampling options included), the step with the
        # draw on the device, one copy back (the drawn ids and the kernels' error flags).
        result = self.model_runner.step(items, sample=True)
        self.h2d_bytes += self.model_runner.last_h2d_bytes
        sampled = {}
        if samplers:
            S = len(samplers)
            self._tokens_dev[:S].copy_(result.tokens)
            self._tokens_dev[S:S + 4].copy_(self.model_runner.error_flag)
            self._tokens_pin[:S + 4].copy_(self._tokens_dev[:S + 4])
            self.d2h_bytes += (S + 4) * 4
            got = self._tokens_pin[:S + 4].tolist()
            if any(got[S:]):
                self.model_runner.check_device_errors()
            sampled = {s.seq_id: t for s, t in zip(samplers, got[:S])}
        emitted = self.scheduler.postprocess(seqs, [sampled.get(s.seq_id) for s in seqs])
        outputs = [(s.seq_id, s.completion_token_ids) for s in emitted if s.is_finished]
        return outputs, num_prefill, num_decode, [s.seq_id for s in emitted]

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    def generate(self, prompts, sampling_params, use_tqdm: bool = True, priorities: Optional[list[int]] = None):
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        priorities = priorities or [0] * len(prompts)
        ids = [self.add_request(p, sp, pr) for p, sp, pr in zip(prompts, sampling_params, priorities)]
        pbar = None
        if use_tqdm:
            from tqdm.auto import tqdm
            pbar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
        outputs = {}
        while not self.is_finished():
            t = perf_counter()
            out, num_prefill, num_decode, _ = self.step()
            if pbar is not None:
                dt = perf_counter() - t
                pbar.set_postfix({"prefill": num_prefill, "decode": num_decode,
                                  "tok/s": f"{(num_prefill + num_decode) / max(dt, 1e-9):.0f}"})
                pbar.update(len(out))
            for seq_id, toks in out:
                outputs[seq_id] = toks
        if pbar is not None:
            pbar.close()
        result = []
        for seq_id in ids:
            toks = outputs[seq_id]
            text = self.tokenizer.decode(toks, skip_special_tokens=True) if self.tokenizer is not None else None
            result.append({"text": text, "token_ids": toks})
        return result
