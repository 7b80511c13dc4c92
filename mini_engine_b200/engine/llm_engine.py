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


class _NoEvent:
    """Stands in for a CUDA event where the runner is not on a CUDA device (host-side tests with a fake runner)."""

    def record(self):
        pass

    def synchronize(self):
        pass


class LLMEngine:
    def __init__(self, model: str, **kwargs):
        names = {f.name for f in fields(EngineConfig)}
        config = EngineConfig(model, **{k: v for k, v in kwargs.items() if k in names})
        self.config = config
        # ``model_runner=``: an object with ModelRunner's surface (step, result_dev, token_feedback, error_flag,
        # make_cache_manager, ...) in place of the real one; host-side tests drive the engine's loop with a fake.
        self.model_runner = kwargs.get("model_runner") or ModelRunner(
            config.model, dtype=config.dtype, page_size=config.kvcache_block_size,
            num_pages=config.num_kvcache_blocks, max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens, max_model_len=config.max_model_len,
            gpu_memory_utilization=config.gpu_memory_utilization, use_cuda_graphs=config.use_cuda_graphs,
            model_config=config.model_config, random_weights_seed=config.seed if config.random_weights else None)
        config.num_kvcache_blocks = self.model_runner.num_pages
        self.tokenizer = _load_tokenizer(config.model)
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            config.eos = self.tokenizer.eos_token_id        # engine/llm_engine.py:19
        self.cache = self.model_runner.make_cache_manager(config.enable_prefix_caching)
        self.scheduler = Scheduler(config, self.cache)
        on_gpu = self.model_runner.device.type == "cuda"
        self._result_pins = [torch.empty(config.max_num_seqs + 4, dtype=torch.int32, pin_memory=on_gpu) for _ in range(3)]
        self._result_events = [torch.cuda.Event() if on_gpu else _NoEvent() for _ in range(3)]
        self._turn = 0
        self._ahead = None                 # (requests, handle) of a step that is already running on the device
        self.steps_ahead_used = 0          # steps launched ahead of the host whose results were kept ...
        self.steps_ahead_dropped = 0       # ... and those the scheduler decided otherwise about
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.num_steps = 0                 # steps whose results were used (a dropped guess is not one)

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
    # One copy to the device (the step's metadata, sampling options included), the step with the draw on the
    # device, one copy back (the kernels' error flags and the drawn ids).  The copy back is asynchronous: while
    # the device runs a decode step, the host launches the step that will most likely follow it (the same
    # requests, one token further, each continuing from the token the device is about to draw: a token id ~j in
    # the metadata means row j of the step before) and only then waits for the first step's tokens.  If the
    # scheduler then decides on exactly that step, its results are kept; if not (a request ended on its
    # end-of-sequence token, a new request arrived, pages ran out) they are dropped, which costs a millisecond
    # of device time and changes nothing: the dropped step wrote the keys and values that the real one writes
    # again, and draws depend on (seed, position) only.
    def _launch(self, seqs, items=None) -> dict:
        if items is None:
            items = []
            for s in seqs:
                a, n = s.num_computed_tokens, s.num_scheduled_tokens
                wants = s.samples_this_step
                items.append(StepItem(s, s.scheduled_tokens(), a, [n - 1] if wants else [],
                                      (s.sampling_params.temperature, self._seed_of(s)) if wants else None))
        rows = [i for i, it in enumerate(items) if it.want]
        result = self.model_runner.step(items, sample=True)
        self.h2d_bytes += self.model_runner.last_h2d_bytes
        k = self._turn = (self._turn + 1) % 3
        S = len(rows)
        dev = self.model_runner.result_dev
        dev[:4].copy_(self.model_runner.error_flag)
        if S:
            dev[4:4 + S].copy_(result.tokens)
        self._result_pins[k][:4 + S].copy_(dev[:4 + S], non_blocking=True)
        self._result_events[k].record()
        self.d2h_bytes += (4 + S) * 4
        return {"turn": k, "rows": rows, "take": list(range(S))}

    def _collect(self, seqs, handle) -> list:
        """The tokens of a launched step, one per request (None where the request drew none)."""
        k = handle["turn"]
        self._result_events[k].synchronize()
        got = self._result_pins[k][:4 + len(handle["rows"])].tolist()
        if any(got[:4]):
            self.model_runner.check_device_errors()
        tokens = [None] * len(seqs)
        for i, r in zip(handle["for"] if "for" in handle else handle["rows"], handle["take"]):
            tokens[i] = got[4 + r]
        return tokens

    def _launch_ahead(self, seqs, handle):
        """The step that follows a decode step of ``seqs`` if nothing unforeseen happens; None if it is not worth
        or not possible to guess.  ``handle`` is the launched step of ``seqs``: it knows in which row of the
        device's result each request's token lies (the rows of a kept guess are those of the batch that was
        guessed, which may hold requests that have ended since)."""
        if not self.config.overlap_steps or self.scheduler.waiting:
            return None
        if self.model_runner.state_needs:
            # A dropped guess is harmless only because keys and values are written again by the real step; a mixer
            # with state of its own would have advanced that state twice.
            return None
        if any(s.num_scheduled_tokens != 1 or not s.samples_this_step for s in seqs):
            return None
        row_of = dict(zip(handle["for"] if "for" in handle else handle["rows"], handle["take"]))
        ahead, items = [], []
        for j, s in enumerate(seqs):
            if s.num_completion_tokens + 1 >= s.sampling_params.max_tokens or len(s) + 1 >= self.config.max_model_len:
                continue                             # this step is the request's last
            if not self.cache.allocate(s, 2):        # room for the token after the one being drawn; nobody is evicted for a guess
                return None
            ahead.append(s)
            items.append(StepItem(s, [~row_of[j]], len(s), [0], (s.sampling_params.temperature, self._seed_of(s))))
        if not ahead:
            return None
        return ahead, self._launch(ahead, items)

    def step(self):
        self.num_steps += 1
        if self._ahead is not None:
            seqs, handle = self._ahead               # launched during the call before this one
            self._ahead = None
        else:
            seqs = self.scheduler.schedule()
            handle = self._launch(seqs)
        num_decode = sum(1 for s in seqs if s.num_scheduled_tokens == 1)
        num_prefill = sum(s.num_scheduled_tokens for s in seqs if s.num_scheduled_tokens > 1)
        guess = self._launch_ahead(seqs, handle)
        tokens = self._collect(seqs, handle)
        emitted = self.scheduler.postprocess(seqs, tokens)
        if guess is not None:
            ahead, ahead_handle = guess
            if self.scheduler.is_finished():
                self.steps_ahead_dropped += 1
            else:
                nxt = self.scheduler.schedule()
                expect = [s for s in ahead if not s.is_finished]
                same = (len(nxt) == len(expect) and all(a is b for a, b in zip(nxt, expect))
                        and all(s.num_scheduled_tokens == 1 and s.samples_this_step for s in nxt))
                if same:
                    where = {id(s): r for r, s in enumerate(ahead)}
                    ahead_handle["for"] = list(range(len(nxt)))
                    ahead_handle["take"] = [where[id(s)] for s in nxt]
                    self._ahead = (nxt, ahead_handle)
                    self.steps_ahead_used += 1
                else:
                    self.steps_ahead_dropped += 1
                    self._ahead = (nxt, self._launch(nxt))
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
