"""Runs the reference's own scheduler and block manager on the CPU and stores what they decide.

Usage:  python tests/golden/make_scheduler_golden.py PATH_OF_THE_REFERENCE_TREE     (or $MINI_ENGINE_REF)

The reference's ``engine.scheduler.Scheduler`` (with its ``BlockManager`` and ``Sequence``) is imported from the
given tree with a plain namespace as its configuration (engine/scheduler.py:10-18 reads ``max_num_seqs,
max_num_batched_tokens, long_prefill_token_threshold, enable_chunked_prefill, scheduling_policy, eos,
kvcache_block_size, max_model_len, num_kvcache_blocks``) and driven by ``tests/scheduler_trace.py`` through the
cases listed there.  The records go to ``tests/golden/scheduler_traces.json``.
"""
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def reference_adapter_factory(ref_path: str):
    """A factory of adapters around the reference's Scheduler (imported from ``ref_path``)."""
    if not os.path.isfile(os.path.join(ref_path, "engine", "scheduler.py")):
        raise FileNotFoundError(f"{ref_path!r} is not the reference tree (no engine/scheduler.py)")
    sys.path.insert(0, ref_path)
    try:
        from engine.scheduler import Scheduler                    # the reference's
        from engine.sequence import Sequence
        from sampling_params import SamplingParams
    finally:
        sys.path.remove(ref_path)

    class Adapter:
        def __init__(self, num_pages, page_size, budget, max_seqs, chunked, threshold, policy, eos, max_model_len):
            Sequence.block_size = page_size                       # a class constant there (engine/sequence.py:15)
            cfg = types.SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=budget,
                                        long_prefill_token_threshold=threshold, enable_chunked_prefill=chunked,
                                        scheduling_policy=policy, eos=eos, kvcache_block_size=page_size,
                                        max_model_len=max_model_len, num_kvcache_blocks=num_pages)
            self.s = Scheduler(cfg)

        def add(self, toks, max_tokens, ignore_eos, priority):
            seq = Sequence(list(toks), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=ignore_eos), priority)
            try:
                self.s.add(seq)
            except ValueError:
                return None
            return seq.seq_id

        def is_finished(self): return self.s.is_finished()
        def schedule(self): return self.s.schedule()
        def postprocess(self, batch, tokens): self.s.postprocess(batch, tokens)
        def id_of(self, q): return q.seq_id
        def computed(self, q): return q.num_computed_tokens
        def scheduled(self, q): return q.num_scheduled_tokens
        def samples(self, q): return q.samples_this_step
        def tokens(self, q): return q.token_ids
        def table(self, q): return q.block_table
        def running(self): return self.s.running
        def waiting(self): return list(self.s.waiting)
        def num_free_pages(self): return self.s.block_manager.num_free_blocks
        def num_preemptions(self): return self.s.num_preemptions

    return Adapter


if __name__ == "__main__":
    import scheduler_trace
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MINI_ENGINE_REF", "")
    make = reference_adapter_factory(ref)
    out = {case[0]: scheduler_trace.run_case(case, make) for case in scheduler_trace.CASES}
    for name, rec in out.items():
        steps = [r for r in rec if "batch" in r]
        print(f"{name}: {len(steps)} steps, {steps[-1]['preemptions']} preemptions, "
              f"{sum(1 for r in rec if r.get('add') == -1)} requests refused")
    path = os.path.join(HERE, "scheduler_traces.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")
