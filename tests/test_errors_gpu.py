"""What a kernel reports through the step's error word reaches the host, is cleared, and the engine goes on."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_once_and_the_next_step_is_clean():
    """The bounded waits of the tensor-map kernels give up by setting flag 1 of the error word.  No real load can
    be made to miss, so a test kernel waits on a barrier that nothing completes (no copy in flight, nothing traps
    or hangs): the call returns, the runner raises and clears the word, and an ordinary step behind it is right."""
    from mini_engine_b200 import ops
    from mini_engine_b200.engine.replay import TraceReplayer
    name = "D"                                         # head size 64: its bfloat16 steps run the tensor-map kernels
    cfg, _, page = helpers.config_of(name)
    rp = TraceReplayer(helpers.model_folder(name), "bfloat16", 256, page_size=page)
    runner = rp.runner
    assert ops.wait_expires_selftest(runner.error_flag, limit=3000) == 3000
    assert runner.error_flag.tolist() == [0, 1, 0, 0]
    _, flags = ops._stream_work_buffers(runner.device)   # a streaming product that gave up may leave a neighbour's flag set
    flags[3] = 1
    with pytest.raises(RuntimeError, match="a bounded wait ran out"):
        runner.check_device_errors()
    runner.check_device_errors()                       # cleared by the report
    assert int(flags.sum()) == 0                       # ... and so are the flags between the streaming products' blocks
    (r,) = helpers.random_requests(cfg["vocab_size"], (150,), seed=3)
    steps = helpers.trace_decode_tail([r], tail=4)
    got = helpers.collect(steps, [rp.run_step(st) for st in steps])["d0"]
    assert np.abs(got - helpers.plain_logits(name, r)).max() <= helpers.TOL["bfloat16"]
    assert runner.error_flag.tolist() == [0, 0, 0, 0]


def test_the_engine_raises_at_the_step_that_reads_the_word():
    from mini_engine_b200 import LLM, SamplingParams, ops
    llm = LLM(helpers.model_folder("A"), dtype="float32", kvcache_block_size=16, num_kvcache_blocks=32, max_num_seqs=4,
              max_num_batched_tokens=64, max_model_len=128)
    llm.add_request([1, 2, 3, 4], SamplingParams(temperature=0, max_tokens=4))
    ops.wait_expires_selftest(llm.model_runner.error_flag, limit=100)
    with pytest.raises(RuntimeError, match="flags \\[0, 1, 0, 0\\]"):
        llm.step()
    torch.cuda.synchronize()
    assert llm.model_runner.error_flag.tolist() == [0, 0, 0, 0]
