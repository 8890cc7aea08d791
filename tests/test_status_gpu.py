"""The failure path of the kernels' bounded waits, reached without hanging or faulting anything: a self-test kernel
waits, through the package's one wait loop, on a barrier that nothing completes and on which no copy is in flight;
after its few thousand tries it reports the wait-timeout code and returns.  The engine turns the code into one
Python error, clears it, and goes on working."""

import pytest
import torch

from models_util import model_folder

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_reports_and_the_engine_goes_on():
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.engine.step import KernelStatusError
    from ampere_kv_engine_b200.kernels import ops
    engine = Engine.from_pretrained(model_folder("A"), config=EngineConfig(dtype="bfloat16", num_pages=16))
    runner = engine.runner
    seq = runner.open("r")
    before = runner.step([SeqStep(seq, [3, 1, 4, 1, 5], [4])]).clone()
    runner.raise_on_status()
    ops.ext().wait_selftest(5000, runner.status)
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 5            # kWaitTimeout
    with pytest.raises(KernelStatusError, match="bounded wait"):
        runner.raise_on_status()
    assert int(runner.status.item()) == 0
    # first writer wins: a code that is already there is not overwritten by a later timeout
    runner.status.fill_(3)
    ops.ext().wait_selftest(100, runner.status)
    with pytest.raises(KernelStatusError, match="token id"):
        runner.raise_on_status()
    # the context is whole: the same request again gives the same logits
    runner.close(seq)
    seq = runner.open("r")
    again = runner.step([SeqStep(seq, [3, 1, 4, 1, 5], [4])])
    runner.raise_on_status()
    torch.testing.assert_close(again, before, atol=0, rtol=0)
    with pytest.raises(RuntimeError, match="limit"):
        ops.ext().wait_selftest(0, runner.status)
