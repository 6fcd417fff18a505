"""A kernel whose bounded wait ran out fails the step it belongs to, on a real device.

The wait is made to run out in the one harmless way: a test-only kernel
(``tests/csrc/wait_probe.cu``) waits on an mbarrier nothing arrives at, with the engine's own
bounded wait compiled with a limit of three milliseconds; it then writes the refusal code to
the device's status word, as the tensor-core kernels do, and returns normally. Nothing traps,
faults or keeps spinning, and the context stays usable, which the tests go on to show.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import pytest
import torch

import engine_support as es
from cases import INIT_LOUD, TINY_A, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def wait_probe(tmp_path_factory):
    from ayaka_b200.kernels.build import CSRC, _nvcc

    out = tmp_path_factory.mktemp("probe") / "libwait_probe.so"
    subprocess.run(
        [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--shared",
         "-Xcompiler", "-fPIC", "-DAYK_WAIT_NS=3000000ull", "-I", str(CSRC), "-o", str(out),
         str(ROOT / "tests" / "csrc" / "wait_probe.cu")], check=True)
    library = ctypes.CDLL(str(out))

    def run(device: torch.device) -> None:
        from ayaka_b200.kernels.flags import status_word

        status = library.ayk_wait_probe(
            ctypes.c_void_p(status_word(device).data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream))
        assert status == 0

    return run


def test_the_replay_path_sees_a_wait_that_ran_out(tmp_path, wait_probe):
    from ayaka_b200.engine.runner import StepEntry
    from ayaka_b200.errors import BackendError

    folder, _ = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "float32")
    core = es.build_core(folder, "float32", num_blocks=16)
    tokens = random_tokens(256, 20, 5)
    first = core.step([StepEntry("r", tokens, [19])]).clone()
    core.runner.check_device_flags()
    core.release("r")
    wait_probe(core.device)
    with pytest.raises(BackendError, match="bounded wait"):
        core.runner.check_device_flags()
    core.runner.check_device_flags()  # cleared
    again = core.step([StepEntry("r", tokens, [19])])
    assert torch.equal(first, again)  # the context is as usable as before
    core.release("r")
    core.manager.check_integrity()


@pytest.mark.parametrize("graphs", [False, True])
def test_generation_ends_the_step_s_requests_and_goes_on(tmp_path, wait_probe, graphs):
    from ayaka_b200 import LLM, EngineConfig, SamplingParams
    from ayaka_b200.engine.outputs import FinishReason

    folder, _ = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "bfloat16")
    config = EngineConfig(model=str(folder), dtype="bfloat16", max_running=4, num_blocks=32,
                          max_tokens_per_step=64, cuda_graph=graphs)
    prompts = [tuple(random_tokens(256, n, 40 + n)) for n in (5, 17, 9)]
    params = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    with LLM.from_config(config) as llm:
        good = llm.generate(prompts, params)
        assert all(o.outputs[0].finish_reason is FinishReason.LENGTH for o in good)
        wait_probe(llm.core.device)
        failed = llm.generate(prompts, params)
        assert all(o.outputs[0].finish_reason is FinishReason.ERROR for o in failed)
        assert all("bounded wait" in o.error for o in failed)
        # no token of the failed step was delivered
        assert all(len(o.outputs[0].token_ids) == 0 for o in failed)
        llm.core.manager.check_integrity()
        assert llm.core.manager.live_requests() == []
        after = llm.generate(prompts, params)
        assert [o.outputs[0].token_ids for o in after] == [o.outputs[0].token_ids for o in good]
