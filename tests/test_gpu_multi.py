"""Multi-GPU tests: each case launches tests/mp_worker.py with one rank per GPU."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, *args, env_extra=None, timeout=600):
    env = dict(os.environ)
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(HERE, "mp_worker.py"), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0 and "WORKER-OK" in r.stdout, f"{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return r.stdout


def _n():
    return min(torch.cuda.device_count(), 8)


@pytest.mark.parametrize("mode", ["peer", "multimem"])
def test_allreduce_oneshot_twoshot(mode):
    _run(_n(), "allreduce", mode)


@pytest.mark.parametrize("ar_mode", ["exact", "deferred_ref", "deferred_consistent"])
def test_tp_engine_tiny(ar_mode):
    _run(2, "tp_engine", ar_mode, "multimem")


def test_tp_engine_tiny_peer_loads():
    _run(2, "tp_engine", "exact", "peer")


@pytest.mark.parametrize("mode", ["peer", "multimem"])
def test_fused_projection_exchange_at_model_shapes(mode):
    """o_proj and down_proj of the 27B model sharded over every GPU of the box, 1 and 5 rows."""
    _run(_n(), "fused_shapes", mode)


@pytest.mark.parametrize("mode", ["peer", "multimem"])
def test_sequence_parallel_reduce_scatter_norm_allgather(mode):
    _run(_n(), "seq_parallel", mode)


def test_speculative_and_many_row_steps_under_tp():
    _run(2, "spec")


def test_device_sampling_under_tp():
    _run(2, "sample")


def test_bounded_wait_times_out_cleanly():
    _run(2, "wait_timeout", env_extra={"NCCL_NVLS_ENABLE": "0"})


def test_failure_detection_and_recovery_in_the_tp_engine():
    _run(2, "failure_detection", env_extra={"NCCL_NVLS_ENABLE": "0"})


def test_tp_engine_medium_all_gpus():
    """TP over every GPU of the box (8: KV heads replicated on rank pairs) against the oracle."""
    n = _n()
    if n < 4:
        pytest.skip("needs >= 4 GPUs")
    _run(8 if n >= 8 else 4, "tp_engine", "exact", "multimem", "medium")
