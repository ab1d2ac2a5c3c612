"""Tensor-parallel fused kernels on real GPUs (2 ranks, one process per GPU). See workers/tp_worker.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, env_extra=None, port=29541, worker="tp_worker.py", ok="TP_WORKER_OK"):
    env = dict(os.environ)
    env.update({"NCCL_NVLS_ENABLE": "0"})
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "workers", worker)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    first_tb = r.stderr.find("Traceback")       # the worker's own traceback comes before the launcher's summary
    assert r.returncode == 0 and ok in r.stdout, r.stdout[-2000:] + r.stderr[max(0, first_tb):][:4000] + r.stderr[-1500:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_fused():
    _run(2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_nccl_baseline_mode():
    _run(2, {"SKEIN_COMM": "nccl"}, port=29542)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_in_switch_reduction():
    """The same checks with the partials summed inside the NVSwitch (multimem.ld_reduce on a multicast mapping)."""
    _run(2, {"SKEIN_MULTIMEM": "1"}, port=29549, ok="multimem 1")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_fused():
    _run(4, port=29543)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_in_switch_reduction():
    _run(4, {"SKEIN_MULTIMEM": "1"}, port=29551, ok="multimem 1")


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp8_fused():
    _run(8, port=29552)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp8_in_switch_reduction():
    _run(8, {"SKEIN_MULTIMEM": "1"}, port=29553, ok="multimem 1")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_fused():
    """Expert parallelism over 2 GPUs: experts divided, owner-aware combine pulls each row from its owner."""
    _run(2, {"SKEIN_TEST_TP": "1"}, port=29544, worker="ep_worker.py", ok="EP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_fp8_experts():
    """The same with block-scaled fp8 expert weights: grouped fp8 GEMMs, fp8 publish epilogue, owner-aware combine."""
    _run(2, {"SKEIN_TEST_TP": "1", "SKEIN_TEST_FP8": "1"}, port=29547, worker="ep_worker.py", ok="EP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_token_dispatch_with_data_parallel_attention():
    """Token-routed expert parallelism: dispatch / combine round trip with identity experts, and a tiny Mixtral served
    EP=2 through the engine with every rank attending only over its own slice of the sequences."""
    _run(2, port=29555, worker="ep_dp_worker.py", ok="EP_DP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_ep4_token_dispatch_with_data_parallel_attention():
    _run(4, port=29556, worker="ep_dp_worker.py", ok="EP_DP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_ep8_token_dispatch_with_data_parallel_attention():
    _run(8, port=29557, worker="ep_dp_worker.py", ok="EP_DP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp2_ep2_fused():
    _run(4, {"SKEIN_TEST_TP": "2"}, port=29545, worker="ep_worker.py", ok="EP_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pull_collectives_match_the_library():
    """all-gather, reduce-scatter, all-to-all and all-reduce as publish + one pull kernel over peer memory."""
    _run(2, port=29548, worker="coll_worker.py", ok="COLL_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_prefill_decode_disaggregation_over_peer_memory():
    """A prompt prefilled on GPU 0, its KV pages stored into GPU 1's pools by the page-copy kernel over NVLink, decoded
    on GPU 1: same tokens as prefill + decode on one GPU. See workers/disagg_worker.py."""
    _run(2, port=29554, worker="disagg_worker.py", ok="DISAGG_WORKER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pp2_gpu(tmp_path):
    """Two pipeline stages on two GPUs (NCCL point-to-point of the residual stream, token feedback, micro-batched
    pipelined decode) produce exactly the single-stage tokens. See workers/pp_worker.py."""
    from skein_b200.parallel import launcher

    procs = []
    for l in launcher.plan_launch([0, 1], str(tmp_path / "rdv")):
        _, env = launcher.build_command(l, [])
        env.update({"PP_WORKER_DEVICE": "cuda", "NCCL_NVLS_ENABLE": "0"})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "workers", "pp_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=200) for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[1][-2000:] for o in outs)
    assert "PP_WORKER_OK" in outs[0][0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_silent_rank_is_detected_by_the_bounded_wait():
    """A rank that stops publishing makes the peer's wait run out after its budget: an error status, not a hang."""
    _run(2, port=29546, worker="tp_timeout_worker.py", ok="TP_TIMEOUT_OK")
