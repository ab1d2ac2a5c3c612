"""Pipeline parallelism with two CPU ranks (gloo): see workers/pp_worker.py."""
import os
import subprocess
import sys

import pytest

from skein_b200.parallel import launcher

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("stages", [2, 3])
def test_pipeline_stages_match_single_stage(tmp_path, stages):
    """Stage-by-stage steps, the micro-batched pipelined decode and the serving engine with one group of sequences per
    stage in flight, each against the single-stage model."""
    procs = []
    for l in launcher.plan_launch(list(range(stages)), str(tmp_path / "rdv")):
        _, env = launcher.build_command(l, [])
        env["CUDA_VISIBLE_DEVICES"] = ""
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "workers", "pp_worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[1][-2000:] for o in outs)
    assert "PP_WORKER_OK" in outs[0][0] and "PP_CONTINUOUS_OK" in outs[0][0] and "PP_CONTINUOUS_FAILURE_OK" in outs[0][0]


def test_lock_step_control_agrees_on_a_failure_across_two_cpu_ranks(tmp_path):
    """See workers/control_worker.py: a step that fails on one rank is dropped on every rank, the ranks re-arm behind a
    barrier and keep serving; the pickled payload is only broadcast on iterations that have one."""
    procs = []
    for l in launcher.plan_launch([0, 1], str(tmp_path / "rdv")):
        _, env = launcher.build_command(l, [])
        env["CUDA_VISIBLE_DEVICES"] = ""
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "workers", "control_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[1][-3000:] for o in outs)
    assert "CONTROL_WORKER_OK" in outs[0][0]
