"""Typed runtime switches: defaults, TOML / environment / override precedence, validation, export to the environment.
The reference has no counterpart to test against: its switches are ~95 ad-hoc environment reads."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from skein_b200.utils.runtime_config import RuntimeConfig, RuntimeConfigError

ROOT = Path(__file__).resolve().parent.parent


def test_defaults_are_the_fast_path_and_round_trip_through_the_environment():
    d = RuntimeConfig()
    assert (d.comm, d.attn_decode, d.fuse_route, d.fuse_rope, d.pack_moe, d.pdl, d.multimem) == ("fused", "auto", True, True, True, False, False)
    env = d.to_env()
    assert env["SKEIN_COMM"] == "fused" and env["SKEIN_PDL"] == "0" and "SKEIN_TUNE_CACHE" not in env and "SKEIN_ATTN_SPLITS" not in env
    assert RuntimeConfig.from_env(env) == d
    c = RuntimeConfig(comm="nccl", attn_splits=4, tune_cache="/x/k.json", fuse_rope=False)
    assert RuntimeConfig.from_env(c.to_env()) == c


def test_precedence_file_then_environment_then_overrides():
    toml = '[runtime]\ncomm = "nccl"\nprofile = 2\nfuse_route = false\n'
    cfg = RuntimeConfig.resolve(toml, env={"SKEIN_PROFILE": "1", "UNRELATED": "x"}, overrides={"fuse_route": True, "pdl": None})
    assert (cfg.comm, cfg.profile, cfg.fuse_route, cfg.pdl) == ("nccl", 1, True, False)
    env = {"SKEIN_TUNE_CACHE": "/old", "SKEIN_ATTN_SPLITS": "3"}
    RuntimeConfig().apply_to_env(env)
    assert "SKEIN_TUNE_CACHE" not in env and "SKEIN_ATTN_SPLITS" not in env and env["SKEIN_FUSE_ROPE"] == "1"


@pytest.mark.parametrize("toml,msg", [
    ('[runtime]\ncom = "fused"\n', "unknown runtime key"),
    ('[runtime]\ncomm = "mpi"\n', "expected one of"),
    ('[runtime]\nprofile = 7\n', "expected one of"),
    ('[runtime]\nprofile = true\n', "not a valid int"),
    ('[runtime]\nfuse_rope = "maybe"\n', "expected a boolean"),
    ('[runtime]\nattn_splits = 64\n', "0..16"),
    ('[runtime]\nmultimem = true\ncomm = "nccl"\n', "needs runtime.comm"),
    ('runtime = 3\n', "must be a table"),
    ('[runtime\n', "runtime config"),
])
def test_bad_files_are_rejected_before_anything_runs(toml, msg):
    with pytest.raises(RuntimeConfigError) as e:
        RuntimeConfig.from_toml(toml)
    assert msg in str(e.value)


def test_cli_applies_the_file_and_reports_bad_ones(tmp_path):
    bad = tmp_path / "bad.toml"
    bad.write_text('[runtime]\ncomm = "mpi"\n')
    r = subprocess.run([sys.executable, "-m", "skein_b200.cli.main", "--output", "json", "--runtime-config", str(bad), "extract",
                        "--model", "m", "--cluster", "c", "--trace", "t", "--drift", "d", "--cost", "k"],
                       capture_output=True, text=True, cwd=ROOT, env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 1
    assert json.loads(r.stderr.strip().splitlines()[-1])["error"]["kind"] == "RuntimeConfigError"
