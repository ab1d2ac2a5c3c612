"""CLI (argument parsing, extract determinism, JSON output and error objects, compile -> verify -> serve on CPU),
calibration (corpus validation, statistics, byte-stable writers, prompt sampling) and the launcher/rendezvous.

Mirrors crates/skein_cli/tests/{arg_parsing,extract_e2e,output_formats}.rs, crates/skein_calibrate/tests/
{corpus_loading,cost_writer_byte_stable}.rs and the unit tests in launcher.rs:81-110, rendezvous.rs:101-118.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from skein_b200 import calibrate as cal
from skein_b200.cli.main import build_parser, main
from skein_b200.parallel import launcher

ROOT = Path(__file__).resolve().parent.parent
ARGS = ["--model", str(ROOT / "configs/mixtral_8x7b_config.json"), "--cluster", str(ROOT / "cluster/h100_2x.toml"), "--trace",
        str(ROOT / "cluster/sample_trace.jsonl"), "--drift", str(ROOT / "models/mixtral_8x7b_drift.toml"), "--cost", str(ROOT / "cluster/cost_constants.toml")]
TINY = {"architectures": ["MixtralForCausalLM"], "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2, "num_attention_heads": 4,
        "num_key_value_heads": 2, "head_dim": 128, "num_local_experts": 4, "num_experts_per_tok": 2, "vocab_size": 512, "rope_theta": 1e6,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 512}


def test_arg_parsing_all_subcommands():
    p = build_parser()
    a = p.parse_args(["--output", "json", "extract", *ARGS, "--out", "x.json"])
    assert a.command == "extract" and a.output == "json" and a.out == "x.json"
    a = p.parse_args(["compile", *ARGS, "--weights", "w/", "--enforce-parity", "--n-parity-prompts", "3"])
    assert a.enforce_parity and a.n_parity_prompts == 3 and a.out == "artifacts/"
    a = p.parse_args(["verify", "--artifact", "a", "--enforce", "--hf-reference", "--n-prompts", "7"])
    assert a.enforce and a.hf_reference and a.n_prompts == 7 and a.cost == "cluster/cost_constants.toml"
    a = p.parse_args(["serve", "--artifact", "a", "--gpus", "0,1", "--prompt", "hi"])
    assert a.port == 8080 and a.max_new_tokens == 32 and a.rendezvous == "/tmp/skein_rendezvous" and a.gpus == "0,1"
    a = p.parse_args(["calibrate", "--hardware", "b200", "--model", "m", "--corpus", "c"])
    assert a.out_cost == "cluster/cost_constants.toml" and a.out_drift_dir == "models/"
    a = p.parse_args(["bench", "--artifact", "a", "--workload", "w", "--baseline", "http://x", "--metrics", "throughput,goodput"])
    assert a.metrics == "throughput,goodput"
    with pytest.raises(SystemExit):
        p.parse_args(["extract"])                       # required inputs missing


def test_extract_end_to_end_deterministic_json(tmp_path, capsys):
    out1, out2 = tmp_path / "p1.json", tmp_path / "p2.json"
    assert main(["--output", "json", "extract", *ARGS, "--out", str(out1)]) == 0
    rep1 = json.loads(capsys.readouterr().out)
    assert main(["--output", "json", "extract", *ARGS, "--out", str(out2)]) == 0
    rep2 = json.loads(capsys.readouterr().out)
    assert out1.read_bytes() == out2.read_bytes() and rep1["content_hash"] == rep2["content_hash"]
    assert set(rep1) >= {"plan_path", "content_hash", "cost_us", "search", "summary"} and rep1["search"]["raw"] == 560
    assert main(["extract", *ARGS, "--out", str(out1)]) == 0
    assert "placement   tp=" in capsys.readouterr().out


def test_bench_writes_synthetic_traces(tmp_path, capsys):
    """`bench --synth` generates the uniform and the burst workload as a trace file (seeded, reproducible) that the other
    commands read like any recorded trace."""
    p1, p2, p3 = tmp_path / "a.jsonl", tmp_path / "b.jsonl", tmp_path / "c.jsonl"
    assert main(["--output", "json", "bench", "--synth", "burst", "--synth-requests", "40", "--write-trace", str(p1)]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["requests"] == 40 and rep["kind"] == "burst"
    assert main(["bench", "--synth", "burst", "--synth-requests", "40", "--write-trace", str(p2)]) == 0
    assert main(["bench", "--synth", "uniform", "--synth-requests", "40", "--synth-seed", "3", "--write-trace", str(p3)]) == 0
    capsys.readouterr()
    assert p1.read_bytes() == p2.read_bytes() != p3.read_bytes()
    lines = [json.loads(l) for l in p1.read_text().splitlines()]
    assert "slo" in lines[0] and len(lines) == 41
    reqs = lines[1:]
    assert all(1 <= r["prompt_tokens"] <= 8192 and 32 <= r["output_tokens"] <= 1024 for r in reqs)
    assert [r["arrival_ms"] for r in reqs] == sorted(r["arrival_ms"] for r in reqs)
    # the planner takes the generated trace
    assert main(["--output", "json", "extract", *[a if a != str(ROOT / "cluster/sample_trace.jsonl") else str(p3) for a in ARGS],
                 "--out", str(tmp_path / "plan.json")]) == 0
    capsys.readouterr()


def test_errors_are_json_objects_on_stderr(tmp_path, capsys):
    bad = tmp_path / "cluster.toml"
    bad.write_text((ROOT / "cluster/h100_2x.toml").read_text().replace("num_devices = 2", "num_devices = 5"))
    args = list(ARGS)
    args[3] = str(bad)
    assert main(["--output", "json", "extract", *args, "--out", str(tmp_path / "p.json")]) == 1
    err = json.loads(capsys.readouterr().err)
    assert err["error"]["kind"] == "ClusterError" and "num_devices" in err["error"]["message"]


def test_compile_verify_serve_job_cpu(tmp_path, capsys):
    cfg = tmp_path / "tiny_config.json"
    cfg.write_text(json.dumps(TINY))
    drift = tmp_path / "tiny_drift.toml"
    drift.write_text((ROOT / "models/mixtral_8x7b_drift.toml").read_text())
    common = ["--model", str(cfg), "--cluster", str(ROOT / "cluster/b200_1x.toml"), "--trace", str(ROOT / "cluster/sample_trace.jsonl"),
              "--drift", str(drift), "--cost", str(ROOT / "cluster/cost_constants.toml")]
    assert main(["--output", "json", "compile", *common, "--out", str(tmp_path / "art"), "--n-parity-prompts", "2", "--enforce-parity"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["parity"]["passed"] and (tmp_path / "art" / "LATEST").is_symlink()
    art = str(tmp_path / "art" / "LATEST")
    art = str((tmp_path / "art" / os.readlink(art)))
    assert main(["--output", "json", "verify", "--artifact", art, "--enforce", "--cost", str(ROOT / "cluster/cost_constants.toml"), "--n-prompts", "2"]) == 0
    assert json.loads(capsys.readouterr().out)["passed"]
    assert main(["--output", "json", "verify", "--artifact", art, "--hf-reference", "--cost", str(ROOT / "cluster/cost_constants.toml"), "--n-prompts", "2"]) == 0
    hf = json.loads(capsys.readouterr().out)
    assert hf["avg_final_kl"] < 0.05                    # runtime graph vs cache-free dense oracle
    # generation job through the worker (single rank, CPU)
    r = subprocess.run([sys.executable, "-m", "skein_b200.cli.main", "serve", "--artifact", art, "--prompt", "hello", "--max-new-tokens", "4",
                        "--max-seq-len", "128"], capture_output=True, text=True, cwd=ROOT, timeout=300,
                       env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert len(out["generated"][0]) == 4 and out["tokens_per_s"] > 0
    # trace replay
    assert main(["--output", "json", "bench", "--artifact", art, "--workload", str(ROOT / "cluster/sample_trace.jsonl"), "--max-requests", "2",
                 "--time-scale", "1000"]) == 0
    b = json.loads(capsys.readouterr().out)
    assert b["requests_ok"] + b["requests_rejected"] == 2 and b["drift_compliance"] is True
    assert "throughput_tok_s" in b and "goodput_req_s" in b
    # --metrics chooses the headline figures; an unknown name is refused
    assert main(["--output", "json", "bench", "--artifact", art, "--workload", str(ROOT / "cluster/sample_trace.jsonl"), "--max-requests", "1",
                 "--time-scale", "1000", "--metrics", "throughput"]) == 0
    b1 = json.loads(capsys.readouterr().out)
    assert "throughput_tok_s" in b1 and "goodput_req_s" not in b1 and "drift_compliance" not in b1 and "requests_ok" in b1
    assert main(["--output", "json", "bench", "--artifact", art, "--workload", str(ROOT / "cluster/sample_trace.jsonl"), "--metrics", "latency"]) != 0
    assert "unknown metric" in capsys.readouterr().err


def test_pipeline_artifact_served_by_two_cpu_rank_processes(tmp_path):
    """`serve --gpus 0,1` on a PP=2 artifact: the launcher starts two rank processes (gloo on CPU), watches their
    heartbeats, and reports none failed."""
    cfg = tmp_path / "tiny_config.json"
    cfg.write_text(json.dumps(TINY))
    drift = tmp_path / "tiny_drift.toml"
    drift.write_text((ROOT / "models/mixtral_8x7b_drift.toml").read_text())
    env = {**os.environ, "CUDA_VISIBLE_DEVICES": "", "SKEIN_FORCE_TP": "1", "SKEIN_FORCE_PP": "2", "SKEIN_FORCE_EP": "1"}
    cli = [sys.executable, "-m", "skein_b200.cli.main", "--output", "json"]
    r = subprocess.run([*cli, "compile", "--model", str(cfg), "--cluster", str(ROOT / "cluster/b200_2x.toml"), "--trace",
                        str(ROOT / "cluster/sample_trace.jsonl"), "--drift", str(drift), "--cost", str(ROOT / "cluster/cost_constants.toml"),
                        "--out", str(tmp_path / "art"), "--n-parity-prompts", "2", "--enforce-parity"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    art = str(tmp_path / "art" / os.readlink(tmp_path / "art" / "LATEST"))
    assert json.loads((Path(art) / "plan.json").read_text())["parallelism"] == {"tp": 1, "pp": 2, "ep": 1}
    r = subprocess.run([*cli, "serve", "--artifact", art, "--gpus", "0,1", "--prompt", "hello", "--max-new-tokens", "4",
                        "--max-seq-len", "128", "--rendezvous", str(tmp_path / "rdv")],
                       capture_output=True, text=True, cwd=ROOT, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1]) == {"failed": 0, "ranks": 2}
    assert sorted(p.name for p in (tmp_path / "rdv.hb").glob("*.hb")) == ["rank_0.hb", "rank_1.hb"]

    # the same two ranks behind the HTTP front end (rank 0 hosts it and announces every step to rank 1); SIGTERM to the
    # launcher reaches rank 0 only, which stops the group between steps: both ranks exit 0
    import signal
    import socket
    import time
    import urllib.request
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    p = subprocess.Popen([*cli, "serve", "--artifact", art, "--gpus", "0,1", "--port", str(port), "--max-seq-len", "128",
                          "--rendezvous", str(tmp_path / "rdv_http")], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         cwd=ROOT, env={**env, "SKEIN_PP_CONTINUOUS": "1"})     # one group of sequences per stage kept in flight
    try:
        up = False
        for _ in range(600):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/healthz", timeout=1) as h:
                    up = h.status == 200
                    break
            except OSError:
                assert p.poll() is None, p.stderr.read()[-2000:]
                time.sleep(0.2)
        assert up
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", headers={"Content-Type": "application/json"},
                                     data=json.dumps({"prompt": "hello", "max_tokens": 4}).encode())
        with urllib.request.urlopen(req, timeout=120) as resp:
            body = json.loads(resp.read().decode())
        assert len(body["tokens"]) == 4 and body["finish_reason"] == "length"
        # the trace replayed against the running two-rank server over HTTP/SSE (how a multi-rank artifact is benchmarked)
        trace = tmp_path / "t.jsonl"
        trace.write_text(json.dumps({"slo": {"ttft_p95_ms": 60000, "tpot_p95_ms": 60000, "max_accuracy_drift": 0.01,
                                             "recompile_drift_threshold_kl": 0.05}}) + "\n" +
                         "".join(json.dumps({"prompt_tokens": 10 + i, "output_tokens": 3, "arrival_ms": 5 * i}) + "\n" for i in range(3)))
        rb = subprocess.run([*cli, "bench", "--url", f"http://127.0.0.1:{port}", "--workload", str(trace), "--vocab-size", "300",
                             "--max-seq-len", "128"], capture_output=True, text=True, cwd=ROOT, timeout=180, env=env)
        assert rb.returncode == 0, rb.stderr[-2000:]
        bj = json.loads(rb.stdout.strip().splitlines()[-1])
        assert bj["requests_ok"] == 3 and bj["requests_failed"] == 0 and bj["ttft_p50_ms"] > 0 and bj["throughput_tok_s"] > 0
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10) as h:
            assert "skein_pipeline_groups_in_flight_max 1" in h.read().decode()
        p.send_signal(signal.SIGTERM)
        out, err = p.communicate(timeout=90)
    finally:
        if p.poll() is None:
            p.kill()
    assert p.returncode == 0, err[-2000:]
    assert json.loads(out.strip().splitlines()[-1]) == {"failed": 0, "ranks": 2}


# ---- calibration ----------------------------------------------------------------------------------------------------
CORPUS = """workload_trace_path = "traces/t.jsonl"
n_drift_prompts = 4
sampling_strategy = "stratified_by_length"
sampling_seed = 0
[[kernel_samples]]
op_kind = "gemm"
dtype = "bf16"
shape = [4096, 4096]
repeats = 10
"""


@pytest.mark.parametrize("old,new,msg", [
    ('n_drift_prompts = 4', 'n_drift_prompts = 0', "n_drift_prompts"),
    ('"stratified_by_length"', '"alphabetical"', "sampling_strategy"),
    ('op_kind = "gemm"', 'op_kind = "fft"', "op_kind"),
    ('dtype = "bf16"', 'dtype = "fp4"', "dtype"),
    ('shape = [4096, 4096]', 'shape = [4096, 0]', "shape"),
    ('shape = [4096, 4096]', 'shape = []', "shape"),
    ('repeats = 10', 'repeats = 0', "repeats"),
    ('workload_trace_path = "traces/t.jsonl"', 'workload_trace_path = ""', "workload_trace_path"),
    ('n_drift_prompts = 4\n', '', "n_drift_prompts"),
])
def test_corpus_rejections(old, new, msg):
    assert cal.Corpus.from_toml(CORPUS).kernel_samples[0].shape == [4096, 4096]
    with pytest.raises(cal.CalibrationError, match=msg):
        cal.Corpus.from_toml(CORPUS.replace(old, new))
    with pytest.raises(cal.CalibrationError, match="kernel_samples"):
        cal.Corpus.from_toml(CORPUS.split("[[kernel_samples]]")[0])


def test_statistics_and_prompt_sampling():
    assert cal.median([3, 1, 2]) == 2 and cal.median([]) == 0.0 and cal.median([1, 2, 3, 4]) == 3
    assert cal.p95([10.0]) == 10.0 and cal.p95(list(map(float, range(1, 101)))) == pytest.approx(95.05)
    lengths = [5, 500, 50, 5000, 20, 200, 2000, 10]
    a = cal.sample_prompts(lengths, 4, "stratified_by_length", 0)
    assert a == cal.sample_prompts(lengths, 4, "stratified_by_length", 0) and len(a) == 4
    assert cal.sample_prompts(lengths, 3, "first_n", 9) == [0, 1, 2]
    assert cal.sample_prompts(lengths, 4, "uniform_random", 1) != cal.sample_prompts(lengths, 4, "uniform_random", 2)
    # one prompt per length stratum
    srt = sorted(range(8), key=lambda i: lengths[i])
    strata = [set(srt[0:2]), set(srt[2:4]), set(srt[4:6]), set(srt[6:8])]
    assert all(len(s & set(a)) == 1 for s in strata)


def test_cost_writer_is_byte_stable_and_preserves_unmeasured_entries():
    text = (ROOT / "cluster/cost_constants.toml").read_text()
    assert cal.write_cost_constants(text, {}) == text
    new = cal.write_cost_constants(text, {("gemm", "bf16"): 0.91, ("attention", "bf16"): 0.33}, {"ring_allreduce": 0.8}, {"b200": 6600.0})
    changed = [(a, b) for a, b in zip(text.split("\n"), new.split("\n")) if a != b]
    assert len(changed) == 4 and len(text.split("\n")) == len(new.split("\n"))
    assert "bf16     = 0.91" in new and "ring_allreduce = 0.8" in new and "b200      = 6600.0" in new
    assert "fp8_e4m3 = 0.76" in new                       # unmeasured entry untouched
    # the measured streaming share per weight dtype is rewritten in place as well
    st = cal.write_cost_constants(text, {}, stream_efficiency={"bf16": 0.99, "fp8_e4m3": 0.66})
    assert "[stream_efficiency]\nbf16     = 0.99" in st and "fp8_e4m3 = 0.66" in st and "int8     = 0.6" in st
    assert len(st.split("\n")) == len(text.split("\n"))
    assert cal.write_cost_constants(new, {("gemm", "bf16"): 0.91}) == new
    # comments after values survive; a new key lands inside its section
    t2 = cal.rewrite_toml_values("[a]\nx = 1.0   # keep me\n[b]\ny = 2.0\n", {("a", "x"): 3.5, ("a", "z"): 7.0})
    assert t2 == "[a]\nx = 3.5   # keep me\nz = 7.0\n[b]\ny = 2.0\n"


def test_fixed_costs_fitted_from_a_measured_step(tmp_path, capsys):
    """`calibrate --fit-step-ms`: the measured step of a one-GPU plan gives the per-kernel fixed cost, a tensor-parallel one the
    fixed cost per all-reduce, an expert-parallel one the cost per exchange; the writer touches that entry only."""
    from skein_b200 import core
    cfg = (ROOT / "configs/mixtral_8x7b_config.json").read_text()
    text = (ROOT / "cluster/cost_constants.toml").read_text()
    meta = json.loads(core.model_meta(cfg))

    def plan(tp=1, ep=1, pp=1, batch=64, dtype="bf16"):
        return json.dumps({
            "parallelism": {"tp": tp, "pp": pp, "ep": ep}, "kv": {"layout": {"kind": "paged", "page_size": 16}, "kv_sharded": True},
            "batching": {"kind": "continuous", "max_batch": batch},
            "dtype_map": {"per_layer": [{"weight": dtype, "activation": "bf16", "kv_cache": "bf16"}] * meta["num_layers"]},
            "execution": {"cuda_graphs": {"enable": True, "capture_classes": [{"batch_size": 1 + i, "kv_class": 0} for i in range(4)]},
                          "spec_decode": {"enable": False, "draft": None}, "prefix_cache": {"enable": True, "reuse_policy": "lru_by_last_access"}},
            "disaggregation": None, "model_meta": meta})
    cl = lambda n: (ROOT / f"cluster/b200_{n}x.toml").read_text()  # noqa: E731
    one = cal.fit_fixed_costs(plan(), cfg, cl(1), text, 16.99, kv_tokens=608)
    assert list(one) == [("", "kernel_overhead_us")] and 6.0 < one[("", "kernel_overhead_us")] < 7.0
    ar = cal.fit_fixed_costs(plan(tp=2), cfg, cl(2), text, 9.95, kv_tokens=608)
    assert list(ar) == [("collective_fixed_us", "ring_allreduce")] and 6.0 < ar[("collective_fixed_us", "ring_allreduce")] < 11.0
    a2a = cal.fit_fixed_costs(plan(ep=8, batch=256, dtype="fp8_e4m3"), cfg, cl(8), text, 7.66, kv_tokens=1040)
    assert 50.0 < a2a[("collective_fixed_us", "alltoall")] < 66.0
    # a step faster than the model's streaming time fits a zero, never a negative cost
    assert cal.fit_fixed_costs(plan(), cfg, cl(1), text, 1.0)[("", "kernel_overhead_us")] == 0.0
    with pytest.raises(cal.CalibrationError, match="one GPU"):
        cal.fit_fixed_costs(plan(tp=2, ep=4), cfg, cl(8), text, 5.0)
    # through the command line: only the fitted entry of the file changes
    cost, pj = tmp_path / "cost.toml", tmp_path / "plan.json"
    cost.write_text(text)
    pj.write_text(plan(tp=8))
    corpus = tmp_path / "corpus.toml"
    corpus.write_text(CORPUS)
    assert main(["--output", "json", "calibrate", "--hardware", "b200", "--model", str(ROOT / "configs/mixtral_8x7b_config.json"),
                 "--corpus", str(corpus), "--out-cost", str(cost), "--fit-step-ms", "4.44", "--fit-plan", str(pj),
                 "--fit-cluster", str(ROOT / "cluster/b200_8x.toml"), "--fit-kv-tokens", "608"]) == 0
    rep = json.loads(capsys.readouterr().out)
    new = cost.read_text()
    changed = [(a, b) for a, b in zip(text.split("\n"), new.split("\n")) if a != b]
    assert len(changed) == 1 and changed[0][0] == "ring_allreduce = 8.0" and rep["fitted"]["collective_fixed_us.ring_allreduce"] > 8.0


def test_drift_writer_monotonic():
    text = (ROOT / "models/mixtral_8x7b_drift.toml").read_text()
    a = cal.write_drift_table(text, {(3, "weight", "fp8_e4m3"): 0.02})
    assert "[layer.3.weight]\nfp8_e4m3 = 0.02" in a
    assert cal.write_drift_table(a, {(3, "weight", "fp8_e4m3"): 0.01}) == a
    assert cal.calibrate_drift([{"layer": 0, "mse": 0.5}, {"layer": 1, "mse": 0.1}],
                               {"dtype_map": {"per_layer": [{"weight": "bf16", "activation": "bf16", "kv_cache": "bf16"},
                                                            {"weight": "fp8_e4m3", "activation": "bf16", "kv_cache": "bf16"}]}}) == {(1, "weight", "fp8_e4m3"): 0.1}


# ---- launcher / rendezvous ---------------------------------------------------------------------------------------------
def test_launch_plan_and_commands():
    plan = launcher.plan_launch(launcher.parse_gpus("3,5"), "/tmp/rdv")
    assert [(l.rank, l.world_size, l.gpu) for l in plan] == [(0, 2, 3), (1, 2, 5)]
    cmd, env = launcher.build_command(plan[1], ["--artifact", "a"], base_env={})
    assert cmd[1:4] == ["-m", "skein_b200.parallel.worker", "--artifact"]
    # every rank sees all devices of the job (peer buffers are CUDA IPC mappings) and computes on its own
    assert env == {"SKEIN_RANK": "1", "SKEIN_WORLD_SIZE": "2", "SKEIN_RENDEZVOUS": "/tmp/rdv", "CUDA_VISIBLE_DEVICES": "3,5",
                   "SKEIN_LOCAL_DEVICE": "1"}
    # --gpus ids index what the launcher itself can see
    assert launcher.build_command(plan[0], [], base_env={"CUDA_VISIBLE_DEVICES": "0,2,4,6,7,1"})[1]["CUDA_VISIBLE_DEVICES"] == "6,1"
    with pytest.raises(ValueError):
        launcher.build_command(plan[1], [], base_env={"CUDA_VISIBLE_DEVICES": "0,1"})
    with pytest.raises(ValueError):
        launcher.parse_gpus("1,1")
    with pytest.raises(ValueError):
        launcher.parse_gpus("")


def test_a_lost_rank_ends_the_job():
    """One rank exits with an error while the other would run for a minute: the survivor is terminated after the grace period."""
    import time as _t
    procs = [subprocess.Popen([sys.executable, "-c", "import sys; sys.exit(3)"]),
             subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)"])]
    t0 = _t.monotonic()
    codes = launcher.wait_ranks(procs, grace_s=0.5)
    assert codes[0] == 3 and codes[1] != 0 and _t.monotonic() - t0 < 20
    ok = [subprocess.Popen([sys.executable, "-c", "pass"]) for _ in range(2)]
    assert launcher.wait_ranks(ok) == [0, 0]
    # a lost rank with restarts allowed: the whole group starts again, and the second attempt succeeds
    attempts = []

    def spawn():
        attempts.append(1)
        bad = "import sys; sys.exit(7)" if len(attempts) == 1 else "pass"
        return [subprocess.Popen([sys.executable, "-c", bad]), subprocess.Popen([sys.executable, "-c", "pass"])]

    notes = []
    assert launcher.supervise(spawn, restarts=2, grace_s=0.5, log=notes.append) == (0, 2)
    assert len(notes) == 1 and "restart 1 of 2" in notes[0]
    attempts.clear()
    always_bad = lambda: [subprocess.Popen([sys.executable, "-c", "import sys; sys.exit(1)"])]
    assert launcher.supervise(always_bad, restarts=1, grace_s=0.2) == (1, 2)      # gives up after the allowed restarts
    # a rank that is alive but has stopped beating is terminated by the launcher's monitor and counts as lost
    import tempfile
    from skein_b200.parallel.watchdog import Monitor
    hb = tempfile.mkdtemp()
    # the fake ranks load watchdog.py by path: no package import, so they start beating within milliseconds
    beating = ("import importlib.util, time; sp = importlib.util.spec_from_file_location('wd', %r); wd = importlib.util.module_from_spec(sp); "
               "sp.loader.exec_module(wd); h = wd.Heartbeat(%r, %%d, interval_s=0.1).start(); time.sleep(%%f); %%s"
               ) % (str(ROOT / "skein_b200/parallel/watchdog.py"), hb)
    procs = [subprocess.Popen([sys.executable, "-c", beating % (0, 60.0, "h.stop()")]),
             subprocess.Popen([sys.executable, "-c", beating % (1, 1.0, "h.stop(); time.sleep(60)")])]     # stalls after 1 s
    notes = []
    t0 = _t.monotonic()
    codes = launcher.wait_ranks(procs, grace_s=0.5, monitor=Monitor(hb, 2, interval_s=0.1, missed_beats=10), log=notes.append)
    assert codes[1] != 0 and codes[0] != 0 and _t.monotonic() - t0 < 45
    assert any("rank 1 stopped beating" in n for n in notes)
    slow = [subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)"])]
    assert launcher.wait_ranks(slow, timeout_s=0.3)[0] != 0          # an overall limit ends a job that never finishes


def test_rendezvous_publish_fetch_and_timeout(tmp_path):
    p = str(tmp_path / "rdv")
    with pytest.raises(launcher.RendezvousError, match="did not appear"):
        launcher.fetch(p, timeout_s=0.1)
    launcher.publish(p, b"hello")
    assert launcher.fetch(p, 1.0) == b"hello" and not list(tmp_path.glob("*.tmp"))


def test_two_cpu_ranks_meet_and_failure_is_counted(tmp_path):
    script = ("import sys; sys.path.insert(0, %r)\nfrom skein_b200.parallel import launcher\nimport torch, torch.distributed as dist\n"
              "r, w, p = launcher.world_from_env()\nif len(sys.argv) > 1 and r == 1: sys.exit(3)\n"
              "launcher.init_process_group(r, w, p, 'gloo', timeout_s=30)\nt = torch.tensor([float(r + 1)])\ndist.all_reduce(t)\n"
              "assert t.item() == 3.0\ndist.destroy_process_group()\n") % str(ROOT)
    f = tmp_path / "rank.py"
    f.write_text(script)

    def run(extra):
        procs = []
        for l in launcher.plan_launch([0, 1], str(tmp_path / "rdv")):
            _, env = launcher.build_command(l, [])
            procs.append(subprocess.Popen([sys.executable, str(f), *extra], env=env))
        return sum(p.wait(120) != 0 for p in procs)

    assert run([]) == 0
