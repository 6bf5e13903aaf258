"""Launchers (``surogate_b200/launch``): run directories, feed filtering, providers, config building, memory fit, and the local /
SSH / dstack / Modal targets against stand-in processes (no ssh, dstack or modal client is installed, none is called)."""
import io
import json
import os
import subprocess
import sys
import time

import pytest
import yaml

from surogate_b200.launch import LaunchFields, ProviderRecord, ProviderStore, build_config, estimate_run_memory_gb, fit_verdict, list_runs, new_run, params_billions, provider_id
from surogate_b200.launch import artifacts, configs, dstack, local, modal, runs, ssh, stream
from surogate_b200.launch.records import parse_feed_line


def test_feed_line_filter_keeps_records_and_drops_log_text():
    assert parse_feed_line('{"step": 3, "ts": 1.0, "train/loss": 2.5}')["step"] == 3
    assert parse_feed_line('{"type": "gpu", "gpu_id": 0, "step": 1}') is not None
    assert parse_feed_line('{"type": "config", "model": "m"}') is not None
    for junk in ("", ":: step 3 loss 2.5", "[1, 2]", '{"type": "weird"}', '{"step": "x"}', '{"step": true}', '{"loss": 1.0}', '{"step": 3'):
        assert parse_feed_line(junk) is None, junk


def test_run_directories_history_and_status(tmp_path):
    root = str(tmp_path / "runs")
    a = new_run("local-my run/1", root, now=1_700_000_000)
    b = new_run("local-my run/1", root, now=1_700_000_000)  # same second, same label: a directory of its own
    assert a.dir != b.dir and os.path.basename(a.dir).endswith("local-my-run-1") and a.feed.endswith("metrics.jsonl")
    a.write_meta(mode="sft", model="Qwen/Qwen3-0.6B", max_steps=3)
    with open(a.feed, "w") as f:
        f.write('{"type": "config", "model": "m"}\nnot json\n')
        for i in range(3):
            f.write(json.dumps({"step": i + 1, "ts": 0.0, "train/loss": 3.0 - i, "train/tokens_per_second": 10.0}) + "\n")
        f.write(json.dumps({"step": 3, "ts": 0.0, "eval/loss": 2.2}) + "\n" + json.dumps({"step": 2, "ts": 0.0, "eval/loss": 2.0}) + "\n")
    os.makedirs(os.path.join(a.output, "checkpoint-2"))
    os.makedirs(os.path.join(a.output, "checkpoints", "step_00000003"))
    with open(os.path.join(a.output, "checkpoint-2", "w.bin"), "wb") as f:
        f.write(b"x" * 100)
    os.symlink(a.output, os.path.join(a.output, "loop"))
    assert [c["step"] for c in runs.list_checkpoints(a.output)] == [3, 2] and runs.path_size(a.output) == 100
    s = runs.summarise_feed(a.feed)
    assert s["records"] == 6 and s["step"] == 3 and s["loss"] == 1.0 and s["best_eval_loss"] == 2.0
    b.write_meta(mode="sft", max_steps=10, remote={"kind": "ssh", "host": "h", "session": "s", "dir": "d"})
    with open(b.feed, "w") as f:
        f.write(json.dumps({"step": 1, "ts": 0.0, "train/loss": 1.0}) + "\n")
    later = time.time() + 3600
    rows = {r["run"]: r for r in list_runs(root, now=later)}
    assert rows[a.id]["status"] == "done" and rows[a.id]["checkpoints"] == 2 and rows[a.id]["where"] == "local"
    assert rows[b.id]["status"] == "stopped" and rows[b.id]["where"] == "ssh"
    assert {r["status"] for r in list_runs(root)} == {"running"}  # both were written within the last minute
    c = new_run("empty", root)
    assert {r["run"]: r["status"] for r in list_runs(root, now=later)}[c.id] == "idle"
    # a pid file naming a live process of another start time is not this run
    runs.write_pid_file(a, os.getpid())
    assert runs.pid_alive(a.pid_file)
    rec = json.load(open(a.pid_file))
    json.dump({"pid": rec["pid"], "start": (rec["start"] or 0) + 1}, open(a.pid_file, "w"))
    assert not runs.pid_alive(a.pid_file)
    assert "loss" in runs.tail_bytes(a.feed, 64)


def test_provider_store_keeps_metadata_only(tmp_path):
    store = ProviderStore(str(tmp_path / "p" / "providers.json"))
    assert store.load() == []
    store.save(ProviderRecord(id=provider_id("ssh", " gpu-box "), kind="ssh", label="box", host="me@gpu-box:2222", gpu="B200:8"))
    store.save(ProviderRecord(id=provider_id("ssh", "a-1"), kind="ssh", label="a-1", host="a-1"))
    store.save(ProviderRecord(id=provider_id("ssh", "a_1"), kind="ssh", label="a_1", host="a_1"))  # distinct hosts stay distinct
    store.save(ProviderRecord(id=provider_id("dstack", "runpod"), kind="dstack", label="RunPod", backend="runpod"))
    store.save(ProviderRecord(id=provider_id("ssh", "gpu-box"), kind="ssh", label="renamed", host="me@gpu-box"))  # same id: updated in place, sorts last
    ids = [r.id for r in store.load()]
    assert ids == ["ssh:a-1", "ssh:a_1", "dstack:runpod", "ssh:gpu-box"] and store.get("ssh:gpu-box").label == "renamed"
    with pytest.raises(ValueError):
        store.save(ProviderRecord(id="x", kind="dstack", label="x", backend="nope"))
    with pytest.raises(ValueError):
        store.save(ProviderRecord(id="x", kind="k8s", label="x"))
    assert [r.id for r in store.delete("ssh:a-1")] == ["ssh:a_1", "dstack:runpod", "ssh:gpu-box"]
    text = open(store.path).read()
    assert "api_key" not in text and "secret" not in text
    open(store.path, "w").write("{broken")
    assert store.load() == []


def test_config_from_launch_fields_is_a_valid_training_config():
    from surogate_b200.config.sft_config import SFTConfig

    f = LaunchFields(model="Qwen/Qwen3-0.6B", dataset_path="data: tricky name.jsonl", max_steps=7, lora_rank=8)
    assert f.problems() == [] and "no model picked" in LaunchFields().problems()
    text = build_config(f, n_gpus=2, metrics_path="/tmp/run 1/metrics.jsonl")
    d = yaml.safe_load(text)
    assert d["datasets"] == [{"path": "data: tricky name.jsonl", "type": "auto"}] and d["gpus"] == 2 and d["report_to"] == ["surogate"]
    cfg = SFTConfig.from_dict(d)
    assert cfg.max_steps == 7 and cfg.lora and cfg.lora_rank == 8 and cfg.recipe.replace('_', '-') == "fp8-hybrid" and cfg.surogate_metrics_path == "/tmp/run 1/metrics.jsonl"
    over = configs.resume_overlay(configs.monitoring_overlay(text, 4, "/tmp/a.jsonl"), "/tmp/b.jsonl")
    d2 = configs.load_overlaid(over)
    assert d2["gpus"] == 4 and d2["surogate_metrics_path"] == "/tmp/b.jsonl" and d2["resume_from_checkpoint"] is True and d2["max_steps"] == 7
    assert configs.build_command([0, 3], "my cfg.yaml") == "CUDA_VISIBLE_DEVICES=0,3 surogate sft 'my cfg.yaml'"
    assert configs.build_command([], "c.yaml", "pt", "/opt/s") == "/opt/s pt c.yaml"


def test_memory_estimate_orders_runs_sensibly():
    assert params_billions("Qwen/Qwen3-30B-A3B") == (30.0, 3.0) and params_billions("meta-llama/Llama-3.1-70B-Instruct") == (70.0, 70.0)
    assert params_billions("HuggingFaceTB/SmolLM2-135M") == (0.135, 0.135) and params_billions("gpt2") is None
    lora, full = estimate_run_memory_gb("Qwen/Qwen3-8B", lora=True), estimate_run_memory_gb("Qwen/Qwen3-8B", lora=False)
    assert lora < full and estimate_run_memory_gb("Qwen/Qwen3-8B", lora=True, qlora="nf4") < lora
    assert estimate_run_memory_gb("Qwen/Qwen3-8B", lora=False, gpus=8, zero_level=3) < full / 3
    assert estimate_run_memory_gb("Qwen/Qwen3-8B", lora=False, optimizer="adamw") > full
    assert estimate_run_memory_gb("Qwen/Qwen3-8B", sequence_len=8192) > estimate_run_memory_gb("Qwen/Qwen3-8B", sequence_len=1024)
    assert estimate_run_memory_gb("Qwen/Qwen3-8B", recompute=False) > estimate_run_memory_gb("Qwen/Qwen3-8B", recompute=True)
    assert estimate_run_memory_gb("gpt2") is None
    assert [fit_verdict(10, f) for f in (20, 11, 9, None)] == ["fits", "tight", "risk", "unknown"] and fit_verdict(None, 5) == "unknown"


def test_metrics_pump_splits_a_stream_into_feed_and_log(tmp_path):
    child = ("import sys, json\n"
             "print('provisioning...'); print(json.dumps({'step': 1, 'ts': 0, 'train/loss': 2.0})); print(':: step 1 loss 2.0')\n"
             "print(json.dumps({'type': 'gpu', 'gpu_id': 0, 'step': 1})); sys.stderr.write('warning: x\\n'); print('SUROGATE_EXIT 0')\n")
    proc = subprocess.Popen([sys.executable, "-c", child], stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    seen = []
    t = stream.pump_metrics(proc, str(tmp_path / "feed"), str(tmp_path / "log"), on_line=seen.append)
    proc.wait()
    t.join(10)
    time.sleep(0.1)
    feed = [json.loads(l) for l in open(tmp_path / "feed")]
    assert [r.get("step") for r in feed] == [1, 1] and feed[1]["type"] == "gpu"
    log = open(tmp_path / "log").read()
    assert "provisioning" in log and "train/loss" in log and "warning: x" in log
    assert seen == ["provisioning...", ":: step 1 loss 2.0", "SUROGATE_EXIT 0"]


def test_mirror_reconnects_without_duplicating_bytes(tmp_path):
    remote = tmp_path / "remote.jsonl"
    remote.write_text("line1\nline2\n")
    offsets = []

    def command(offset):  # stands in for ``ssh host tail -c +N -F file``: print from the offset, then drop the link
        offsets.append(offset)
        return [sys.executable, "-c", f"import sys; sys.stdout.write(open({str(remote)!r}).read()[{offset}:])"]

    m = stream.Mirror(command, str(tmp_path / "local.jsonl"), backoff=(0.05,)).start()
    deadline = time.time() + 10
    while len(offsets) < 2 and time.time() < deadline:
        time.sleep(0.02)
    with open(remote, "a") as f:
        f.write("line3\n")
    while m.bytes < 18 and time.time() < deadline:
        time.sleep(0.02)
    m.stop()
    assert open(tmp_path / "local.jsonl").read() == "line1\nline2\nline3\n" and offsets[0] == 0 and 12 in offsets and m.attempts >= 1


def test_local_launch_runs_a_detached_process_with_its_own_feed(tmp_path):
    fake = tmp_path / "fake_surogate"
    fake.write_text("#!/bin/sh\necho \"mode=$1 cfg=$2 gpus=$CUDA_VISIBLE_DEVICES\"\necho '{\"step\": 1, \"ts\": 0, \"train/loss\": 1.5}' >> \"$SUROGATE_METRICS_PATH\"\nsleep 30\n")
    fake.chmod(0o755)
    res = local.launch_local("model: Qwen/Qwen3-0.6B\nmax_steps: 5\noutput_dir: ./out\n", "demo", gpu_ids=[1, 2], root=str(tmp_path / "runs"), surogate_bin=str(fake))
    assert res["ok"]
    run = res["run"]
    cfg = configs.load_overlaid(open(run.config).read())
    assert cfg["gpus"] == 2 and cfg["surogate_metrics_path"] == run.feed and cfg["output_dir"] == run.output and cfg["report_to"] == ["surogate"]
    deadline = time.time() + 10
    while (not os.path.exists(run.feed) or not open(run.log).read()) and time.time() < deadline:
        time.sleep(0.05)
    assert "mode=sft" in open(run.log).read() and "gpus=1,2" in open(run.log).read()
    assert runs.summarise_feed(run.feed)["step"] == 1 and run.read_meta()["gpus"] == [1, 2] and run.read_meta()["max_steps"] == 5
    assert list_runs(str(tmp_path / "runs"))[0]["status"] == "running"
    assert local.stop_local(run)
    deadline = time.time() + 10
    while runs.pid_alive(run.pid_file) and time.time() < deadline:
        try:
            os.waitpid(res["pid"], os.WNOHANG)
        except ChildProcessError:
            pass
        time.sleep(0.05)
    assert not runs.pid_alive(run.pid_file) and not local.stop_local(run)
    assert local.surogate_argv("sft", "c.yaml", 4)[1:5] == ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4"]


class _Done:
    def __init__(self, rc=0, out="", err=""):
        self.returncode, self.stdout, self.stderr = rc, out, err


def test_ssh_launch_copies_the_config_and_starts_a_tmux_session(tmp_path):
    t = ssh.parse_target("me@gpu-box:2222")
    assert (t.host, t.port) == ("me@gpu-box", 2222) and ssh.parse_target("alias").port is None
    assert ssh.ssh_args(t)[-2:] == ["-p", "2222"] and ssh.scp_args(t)[-2:] == ["-P", "2222"] and "BatchMode=yes" in ssh.ssh_args(t)
    calls = []

    def run(argv, **kw):
        calls.append(argv)
        return _Done()

    res = ssh.launch_remote(t, "model: m\nmax_steps: 9\n", "demo", gpu_ids=[0, 1], root=str(tmp_path), run=run, mirror=False)
    assert res["ok"] and [c[0] for c in calls] == ["ssh", "scp", "ssh"]
    rd = res["run"]
    remote_dir = f"~/.surogate-watch/remote/{rd.id}"
    assert calls[0][-1] == f"mkdir -p {remote_dir}" and calls[1][-1] == f"me@gpu-box:{remote_dir}/config.yaml"
    line = calls[2][-1]
    assert f"tmux new-session -d -s {res['session']}" in line and "CUDA_VISIBLE_DEVICES=0,1" in line and f"SUROGATE_METRICS_PATH={remote_dir}/metrics.jsonl" in line
    assert "surogate sft config.yaml > train.log 2>&1 < /dev/null" in line
    meta = rd.read_meta()
    assert meta["remote"] == {"kind": "ssh", "host": "me@gpu-box:2222", "session": res["session"], "dir": remote_dir} and meta["max_steps"] == 9
    assert ssh.follow_command(t, "/r/metrics.jsonl")(120)[-5:] == ["tail", "-c", "+121", "-F", "/r/metrics.jsonl"]
    # a failing step reports the tool's last error line and starts nothing further
    calls.clear()
    res = ssh.launch_remote(t, "model: m\n", "demo", root=str(tmp_path), run=lambda argv, **kw: calls.append(argv) or _Done(255, err="x\nPermission denied (publickey)."), mirror=False)
    assert not res["ok"] and res["reason"] == "Permission denied (publickey)." and len(calls) == 1
    started = []
    assert ssh.stop_remote(t, "sur_ok-1", popen=lambda argv, **kw: started.append(argv)) and started[0][-1] == "tmux kill-session -t sur_ok-1"
    assert not ssh.stop_remote(t, "x; rm -rf ~", popen=lambda *a, **k: started.append(a)) and len(started) == 1
    gpus = ssh.parse_gpu_csv("0, NVIDIA B200, 183359, 12, 3, 10.0\n1, NVIDIA B200, 183359, 100000, 97, 10.0\nnonsense\n")
    assert [g["index"] for g in gpus] == [0, 1] and gpus[1]["util"] == 97.0 and gpus[0]["compute_cap"] == 10.0
    hosts = str(tmp_path / "hosts")
    for h in ("a", "b", "a"):
        ssh.recent_hosts(hosts, remember=h)
    assert ssh.recent_hosts(hosts) == ["a", "b"]
    # fetching an ssh run's outputs is one recursive scp into the run's output directory
    scp = []
    out = artifacts.fetch_artifacts(rd, runner=lambda argv, **kw: scp.append(argv) or _Done(0, "ok"))
    assert out == {"ok": True, "dest": rd.output} and scp[0][:2] == ["scp", "-r"] and scp[0][-2:] == [f"me@gpu-box:{remote_dir}/output/.", rd.output]


def test_dstack_backend_config_is_merged_never_clobbered(tmp_path):
    key = tmp_path / "sa.json"
    key.write_text('{"private": 1}\n')
    assert dstack.backend_entry("gcp", {"project_id": "p", "data_file": str(key)})["creds"]["data"] == '{"private": 1}'
    assert dstack.backend_entry("nebius", {"service_account_id": "s", "public_key_id": "k", "private_key_file": "-----BEGIN\nabc/def\n-----END\n"})["creds"][
        "private_key_content"].startswith("-----BEGIN")
    with pytest.raises(ValueError, match="could not read"):
        dstack.backend_entry("gcp", {"project_id": "p", "data_file": "~/no/such/file.json"})
    with pytest.raises(ValueError, match="missing API key"):
        dstack.backend_entry("runpod", {})
    with pytest.raises(ValueError, match="unknown backend"):
        dstack.backend_entry("k8s", {})
    existing = {"projects": [{"name": "other", "backends": [{"type": "aws"}]}, {"name": "main", "backends": [{"type": "lambda", "creds": {"api_key": "old"}}, {"type": "gcp"}]}], "x": 1}
    doc = dstack.merge_backend(existing, "lambda", {"api_key": "new"})
    main = doc["projects"][1]
    assert [b["type"] for b in main["backends"]] == ["lambda", "gcp"] and main["backends"][0]["creds"]["api_key"] == "new"
    assert doc["projects"][0] == {"name": "other", "backends": [{"type": "aws"}]} and doc["x"] == 1
    assert dstack.merge_backend(None, "runpod", {"api_key": "k"}) == {"projects": [{"name": "main", "backends": [{"type": "runpod", "creds": {"type": "api_key", "api_key": "k"}}]}]}
    with pytest.raises(ValueError, match="not a list"):
        dstack.merge_backend({"projects": {"main": {}}}, "runpod", {"api_key": "k"})
    path = tmp_path / "dstack" / "config.yml"
    assert dstack.configure_backend("runpod", {"api_key": "k1"}, str(path))["ok"] and oct(os.stat(path).st_mode & 0o777) == "0o600"
    assert dstack.configure_backend("aws", {"access_key": "a", "secret_key": "s"}, str(path))["ok"] and os.path.exists(str(path) + ".bak")
    types = [b["type"] for b in yaml.safe_load(open(path))["projects"][0]["backends"]]
    assert types == ["runpod", "aws"]
    path.write_text("projects: [unclosed")
    res = dstack.configure_backend("runpod", {"api_key": "k"}, str(path))
    assert not res["ok"] and "not a valid dstack config" in res["reason"] and path.read_text() == "projects: [unclosed"


def test_dstack_task_embeds_the_config_and_streams_the_feed(tmp_path):
    cfg_text = "model: Qwen/Qwen3-8B\nmax_steps: 4\ndatasets:\n  - path: d.jsonl\n"
    text = dstack.task_yaml("sur-x", dstack.DstackConfig("B200", 8, "img:1", "runpod", "eu"), cfg_text)
    spec = yaml.safe_load(text)
    assert spec["type"] == "task" and spec["resources"] == {"gpu": "B200:8"} and spec["backends"] == ["runpod"] and spec["regions"] == ["eu"]
    script = spec["commands"][0]
    body = script.split("<<'SUROGATE_CONFIG_YAML'\n", 1)[1].split("\nSUROGATE_CONFIG_YAML\n", 1)
    assert yaml.safe_load(body[0]) == yaml.safe_load(cfg_text)
    assert "SUROGATE_METRICS_PATH=metrics.jsonl surogate sft config.yaml > train.log 2>&1 &" in body[1] and body[1].rstrip().endswith("tail -n +1 -F metrics.jsonl")
    assert "|" in text.split("commands:")[1].splitlines()[1]  # a literal block, so the here-document survives as written
    with pytest.raises(ValueError):
        dstack.task_spec("n", dstack.DstackConfig(), "x: SUROGATE_CONFIG_YAML\n")
    child = "import json; print('Provisioning...'); print(json.dumps({'step': 1, 'ts': 0, 'train/loss': 3.0}))"
    started = []

    def popen(argv, **kw):
        started.append(argv)
        return subprocess.Popen([sys.executable, "-c", child], stdout=kw["stdout"], stderr=kw["stderr"])

    res = dstack.launch_dstack(dstack.DstackConfig("B200", 2), cfg_text, "demo", root=str(tmp_path), popen=popen)
    assert res["ok"] and started[0][:4] == ["dstack", "apply", "-y", "--name"] and started[0][4] == res["name"] and len(res["name"]) <= 40
    res["proc"].wait()
    deadline = time.time() + 10
    while runs.summarise_feed(res["feed"])["records"] < 1 and time.time() < deadline:
        time.sleep(0.05)
    rd = res["run"]
    assert runs.summarise_feed(rd.feed)["loss"] == 3.0 and "Provisioning" in open(rd.log).read() and os.path.exists(os.path.join(rd.dir, "task.dstack.yml"))
    assert rd.read_meta()["remote"]["kind"] == "dstack" and not artifacts.fetchable(rd) and not artifacts.fetch_artifacts(rd)["ok"]
    stops = []
    assert dstack.stop_dstack(res["name"], popen=lambda argv, **kw: stops.append(argv)) and stops[0] == ["dstack", "stop", "-y", res["name"]]
    bad = dstack.launch_dstack(dstack.DstackConfig(), cfg_text, "demo", root=str(tmp_path), popen=lambda *a, **k: (_ for _ in ()).throw(FileNotFoundError("dstack")))
    assert not bad["ok"] and "dstack" in bad["reason"]


def test_modal_driver_and_launch(tmp_path):
    compile(modal.DRIVER, "modal_driver.py", "exec")  # the generated driver is valid Python
    assert "sandbox.id" in modal.DRIVER and "SUROGATE_EXIT" in modal.DRIVER and "terminate()" in modal.DRIVER
    env = modal.driver_env(modal.ModalConfig("H100", 2), "a: 1\n", "vol")
    assert env["SUROGATE_LAUNCH_GPU"] == "H100" and env["SUROGATE_LAUNCH_COUNT"] == "2"
    import base64

    assert base64.b64decode(env["SUROGATE_LAUNCH_CONFIG_B64"]).decode() == "a: 1\n"
    assert not modal.launch_modal(modal.ModalConfig("TPU"), "a: 1\n", "x", root=str(tmp_path))["ok"]
    started = []

    def popen(argv, **kw):
        started.append((argv, kw.get("env", {})))
        return subprocess.Popen([sys.executable, "-c", "import json; print(json.dumps({'step': 2, 'ts': 0, 'train/loss': 1.0})); print('SUROGATE_EXIT 0')"],
                                stdout=kw["stdout"], stderr=kw["stderr"])

    res = modal.launch_modal(modal.ModalConfig("B200", 1), "model: m\noutput_dir: ./x\n", "demo", root=str(tmp_path), popen=popen)
    assert res["ok"] and started[0][0][:4] == ["uv", "run", "--with", "modal"] and started[0][1]["SUROGATE_LAUNCH_VOLUME"] == res["volume"]
    rd = res["run"]
    assert configs.load_overlaid(open(rd.config).read())["output_dir"] == "/outputs/model"  # outputs land on the Volume
    res["proc"].wait()
    deadline = time.time() + 10
    while runs.summarise_feed(rd.feed)["records"] < 1 and time.time() < deadline:
        time.sleep(0.05)
    assert runs.summarise_feed(rd.feed)["step"] == 2 and "SUROGATE_EXIT 0" in open(rd.log).read()
    assert not modal.stop_modal(rd)  # no sandbox id yet, driver gone: nothing to stop
    open(os.path.join(rd.dir, "sandbox.id"), "w").write("sb-123")
    kills = []
    assert modal.stop_modal(rd, popen=lambda argv, **kw: kills.append(argv)) and "modal.Sandbox.from_id('sb-123').terminate()" in kills[0][-1]
    open(os.path.join(rd.dir, "sandbox.id"), "w").write("x'); import os; os.system('boom")
    assert not modal.stop_modal(rd, popen=lambda argv, **kw: kills.append(argv)) and len(kills) == 1
    got = []
    out = artifacts.fetch_artifacts(rd, runner=lambda argv, **kw: got.append(argv) or _Done())
    assert out["ok"] and got[0] == ["modal", "volume", "get", "--force", res["volume"], "/model", rd.output] and got[1][5] == "/train.log"


def test_launch_command_line(tmp_path, capsys):
    from surogate_b200.cli import launch as cli
    from surogate_b200.cli.main import COMMAND_MAPPING

    assert COMMAND_MAPPING["launch"] == "surogate_b200.cli.launch"
    root = str(tmp_path / "runs")
    assert cli.main(["run", "--model", "Qwen/Qwen3-0.6B", "--dataset", "d.jsonl", "--target", "dstack", "--count", "2", "--dry-run"]) == 0
    out = capsys.readouterr().out
    assert "model: Qwen/Qwen3-0.6B" in out and "# --- dstack task ---" in out and "gpu: B200:2" in out
    with pytest.raises(SystemExit, match="no dataset picked"):
        cli.main(["run", "--model", "m", "--dry-run"])
    store = str(tmp_path / "providers.json")
    assert cli.main(["providers", "add", "--kind", "ssh", "--key", "me@box", "--gpu", "B200:8", "--store", store]) == 0
    assert "ssh:me@box" in capsys.readouterr().out
    assert cli.main(["providers", "remove", "--key", "ssh:me@box", "--store", store]) == 0 and "(none)" in capsys.readouterr().out
    assert cli.main(["dstack-backend", "runpod", "api_key=k", "--config-path", str(tmp_path / "d.yml")]) == 0
    assert cli.main(["dstack-backend", "runpod", "--config-path", str(tmp_path / "d.yml")]) == 1
    capsys.readouterr()
    assert cli.main(["fit", "--model", "Qwen/Qwen3-8B", "--full", "--gpus", "8", "--zero-level", "3"]) == 0 and "GB per GPU" in capsys.readouterr().out
    rd = new_run("x", root)
    rd.write_meta(mode="sft", max_steps=1)
    assert cli.main(["--runs-dir", root, "runs"]) == 0 and rd.id in capsys.readouterr().out
    assert cli.main(["--runs-dir", root, "stop", rd.id]) == 1 and cli.main(["--runs-dir", root, "fetch", rd.id]) == 0


def test_interactive_dashboard_state_machine(tmp_path):
    """Keys drive the pages: search and line up a model and a dataset, edit launch fields, start a run (through an injected
    launcher), follow it in Monitor, stop it from Runs; every frame renders at any size."""
    from surogate_b200.cli.dashboard import EDITABLE, KEYMAP, PAGES, Dashboard

    feed = tmp_path / "feed.jsonl"
    feed.write_text(json.dumps({"step": 1, "ts": 0, "train/loss": 2.5, "max_steps": 10}) + "\n")
    started = []

    def launcher(target, text, label):
        started.append((target, yaml.safe_load(text), label))
        rd = new_run(f"local-{label}", str(tmp_path / "runs"))
        with open(rd.feed, "w") as f:
            f.write(json.dumps({"step": 3, "ts": 0, "train/loss": 1.25, "max_steps": 7}) + "\n")
        rd.write_meta(mode="sft", model="m", max_steps=7)
        return {"ok": True, "feed": rd.feed, "run": rd}

    d = Dashboard(str(feed), str(tmp_path / "runs"), gpus=lambda: [{"index": 0, "name": "B200", "mem_total": 180 * 2**30, "mem_used": 2**30, "gpu_util": 10}],
                  search_models=lambda q, n: [{"id": "Qwen/Qwen3-0.6B", "architectures": ["Qwen3ForCausalLM"], "downloads": 5}, {"id": "x/y", "architectures": ["Nope"], "downloads": 1}],
                  search_datasets=lambda q, n: [{"id": "org/data", "downloads": 3}], launcher=launcher)
    d.state.poll()
    assert "step 1/10" in d.render(100, 30) and d.name == "Monitor"
    for key in "3/":
        d.on_key(key)
    for ch in "qwen":
        d.on_key(ch)                                   # typed into the search box: 'q' does not quit here
    assert d.input == "qwen" and not d.quit
    d.on_key("backspace")
    d.on_key("enter")
    assert len(d.rows["Models"]) == 2 and "2 result(s) for 'qwe'" in d.message
    frame = d.render(120, 30)
    assert "> " in frame and "Qwen/Qwen3-0.6B" in frame and "yes" in frame
    d.on_key("enter")
    assert d.fields.model == "Qwen/Qwen3-0.6B"
    d.on_key("down")
    d.on_key("enter")
    assert d.fields.model == "x/y" and "not supported" in d.message
    d.on_key("up")
    d.on_key("enter")
    d.on_key("4")
    d.on_key("/")
    for ch in "data":
        d.on_key(ch)
    d.on_key("enter")
    d.on_key("enter")
    assert d.fields.dataset_path == "org/data"
    d.on_key("2")
    assert "GB per GPU" in d.render(100, 30) and "fits" in d.render(100, 30)
    d.on_key("5")
    i = EDITABLE.index("max_steps")
    for _ in range(i):
        d.on_key("down")
    d.on_key("enter")
    assert d.input == "200"
    for _ in range(3):
        d.on_key("backspace")
    for ch in "7x":
        d.on_key(ch)
    d.on_key("enter")
    assert d.fields.max_steps == 200 and "not a valid value" in d.message          # '7x' is refused, the old value stays
    d.on_key("enter")
    for _ in range(3):
        d.on_key("backspace")
    d.on_key("7")
    d.on_key("enter")
    assert d.fields.max_steps == 7
    lora = EDITABLE.index("lora")
    for _ in range(lora - i):
        d.on_key("down")
    d.on_key("enter")
    assert d.fields.lora is False                                                    # booleans toggle
    d.on_key("t")
    d.on_key("+")
    assert d.target == "ssh" and d.gpu_count == 2 and "ssh (h: set host)" in d.render(100, 40)
    for _ in range(3):
        d.on_key("t")
    assert d.target == "local"
    for _ in range(len(EDITABLE) - lora):
        d.on_key("down")
    d.on_key("enter")                                                                # [ start the run ]
    assert started and started[0][0] == "local" and started[0][1]["max_steps"] == 7 and started[0][1]["lora"] is False and started[0][1]["gpus"] == 2
    assert d.name == "Monitor" and "started on local" in d.message
    d.state.poll()
    assert "step 3/7" in d.render(100, 30)
    d.on_key("6")
    assert len(d.rows["Runs"]) == 1 and "running" in d.render(140, 30)
    d.on_key("s")
    assert d.message.startswith("stop:")
    d.on_key("enter")
    assert d.name == "Monitor" and "following" in d.message
    d.on_key("?")
    assert "switch page" in d.render(100, 40)
    d.on_key("x")
    assert not d.help
    d.on_key("tab")
    assert d.name == "GPUs"
    for size in ((60, 10), (200, 60), (20, 5)):
        for page in range(len(PAGES)):
            d.go(page)
            frame = d.render(*size)
            assert len(frame.splitlines()) <= max(size[1], 8) + 2 and all(len(l) <= max(60, size[0]) for l in frame.splitlines())
    empty = Dashboard(str(tmp_path / "none.jsonl"), str(tmp_path / "no-runs"), gpus=lambda: [])
    empty.on_key("5")
    for _ in range(len(EDITABLE)):
        empty.on_key("down")
    empty.on_key("enter")
    assert "cannot start: no model picked" in empty.message
    empty.on_key("6")
    assert "(nothing yet)" in empty.render(100, 20)
    empty.on_key("q")
    assert empty.quit and KEYMAP["\x1b[A"] == "up" and KEYMAP["\r"] == "enter"
