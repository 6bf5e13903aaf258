"""A run inside a Modal GPU sandbox.

The launcher writes a small driver script next to the run and starts it with ``uv run --with modal`` (the SDK is then importable
however the user installed the client; it authenticates from the user's Modal token file).  The driver creates a sandbox from a
trainer image with a named Volume mounted at ``/outputs``, writes the config into it, runs the trainer with feed and log on the
Volume, and prints both back: feed records drive the monitor, log lines surface progress and any crash, and a final
``SUROGATE_EXIT <code>`` line reports the trainer's status.  The sandbox id is saved beside the run so the sandbox can be ended
later by a fresh process: a launcher that died must never strand a paid GPU.

Parity: jackalope/src/modal.ts.
"""
from __future__ import annotations

import base64
import os
import re
import subprocess
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .configs import load_overlaid
from .runs import RunDir, new_run
from .stream import pump_metrics, register

MODAL_GPUS = ("T4", "L4", "A10", "L40S", "A100-40GB", "A100-80GB", "H100", "H200", "B200")
DEFAULT_IMAGE = "surogate-b200:latest"

DRIVER = r'''"""Driver of one training run in a Modal sandbox; every input comes from the environment."""
import base64
import os
import signal
import sys

import modal

env = os.environ
gpu = env.get("SUROGATE_LAUNCH_GPU", "B200")
count = env.get("SUROGATE_LAUNCH_COUNT", "1")
gpu = gpu if count in ("", "1") else f"{gpu}:{count}"
mode = env.get("SUROGATE_LAUNCH_MODE", "sft")
config_b64 = env["SUROGATE_LAUNCH_CONFIG_B64"]
base64.b64decode(config_b64)  # fail here, not on the sandbox, if the payload is damaged

app = modal.App.lookup("surogate-launch", create_if_missing=True)
volume = modal.Volume.from_name(env.get("SUROGATE_LAUNCH_VOLUME", "surogate-run"), create_if_missing=True)
# the image's own entry point is cleared: the sandbox must idle until exec() starts the trainer
image = modal.Image.from_registry(env.get("SUROGATE_LAUNCH_IMAGE", "surogate-b200:latest"), add_python="3.12").entrypoint([])

print(f"launch: creating a {gpu} sandbox", file=sys.stderr, flush=True)
sandbox = modal.Sandbox.create(app=app, image=image, gpu=gpu, timeout=24 * 3600, volumes={"/outputs": volume}, workdir="/root")
try:
    with open("sandbox.id", "w") as f:
        f.write(sandbox.object_id or "")
except OSError:
    pass


def end(*_):
    try:
        sandbox.terminate()
    finally:
        os._exit(1)


signal.signal(signal.SIGTERM, end)
signal.signal(signal.SIGINT, end)
try:
    sandbox.exec("bash", "-lc", f"mkdir -p /outputs && echo {config_b64} | base64 -d > /root/config.yaml").wait()
    script = (
        "cd /root && touch /outputs/metrics.jsonl /outputs/train.log && "
        f"(SUROGATE_METRICS_PATH=/outputs/metrics.jsonl surogate {mode} config.yaml > /outputs/train.log 2>&1; echo $? > /outputs/DONE) & "
        "tail -n +1 -F /outputs/metrics.jsonl & FEED=$!; tail -n +1 -F /outputs/train.log & LOG=$!; "
        "while [ ! -f /outputs/DONE ]; do sleep 2; done; sleep 2; kill $FEED $LOG 2>/dev/null; echo SUROGATE_EXIT $(cat /outputs/DONE)"
    )
    proc = sandbox.exec("bash", "-lc", script)
    for line in proc.stdout:
        sys.stdout.write(line)
        sys.stdout.flush()
    proc.wait()
finally:
    sandbox.terminate()
'''


@dataclass
class ModalConfig:
    gpu: str = "B200"
    count: int = 1
    image: str = DEFAULT_IMAGE


def volume_name(run_id: str) -> str:
    return re.sub(r"[^a-z0-9-]", "-", f"surogate-{run_id}".lower())[:50]


def driver_env(cfg: ModalConfig, config_text: str, volume: str, mode: str = "sft") -> Dict[str, str]:
    return {"SUROGATE_LAUNCH_GPU": cfg.gpu, "SUROGATE_LAUNCH_COUNT": str(max(1, cfg.count)), "SUROGATE_LAUNCH_MODE": mode,
            "SUROGATE_LAUNCH_IMAGE": cfg.image or DEFAULT_IMAGE, "SUROGATE_LAUNCH_VOLUME": volume,
            "SUROGATE_LAUNCH_CONFIG_B64": base64.b64encode(config_text.encode()).decode()}


def launch_modal(cfg: ModalConfig, config_text: str, label: str, mode: str = "sft", root: Optional[str] = None, popen=subprocess.Popen) -> Dict[str, Any]:
    if cfg.gpu not in MODAL_GPUS:
        return {"ok": False, "reason": f"Modal offers {', '.join(MODAL_GPUS)}; got {cfg.gpu}"}
    rd = new_run(f"modal-{label}", root)
    volume = volume_name(rd.id)
    on_volume = config_text.rstrip() + "\noutput_dir: /outputs/model\n"  # outputs must land on the Volume to be fetched later
    driver = os.path.join(rd.dir, "modal_driver.py")
    try:
        with open(rd.config, "w") as f:
            f.write(on_volume)
        with open(driver, "w") as f:
            f.write(DRIVER)
        proc = popen(["uv", "run", "--with", "modal", "python", driver], cwd=rd.dir, env=dict(os.environ, **driver_env(cfg, on_volume, volume, mode)),
                     stdin=subprocess.DEVNULL, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    except OSError as e:
        return {"ok": False, "reason": f"could not start the Modal driver ({e}); is uv installed?", "run": rd}
    pump_metrics(proc, rd.feed, rd.log)
    register(proc)
    c = load_overlaid(on_volume)
    rd.write_meta(mode=mode, label=f"modal-{label}", model=c.get("model"), recipe=c.get("recipe"), max_steps=c.get("max_steps"),
                  remote={"kind": "modal", "host": f"Modal · {cfg.gpu}:{cfg.count}", "session": volume, "dir": "(modal volume)"})
    return {"ok": True, "run": rd, "feed": rd.feed, "name": volume, "volume": volume, "proc": proc}


def stop_modal(run: RunDir, proc: Optional[subprocess.Popen] = None, popen=subprocess.Popen) -> bool:
    """End the sandbox by its saved id from a fresh process (works after the driver has gone), then end the local driver."""
    stopped = False
    try:
        with open(os.path.join(run.dir, "sandbox.id")) as f:
            sid = f.read().strip()
    except OSError:
        sid = ""
    if sid and re.fullmatch(r"[A-Za-z0-9_-]+", sid):
        try:
            popen(["uv", "run", "--with", "modal", "python", "-c", f"import modal; modal.Sandbox.from_id({sid!r}).terminate()"],
                  stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL, start_new_session=True)
            stopped = True
        except OSError:
            pass
    if proc is not None and proc.poll() is None:
        proc.terminate()
        stopped = True
    return stopped
