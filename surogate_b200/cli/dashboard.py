"""Interactive terminal dashboard: pages for the live run, GPUs, models, datasets, a launch form and the run history.

``surogate monitor --interactive`` (and ``surogate jackalope`` on a terminal) opens it.  The application is a small state machine:
``Dashboard.on_key(key)`` changes the state, ``Dashboard.render(width, height)`` draws the current page as text; the terminal
loop in ``run`` only reads keys and repaints, so everything else is testable without a terminal.

    1-6 / Tab    switch page (Monitor, GPUs, Models, Datasets, Launch, Runs)
    up / down    move the selection (models, datasets, launch fields, runs)
    /            type a search text or a path (Models, Datasets); Enter runs it, the selection is lined up for a launch
    Enter        Launch page: edit the selected field / start the run;   Runs page: follow the selected run in Monitor
    s            Runs page: stop the selected run        f   fetch its outputs
    t            Launch page: cycle the target (local, ssh, dstack, modal)
    ?            help         q   quit

Parity: jackalope/src/ui/{App,Pages,Browse,Launch,Monitor,Sidebar,HelpOverlay}.tsx.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import fields
from typing import Any, Callable, Dict, List, Optional

from . import monitor
from ..launch.configs import LaunchFields, build_config

PAGES = ["Monitor", "GPUs", "Models", "Datasets", "Launch", "Runs"]
TARGETS = ["local", "ssh", "dstack", "modal"]
EDITABLE = ["model", "dataset_path", "dataset_type", "recipe", "max_steps", "learning_rate", "per_device_batch", "grad_accum", "sequence_len", "lora", "lora_rank",
            "optimizer", "output_dir"]


class Dashboard:
    def __init__(self, feed: str = monitor.DEFAULT_FEED, runs_dir: Optional[str] = None, gpus: Callable[[], List[Dict[str, Any]]] = monitor.live_gpus,
                 search_models=None, search_datasets=None, launcher: Optional[Callable[..., Dict[str, Any]]] = None):
        self.state = monitor.FeedState(feed)
        self.runs_dir, self.gpus = runs_dir, gpus
        self.search_models, self.search_datasets, self.launcher = search_models, search_datasets, launcher
        self.page = 0
        self.fields = LaunchFields()
        self.target, self.ssh_host, self.gpu_type, self.gpu_count = "local", "", "B200", 1
        self.rows: Dict[str, List[Dict[str, Any]]] = {"Models": [], "Datasets": [], "Runs": []}
        self.sel: Dict[str, int] = {"Models": 0, "Datasets": 0, "Launch": 0, "Runs": 0}
        self.input: Optional[str] = None        # text being typed (search box or a field's new value)
        self.input_for: Optional[str] = None
        self.message = ""
        self.help = False
        self.quit = False

    # ------------------------------------------------------------------ state changes
    @property
    def name(self) -> str:
        return PAGES[self.page]

    def refresh_runs(self) -> None:
        from ..launch.runs import list_runs

        self.rows["Runs"] = list_runs(self.runs_dir)
        self.sel["Runs"] = min(self.sel["Runs"], max(0, len(self.rows["Runs"]) - 1))

    def go(self, page: int) -> None:
        self.page = page % len(PAGES)
        self.input = self.input_for = None
        if self.name == "Runs":
            self.refresh_runs()

    def _move(self, d: int) -> None:
        n = {"Models": len(self.rows["Models"]), "Datasets": len(self.rows["Datasets"]), "Launch": len(EDITABLE) + 1, "Runs": len(self.rows["Runs"])}.get(self.name, 0)
        if n:
            self.sel[self.name] = (self.sel[self.name] + d) % n

    def _submit_input(self) -> None:
        text, what = (self.input or "").strip(), self.input_for
        self.input = self.input_for = None
        if what == "search" and text:
            try:
                if self.name == "Models":
                    self.rows["Models"] = monitor.browse_models(text, search=self.search_models)
                else:
                    self.rows["Datasets"] = monitor.browse_datasets(text, search=self.search_datasets)
                self.sel[self.name] = 0
                self.message = f"{len(self.rows[self.name])} result(s) for '{text}'"
            except Exception as e:  # noqa: BLE001 - no network, a path that does not exist: say so, stay usable
                self.message = f"search failed: {e}"
        elif what == "ssh":
            self.ssh_host = text
        elif what in EDITABLE:
            cur = getattr(self.fields, what)
            try:
                value: Any = (text.lower() in ("1", "true", "yes", "on")) if isinstance(cur, bool) else type(cur)(text) if not isinstance(cur, str) else text
                setattr(self.fields, what, value)
            except ValueError:
                self.message = f"'{text}' is not a valid value for {what}"

    def _pick(self) -> None:
        rows = self.rows.get(self.name) or []
        if not rows:
            return
        row = rows[self.sel[self.name]]
        if self.name == "Models":
            self.fields.model = row["id"]
            self.message = f"model {row['id']} lined up" + ("" if row.get("trainable", True) else " (architecture not supported)")
        elif self.name == "Datasets":
            self.fields.dataset_path, self.fields.dataset_type = row["id"], row.get("type") or "auto"
            self.message = f"dataset {row['id']} lined up"
        elif self.name == "Runs":
            self.state = monitor.FeedState(os.path.join(row["dir"], "metrics.jsonl"))
            self.message = f"following {row['run']}"
            self.go(0)

    def start_run(self) -> None:
        bad = self.fields.problems()
        if bad:
            self.message = "cannot start: " + "; ".join(bad)
            return
        text = build_config(self.fields, n_gpus=self.gpu_count)
        label = os.path.basename(self.fields.model.rstrip("/")) or "run"
        try:
            res = (self.launcher or self._launch)(self.target, text, label)
        except Exception as e:  # noqa: BLE001
            res = {"ok": False, "reason": str(e)}
        if not res.get("ok"):
            self.message = f"launch failed: {res.get('reason')}"
            return
        self.state = monitor.FeedState(res["feed"])
        self.message = f"started on {self.target}: {res['feed']}"
        self.go(0)

    def _launch(self, target: str, text: str, label: str) -> Dict[str, Any]:
        if target == "local":
            from ..launch.local import launch_local

            return launch_local(text, label, root=self.runs_dir)
        if target == "ssh":
            from ..launch.ssh import launch_remote, parse_target

            if not self.ssh_host:
                return {"ok": False, "reason": "no ssh host set (press h on the Launch page)"}
            return launch_remote(parse_target(self.ssh_host), text, label, root=self.runs_dir)
        if target == "dstack":
            from ..launch.dstack import DstackConfig, launch_dstack

            return launch_dstack(DstackConfig(self.gpu_type, self.gpu_count), text, label, root=self.runs_dir)
        from ..launch.modal import ModalConfig, launch_modal

        return launch_modal(ModalConfig(self.gpu_type, self.gpu_count), text, label, root=self.runs_dir)

    def _run_action(self, what: str) -> None:
        rows = self.rows["Runs"]
        if not rows:
            return
        from .launch import main as launch_cli

        argv = (["--runs-dir", self.runs_dir] if self.runs_dir else []) + [what, rows[self.sel["Runs"]]["run"]]
        import contextlib
        import io

        buf = io.StringIO()
        with contextlib.redirect_stdout(buf), contextlib.redirect_stderr(buf):
            rc = launch_cli(argv)
        self.message = f"{what}: " + (buf.getvalue().strip().splitlines() or ["done" if rc == 0 else "nothing to do"])[-1]
        self.refresh_runs()

    def on_key(self, key: str) -> None:
        """``key``: one character, or 'up' / 'down' / 'enter' / 'tab' / 'backspace' / 'esc'."""
        if self.input is not None:
            if key == "enter":
                self._submit_input()
            elif key == "esc":
                self.input = self.input_for = None
            elif key == "backspace":
                self.input = self.input[:-1]
            elif len(key) == 1 and key.isprintable():
                self.input += key
            return
        if self.help:
            self.help = False
            return
        if key == "q":
            self.quit = True
        elif key == "?":
            self.help = True
        elif key == "tab":
            self.go(self.page + 1)
        elif key in "123456" and len(key) == 1:
            self.go(int(key) - 1)
        elif key == "up":
            self._move(-1)
        elif key == "down":
            self._move(1)
        elif key == "/" and self.name in ("Models", "Datasets"):
            self.input, self.input_for = "", "search"
        elif key == "enter":
            if self.name == "Launch":
                i = self.sel["Launch"]
                if i == len(EDITABLE):
                    self.start_run()
                elif isinstance(getattr(self.fields, EDITABLE[i]), bool):
                    setattr(self.fields, EDITABLE[i], not getattr(self.fields, EDITABLE[i]))
                else:
                    self.input, self.input_for = str(getattr(self.fields, EDITABLE[i])), EDITABLE[i]
            else:
                self._pick()
        elif self.name == "Launch" and key == "t":
            self.target = TARGETS[(TARGETS.index(self.target) + 1) % len(TARGETS)]
        elif self.name == "Launch" and key == "h":
            self.input, self.input_for = self.ssh_host, "ssh"
        elif self.name == "Launch" and key in "+-":
            self.gpu_count = max(1, self.gpu_count + (1 if key == "+" else -1))
        elif self.name == "Runs" and key == "s":
            self._run_action("stop")
        elif self.name == "Runs" and key == "f":
            self._run_action("fetch")
        elif self.name == "Runs" and key == "r":
            self.refresh_runs()

    # ------------------------------------------------------------------ drawing
    def _listing(self, rows: List[Dict[str, Any]], cols: List[str], sel: int, height: int) -> List[str]:
        if not rows:
            return ["(nothing yet)"]
        shown = [{c: r.get(c, "") for c in cols} for r in rows]
        lines = monitor.table(shown).splitlines()
        top = max(0, min(sel - height // 2, len(rows) - height))
        body = lines[2:][top:top + max(1, height)]
        return lines[:2] + [("> " if top + i == sel else "  ") + l for i, l in enumerate(body)]

    def render(self, width: int = 100, height: int = 30) -> str:
        w = max(60, width)
        tabs = "  ".join(f"[{i + 1} {p}]" if i == self.page else f" {i + 1} {p} " for i, p in enumerate(PAGES))
        out = [tabs[:w], "─" * w]
        body_h = max(5, height - 6)
        if self.help:
            out += [l.strip() for l in (__doc__ or "").splitlines() if "   " in l and not l.strip().startswith("Parity")]
        elif self.name == "Monitor":
            out += monitor.render(self.state, w, None).splitlines()
        elif self.name == "GPUs":
            gpus = self.gpus() or []
            from ..launch.fit import estimate_run_memory_gb, fit_verdict

            est = estimate_run_memory_gb(self.fields.model, self.fields.recipe, self.fields.lora, per_device_batch=self.fields.per_device_batch,
                                         sequence_len=self.fields.sequence_len, recompute=self.fields.recompute) if self.fields.model else None
            out.append(f"run estimate: {'pick a model first' if not self.fields.model else 'unknown' if est is None else f'~{est} GB per GPU'}")
            for i, g in enumerate(gpus):
                total, used = float(g.get("mem_total", 0) or 0), float(g.get("mem_used", 0) or 0)
                free = (total - used) / 2 ** 30 if total else None
                out.append(f"gpu{g.get('index', i)}  {g.get('name', '')}  {monitor.bar(float(g.get('gpu_util', 0) or 0) / 100.0)}  "
                           f"{'?' if free is None else f'{free:.0f} GB free'}  {fit_verdict(est, free)}")
            if not gpus:
                out.append("no local GPUs visible (NVML not available); saved providers: surogate launch providers")
        elif self.name in ("Models", "Datasets"):
            cols = ["id", "architecture", "trainable", "downloads"] if self.name == "Models" else ["id", "type", "bytes", "downloads"]
            out.append("press / and type a HuggingFace search text, or a path starting with / ~ .   Enter lines the selection up for a launch")
            out += self._listing(self.rows[self.name], cols, self.sel[self.name], body_h - 3)
        elif self.name == "Launch":
            for i, name in enumerate(EDITABLE):
                out.append(("> " if i == self.sel["Launch"] else "  ") + f"{name:18s} {getattr(self.fields, name)}")
            out.append(("> " if self.sel["Launch"] == len(EDITABLE) else "  ") + "[ start the run ]")
            where = {"ssh": f"ssh {self.ssh_host or '(h: set host)'}", "dstack": f"dstack {self.gpu_type}:{self.gpu_count}", "modal": f"Modal {self.gpu_type}:{self.gpu_count}"}
            out.append(f"target (t): {where.get(self.target, 'this machine')}    GPUs (+/-): {self.gpu_count}")
        elif self.name == "Runs":
            out.append("Enter follows a run   s stops it   f fetches its outputs   r refreshes")
            out += self._listing(self.rows["Runs"], ["run", "status", "where", "model", "step", "max_steps", "loss", "eval_loss", "checkpoints"], self.sel["Runs"], body_h - 3)
        out = out[:height - 2]
        out += [""] * max(0, height - 2 - len(out))
        prompt = f"{self.input_for}> {self.input}_" if self.input is not None else self.message
        out += ["─" * w, (prompt or "? help   q quit")[:w]]
        return "\n".join(l[:w] for l in out)


# ---------------------------------------------------------------------- terminal loop
KEYMAP = {"\x1b[A": "up", "\x1b[B": "down", "\r": "enter", "\n": "enter", "\t": "tab", "\x7f": "backspace", "\x08": "backspace", "\x1b": "esc"}


def read_key(fd: int, timeout_s: float) -> Optional[str]:
    import select

    r, _, _ = select.select([fd], [], [], timeout_s)
    if not r:
        return None
    data = os.read(fd, 8).decode("utf-8", "ignore")
    return KEYMAP.get(data, data[:1] if data else None)


def run(dash: Dashboard, interval_s: float = 0.5) -> int:
    """Raw-mode loop on the controlling terminal: poll the feed, repaint, read a key.  The terminal's settings are restored on
    every way out."""
    import shutil
    import termios
    import tty

    fd = sys.stdin.fileno()
    saved = termios.tcgetattr(fd)
    try:
        tty.setcbreak(fd)
        sys.stdout.write("\x1b[?1049h\x1b[?25l")   # alternate screen, cursor hidden
        last = 0.0
        while not dash.quit:
            if time.time() - last >= interval_s:
                dash.state.poll()
                size = shutil.get_terminal_size((100, 30))
                sys.stdout.write("\x1b[H\x1b[2J" + dash.render(size.columns, size.lines))
                sys.stdout.flush()
                last = time.time()
            key = read_key(fd, interval_s)
            if key is not None:
                dash.on_key(key)
                last = 0.0
    except KeyboardInterrupt:
        pass
    finally:
        sys.stdout.write("\x1b[?25h\x1b[?1049l")
        sys.stdout.flush()
        termios.tcsetattr(fd, termios.TCSADRAIN, saved)
    return 0
