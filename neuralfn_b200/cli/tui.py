"""Terminal front ends: a Rich dashboard for training event streams and an interactive chat
loop for a resident model.

``TrainDashboard`` consumes the JSON lines a native training run prints
(``{"event": "train_step" | "validation" | "checkpoint" | "complete", ...}``) and keeps panels
with progress, throughput, loss curve (sparkline) and the last checkpoint; ``tee`` writes the
raw lines to a log file as well. ``run_train_dashboard`` wraps a child process.

``InferTUI`` is a line-oriented chat loop over ``NativeInferenceModel``: plain lines are user
turns; ``/show`` prints session and speculative-decoding statistics, ``/reset`` clears the
conversation, ``/mode greedy|sample`` switches decoding, ``/tokens N`` sets the reply budget,
``/quit`` leaves. Input and output streams are injectable, so it is testable without a terminal.

Behavioural counterparts: the reference's Rich train TUI (``cli/nfn.py:2323-3125, 3489-3855``) and
``cli/native_infer_tui.py`` (``/show``, ``/reset``, ``/mode``).
"""
from __future__ import annotations

import json
import subprocess
import sys
import time
from typing import IO, Iterable, Sequence

__all__ = ["TrainDashboard", "run_train_dashboard", "InferTUI", "sparkline"]

_BARS = "▁▂▃▄▅▆▇█"


def sparkline(values: Sequence[float], width: int = 40) -> str:
    vals = [v for v in values if v == v][-width:]
    if not vals:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    return "".join(_BARS[min(7, int((v - lo) / span * 7.999))] for v in vals)


class TrainDashboard:
    def __init__(self, total_steps: int | None = None, tee: IO[str] | None = None) -> None:
        self.total_steps, self.tee = total_steps, tee
        self.step, self.losses, self.val_losses = 0, [], []
        self.tokens_per_second = 0.0
        self.last_checkpoint, self.status, self.started = "", "running", time.time()
        self.other: list[str] = []

    def feed(self, line: str) -> None:
        if self.tee is not None:
            self.tee.write(line if line.endswith("\n") else line + "\n")
        line = line.strip()
        if not line.startswith("{"):
            if line:
                self.other = (self.other + [line])[-5:]
            return
        try:
            ev = json.loads(line)
        except json.JSONDecodeError:
            self.other = (self.other + [line])[-5:]
            return
        kind = ev.get("event")
        if kind == "train_step":
            self.step = int(ev.get("step", self.step))
            if "loss" in ev:
                self.losses.append(float(ev["loss"]))
            self.tokens_per_second = float(ev.get("tokens_per_second", self.tokens_per_second))
        elif kind == "validation":
            self.val_losses.append(float(ev.get("loss", float("nan"))))
        elif kind == "checkpoint":
            self.last_checkpoint = str(ev.get("path", ""))
        elif kind == "complete" or ev.get("status") == "ok":
            self.status = "complete"
            self.total_steps = self.total_steps or ev.get("steps")
            self.tokens_per_second = float(ev.get("train_compute_tokens_per_second", self.tokens_per_second))
        elif kind == "error":
            self.status = "failed: " + str(ev.get("message", ""))

    def render(self):
        """A Rich renderable (a plain string when Rich is missing)."""
        frac = (self.step / self.total_steps) if self.total_steps else 0.0
        rows = [("status", self.status), ("step", f"{self.step}" + (f" / {self.total_steps} ({100 * frac:.1f} %)" if self.total_steps else "")),
                ("tokens/s", f"{self.tokens_per_second:,.0f}"), ("train loss", f"{self.losses[-1]:.4f}" if self.losses else "-"),
                ("loss curve", sparkline(self.losses)), ("val loss", f"{self.val_losses[-1]:.4f}" if self.val_losses else "-"),
                ("checkpoint", self.last_checkpoint or "-"), ("elapsed", f"{time.time() - self.started:,.0f} s")]
        try:
            from rich.panel import Panel
            from rich.table import Table
        except ImportError:  # pragma: no cover
            return "\n".join(f"{k:12s} {v}" for k, v in rows)
        t = Table.grid(padding=(0, 2))
        for k, v in rows:
            t.add_row(f"[bold]{k}[/bold]", str(v))
        for line in self.other:
            t.add_row("", f"[dim]{line[:100]}[/dim]")
        return Panel(t, title="nfn train", border_style="green" if self.status == "complete" else "cyan")


def run_train_dashboard(argv: Sequence[str], total_steps: int | None = None, log_file: str | None = None) -> int:  # pragma: no cover - needs a terminal
    """Runs ``argv`` as a child, renders its JSON-line events live, returns its exit code."""
    from rich.live import Live
    tee = open(log_file, "a", encoding="utf-8") if log_file else None
    dash = TrainDashboard(total_steps, tee)
    proc = subprocess.Popen(list(argv), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, bufsize=1)
    try:
        with Live(dash.render(), refresh_per_second=4) as live:
            for line in proc.stdout:  # type: ignore[union-attr]
                dash.feed(line)
                live.update(dash.render())
        return proc.wait()
    finally:
        if tee:
            tee.close()


class InferTUI:
    def __init__(self, model, renderer=None, *, max_new_tokens: int = 128, stdin: Iterable[str] | None = None, stdout: IO[str] | None = None,
                 proposer_factory=None) -> None:
        from ..serving.chat import ChatRenderer
        self.model, self.renderer = model, renderer or ChatRenderer()
        self.max_new_tokens, self.mode = max_new_tokens, "greedy"
        self.stdin, self.out = stdin if stdin is not None else sys.stdin, stdout or sys.stdout
        self.proposer_factory = proposer_factory
        self.history: list = []
        self.session = model.create_session()
        self.totals = {"turns": 0, "prompt_tokens": 0, "completion_tokens": 0, "proposed": 0, "accepted": 0, "seconds": 0.0}

    def _say(self, text: str) -> None:
        self.out.write(text + "\n")
        self.out.flush()

    def command(self, line: str) -> bool:
        """Handles a ``/command``; returns False when the loop should end."""
        parts = line.split()
        cmd = parts[0].lower()
        if cmd in ("/quit", "/exit"):
            return False
        if cmd == "/reset":
            self.session.reset()
            self.history.clear()
            self._say("(conversation cleared)")
        elif cmd == "/mode":
            if len(parts) == 2 and parts[1] in ("greedy", "sample"):
                self.mode = parts[1]
            self._say(f"(mode: {self.mode})")
        elif cmd == "/tokens" and len(parts) == 2 and parts[1].isdigit():
            self.max_new_tokens = int(parts[1])
            self._say(f"(reply budget: {self.max_new_tokens} tokens)")
        elif cmd == "/show":
            t = self.totals
            rate = t["completion_tokens"] / t["seconds"] if t["seconds"] > 0 else 0.0
            acc = f"{t['accepted']}/{t['proposed']}" if t["proposed"] else "off"
            self._say(f"turns {t['turns']} | prompt tokens {t['prompt_tokens']} | reply tokens {t['completion_tokens']} | {rate:.1f} tok/s | "
                      f"speculative accepted {acc} | cached {self.session.cached_tokens} | mode {self.mode}")
        else:
            self._say("commands: /show /reset /mode greedy|sample /tokens N /quit")
        return True

    def turn(self, text: str) -> str:
        from ..serving.chat import ChatMessage, parse_assistant_response
        from ..serving.inference import GenerationConfig
        self.history.append(ChatMessage("user", text))
        prompt = self.renderer.render(self.history, include_assistant_prompt=True)
        ids = self.model.codec.encode(prompt)
        have = list(self.session.token_ids)
        keep = 0
        while keep < min(len(have), len(ids) - 1) and have[keep] == ids[keep]:
            keep += 1
        self.session.truncate(keep)  # reuse the shared prefix of the previous turns
        t0 = time.time()
        self.session.prefill(ids[keep:])
        cfg = GenerationConfig(max_new_tokens=self.max_new_tokens, temperature=0.0 if self.mode == "greedy" else 0.8, top_p=0.95,
                               stop_token_ids=tuple(self.model.manifest.get("stop_token_ids", ())))
        res = self.session.decode(cfg, proposer=self.proposer_factory() if self.proposer_factory else None)
        shown = parse_assistant_response(res.text, self.renderer).visible_text
        self.history.append(ChatMessage("assistant", shown))
        t = self.totals
        t["turns"] += 1
        t["prompt_tokens"] += len(ids) - keep
        t["completion_tokens"] += res.completion_tokens
        t["proposed"] += res.speculative_proposed_tokens
        t["accepted"] += res.speculative_accepted_tokens
        t["seconds"] += time.time() - t0
        return shown

    def run(self) -> int:
        self._say("nfn infer - /show /reset /mode /tokens /quit")
        for raw in self.stdin:
            line = raw.strip()
            if not line:
                continue
            if line.startswith("/"):
                if not self.command(line):
                    break
                continue
            self._say(self.turn(line))
        self.session.close()
        return 0
