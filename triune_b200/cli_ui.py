"""Terminal rendering for the command line: banner, key/value cards, tables, notices, the telemetry line after a
generation, a spinner. With ``rich`` installed and a terminal attached the output is styled; otherwise (pipes, logs,
machines without ``rich``) the same information is printed as plain text. Everything goes through ``print`` so that
captured output in tests and logs sees it. Parity: ``triune/cli_ui.py:25-396`` of the reference (same function names and
arguments)."""

from __future__ import annotations

import contextlib
import io
import os
import shutil
import sys
from typing import Any, Iterable, List, Optional, Sequence, Tuple

try:
    from rich import box
    from rich.console import Console
    from rich.panel import Panel
    from rich.rule import Rule
    from rich.table import Table
    from rich.text import Text

    HAS_RICH = True
except ImportError:  # plain text only
    HAS_RICH = False

_TIER_STYLE = (("REFLEX", "REFLEX", "bold green", "32"), ("LIMBIC", "LIMBIC", "bold yellow", "33"), ("CORTEX", "CORTEX", "bold magenta", "35"),
               ("OLLAMA", "OLLAMA", "bold blue", "34"), ("SPEC", "SPECULATIVE", "bold cyan", "36"))


def ensure_utf8_stdio() -> None:
    """Make stdout / stderr UTF-8 (Windows consoles and pipes default to a code page that cannot print box characters)."""
    os.environ.setdefault("PYTHONUTF8", "1")
    os.environ.setdefault("PYTHONIOENCODING", "utf-8")
    for stream in (sys.stdout, sys.stderr):
        reconf = getattr(stream, "reconfigure", None)
        if callable(reconf):
            try:
                reconf(encoding="utf-8", errors="replace")
            except (ValueError, OSError):
                pass


def is_tty() -> bool:
    try:
        return bool(sys.stdout.isatty())
    except (AttributeError, ValueError):
        return False


def _width() -> int:
    cols = shutil.get_terminal_size(fallback=(120, 30)).columns
    return max(60, min(cols, 140 if is_tty() else 120))


def emit_renderable(renderable: Any) -> None:
    """Render a rich object (or anything printable) to text and ``print`` it: colours only on a terminal."""
    if not HAS_RICH or isinstance(renderable, str) and not is_tty():
        print(_strip_markup(str(renderable)))
        return
    buf = io.StringIO()
    tty = is_tty()
    Console(file=buf, width=_width(), force_terminal=tty, color_system="truecolor" if tty else None, legacy_windows=False,
            highlight=False).print(renderable)
    print(buf.getvalue().rstrip("\n"))


def _strip_markup(text: str) -> str:
    if HAS_RICH:
        try:
            return Text.from_markup(text).plain
        except Exception:
            return text
    import re

    return re.sub(r"\[/?[a-z_ #0-9]*\]", "", text)


def _tier(route: str) -> Tuple[str, str, str]:
    r = str(route or "AUTO").upper()
    for key, label, style, ansi in _TIER_STYLE:
        if key in r:
            return label, style, ansi
    return (r or "AUTO"), "bold white", "37"


def route_badge_markup(route: str) -> str:
    """The exit tier (or backend) of a reply as rich markup: green Reflex, yellow Limbic, magenta Cortex, blue Ollama."""
    label, style, _ = _tier(route)
    return f"[{style}] {label} [/]"


def route_badge_ansi(route: str) -> str:
    """The same badge with ANSI colours for prompts that bypass rich; plain ``[LABEL]`` when stdout is not a terminal."""
    label, _, ansi = _tier(route)
    return f"\x1b[1;{ansi}m[{label}]\x1b[0m" if is_tty() else f"[{label}]"


def render_banner(title: str = "TRIUNE B200", subtitle: Optional[str] = None, badge: Optional[str] = None) -> None:
    if not HAS_RICH:
        print(f"\n== {title}{f'  [{badge}]' if badge else ''} ==")
        if subtitle:
            print(f"   {subtitle}")
        return
    head = Text(title, style="bold cyan")
    if badge:
        head.append(f"  {badge}", style="bold black on cyan")
    if subtitle:
        head.append(f"\n{subtitle}", style="dim")
    emit_renderable(Panel(head, box=box.ROUNDED, border_style="cyan", padding=(0, 2), expand=False))


def render_kv_panel(title: str, rows: Iterable[Tuple[str, Any]], *, border_style: str = "bright_black", footer: Optional[str] = None) -> None:
    rows = [(str(k), v) for k, v in rows]
    if not HAS_RICH:
        print(f"\n[{title}]")
        w = max((len(k) for k, _ in rows), default=12)
        for k, v in rows:
            print(f"  {k:<{w}} : {v}")
        if footer:
            print(f"  {footer}")
        return
    grid = Table.grid(padding=(0, 2))
    grid.add_column(style="dim", no_wrap=True)
    grid.add_column(style="white", overflow="fold")
    for k, v in rows:
        grid.add_row(k, str(v))
    emit_renderable(Panel(grid, title=f"[bold]{title}[/]", title_align="left", subtitle=footer, subtitle_align="left",
                          box=box.ROUNDED, border_style=border_style, expand=False))


def render_table(title: str, columns: Sequence[Tuple[str, str, str]], rows: Sequence[Sequence[Any]], *, caption: Optional[str] = None,
                 border_style: str = "bright_black") -> None:
    """``columns`` are (header, justification, style) triples."""
    if not HAS_RICH:
        print(f"\n{title}")
        widths = [max(len(str(h)), *(len(str(r[i])) for r in rows)) if rows else len(str(h)) for i, (h, _, _) in enumerate(columns)]
        line = "  ".join(f"{str(h):<{w}}" for (h, _, _), w in zip(columns, widths))
        print(line)
        print("-" * len(line))
        for r in rows:
            print("  ".join(f"{str(c):>{w}}" if j == "right" else f"{str(c):<{w}}" for c, w, (_, j, _) in zip(r, widths, columns)))
        if caption:
            print(caption)
        return
    t = Table(title=title, title_justify="left", caption=caption, caption_justify="left", box=box.ROUNDED, border_style=border_style,
              header_style="bold", show_lines=False)
    for header, justify, style in columns:
        t.add_column(str(header), justify=justify or "left", style=style or None, overflow="fold")
    for r in rows:
        t.add_row(*[str(c) for c in r])
    emit_renderable(t)


def render_notice(message: str, level: str = "info") -> None:
    icon = {"info": "•", "success": "✓", "warn": "!", "error": "✗"}.get(level, "•")
    style = {"info": "cyan", "success": "bold green", "warn": "bold yellow", "error": "bold red"}.get(level, "cyan")
    if not HAS_RICH:
        print(f"{icon} {message}")
        return
    emit_renderable(Text.assemble((f"{icon} ", style), (str(message), style if level == "error" else "")))


def render_telemetry_bar(route: str, *, tok_sec: float = 0.0, ttft_ms: Optional[float] = None, tokens: int = 0, latency_ms: float = 0.0,
                         vram_gb: float = 0.0, load_s: Optional[float] = None, extra: Optional[str] = None) -> None:
    """One line under a generation: exit tier, decode rate, time to first token, token count and latency, device memory."""
    parts = [route_badge_markup(route), f"[bold cyan]{tok_sec:.1f} tok/s[/]", f"[dim]TTFT[/] [yellow]{f'{ttft_ms:.1f}ms' if ttft_ms else 'N/A'}[/]",
             f"[dim]Tokens[/] [white]{tokens}[/] [dim]({latency_ms:.0f}ms)[/]"]
    if vram_gb > 0:
        parts.append(f"[dim]VRAM[/] [white]{vram_gb:.2f}GB[/]")
    if load_s is not None:
        parts.append(f"[dim]Load[/] [white]{load_s:.1f}s[/]")
    if extra:
        parts.append(f"[dim]{extra}[/]")
    line = "  [dim]│[/]  ".join(parts)
    if not HAS_RICH:
        print(_strip_markup(line))
        return
    emit_renderable(Text.from_markup(line))


def render_rule(title: str = "") -> None:
    if not HAS_RICH:
        print(f"\n--- {title} ---" if title else "\n" + "-" * 60)
        return
    emit_renderable(Rule(title=title, style="bright_black"))


@contextlib.contextmanager
def _note(message: str):
    print(f"... {message}")
    yield


def status_spinner(message: str):
    """Context manager: an animated spinner on a terminal, a single status line elsewhere."""
    if HAS_RICH and is_tty():
        return Console(force_terminal=True, legacy_windows=False).status(f"[cyan]{message}[/]", spinner="dots")
    return _note(message)


_COMMAND_GROUPS: List[Tuple[str, List[Tuple[str, str]]]] = [
    ("Run", [("chat", "interactive chat with a checkpoint, a Hugging Face directory, a GGUF file or ollama:<tag>"),
             ("infer", "one prompt, one reply (--depth reflex|limbic|cortex|auto, --speculative)"),
             ("serve", "OpenAI-compatible HTTP server with the Studio page"), ("desktop / studio", "start or reuse the server and open its page")]),
    ("Train", [("train", "pre-train from a run configuration (one process per GPU under torchrun)"), ("finetune", "LoRA fine-tuning on a text or JSONL file"),
               ("adapter", "list, merge or export LoRA adapters"), ("rescue", "repair a starved deep exit of a checkpoint")]),
    ("Models", [("models", "the model presets"), ("scan", "model files on this machine (checkpoints, Hugging Face, GGUF, Ollama)"),
                ("transmute", "convert a dense Hugging Face model into the multi-exit MoE layout"), ("checkpoint / export", "inspect, merge and export checkpoints"),
                ("cache / cache-nvfp4", "build an NVFP4 layer cache on disk")]),
    ("Machine", [("doctor / info", "what this installation can do on this machine"), ("gpucheck", "GPU, driver and kernel extension check"),
                 ("plan-memory", "memory plan of a model and batch on a GPU"), ("bench / benchmark", "training throughput"), ("profile", "time one training step by phase"),
                 ("native / build-native", "build the CUDA extension and the C engine"), ("install / uninstall", "set this machine up")]),
    ("Extend", [("plugin", "scaffold, sign and list plugins"), ("agent", "run the agent harness on a goal"), ("sandbox", "run Python in the restricted sandbox"),
                ("tokenizer", "train or inspect tokenizers"), ("eval", "evaluation suites")]),
]


def render_help_overview() -> None:
    """The grouped command overview shown by ``--help`` on a terminal."""
    render_banner("TRIUNE B200", subtitle="python -m triune_b200 <command> [options]   (add -h to a command for its options)")
    for group, cmds in _COMMAND_GROUPS:
        render_table(group, [("command", "left", "bold cyan"), ("what it does", "left", "")], [[c, d] for c, d in cmds])
