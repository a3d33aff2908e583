"""Terminal chat with a training checkpoint.

    python scripts/chat_tui.py <checkpoint_dir> --tokenizer <name or dir>
           [--model-name glm4 --flavor 106B] [--format chatml|plain|raw] [--system "..."]
           [--temperature 0.7 --top-k 50 --max-new-tokens 256 --window 4096]
           [--stream-layers 4] [--plain-ui]

A Textual application (message log, input box, status line; ctrl+r resets the conversation, ctrl+s
saves a transcript, escape interrupts generation).  ``--plain-ui`` is a line-based loop for dumb
terminals.  ``--stream-layers N`` keeps the transformer blocks in pinned host memory and streams N at
a time through the GPU, for checkpoints larger than the device (reference: scripts/chat_tui.py).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from maester_b200.chat import FORMATTERS, ChatSession, GenerationConfig, LayerStreamingRunner, load_model_from_dcp  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="Chat with a DCP checkpoint")
    ap.add_argument("checkpoint_dir")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--model-name")
    ap.add_argument("--flavor")
    ap.add_argument("--format", choices=sorted(FORMATTERS), default="chatml")
    ap.add_argument("--system")
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--window", type=int, default=4096)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--stream-layers", type=int, default=0)
    ap.add_argument("--plain-ui", action="store_true")
    return ap.parse_args(argv)


def build_session(a) -> ChatSession:
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.tokenizer)
    load_device = "cpu" if a.stream_layers else a.device
    model, _ = load_model_from_dcp(a.checkpoint_dir, a.model_name, a.flavor, device=load_device, seq_len=a.window)
    if a.stream_layers:
        model = LayerStreamingRunner(model.to(torch.bfloat16), torch.device(a.device), block=a.stream_layers)
        model.device = torch.device(a.device)
    fmt_cls = FORMATTERS[a.format]
    fmt = fmt_cls(system=a.system) if a.format == "chatml" else fmt_cls()
    return ChatSession(model, tok, fmt, GenerationConfig(a.max_new_tokens, a.temperature, a.top_k, a.window))


def run_plain(session: ChatSession) -> None:
    print("type /reset to clear the conversation, /quit to leave")
    while True:
        try:
            text = input("you> ").strip()
        except (EOFError, KeyboardInterrupt):
            break
        if text in ("/quit", "/exit"):
            break
        if text == "/reset":
            session.reset()
            continue
        if not text:
            continue
        print("model> ", end="", flush=True)
        for piece in session.stream(text):
            print(piece, end="", flush=True)
        print()


def run_tui(session: ChatSession, title: str) -> None:
    from textual.app import App, ComposeResult
    from textual.binding import Binding
    from textual.widgets import Footer, Header, Input, RichLog, Static

    class ChatApp(App):
        TITLE = title
        CSS = "RichLog {height: 1fr;} #status {height: 1; color: $text-muted;}"
        BINDINGS = [Binding("ctrl+r", "reset", "Reset"), Binding("ctrl+s", "save", "Save transcript"),
                    Binding("escape", "interrupt", "Stop"), Binding("ctrl+q", "quit", "Quit")]

        def compose(self) -> ComposeResult:
            yield Header()
            yield RichLog(wrap=True, markup=False, id="log")
            yield Static("ready", id="status")
            yield Input(placeholder="message", id="inp")
            yield Footer()

        def on_input_submitted(self, event: Input.Submitted) -> None:
            text = event.value.strip()
            event.input.value = ""
            if text:
                self.query_one("#log", RichLog).write(f"you: {text}")
                self.run_worker(lambda: self._generate(text), thread=True, exclusive=True)

        def _generate(self, text: str) -> None:
            log, status = self.query_one("#log", RichLog), self.query_one("#status", Static)
            self.call_from_thread(status.update, "generating ...")
            reply, n = "", 0
            for piece in session.stream(text):
                reply += piece
                n += 1
                self.call_from_thread(status.update, f"generating ... {len(reply)} chars")
            self.call_from_thread(log.write, f"model: {reply}")
            self.call_from_thread(status.update, f"ready ({len(session.history)} messages)")

        def action_reset(self) -> None:
            session.reset()
            self.query_one("#log", RichLog).clear()

        def action_save(self) -> None:
            session.save_transcript("chat_transcript.json")
            self.query_one("#status", Static).update("saved chat_transcript.json")

        def action_interrupt(self) -> None:
            session.stop()

    ChatApp().run()


def main(argv=None) -> None:
    a = parse_args(argv)
    session = build_session(a)
    if a.plain_ui or not sys.stdout.isatty():
        run_plain(session)
    else:
        run_tui(session, f"maester_b200 chat - {os.path.basename(os.path.normpath(a.checkpoint_dir))}")


if __name__ == "__main__":
    main()
