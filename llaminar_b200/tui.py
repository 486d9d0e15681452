"""Full-screen interactive chat (`chat --tui`): transcript pane with scroll-back, input line with history, status bar.

The reference's interactive mode is an FTXUI application (reference: src/v2/app/modes/InteractiveChatMode.cpp,
src/v2/utils/ChatUI.cpp).  Here the terminal-independent parts (conversation state, wrapping, scrolling, line editing)
are plain classes that are tested without a terminal; `run` is a thin `curses` driver around them.  Generation goes
through the same engine calls as the line-oriented `chat` command, one step per screen refresh, so tokens appear as
they are produced.
"""
from __future__ import annotations

import textwrap
import time
from dataclasses import dataclass, field


class ChatSession:
    """Conversation state and token streaming over an engine (or its replicated front on rank 0)."""

    def __init__(self, drive, tok, template, ctx_size: int, make_sampling, system_prompt: str | None = None):
        self.drive, self.tok, self.template, self.ctx_size, self.make_sampling = drive, tok, template, ctx_size, make_sampling
        self.base = [{"role": "system", "content": system_prompt}] if system_prompt else []
        self.history: list[dict] = list(self.base)
        self.eos = tuple(dict.fromkeys(i for i in (tok.eos_id, tok.vocab.get("<|im_end|>"), tok.vocab.get("<|endoftext|>"))
                                       if i is not None))
        self.prompt_tokens = 0
        self.generated = 0
        self.last_tok_s = 0.0

    def reset(self) -> None:
        self.history = list(self.base)
        self.prompt_tokens = self.generated = 0
        self.drive.clear_cache()

    @property
    def context_used(self) -> int:
        return self.prompt_tokens + self.generated

    def ask(self, text: str):
        """Generator of (kind, piece) with kind "reasoning" or "content" while the answer streams; the finished answer
        joins the history.  Raises ValueError when the conversation no longer fits the context window."""
        from .tokenizer.bpe import StreamDecoder
        from .tokenizer.chat_template import ThinkSplitter
        self.history.append({"role": "user", "content": text})
        ids = self.tok.encode(self.template.render(self.history), add_special=True)
        if len(ids) + 2 >= self.ctx_size:
            self.history.pop()
            raise ValueError("context window exhausted; /reset to start over")
        sp = self.make_sampling()
        sp.max_tokens = min(sp.max_tokens, self.ctx_size - len(ids) - 1)
        sp.stop_token_ids = self.eos
        req = self.drive.add_request(ids, sp)
        self.prompt_tokens, self.generated = len(ids), 0
        dec, split, answer = StreamDecoder(self.tok), ThinkSplitter(), []
        t0 = time.perf_counter()

        def emit(pair):
            r, c = pair
            if r:
                yield "reasoning", r
            if c:
                answer.append(c)
                yield "content", c

        try:
            while req.state != "finished":
                for o in self.drive.step():
                    if o.rid != req.rid:
                        continue
                    for t in o.new_tokens:
                        self.generated += 1
                        self.last_tok_s = self.generated / max(time.perf_counter() - t0, 1e-9)
                        yield from emit(split.push(dec.push(t)))
            yield from emit(split.push(dec.flush()))
            yield from emit(split.flush())
        finally:
            if req.state != "finished":                    # the consumer went away in mid-answer
                self.drive.abort(req.rid)
            self.drive.requests.pop(req.rid, None)
            self.history.append({"role": "assistant", "content": "".join(answer)})


@dataclass
class ChatView:
    """What is on the screen, independent of the terminal: transcript entries, wrapped lines, scroll offset."""
    width: int = 80
    height: int = 24
    entries: list = field(default_factory=list)          # [role, text]
    scroll: int = 0                                       # lines above the bottom (0 follows the newest text)

    PREFIX = {"user": "you  ", "assistant": "model", "reasoning": "think", "system": "sys  ", "info": "     "}

    def add(self, role: str, text: str = "") -> None:
        self.entries.append([role, text])

    def append(self, role: str, text: str) -> None:
        """Streams text into the last entry of this role (a new entry when the role changes)."""
        if not self.entries or self.entries[-1][0] != role:
            self.add(role)
        self.entries[-1][1] += text

    def lines(self) -> list[tuple[str, str]]:
        """(role, line) for the whole transcript, wrapped to the pane; the role label is on an entry's first line."""
        body = max(self.width - 8, 8)
        out = []
        for role, text in self.entries:
            first = True
            for para in (text.split("\n") if text else [""]):
                for ln in textwrap.wrap(para, body, replace_whitespace=False, drop_whitespace=False) or [""]:
                    out.append((role, f"{self.PREFIX.get(role, role[:5]):<5} | {ln}" if first else f"      | {ln}"))
                    first = False
        return out

    @property
    def pane_height(self) -> int:
        return max(self.height - 3, 1)                    # status bar, separator, input line

    def visible(self) -> list[tuple[str, str]]:
        ls = self.lines()
        self.scroll = max(0, min(self.scroll, max(len(ls) - self.pane_height, 0)))
        end = len(ls) - self.scroll
        return ls[max(end - self.pane_height, 0):end]

    def scroll_by(self, delta: int) -> None:
        self.scroll = max(0, self.scroll + delta)
        self.visible()                                    # clamps

    def resize(self, width: int, height: int) -> None:
        self.width, self.height = max(width, 20), max(height, 5)

    def status(self, model: str, used: int, ctx: int, tok_s: float, busy: bool) -> str:
        s = f" {model} | context {used}/{ctx} | {tok_s:5.1f} tok/s | {'generating...' if busy else 'Enter: send  PgUp/PgDn: scroll  /reset  /exit'}"
        return s[:self.width - 1].ljust(self.width - 1)


class LineEditor:
    """Single-line input with a cursor and a history of sent lines."""

    def __init__(self):
        self.buf, self.cur = "", 0
        self.sent: list[str] = []
        self._hist = 0

    def key(self, k) -> str | None:
        """Feeds one key (a printable string, or a name such as "LEFT", "BACKSPACE", "ENTER"); returns the line on ENTER."""
        if k == "ENTER":
            line, self.buf, self.cur = self.buf, "", 0
            if line.strip():
                self.sent.append(line)
            self._hist = len(self.sent)
            return line
        if k == "BACKSPACE":
            if self.cur:
                self.buf, self.cur = self.buf[:self.cur - 1] + self.buf[self.cur:], self.cur - 1
        elif k == "DELETE":
            self.buf = self.buf[:self.cur] + self.buf[self.cur + 1:]
        elif k == "LEFT":
            self.cur = max(self.cur - 1, 0)
        elif k == "RIGHT":
            self.cur = min(self.cur + 1, len(self.buf))
        elif k == "HOME":
            self.cur = 0
        elif k == "END":
            self.cur = len(self.buf)
        elif k == "KILL":                                  # ctrl-u
            self.buf, self.cur = "", 0
        elif k in ("UP", "DOWN"):
            self._hist = max(0, min(self._hist + (-1 if k == "UP" else 1), len(self.sent)))
            self.buf = self.sent[self._hist] if self._hist < len(self.sent) else ""
            self.cur = len(self.buf)
        elif isinstance(k, str) and len(k) == 1 and k.isprintable():
            self.buf, self.cur = self.buf[:self.cur] + k + self.buf[self.cur:], self.cur + 1
        return None

    def window(self, width: int) -> tuple[str, int]:
        """The part of the buffer that fits ``width`` columns around the cursor, and the cursor's column in it."""
        width = max(width, 4)
        start = max(0, self.cur - width + 1)
        return self.buf[start:start + width], self.cur - start


def _key_name(ch) -> str | None:
    import curses
    if isinstance(ch, str):
        if ch in ("\n", "\r"):
            return "ENTER"
        if ch in ("\x7f", "\b"):
            return "BACKSPACE"
        if ch == "\x15":
            return "KILL"
        return ch if ch.isprintable() else None
    return {curses.KEY_ENTER: "ENTER", curses.KEY_BACKSPACE: "BACKSPACE", curses.KEY_DC: "DELETE", curses.KEY_LEFT: "LEFT",
            curses.KEY_RIGHT: "RIGHT", curses.KEY_HOME: "HOME", curses.KEY_END: "END", curses.KEY_UP: "UP",
            curses.KEY_DOWN: "DOWN", curses.KEY_PPAGE: "PGUP", curses.KEY_NPAGE: "PGDN", curses.KEY_RESIZE: "RESIZE"}.get(ch)


def run(session: ChatSession, model_name: str) -> None:
    """Runs the full-screen interface until /exit or end of input."""
    import curses

    def main(scr):
        curses.curs_set(1)
        scr.keypad(True)
        has_color = curses.has_colors()
        if has_color:
            curses.use_default_colors()
            for i, c in enumerate((curses.COLOR_CYAN, curses.COLOR_GREEN, curses.COLOR_YELLOW), start=1):
                curses.init_pair(i, c, -1)
        attr = {"user": curses.color_pair(1) if has_color else curses.A_BOLD, "assistant": curses.color_pair(2) if has_color else 0,
                "reasoning": (curses.color_pair(3) if has_color else 0) | curses.A_DIM, "info": curses.A_DIM, "system": curses.A_DIM}
        view, edit = ChatView(), LineEditor()
        stream = None
        view.add("info", "full-screen chat; /reset clears the conversation, /exit leaves")

        def draw():
            h, w = scr.getmaxyx()
            view.resize(w, h)
            scr.erase()
            for y, (role, ln) in enumerate(view.visible()):
                scr.addnstr(y, 0, ln, w - 1, attr.get(role, 0))
            scr.addnstr(h - 3, 0, "-" * (w - 1), w - 1, curses.A_DIM)
            text, col = edit.window(w - 4)
            scr.addnstr(h - 2, 0, "> " + text, w - 1)
            scr.addnstr(h - 1, 0, view.status(model_name, session.context_used, session.ctx_size, session.last_tok_s,
                                              stream is not None), w - 1, curses.A_REVERSE)
            scr.move(h - 2, min(2 + col, w - 2))
            scr.refresh()

        while True:
            draw()
            scr.timeout(0 if stream is not None else -1)      # poll the keyboard between engine steps while generating
            try:
                ch = scr.get_wch()
            except curses.error:
                ch = None
            k = _key_name(ch) if ch is not None else None
            if k == "PGUP":
                view.scroll_by(view.pane_height // 2)
            elif k == "PGDN":
                view.scroll_by(-(view.pane_height // 2))
            elif k is not None and k != "RESIZE":
                line = edit.key(k)
                if line is not None and line.strip() in ("/exit", "/quit"):
                    if stream is not None:
                        stream.close()                        # aborts the request that is still generating
                    return
                if line is not None and stream is None:
                    line = line.strip()
                    if line == "/reset":
                        session.reset()
                        view.entries.clear()
                        view.add("info", "conversation cleared")
                    elif line:
                        view.add("user", line)
                        view.scroll = 0
                        stream = session.ask(line)
            if stream is not None:
                try:
                    kind, piece = next(stream)
                    view.append("reasoning" if kind == "reasoning" else "assistant", piece)
                except StopIteration:
                    stream = None
                except ValueError as exc:
                    view.add("info", str(exc))
                    stream = None

    curses.wrapper(main)
