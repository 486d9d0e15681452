"""Chat-template rendering (Jinja2) and the reasoning / content splitter for thinking models.

The checkpoint's `tokenizer.chat_template` is rendered with messages, tools, `add_generation_prompt`
and `enable_thinking`; `--chat-template` may override it with a file or a built-in name (reference:
src/v2/utils/ChatTemplate.cpp, src/v2/app/ChatTemplateResolver.cpp; the reference vendors a Jinja subset
interpreter, here the jinja2 package does the work).
"""
from __future__ import annotations

import json
import os

CHATML = (
    "{%- for message in messages %}{{- '<|im_start|>' + message.role + '\\n' + (message.content or '') + '<|im_end|>\\n' }}"
    "{%- endfor %}{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- endif %}"
)
BUILTIN = {"chatml": CHATML}


def _raise(msg):
    raise ValueError(msg)


class ChatTemplate:
    def __init__(self, source: str | None, bos_token: str = "", eos_token: str = ""):
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        self.source = source or CHATML
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, undefined=jinja2.Undefined)
        env.filters["tojson"] = lambda x, indent=None, ensure_ascii=False: json.dumps(x, ensure_ascii=ensure_ascii, indent=indent)
        env.globals["raise_exception"] = _raise
        env.globals["strftime_now"] = lambda fmt: __import__("datetime").datetime.now().strftime(fmt)
        self._tpl = env.from_string(self.source)
        self.bos_token, self.eos_token = bos_token, eos_token

    @staticmethod
    def resolve(override: str | None, from_checkpoint: str | None, **kw) -> "ChatTemplate":
        if override:
            if override in BUILTIN:
                return ChatTemplate(BUILTIN[override], **kw)
            if os.path.exists(override):
                with open(override) as f:
                    return ChatTemplate(f.read(), **kw)
            raise FileNotFoundError(f"--chat-template: '{override}' is neither a file nor one of {sorted(BUILTIN)}")
        return ChatTemplate(from_checkpoint, **kw)

    @property
    def expects_thinking(self) -> bool:
        return "</think>" in self.source or "enable_thinking" in self.source

    def render(self, messages: list[dict], tools: list | None = None, add_generation_prompt: bool = True,
               enable_thinking: bool = True) -> str:
        return self._tpl.render(messages=messages, tools=tools or None, add_generation_prompt=add_generation_prompt,
                                enable_thinking=enable_thinking, bos_token=self.bos_token, eos_token=self.eos_token)


class ThinkSplitter:
    """Routes streamed text into `reasoning_content` (inside <think>…</think>) and `content`.

    `starts_in_thinking`: the template already opened a <think> block in the prompt.  Only the first
    closing tag ends the reasoning; a later one is ordinary content.  Partial tags at chunk borders are
    held back until they can be classified.
    """
    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, starts_in_thinking: bool = False):
        self.in_think = starts_in_thinking
        self.closed = False
        self._buf = ""
        self._strip_content_lead = False

    def _hold(self, text: str, tags) -> int:
        """Length of the longest suffix of text that is a proper prefix of one of the tags."""
        for n in range(min(len(text), max(len(t) for t in tags) - 1), 0, -1):
            if any(t.startswith(text[-n:]) for t in tags):
                return n
        return 0

    def push(self, text: str) -> tuple[str, str]:
        """Returns (reasoning_delta, content_delta)."""
        self._buf += text
        reasoning, content = "", ""
        while self._buf:
            if self.in_think:
                i = self._buf.find(self.CLOSE)
                if i >= 0:
                    reasoning += self._buf[:i]
                    self._buf = self._buf[i + len(self.CLOSE):]
                    self.in_think, self.closed = False, True
                    self._strip_content_lead = True
                    continue
                keep = self._hold(self._buf, (self.CLOSE,))
                reasoning += self._buf[:len(self._buf) - keep]
                self._buf = self._buf[len(self._buf) - keep:]
                break
            if not self.closed:
                i = self._buf.find(self.OPEN)
                if i >= 0:
                    content += self._buf[:i]
                    self._buf = self._buf[i + len(self.OPEN):]
                    self.in_think = True
                    continue
                keep = self._hold(self._buf, (self.OPEN,))
            else:
                keep = 0
            out = self._buf[:len(self._buf) - keep]
            if self._strip_content_lead:
                stripped = out.lstrip()
                if stripped:
                    self._strip_content_lead = False
                out = stripped
            content += out
            self._buf = self._buf[len(self._buf) - keep:]
            break
        return reasoning, content

    def flush(self) -> tuple[str, str]:
        rest, self._buf = self._buf, ""
        return (rest, "") if self.in_think else ("", rest)
