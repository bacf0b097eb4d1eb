"""Incremental tool-call parsers: the model's DSML block (DeepSeek) and the ``<tool_call>`` XML/JSON dialect
(Qwen) become OpenAI-style tool-call deltas while the text is still streaming.

Reference behaviour: crates/sparkflash-api/src/tool_parser.rs and tool_block.rs (calls are surfaced
incrementally, the arguments string grows parameter by parameter; text outside the block stays content; a
partial tag at the end of a delta is held back until it is decided).
"""
from __future__ import annotations

import ast
import json
import re
import uuid
from dataclasses import dataclass

from .encoding import DSML


@dataclass
class ToolDelta:
    index: int
    id: str | None
    name: str | None
    arguments_delta: str


def _value_json(raw: str, is_string: bool) -> str:
    if is_string:
        return json.dumps(raw, ensure_ascii=False)
    t = raw.strip()
    try:
        return json.dumps(json.loads(t), ensure_ascii=False)
    except ValueError:
        pass
    try:
        return json.dumps(ast.literal_eval(t), ensure_ascii=False)     # python-style spelling: True / None / 'x'
    except (ValueError, SyntaxError):
        return json.dumps(raw, ensure_ascii=False)


def _holdback(buf: str, tags: list[str]) -> int:
    """How many trailing characters of ``buf`` could still grow into one of ``tags``."""
    best = 0
    for t in tags:
        for k in range(min(len(t) - 1, len(buf)), 0, -1):
            if buf.endswith(t[:k]):
                best = max(best, k)
                break
    return best


class DsmlToolParser:
    """Feed text deltas; get (content_delta, [ToolDelta...]) back."""

    OPEN, CLOSE = f"<{DSML} calls>", f"</{DSML} calls>"
    INV = re.compile(rf'<{DSML} invoke name="([^"]*)">')
    INV_CLOSE = f"</{DSML} invoke>"
    PARAM = re.compile(rf'<{DSML} parameter name="([^"]*)" string="(true|false)">(.*?)</{DSML} parameter>', re.S)

    def __init__(self, in_block: bool = False):
        self.buf = ""
        self.in_block = in_block      # tool_choice=required prompts end inside an opened block
        self.index = -1
        self.in_call = False
        self.n_params = 0
        self.calls: list[dict] = []

    def feed(self, text: str, final: bool = False) -> tuple[str, list[ToolDelta]]:
        self.buf += text
        content, deltas = "", []
        while True:
            if not self.in_block:
                i = self.buf.find(self.OPEN)
                if i >= 0:
                    content += self.buf[:i]
                    self.buf = self.buf[i + len(self.OPEN):]
                    self.in_block = True
                    continue
                keep = 0 if final else _holdback(self.buf, [self.OPEN])
                content += self.buf[:len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            if not self.in_call:
                m = self.INV.search(self.buf)
                c = self.buf.find(self.CLOSE)
                if c >= 0 and (m is None or c < m.start()):
                    self.buf = self.buf[c + len(self.CLOSE):]
                    self.in_block = False
                    continue
                if m is None:
                    break
                self.index += 1
                self.in_call, self.n_params = True, 0
                call = {"id": "call_" + uuid.uuid4().hex[:24], "name": m.group(1), "arguments": ""}
                self.calls.append(call)
                deltas.append(ToolDelta(self.index, call["id"], call["name"], ""))
                self.buf = self.buf[m.end():]
                continue
            m = self.PARAM.search(self.buf)
            e = self.buf.find(self.INV_CLOSE)
            if m is not None and (e < 0 or m.start() < e):
                frag = ("{" if self.n_params == 0 else ", ") + json.dumps(m.group(1)) + ": " + _value_json(m.group(3), m.group(2) == "true")
                self.n_params += 1
                self.calls[-1]["arguments"] += frag
                deltas.append(ToolDelta(self.index, None, None, frag))
                self.buf = self.buf[m.end():]
                continue
            if e >= 0:
                frag = "{}" if self.n_params == 0 else "}"
                self.calls[-1]["arguments"] += frag
                deltas.append(ToolDelta(self.index, None, None, frag))
                self.buf = self.buf[e + len(self.INV_CLOSE):]
                self.in_call = False
                continue
            break
        if final and self.in_call:      # the stream ended inside a call: close what was parsed
            frag = "{}" if self.n_params == 0 else "}"
            self.calls[-1]["arguments"] += frag
            deltas.append(ToolDelta(self.index, None, None, frag))
            self.in_call = False
        return content, deltas


class XmlToolParser:
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Qwen dialect; reference: crates/sparkflash-api/src/qwen.rs)."""

    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self):
        self.buf = ""
        self.index = -1
        self.calls: list[dict] = []

    def feed(self, text: str, final: bool = False) -> tuple[str, list[ToolDelta]]:
        self.buf += text
        content, deltas = "", []
        while True:
            i = self.buf.find(self.OPEN)
            if i < 0:
                keep = 0 if final else _holdback(self.buf, [self.OPEN])
                content += self.buf[:len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            j = self.buf.find(self.CLOSE, i)
            if j < 0:
                content += self.buf[:i]
                self.buf = self.buf[i:]
                if final:
                    self.buf = ""
                break
            content += self.buf[:i]
            body = self.buf[i + len(self.OPEN):j].strip()
            self.buf = self.buf[j + len(self.CLOSE):]
            try:
                obj = json.loads(body)
                name, args = obj.get("name", ""), obj.get("arguments", {})
            except ValueError:
                name, args = "", {"arguments": body}
            self.index += 1
            call = {"id": "call_" + uuid.uuid4().hex[:24], "name": name,
                    "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}
            self.calls.append(call)
            deltas.append(ToolDelta(self.index, call["id"], name, call["arguments"]))
        return content, deltas
