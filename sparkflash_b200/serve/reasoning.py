"""Reasoning split, stop strings and the decode-side loop detector: three small streaming filters between
the detokeniser and the API events.

Reference behaviour: crates/sparkflash-api/src/reasoning.rs (text before ``</think>`` is the reasoning
channel when the prompt opened a thinking block), crates/sparkflash-api/src/loop_abort.rs:15-60 (an n-gram
repeated back to back, or the same long line repeated, ends the sequence).
"""
from __future__ import annotations

from collections import deque

from .encoding import THINK_END, THINK_START
from .tool_parser import _holdback


class ReasoningSplitter:
    def __init__(self, thinking: bool):
        self.in_think = thinking
        self.buf = ""

    def feed(self, text: str, final: bool = False) -> tuple[str, str]:
        """-> (reasoning_delta, content_delta)"""
        self.buf += text
        reasoning = content = ""
        while True:
            if self.in_think:
                i = self.buf.find(THINK_END)
                if i >= 0:
                    reasoning += self.buf[:i]
                    self.buf = self.buf[i + len(THINK_END):]
                    self.in_think = False
                    continue
                keep = 0 if final else _holdback(self.buf, [THINK_END])
                reasoning += self.buf[:len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
            i = self.buf.find(THINK_START)
            if i >= 0:          # the model opened a block of its own
                content += self.buf[:i]
                self.buf = self.buf[i + len(THINK_START):]
                self.in_think = True
                continue
            keep = 0 if final else _holdback(self.buf, [THINK_START])
            content += self.buf[:len(self.buf) - keep]
            self.buf = self.buf[len(self.buf) - keep:]
            break
        return reasoning, content


class StopStrings:
    """Holds back text that may still become a stop string; ``hit`` is set once one matched (the stop
    string itself is not emitted)."""

    def __init__(self, stops: list[str]):
        self.stops = [s for s in stops if s]
        self.buf = ""
        self.hit: str | None = None

    def feed(self, text: str, final: bool = False) -> str:
        if self.hit is not None:
            return ""
        self.buf += text
        first, which = -1, None
        for s in self.stops:
            i = self.buf.find(s)
            if i >= 0 and (first < 0 or i < first):
                first, which = i, s
        if which is not None:
            out, self.buf, self.hit = self.buf[:first], "", which
            return out
        keep = 0 if final else _holdback(self.buf, self.stops)
        out, self.buf = self.buf[:len(self.buf) - keep], self.buf[len(self.buf) - keep:]
        return out


class LoopAbortDetector:
    """Exact and structural: the last n*(R-1) tokens satisfy token[i] == token[i-n]  <=>  an n-gram repeated R
    times back to back; and R identical consecutive lines of at least ``min_line_bytes``."""

    LINE_CAP = 8192

    def __init__(self, ngram: int = 8, max_repeats: int = 8, max_line_repeats: int = 4, min_line_bytes: int = 16):
        self.n, self.R, self.LR, self.min_line = ngram, max_repeats, max_line_repeats, min_line_bytes
        self.ring: deque[int] = deque(maxlen=ngram)
        self.run = 0
        self.line, self.prev_line, self.line_run = "", None, 0
        self.overflow = False

    def push_token(self, tok: int) -> bool:
        if len(self.ring) == self.n and self.ring[0] == tok:
            self.run += 1
        else:
            self.run = 0
        self.ring.append(tok)
        return self.run >= self.n * (self.R - 1)

    def push_text(self, text: str) -> bool:
        fired = False
        for ch in text:
            if ch != "\n":
                if len(self.line) < self.LINE_CAP:
                    self.line += ch
                else:
                    self.overflow = True
                continue
            line, self.line = self.line, ""
            ok = not self.overflow and len(line.encode()) >= self.min_line
            self.overflow = False
            if ok and line == self.prev_line:
                self.line_run += 1
            else:
                self.line_run = 1 if ok else 0
            self.prev_line = line if ok else None
            fired = fired or self.line_run >= self.LR
        return fired
