"""Chat encoding of DeepSeek-V4.1: messages -> one prompt string (special tokens spelled literally, the
tokenizer maps each to a single id), DSML tool markup, thinking mode and the reasoning-effort line.

Behaviour follows docs/architecture/07-encoding-protocol.md of the reference (sections 1-5): the effort
table is the checkpoint encoder's (low 25, high 50, xhigh 75, max 100; default high), later system messages
keep their own marker, tool results are re-ordered to the order of the calls, arguments are spelled
python-style.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_START, THINK_END = "<think>", "</think>"
SYSTEM, USER, ASSISTANT, REMINDER = "<｜System｜>", "<｜User｜>", "<｜Assistant｜>", "<｜latest_reminder｜>"
DSML = "｜DSML｜"
IMAGE = "<｜image｜>"         # one placeholder per image; the server expands it into the image span
SPECIAL_TOKENS = [BOS, EOS, THINK_START, THINK_END, SYSTEM, USER, ASSISTANT, REMINDER, DSML, IMAGE]

EFFORT_SCORE = {"minimal": 25, "low": 25, "medium": 50, "high": 50, "xhigh": 75, "max": 100}
DEFAULT_EFFORT = 50


@dataclass
class ToolCall:
    id: str
    name: str
    arguments: str        # JSON text


@dataclass
class Message:
    role: str                     # system | user | assistant | tool | latest_reminder
    content: str = ""
    reasoning: str | None = None
    tool_calls: list[ToolCall] = field(default_factory=list)
    tool_call_id: str | None = None
    images: list[Any] = field(default_factory=list)


def python_repr(v: Any) -> str:
    """Python-style spelling of a JSON value: True/False/None, single-quoted strings, json.dumps spacing."""
    if v is True:
        return "True"
    if v is False:
        return "False"
    if v is None:
        return "None"
    if isinstance(v, str):
        return repr(v)
    if isinstance(v, (int, float)):
        return repr(v)
    if isinstance(v, list):
        return "[" + ", ".join(python_repr(x) for x in v) + "]"
    if isinstance(v, dict):
        return "{" + ", ".join(f"{python_repr(str(k))}: {python_repr(x)}" for k, x in v.items()) + "}"
    return repr(v)


def render_tool_call(name: str, arguments: str) -> str:
    try:
        args = json.loads(arguments) if arguments.strip() else {}
        if not isinstance(args, dict):
            raise ValueError
    except ValueError:
        args = {"arguments": arguments}
    params = []
    for k, v in args.items():
        is_str = isinstance(v, str)
        params.append(f'<{DSML} parameter name="{k}" string="{"true" if is_str else "false"}">{v if is_str else python_repr(v)}</{DSML} parameter>')
    return f'<{DSML} invoke name="{name}">\n' + "\n".join(params) + f"\n</{DSML} invoke>"


def render_tool_calls(calls: list[ToolCall]) -> str:
    return f"<{DSML} calls>\n" + "\n".join(render_tool_call(c.name, c.arguments) for c in calls) + f"\n</{DSML} calls>"


def tool_prompt(tools: list[dict]) -> str:
    schemas = "\n".join(python_repr(t.get("function", t)) for t in tools)
    return (
        "## Tools\n\nYou have access to a set of tools to help answer the user's question. "
        f'You can invoke tools by writing a "<{DSML} calls>" block like the following:\n\n'
        f"<{DSML} calls>\n<{DSML} invoke name=\"$TOOL_NAME\">\n"
        f"<{DSML} parameter name=\"$PARAMETER_NAME\" string=\"true|false\">$PARAMETER_VALUE</{DSML} parameter>\n...\n"
        f"</{DSML} invoke>\n<{DSML} invoke name=\"$TOOL_NAME2\">\n...\n</{DSML} invoke>\n</{DSML} calls>\n\n"
        'String parameters should be specified as is and set string="true". For all other types (numbers, booleans, '
        'arrays, objects), pass the value in JSON format and set string="false".\n\n'
        "If thinking_mode is enabled (triggered by <think>), you MUST output your complete reasoning inside "
        "<think>...</think> BEFORE any tool calls or final response.\n\n"
        "Otherwise, output directly after </think> with tool calls or final response.\n\n"
        f"### Available Tool Schemas\n\n{schemas}\n\n"
        "You MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls."
    )


def resolve_thinking(reasoning_effort: str | int | None, thinking: dict | None, default_thinking: bool) -> tuple[bool, int | None]:
    """(thinking on?, effort score 1..100 or None) from the request fields; the typed ``thinking`` object wins."""
    score: int | None = None
    on = default_thinking
    if isinstance(reasoning_effort, int) and not isinstance(reasoning_effort, bool):
        if not 1 <= reasoning_effort <= 100:
            raise ValueError("reasoning_effort must lie in 1..100")
        on, score = True, reasoning_effort
    elif isinstance(reasoning_effort, str):
        if reasoning_effort == "none":
            on = False
        elif reasoning_effort in EFFORT_SCORE:
            on, score = True, EFFORT_SCORE[reasoning_effort]
        else:
            raise ValueError(f"unknown reasoning_effort {reasoning_effort!r}")
    if thinking is not None:
        t = thinking.get("type")
        if t not in ("enabled", "disabled"):
            raise ValueError("thinking.type must be enabled or disabled")
        on = t == "enabled"
    if not on:
        return False, None
    return True, score if score is not None else DEFAULT_EFFORT


def normalise(messages: list[Message], need_system: bool) -> list[Message]:
    out: list[Message] = []
    for m in messages:
        if m.role == "user" and out and out[-1].role == "user":
            out[-1] = Message("user", out[-1].content + "\n\n" + m.content, images=out[-1].images + m.images)
        else:
            out.append(m)
    # tool results follow the order of the preceding assistant's calls
    i = 0
    while i < len(out):
        if out[i].role == "assistant" and out[i].tool_calls:
            j = i + 1
            while j < len(out) and out[j].role == "tool":
                j += 1
            order = {c.id: k for k, c in enumerate(out[i].tool_calls)}
            out[i + 1:j] = sorted(out[i + 1:j], key=lambda t: order.get(t.tool_call_id, len(order)))
            i = j
        else:
            i += 1
    if need_system and (not out or out[0].role != "system"):
        out.insert(0, Message("system", ""))
    return out


def render_prompt(messages: list[Message], tools: list[dict] | None = None, thinking: bool = False, effort: int | None = None,
                  tool_choice_required: bool = False, json_hint: str | None = None) -> str:
    """The whole generation prompt.  ``json_hint``: text appended to the first system message for a JSON
    response format (the constraint itself is enforced at the head, not by this hint)."""
    tools = tools or []
    msgs = normalise(messages, bool(tools) or json_hint is not None)
    parts = [BOS]
    for i, m in enumerate(msgs):
        prev = msgs[i - 1].role if i else None
        if m.role == "system":
            body = m.content
            if i == 0:
                extra = []
                if tools:
                    extra.append(tool_prompt(tools))
                if json_hint:
                    extra.append(json_hint)
                if extra:
                    body = "\n\n".join([body] * bool(body) + extra)
            line = f"Reasoning Effort: {effort} (range 1-100, the higher the value, the more thorough the reasoning)\n\n" if (i == 0 and thinking and effort) else ""
            parts.append(SYSTEM + line + body)
        elif m.role in ("user", "tool"):
            if i == 0 and thinking and effort:
                parts.append(SYSTEM + f"Reasoning Effort: {effort} (range 1-100, the higher the value, the more thorough the reasoning)\n\n")
            parts.append("\n\n" if prev in ("user", "tool") else USER)
            parts.append(m.content if m.role == "user" else f"<tool_result>{m.content}</tool_result>")
        elif m.role == "latest_reminder":
            parts.append(REMINDER + m.content)
        elif m.role == "assistant":
            think = (m.reasoning or "") + THINK_END if (thinking and i > 0 and m.reasoning) else ""
            calls = "\n\n" + render_tool_calls(m.tool_calls) if m.tool_calls else ""
            if think:
                parts.append(ASSISTANT + THINK_START + think + m.content + calls + EOS)
            else:
                parts.append(ASSISTANT + THINK_END + m.content + calls + EOS)
        else:
            raise ValueError(f"unknown role {m.role!r}")
    parts.append(ASSISTANT + (THINK_START if thinking else THINK_END))
    if tool_choice_required and tools:
        parts.append(f"\n\n<{DSML} calls>\n")
    return "".join(parts)
