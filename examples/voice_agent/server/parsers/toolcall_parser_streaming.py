"""Streaming extraction of tool calls from LLM output of the form ``<TOOLCALL>[{"name": ..., "arguments": {...}}, ...]</TOOLCALL>``.
Text outside the tags is content for the voice; inside, JSON objects are emitted one by one as soon as each is complete (brace
matching that respects strings and escapes), so a tool can start before the model has finished listing the others.

(reference: ``examples/voice_agent/server/parsers/nemotron_toolcall_parser_streaming.py``, a serving-engine plug-in; this parser
is engine-independent.)"""
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List


@dataclass
class ToolDelta:
    content: str = ""
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)
    errors: List[str] = field(default_factory=list)


class StreamingToolCallParser:
    def __init__(self, start: str = "<TOOLCALL>", end: str = "</TOOLCALL>"):
        self.start, self.end = start, end
        self.inside = False
        self._buf = ""
        self.n_calls = 0

    @staticmethod
    def _held(text: str, tag: str) -> int:
        for n in range(min(len(tag) - 1, len(text)), 0, -1):
            if text.endswith(tag[:n]):
                return n
        return 0

    def _take_objects(self, out: ToolDelta) -> None:
        """Pops every complete top-level ``{...}`` from the buffer."""
        while True:
            i = self._buf.find("{")
            if i < 0:
                return
            depth, in_str, esc = 0, False, False
            endpos = -1
            for j in range(i, len(self._buf)):
                c = self._buf[j]
                if in_str:
                    if esc:
                        esc = False
                    elif c == "\\":
                        esc = True
                    elif c == '"':
                        in_str = False
                elif c == '"':
                    in_str = True
                elif c == "{":
                    depth += 1
                elif c == "}":
                    depth -= 1
                    if depth == 0:
                        endpos = j
                        break
            if endpos < 0:
                return
            raw, self._buf = self._buf[i:endpos + 1], self._buf[endpos + 1:]
            try:
                obj = json.loads(raw)
                args = obj.get("arguments", obj.get("parameters", {}))
                if isinstance(args, str):
                    args = json.loads(args)
                out.tool_calls.append({"id": f"call_{self.n_calls}", "type": "function", "function": {"name": obj["name"], "arguments": args}})
                self.n_calls += 1
            except (ValueError, KeyError, TypeError) as e:
                out.errors.append(f"unparsable tool call {raw[:80]!r}: {e}")

    def feed(self, delta_text: str) -> ToolDelta:
        out = ToolDelta()
        self._buf += delta_text
        while True:
            if not self.inside:
                k = self._buf.find(self.start)
                if k < 0:
                    h = self._held(self._buf, self.start)
                    out.content += self._buf[:len(self._buf) - h]
                    self._buf = self._buf[len(self._buf) - h:]
                    return out
                out.content += self._buf[:k]
                self._buf = self._buf[k + len(self.start):]
                self.inside = True
            else:
                k = self._buf.find(self.end)
                if k < 0:
                    self._take_objects(out)
                    return out
                tail = self._buf[k + len(self.end):]
                self._buf = self._buf[:k]
                self._take_objects(out)
                self._buf = tail
                self.inside = False

    def flush(self) -> ToolDelta:
        out = ToolDelta()
        if self.inside:
            self._take_objects(out)
            if self._buf.strip(" \n[],"):
                out.errors.append(f"generation ended inside a tool call: {self._buf[:80]!r}")
        else:
            out.content = self._buf
        self._buf = ""
        return out
