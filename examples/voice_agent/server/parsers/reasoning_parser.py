"""Streaming split of an LLM's output into *reasoning* (between ``<think>`` and ``</think>``) and *content*.  The voice agent
speaks only the content, so the split has to work on partial text: a tag can arrive cut in half at a chunk boundary, and a model
started with a reasoning prompt may emit ``</think>`` without ever emitting ``<think>``.

(reference: ``examples/voice_agent/server/parsers/nano_v3_reasoning_parser.py``, a plug-in for a serving engine; this parser is
engine-independent: feed it text deltas.)"""
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass
class Delta:
    reasoning: str = ""
    content: str = ""


class StreamingReasoningParser:
    def __init__(self, start: str = "<think>", end: str = "</think>", starts_in_reasoning: bool = False):
        self.start, self.end = start, end
        self.in_reasoning = starts_in_reasoning
        self._held = ""                                      # tail that may be the beginning of a tag

    def _longest_tag_prefix(self, text: str) -> int:
        """Length of the longest suffix of ``text`` that is a proper prefix of the tag expected next."""
        tag = self.end if self.in_reasoning else self.start
        for n in range(min(len(tag) - 1, len(text)), 0, -1):
            if text.endswith(tag[:n]):
                return n
        return 0

    def feed(self, delta_text: str) -> Delta:
        text = self._held + delta_text
        self._held = ""
        out = Delta()
        while text:
            tag = self.end if self.in_reasoning else self.start
            k = text.find(tag)
            if k < 0 and not self.in_reasoning:
                e = text.find(self.end)                       # a closing tag without an opening one: everything before it was reasoning
                if e >= 0:
                    out.reasoning += out.content + text[:e]
                    out.content = ""
                    text = text[e + len(self.end):]
                    continue
            if k < 0:
                hold = self._longest_tag_prefix(text)
                if not self.in_reasoning:
                    hold = max(hold, self._suffix_prefix(text, self.end))
                body, self._held = (text[:-hold], text[-hold:]) if hold else (text, "")
                if self.in_reasoning:
                    out.reasoning += body
                else:
                    out.content += body
                break
            if self.in_reasoning:
                out.reasoning += text[:k]
            else:
                out.content += text[:k]
            self.in_reasoning = not self.in_reasoning
            text = text[k + len(tag):]
        return out

    @staticmethod
    def _suffix_prefix(text: str, tag: str) -> int:
        for n in range(min(len(tag) - 1, len(text)), 0, -1):
            if text.endswith(tag[:n]):
                return n
        return 0

    def flush(self) -> Delta:
        """End of generation: whatever was held back was not a tag after all."""
        held, self._held = self._held, ""
        return Delta(reasoning=held) if self.in_reasoning else Delta(content=held)


def split_reasoning(text: str, start: str = "<think>", end: str = "</think>") -> Tuple[Optional[str], str]:
    """Whole-text version: ``(reasoning or None, content)``."""
    p = StreamingReasoningParser(start, end)
    d = p.feed(text)
    f = p.flush()
    reasoning, content = d.reasoning + f.reasoning, d.content + f.content
    return (reasoning.strip() or None), content.strip()
