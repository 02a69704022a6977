"""The Qwen3 chat template as text (no Jinja):
    <|im_start|>{role}\\n{content}<|im_end|>\\n   per message,
    then <|im_start|>assistant\\n, and an empty <think> block when thinking is off.

Reference: src/chat/chat_template.cpp:86-117; its validation (:26-83): at least one
message, an optional system message only in front, then user and assistant in turn
starting with user, and a generation prompt only after a user message.
"""
from __future__ import annotations

from typing import List, Tuple

ROLES = ("system", "user", "assistant")


def apply_chat_template(messages: List[Tuple[str, str]], add_generation_prompt: bool = True,
                        enable_thinking: bool = True) -> str:
    if not messages:
        raise ValueError("chat template needs at least one message")
    index = 1 if messages[0][0] == "system" else 0
    if index == len(messages):
        raise ValueError("chat template needs a user message after the system message")
    expected = "user"
    for role, _ in messages[index:]:
        if role not in ROLES:
            raise ValueError(f"unknown role {role!r}")
        if role == "system":
            raise ValueError("a system message may only come first")
        if role != expected:
            raise ValueError("user and assistant messages must alternate, starting with user")
        expected = "assistant" if expected == "user" else "user"
    if add_generation_prompt and messages[-1][0] != "user":
        raise ValueError("a generation prompt needs a user message last")
    parts = [f"<|im_start|>{role}\n{content}<|im_end|>\n" for role, content in messages]
    if add_generation_prompt:
        parts.append("<|im_start|>assistant\n")
        if not enable_thinking:
            parts.append("<think>\n\n</think>\n\n")
    return "".join(parts)


def parse_answer(text: str) -> Tuple[str, bool, bool]:
    """(final answer, a thinking block was seen, the thinking block was closed) of a raw response, as the reference
    reads it (apps/qwen3_chat.cpp:593-643): everything after the LAST </think>, with the line breaks right behind
    the tag dropped; an opening tag without a closing one means the model stopped while it was still thinking - no
    final answer; a response without either tag is the answer itself."""
    end = text.rfind("</think>")
    if end >= 0:
        return text[end + len("</think>"):].lstrip("\n\r"), True, True
    if "<think>" in text:
        return "", True, False
    return text, False, True


def split_thinking(text: str) -> Tuple[str, str]:
    """(thinking, answer) of a response that may open with a <think>...</think> block: `parse_answer`'s final
    answer beside the text of the thinking block (for printing it apart from the answer)."""
    answer, saw, closed = parse_answer(text)
    if not saw:
        return "", answer
    start = text.find("<think>")
    begin = start + len("<think>") if start >= 0 else 0
    end = text.rfind("</think>") if closed else len(text)
    return text[begin:end].strip(), answer
