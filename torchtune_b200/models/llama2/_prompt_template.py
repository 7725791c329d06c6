"""Llama-2 chat format (parity: torchtune/models/llama2/_prompt_template.py)."""
from typing import List

from ...data._messages import Message


class Llama2ChatTemplate:
    """``[INST] <<SYS>>\\n{system}\\n<</SYS>>\\n\\n{user} [/INST] {assistant}`` — the system prompt is
    folded into the first user turn that follows it."""

    template = {
        "system": ("<<SYS>>\n", "\n<</SYS>>\n\n"),
        "user": ("[INST] ", " [/INST] "),
        "assistant": ("", ""),
        "ipython": ("", ""),
    }

    def __call__(self, messages: List[Message], inference: bool = False) -> List[Message]:
        pending_system = []
        out = []
        for m in messages:
            content = m.content
            if m.role == "system":
                before, after = self.template["system"]
                pending_system = [{"type": "text", "content": before}] + m.content + [{"type": "text", "content": after}]
                continue
            if m.role == "user":
                before, after = self.template["user"]
                content = [{"type": "text", "content": before}] + pending_system + m.content + [{"type": "text", "content": after}]
            out.append(Message(role=m.role, content=content, masked=m.masked, ipython=m.ipython, eot=m.eot))
        return out
