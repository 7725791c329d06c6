"""Mistral instruct format (parity: torchtune/models/mistral/_prompt_template.py)."""
from typing import List

from ...data._messages import Message


class MistralChatTemplate:
    """``[INST] {user} [/INST] {assistant}``; system prompts are not part of the format."""

    template = {"system": None, "user": ("[INST] ", " [/INST] "), "assistant": ("", ""), "ipython": ("", "")}

    def __call__(self, messages: List[Message], inference: bool = False) -> List[Message]:
        out = []
        for m in messages:
            if m.role == "system":
                raise ValueError("System prompts are not supported in MistralChatTemplate")
            before, after = self.template[m.role]
            content = [{"type": "text", "content": before}] + m.content + [{"type": "text", "content": after}]
            out.append(Message(role=m.role, content=content, masked=m.masked, ipython=m.ipython, eot=m.eot))
        return out
