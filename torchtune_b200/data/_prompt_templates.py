"""Prompt templates: per-role text wrapped around message content
(parity: torchtune/data/_prompt_templates.py:16-288)."""
from __future__ import annotations

from functools import partial
from typing import Dict, List, Protocol, Tuple, Union

from ._messages import Message, Role

_TemplateType = Union[str, Dict[Role, Tuple[str, str]]]


class PromptTemplateInterface(Protocol):
    """``template`` maps a role to ``(text before, text after)``; calling the template returns
    new messages with those texts added as extra text parts."""

    template: Dict[Role, Tuple[str, str]]

    def __call__(self, messages: List[Message], inference: bool = False) -> List[Message]: ...


def _wrap(message: Message, before: str, after: str) -> Message:
    content = list(message.content)
    if isinstance(before, str) and before:
        content = [{"type": "text", "content": before}] + content
    if isinstance(after, str) and after:
        content = content + [{"type": "text", "content": after}]
    return Message(role=message.role, content=content, masked=message.masked, ipython=message.ipython, eot=message.eot)


class PromptTemplate(PromptTemplateInterface):
    """Template given directly as ``{role: (prepend, append)}``.  Tags around assistant turns
    count towards the loss; tags around other roles normally do not."""

    def __init__(self, template: Dict[Role, Tuple[str, str]]):
        self.template = template

    def __call__(self, messages: List[Message], inference: bool = False) -> List[Message]:
        out = []
        for m in messages:
            before, after = self.template.get(m.role, ("", ""))
            out.append(_wrap(m, before, after))
        return out


class ChatMLTemplate(PromptTemplateInterface):
    """OpenAI Chat Markup Language: ``<|im_start|>role\\n … <|im_end|>\\n`` around every turn;
    a trailing *empty* assistant turn (generation prompt) gets only its opening tag."""

    template = {
        "system": ("<|im_start|>system\n", "<|im_end|>\n"),
        "user": ("<|im_start|>user\n", "<|im_end|>\n"),
        "assistant": ("<|im_start|>assistant\n", "<|im_end|>\n"),
        "ipython": ("", ""),
    }

    def __call__(self, messages: List[Message], inference: bool = False) -> List[Message]:
        out = []
        for i, m in enumerate(messages):
            before, after = self.template[m.role]
            open_ended = m.role == "assistant" and i == len(messages) - 1 and len(m.text_content) == 0
            out.append(_wrap(m, before, "" if open_ended else after))
        return out


GrammarErrorCorrectionTemplate = partial(PromptTemplate, template={"user": ("Correct this to standard English: ", "\n---\nCorrected: ")})
GrammarErrorCorrectionTemplate.__doc__ = "``Correct this to standard English: {user}\\n---\\nCorrected: {assistant}``"
SummarizeTemplate = partial(PromptTemplate, template={"user": ("Summarize this dialogue:\n", "\n---\nSummary:\n")})
SummarizeTemplate.__doc__ = "``Summarize this dialogue:\\n{user}\\n---\\nSummary:\\n{assistant}``"
QuestionAnswerTemplate = partial(PromptTemplate, template={"user": ("Question: ", "\n\nAnswer: ")})
QuestionAnswerTemplate.__doc__ = "``Question: {user}\\n\\nAnswer: {assistant}``"


def _get_prompt_template(prompt_template: _TemplateType) -> PromptTemplateInterface:
    """A dotted path names a template class (instantiated without arguments); a dict becomes a
    :class:`PromptTemplate`."""
    if isinstance(prompt_template, str):
        from ..config._resolve import get_component_from_path

        return get_component_from_path(prompt_template)()
    if isinstance(prompt_template, dict) or hasattr(prompt_template, "keys"):
        return PromptTemplate({k: tuple(v) for k, v in dict(prompt_template).items()})
    raise ValueError(f"Prompt template must be a dotpath string or dictionary with custom template, got {type(prompt_template)}")
