"""Conversation messages and dataset-row → messages transforms
(parity: torchtune/data/_messages.py:23-935).

All transforms share one base that resolves the column map, the optional replacement system
prompt and the masking strategy; each subclass only states how a row becomes a list of
:class:`Message`.
"""
from __future__ import annotations

from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Literal, Mapping, Optional, Sequence, Union
from warnings import warn

Role = Literal["system", "user", "assistant", "ipython", "tool"]


class MaskingStrategy(Enum):
    TRAIN_ON_ALL = "train_on_all"
    TRAIN_ON_ASSISTANT = "train_on_assistant"
    TRAIN_ON_LAST = "train_on_last"


class Message:
    """One turn of a conversation.

    ``content`` is text or a list of ``{"type": "text"|"image", "content": ...}`` parts;
    ``masked`` excludes the turn from the loss; ``ipython`` marks an assistant tool call;
    ``eot`` says the turn hands control to the other party (False for tool returns and for an
    assistant message that is followed by a tool return).
    """

    def __init__(self, role: Role, content: Union[str, List[Dict[str, Any]]], masked: bool = False, ipython: bool = False, eot: bool = True):
        self.role = role
        if isinstance(content, str):
            content = [{"type": "text", "content": content}]
        assert isinstance(content, list), f"content must be of type list[dict[str, Any]], got {content}"
        self.content = content
        self.masked = masked
        self.ipython = ipython
        self.eot = eot
        if self.ipython and self.contains_media:
            raise ValueError(f"Media tokens in tool calls are not supported. Both are set in message: {self.text_content}")
        if self.ipython and self.role != "assistant":
            raise ValueError(f"Only assistant messages can be tool calls. Found role {self.role} in message: {self.text_content}")

    @classmethod
    def from_dict(cls, d: dict) -> "Message":
        return cls(role=d["role"], content=d["content"], masked=d.get("masked", False), ipython=d.get("ipython", False), eot=d.get("eot", True))

    def get_media(self) -> List[Any]:
        return [part["content"] for part in self.content if part["type"] == "image"]

    @property
    def contains_media(self) -> bool:
        return any(part["type"] == "image" for part in self.content)

    @property
    def text_content(self) -> str:
        return "".join(part["content"] for part in self.content if part["type"] == "text")

    def __repr__(self) -> str:
        return f"Message(role='{self.role}', content={[part['content'] for part in self.content]!r})"


def mask_messages(messages: List[Message], masking_strategy: Union[str, MaskingStrategy]) -> None:
    """Set ``masked`` on every message: system turns are always masked; ``train_on_all`` masks
    only user turns that carry images; ``train_on_assistant`` masks everything but assistant
    turns; ``train_on_last`` leaves only the final assistant turn unmasked."""
    strategy = MaskingStrategy(masking_strategy)
    last_assistant = max((i for i, m in enumerate(messages) if m.role == "assistant"), default=-1)
    for i, m in enumerate(messages):
        if m.role == "system":
            m.masked = True
        elif strategy is MaskingStrategy.TRAIN_ON_LAST:
            m.masked = i != last_assistant
        elif strategy is MaskingStrategy.TRAIN_ON_ALL:
            m.masked = m.role == "user" and m.contains_media
        else:
            m.masked = m.role != "assistant"


def validate_messages(messages: List[Message]) -> None:
    """Raise ``ValueError`` unless the list is a well-formed conversation: at least one
    exchange, a system turn only in first place, no two user turns in a row, no assistant turn
    without a preceding user/tool turn, tool returns only after a tool call."""
    if len(messages) < 2:
        raise ValueError(f"Messages must be at least length 2, but got {len(messages)} messages")
    prev = Message(role="assistant", content="")
    for i, m in enumerate(messages):
        if m.role == "assistant" and prev.role not in ("user", "tool", "ipython"):
            raise ValueError(f"Assistant message before expected user, tool or ipython message at index {i} in messages")
        if m.role == "user" and prev.role == "user":
            raise ValueError(f"Two consecutive user messages at index {i} and {i - 1} in messages")
        if m.role == "system" and i > 0:
            raise ValueError(f"System message at index {i} in messages, but system messages must come first")
        if m.role in ("tool", "ipython") and not prev.ipython:
            raise ValueError(f"Tool or ipython message at index {i} must follow an ipython message")
        prev = m


class _ToMessages:
    """Shared plumbing.  ``required`` names the logical columns a user-supplied ``column_map``
    must contain; ``defaults`` is the identity map used otherwise."""

    required: Sequence[str] = ()
    defaults: Dict[str, str] = {}

    def __init__(self, train_on_input: Optional[bool], column_map: Optional[Dict[str, str]], new_system_prompt: Optional[str], masking_strategy: Optional[str]):
        if train_on_input is not None:
            warn(
                "train_on_input is deprecated and will be removed in a future release. Please use masking_strategy instead."
                "You should replace train_on_input=True with masking_strategy='train_on_all', and "
                "train_on_input=False with masking_strategy='train_on_assistant'.",
                DeprecationWarning,
                stacklevel=3,
            )
            masking_strategy = "train_on_all" if train_on_input else "train_on_assistant"
        self.masking_strategy = masking_strategy
        self.new_system_prompt = new_system_prompt
        if column_map:
            for key in self.required:
                if key not in column_map:
                    raise ValueError(f"Expected a key of '{key}' in column_map but found {column_map.keys()}.")
            self._column_map = dict(column_map)
        else:
            self._column_map = dict(self.defaults)

    def _system(self) -> List[Message]:
        if self.new_system_prompt is None:
            return []
        return [Message(role="system", content=self.new_system_prompt, masked=True, eot=True)]

    def _finish(self, messages: List[Message]) -> Dict[str, Any]:
        mask_messages(messages, self.masking_strategy)
        return {"messages": messages}

    def _image_for(self, sample: Mapping[str, Any], image_dir: Optional[Path]):
        """The sample's image (loaded if given as a path) or ``None`` for text-only rows."""
        col = self._column_map.get("image")
        if not ("image" in sample or (col is not None and col in sample)):
            return None
        from ._utils import load_image

        value = sample[col if col is not None else "image"]
        if isinstance(value, (str, Path)):
            path = Path(value)
            return load_image(image_dir / path if image_dir is not None else path)
        return value


class InputOutputToMessages(_ToMessages):
    """Rows with an ``input`` and an ``output`` column (optionally an ``image``) → one
    user/assistant exchange."""

    required = ("input", "output")
    defaults = {"input": "input", "output": "output", "image": "image"}

    def __init__(self, train_on_input: Optional[bool] = None, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, image_dir: Optional[Path] = None, masking_strategy: Optional[str] = "train_on_assistant"):
        super().__init__(train_on_input, column_map, new_system_prompt, masking_strategy)
        if "image" not in self._column_map and image_dir is not None:
            raise ValueError(f"image_dir is specified as {image_dir} but 'image' is not in column_map. Please specify an 'image' key in column_map.")
        self.image_dir = image_dir

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        image = self._image_for(sample, self.image_dir)
        user: List[Dict[str, Any]] = [{"type": "text", "content": sample[self._column_map["input"]]}]
        if image is not None:
            user.insert(0, {"type": "image", "content": image})
        return self._finish(
            self._system()
            + [Message(role="user", content=user, eot=True), Message(role="assistant", content=[{"type": "text", "content": sample[self._column_map["output"]]}], eot=True)]
        )


class ChosenRejectedToMessages(_ToMessages):
    """Preference rows: ``chosen`` and ``rejected`` are each a list of ``{role, content}``
    dicts; returns ``{"chosen": [...], "rejected": [...]}``."""

    required = ("chosen", "rejected")
    defaults = {"chosen": "chosen", "rejected": "rejected"}

    def __init__(self, train_on_input: Optional[bool] = None, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, masking_strategy: Optional[str] = "train_on_assistant"):
        super().__init__(train_on_input, column_map, new_system_prompt, masking_strategy)

    def _side(self, turns: Sequence[Mapping[str, Any]]) -> List[Message]:
        out = self._system()
        for t in turns:
            if t["role"] == "system" and self.new_system_prompt is not None:
                continue
            out.append(Message.from_dict(t))
        mask_messages(out, self.masking_strategy)
        return out

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        return {"chosen": self._side(sample[self._column_map["chosen"]]), "rejected": self._side(sample[self._column_map["rejected"]])}


class ShareGPTToMessages(_ToMessages):
    """``{"conversations": [{"from": "system|human|gpt", "value": ...}]}`` rows; an optional
    image is attached to the first human turn (at ``image_tag`` positions, or prepended when
    ``image_tag`` is None)."""

    required = ("conversations",)
    defaults = {"conversations": "conversations", "image": "image"}
    _ROLES = {"system": "system", "human": "user", "gpt": "assistant"}

    def __init__(self, train_on_input: Optional[bool] = None, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, image_dir: Optional[Path] = None, image_tag: Optional[str] = "<image>", masking_strategy: Optional[str] = "train_on_assistant"):
        super().__init__(train_on_input, column_map, new_system_prompt, masking_strategy)
        self.image_dir = image_dir
        self.image_tag = image_tag

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        from ._utils import format_content_with_images

        messages = self._system()
        image = self._image_for(sample, self.image_dir)
        for turn in sample[self._column_map["conversations"]]:
            role = self._ROLES[turn["from"]]
            content: Any = turn["value"]
            if role == "system" and self.new_system_prompt is not None:
                continue
            if role == "user" and image is not None:
                if self.image_tag is None:
                    content = [{"type": "image", "content": image}, {"type": "text", "content": content}]
                else:
                    content = format_content_with_images(content, image_tag=self.image_tag, images=[image])
                image = None  # only the first human turn carries it
            messages.append(Message(role=role, content=content))
        return self._finish(messages)


class OpenAIToMessages(_ToMessages):
    """OpenAI chat-completion rows: ``{"messages": [{"role", "content"}]}`` where content is
    text or a list of ``{"type": "text"|"image_url", ...}`` parts.  Tool returns and
    assistant turns followed by a tool return do not end the turn."""

    required = ("messages",)
    defaults = {"messages": "messages"}

    def __init__(self, train_on_input: Optional[bool] = None, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, masking_strategy: Optional[str] = "train_on_assistant"):
        super().__init__(train_on_input, column_map, new_system_prompt, masking_strategy)

    @staticmethod
    def _convert_from_openai_content(content: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        from ._utils import load_image

        out = []
        for part in content:
            if part["type"] == "text":
                out.append({"type": "text", "content": part["text"]})
            elif part["type"] == "image_url":
                out.append({"type": "image", "content": load_image(part["image_url"]["url"])})
        return out

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        rows = sample[self._column_map["messages"]]
        messages = self._system()
        for i, row in enumerate(rows):
            if row["role"] == "system" and self.new_system_prompt is not None:
                continue
            content = self._convert_from_openai_content(row["content"]) if isinstance(row["content"], list) else row["content"]
            eot = True
            if row["role"] in ("tool", "ipython"):
                eot = False
            elif row["role"] == "assistant" and i + 1 < len(rows) and rows[i + 1]["role"] in ("tool", "ipython"):
                eot = False
            messages.append(Message(role=row["role"], content=content, eot=eot))
        return self._finish(messages)


class AlpacaToMessages(_ToMessages):
    """Alpaca rows (``instruction``, optional ``input``, ``output``) rendered with the
    standard Alpaca prompt (with / without the input block)."""

    required = ("instruction", "output")
    defaults = {"instruction": "instruction", "input": "input", "output": "output"}
    _HEAD = "Below is an instruction that describes a task"
    template = {
        "prompt_input": _HEAD + ", paired with an input that provides further context. Write a response that appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n",
        "prompt_no_input": _HEAD + ". Write a response that appropriately completes the request.\n\n### Instruction:\n{instruction}\n\n### Response:\n",
    }

    def __init__(self, train_on_input: Optional[bool] = None, column_map: Optional[Dict[str, str]] = None, masking_strategy: Optional[str] = "train_on_all"):
        super().__init__(train_on_input, column_map, None, masking_strategy)

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        extra = self._column_map.get("input", "input")
        instruction = sample[self._column_map["instruction"]]
        if extra in sample and sample[extra]:
            prompt = self.template["prompt_input"].format(instruction=instruction, input=sample[extra])
        else:
            prompt = self.template["prompt_no_input"].format(instruction=instruction)
        return self._finish([Message(role="user", content=prompt, eot=True), Message(role="assistant", content=sample[self._column_map["output"]], eot=True)])
