"""Image + text SFT datasets (parity: torchtune/datasets/multimodal/{_llava_instruct,_the_cauldron,_vqa,_multimodal}.py).

Every builder pairs a message transform (rows → :class:`~torchtune_b200.data.Message` lists whose user turns carry
``{"type": "image"}`` parts) with the model's multimodal transform (tokenizer + image tiling + cross-attention
mask).  Packing is not supported for multimodal samples."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Dict, Mapping, Optional

from ...data import InputOutputToMessages, Message, ShareGPTToMessages
from .._sft import SFTDataset, SFTTransform


def _no_packing(packed: bool) -> None:
    if packed:
        raise ValueError("Multimodal datasets don't support packing yet.")


class TheCauldronToMessages:
    """Rows ``{"images": [img, …], "texts": [{"user": …, "assistant": …}, …]}`` → alternating user / assistant
    messages; all images are attached in front of the first user turn; user turns are masked from the loss."""

    def __init__(self, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None):
        self.new_system_prompt = new_system_prompt
        if column_map is not None:
            for needed in ("images", "texts"):
                if needed not in column_map:
                    raise ValueError(f"column_map must map '{needed}' to your expected column name if specified")
            self._column_map = column_map
        else:
            self._column_map = {"texts": "texts", "images": "images"}

    def __call__(self, sample: Mapping[str, Any]) -> Mapping[str, Any]:
        images = [{"type": "image", "content": img} for img in sample[self._column_map["images"]]]
        messages = []
        if self.new_system_prompt is not None:
            messages.append(Message(role="system", content=self.new_system_prompt, masked=True, eot=True))
        for i, turn in enumerate(sample[self._column_map["texts"]]):
            user = [{"type": "text", "content": turn["user"]}]
            messages.append(Message(role="user", content=(images + user) if i == 0 else user, masked=True))
            messages.append(Message(role="assistant", content=[{"type": "text", "content": turn["assistant"]}]))
        return {"messages": messages}


def the_cauldron_dataset(model_transform: Callable, *, subset: str = "ocrvqa", source: str = "HuggingFaceM4/the_cauldron", column_map: Optional[Dict[str, str]] = None,
                         new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> SFTDataset:
    """One subset of The Cauldron (a collection of 50 vision-language datasets in a common schema)."""
    _no_packing(packed)
    return SFTDataset(model_transform=model_transform, source=source, message_transform=TheCauldronToMessages(column_map, new_system_prompt), name=subset, filter_fn=filter_fn, split=split, **load_dataset_kwargs)


def the_cauldron_transform(model_transform: Optional[Callable] = None, texts_col: str = "texts", images_col: str = "images", new_system_prompt: Optional[str] = None) -> SFTTransform:
    return SFTTransform(message_transform=TheCauldronToMessages({"texts": texts_col, "images": images_col}, new_system_prompt), model_transform=model_transform)


def llava_instruct_dataset(model_transform: Callable, *, source: str = "liuhaotian/LLaVA-Instruct-150K", image_dir: str = "coco/train2017/", column_map: Optional[Dict[str, str]] = None,
                           new_system_prompt: Optional[str] = None, packed: bool = False, filter_fn: Optional[Callable] = None, split: str = "train", data_files: str = "llava_instruct_150k.json",
                           **load_dataset_kwargs: Any) -> SFTDataset:
    """LLaVA-Instruct-150K: ShareGPT-style conversations whose first human turn refers to a COCO image (``<image>`` tag)
    loaded from ``image_dir``."""
    _no_packing(packed)
    transform = ShareGPTToMessages(train_on_input=False, column_map=column_map, new_system_prompt=new_system_prompt, image_dir=Path(image_dir), image_tag="<image>")
    return SFTDataset(model_transform=model_transform, source=source, message_transform=transform, filter_fn=filter_fn, split=split, data_files=data_files, **load_dataset_kwargs)


def vqa_dataset(model_transform: Callable, *, source: str, image_dir: Optional[str] = None, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, packed: bool = False,
                filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> SFTDataset:
    """Generic visual question answering rows: ``input`` (question), ``output`` (answer), ``image`` (PIL image or path)."""
    _no_packing(packed)
    transform = InputOutputToMessages(column_map=column_map, new_system_prompt=new_system_prompt, image_dir=Path(image_dir) if image_dir is not None else None)
    return SFTDataset(source=source, message_transform=transform, model_transform=model_transform, filter_fn=filter_fn, split=split, **load_dataset_kwargs)


def multimodal_chat_dataset(model_transform: Callable, *, source: str, column_map: Optional[Dict[str, str]] = None, new_system_prompt: Optional[str] = None, packed: bool = False,
                            image_tag: Optional[str] = None, image_dir: Optional[str] = None, filter_fn: Optional[Callable] = None, split: str = "train", **load_dataset_kwargs: Any) -> SFTDataset:
    """Generic multi-turn image chat in ShareGPT format; ``image_tag`` marks where the image goes in the first human turn."""
    _no_packing(packed)
    transform = ShareGPTToMessages(train_on_input=False, column_map=column_map, new_system_prompt=new_system_prompt, image_dir=Path(image_dir) if image_dir is not None else None, image_tag=image_tag)
    return SFTDataset(source=source, message_transform=transform, model_transform=model_transform, filter_fn=filter_fn, split=split, **load_dataset_kwargs)
