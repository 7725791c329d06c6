"""Small data helpers (parity: torchtune/data/_utils.py:25-347)."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, TypeVar, Union
from urllib import request

T = TypeVar("T")


def truncate(tokens: List[Any], max_seq_len: int, eos_id: Optional[Any] = None, truncation_type: str = "right") -> List[Any]:
    """Keep the first (``right``) or last (``left``) ``max_seq_len`` tokens; when ``eos_id`` is
    given the final kept token is forced to it."""
    if truncation_type == "left":
        kept = tokens[-max_seq_len:]
    elif truncation_type == "right":
        kept = tokens[:max_seq_len]
    else:
        raise ValueError(f"truncation_type must be 'left' or 'right', got {truncation_type}")
    if eos_id is not None and kept and kept[-1] != eos_id:
        kept[-1] = eos_id
    return kept


def load_image(image_loc: Union[Path, str]):
    """Open a local path or an http(s) URL as a ``PIL.Image``."""
    from PIL import Image

    loc = str(image_loc)
    try:
        if loc.startswith("http"):
            with request.urlopen(loc) as resp:  # noqa: S310 (caller supplied URL)
                from io import BytesIO

                image = Image.open(BytesIO(resp.read()))
                image.load()
                return image
        image = Image.open(image_loc)
        image.load()
        return image
    except Exception as exc:
        raise ValueError(f"Failed to load image from {image_loc}") from exc


def format_content_with_images(content: str, *, image_tag: str, images: List[Any]) -> List[Dict[str, Any]]:
    """Split ``content`` at every ``image_tag`` and interleave the images in order."""
    n_tags = content.count(image_tag)
    if len(images) != n_tags:
        raise ValueError(f"Number of images ({len(images)}) does not match number of image tags ({n_tags}) in content: {content}")
    pieces = content.split(image_tag)
    queue = list(images)
    out: List[Dict[str, Any]] = []
    for i, text in enumerate(pieces):
        if text:
            out.append({"type": "text", "content": text})
        if i < len(pieces) - 1:
            out.append({"type": "image", "content": queue.pop(0)})
    return out


def chain(*funcs: Callable) -> Callable:
    """``chain(f, g, h)(x) == h(g(f(x)))``."""

    def composed(x):
        for fn in funcs:
            x = fn(x)
        return x

    return composed


def load_hf_dataset(source: str, transform: Callable, filter_fn: Optional[Callable] = None, shuffle: bool = True, seed: int = 0, num_workers: int = 0, parallel_method: str = "thread", streaming: bool = False, **load_dataset_kwargs: Any):
    """Load a HF dataset and apply ``transform`` lazily; returns an iterable of samples.
    (The reference builds a torchdata node graph here; this returns a plain mapped dataset.)"""
    from datasets import load_dataset

    ds = load_dataset(source, streaming=streaming, **load_dataset_kwargs)
    if filter_fn is not None:
        ds = ds.filter(filter_fn)
    if shuffle and not streaming:
        ds = ds.shuffle(seed=seed)

    class _Mapped:
        def __len__(self):
            return len(ds)

        def __getitem__(self, i):
            return transform(ds[i])

        def __iter__(self):
            for row in ds:
                yield transform(row)

    return _Mapped()


def get_multi_dataset(datasets: Dict[str, Any], weights: Dict[str, float], stop_criteria: str = "CYCLE_UNTIL_ALL_DATASETS_EXHAUSTED", seed: int = 0):
    """Weighted interleaving of several iterables (generator)."""
    import random

    rng = random.Random(seed)
    names = list(datasets)
    iters = {n: iter(datasets[n]) for n in names}
    exhausted = set()

    def gen():
        while True:
            n = rng.choices(names, weights=[weights[k] for k in names])[0]
            try:
                yield next(iters[n])
            except StopIteration:
                exhausted.add(n)
                if stop_criteria == "FIRST_DATASET_EXHAUSTED" or len(exhausted) == len(names):
                    return
                iters[n] = iter(datasets[n])

    return gen()


def get_dataloader(dataset, model_transform: Callable, batch_size: int, collate_fn: Optional[Callable] = None, drop_last: bool = True, num_workers: int = 0, pin_memory: bool = True):
    """Batching iterator over an iterable dataset with a model transform applied per sample."""

    def gen():
        batch = []
        for sample in dataset:
            batch.append(model_transform(sample))
            if len(batch) == batch_size:
                yield collate_fn(batch) if collate_fn else batch
                batch = []
        if batch and not drop_last:
            yield collate_fn(batch) if collate_fn else batch

    return gen()
