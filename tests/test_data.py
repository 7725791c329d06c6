import json

import pytest
import torch

from torchtune_b200.data import (
    AlpacaToMessages,
    ChatMLTemplate,
    ChosenRejectedToMessages,
    InputOutputToMessages,
    Message,
    OpenAIToMessages,
    PromptTemplate,
    ShareGPTToMessages,
    left_pad_sequence,
    mask_messages,
    padded_collate_dpo,
    padded_collate_packed,
    padded_collate_sft,
    truncate,
    validate_messages,
)
from torchtune_b200.datasets import ConcatDataset, PackedDataset, alpaca_dataset, chat_dataset, preference_dataset


class WordTokenizer:
    """Token = length of each whitespace-separated word; bos 0, eos -1 (test double)."""

    max_seq_len = None
    pad_id = 0

    def encode(self, text, add_bos=True, add_eos=True, **kw):
        ids = [len(w) for w in text.split()]
        return ([0] if add_bos else []) + ids + ([-1] if add_eos else [])

    def tokenize_messages(self, messages, **kw):
        tokens, mask = [0], [True]
        for m in messages:
            ids = self.encode(m.text_content, add_bos=False, add_eos=False)
            tokens += ids
            mask += [m.masked] * len(ids)
        return tokens + [-1], mask + [True]

    def __call__(self, sample, inference=False):
        sample["tokens"], sample["mask"] = self.tokenize_messages(sample.pop("messages"))
        return sample


def test_message_masking_strategies_and_validation():
    msgs = [Message("system", "s"), Message("user", "u"), Message("assistant", "a1"), Message("user", "u2"), Message("assistant", "a2")]
    mask_messages(msgs, "train_on_assistant")
    assert [m.masked for m in msgs] == [True, True, False, True, False]
    mask_messages(msgs, "train_on_last")
    assert [m.masked for m in msgs] == [True, True, True, True, False]
    mask_messages(msgs, "train_on_all")
    assert [m.masked for m in msgs] == [True, False, False, False, False]
    validate_messages(msgs)
    with pytest.raises(ValueError):
        validate_messages([Message("user", "a"), Message("user", "b")])
    with pytest.raises(ValueError):
        validate_messages([Message("user", "a"), Message("system", "b")])
    with pytest.raises(ValueError):
        Message("user", "x", ipython=True)


def test_row_transforms():
    out = InputOutputToMessages(new_system_prompt="be nice")({"input": "hi", "output": "yo"})["messages"]
    assert [m.role for m in out] == ["system", "user", "assistant"] and out[1].masked and not out[2].masked
    sg = ShareGPTToMessages()({"conversations": [{"from": "system", "value": "s"}, {"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]})["messages"]
    assert [m.role for m in sg] == ["system", "user", "assistant"]
    oa = OpenAIToMessages()({"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "call"}, {"role": "tool", "content": "3"}, {"role": "assistant", "content": "a"}]})["messages"]
    assert [m.eot for m in oa] == [True, False, False, True]
    cr = ChosenRejectedToMessages()({"chosen": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "good"}], "rejected": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "bad"}]})
    assert cr["chosen"][1].text_content == "good" and cr["rejected"][0].masked
    with pytest.raises(ValueError):
        InputOutputToMessages(column_map={"input": "a"})


def test_templates():
    msgs = [Message("user", "hi"), Message("assistant", "")]
    out = ChatMLTemplate()(msgs)
    assert out[0].text_content == "<|im_start|>user\nhi<|im_end|>\n" and out[1].text_content == "<|im_start|>assistant\n"
    t = PromptTemplate({"user": ("Q: ", "\nA: ")})(msgs)
    assert t[0].text_content == "Q: hi\nA: " and t[1].text_content == ""


def test_truncate_and_collate():
    assert truncate([1, 2, 3, 4], 3, eos_id=9) == [1, 2, 9] and truncate([1, 2, 3, 4], 2, truncation_type="left") == [3, 4]
    b = padded_collate_sft([{"tokens": [1, 2, 3], "labels": [4, 5, 6]}, {"tokens": [7], "labels": [10]}], padding_idx=0, ignore_idx=-100)
    assert b["tokens"].tolist() == [[1, 2, 3], [7, 0, 0]] and b["labels"].tolist() == [[4, 5, 6], [10, -100, -100]]
    b8 = padded_collate_sft([{"tokens": [1, 2, 3], "labels": [4, 5, 6]}], pad_to_multiple_of=4)
    assert b8["tokens"].shape[1] == 4
    assert left_pad_sequence([torch.tensor([1, 2, 3]), torch.tensor([4])], batch_first=True).tolist() == [[1, 2, 3], [0, 0, 4]]
    ids, lbl = padded_collate_dpo([{"chosen_input_ids": [1, 2], "chosen_labels": [1, 2], "rejected_input_ids": [3], "rejected_labels": [3]}])
    assert ids.tolist() == [[1, 2], [3, 0]] and lbl.tolist() == [[1, 2], [3, -100]]


def test_packed_dataset_and_collate():
    samples = [{"tokens": list(range(1, n + 1)), "labels": list(range(1, n + 1))} for n in (3, 4, 2, 5)]
    ds = PackedDataset(samples, max_seq_len=6, padding_idx=0)
    assert len(ds) == 3
    assert ds[0]["tokens"].tolist() == [1, 2, 3, 0, 0, 0] and ds[0]["seq_lens"].tolist() == [3, 3]
    assert ds[1]["tokens"].tolist() == [1, 2, 3, 4, 1, 2] and ds[1]["input_pos"].tolist() == [0, 1, 2, 3, 0, 1] and ds[1]["seq_lens"].tolist() == [4, 2]
    for p in ds.packs:
        assert int(p["seq_lens"].sum()) == 6 and p["labels"].numel() == 6
    split = PackedDataset(samples, max_seq_len=6, split_across_pack=True)
    assert split[0]["tokens"].tolist() == [1, 2, 3, 1, 2, 3] and split[1]["tokens"].tolist()[:1] == [4]
    batch = padded_collate_packed([ds[0], ds[1]])
    dense = batch["mask"].dense(2, 6, 6, "cpu")
    assert dense[1, 4, 3].item() is False and dense[1, 5, 4].item() is True and dense[1, 3, 0].item() is True
    with pytest.raises(ValueError):
        ConcatDataset([ds, samples])


def test_dataset_builders_on_local_json(tmp_path):
    alpaca = tmp_path / "alpaca.json"
    alpaca.write_text(json.dumps([{"instruction": "Say hi", "input": "", "output": "hi there"}, {"instruction": "Add", "input": "1 2", "output": "3"}]))
    ds = alpaca_dataset(WordTokenizer(), source="json", data_files=str(alpaca), split="train")
    row = ds[0]
    assert len(row["tokens"]) == len(row["labels"]) and row["labels"][-1] == -100 and row["labels"][0] == row["tokens"][1]
    masked = alpaca_dataset(WordTokenizer(), source="json", data_files=str(alpaca), split="train", train_on_input=False)[0]
    assert masked["labels"].count(-100) > row["labels"].count(-100)
    chat = tmp_path / "chat.json"
    chat.write_text(json.dumps([{"conversations": [{"from": "human", "value": "a b"}, {"from": "gpt", "value": "c"}]}]))
    assert len(chat_dataset(WordTokenizer(), source="json", data_files=str(chat), conversation_column="conversations", conversation_style="sharegpt", split="train")[0]["tokens"]) == 5
    pref = tmp_path / "pref.json"
    pref.write_text(json.dumps([{"chosen": [{"role": "user", "content": "q q"}, {"role": "assistant", "content": "good"}], "rejected": [{"role": "user", "content": "q q"}, {"role": "assistant", "content": "bad one"}]}]))
    p = preference_dataset(WordTokenizer(), source="json", data_files=str(pref), split="train")[0]
    assert p["chosen_labels"][:3] == [-100, -100, -100] and p["chosen_labels"][3] == 4 and len(p["rejected_input_ids"]) == 6


def test_torchdata_guards(monkeypatch):
    from torchtune_b200.data import _torchdata

    @_torchdata.requires_torchdata
    def build():
        return "built"

    monkeypatch.setattr(_torchdata, "_installed", lambda: True)
    assert build() == "built" and build.__name__ == "build"
    monkeypatch.setattr(_torchdata, "_installed", lambda: False)
    import pytest as _pytest

    with _pytest.raises(ImportError, match="torchdata"):
        build()
