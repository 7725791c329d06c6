"""Wrappers over the Hugging Face ``tokenizers`` library
(parity: torchtune/modules/transforms/tokenizers/_hf_tokenizer.py:19-330)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

from ....data._messages import Message
from ....data._utils import truncate


class HuggingFaceBaseTokenizer:
    """Loads ``tokenizer.json``; BOS/EOS ids come from ``tokenizer_config.json`` or, failing
    that, ``generation_config.json``.  If the underlying tokenizer already adds BOS/EOS itself
    they are not added twice."""

    def __init__(self, tokenizer_json_path: str, *, tokenizer_config_json_path: Optional[str] = None, generation_config_path: Optional[str] = None):
        from tokenizers import Tokenizer

        self.tokenizer = Tokenizer.from_file(tokenizer_json_path)
        if tokenizer_config_json_path is None and generation_config_path is None:
            raise ValueError("At least one of tokenizer_config_json_path or generation_config_path must be specified.")
        self.config = json.load(open(tokenizer_config_json_path)) if tokenizer_config_json_path else None
        self.generation_config = json.load(open(generation_config_path)) if generation_config_path else None
        self._infer_bos_eos_tokens()
        self._infer_should_add_bos_eos()

    @staticmethod
    def _get_token_from_config(config: Dict[str, Any], key: str) -> str:
        tok = config.get(key)
        if isinstance(tok, dict):
            if "content" not in tok:
                raise ValueError(f"Could not parse {key} from config")
            tok = tok["content"]
        elif not isinstance(tok, str):
            raise ValueError(f"Could not parse {key} from config")
        return tok

    def _infer_bos_eos_tokens(self) -> None:
        self.bos_id = self.eos_id = None
        self.bos_token = self.eos_token = None
        if self.config:
            for name in ("bos", "eos"):
                try:
                    token = self._get_token_from_config(self.config, f"{name}_token")
                except ValueError:
                    continue
                setattr(self, f"{name}_token", token)
                setattr(self, f"{name}_id", self.tokenizer.token_to_id(token))
        if self.generation_config:
            if self.bos_id is None:
                self.bos_id = self.generation_config.get("bos_token_id")
            if self.eos_id is None:
                self.eos_id = self.generation_config.get("eos_token_id")
        if self.bos_id is None or self.eos_id is None:
            raise ValueError("Could not infer BOS and EOS token IDs from config")

    def _infer_should_add_bos_eos(self) -> None:
        probe = self.tokenizer.encode("Lorem ipsum", add_special_tokens=True).ids
        self.hf_adds_bos = bool(probe) and probe[0] == self.bos_id
        self.hf_adds_eos = bool(probe) and probe[-1] == self.eos_id

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, **_) -> List[int]:
        ids = self.tokenizer.encode(text, add_special_tokens=True).ids
        if add_bos and not self.hf_adds_bos:
            ids.insert(0, self.bos_id)
        if add_eos and not self.hf_adds_eos:
            ids.append(self.eos_id)
        return ids

    def decode(self, token_ids: List[int]) -> str:
        return self.tokenizer.decode(token_ids)


def _infer_special_tokens_from_hf_config(config: Dict[str, Any]) -> List[str]:
    found = set()
    for key in ("bos_token", "eos_token", "pad_token", "unk_token", "sep_token", "cls_token", "mask_token"):
        tok = config.get(key)
        if isinstance(tok, str):
            found.add(tok)
        elif isinstance(tok, dict) and isinstance(tok.get("content"), str):
            found.add(tok["content"])
    for tok in config.get("additional_special_tokens", []) or []:
        if isinstance(tok, str):
            found.add(tok)
        elif isinstance(tok, dict) and isinstance(tok.get("content"), str):
            found.add(tok["content"])
    for entry in (config.get("added_tokens_decoder") or {}).values():
        if isinstance(entry, dict) and entry.get("special") and isinstance(entry.get("content"), str):
            found.add(entry["content"])
    return list(found)


class HuggingFaceModelTokenizer:
    """Model tokenizer driven by the Jinja ``chat_template`` stored in ``tokenizer_config.json``.
    Masks are derived by rendering growing prefixes of the conversation and attributing the new
    tokens of each step to the message that produced them."""

    def __init__(self, tokenizer_json_path: str, *, tokenizer_config_json_path: Optional[str] = None, generation_config_path: Optional[str] = None, truncation_type: str = "right", max_seq_len: Optional[int] = None):
        import jinja2

        self.base_tokenizer = HuggingFaceBaseTokenizer(tokenizer_json_path, tokenizer_config_json_path=tokenizer_config_json_path, generation_config_path=generation_config_path)
        if not tokenizer_config_json_path:
            raise ValueError("A tokenizer_config.json with a chat_template is required")
        cfg = json.load(open(tokenizer_config_json_path))
        self.special_tokens_list = _infer_special_tokens_from_hf_config(cfg)
        self.special_tokens = {t: self.base_tokenizer.tokenizer.token_to_id(t) for t in self.special_tokens_list}
        env = jinja2.Environment()
        env.globals["raise_exception"] = self._raise_helper
        self.template = env.from_string(cfg["chat_template"])
        self.top_level_variables = {k: v["content"] if isinstance(v, dict) and "content" in v else v for k, v in cfg.items() if k.endswith("_token")}
        self.truncation_type = truncation_type
        self.max_seq_len = max_seq_len

    @staticmethod
    def _raise_helper(message: str):
        import jinja2

        raise jinja2.exceptions.TemplateError(message)

    def render_template(self, messages: List[Dict[str, str]], add_eos: bool = True) -> str:
        return self.template.render(messages=messages, add_generation_prompt=not add_eos, **self.top_level_variables)

    def tokenize_messages(self, messages: List[Message], add_eos: bool = True) -> Tuple[List[int], List[bool]]:
        tokens: List[int] = []
        mask: List[bool] = []
        prev_rendered = ""
        as_dicts: List[Dict[str, str]] = []
        for i, m in enumerate(messages):
            as_dicts.append({"role": m.role, "content": m.text_content})
            last = i == len(messages) - 1
            rendered = self.render_template(as_dicts, add_eos=add_eos if last else True)
            delta = rendered[len(prev_rendered) :] if rendered.startswith(prev_rendered) else rendered
            prev_rendered = rendered
            ids = self.base_tokenizer.encode(delta, add_bos=False, add_eos=False)
            tokens += ids
            mask += [m.masked] * len(ids)
            if self.max_seq_len and len(tokens) >= self.max_seq_len:
                break
        if self.max_seq_len:
            tokens = truncate(tokens, self.max_seq_len, self.base_tokenizer.eos_id if add_eos else None, self.truncation_type)
            mask = truncate(mask, self.max_seq_len, True if add_eos else None, self.truncation_type)
        return tokens, mask

    def __call__(self, sample: Dict[str, Any], inference: bool = False) -> Dict[str, Any]:
        messages = sample.pop("messages")
        tokens, mask = self.tokenize_messages(messages, add_eos=not inference)
        sample["tokens"], sample["mask"] = tokens, mask
        return sample
