import pytest

from tokenizer_assets import write_gpt2_files, write_sentencepiece_model, write_tiktoken_file
from torchtune_b200.data import Message
from torchtune_b200.modules.transforms.tokenizers import GPT2BaseTokenizer, SentencePieceBaseTokenizer, TikTokenBaseTokenizer, tokenize_messages_no_special_tokens


def test_tiktoken_round_trip_and_long_runs(tmp_path):
    from torchtune_b200.models.llama3._tokenizer import CL100K_PATTERN

    tok = TikTokenBaseTokenizer(str(write_tiktoken_file(tmp_path / "tt.model")), "t", CL100K_PATTERN, bos_id=1000, eos_id=1001, special_tokens={"<|a|>": 1000, "<|b|>": 1001})
    ids = tok.encode("hello world", add_bos=True, add_eos=True)
    assert ids[0] == 1000 and ids[-1] == 1001
    assert tok.decode(ids[1:-1]) == "hello world"
    assert len(ids) < 2 + len("hello world")  # merges were applied
    pieces = list(tok._split_long_repetitions("a" * 10 + " " * 3 + "b" * 7, 4))
    import re

    assert "".join(pieces) == "a" * 10 + " " * 3 + "b" * 7
    assert all(len(run) <= 4 for piece in pieces for run in re.findall(r"\s+|\S+", piece))
    assert tok.encode("") == []


def test_llama3_tokenizer_layout(tmp_path):
    from torchtune_b200.models.llama3 import llama3_tokenizer

    tok = llama3_tokenizer(str(write_tiktoken_file(tmp_path / "tt.model")), max_seq_len=None)
    msgs = [Message(role="user", content="hello world", masked=True), Message(role="assistant", content="hello")]
    tokens, mask = tok.tokenize_messages(msgs)
    assert tokens[0] == tok.bos_id and tokens[-1] == tok.eos_id and mask[0] and mask[-1]
    assert tokens.count(tok.start_header_id) == 2 and tokens.count(tok.eot_id) == 2
    assert tok.decode(tokens) == "hello worldhello"
    # generation prompt: the last message is left open
    open_tokens, _ = tok.tokenize_messages(msgs[:1] + [Message(role="assistant", content="")], add_end_tokens=False)
    assert open_tokens[-1] != tok.eos_id and open_tokens.count(tok.eot_id) == 1
    # tool call: eom instead of eot, python tag in front
    call = Message(role="assistant", content="hello", ipython=True, eot=False)
    ids = tok.tokenize_message(call)
    assert ids[-1] == tok.eom_id and tok.python_tag in ids
    # truncation forces eos
    tok.max_seq_len = 8
    t2, m2 = tok.tokenize_messages(msgs)
    assert len(t2) == 8 and t2[-1] == tok.eos_id and m2[-1] is True
    out = tok({"messages": msgs})
    assert set(out) == {"tokens", "mask"}


def test_sentencepiece_and_plain_message_tokenization(tmp_path):
    sp = SentencePieceBaseTokenizer(str(write_sentencepiece_model(tmp_path)))
    ids = sp.encode("Hello world", add_bos=True, add_eos=True)
    assert ids[0] == sp.bos_id and ids[-1] == sp.eos_id and sp.decode(ids) == "Hello world"
    trimmed = sp.encode("world", add_bos=False, add_eos=False, trim_leading_whitespace=True)
    assert sp.decode(trimmed) == "world"

    class Tok:
        max_seq_len = None

        def encode(self, text, **kw):
            return sp.encode(text, **kw)

    msgs = [Message(role="user", content="Hello world ", masked=True), Message(role="assistant", content="fine")]
    tokens, mask = tokenize_messages_no_special_tokens(Tok(), msgs, bos_id=sp.bos_id, eos_id=sp.eos_id)
    assert tokens[0] == sp.bos_id and tokens[-1] == sp.eos_id
    assert mask[0] is True and mask[-1] is False and len(tokens) == len(mask)


def test_gpt2_bpe(tmp_path):
    vocab, merges = write_gpt2_files(tmp_path)
    tok = GPT2BaseTokenizer(str(vocab), str(merges), unk_id=0, bos_id=None, eos_id=None)
    ids = tok.encode("hello world")
    assert len(ids) == 2 and tok.decode(ids) == "hello world"
    assert tok.decode(tok.encode("héllo ∑")) == "héllo ∑"
