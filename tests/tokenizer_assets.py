"""Tiny tokenizer files generated on the fly for tests (no binary assets in the tree)."""
import base64
import json
from pathlib import Path

CORPUS = [
    "Hello world! How are you today?",
    "The quick brown fox jumps over the lazy dog.",
    "Fine-tuning large language models on Blackwell GPUs is fun.",
    "You are a helpful assistant.",
    "What is the capital of France? The capital of France is Paris.",
    "1 2 3 4 5 6 7 8 9 10 one two three four five six seven eight nine ten",
] * 20


def write_tiktoken_file(path: Path) -> Path:
    """All 256 single bytes plus a handful of merged byte pairs, in tiktoken's text format."""
    tokens = [bytes([b]) for b in range(256)]
    for word in (b"he", b"ll", b"llo", b"hello", b" w", b"or", b" wor", b"ld", b" world", b"th", b" th", b" the", b"in", b"er", b"an", b"re", b"on", b"at", b"en", b"ou"):
        if word not in tokens:
            tokens.append(word)
    with open(path, "w") as f:
        for rank, tok in enumerate(tokens):
            f.write(f"{base64.b64encode(tok).decode()} {rank}\n")
    return path


def write_sentencepiece_model(dirpath: Path, vocab_size: int = 200) -> Path:
    import sentencepiece as spm

    corpus = dirpath / "corpus.txt"
    corpus.write_text("\n".join(CORPUS))
    prefix = dirpath / "spm_tiny"
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(prefix), vocab_size=vocab_size, model_type="bpe", bos_id=1, eos_id=2, unk_id=0, pad_id=-1, minloglevel=2, hard_vocab_limit=False)
    return Path(str(prefix) + ".model")


def write_gpt2_files(dirpath: Path):
    """Byte-level vocab with a few merges in GPT-2's vocab.json / merges.txt format."""
    from torchtune_b200.modules.transforms.tokenizers._gpt2 import bytes_to_unicode

    table = bytes_to_unicode()
    vocab = {table[b]: b for b in range(256)}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("o", "r"), ("Ġw", "or"), ("l", "d"), ("Ġwor", "ld")]
    for a, b in merges:
        vocab.setdefault(a + b, len(vocab))
    for special in ("<|endoftext|>", "<|im_start|>", "<|im_end|>"):
        vocab[special] = len(vocab)
    (dirpath / "vocab.json").write_text(json.dumps(vocab))
    (dirpath / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n")
    return dirpath / "vocab.json", dirpath / "merges.txt"
