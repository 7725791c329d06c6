"""``tune download`` without a network: the Hub client is replaced by a fake, and the command's own behaviour is checked —
default output directory, ignore patterns and token forwarded, the repo id remembered next to the files, and the two Hub
errors turned into the CLI's messages (torchtune/_cli/download.py:120-190)."""
import json
import sys

import pytest

from torchtune_b200._cli import tune


def _run(monkeypatch, argv):
    monkeypatch.setattr(sys, "argv", ["tune"] + argv)
    parser = tune.TuneCLIParser()
    parser.run(parser.parse_args())


def test_download_from_the_hub_writes_files_and_remembers_the_repo(monkeypatch, tmp_path, capsys):
    import huggingface_hub

    calls = {}

    def fake_snapshot_download(repo_id, local_dir=None, ignore_patterns=None, token=None, **_):
        calls.update(repo_id=repo_id, local_dir=local_dir, ignore_patterns=ignore_patterns, token=token)
        out = tmp_path / "model" if local_dir is None else __import__("pathlib").Path(local_dir)
        out.mkdir(parents=True, exist_ok=True)
        (out / "model-00001-of-00001.safetensors").write_bytes(b"weights")
        (out / "config.json").write_text("{}")
        return str(out)

    monkeypatch.setattr(huggingface_hub, "snapshot_download", fake_snapshot_download)
    target = tmp_path / "llama"
    _run(monkeypatch, ["download", "meta-llama/Llama-3.1-8B", "--output-dir", str(target), "--ignore-patterns", "original/consolidated*", "--hf-token", "tok"])
    assert calls == {"repo_id": "meta-llama/Llama-3.1-8B", "local_dir": str(target), "ignore_patterns": "original/consolidated*", "token": "tok"}
    assert json.loads((target / "original_repo_id.json").read_text()) == {"repo_id": "meta-llama/Llama-3.1-8B"}
    printed = capsys.readouterr().out
    assert "Successfully downloaded model repo" in printed and "model-00001-of-00001.safetensors" in printed


def test_download_default_directory_is_named_after_the_model(monkeypatch, tmp_path):
    import huggingface_hub

    seen = {}

    def fake_snapshot_download(repo_id, local_dir=None, **_):
        seen["local_dir"] = local_dir
        (tmp_path / "x").mkdir(exist_ok=True)
        return str(tmp_path / "x")

    monkeypatch.setattr(huggingface_hub, "snapshot_download", fake_snapshot_download)
    _run(monkeypatch, ["download", "org/My-Model"])
    assert seen["local_dir"] == "/tmp/My-Model"


@pytest.mark.parametrize("error,needle", [("GatedRepoError", "gated repository"), ("RepositoryNotFoundError", "not found on the Hugging Face Hub")])
def test_download_hub_errors_become_cli_errors(monkeypatch, tmp_path, capsys, error, needle):
    import huggingface_hub
    from huggingface_hub import utils as hub_utils

    exc_type = getattr(hub_utils, error)

    def failing(*_, **__):
        raise exc_type.__new__(exc_type)  # the Hub's constructors want a response object; the CLI only looks at the type

    monkeypatch.setattr(huggingface_hub, "snapshot_download", failing)
    with pytest.raises(SystemExit) as exit_info:
        _run(monkeypatch, ["download", "org/private", "--output-dir", str(tmp_path / "o")])
    assert exit_info.value.code == 2
    assert needle in capsys.readouterr().err
