"""Push protocol for policy weights between two jobs that share no default process group: a parameter server (rank 0) and an
inference-side worker (rank 1) over a stateless gloo group, as child processes on CPU."""
import socket

import pytest
import torch
import torch.multiprocessing as mp
from torch import nn


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model(seed: int) -> nn.Module:
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))


def _server(port: int, out) -> None:
    from torchtune_b200.dev.rl.workers import BroadcastParameterServer

    src = _model(1)
    ps = BroadcastParameterServer(src.state_dict())
    ps.init_update_group("127.0.0.1", port, world_size=2, timeout_s=60)
    ps.publish(src.state_dict())
    v1 = ps.push()
    with torch.no_grad():
        for p in src.parameters():
            p.add_(1.0)
    ps.publish(src.state_dict())
    v2 = ps.push()
    ps.close()
    out.put(("server", v1, v2, {k: v.tolist() for k, v in src.state_dict().items()}))


def _worker(port: int, out) -> None:
    import torch.distributed as dist

    from torchtune_b200.dev.rl.workers import GeneratorWeightWorker

    model = _model(2)
    w = GeneratorWeightWorker(model, device=torch.device("cpu"))
    w.init_weight_update_group("127.0.0.1", port, rank_offset=1, world_size=2, timeout_s=60)
    v1 = w.receive()
    v2 = w.receive()
    w.close()
    out.put(("worker", v1, v2, {k: v.tolist() for k, v in model.state_dict().items()}, dist.is_initialized()))


@pytest.mark.timeout(180)
def test_weights_and_version_cross_a_stateless_group():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_server, args=(port, out)), ctx.Process(target=_worker, args=(port, out))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        item = out.get(timeout=120)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    sv1, sv2, sent = got["server"]
    wv1, wv2, received, default_group = got["worker"]
    assert (sv1, sv2) == (1, 2) and (wv1, wv2) == (1, 2)
    assert not default_group  # the bridge leaves torch.distributed's global state alone
    for k in sent:
        assert sent[k] == received[k]


def test_worker_refuses_the_server_rank():
    from torchtune_b200.dev.rl.workers import GeneratorWeightWorker

    with pytest.raises(ValueError):
        GeneratorWeightWorker(_model(0), device=torch.device("cpu")).init_weight_update_group("127.0.0.1", 1, rank_offset=0, world_size=2)


def test_old_tokenizer_path_warns_and_resolves():
    import importlib
    import sys

    sys.modules.pop("torchtune_b200.modules.tokenizers", None)
    with pytest.warns(DeprecationWarning):
        mod = importlib.import_module("torchtune_b200.modules.tokenizers")
    from torchtune_b200.modules.transforms.tokenizers import ModelTokenizer

    assert mod.ModelTokenizer is ModelTokenizer
