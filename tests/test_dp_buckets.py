"""Layout of the bucketed flat parameter store: one bucket per decoder layer, every rank owns the slice with its index of
every bucket, and optimizer state moves between the per-rank and the flat-parameter order without loss."""
import torch

from torchtune_b200.models.llama3_1 import llama3_1
from torchtune_b200.parallel.dp import FlatParameters

ARCH = dict(vocab_size=64, num_layers=3, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48, norm_eps=1e-5, rope_base=10000)


def _flat(world):
    model = llama3_1(**ARCH)
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    return model, FlatParameters(named, world, torch.device("cpu"))


def test_buckets_follow_layers_and_are_divisible():
    for world in (1, 2, 8):
        model, flat = _flat(world)
        assert flat.bucket_keys == [None, "layers.0", "layers.1", "layers.2", None]
        assert len(flat.buckets) == 5
        cursor = 0
        for (start, size), piece in zip(flat.buckets, flat.pieces):
            assert start == cursor and size % (8 * world) == 0 and piece * world == size
            cursor += size
        assert cursor == flat.total and flat.shard == sum(flat.pieces)
        # every parameter lies inside the bucket of its layer and the model still works on the re-homed storage
        for name, p, off in zip(flat.names, flat.params, flat.offsets):
            b = next(i for i, (s, n) in enumerate(flat.buckets) if s <= off < s + n)
            assert off + p.numel() <= flat.buckets[b][0] + flat.buckets[b][1]
            key = flat.bucket_keys[b]
            assert (key is None and not name.startswith("layers.")) or name.startswith(key + ".")
        out = model(torch.randint(0, 64, (1, 8)))
        assert out.shape == (1, 8, 64)


def test_ownership_covers_every_element_once_and_state_round_trips():
    world = 4
    _, flat = _flat(world)
    seen = torch.zeros(flat.total, dtype=torch.int32)
    for r in range(world):
        for b in range(len(flat.buckets)):
            begin, count, off = flat.owned(b, r)
            seen[begin : begin + count] += 1
            assert off == flat.state_offsets[b] and begin % 8 == 0 and count % 8 == 0
    assert bool((seen == 1).all())
    full = torch.arange(flat.total, dtype=torch.float32)
    shards = []
    for r in range(world):
        sh = torch.empty(flat.shard)
        flat.full_to_shard(full, r, sh)
        shards.append(sh)
    assert torch.equal(flat.shards_to_full(shards), full)
