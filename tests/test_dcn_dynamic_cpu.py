"""DCN v2 over the dynamic hash-table collection (CPU host table): trains, admits on the second sighting, and the
incremental dump returns the rows touched since the given score."""
import torch

from recsdk_b200.dynamic import incremental_dump
from recsdk_b200.models.dcn_bench import build, make_batch
from recsdk_b200.parallel.comm import ShardingEnv


def test_dcn_dynamic_trains_and_dumps():
    torch.manual_seed(0)
    model, opt, emb, dense = build(torch.device("cpu"), ShardingEnv(1, 0, None), 1 << 14)
    gen = torch.Generator().manual_seed(1)
    batches = [make_batch(64, gen, key_bits=12, max_len=3) for _ in range(4)]
    losses = []
    for ep in range(4):
        for b in batches:
            opt.zero_grad()
            loss, _ = model(b)
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
    assert sum(losses[-4:]) < sum(losses[:4])
    out, scores = incremental_dump(model, 0, None)
    (tabs,) = out.values()
    keys, vals = tabs["tab"]
    assert keys.numel() > 0 and vals.shape == (keys.numel(), 64)
