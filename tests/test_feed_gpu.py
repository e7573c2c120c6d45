"""HostBatchFeed: batches come out in order, bit-identical to the pinned host tensors, also
when the buffers are reused several times and the consumer works on them on its stream."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_feed_order_and_contents():
    from picassoplus_b200.parallel import HostBatchFeed
    g = torch.Generator().manual_seed(3)
    batches = []
    for rows in (1000, 257, 4096, 1, 3000):
        batches.append(dict(a=torch.randn(rows, 7, generator=g).pin_memory(),
                            b=torch.randint(0, 1 << 30, (rows * 2, 3), generator=g, dtype=torch.int32).pin_memory()))
    dev = torch.device("cuda", 0)
    feed = HostBatchFeed(batches, dev, depth=2)
    assert feed.bytes_per_pass == sum(t.numel() * t.element_size() for b in batches for t in b.values())
    for _ in range(3):                                  # buffers are reused across passes
        sums = []
        for i, d in enumerate(feed):
            assert d["a"].shape == batches[i]["a"].shape and d["b"].shape == batches[i]["b"].shape
            assert d["a"].data_ptr() % 16 == 0
            # consumer work on the current stream that reads the buffer after the next copy was issued
            sums.append((d["a"].double().sum(), d["b"].long().sum(), d["a"].clone(), d["b"].clone()))
        torch.cuda.synchronize()
        for i, (sa, sb, ca, cb) in enumerate(sums):
            assert torch.equal(ca.cpu(), batches[i]["a"]) and torch.equal(cb.cpu(), batches[i]["b"])
            assert float(sa) == float(batches[i]["a"].double().sum()) and int(sb) == int(batches[i]["b"].long().sum())


def test_feed_cycle_crosses_pass_boundaries():
    """cycle(): pass after pass as one stream (odd batch count, two buffers: the buffer of a batch
    alternates between passes), contents and order stay exact."""
    from picassoplus_b200.parallel import HostBatchFeed
    g = torch.Generator().manual_seed(5)
    batches = [dict(a=torch.randn(rows, 5, generator=g).pin_memory()) for rows in (513, 64, 2049)]
    feed = HostBatchFeed(batches, torch.device("cuda", 0), depth=2)
    it = feed.cycle()
    kept = []
    for i in range(10):
        d = next(it)
        assert d["a"].shape == batches[i % 3]["a"].shape
        kept.append(d["a"].clone())
    torch.cuda.synchronize()
    for i, c in enumerate(kept):
        assert torch.equal(c.cpu(), batches[i % 3]["a"])
