"""Device chunk pool: pooled allocations, elastic ranges, exhaustion as an error code."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pool_alloc_free_elastic_and_exhaustion():
    from titanic_flash_41_b200.utils.vmm import ChunkPool, PoolExhausted
    pool = ChunkPool(n_chunks=6, chunk_bytes=2 << 20)
    try:
        total, free = pool.counts()
        assert total == 6 and free == 6 and pool.chunk >= 2 << 20
        a = pool.alloc(3 * pool.chunk - 100)                 # 3 chunks
        ta = a.tensor(3 * pool.chunk - 100)
        ta.copy_(torch.arange(ta.numel(), device="cuda") % 251)
        assert pool.counts()[1] == 3
        # elastic range: addresses stay, the tail comes and goes
        e = pool.reserve(8 * pool.chunk, pool.chunk)
        te = e.tensor()
        te.fill_(7)
        base = e.base
        e.resize(2 * pool.chunk + 5)                         # grows to 3 chunks
        assert e.base == base and pool.counts()[1] == 0
        t3 = e.tensor(3 * pool.chunk)
        assert int(t3[: pool.chunk].min()) == 7              # the mapped prefix kept its contents
        t3[pool.chunk:].fill_(9)
        with pytest.raises(PoolExhausted):
            pool.alloc(1)
        with pytest.raises(PoolExhausted):
            e.resize(4 * pool.chunk)
        torch.cuda.synchronize()
        e.resize(pool.chunk)
        assert pool.counts()[1] == 2 and int(e.tensor()[100]) == 7
        # data of the first allocation is intact
        want = torch.arange(ta.numel(), device="cuda") % 251
        assert torch.equal(ta.long(), want)
        torch.cuda.synchronize()
        del ta, te, t3
        a.free()
        e.free()
        assert pool.counts() == (6, 6)
        b = pool.alloc(6 * pool.chunk)                       # every chunk is reusable
        b.tensor().zero_()
        torch.cuda.synchronize()
        b.free()
    finally:
        pool.destroy()
    assert torch.ones(3, device="cuda").sum().item() == 3.0


def test_state_image_in_the_pool_round_trips_and_returns_chunks():
    from titanic_flash_41_b200.serve import state_image as SI
    from titanic_flash_41_b200.utils.vmm import ChunkPool, PoolExhausted
    pool = ChunkPool(n_chunks=4, chunk_bytes=2 << 20)
    try:
        a = torch.randn(300, 1000, device="cuda")
        b = torch.randint(0, 255, (7, 33), dtype=torch.uint8, device="cuda")
        img = SI.capture([1, 2, 3], [("a", a), ("b", b)], pool=pool)
        assert pool.counts()[1] < 4 and img.tier == "device"
        want = SI.capture([1, 2, 3], [("a", a), ("b", b)]).digest()
        assert img.digest() == want
        a2, b2 = torch.zeros_like(a), torch.zeros_like(b)
        SI.restore_into(img, {"a": a2, "b": b2})
        assert torch.equal(a, a2) and torch.equal(b, b2)
        with pytest.raises(PoolExhausted):
            SI.capture([1], [("big", torch.zeros(5 * pool.chunk, dtype=torch.uint8, device="cuda"))], pool=pool)
        img.to_host(pin=False)                         # leaves the device tier: chunks go back
        assert pool.counts() == (4, 4) and img.digest() == want
    finally:
        pool.destroy()
