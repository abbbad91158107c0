"""Engram hash history (CPU) and device ops (GPU)."""
import os

import numpy as np
import pytest
import torch

from titanic_flash_41_b200.models import engram as EG


def test_hash_history_is_causal_and_transactional():
    md = EG.HashMetadata.synthetic(1000, seed=1, image_token=999)
    h = EG.HashHistory(lineage=7)
    toks = [5, 17, 300, 42, 8, 999, 11, 12, 13, 14]
    whole = h.prepare(toks, md)
    assert whole.rows.shape == (10, 2, 24)
    # every id falls inside its head's slice of the table
    for t in range(2):
        for j in range(24):
            lo = int(md.offsets[t][j])
            assert ((whole.rows[:, t, j] >= lo) & (whole.rows[:, t, j] < lo + int(md.primes[t][j]))).all()
    # committing a prefix and hashing the rest reproduces the same rows (speculative acceptance)
    spec = h.prepare(toks[:4], md)
    h.commit(spec, 3)
    assert h.position == 3 and h.generation == 1
    rest = h.prepare(toks[3:], md)
    assert np.array_equal(rest.rows, whole.rows[3:])
    with pytest.raises(ValueError, match="stale"):
        h.commit(spec, 1)
    # rows whose window touches an image token only depend on the tokens after it
    other = list(toks)
    other[4] = 77
    h2 = EG.HashHistory(lineage=9)
    b2 = h2.prepare(other, md)
    assert np.array_equal(b2.rows[9], whole.rows[9]) and not np.array_equal(b2.rows[4], whole.rows[4])
    assert np.array_equal(b2.rows[6][:, :8], whole.rows[6][:, :8])      # bigram of (11, image) is blocked -> pad
    # padded launch: padding rows cannot be committed
    pad = h.prepare_padded(toks[3:5] + [md.pad_token] * 3, 2, md)
    assert len(pad.tokens) == 2 and pad.rows.shape[0] == 5
    with pytest.raises(ValueError):
        h.commit(pad, 3)


def test_row_format_round_trip(tmp_path):
    v = torch.randn(50, 256) * 3
    packed = EG.pack_rows(v)
    assert packed.shape == (50, 264)
    assert (EG.unpack_rows(packed) - v).abs().max() < 0.07 * v.abs().max()
    p = os.path.join(str(tmp_path), "t.bin")
    EG.write_table(p, packed, row_start=100)
    back, start = EG.read_table(p)
    assert start == 100 and torch.equal(back, packed)
    with open(p, "r+b") as f:
        f.truncate(4096 + 10 * 264)
    with pytest.raises(ValueError, match="truncated"):
        EG.read_table(p)


@pytest.mark.gpu
def test_device_lookup_and_gate_match_references():
    dev = "cuda"
    v = torch.randn(300, 256) * 2
    packed = EG.pack_rows(v)
    tab = EG.EngramTable(packed[100:200], 100, dev)
    ids = torch.tensor([100, 150, 199, 99, 200, 5], dtype=torch.int64)
    got = tab.lookup(ids).float().cpu()
    want = EG.unpack_rows(packed)[ids].bfloat16().float()
    want[3:] = 0                                            # not owned by this rank
    assert torch.equal(got, want)
    g = torch.Generator().manual_seed(0)
    r, m, d = 9, 4, 1024
    x = torch.randn(r, m, d, generator=g).bfloat16()
    kv = torch.randn(r, m + 1, d, generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(m, d, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(m, d, generator=g)).bfloat16()
    out = EG.gate(x.to(dev), kv.to(dev), qw.to(dev), kw.to(dev), 1e-6).float().cpu()
    ref = EG.gate_reference(x.float(), kv.float(), qw.float(), kw.float(), 1e-6)
    assert (out - ref).abs().max() < 0.03


def test_engram_layer_in_the_oracle_model():
    """Engram in the model path: chunked == whole, overwritten speculative rows leave no trace, and the
    memory actually changes the logits."""
    from titanic_flash_41_b200.config import EngramConfig, tiny_config
    from titanic_flash_41_b200.models import oracle
    cfg = tiny_config(engram=EngramConfig(layers=(0, 1), rows_per_table=1500))
    W = oracle.init_weights(cfg, 1)
    assert W["engram.0.table"].shape[1] == 256 and "layers.1.engram.wkv.weight" in W
    m = oracle.OracleModel(cfg, W)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(3, cfg.vocab, (30,), generator=g)
    s1 = m.new_session(64)
    whole = m.forward(toks, s1)
    s2 = m.new_session(64)
    a = m.forward(toks[:13], s2)
    b = m.forward(toks[13:], s2)
    assert torch.allclose(torch.cat([a, b]), whole, atol=2e-4, rtol=1e-4)
    # speculative rows at positions 30.. are replaced by other tokens: same result as never having run them
    m.forward(torch.randint(3, cfg.vocab, (4,), generator=g), s2, commit=False)
    nxt = torch.randint(3, cfg.vocab, (4,), generator=g)
    x = m.forward(nxt, s2, start=30)
    y = m.forward(nxt, s1)
    assert torch.allclose(x, y, atol=2e-4, rtol=1e-4)
    # without the memory the model is a different function
    plain = oracle.OracleModel(tiny_config(), {k: v for k, v in W.items() if "engram" not in k})
    assert not torch.allclose(plain.forward(toks, plain.new_session(64)), whole, atol=1e-3)


def test_row_store_on_disk_with_set_associative_host_cache(tmp_path):
    """Rows come back exactly as written; repeated ids hit the host cache; a full set evicts its
    least recently used way; ids outside the store's interval read as zero rows."""
    import os

    import numpy as np
    import torch

    from titanic_flash_41_b200.models import engram as EG
    from titanic_flash_41_b200.utils import build
    build.build(verbose=False)                         # the batched reader lives in the host runtime library
    rows = 5000
    packed = EG.pack_rows(torch.randn(rows, 256, generator=torch.Generator().manual_seed(3)))
    path = os.path.join(str(tmp_path), "table.bin")
    EG.write_table(path, packed, row_start=1000)
    store = EG.EngramRowStore(path, cache_rows=64, ways=4, threads=4)
    assert (store.row_start, store.row_end) == (1000, 6000) and store.sets == 16
    ids = np.array([1000, 1005, 5999, 999, 6000, 1005, 2500], dtype=np.int64)
    got = store.lookup(ids)
    want = packed.numpy()
    assert (got[0] == want[0]).all() and (got[1] == want[5]).all() and (got[2] == want[4999]).all()
    assert (got[3] == 0).all() and (got[4] == 0).all() and (got[5] == want[5]).all() and (got[6] == want[1500]).all()
    assert store.stats["reads"] == 4 and store.stats["foreign"] == 2       # the repeated id was read once
    again = store.lookup(ids)
    assert (again == got).all() and store.stats["reads"] == 4 and store.stats["hits"] >= 5
    # five rows of one set in a 4-way cache: the oldest one is evicted and read again
    same_set = np.array([1000 + 16 * k for k in range(5)], dtype=np.int64)
    store.lookup(same_set[:4])
    store.lookup(same_set[4:])
    before = store.stats["reads"]
    store.lookup(same_set[1:2])
    assert store.stats["reads"] == before              # still cached
    store.lookup(same_set[0:1])
    assert store.stats["reads"] == before + 1          # was the least recently used way
    big = np.random.default_rng(0).integers(1000, 6000, size=3000)
    assert (store.lookup(big) == want[big - 1000]).all()
