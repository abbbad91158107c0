"""Single-rank sanity of the PyTorch oracle and the TP=2 gloo plumbing check."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from titanic_flash_41_b200.config import tiny_config
from titanic_flash_41_b200.models import oracle


def _prompts(cfg, batch=2, n=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab, (n,), generator=g) for _ in range(batch)]


def test_chunked_prefill_equals_one_shot():
    cfg = tiny_config()
    W = oracle.init_weights(cfg, 0)
    m = oracle.OracleModel(cfg, W)
    p = _prompts(cfg, 1, 50)[0]
    s1 = m.new_session(64)
    full = m.forward(p, s1)
    s2 = m.new_session(64)
    parts = [m.forward(p[a:b], s2) for a, b in ((0, 7), (7, 30), (30, 31), (31, 50))]
    assert torch.allclose(torch.cat(parts), full, atol=2e-5)


def test_mixed_compression_ratios_per_source_layer():
    """Two source layers with their own ratios (the reference pools pairs in layers 2-19 and keeps every
    token from layer 20 on, src/config.rs:252-280): each stream gets position // ratio entries, chunked
    prefill equals one shot, and the coarser stream changes the logits against a uniform fine one."""
    kw = dict(n_layers=3, kv_source_layers=(0, 1), index_source_layers=(0, 1, 2), index_topk=8)
    cfg = tiny_config(compress_ratio=1, compress_ratios=(2, 1), **kw)
    assert [cfg.ratio_of(l) for l in range(3)] == [2, 1, 1] and cfg.max_ratio == 2
    W = oracle.init_weights(cfg, 0)
    m = oracle.OracleModel(cfg, W)
    p = _prompts(cfg, 1, 51)[0]
    s1 = m.new_session(64)
    full = m.forward(p, s1)
    assert s1.comp["layers.0"].shape[0] == 64 // 2 + 1 and s1.comp["layers.1"].shape[0] == 64 + 1
    # 25 complete pairs in the coarse stream, 51 entries in the fine one
    assert bool(s1.comp["layers.0"][:25].abs().sum(-1).gt(0).all()) and not bool(s1.comp["layers.0"][25:].any())
    assert bool(s1.comp["layers.1"][:51].abs().sum(-1).gt(0).all()) and not bool(s1.comp["layers.1"][51:].any())
    assert m.last_selection[2].shape == (51, 8) and int(m.last_selection[2].max()) <= 50
    assert int(m.last_selection[0].max()) <= 24
    s2 = m.new_session(64)
    parts = [m.forward(p[a:b], s2) for a, b in ((0, 7), (7, 30), (30, 31), (31, 51))]
    assert torch.allclose(torch.cat(parts), full, atol=2e-5)
    uni = oracle.OracleModel(tiny_config(compress_ratio=1, **kw), W)
    assert not torch.allclose(uni.forward(p, uni.new_session(64)), full, atol=1e-3)
    with pytest.raises(ValueError):
        tiny_config(compress_ratio=2, compress_ratios=(2, 3), **kw)
    with pytest.raises(ValueError):
        tiny_config(compress_ratio=1, compress_ratios=(2,), **kw)


def test_rollback_of_speculative_rows():
    cfg = tiny_config()
    m = oracle.OracleModel(cfg, oracle.init_weights(cfg, 1))
    p = _prompts(cfg, 1, 40, 3)[0]
    s = m.new_session(64)
    m.forward(p[:30], s)
    junk = torch.randint(0, cfg.vocab, (6,))
    m.forward(junk, s, commit=False)            # rejected speculative rows
    got = m.forward(p[30:], s)
    s2 = m.new_session(64)
    want = m.forward(p, s2)[30:]
    assert torch.allclose(got, want, atol=2e-5)


def test_hyper_connections_and_lora_variants_run():
    cfg = tiny_config(hc_mult=4, q_lora_rank=64, o_groups=2, o_lora_rank=32,
                      scoring="sqrtsoftplus", router_bias=True, route_scale=1.5, swiglu_limit=10.0)
    m = oracle.OracleModel(cfg, oracle.init_weights(cfg, 2))
    s = m.new_session(40)
    lg = m.forward(_prompts(cfg, 1, 33)[0], s)
    assert lg.shape == (33, cfg.vocab) and torch.isfinite(lg).all()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_config(variant):
    if variant == "mixed":                       # two compressed streams with their own ratios
        return tiny_config(n_layers=3, compress_ratio=1, compress_ratios=(2, 1), kv_source_layers=(0, 1),
                           index_source_layers=(0, 1, 2), index_topk=8)
    return tiny_config()


def _tp_worker(rank, world, port, q, moe_parallel, variant="plain"):
    import torch.distributed as dist
    from titanic_flash_41_b200.parallel.comm import DistComm
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cfg = _tp_config(variant)
    W = oracle.shard_weights(oracle.init_weights(cfg, 0), cfg, rank, world, moe_parallel)
    m = oracle.OracleModel(cfg, W, DistComm(), moe_parallel)
    toks, logits = oracle.greedy_generate(m, _prompts(cfg), 16)
    if rank == 0:
        q.put((toks, [l.numpy() for l in logits]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("moe_parallel,variant", [("ep", "plain"), ("tp", "plain"), ("ep", "mixed")])
def test_tp2_gloo_matches_single_rank(moe_parallel, variant):
    """Tiny 2-layer MoE decoder, batch 2, 64 prompt ids then 16 greedy steps: logits of the
    TP=2 gloo run within 1e-4 of the single-rank run ("mixed": three layers, two compressed streams
    with their own ratios)."""
    cfg = _tp_config(variant)
    ref = oracle.OracleModel(cfg, oracle.init_weights(cfg, 0))
    toks1, logits1 = oracle.greedy_generate(ref, _prompts(cfg), 16)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q, moe_parallel, variant)) for r in range(2)]
    for p in procs:
        p.start()
    toks2, logits2 = q.get(timeout=300)
    for p in procs:
        p.join(60)
    assert toks1 == toks2
    for a, b in zip(logits1, logits2):
        assert torch.allclose(a, torch.from_numpy(b), atol=1e-4)


def test_reference_feature_set_composes_at_toy_widths():
    """Everything the reference model combines, at toy widths on the CPU oracle: per-source compression
    ratios, four residual copies, low-rank query, grouped low-rank output, n-gram memory layers, a
    two-layer drafter with Markov correction and confidence head.  Chunked prefill equals one shot, the
    serving backend decodes with causal stopping, and a state image restores the conversation exactly."""
    from titanic_flash_41_b200.config import DraftConfig, EngramConfig, RopeConfig, reference_1017_config
    from titanic_flash_41_b200.serve.backend import OracleBackend
    from titanic_flash_41_b200.spec.decoder import DecodeSlot
    cfg = reference_1017_config(
        n_layers=5, hidden=128, vocab=512, n_heads=4, head_dim=32, q_lora_rank=32, o_groups=2, o_lora_rank=16, window=16,
        kv_source_layers=(1, 3), compress_ratios=(2, 1), index_source_layers=(1, 3, 4), index_heads=2, index_dim=32,
        index_topk=8, candidate_blocks=0, late_start=4, n_experts=8, topk=2, moe_inter=64, shared_inter=64,
        rope=RopeConfig(theta=10000.0, compress_theta=160000.0, dim=16), dense_quant="none", expert_quant="none",
        kv_quant="none", draft=DraftConfig(layers=2, depth=4, condition_layers=1, markov_rank=16, confidence_head=True),
        vision=None, engram=EngramConfig(layers=(1, 2), rows_per_table=64, width=256, heads=2, ngram=3, tables=2))
    assert cfg.hc_mult == 4 and [cfg.ratio_of(l) for l in range(5)] == [1, 2, 2, 1, 1]
    W = oracle.init_weights(cfg, 0)
    m = oracle.OracleModel(cfg, W)
    p = _prompts(cfg, 1, 45, 5)[0]
    s1, s2 = m.new_session(64), m.new_session(64)
    full = m.forward(p, s1)
    parts = torch.cat([m.forward(p[a:b], s2) for a, b in ((0, 9), (9, 31), (31, 45))])
    assert torch.isfinite(full).all() and torch.allclose(parts, full, atol=5e-5)

    def decode(backend, slot, rounds):
        for _ in range(rounds):
            toks = backend.decode_step([slot])[0]
            assert 1 <= len(toks) <= slot.verified + 1 <= 5 and len(slot.confidence) >= slot.verified
        return list(slot.emitted)
    b = OracleBackend(cfg, W, regions=2, max_context=128, chunk=16)
    prompt = p.tolist()
    lg = b.prefill(0, prompt, 0, None)
    mk = lambda region, length, anchor, emitted=(): DecodeSlot(region=region, length=length, anchor=anchor, seed=1, temperature=0.7,
                                                              top_p=0.9, recent=(prompt + list(emitted))[-8:])
    sl = mk(0, 45, int(lg.argmax()))
    first = decode(b, sl, 3)
    img = b.snapshot(0, prompt + first[: sl.length - 45])
    anchor = sl.anchor
    rest = decode(b, sl, 3)[len(first):]
    # the same conversation restored into the other region continues with the same tokens
    b.restore(1, img)
    sl2 = mk(1, img.length, anchor, first)
    sl2.emitted = list(first)
    assert decode(b, sl2, 3)[len(first):] == rest
