"""End-to-end: the CUDA engine against the PyTorch oracle on the same (quantised) weights."""
import pytest
import torch

from titanic_flash_41_b200.config import EngineConfig, ModelConfig, RopeConfig
from titanic_flash_41_b200.models import engine as E
from titanic_flash_41_b200.models import oracle

pytestmark = pytest.mark.gpu


def _row_err(got, want):
    return (got - want).abs().amax(-1) / want.abs().max()


def small_config(**over):
    kw = dict(name="small", n_layers=3, hidden=512, vocab=2048, n_heads=4, head_dim=128, window=32,
              compress_ratio=4, kv_source_layers=(0,), index_source_layers=(0, 2), index_heads=4,
              index_dim=128, index_topk=16, n_experts=8, topk=2, moe_inter=256, n_shared=1,
              shared_inter=256, scoring="sqrtsoftplus", router_bias=True, route_scale=1.5,
              swiglu_limit=10.0, rope=RopeConfig(theta=10000.0, compress_theta=160000.0, dim=64),
              dense_quant="fp8_block128", expert_quant="mxfp4", kv_quant="v41", init_std=0.05)
    kw.update(over)
    return ModelConfig(**kw)


def test_engine_matches_oracle_prefill_and_decode():
    cfg = small_config()
    W = oracle.init_weights(cfg, 0)
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=g)
    s = ref.new_session(256)
    want = ref.forward(prompt, s)
    got = eng.forward(E.StepPlan.build([(1, 0, prompt.tolist())])).cpu()
    eng.status.check()
    # a near-tie in the router can flip an expert for a row, so rows are assessed statistically (the median
    # of this small random model moves between 0.04 and 0.10 with the weight seed alone)
    err = _row_err(got, want)
    assert err.median() < 0.11 and (err < 0.15).float().mean() >= 0.7, err
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.7
    # decode 6 verification blocks of 4 rows (teacher-forced from the oracle's greedy tokens)
    pos, errs = 77, []
    for step in range(6):
        toks = torch.randint(0, cfg.vocab, (4,), generator=g)
        want = ref.forward(toks, s)
        got = eng.forward(E.StepPlan.build([(1, pos, toks.tolist())])).cpu()
        pos += 4
        errs.append(_row_err(got, want))
    eng.status.check()
    errs = torch.cat(errs)
    assert errs.median() < 0.11 and (errs < 0.15).float().mean() >= 0.7, errs


def test_mixed_compression_ratios_match_oracle_and_travel_in_state_images():
    """Two compressed streams with their own ratios (pairs pooled at the first source, every token kept
    at the second: the reference's layers 2-19 / 20-39, src/config.rs:252-280): prefill and decode rows
    against the oracle, then the state image of the conversation restored into another region
    continues with identical logits."""
    from titanic_flash_41_b200.serve.backend import EngineBackend
    # index_topk above the entry count and every expert routed: nothing discrete can flip on a
    # near-tie (selection and routing have their own tests), so EVERY row must agree closely
    cfg = small_config(n_layers=4, compress_ratio=1, compress_ratios=(2, 1), kv_source_layers=(0, 2),
                       index_source_layers=(0, 2, 3), index_topk=128, topk=8)
    W = oracle.init_weights(cfg, 0)
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=g)
    s = ref.new_session(256)
    want = ref.forward(prompt, s)
    got = eng.forward(E.StepPlan.build([(1, 0, prompt.tolist())])).cpu()
    eng.status.check()
    err = _row_err(got, want)
    assert err.max() < 0.15 and err.median() < 0.07, err
    # 38 pairs in the coarse stream, 77 entries in the fine one; nothing written past them
    assert bool(eng.comp[0, 1, :38].any(-1).all()) and not bool(eng.comp[0, 1, 38:].any())
    assert bool(eng.comp[1, 1, :77].any(-1).all()) and not bool(eng.comp[1, 1, 77:].any())
    pos, errs = 77, []
    for step in range(4):
        toks = torch.randint(0, cfg.vocab, (4,), generator=g)
        want = ref.forward(toks, s)
        got = eng.forward(E.StepPlan.build([(1, pos, toks.tolist())])).cpu()
        pos += 4
        errs.append(_row_err(got, want))
    eng.status.check()
    errs = torch.cat(errs)
    assert errs.max() < 0.15 and errs.median() < 0.07, errs
    be = EngineBackend(eng, chunk=128)
    img = be.snapshot(1, list(range(pos)))
    be.restore(0, img)
    toks = torch.randint(0, cfg.vocab, (4,), generator=g).tolist()
    a = eng.forward(E.StepPlan.build([(1, pos, toks)])).cpu()
    b = eng.forward(E.StepPlan.build([(0, pos, toks)])).cpu()
    eng.status.check()
    assert torch.equal(a, b)


def test_block_scaled_expert_path_matches_register_path_and_oracle():
    """Decode rows with the routed experts on block-scaled tcgen05 MMAs.  MXFP8 activations are a
    different arithmetic from f16 ones (the W4A8 form of the reference's expert kernels): the
    oracle's logits move by some amount when its experts see MXFP8 activations, and the engine's
    move by no more than that when it switches from the register-fed f16 form to this one."""
    cfg = small_config(moe_inter=512)
    W = oracle.init_weights(cfg, 0)
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    assert eng._moe_mx_ok(4) and "x8" in eng._bufs(4)
    old = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,),
                                                  moe_block_scaled=False), W)
    assert "x8" not in old._bufs(4)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (77,), generator=g)
    s, s_mx = ref.new_session(256), ref.new_session(256)
    ref.forward(prompt, s)
    ref.forward(prompt, s_mx)
    eng.forward(E.StepPlan.build([(1, 0, prompt.tolist())]))
    old.forward(E.StepPlan.build([(1, 0, prompt.tolist())]))
    pos, errs, errs_old, between, oracle_shift = 77, [], [], [], []
    for step in range(6):
        toks = torch.randint(0, cfg.vocab, (4,), generator=g)
        ref.expert_act_mx8 = False
        want = ref.forward(toks, s)
        ref.expert_act_mx8 = True          # the oracle's experts see MXFP8 activations as the kernel's do
        want_mx = ref.forward(toks, s_mx)
        got = eng.forward(E.StepPlan.build([(1, pos, toks.tolist())])).cpu()
        got_old = old.forward(E.StepPlan.build([(1, pos, toks.tolist())])).cpu()
        pos += 4
        errs.append(_row_err(got, want_mx))
        errs_old.append(_row_err(got_old, want))
        between.append(_row_err(got, got_old))
        oracle_shift.append(_row_err(want_mx, want))
    eng.status.check()
    ref.expert_act_mx8 = False
    errs, errs_old, between, oracle_shift = (torch.cat(v) for v in (errs, errs_old, between, oracle_shift))
    assert errs_old.median() < 0.11, errs_old
    assert between.median() < 1.5 * oracle_shift.median() + 0.01, (between, oracle_shift)
    # rounding decisions of two noisy paths are independent: the distances add in quadrature
    bound = (errs_old.median() ** 2 + 2 * oracle_shift.median() ** 2) ** 0.5 + 0.02
    assert errs.median() < bound and (errs < 0.2).float().mean() >= 0.6, (errs, bound)
    # a block of 24 rows (deeper drafts, more conversations): the 32-column form of the tensor-core
    # kernel against the register-fed form, with every expert routed so that nothing discrete flips
    cfg24 = small_config(moe_inter=512, topk=8)
    W24 = oracle.init_weights(cfg24, 0)
    new24 = E.Engine.from_weights(cfg24, ecfg, W24)
    old24 = E.Engine.from_weights(cfg24, EngineConfig(reference_matmul=True, regions=2, max_context=512,
                                                      prefill_widths=(128,), moe_block_scaled=False), W24)
    assert "x8" in new24._bufs(24) and "x8" not in old24._bufs(24)
    toks = torch.randint(0, cfg.vocab, (24,), generator=g).tolist()
    outs = []
    for e in (new24, old24):
        e.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
        outs.append(e.forward(E.StepPlan.build([(0, 77, toks)])).cpu())
        e.status.check()
    d24 = _row_err(outs[0], outs[1])
    assert d24.max() < 0.12 and d24.median() < 0.06, d24


def test_index_scoring_in_row_tiles_is_bitwise_the_same():
    """Long contexts bound the fp32 score matrix by scoring and selecting a tile of rows at a time: the
    selections and the logits do not change."""
    cfg = small_config()
    W = oracle.init_weights(cfg, 0)
    mk = lambda nbytes: E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512,
                                                               prefill_widths=(256,), index_score_bytes=nbytes), W)
    whole, tiled = mk(2 << 30), mk(256 << 10)         # 256 KB: tiles of 64 rows of 1,024 scores
    prompt = torch.randint(0, cfg.vocab, (239,), generator=torch.Generator().manual_seed(8)).tolist()
    a = whole.forward(E.StepPlan.build([(0, 0, prompt)]))
    b = tiled.forward(E.StepPlan.build([(0, 0, prompt)]))
    tiled.status.check()
    assert ("scores", 239) in whole._scratch and "scores_flat" in tiled._scratch and ("scores", 239) not in tiled._scratch
    assert tiled._scratch["scores_flat"].numel() == 64 * 1024
    for li in cfg.index_source_layers:
        assert torch.equal(whole._bufs(239)["sel"][li], tiled._bufs(239)["sel"][li])
    assert torch.equal(a, b)


def test_two_regions_batched_decode_equals_separate():
    cfg = small_config()
    W = oracle.init_weights(cfg, 3)
    ecfg = EngineConfig(reference_matmul=True, regions=3, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W)
    g = torch.Generator().manual_seed(2)
    pa, pb = (torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (40, 61))
    eng.forward(E.StepPlan.build([(0, 0, pa)]))
    eng.forward(E.StepPlan.build([(2, 0, pb)]))
    ta, tb = [5, 6, 7, 8], [9, 10, 11, 12]
    both = eng.forward(E.StepPlan.build([(0, 40, ta), (2, 61, tb)])).clone()
    # the same rows again one conversation at a time (positions are overwritten in place)
    a = eng.forward(E.StepPlan.build([(0, 40, ta)])).clone()
    b = eng.forward(E.StepPlan.build([(2, 61, tb)])).clone()
    assert torch.allclose(both[:4], a, atol=2e-3, rtol=1e-3)
    assert torch.allclose(both[4:], b, atol=2e-3, rtol=1e-3)
    eng.status.check()


def test_determinism_run_to_run():
    cfg = small_config()
    ecfg = EngineConfig(reference_matmul=True, regions=1, max_context=256, prefill_widths=(64,))
    eng = E.Engine.from_weights(cfg, ecfg, oracle.init_weights(cfg, 5))
    p = list(range(3, 35))
    a = eng.forward(E.StepPlan.build([(0, 0, p)])).clone()
    b = eng.forward(E.StepPlan.build([(0, 0, p)])).clone()
    assert torch.equal(a, b)


@pytest.mark.parametrize("mx", [True, False])
def test_tensor_core_prefill_path_matches_staging_per_call(mx):
    """Rows beyond the small-M limit run on the tcgen05 GEMMs: block-scaled by the tensor core
    (MXFP8 activations, FP8 weights with UE8M0 scales, MXFP4 experts as stored) or, with
    ``prefill_mx`` off, with fp32 scales promoted in software (experts re-expressed as
    block-scaled FP8 in one grouped launch).  FP8 activations put ~2.6% of noise
    on every GEMM, which this small random model amplifies through its discrete choices (router,
    top-k), so each call is checked against the dequantised-weight PyTorch product on the SAME
    input rather than through the end-to-end logits."""
    from titanic_flash_41_b200.ops import bigpath
    cfg = small_config(moe_inter=256)
    W = oracle.init_weights(cfg, 0)
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=1024, prefill_widths=(512,), prefill_mx=mx)
    eng = E.Engine.from_weights(cfg, ecfg, W)
    bp = bigpath.BigPath(eng)
    errs = []

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-9))

    def dense_checker(e, x16, w, out, M, w3=None):
        o2 = torch.zeros_like(out)
        bp.gemm(e, x16, w, o2, M, w3)
        e.big_gemm = None
        e._linear(x16, w, out, M, w3)            # dequantised weights through torch.matmul
        e.big_gemm = dense_checker
        errs.append(rel(o2[:M, : w.q.shape[0]], out[:M, : w.q.shape[0]]))

    def moe_checker(e, L, T, b):
        e._moe_large(L, T, b)                    # per-expert PyTorch loop on dequantised weights
        shared = None
        if cfg.n_shared:
            e._linear(b["h16"], L.sw1, b["s_act"], T, w3=L.sw3)
            e._linear(b["s_act"], L.sw2, b["s_y"], T)
            shared = b["s_y"]
        from titanic_flash_41_b200.ops import native
        native.call("tf_moe_combine", b["y_pair"], b["ids"], b["wts"], shared, b["delta"], T, cfg.hidden,
                    cfg.topk, 0, cfg.n_experts)
        want = b["delta"][:T].clone()
        bp.moe(e, L, T, b)
        errs.append(rel(b["delta"][:T], want))
        b["delta"][:T].copy_(want)

    eng.big_gemm = dense_checker
    eng.big_moe_full = moe_checker
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (300,), generator=g)
    eng._scratch.clear()
    eng.big_moe_full = None
    b = eng._bufs(300)                           # full-size expert scratch for the staging loop
    eng.big_moe_full = moe_checker
    got = eng.forward(E.StepPlan.build([(0, 0, prompt.tolist())]))
    torch.cuda.synchronize()
    eng.status.check()
    assert len(errs) >= 3 * 5 and max(errs) < 0.06, errs
    assert torch.isfinite(got).all()
    assert (bp._mx_layer is not None) == mx          # the routed experts took the form that was asked for


def test_chunked_prefill_with_late_group_and_spec_decode():
    from titanic_flash_41_b200.ops import bigpath
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.serve.prefill import run_prefill
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    cfg = small_config(n_layers=4, kv_source_layers=(0, 1), index_source_layers=(0, 1, 3), late_start=2,
                       draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=2048, prefill_widths=(256,))
    eng = E.Engine.from_weights(cfg, ecfg, W)
    bigpath.attach(eng)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g, dtype=torch.int32) for n in (700, 333)]
    slots = []
    for r, p in enumerate(prompts):
        lg = run_prefill(eng, r, p, 256)
        assert lg.shape == (1, cfg.vocab) and torch.isfinite(lg).all()
        slots.append(DecodeSlot(region=r, length=int(p.numel()), anchor=int(lg.argmax()), seed=r + 1))
    dec = SpecDecoder(eng, 2, temperature=0.6, top_p=0.95, use_graph=True)
    n0 = [s.length for s in slots]
    for _ in range(6):
        out = dec.step(slots)
        assert all(1 <= len(o) <= 4 for o in out)
    eng.status.check()
    assert all(s.length - a == len(s.emitted) for s, a in zip(slots, n0))
    assert all(0 <= t < cfg.vocab for s in slots for t in s.emitted)
    # graph replay and eager execution of the same step agree
    dec2 = SpecDecoder(eng, 2, temperature=0.6, top_p=0.95, use_graph=False)
    snap = [(s.length, s.anchor) for s in slots]
    a = dec.step([DecodeSlot(region=i, length=l, anchor=t, seed=9) for i, (l, t) in enumerate(snap)])
    b = dec2.step([DecodeSlot(region=i, length=l, anchor=t, seed=9) for i, (l, t) in enumerate(snap)])
    assert [x[0] for x in a] == [x[0] for x in b]


def test_layer_major_prefill_matches_chunk_major():
    """Sweeping the encoder layer by layer over all chunks (experts converted once per layer) must
    give the same logits and the same cached state as the chunk-by-chunk order."""
    from titanic_flash_41_b200.ops import bigpath
    from titanic_flash_41_b200.serve.prefill import run_prefill
    cfg = small_config(n_layers=4, kv_source_layers=(0, 1), index_source_layers=(0, 1, 3), late_start=2)
    W = oracle.init_weights(cfg, 0)
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=2048, prefill_widths=(256,)), W)
    bigpath.attach(eng)
    g = torch.Generator().manual_seed(5)
    p = torch.randint(0, cfg.vocab, (900,), generator=g, dtype=torch.int32)
    a = run_prefill(eng, 0, p, 256, layer_major=False)
    b = run_prefill(eng, 1, p, 256, layer_major=True)
    torch.cuda.synchronize()
    eng.status.check()
    assert int(a.argmax()) == int(b.argmax())
    assert float((a - b).abs().max() / a.abs().max()) < 2e-2
    for li in range(len(eng.layers)):
        w = eng.win[li]
        same = (w[0] == w[1]).float().mean()
        assert same > 0.98, (li, float(same))


@pytest.mark.parametrize("geom", ["lora_q", "grouped_wo", "hc", "all"])
def test_reference_geometry_matches_oracle(geom):
    """Low-rank query, grouped low-rank output projection and the multi-copy residual (mHC) — the
    geometry of the reference model proper — on the CUDA engine against the fp32 oracle."""
    over = {}
    if geom in ("lora_q", "all"):
        over.update(q_lora_rank=128)
    if geom in ("grouped_wo", "all"):
        over.update(o_groups=2, o_lora_rank=128)
    if geom in ("hc", "all"):
        over.update(hc_mult=4)
    cfg = small_config(**over)
    W = oracle.init_weights(cfg, 0)
    if cfg.hc_mult > 1:                       # make the mixing coefficients row-dependent
        g0 = torch.Generator().manual_seed(9)
        for k in W:
            if k.endswith("_base") and "hc_" in k:
                W[k] = torch.randn(W[k].shape, generator=g0) * 0.3
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (61,), generator=g)
    s = ref.new_session(256)
    want = ref.forward(prompt, s)
    got = eng.forward(E.StepPlan.build([(1, 0, prompt.tolist())])).cpu()
    eng.status.check()
    err = _row_err(got, want)
    # rows whose router decision flips on a near-tie differ a lot; assess the rows statistically
    med, lim, frac = (0.15, 0.25, 0.55) if cfg.hc_mult > 1 else (0.1, 0.2, 0.7)   # bf16 residual copies feed the mix
    assert err.median() < med and (err < lim).float().mean() >= frac, err
    pos, errs = 61, []
    for step in range(8):
        toks = torch.randint(0, cfg.vocab, (4,), generator=g)
        want = ref.forward(toks, s)
        got = eng.forward(E.StepPlan.build([(1, pos, toks.tolist())])).cpu()
        pos += 4
        errs.append(_row_err(got, want))
    eng.status.check()
    errs = torch.cat(errs)
    assert errs.median() < med and (errs < lim).float().mean() >= frac, errs


@pytest.mark.parametrize("hc", [1, 4])
def test_engram_layers_match_oracle(hc):
    """Hashed n-gram memory in the engine's layer loop (table lookup, projection, gate) against the oracle."""
    from titanic_flash_41_b200.config import EngramConfig
    cfg = small_config(engram=EngramConfig(layers=(0, 2), rows_per_table=1500), hc_mult=hc)
    W = oracle.init_weights(cfg, 0)
    rt = {}
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,)), W, roundtrip=rt)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(3, cfg.vocab, (50,), generator=g)
    s = ref.new_session(256)
    want = ref.forward(prompt, s)
    got = eng.forward(E.StepPlan.build([(1, 0, prompt.tolist())]).attach_engram(cfg, [[]])).cpu()
    eng.status.check()
    err = _row_err(got, want)
    med, lim, frac = (0.15, 0.25, 0.55) if cfg.hc_mult > 1 else (0.1, 0.2, 0.7)   # bf16 residual copies feed the mix
    assert err.median() < med and (err < lim).float().mean() >= frac, err
    hist, pos, errs = prompt.tolist(), 50, []
    for step in range(6):
        toks = torch.randint(3, cfg.vocab, (4,), generator=g)
        want = ref.forward(toks, s)
        got = eng.forward(E.StepPlan.build([(1, pos, toks.tolist())]).attach_engram(cfg, [hist[-3:]])).cpu()
        hist += toks.tolist()
        pos += 4
        errs.append(_row_err(got, want))
    eng.status.check()
    errs = torch.cat(errs)
    assert errs.median() < med and (errs < lim).float().mean() >= frac, errs
    # a plan without hashes is refused for this model
    with pytest.raises(ValueError, match="attach_engram"):
        eng.forward(E.StepPlan.build([(1, pos, [5, 6])]))


def test_engram_ids_hashed_on_the_device_equal_the_host_hashes():
    """Two conversations in one launch, one at its start (blocked orders), one mid-stream: the ids
    written by tf_engram_hash equal HashHistory's, and the logits equal those of host-hashed plans
    bit for bit; a speculative decoder on an Engram model commits the same tokens on both paths."""
    from titanic_flash_41_b200.config import DraftConfig, EngramConfig
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    cfg = small_config(engram=EngramConfig(layers=(0, 2), rows_per_table=1500), draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,)), W)
    g = torch.Generator().manual_seed(4)
    a = torch.randint(3, cfg.vocab, (9,), generator=g).tolist()
    hist = torch.randint(3, cfg.vocab, (40,), generator=g).tolist()
    eng.forward(E.StepPlan.build([(1, 0, hist)]).attach_recent(cfg, [[]]))
    bt = torch.randint(3, cfg.vocab, (9,), generator=g).tolist()
    blocks = [(0, 0, a), (1, 40, bt)]
    prevs = [[], hist[-3:]]
    host = E.StepPlan.build(blocks).attach_engram(cfg, prevs)
    want = eng.forward(host).clone()
    dev_plan = E.StepPlan.build(blocks).attach_recent(cfg, prevs)
    got = eng.forward(dev_plan).clone()
    eng.status.check()
    ids = eng._bufs(18)["eg_ids"][:, :18].cpu()                      # [tables, T, ids]
    assert torch.equal(ids, torch.from_numpy(host.engram_ids.transpose(1, 0, 2).copy()))
    assert torch.equal(got, want)
    with pytest.raises(ValueError, match="attach_recent"):
        eng.forward(E.StepPlan.build([(1, 49, [5, 6])]))
    # speculative decoding: proposals are sampled inside the graph, so only the device can hash them
    toks = {}
    for use_graph in (True, False):
        eng.forward(E.StepPlan.build([(1, 0, hist)]).attach_recent(cfg, [[]]))
        dec = SpecDecoder(eng, 1, temperature=0.6, top_p=0.95, use_graph=use_graph)
        slots = [DecodeSlot(region=1, length=40, anchor=7, seed=3, recent=hist[-3:])]
        toks[use_graph] = [t for _ in range(5) for t in dec.step(slots)[0]]
        eng.status.check()
        assert slots[0].recent == (hist + toks[use_graph])[-3:]
    assert toks[True] == toks[False]


def test_two_level_candidates_in_the_layer_loop():
    """Long decode rows: the candidate source layer publishes its best blocks of 8 keys and the
    index layer after it selects only among them; short rows and prefill chunks score densely."""
    from titanic_flash_41_b200.ops import two_level as TL
    cfg = small_config(candidate_blocks=4, index_topk=8)
    W = oracle.init_weights(cfg, 0)
    mk = lambda tl: E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(256,),
                                                            two_level_index_min=tl), W)
    eng, dense = mk(16), mk(0)
    assert eng.candidate_source == 0
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (230,), generator=g).tolist()
    calls = []
    orig = TL.consume
    TL.consume = lambda *a, **k: (calls.append(a[3].clone()), orig(*a, **k))[1]
    try:
        a = eng.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
        b = dense.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
        assert not calls and torch.equal(a, b)                     # a prefill chunk never takes the sparse path
        toks = [5, 6, 7, 8]
        a = eng.forward(E.StepPlan.build([(0, 230, toks)])).clone()
        b = dense.forward(E.StepPlan.build([(0, 230, toks)])).clone()
        eng.status.check()
    finally:
        TL.consume = orig
    assert len(calls) == 1                                          # layer 2 consumed what layer 0 published
    cand = calls[0]
    assert cand.shape == (4, 32)
    sel = eng._bufs(4)["sel"][2][:4]
    cnt = eng._bufs(4)["selcnt"][2][:4]
    for r in range(4):
        c = set(cand[r][cand[r] >= 0].tolist())
        picked = sel[r][: int(cnt[r])].tolist()
        assert int(cnt[r]) == min(cfg.index_topk, len(c)) and set(picked) <= c and picked == sorted(picked)
    # the source layer itself selects densely on both engines
    assert torch.equal(eng._bufs(4)["sel"][0][:4], dense._bufs(4)["sel"][0][:4])
    # selecting among 32 candidates instead of all keys is an approximation: with 8 picks per row on
    # this small random model the logits move by a few tenths; the structural checks above are exact
    err = _row_err(a.cpu(), b.cpu())
    assert err.median() < 0.5, err


def test_two_level_selection_inside_the_captured_decode_graph():
    """Contexts long enough for two-level selection decode under a CUDA graph: the replayed graph commits
    what the eager step commits (the candidate tensors are allocated inside the capture)."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    cfg = small_config(candidate_blocks=4, index_topk=8, draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=1024, prefill_widths=(256,),
                                                  two_level_index_min=16), W)
    prompt = torch.randint(0, cfg.vocab, (230,), generator=torch.Generator().manual_seed(6)).tolist()
    outs = []
    for region, graph in ((0, True), (1, False)):
        lg = eng.forward(E.StepPlan.build([(region, 0, prompt)], logits="last"))
        sl = DecodeSlot(region=region, length=230, anchor=int(lg.argmax()), seed=4, temperature=0.0, top_p=1.0)
        dec = SpecDecoder(eng, 1, use_graph=graph)
        dec.hidden.copy_(eng.last_hidden[-1:])
        for _ in range(6):
            dec.step([sl])
        eng.status.check()
        outs.append(list(sl.emitted))
    assert outs[0] == outs[1] and len(outs[0]) >= 6


def test_draft_head_with_markov_correction_matches_oracle():
    """Draft logits = draft head + rank-r bigram term of the token each row was fed."""
    from titanic_flash_41_b200.config import DraftConfig
    cfg = small_config(draft=DraftConfig(layers=1, depth=3, markov_rank=256))
    plain = small_config(draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    assert W["mtp.0.markov_head.head.weight"].shape == (cfg.vocab, 256)
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    base = E.Engine.from_weights(plain, ecfg, {k: v for k, v in W.items() if "markov" not in k})
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (60,), generator=g)
    s = ref.new_session(256)
    ref.forward(prompt, s)
    hid_ref = ref.last_hidden[-1:].clone()
    for e in (eng, base):
        e.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
    hid = eng.last_hidden[-1:].clone()
    toks = torch.tensor([11, 900, 5, 1300])
    want = []
    for t in toks.tolist():                                    # four candidate anchors at position 60
        lg, _ = ref.draft_forward(torch.tensor([t]), hid_ref, s, 60)
        want.append(lg[0])
    want = torch.stack(want)
    got, got_plain = [], []
    for t in toks.tolist():
        for e, out in ((eng, got), (base, got_plain)):
            b = e._bufs(1)
            e.upload_plan(E.StepPlan.build([(0, 60, [t])]), b)
            out.append(e.draft_run(1, b, hid, torch.arange(1, device="cuda"))[0].clone())
    got, got_plain = torch.stack(got).cpu(), torch.stack(got_plain).cpu()
    eng.status.check()
    err = _row_err(got, want)
    assert err.median() < 0.1, err
    # the correction is exactly the bigram term
    bias = (W["mtp.0.markov_head.embed.weight"][toks].bfloat16().float()
            @ W["mtp.0.markov_head.head.weight"].bfloat16().float().t())
    assert (got - got_plain - bias).abs().max() <= 2e-3 * bias.abs().max() + 1e-3
    assert bias.abs().max() > 0.5


@pytest.mark.parametrize("hc", [1, 4])
def test_confidence_head_and_causal_stopping_in_the_decode_graph(hc):
    """The drafter's confidences against the oracle, the device's stopping rule against the host rule
    on the same confidences, never more accepted than verified, and (sharp law) the same text
    whatever the ladder."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    from titanic_flash_41_b200.spec.verify import causal_rows
    # every expert routed: no discrete flips between the engine and the oracle
    mk = lambda ladder: small_config(topk=8, hc_mult=hc, draft=DraftConfig(layers=1, depth=3, markov_rank=256,
                                                                           confidence_head=True, confidence_ladder=ladder))
    cfg = mk((0.15, 0.25, 0.20))
    W = oracle.init_weights(cfg, 0)
    rt = {}
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W, roundtrip=rt)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (60,), generator=g)
    s = ref.new_session(256)
    ref.forward(prompt, s)
    hid_ref = ref.last_hidden[-1:].clone()
    eng.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
    hid = eng.last_hidden[-1:].clone()
    toks = [11, 900, 5, 1300, 77, 1999]
    conf = torch.zeros(1, 3, device="cuda")
    cum, nver = torch.zeros(1, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    ladder = torch.tensor([0.15, 0.25, 0.20], device="cuda")
    want, got = [], []
    for t in toks:
        _, x = ref.draft_forward(torch.tensor([t]), hid_ref, s, 60)
        want.append(float(ref.draft_confidence(torch.tensor([t]), x)[0]))
        b = eng._bufs(1)
        eng.upload_plan(E.StepPlan.build([(0, 60, [t])]), b)
        eng.draft_run(1, b, hid, torch.arange(1, device="cuda"))
        eng.draft_confidence(1, b, 0, 3, ladder, conf, cum, nver)
        got.append(float(conf[0, 0]))
        assert int(nver[0]) == 1 and float(cum[0]) == got[-1]
    eng.status.check()
    want, got = torch.tensor(want), torch.tensor(got)
    assert (want - got).abs().max() < 0.08, (want, got)
    assert want.std() > 0.05                                     # the head is not a constant
    # the decode loop: rule on the device == rule on the host, accepted <= verified
    texts, stopped = [], 0
    for lad in ((0.15, 0.25, 0.20), (0.0,), (2.0,)):
        e = E.Engine.from_weights(mk(lad), ecfg, W)
        lg = e.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
        sl = DecodeSlot(region=0, length=60, anchor=int(lg.argmax()), seed=3, temperature=0.0, top_p=1.0)
        dec = SpecDecoder(e, 1, use_graph=True)
        assert dec.causal
        dec.hidden.copy_(e.last_hidden[-1:])
        while len(sl.emitted) < 20:
            n = len(dec.step([sl])[0])
            assert len(sl.confidence) == 3 and sl.verified == causal_rows(sl.confidence, lad)
            assert n - 1 <= sl.verified
            stopped += sl.verified < 3
        e.status.check()
        texts.append(sl.emitted[:20])
    assert texts[0] == texts[1] == texts[2]
    assert stopped > 0


def test_draft_subset_head_in_four_bits_matches_oracle_and_proposes_subset_tokens():
    """The drafter's vocabulary-subset head: MXFP4 rows x MXFP8 activations on the block-scaled GEMV."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    cfg = small_config(draft=DraftConfig(layers=1, depth=3, subset_rows=1024))
    W = oracle.init_weights(cfg, 0)
    ids = W["mtp.head_subset.ids"]
    assert ids.shape == (1024,) and bool((ids[1:] > ids[:-1]).all())
    rt = {}
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,)), W, roundtrip=rt)
    assert "head_mx" in eng.draft_extra and torch.equal(rt["mtp.head_subset.ids"], ids)
    ref = oracle.OracleModel(cfg, rt)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (60,), generator=g)
    s = ref.new_session(256)
    ref.forward(prompt, s)
    hid_ref = ref.last_hidden[-1:].clone()
    eng.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
    hid = eng.last_hidden[-1:].clone()
    inside = torch.zeros(cfg.vocab, dtype=torch.bool)
    inside[ids] = True
    errs = []
    for t in (11, 900, 5, 1300):
        want, _ = ref.draft_forward(torch.tensor([t]), hid_ref, s, 60)
        b = eng._bufs(1)
        eng.upload_plan(E.StepPlan.build([(0, 60, [t])]), b)
        got = eng.draft_run(1, b, hid, torch.arange(1, device="cuda"))[0].cpu()
        assert bool(torch.isinf(got[~inside]).all()) and bool(torch.isfinite(got[inside]).all())
        assert bool(torch.isinf(want[0][~inside]).all())
        errs.append(float((got[inside] - want[0][inside]).abs().max() / want[0][inside].abs().max()))
    eng.status.check()
    assert sorted(errs)[len(errs) // 2] < 0.1, errs
    # speculative decoding with the subset head: every proposal is a subset token, the committed
    # tokens do not depend on graph capture
    runs = {}
    for use_graph in (True, False):
        eng.forward(E.StepPlan.build([(0, 0, prompt.tolist())], logits="last"))
        dec = SpecDecoder(eng, 1, temperature=0.8, top_p=0.95, use_graph=use_graph)
        slots = [DecodeSlot(region=0, length=60, anchor=7, seed=5)]
        toks = []
        for _ in range(5):
            toks += dec.step(slots)[0]
            assert bool(inside[dec.h_out[2:, 0].long()].all())
        runs[use_graph] = toks
        eng.status.check()
    assert runs[True] == runs[False]


def test_reference_model_widths_run_on_the_engine():
    """The reference model's real widths (hidden 5120, 512-wide latent heads, low-rank query 1280, eight
    output groups of rank 1024, four residual copies, 32 index heads, expert width 2304) with few layers and
    experts: prefill and a decode block produce finite logits and no kernel reports a problem."""
    from titanic_flash_41_b200.config import DraftConfig, reference_1017_config
    cfg = reference_1017_config(n_layers=4, kv_source_layers=(1, 2), compress_ratios=(2, 1), index_source_layers=(1, 2, 3),
                                late_start=3, n_experts=32,
                                draft=DraftConfig(layers=1, depth=3), engram=None, dense_quant="fp8_block128", vocab=16384)
    eng = E.Engine.random_init(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=4096, prefill_widths=(256,)), seed=0, max_chunk=256)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(3, cfg.vocab, (200,), generator=g).tolist()
    lg = eng.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
    torch.cuda.synchronize()
    eng.status.check()
    assert lg.shape == (1, cfg.vocab) and bool(torch.isfinite(lg).all())
    lg = eng.forward(E.StepPlan.build([(0, 200, [5, 6, 7, 8])]))
    torch.cuda.synchronize()
    eng.status.check()
    assert lg.shape == (4, cfg.vocab) and bool(torch.isfinite(lg).all()) and float(lg.std()) > 0


def test_startup_self_check_and_bitwise_determinism_on_the_engine():
    """Two runs of the fixture (prefill + speculative decode under CUDA graphs) in different regions give
    identical tokens, logits and state digests."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.serve.backend import EngineBackend
    from titanic_flash_41_b200.serve.warmup import self_check
    cfg = small_config(draft=DraftConfig(layers=1, depth=3))
    W = oracle.init_weights(cfg, 0)
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(64,)), W)
    rep = self_check(EngineBackend(eng, chunk=64), steps=4)
    assert rep["tokens"] >= 5


def test_memory_report_accounts_for_what_the_engine_holds():
    cfg = small_config()
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,)),
                                oracle.init_weights(cfg, 0))
    eng.forward(E.StepPlan.build([(0, 0, [1, 2, 3, 4])]))
    rep = eng.memory_report()
    nb = lambda t: t.untyped_storage().nbytes()
    assert rep["total"] == sum(v for k, v in rep.items() if k != "total")
    assert rep["kv_state"] == sum(nb(t) for t in (eng.win, eng.comp, eng.keys, eng.carry))
    assert rep["expert_weights"] == sum(nb(getattr(L, f)) for L in eng.layers + eng.draft_layers
                                        for f in ("ew1", "ew3", "ew2", "es1", "es3", "es2") if getattr(L, f) is not None)
    assert rep["dense_weights"] > 0 and rep["row_scratch"] > 0 and rep["embeddings_and_heads"] >= nb(eng.embed_w)


def test_graph_clock_times_the_kernels_inside_a_replayed_graph():
    """Device timestamps captured with the decode graph: every replay refreshes them; the per-kernel
    table covers the kernels of the step and adds up to about the span of the step."""
    from titanic_flash_41_b200.config import DraftConfig
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    from titanic_flash_41_b200.utils.trace import GraphClock
    cfg = small_config(draft=DraftConfig(layers=1, depth=3))
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,)),
                                oracle.init_weights(cfg, 0))
    prompt = torch.randint(0, cfg.vocab, (60,), generator=torch.Generator().manual_seed(2)).tolist()
    lg = eng.forward(E.StepPlan.build([(0, 0, prompt)], logits="last"))
    sl = DecodeSlot(region=0, length=60, anchor=int(lg.argmax()), seed=3)
    dec = SpecDecoder(eng, 1, use_graph=True)
    dec.clock = GraphClock()
    dec.hidden.copy_(eng.last_hidden[-1:])
    dec.step([sl])
    first = dec.clock.ring[: 2 * len(dec.clock.marks)].clone()
    dec.step([sl])
    second = dec.clock.ring[: 2 * len(dec.clock.marks)].clone()
    eng.status.check()
    assert len(dec.clock.marks) > 50 and bool((second > first).all())          # the replay wrote new times
    rows = dec.clock.table()
    names = {r[0] for r in rows}
    assert {"tf_sparse_attention", "tf_attn_prep", "tf_sample_chunks"} <= names
    total, span = sum(r[2] for r in rows), dec.clock.span_us()
    assert 0 < span < 1e5 and 0.3 * span <= total <= 1.3 * span, (total, span)   # gaps are not charged; side branches overlap
    assert all(r[2] > 0 for r in rows)
    assert "inside the graph" in dec.clock.report()
