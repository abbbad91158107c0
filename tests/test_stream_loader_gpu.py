"""Streamed loading of a checkpoint in its stored formats (models/stream_loader.py) against the
dequantise-and-requantise path: identical device weights for block-128 FP8 + MXFP4 checkpoints, a
bounded host footprint, digests, and the 32x32-UE8M0 dense format re-expressed on the device."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(**over):
    from tests.test_engine_gpu import small_config
    from titanic_flash_41_b200.config import DraftConfig
    kw = dict(draft=DraftConfig(layers=1, depth=3, markov_rank=128), n_layers=3)
    kw.update(over)
    return small_config(**kw)


def test_streamed_engine_equals_the_dequantising_loader(tmp_path):
    from titanic_flash_41_b200.config import EngineConfig
    from titanic_flash_41_b200.formats.safetensors import Checkpoint
    from titanic_flash_41_b200.models import engine as E, loader, oracle, stream_loader
    cfg = _cfg()
    W = oracle.init_weights(cfg, 2)
    loader.export_checkpoint(W, cfg, str(tmp_path), shard_bytes=1 << 22)
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    ck = Checkpoint.scan(str(tmp_path))
    # this checkpoint's block scales are amax / 448 (not powers of two): re-quantise by the same rule
    E.POW2_SCALES = False
    try:
        a = E.Engine.from_weights(cfg, ecfg, loader.checkpoint_weights(ck, cfg))
    finally:
        E.POW2_SCALES = True
    b = stream_loader.load_engine(str(tmp_path), cfg, ecfg)
    for la, lb in zip(a.layers + a.draft_layers, b.layers + b.draft_layers):
        assert la.offs == lb.offs
        for nm in ("proj", "wo", "sw1", "sw3", "sw2"):
            # the streamed engine holds the checkpoint's own bytes; the other path re-quantises what it
            # dequantised, which reproduces them up to the rounding of (448 * s) / 448
            wa, wb = getattr(la, nm), getattr(lb, nm)
            da, db = E.dequant_fp8(wa), E.dequant_fp8(wb)
            assert da.shape == db.shape, nm
            # (the re-derived block scale fl(fl(448 s) / 448) can sit one ulp from s)
            assert torch.allclose(da, db, rtol=1e-6, atol=0), nm
        for nm in ("ew1", "ew3", "ew2", "es1", "es3", "es2", "gate", "attn_norm", "kv_norm"):
            ta, tb = getattr(la, nm), getattr(lb, nm)
            if nm.startswith("e"):
                # FP4 group scales may renormalise on re-quantisation; the decoded values may not move
                continue
            assert torch.equal(ta, tb), nm
        for nm in ("w1", "w3", "w2"):
            da = E.dequant_mxfp4(getattr(la, "e" + nm), getattr(la, "es" + nm[1]))
            db = E.dequant_mxfp4(getattr(lb, "e" + nm), getattr(lb, "es" + nm[1]))
            assert torch.equal(da, db), nm
    assert torch.equal(a.embed_w, b.embed_w) and torch.equal(a.head_w, b.head_w)
    assert torch.equal(a.draft_extra["markov_head"], b.draft_extra["markov_head"])
    toks = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    la = a.forward(E.StepPlan.build([(0, 0, toks)]))
    lb = b.forward(E.StepPlan.build([(0, 0, toks)]))
    rel = (la - lb).abs().amax(-1) / la.abs().amax(-1)
    assert float(rel.median()) < 0.02, rel
    # and the streamed weights ARE the stored bytes
    raw = ck.read("layers.0.attn.wkv.weight").view(torch.uint8)
    o = b.layers[0].offs["kv"]
    assert torch.equal(b.layers[0].proj.q[o:o + raw.shape[0]].view(torch.uint8).cpu(), raw)
    # the host never held more than about one layer, and every loaded tensor has its digest on record
    rep = b.load_report
    total = sum(t.nbytes for t in ck.tensors.values())
    assert rep["peak_host_bytes"] < total / 2 and rep["tensors"] > 50
    assert all(len(h) == 64 for h in rep["sha256"].values())
    # an expert scale byte above the kernels' headroom is refused
    name = "layers.0.ffn.experts.0.w1.scale"
    t = ck.tensors[name]
    with open(t.file, "r+b") as f:
        f.seek(t.begin)
        f.write(bytes([250]))
    from titanic_flash_41_b200.formats.safetensors import CheckpointError
    with pytest.raises(CheckpointError, match="247"):
        stream_loader.load_engine(str(tmp_path), cfg, ecfg)


def test_ue8m0_32_dense_scales_are_reexpressed_on_the_device(tmp_path):
    """The reference's dense format (e4m3 + one UE8M0 scale per 32x32): logits of the streamed engine
    agree with the engine built from the dequantised checkpoint within the quantisation noise."""
    from titanic_flash_41_b200.config import EngineConfig
    from titanic_flash_41_b200.formats.safetensors import Checkpoint
    from titanic_flash_41_b200.models import engine as E, loader, oracle, stream_loader
    cfg = _cfg(dense_quant="fp8_ue8m0_32")
    W = oracle.init_weights(cfg, 4)
    loader.export_checkpoint(W, cfg, str(tmp_path), shard_bytes=1 << 22)
    ecfg = EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(128,))
    ck = Checkpoint.scan(str(tmp_path))
    Wd = loader.checkpoint_weights(ck, cfg)
    b = stream_loader.load_engine(str(tmp_path), cfg, ecfg)
    # the re-expressed matrix decodes to (almost) the stored values
    got = E.dequant_fp8(b.layers[0].wo)
    want = Wd["layers.0.attn.wo.weight"].to(got.device)
    assert float((got - want).abs().max()) <= 0.07 * float(want.abs().max())
    assert float((got - want).abs().mean()) <= 0.01 * float(want.abs().mean()) + 1e-6
    a = E.Engine.from_weights(cfg, ecfg, Wd)
    toks = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    la = a.forward(E.StepPlan.build([(0, 0, toks)]))
    lb = b.forward(E.StepPlan.build([(0, 0, toks)]))
    rel = (la - lb).abs().amax(-1) / la.abs().amax(-1)          # a near-tie in the router can flip an expert of a row
    assert float(rel.median()) < 0.3, rel
