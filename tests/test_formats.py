"""Codecs, safetensors scan, rank plan and staged atlas."""
import json
import os
import struct

import pytest
import torch

from titanic_flash_41_b200.config import ModelConfig, tiny_config
from titanic_flash_41_b200.formats import atlas, codecs, layout
from titanic_flash_41_b200.formats.safetensors import Checkpoint, CheckpointError, write_safetensors


def test_codecs_round_trip_and_row_sizes():
    x = torch.randn(7, 512)
    q, s = codecs.mxfp8_quant(x)
    assert (codecs.mxfp8_dequant(q, s) - x).abs().max() < 0.07 * x.abs().max()
    assert codecs.kv_v41_encode(x).shape[-1] == 528 and codecs.kv_v41fp4_encode(x).shape[-1] == 288
    assert codecs.index_key_encode(torch.randn(3, 128)).shape[-1] == 68
    assert (codecs.kv_v41_decode(codecs.kv_v41_encode(x), 512) - x).abs().max() < 0.1 * x.abs().max()
    p, sc = codecs.mxfp4_quant(x)
    assert p.shape == (7, 256) and sc.shape == (7, 16) and int(sc.max()) <= 247
    assert (codecs.mxfp4_dequant(p, sc) - x).abs().mean() < 0.15 * x.abs().mean() + 0.05
    assert torch.equal(codecs.ue8m0_decode(torch.tensor([127, 128, 0], dtype=torch.uint8))[:2], torch.tensor([1.0, 2.0]))
    assert torch.isnan(codecs.ue8m0_decode(torch.tensor([255], dtype=torch.uint8)))[0]
    w = torch.randn(200, 256)
    for ue in (False, True):
        qq, ss = codecs.fp8_block_quant(w, 128 if not ue else 32, ue)
        assert (codecs.fp8_block_dequant(qq, ss, 128 if not ue else 32) - w).abs().max() < 0.08 * w.abs().max()
    assert ModelConfig.from_json(tiny_config().to_json()).digest() == tiny_config().digest()


def _ckpt(tmp_path, cfg):
    names = {n: (dt, sh) for n, dt, sh in layout.expected_tensors(cfg)}
    tensors, dnames = {}, {}
    g = torch.Generator().manual_seed(0)
    for n, (dt, sh) in names.items():
        if dt == "BF16":
            tensors[n] = torch.randn(*sh, generator=g).bfloat16()
        elif dt == "F32":
            tensors[n] = torch.randn(*sh, generator=g)
        elif dt == "F8_E4M3":
            tensors[n] = torch.randn(*sh, generator=g).to(torch.float8_e4m3fn)
        else:
            tensors[n] = torch.randint(100, 130, sh, generator=g, dtype=torch.uint8)
            dnames[n] = dt
    write_safetensors(os.path.join(tmp_path, "model-00001.safetensors"), tensors, dnames)
    return tensors


def test_scan_plan_stage_and_load(tmp_path):
    cfg = tiny_config(n_layers=1, hidden=256, n_experts=4, moe_inter=128, shared_inter=256, vocab=512,
                      dense_quant="fp8_block128", expert_quant="mxfp4")
    tensors = _ckpt(str(tmp_path), cfg)
    ck = Checkpoint.scan(str(tmp_path))
    layout.validate_checkpoint(ck, cfg)
    with pytest.raises(CheckpointError):
        ck.require("embed.weight", "BF16", (1, 1))
    plans = [layout.RankPlan.build(ck, cfg, r, 2, "ep") for r in range(2)]
    p0 = plans[0].entries
    assert p0["embed.weight"].kind == "shard" and p0["embed.weight"].length == 256
    assert p0["layers.0.attn.wo.weight"].axis == 1 and p0["layers.0.attn.wkv.weight"].kind == "replicated"
    assert p0["layers.0.ffn.experts.0.w1.weight"].kind == "expert_local"
    assert p0["layers.0.ffn.experts.3.w1.weight"].kind == "expert_remote"
    tp = layout.RankPlan.build(ck, cfg, 1, 2, "tp").entries
    assert tp["layers.0.ffn.experts.3.w2.weight"].axis == 1
    assert sum(pl.local_bytes(ck) for pl in plans) > sum(t.nbytes for t in ck.tensors.values())   # replication
    out = os.path.join(str(tmp_path), "rank0")
    meta = atlas.stage(ck, cfg, plans[0], out)
    assert all(e["offset"] % 256 == 0 for e in meta["tensors"])
    loaded = atlas.load_staged(out, cfg)
    assert torch.equal(loaded["embed.weight"], tensors["embed.weight"][:256])
    assert torch.equal(loaded["layers.0.attn.wo.weight"].view(torch.uint8),
                       tensors["layers.0.attn.wo.weight"][:, :128].contiguous().view(torch.uint8))
    assert "layers.0.ffn.experts.3.w1.weight" not in loaded
    assert atlas.device_digest(loaded) == atlas.device_digest(atlas.load_staged(out))
    # a flipped byte is caught by the per-tensor digest
    path = os.path.join(out, "atlas.bin")
    raw = bytearray(open(path, "rb").read())
    raw[meta["tensors"][3]["offset"]] ^= 1
    open(path, "wb").write(bytes(raw))
    with pytest.raises(CheckpointError, match="digest mismatch"):
        atlas.load_staged(out, cfg)


def test_scan_rejects_holes_and_traversal(tmp_path):
    p = os.path.join(str(tmp_path), "a.safetensors")
    head = json.dumps({"x": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(head)) + head + b"\0" * 12)
    with pytest.raises(CheckpointError, match="hole"):
        Checkpoint.scan(str(tmp_path))
    os.remove(p)
    json.dump({"weight_map": {"x": "../evil.safetensors"}}, open(os.path.join(str(tmp_path), "model.safetensors.index.json"), "w"))
    with pytest.raises(CheckpointError, match="escapes"):
        Checkpoint.scan(str(tmp_path))


def test_export_and_reload_matches_oracle_weights(tmp_path):
    from titanic_flash_41_b200.models import loader, oracle
    cfg = tiny_config(dense_quant="fp8_block128", expert_quant="mxfp4")
    W = oracle.init_weights(cfg, seed=3)
    n = loader.export_checkpoint(W, cfg, str(tmp_path), shard_bytes=1 << 20)
    assert n > 1
    ck = Checkpoint.scan(str(tmp_path))
    W2 = loader.checkpoint_weights(ck, cfg)
    assert set(W2) >= {k for k in W if not k.startswith("hc_")}
    for k in ("embed.weight", "layers.0.attn.wq.weight", "layers.1.ffn.experts.w2.weight", "layers.0.ffn.gate.bias"):
        a, b = W[k].float(), W2[k]
        assert a.shape == b.shape and (a - b).abs().max() <= 0.3 * a.abs().max(), k
    # a second export of the reloaded weights reproduces the same bytes: quantisation is idempotent in value
    d2 = os.path.join(str(tmp_path), "again")
    loader.export_checkpoint(W2, cfg, d2, shard_bytes=1 << 20)
    ck2 = Checkpoint.scan(d2)
    for k in ("layers.0.attn.wq.weight", "layers.0.attn.wq.scale"):
        assert torch.equal(ck.read(k).view(torch.uint8), ck2.read(k).view(torch.uint8)), k
    W3 = loader.checkpoint_weights(ck2, cfg)        # FP4 group scales may renormalise; the values may not move
    assert torch.equal(W3["layers.1.ffn.experts.w1.weight"], W2["layers.1.ffn.experts.w1.weight"])
