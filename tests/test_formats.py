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


def test_reference_tensor_names_validate_and_shard(tmp_path):
    """A header-only checkpoint with the reference's names for the parts that have their own naming
    rules (src/layout.rs:86, :275-292, :362): the Markov head of the LAST draft stage, the Engram
    row store as MXFP8 weight + scale, the image-token selection bias.  It must validate, and the
    rank plan must split vocabulary rows / Engram rows while the Markov latents stay whole."""
    from titanic_flash_41_b200.config import DraftConfig, EngramConfig
    cfg = tiny_config(n_layers=2, hidden=256, n_experts=4, moe_inter=128, shared_inter=256, vocab=512,
                      dense_quant="fp8_ue8m0_32", expert_quant="mxfp4", router_bias=True, router_bias_vl=True,
                      image_token=500, draft=DraftConfig(layers=3, depth=3, markov_rank=32),
                      engram=EngramConfig(layers=(1,), tables=1, rows_per_table=40))
    names = {n: (dt, sh) for n, dt, sh in layout.expected_tensors(cfg)}
    for want in ("mtp.2.markov_head.embed.weight", "mtp.2.markov_head.head.weight", "layers.1.engram.embed.weight",
                 "layers.1.engram.embed.scale", "layers.1.engram.wkv.weight", "layers.1.engram.wkv.scale",
                 "layers.1.engram.q_weight", "layers.0.ffn.gate.bias_vl", "layers.1.ffn.gate.bias_vl"):
        assert want in names, want
    assert "mtp.markov_head.head.weight" not in names and "mtp.0.ffn.gate.bias_vl" not in names
    assert names["layers.1.engram.embed.weight"][0] == "F8_E4M3" and names["layers.1.engram.embed.weight"][1][1] == 256
    assert names["layers.1.engram.embed.scale"] == ("F8_E8M0", (names["layers.1.engram.embed.weight"][1][0], 8))
    assert names["layers.0.attn.wkv.scale"][0] == "F8_E8M0"              # 32 x 32 UE8M0 dense scales
    # header-only file: every tensor of the contract with its dtype and shape, zero-filled payload
    header, off = {}, 0
    esize = {"BF16": 2, "F32": 4, "F8_E4M3": 1, "F8_E8M0": 1, "I8": 1, "I64": 8}
    for n, (dt, sh) in names.items():
        nb = esize[dt]
        for v in sh:
            nb *= v
        header[n] = {"dtype": dt, "shape": list(sh), "data_offsets": [off, off + nb]}
        off += nb
    hb = json.dumps(header).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(os.path.join(str(tmp_path), "model-00001.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hb)) + hb)
        f.truncate(8 + len(hb) + off)
    ck = Checkpoint.scan(str(tmp_path))
    layout.validate_checkpoint(ck, cfg)
    plan = layout.RankPlan.build(ck, cfg, 1, 2, "ep").entries
    head = plan["mtp.2.markov_head.head.weight"]
    assert (head.kind, head.axis, head.start, head.length) == ("shard", 0, 256, 256)
    assert plan["mtp.2.markov_head.embed.weight"].kind == "replicated"
    rows = names["layers.1.engram.embed.weight"][1][0]
    eg = plan["layers.1.engram.embed.weight"]
    assert eg.kind == "shard" and eg.start == rows // 2 and eg.start + eg.length == rows
    assert plan["layers.1.engram.embed.scale"].start == eg.start
    assert plan["layers.1.engram.wkv.weight"].kind == "shard" and plan["layers.0.ffn.gate.bias_vl"].kind == "replicated"
    # a checkpoint with the unqualified name is refused
    header["mtp.markov_head.head.weight"] = header.pop("mtp.2.markov_head.head.weight")
    os.remove(os.path.join(str(tmp_path), "model-00001.safetensors"))
    hb = json.dumps(header).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(os.path.join(str(tmp_path), "model-00001.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hb)) + hb)
        f.truncate(8 + len(hb) + off)
    with pytest.raises(CheckpointError):
        layout.validate_checkpoint(Checkpoint.scan(str(tmp_path)), cfg)


def test_image_rows_select_experts_with_the_vl_bias():
    from titanic_flash_41_b200.models import oracle
    cfg = tiny_config(router_bias=True, router_bias_vl=True, image_token=7, scoring="sqrtsoftplus")
    logits = torch.randn(5, cfg.n_experts)
    bias = torch.zeros(cfg.n_experts)
    bias_vl = torch.zeros(cfg.n_experts)
    bias_vl[3] = 100.0                                             # image rows must pick expert 3 first
    img = torch.tensor([False, True, False, True, False])
    ids, wts = oracle.route(logits, cfg, bias, bias_vl, img)
    plain, wplain = oracle.route(logits, cfg, bias)
    assert ids[1, 0] == 3 and ids[3, 0] == 3
    assert torch.equal(ids[[0, 2, 4]], plain[[0, 2, 4]]) and torch.equal(wts[[0, 2, 4]], wplain[[0, 2, 4]])
    # weights stay the UNBIASED scores of the winners
    sp = torch.sqrt(torch.log1p(torch.exp(logits[1])))
    assert torch.allclose(wts[1] / wts[1].sum(), sp[ids[1]] / sp[ids[1]].sum(), atol=1e-6)
