"""Image input planning / patchify (CPU) and the device vision tower against its fp32 oracle (GPU)."""
import io

import numpy as np
import pytest
import torch

from titanic_flash_41_b200.api import vision_input as VI
from titanic_flash_41_b200.config import VisionConfig


def test_plan_token_budget_and_padding():
    p = VI.Plan.new(640, 480)
    assert p.width % 14 == 0 and p.height % 14 == 0 and p.tokens == p.llm_height * (p.llm_width + 1) + 2
    assert p.tokens <= 1024 and p.resize_width <= p.width and p.resize_height <= p.height
    big = VI.Plan.new(8000, 6000)
    assert big.tokens <= 1024 and big.vit_height * big.vit_width <= 9198
    tall = VI.Plan.new(50, 20000)
    assert tall.tokens <= 1024
    small = VI.Plan.new(32, 32)                  # tiny images are scaled up to the minimum area first
    assert small.width * small.height >= 500 * 500
    with pytest.raises(ValueError):
        VI.Plan.new(0, 10)


def test_prepare_patch_layout_and_cache():
    from PIL import Image
    rng = np.random.default_rng(0)
    rgb = rng.integers(0, 256, size=(600, 800, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(rgb).save(buf, format="PNG")
    prep = VI.prepare(buf.getvalue())
    plan = prep.plan
    assert prep.patches.shape == (plan.vit_height * plan.vit_width, 588) and prep.patches.dtype == torch.bfloat16
    assert float(prep.patches.abs().max()) <= 1.0
    # patch (1, 2), channel 1, pixel (3, 4) is canvas pixel (17, 32) of the resized image
    im = np.asarray(Image.fromarray(rgb).resize((plan.resize_width, plan.resize_height), Image.BICUBIC))
    y, x = 14 + 3 - plan.top, 28 + 4 - plan.left
    want = ((im[y, x, 1] / 255.0) - 0.5) / 0.5
    got = float(prep.patches[1 * plan.vit_width + 2, 1 * 196 + 3 * 14 + 4])
    assert abs(got - want) < 0.01
    assert VI.identity(buf.getvalue()) == prep.identity != VI.identity(buf.getvalue(), "high")
    with pytest.raises(ValueError):
        VI.prepare(b"not an image")
    cache = VI.ImageCache(budget_bytes=3 * prep.patches.numel() * 2)
    for i in range(5):
        cache.put(bytes([i]), i, prep.patches.numel() * 2)
    assert cache.get(bytes([0])) is None and cache.get(bytes([4])) == 4 and cache.used <= cache.budget


@pytest.mark.gpu
def test_vision_tower_matches_oracle():
    from titanic_flash_41_b200.models import vision as V
    vc = VisionConfig(layers=2, hidden=256, heads=4, intermediate=384)
    d_model = 512
    W = V.init_vision_weights(vc, d_model, seed=1)
    gh, gw = 7, 10
    g = torch.Generator().manual_seed(2)
    patches = (torch.rand(gh * gw, 588, generator=g) * 2 - 1).bfloat16()
    want = V.VisionOracle(vc, d_model, W).encode(patches.float(), gh, gw)
    got = V.VisionTower(vc, d_model, W).encode(patches, gh, gw).float().cpu()
    assert got.shape == want.shape == (3 * (4 + 1) + 2, d_model)
    rel = float((got - want).norm() / want.norm())
    assert rel < 0.03, rel


def test_media_expansion_and_identity():
    import base64
    from PIL import Image
    from titanic_flash_41_b200.api import media as M
    buf = io.BytesIO()
    Image.fromarray(np.full((600, 600, 3), 200, dtype=np.uint8)).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    cache = VI.ImageCache()
    pm = M.expand([5, 900, 6, 900, 7], [uri, uri], marker_id=900, image_token_id=901, cache=cache)
    n = pm.images[0].plan.tokens
    assert len(pm.tokens) == 3 + 2 * n and pm.tokens[1] == 901 and pm.offsets == [(1, n), (2 + n, n)]
    assert cache.hits == 1 and len(pm.identity) == 64
    assert M.expand([5], [], 900, 901).identity == ""
    for bad in ("http://example.com/x.png", "data:image/png;base64,@@@"):
        with pytest.raises(M.MediaError):
            M.expand([900], [bad], 900, 901)
    with pytest.raises(M.MediaError, match="disagree"):
        M.expand([5], [uri], 900, 901)


@pytest.mark.gpu
def test_prefill_with_image_span_embeddings():
    """Replacing embeddings through ``embeds`` with the tokens' own embeddings is a no-op; other rows change the logits."""
    from tests.test_engine_gpu import small_config
    from titanic_flash_41_b200.config import EngineConfig
    from titanic_flash_41_b200.models import engine as E, oracle
    from titanic_flash_41_b200.serve.prefill import run_prefill
    cfg = small_config()
    W = oracle.init_weights(cfg, 0)
    eng = E.Engine.from_weights(cfg, EngineConfig(reference_matmul=True, regions=2, max_context=512, prefill_widths=(64,)), W)
    p = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(1), dtype=torch.int32)
    base = run_prefill(eng, 0, p, 64)
    offs = torch.arange(70, 90)
    own = eng.embed_w[p[70:90].long().to(eng.dev)]
    same = run_prefill(eng, 1, p, 64, embeds=(offs, own))
    assert torch.equal(base, same)
    other = run_prefill(eng, 1, p, 64, embeds=(offs, own.flip(0)))
    assert not torch.equal(base, other) and torch.isfinite(other).all()
