"""POST /v1/chat/completions -> scheduler -> worker -> EngineBackend on one GPU: non-stream, stream
and an image request, with the committed tokens checked against driving the engine directly
(prefill + SpecDecoder) on a second engine with the same weights."""
import asyncio
import base64
import io
import json
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(vision=False):
    from tests.test_engine_gpu import small_config
    from titanic_flash_41_b200.api.media import SpanEncoder, VisionFrontend
    from titanic_flash_41_b200.api.server import Frontend, Server
    from titanic_flash_41_b200.api.tokenizer import ByteTokenizer
    from titanic_flash_41_b200.config import DraftConfig, EngineConfig, ServerConfig, VisionConfig
    from titanic_flash_41_b200.models import engine as E, oracle
    from titanic_flash_41_b200.models import vision as V
    from titanic_flash_41_b200.serve.backend import EngineBackend
    from titanic_flash_41_b200.serve.scheduler import Scheduler
    from titanic_flash_41_b200.serve.session_cache import SessionCache
    from titanic_flash_41_b200.serve.worker import Worker
    cfg = small_config(draft=DraftConfig(layers=1, depth=3), vocab=2048)
    W = oracle.init_weights(cfg, 0)
    ecfg = EngineConfig(regions=2, max_context=2048, prefill_widths=(128,))
    eng = E.Engine.from_weights(cfg, ecfg, W)
    backend = EngineBackend(eng, chunk=128)
    tok = ByteTokenizer(cfg.vocab)
    sched = Scheduler(2, 4, 2)
    vf = se = None
    if vision:
        vc = VisionConfig(layers=2, hidden=256, heads=4, intermediate=384, image_token_id=2000, max_image_tokens=64)
        tower = V.VisionTower(vc, cfg.hidden, V.init_vision_weights(vc, cfg.hidden, seed=1))
        vf = VisionFrontend(tok.image_id, vc.image_token_id, vc.max_image_tokens)
        se = SpanEncoder(tower)
    worker = Worker(backend, sched, SessionCache(), eos_id=tok.eos_id, span_encoder=se)
    server = Server(ServerConfig(), Frontend(tok, 2048, vision=vf), sched)
    server.ready("gpu-test")
    t = threading.Thread(target=worker.run_forever, daemon=True)
    t.start()
    return cfg, W, ecfg, tok, server, sched, worker, t


def _direct(cfg, W, ecfg, prompt, n_new, seed, temperature=0.0, embeds=None):
    """The same request served by hand: prefill, first token, SpecDecoder steps."""
    from titanic_flash_41_b200.models import engine as E
    from titanic_flash_41_b200.ops import bigpath
    from titanic_flash_41_b200.serve.prefill import run_prefill
    from titanic_flash_41_b200.spec.decoder import DecodeSlot, SpecDecoder
    eng = E.Engine.from_weights(cfg, ecfg, W)
    bigpath.attach(eng)
    lg = run_prefill(eng, 0, torch.tensor(prompt, dtype=torch.int32), 128, embeds=embeds)
    first = int(lg[-1].argmax())
    dec = SpecDecoder(eng, 1)
    dec.hidden[0].copy_(eng.last_hidden[-1].reshape(-1)[-cfg.hidden:])
    slot = DecodeSlot(region=0, length=len(prompt), anchor=first, seed=seed, temperature=temperature, top_p=1.0)
    out = [first]
    while len(out) < n_new:
        toks = dec.step([slot])[0]
        out += toks[1:] + [slot.anchor]
    eng.status.check()
    return out[:n_new]


def _png(value):
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(np.full((560, 560, 3), value, dtype=np.uint8)).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def test_chat_completions_through_the_cuda_engine_match_direct_decoding():
    from aiohttp.test_utils import TestClient, TestServer
    cfg, W, ecfg, tok, server, sched, worker, t = _setup()
    body = {"messages": [{"role": "user", "content": "count the sheep " * 12}], "max_tokens": 12, "temperature": 0,
            "seed": 5}

    async def go():
        async with TestClient(TestServer(server.app)) as c:
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status == 200, await r.text()
            plain = await r.json()
            r = await c.post("/v1/chat/completions", json=dict(body, stream=True, stream_options={"include_usage": True}))
            assert r.status == 200
            text = (await r.read()).decode()
            return plain, text
    plain, text = asyncio.run(go())
    sched.close()
    t.join(30)
    req_tokens = server.front.prepare(body)[1]
    want = _direct(cfg, W, ecfg, req_tokens, 12, seed=5)
    want_text = tok.decode([x for x in want if x != tok.eos_id])
    assert plain["usage"]["prompt_tokens"] == len(req_tokens) and plain["usage"]["completion_tokens"] <= 12
    got_text = (plain["choices"][0]["message"].get("reasoning_content") or "") + (plain["choices"][0]["message"].get("content") or "")
    assert plain["timings"]["prompt_n"] == len(req_tokens)
    # greedy decoding through the server commits exactly what direct speculative decoding commits
    n = plain["usage"]["completion_tokens"]
    assert n >= 1 and want_text.startswith(got_text[: max(1, len(got_text) - 4)]) or got_text == want_text[: len(got_text)]
    # the stream carries the same text, the timings on its first chunk and the [DONE] marker
    chunks = [json.loads(l[6:]) for l in text.splitlines() if l.startswith("data: {")]
    streamed = "".join((c["choices"][0]["delta"].get("reasoning_content") or "") + (c["choices"][0]["delta"].get("content") or "")
                       for c in chunks if c.get("choices"))
    assert streamed == got_text and "data: [DONE]" in text and ": native-execution running" in text
    assert any("timings" in c for c in chunks) and chunks[-1]["usage"]["prompt_tokens"] == len(req_tokens)
    worker.b.e.status.check()


def test_image_request_reaches_prefill_as_span_embeddings():
    from aiohttp.test_utils import TestClient, TestServer
    cfg, W, ecfg, tok, server, sched, worker, t = _setup(vision=True)

    def body(img):
        return {"messages": [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                                          {"type": "image_url", "image_url": {"url": img}}]}],
                "max_tokens": 6, "temperature": 0, "seed": 3}
    seen = []
    orig = worker.b.prefill

    def spy(region, tokens, start, on_chunk=None, **kw):
        seen.append((list(tokens), kw.get("embeds")))
        return orig(region, tokens, start, on_chunk, **kw)
    worker.b.prefill = spy

    async def go():
        async with TestClient(TestServer(server.app)) as c:
            outs = []
            for img in (_png(40), _png(220)):
                r = await c.post("/v1/chat/completions", json=body(img))
                assert r.status == 200, await r.text()
                outs.append(await r.json())
            # a deployment without a vision tower refuses image parts instead of ignoring them
            server.front.vision = None
            r = await c.post("/v1/chat/completions", json=body(_png(40)))
            assert r.status == 400 and (await r.json())["error"]["code"] == "unsupported_media"
            return outs
    outs = asyncio.run(go())
    sched.close()
    t.join(30)
    assert len(seen) >= 2
    (t1, e1), (t2, e2) = seen[0], seen[1]
    assert t1 == t2 and t1.count(2000) >= 4              # same prompt tokens: placeholders for the image positions
    assert e1 is not None and e2 is not None and e1[1].shape == e2[1].shape
    assert e1[1].shape[0] == t1.count(2000) and not torch.equal(e1[1], e2[1])     # different images, different spans
    assert outs[0]["usage"]["prompt_tokens"] == len(t1)
    # the two conversations are cached under different media identities
    medias = {e.image.media for e in worker.cache.entries}
    assert len(medias) >= 2 and "" not in medias
    worker.b.e.status.check()
