"""Images of a chat request: from data URIs to prompt tokens and feature spans.

``expand`` turns each ``<｜image｜>`` marker of the tokenised prompt into as many image-token ids as
the image's plan has language-model positions, records where they sit, and derives the media
identity under which prefix caches key the conversation.  ``spans`` runs the vision tower
(content-keyed cache in front of it) and returns the (offsets, rows) pair that prefill uses to
replace the embeddings at those positions (reference: src/worker_media.rs, src/prompt_media.rs,
src/image_input_cache.rs, src/image_cache.rs).
"""
from __future__ import annotations

import base64
import hashlib
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from . import vision_input as VI

MAX_IMAGES = 16
MAX_ENCODED_BYTES = 32 << 20


class MediaError(ValueError):
    pass


def decode_data_uri(uri: str) -> bytes:
    if not uri.startswith("data:"):
        raise MediaError("only data: URIs are accepted for images (the server makes no outbound requests)")
    head, _, body = uri.partition(",")
    if not head.endswith(";base64"):
        raise MediaError("image data URI must be base64")
    if len(body) * 3 // 4 > MAX_ENCODED_BYTES:
        raise MediaError("image too large")
    try:
        return base64.b64decode(body, validate=True)
    except Exception as e:                                  # noqa: BLE001
        raise MediaError("bad base64 in image data URI") from e


@dataclass
class PromptMedia:
    tokens: List[int]
    images: List[VI.Prepared] = field(default_factory=list)
    offsets: List[Tuple[int, int]] = field(default_factory=list)     # (first prompt offset, count) per image
    identity: str = ""


def expand(tokens: Sequence[int], uris: Sequence[str], marker_id: int, image_token_id: int,
           cache: Optional[VI.ImageCache] = None, max_tokens: int = 1024) -> PromptMedia:
    if len(uris) > MAX_IMAGES:
        raise MediaError(f"at most {MAX_IMAGES} images per request")
    n_mark = sum(1 for t in tokens if t == marker_id)
    if n_mark != len(uris):
        raise MediaError("image markers and image parts disagree")
    preps: List[VI.Prepared] = []
    for u in uris:
        raw = decode_data_uri(u)
        key = VI.identity(raw)
        p = cache.get(key) if cache is not None else None
        if p is None:
            try:
                p = VI.prepare(raw, max_tokens=max_tokens)
            except ValueError as e:
                raise MediaError(str(e)) from e
            if cache is not None:
                cache.put(key, p, p.patches.numel() * 2)
        preps.append(p)
    out, offs, i = [], [], 0
    for t in tokens:
        if t == marker_id:
            n = preps[i].plan.tokens
            offs.append((len(out), n))
            out.extend([image_token_id] * n)
            i += 1
        else:
            out.append(int(t))
    ident = hashlib.sha256(b"".join(p.identity for p in preps)).hexdigest() if preps else ""
    return PromptMedia(out, preps, offs, ident)


class VisionFrontend:
    """What the HTTP front end needs to accept image parts: the tokenizer's image marker, the
    placeholder token id of the language model, the per-image token cap and a content-keyed cache
    of prepared images (CPU decode / resize / patchify happens once per distinct image)."""

    def __init__(self, marker_id: int, image_token_id: int, max_tokens: int = 1024, cache_bytes: int = 256 << 20):
        self.marker_id, self.image_token_id, self.max_tokens = marker_id, image_token_id, max_tokens
        self.cache = VI.ImageCache(cache_bytes)

    def expand(self, tokens: Sequence[int], uris: Sequence[str]) -> PromptMedia:
        return expand(tokens, uris, self.marker_id, self.image_token_id, self.cache, self.max_tokens)


class SpanEncoder:
    """Vision tower + feature cache: prepared images -> rows that replace image-token embeddings."""

    def __init__(self, tower, cache_bytes: int = 1 << 30):
        self.tower, self.cache = tower, VI.ImageCache(cache_bytes)

    def spans(self, pm: PromptMedia) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if not pm.images:
            return None
        offs, rows = [], []
        for prep, (o, n) in zip(pm.images, pm.offsets):
            span = self.cache.get(prep.identity)
            if span is None:
                span = self.tower.encode(prep.patches, prep.plan.vit_height, prep.plan.vit_width)
                self.cache.put(prep.identity, span, span.numel() * 2)
            if span.shape[0] != n:
                raise MediaError("vision span length differs from the plan")
            offs.append(torch.arange(o, o + n))
            rows.append(span)
        return torch.cat(offs), torch.cat(rows)
