"""Image input on the CPU: decode, plan the patch grid, PIL-bicubic resize with centred padding,
pack 14x14 CHW patches as bf16, and cache the result by content.

The plan keeps at most ``max_tokens`` language-model positions per image
(tokens = llm_h * (llm_w + 1) + 2: one newline per feature row plus start / end markers) and pads
with mid-grey (127) so that the padding normalises to ~0 (reference: src/vision_input/mod.rs:55-131
Plan::new, :142 prepare_rgb, :33 identity; src/vision_input/patch.rs:17-80 resize_patchify;
src/image_input_cache.rs content-keyed cache).
"""
from __future__ import annotations

import hashlib
import io
import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

PATCH, DOWNSAMPLE = 14, 3
MIN_PIXELS = 544 * 544
MAX_INPUT_PIXELS = 89_478_485
INVALID = "invalid image"


def _round_even(v: float) -> int:
    return int(round(v))            # Python's round is ties-to-even


@dataclass
class Plan:
    width: int
    height: int
    resize_width: int
    resize_height: int
    top: int
    left: int
    vit_height: int
    vit_width: int
    llm_height: int
    llm_width: int
    tokens: int

    @staticmethod
    def new(ow: int, oh: int, max_tokens: int = 1024) -> "Plan":
        area = ow * oh
        if not (0 < area <= MAX_INPUT_PIXELS):
            raise ValueError(INVALID)
        w, h = ow, oh
        if area < MIN_PIXELS:
            r = math.sqrt(MIN_PIXELS / area)
            w, h = int(w * r), int(h * r)
        out_w, out_h = -(-w // PATCH) * PATCH, -(-h // PATCH) * PATCH
        grid = lambda hh, ww: (-(-(hh // PATCH) // DOWNSAMPLE), -(-(ww // PATCH) // DOWNSAMPLE))
        count = lambda hh, ww: hh * (ww + 1) + 2
        lh, lw = grid(out_h, out_w)
        if count(lh, lw) > max_tokens:
            ratio = h / w
            max_w = math.sqrt((max_tokens - 2) / ratio + 0.25) - 0.5
            max_h = max_w * ratio
            cell = PATCH * DOWNSAMPLE
            if max_w < 1.0:
                out_h, out_w = (max_tokens - 2) // 2 * cell, cell
            elif max_h < 1.0:
                out_h, out_w = cell, (max_tokens - 3) * cell
            else:
                beta = min(math.floor(max_w) * cell / w, math.floor(max_h) * cell / h)
                out_h = int(math.floor(h * beta / PATCH)) * PATCH
                out_w = int(math.floor(w * beta / PATCH)) * PATCH
        lh, lw = grid(out_h, out_w)
        rh, rw = out_h, out_w
        o_ratio, t_ratio = ow / oh, out_w / out_h
        if o_ratio > t_ratio:
            rh = _round_even(oh / ow * out_w)
        elif o_ratio < t_ratio:
            rw = _round_even(ow / oh * out_h)
        if not (0 < rh <= out_h and 0 < rw <= out_w and count(lh, lw) <= max_tokens):
            raise ValueError(INVALID)
        return Plan(out_w, out_h, rw, rh, _round_even((out_h - rh) / 2), _round_even((out_w - rw) / 2),
                    out_h // PATCH, out_w // PATCH, lh, lw, count(lh, lw))


def identity(encoded: bytes, detail: str = "auto") -> bytes:
    return hashlib.sha256(b"tflash-image\0" + detail.encode() + b"\0" + encoded).digest()


def decode_rgb(encoded: bytes) -> np.ndarray:
    """Encoded image bytes -> [H, W, 3] uint8 (alpha composited on white)."""
    from PIL import Image
    try:
        im = Image.open(io.BytesIO(encoded))
        im.load()
    except Exception as e:                                   # noqa: BLE001 - any decoder failure is a bad request
        raise ValueError(INVALID) from e
    if im.mode in ("RGBA", "LA", "P"):
        im = im.convert("RGBA")
        bg = Image.new("RGBA", im.size, (255, 255, 255, 255))
        im = Image.alpha_composite(bg, im)
    return np.asarray(im.convert("RGB"), dtype=np.uint8)


def resize_patchify(rgb: np.ndarray, plan: Plan) -> torch.Tensor:
    """[H, W, 3] uint8 -> [vit_h * vit_w, 3 * 14 * 14] bf16, patch-major, channel-first inside a patch."""
    from PIL import Image
    if rgb.ndim != 3 or rgb.shape[2] != 3:
        raise ValueError(INVALID)
    im = Image.fromarray(rgb).resize((plan.resize_width, plan.resize_height), Image.BICUBIC)
    canvas = np.full((plan.height, plan.width, 3), 127, dtype=np.uint8)
    canvas[plan.top:plan.top + plan.resize_height, plan.left:plan.left + plan.resize_width] = np.asarray(im)
    lut = (((torch.arange(256, dtype=torch.float32) / 255.0) - 0.5) / 0.5).to(torch.bfloat16)
    x = torch.from_numpy(canvas).long()                                      # [H, W, 3]
    gh, gw = plan.vit_height, plan.vit_width
    x = x.view(gh, PATCH, gw, PATCH, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * PATCH * PATCH)
    return lut[x]


@dataclass
class Prepared:
    identity: bytes
    original: Tuple[int, int]
    plan: Plan
    patches: torch.Tensor


def prepare(encoded: bytes, detail: str = "auto", max_tokens: int = 1024) -> Prepared:
    rgb = decode_rgb(encoded)
    plan = Plan.new(rgb.shape[1], rgb.shape[0], max_tokens)
    return Prepared(identity(encoded, detail), (rgb.shape[1], rgb.shape[0]), plan, resize_patchify(rgb, plan))


class ImageCache:
    """Content-keyed LRU of prepared images (and, once encoded, their feature spans) under a byte budget."""

    def __init__(self, budget_bytes: int = 256 << 20):
        self.budget, self.used = budget_bytes, 0
        self.items: "OrderedDict[bytes, Tuple[object, int]]" = OrderedDict()
        self.hits = self.misses = 0

    def get(self, key: bytes):
        it = self.items.get(key)
        if it is None:
            self.misses += 1
            return None
        self.items.move_to_end(key)
        self.hits += 1
        return it[0]

    def put(self, key: bytes, value, nbytes: int) -> bool:
        if nbytes > self.budget:
            return False
        if key in self.items:
            self.used -= self.items.pop(key)[1]
        while self.used + nbytes > self.budget and self.items:
            _, (_, n) = self.items.popitem(last=False)
            self.used -= n
        self.items[key] = (value, nbytes)
        self.used += nbytes
        return True
