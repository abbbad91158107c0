"""Typed configuration objects: model geometry, engine policy, server policy.

One ``ModelConfig`` instantiates every geometry the framework runs: the tiny
plumbing model, the 43-layer / hidden-4096 benchmark model and the
reference's 40-layer / hidden-5120 "1017" checkpoint geometry (reference:
src/config.rs:5-92 and :193-296 validate exactly one geometry; here the same
fields are parameters).  Configs are plain dataclasses that round-trip through
JSON, hash to a stable digest, and are byte-agreed across ranks at start-up
(reference: src/resident_worker.rs:5935-5977 agrees every policy value that
shapes device state).
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


def _canon(obj: Any) -> Any:
    if dataclasses.is_dataclass(obj):
        return {f.name: _canon(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, (list, tuple)):
        return [_canon(x) for x in obj]
    if isinstance(obj, dict):
        return {str(k): _canon(v) for k, v in sorted(obj.items())}
    return obj


class _JsonMixin:
    def to_dict(self) -> Dict[str, Any]:
        return _canon(self)

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"))

    def digest(self) -> str:
        """SHA-256 of the canonical JSON: the value ranks agree on at start-up."""
        return hashlib.sha256(self.to_json().encode()).hexdigest()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]):
        names = {f.name: f for f in dataclasses.fields(cls)}
        unknown = set(d) - set(names)
        if unknown:
            raise ValueError(f"unknown {cls.__name__} field(s): {sorted(unknown)}")
        kw = {}
        for k, v in d.items():
            f = names[k]
            sub = _SUBCONFIGS.get((cls.__name__, k))
            if sub is not None and isinstance(v, dict):
                v = sub.from_dict(v)
            elif isinstance(v, list) and "Tuple" in str(f.type):
                v = tuple(v)
            kw[k] = v
        return cls(**kw)

    @classmethod
    def from_json(cls, s: str):
        return cls.from_dict(json.loads(s))


@dataclass
class RopeConfig(_JsonMixin):
    """Rotary embedding; YaRN when ``factor > 1`` (reference: kernels/core.cu:980-999)."""
    theta: float = 10000.0
    compress_theta: float = 160000.0
    dim: int = 64                      # rotated tail of every head
    factor: float = 1.0                # YaRN scaling factor (1 = plain RoPE)
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_max_position: int = 65536


@dataclass
class DraftConfig(_JsonMixin):
    """Speculative draft head (reference draft network: src/dspark.rs:42)."""
    layers: int = 1                    # decoder layers in the draft head
    depth: int = 3                     # proposals per verification round
    condition_layers: int = 1          # last N target layers whose output feeds the draft
    temperature: float = 0.7           # proposal temperature when sampling
    confidence_head: bool = False      # the drafter scores each proposal before it is verified (causal stopping)
    confidence_ladder: Tuple[float, ...] = (0.15, 0.25, 0.20, 0.15)    # thresholds of proposals 2, 3, ... on the running product
    markov_rank: int = 0               # rank of the Markov (bigram) correction of the draft logits; 0 = none (reference: 256)
    subset_rows: int = 0               # 4-bit vocabulary-subset head of the drafter: it proposes only these many tokens (multiple of 128; 0 = whole vocabulary; reference: 61 % of the vocabulary)


@dataclass
class VisionConfig(_JsonMixin):
    """ViT tower (reference: src/vision.rs:19-44)."""
    layers: int = 32
    hidden: int = 1024
    heads: int = 16
    patch: int = 14
    downsample: int = 3
    intermediate: int = 4096
    max_image_tokens: int = 1024
    image_token_id: int = 129264


@dataclass
class EngramConfig(_JsonMixin):
    """n-gram hashed embedding memory (reference: src/hash_history.rs:6-15)."""
    layers: Tuple[int, ...] = ()
    tables: int = 2
    ngram: int = 4
    heads: int = 8
    width: int = 256                   # fp8 values per row (+ width/32 ue8m0)
    rows_per_table: int = 0


@dataclass
class ModelConfig(_JsonMixin):
    name: str = "tiny"
    n_layers: int = 2
    hidden: int = 256
    vocab: int = 1024
    # attention: MQA over one latent that is both K and V (reference: src/layout.rs:233-239)
    n_heads: int = 4
    head_dim: int = 64
    q_lora_rank: int = 0               # 0 = direct wq; >0 = wq_a -> norm -> wq_b
    o_groups: int = 0                  # 0 = direct wo; >0 = grouped low-rank wo_a -> wo_b
    o_lora_rank: int = 0
    attn_sink: bool = True
    window: int = 32
    # sparse attention over compressed KV
    compress_ratio: int = 4            # tokens pooled per compressed entry at source layers
    #   (with ``compress_ratios``: the finest stream's ratio, which the step metadata counts in)
    compress_ratios: Tuple[int, ...] = ()         # one ratio per kv source layer; () = compress_ratio everywhere
    kv_source_layers: Tuple[int, ...] = (0,)      # layers owning a compressed KV stream
    index_source_layers: Tuple[int, ...] = (0,)   # layers running the indexer (others reuse)
    index_heads: int = 4
    index_dim: int = 32
    index_topk: int = 16
    candidate_blocks: int = 0          # two-level selection: keep this many blocks (0 = off)
    candidate_block: int = 8
    late_start: int = -1               # first layer of the late group (prefill replays only the
                                       # last `window` rows there); -1 = none
    # MoE
    n_experts: int = 8
    topk: int = 2
    moe_inter: int = 512
    n_shared: int = 1
    shared_inter: int = 512
    scoring: str = "softmax"           # "softmax" | "sqrtsoftplus"
    router_bias: bool = False
    router_bias_vl: bool = False       # image-token rows select experts with gate.bias_vl instead of gate.bias
    image_token: int = -1              # token id of image placeholder rows (reference: 129264)
    renorm: bool = True
    route_scale: float = 1.0
    swiglu_limit: float = 0.0          # 0 = no clamp
    # residual
    hc_mult: int = 1                   # 1 = plain residual, 4 = mHC hyper-connections
    sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    rms_eps: float = 1e-6
    rope: RopeConfig = field(default_factory=lambda: RopeConfig(dim=32))
    # quantisation of the stored weights
    dense_quant: str = "none"          # "none" | "fp8_block128" | "fp8_ue8m0_32"
    expert_quant: str = "none"         # "none" | "mxfp4"
    kv_quant: str = "none"             # "none" | "v41" (FP8 window + FP4 compressed)
    init_std: float = 0.02
    max_positions: int = 1048576
    draft: Optional[DraftConfig] = None
    vision: Optional[VisionConfig] = None
    engram: Optional[EngramConfig] = None

    # ---- derived -------------------------------------------------------
    def __post_init__(self):
        self.kv_source_layers = tuple(self.kv_source_layers)
        self.index_source_layers = tuple(self.index_source_layers)
        self.validate()

    def validate(self) -> None:
        def need(ok: bool, msg: str):
            if not ok:
                raise ValueError(f"ModelConfig[{self.name}]: {msg}")
        need(self.n_layers >= 1 and self.hidden % 2 == 0, "bad layers/hidden")
        need(self.rope.dim <= self.head_dim and self.rope.dim % 2 == 0, "rope dim")
        need(self.scoring in ("softmax", "sqrtsoftplus"), "scoring")
        need(self.hc_mult in (1, 4), "hc_mult must be 1 or 4")
        need(self.topk <= self.n_experts, "topk > experts")
        need(all(0 <= l < self.n_layers for l in self.kv_source_layers), "kv source layer range")
        need(set(self.index_source_layers) >= set(self.kv_source_layers) or not self.index_source_layers,
             "every kv source layer must run an indexer")
        need(all(0 <= l < self.n_layers for l in self.index_source_layers), "index source layer range")
        need(self.compress_ratio >= 1, "compress ratio")
        need(self.candidate_block == 8, "candidate blocks are 8 keys (the block-maximum kernel's unit)")
        if self.compress_ratios:
            need(len(self.compress_ratios) == len(self.kv_source_layers), "one compress ratio per kv source layer")
            need(min(self.compress_ratios) == self.compress_ratio, "compress_ratio must be the smallest of compress_ratios")
            need(all(r % self.compress_ratio == 0 for r in self.compress_ratios),
                 "every compress ratio must be a multiple of the smallest")
        need(self.dense_quant in ("none", "fp8_block128", "fp8_ue8m0_32"), "dense_quant")
        need(self.expert_quant in ("none", "mxfp4"), "expert_quant")
        need(self.kv_quant in ("none", "v41"), "kv_quant")
        if self.late_start >= 0:
            need(self.late_start - 1 in self.kv_source_layers or self.late_start == 0,
                 "late group must start right after a kv source layer")

    def kv_source_of(self, layer: int) -> int:
        """Compressed-KV source layer a layer reads (-1: window-only layer)."""
        best = -1
        for s in self.kv_source_layers:
            if s <= layer:
                best = max(best, s)
        return best

    def ratio_of_source(self, source_layer: int) -> int:
        """Tokens pooled per compressed entry in the stream of one kv source layer (reference:
        ``compress_ratios`` per layer, src/config.rs:252-280: 2 for layers 2-19, 1 from layer 20)."""
        if not self.compress_ratios:
            return self.compress_ratio
        return self.compress_ratios[self.kv_source_layers.index(source_layer)]

    def ratio_of(self, layer: int) -> int:
        """Ratio of the compressed stream a layer reads (the finest ratio for window-only layers)."""
        src = self.kv_source_of(layer)
        return self.ratio_of_source(src) if src >= 0 else self.compress_ratio

    @property
    def max_ratio(self) -> int:
        return max(self.compress_ratios) if self.compress_ratios else self.compress_ratio

    def index_source_of(self, layer: int) -> int:
        best = -1
        for s in self.index_source_layers:
            if s <= layer:
                best = max(best, s)
        return best

    @property
    def window_kv_bytes(self) -> int:
        """V4.1 window-cache bytes/token: e4m3 values + one ue8m0 per 32
        (528 for a 512-wide latent; reference src/attention.rs:18-38); the row stride is rounded
        up to 16 bytes so that rows of narrower latents stay vector-load aligned."""
        return -(-(self.head_dim + self.head_dim // 32) // 16) * 16

    @property
    def compressed_kv_bytes(self) -> int:
        """V4.1-FP4 bytes/entry: packed e2m1 + one e4m3 scale per 16 (288 at 512), stride
        rounded up to 16 bytes."""
        return -(-(self.head_dim // 2 + self.head_dim // 16) // 16) * 16

    @property
    def index_key_bytes(self) -> int:
        """Index key: packed e2m1 + one ue8m0 per 32 (68 B at 128 dims)."""
        return self.index_dim // 2 + self.index_dim // 32


_SUBCONFIGS = {
    ("ModelConfig", "rope"): RopeConfig,
    ("ModelConfig", "draft"): DraftConfig,
    ("ModelConfig", "vision"): VisionConfig,
    ("ModelConfig", "engram"): EngramConfig,
}


# ---------------------------------------------------------------------------
# Named geometries
# ---------------------------------------------------------------------------
def tiny_config(**over) -> ModelConfig:
    """2-layer plumbing model: hidden 256, 4 heads x 64, window 32, top-16 indexer over a
    4x-compressed KV, 8 experts top-2 (softmax) + 1 shared, inter 512, vocab 1024."""
    kw = dict(name="tiny", n_layers=2, hidden=256, vocab=1024, n_heads=4, head_dim=64, window=32,
              compress_ratio=4, kv_source_layers=(0,), index_source_layers=(0,), index_heads=4,
              index_dim=32, index_topk=16, n_experts=8, topk=2, moe_inter=512, n_shared=1,
              shared_inter=512, scoring="softmax", renorm=True, rms_eps=1e-6,
              rope=RopeConfig(theta=10000.0, compress_theta=10000.0, dim=32),
              draft=DraftConfig(layers=1, depth=3))
    kw.update(over)
    return ModelConfig(**kw)


def flash_b200_config(**over) -> ModelConfig:
    """Full-size benchmark geometry: 43 layers, hidden 4096, 64 heads x 128, window 128 plus
    FP4-compressed KV (4x), top-2048 BF16 indexer, 256 MXFP4 experts top-6 + 1 shared (inter
    2048), FP8 dense weights with 128x128 block scales, vocab 129280, 1-layer draft head
    depth 3.  Source-layer placement follows the reference's pattern (compressed streams at
    a few source layers, followers reuse them; the late group starts after the last source)."""
    kw = dict(name="flash-b200", n_layers=43, hidden=4096, vocab=129280, n_heads=64, head_dim=128,
              window=128, compress_ratio=4, kv_source_layers=(2, 8, 14, 20),
              index_source_layers=(2, 8, 14, 20, 26, 32, 38), index_heads=8, index_dim=128,
              index_topk=2048, candidate_blocks=2048, candidate_block=8, late_start=21,
              n_experts=256, topk=6, moe_inter=2048, n_shared=1, shared_inter=2048,
              scoring="sqrtsoftplus", router_bias=True, renorm=True, route_scale=1.5,
              swiglu_limit=10.0, rms_eps=1e-6,
              rope=RopeConfig(theta=10000.0, compress_theta=160000.0, dim=64, factor=16.0,
                              original_max_position=65536),
              dense_quant="fp8_block128", expert_quant="mxfp4", kv_quant="v41",
              draft=DraftConfig(layers=1, depth=3))
    kw.update(over)
    return ModelConfig(**kw)


def reference_1017_config(**over) -> ModelConfig:
    """The geometry the reference serves (tests/fixtures/1017-config.json; src/config.rs:193-296)."""
    # per layer [0, 0] + [2] * 18 + [1] * 20: the three early sources pool pairs, layer 20 keeps every token
    kw = dict(name="DeepSeek-V4.1-Flash-1017", n_layers=40, hidden=5120, vocab=129280, n_heads=64,
              head_dim=512, q_lora_rank=1280, o_groups=8, o_lora_rank=1024, window=128,
              compress_ratio=1, compress_ratios=(2, 2, 2, 1), kv_source_layers=(2, 8, 14, 20),
              index_source_layers=(2, 8, 14, 20, 24, 28, 32, 36), index_heads=32, index_dim=128,
              index_topk=512, candidate_blocks=2048, candidate_block=8, late_start=21,
              n_experts=384, topk=6, moe_inter=2304, n_shared=1, shared_inter=2304,
              scoring="sqrtsoftplus", router_bias=True, renorm=True, route_scale=1.5,
              swiglu_limit=10.0, hc_mult=4, sinkhorn_iters=20, hc_eps=1e-6, rms_eps=1e-20,
              rope=RopeConfig(theta=10000.0, compress_theta=160000.0, dim=64, factor=16.0,
                              beta_fast=32.0, beta_slow=1.0, original_max_position=65536),
              dense_quant="fp8_ue8m0_32", expert_quant="mxfp4", kv_quant="v41",
              draft=DraftConfig(layers=3, depth=5, condition_layers=3, markov_rank=256, confidence_head=True),
              vision=VisionConfig(), engram=EngramConfig(layers=(1, 14), rows_per_table=384_000_000))
    kw.update(over)
    return ModelConfig(**kw)


NAMED_MODELS = {"tiny": tiny_config, "flash-b200": flash_b200_config,
                "1017": reference_1017_config}


# ---------------------------------------------------------------------------
# Engine / server policy
# ---------------------------------------------------------------------------
@dataclass
class EngineConfig(_JsonMixin):
    """Per-cohort runtime policy (reference: WorkerConfig src/resident_worker.rs:268-290 and
    the env policy of src/config.rs; here one typed object, no env sprawl)."""
    tp: int = 1
    moe_parallel: str = "ep"           # "ep": whole experts per rank; "tp": column-sliced
    regions: int = 4                   # concurrently admitted conversations
    max_context: int = 131072
    prefill_widths: Tuple[int, ...] = (256, 1024, 4096, 16384)
    session_slots: int = 16            # entries of the session cache (state images of prefixes and finished turns)
    session_budget_bytes: int = 8 << 30   # device bytes the cache may hold; older images move to the host tier
    host_tier_bytes: int = 32 << 30    # pinned host bytes of parked images; beyond it they go to the disk tier
    disk_tier_dir: str = ""            # directory of the disk tier ("" = none: the oldest host images are dropped instead)
    checkpoint_min_tokens: int = 8192  # prompts shorter than this leave no intermediate checkpoints; also the checkpoint spacing
    prefill_slice_ms: int = 500        # a prefill yields to one batched decode step of the other conversations this often
    spin_limit: int = 20_000_000       # bounded device waits (reference src/roce.rs:1196-1199)
    use_cuda_graphs: bool = True
    key_sharded_index_min: int = 262144  # decode rows: split index scoring over the ranks from this many keys (0 = never); below about a million tokens of context the exchange costs more than the scoring it saves
    two_level_index_min: int = 65536   # decode rows: from this many index keys on, layers after the candidate source score only its published blocks (0 = never)
    reference_matmul: bool = False     # validation only: rows beyond the small-M limit may run through dequantised weights and torch.matmul when the tensor-core path is not attached (never set in serving or benchmarks: the engine refuses instead)
    pdl: bool = False                  # launch kernels with programmatic dependent launch (each kernel waits for its predecessor on the device; the next one is already resident)
    sp_prefill: bool = True            # more than one rank: prefill chunks are split by rows over the ranks (every rank keeps the unsharded dense matrices of the encoder layers)
    sp_chunk_rows: int = 0                 # rows of one sequence-parallel prefill chunk over ALL ranks (0: the single-rank chunk); the window ring holds a whole chunk
    index_score_bytes: int = 2 << 30       # most bytes of one fp32 index-score matrix: prefill rows are scored and selected in row tiles beyond it (long contexts)
    prefill_mx: bool = True                # prefill GEMMs on the block-scaled tensor-core form (MXFP8 activations)
    moe_block_scaled: bool = True     # decode rows <= 16: routed experts on block-scaled tcgen05 MMAs (MXFP8 activations)
    seed: int = 0


@dataclass
class ServerConfig(_JsonMixin):
    """HTTP front-end policy (reference: ServerConfig src/http_server.rs:88)."""
    host: str = "127.0.0.1"
    port: int = 8000
    api_key: str = ""
    model_name: str = "DeepSeek-V4.1-Flash-1017"
    max_admitted: int = 4
    queue_limit: int = 16
    background_queue_limit: int = 4
    upload_timeout_s: float = 15.0
    keepalive_s: float = 5.0
    default_max_tokens: int = 262144
    context_cache_bytes: int = 64 << 20


def agree_digest(cfgs: List[_JsonMixin]) -> str:
    h = hashlib.sha256()
    for c in cfgs:
        h.update(c.digest().encode())
    return h.hexdigest()
