"""Plain-PyTorch restatement of the whole model: the numerical oracle and the CPU/gloo path.

Everything here is written for clarity in fp32 (or fp64) on whatever device the weights live
on.  The CUDA path (``models/engine.py``) must agree with this file on the same weights; the
tensor-parallel path must agree with the single-rank run of this file (plumbing check: TP=2
over gloo, logits within 1e-4).

Model structure (generalising the reference's layer: src/decoder.rs:802-850,
src/layer_attention.rs:1121-1455, src/ffn.rs:974-1047):

    x -> [boundary: (mHC collapse) + RMSNorm] -> attention -> sum over ranks -> residual
      -> [boundary] -> MoE FFN (router, routed experts, shared expert) -> sum -> residual

Attention is MQA over one latent per token that is both K and V; every query row attends to
the last ``window`` tokens, to the ``index_topk`` compressed entries its indexer selected and
to a per-head sink; RoPE is applied to q and k and the inverse rotation to the output
(src/layer_attention.rs:1416-1423).  Compressed entries pool ``compress_ratio`` consecutive
tokens with a per-channel softmax gate (ratio-2 form: kernels/core.cu:944-950).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from ..formats import codecs
from ..parallel.comm import Comm, LocalComm


# ---------------------------------------------------------------------------
# elementary math
# ---------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """``(x * rsqrt(mean(x^2) + eps)) * w`` with fp32 statistics (kernels/core.cu:851-857)."""
    xf = x.to(torch.float32)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * w if w is not None else y


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float) -> torch.Tensor:
    """``g=min(gate,L); u=clamp(up,+-L); g*sigmoid(g)*u`` (kernels/core.cu:938-942)."""
    if limit > 0:
        gate = torch.clamp(gate, max=limit)
        up = torch.clamp(up, -limit, limit)
    return gate * torch.sigmoid(gate) * up


def rope_frequencies(dim: int, theta: float, factor: float = 1.0, beta_fast: float = 32.0,
                     beta_slow: float = 1.0, original_max: int = 65536) -> torch.Tensor:
    """``dim/2`` inverse frequencies; YaRN ramp when factor > 1 (kernels/core.cu:980-995)."""
    j = torch.arange(dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * j / dim)
    if factor > 1.0:
        def corr(beta):
            return dim * math.log(original_max / (beta * 2 * math.pi)) / (2 * math.log(theta))
        low = max(math.floor(corr(beta_fast)), 0)
        high = min(math.ceil(corr(beta_slow)), dim // 2 - 1)
        if high == low:
            high = low + 0.001
        smooth = 1.0 - torch.clamp((j - low) / (high - low), 0.0, 1.0)
        f = (f / factor) * (1 - smooth) + f * smooth
    return f.to(torch.float32)


def apply_rope(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor, inverse: bool = False
               ) -> torch.Tensor:
    """Rotate the last ``2*len(freqs)`` dims of x[..., D] (pairs are (2j, 2j+1)) by
    ``pos*freq``; x's leading dims broadcast against pos[T] placed at dim 0."""
    rd = freqs.numel() * 2
    D = x.shape[-1]
    ang = pos.to(torch.float32)[:, None] * freqs.to(x.device)[None, :]         # [T, rd/2]
    cos, sin = torch.cos(ang), torch.sin(ang)
    if inverse:
        sin = -sin
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [rd // 2]
    cos, sin = cos.reshape(shape), sin.reshape(shape)
    head, tail = x[..., : D - rd], x[..., D - rd:]
    a, b = tail[..., 0::2], tail[..., 1::2]
    ra, rb = a * cos - b * sin, a * sin + b * cos
    rot = torch.stack([ra, rb], -1).reshape(tail.shape)
    return torch.cat([head, rot], -1)


def route(logits: torch.Tensor, cfg: ModelConfig, bias: Optional[torch.Tensor],
          bias_vl: Optional[torch.Tensor] = None, image_rows: Optional[torch.Tensor] = None
          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router: returns (expert ids [T,k] in selection order, weights [T,k] fp32).

    ``sqrtsoftplus``: score = sqrt(softplus(x)); selection key = score + bias; weights are the
    unbiased scores of the winners, renormalised and scaled (kernels/moe_frontend.cuh:27-130).
    ``softmax``: score = softmax(x).  Ties go to the lowest expert id."""
    lf = logits.to(torch.float32)
    if cfg.scoring == "sqrtsoftplus":
        sp = torch.where(lf > 20, lf, torch.log1p(torch.exp(torch.clamp(lf, max=20))))
        score = torch.sqrt(sp)
    else:
        score = torch.softmax(lf, -1)
    key = score + bias if (bias is not None and cfg.router_bias) else score
    if bias_vl is not None and image_rows is not None and cfg.router_bias and bool(image_rows.any()):
        # the selection bias is chosen per token: image rows use gate.bias_vl (kernels/moe_frontend.cuh:140)
        key = torch.where(image_rows[:, None], score + bias_vl, key)
    key = torch.nan_to_num(key, nan=float("inf"))
    # stable descending sort => ties resolved by lowest expert id
    order = torch.sort(key, dim=-1, descending=True, stable=True).indices[:, : cfg.topk]
    w = torch.gather(score, 1, order)
    if cfg.renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return order, w * cfg.route_scale


# ---------------------------------------------------------------------------
# mHC boundary (hc_mult = 4)   reference arithmetic: kernels/core.cu:859-936
# ---------------------------------------------------------------------------
def hc_coefficients(x: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
                    iters: int, eps: float, rms_eps: float):
    """x [T,4,d] -> (pre [T,4], post [T,4], comb [T,4,4]).

    24 mixes over the flattened row share one rsqrt; pre = sigmoid(m*s0+b)+eps,
    post = 2*sigmoid(m*s1+b), comb = Sinkhorn(softmax rows + eps)."""
    T, H, d = x.shape
    flat = x.reshape(T, H * d).to(torch.float32)
    inv = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + rms_eps)
    mixes = (flat @ fn.t()) * inv                                   # [T, H*(2+H)]
    pre = torch.sigmoid(mixes[:, :H] * scale[0] + base[:H]) + eps
    post = 2 * torch.sigmoid(mixes[:, H:2 * H] * scale[1] + base[H:2 * H])
    c = (mixes[:, 2 * H:] * scale[2] + base[2 * H:]).reshape(T, H, H)
    c = torch.softmax(c, -1) + eps
    c = c / (c.sum(1, keepdim=True) + eps)                           # column normalise
    for _ in range(iters - 1):
        c = c / (c.sum(2, keepdim=True) + eps)
        c = c / (c.sum(1, keepdim=True) + eps)
    return pre, post, c


def hc_collapse(x: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    return (x.to(torch.float32) * pre[:, :, None]).sum(1)


def hc_post(x: torch.Tensor, a: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """y_c = post_c * a + sum_k comb[k,c] * x_k   (kernels/core.cu:899-907)."""
    return post[:, :, None] * a[:, None, :] + torch.einsum("tkc,tkd->tcd", comb, x.to(torch.float32))


# ---------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------
def init_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random-init N(0, init_std) weights under the reference's tensor names
    (src/layout.rs:220-295)."""
    g = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def mat(name, n, k, std=None):
        W[name] = (torch.randn(n, k, generator=g, dtype=torch.float32) * (std or cfg.init_std)).to(dtype)

    d, H, Dh = cfg.hidden, cfg.n_heads, cfg.head_dim
    mat("embed.weight", cfg.vocab, d)
    mat("head.weight", cfg.vocab, d)
    W["norm.weight"] = torch.ones(d, dtype=dtype)
    if cfg.hc_mult > 1:
        W["hc_head_fn"] = (torch.randn(cfg.hc_mult, cfg.hc_mult * d, generator=g) * cfg.init_std).to(dtype)
        W["hc_head_base"] = torch.zeros(cfg.hc_mult, dtype=dtype)
        W["hc_head_scale"] = torch.ones(1, dtype=dtype)
    n_total = cfg.n_layers + (cfg.draft.layers if cfg.draft else 0)
    for li in range(n_total):
        is_draft = li >= cfg.n_layers
        p = f"mtp.{li - cfg.n_layers}" if is_draft else f"layers.{li}"
        for br in ("attn", "ffn"):
            W[f"{p}.{br}_norm.weight"] = torch.ones(d, dtype=dtype)
            if cfg.hc_mult > 1:
                m = cfg.hc_mult
                mat(f"{p}.hc_{br}_fn", m * (2 + m), m * d)
                W[f"{p}.hc_{br}_base"] = torch.zeros(m * (2 + m), dtype=dtype)
                W[f"{p}.hc_{br}_scale"] = torch.ones(3, dtype=dtype)
        if cfg.q_lora_rank:
            mat(f"{p}.attn.wq_a.weight", cfg.q_lora_rank, d)
            W[f"{p}.attn.q_norm.weight"] = torch.ones(cfg.q_lora_rank, dtype=dtype)
            mat(f"{p}.attn.wq_b.weight", H * Dh, cfg.q_lora_rank)
        else:
            mat(f"{p}.attn.wq.weight", H * Dh, d)
        mat(f"{p}.attn.wkv.weight", Dh, d)
        W[f"{p}.attn.kv_norm.weight"] = torch.ones(Dh, dtype=dtype)
        if cfg.o_groups:
            per = H * Dh // cfg.o_groups
            mat(f"{p}.attn.wo_a.weight", cfg.o_groups * cfg.o_lora_rank, per)
            mat(f"{p}.attn.wo_b.weight", d, cfg.o_groups * cfg.o_lora_rank)
        else:
            mat(f"{p}.attn.wo.weight", d, H * Dh)
        if cfg.attn_sink:
            W[f"{p}.attn.attn_sink"] = (torch.randn(H, generator=g) * 0.5).to(dtype)
        if (not is_draft) and li in cfg.kv_source_layers:
            C = Dh + cfg.index_dim
            mat(f"{p}.attn.compressor.wkv.weight", C, d)
            mat(f"{p}.attn.compressor.wgate.weight", C, d)
            W[f"{p}.attn.compressor.norm.weight"] = torch.ones(Dh, dtype=dtype)
        if (not is_draft) and li in cfg.index_source_layers:
            mat(f"{p}.attn.indexer.wq.weight", cfg.index_heads * cfg.index_dim, d)
            mat(f"{p}.attn.indexer.weights_proj.weight", cfg.index_heads, d, std=1.0 / math.sqrt(d))
        mat(f"{p}.ffn.gate.weight", cfg.n_experts, d, std=1.0 / math.sqrt(d))
        W[f"{p}.ffn.gate.bias"] = torch.zeros(cfg.n_experts, dtype=dtype)
        if cfg.router_bias_vl and not is_draft:
            W[f"{p}.ffn.gate.bias_vl"] = (0.5 * torch.randn(cfg.n_experts, generator=g)).to(dtype)
        for nm, n, k in (("w1", cfg.moe_inter, d), ("w3", cfg.moe_inter, d), ("w2", d, cfg.moe_inter)):
            W[f"{p}.ffn.experts.{nm}.weight"] = (
                torch.randn(cfg.n_experts, n, k, generator=g) * cfg.init_std).to(dtype)
        if cfg.n_shared:
            si = cfg.shared_inter * cfg.n_shared
            mat(f"{p}.ffn.shared_experts.w1.weight", si, d)
            mat(f"{p}.ffn.shared_experts.w3.weight", si, d)
            mat(f"{p}.ffn.shared_experts.w2.weight", d, si)
        if is_draft and li == cfg.n_layers:
            # draft conditioning: [embedding of the anchor ; target hidden] -> d
            mat(f"{p}.main_proj.weight", d, d * (1 + cfg.draft.condition_layers))
            W[f"{p}.enorm.weight"] = torch.ones(d, dtype=dtype)
            W[f"{p}.hnorm.weight"] = torch.ones(d * cfg.draft.condition_layers, dtype=dtype)
            if cfg.draft.subset_rows:
                # vocabulary subset of the drafter's 4-bit head: sorted token ids
                # (reference: src/nvfp4_head.rs over src/latin_subset_v1.bin)
                W["mtp.head_subset.ids"] = torch.sort(
                    torch.randperm(cfg.vocab, generator=g)[: cfg.draft.subset_rows]).values.to(torch.int64)
            if cfg.draft.markov_rank:
                # Markov correction head of the last draft stage (reference: mtp.2.markov_head.{embed,head}.weight)
                mk = f"mtp.{cfg.draft.layers - 1}.markov_head"
                mat(f"{mk}.embed.weight", cfg.vocab, cfg.draft.markov_rank, std=1.0)
                mat(f"{mk}.head.weight", cfg.vocab, cfg.draft.markov_rank,
                    std=1.0 / math.sqrt(cfg.draft.markov_rank))
            if cfg.draft.confidence_head:
                # (reference: mtp.2.confidence_head.proj.weight [1, hidden + Markov rank])
                mat(f"mtp.{cfg.draft.layers - 1}.confidence_head.proj.weight", 1, d + cfg.draft.markov_rank,
                    std=2.0 / math.sqrt(d))
    if cfg.engram is not None and cfg.engram.layers:
        # hashed n-gram memory: one table per Engram layer (values exactly representable in the packed
        # MXFP8 row format), the projection of the looked-up rows to (copies + 1) x hidden, gate weights
        from . import engram as EG
        ec, m = cfg.engram, cfg.hc_mult
        rows = EG.table_rows(cfg)
        ids = (ec.ngram - 1) * ec.heads
        for e, l in enumerate(ec.layers):
            raw = torch.randn(rows, ec.width, generator=g) * 0.5
            W[f"engram.{e}.table"] = EG.unpack_rows(EG.pack_rows(raw)).to(dtype)
            mat(f"layers.{l}.engram.wkv.weight", (m + 1) * d, ids * ec.width, std=1.0 / math.sqrt(ids * ec.width))
            W[f"layers.{l}.engram.q_weight"] = (1 + 0.1 * torch.randn(m, d, generator=g)).to(dtype)
            W[f"layers.{l}.engram.k_weight"] = (1 + 0.1 * torch.randn(m, d, generator=g)).to(dtype)
    return W


def shard_weights(W: Dict[str, torch.Tensor], cfg: ModelConfig, rank: int, world: int,
                  moe_parallel: str = "ep") -> Dict[str, torch.Tensor]:
    """Slice a full weight dict for one rank (reference plan: src/layout.rs:57-144).

    embed/head rows, q heads (wq / wq_b rows), sinks, wo columns (K), shared-expert w1/w3 rows and
    w2 columns are split; routed experts are split whole ("ep") or column-sliced ("tp");
    everything else is replicated."""
    if world == 1:
        return dict(W)
    out = {}

    def sl(t, axis):
        n = t.shape[axis]
        assert n % world == 0, (n, world)
        return t.narrow(axis, rank * (n // world), n // world).contiguous()

    for name, t in W.items():
        if name in ("embed.weight", "head.weight") or name.endswith(".markov_head.head.weight"):
            out[name] = sl(t, 0)
        elif name.endswith((".attn.wq.weight", ".attn.wq_b.weight", ".attn.attn_sink")):
            out[name] = sl(t, 0)
        elif name.endswith(".attn.wo.weight"):
            out[name] = sl(t, 1)
        elif name.endswith(".attn.wo_a.weight"):
            out[name] = sl(t, 0)
        elif name.endswith(".attn.wo_b.weight"):
            out[name] = sl(t, 1)
        elif ".ffn.experts." in name:
            if moe_parallel == "ep":
                out[name] = sl(t, 0)
            else:
                out[name] = sl(t, 2) if name.endswith(".w2.weight") else sl(t, 1)
        elif ".ffn.shared_experts." in name:
            out[name] = sl(t, 1) if name.endswith(".w2.weight") else sl(t, 0)
        else:
            out[name] = t
    return out


# ---------------------------------------------------------------------------
# per-conversation state
# ---------------------------------------------------------------------------
@dataclass
class OracleSession:
    """Committed state of one conversation; every buffer is addressed by absolute position so
    that discarding speculative rows is only a change of ``length`` (the reference keeps carry
    snapshots for the same purpose: src/carry_state.rs)."""
    cfg: ModelConfig
    max_tokens: int
    device: torch.device = torch.device("cpu")
    dtype: torch.dtype = torch.float32
    length: int = 0
    window: Dict[str, torch.Tensor] = field(default_factory=dict)     # prefix -> [max_tokens, Dh]
    comp: Dict[str, torch.Tensor] = field(default_factory=dict)       # src prefix -> [maxC, Dh]
    keys: Dict[str, torch.Tensor] = field(default_factory=dict)       # src prefix -> [maxC, Di]
    carry: Dict[str, torch.Tensor] = field(default_factory=dict)      # src prefix -> [max_tokens, 2, C]
    tokens: List[int] = field(default_factory=list)
    token_at: Optional[torch.Tensor] = None                           # [max_tokens] token id by position (Engram)

    def buf(self, store: Dict[str, torch.Tensor], key: str, rows: int, *shape) -> torch.Tensor:
        if key not in store:
            store[key] = torch.zeros(rows, *shape, dtype=self.dtype, device=self.device)
        return store[key]


class OracleModel:
    """Reference forward pass. ``forward`` runs consecutive rows of ONE conversation (a prefill
    chunk or a verification block) against that conversation's state; ``forward_batch`` runs
    several conversations' rows and concatenates the logits."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], comm: Optional[Comm] = None,
                 moe_parallel: str = "ep", dtype=torch.float32):
        self.cfg, self.W, self.comm = cfg, weights, comm or LocalComm()
        self.moe_parallel = moe_parallel
        self.dtype = dtype
        r = cfg.rope
        self.freqs = rope_frequencies(r.dim, r.theta, r.factor, r.beta_fast, r.beta_slow,
                                      r.original_max_position)
        self.cfreqs = rope_frequencies(r.dim, r.compress_theta, r.factor, r.beta_fast, r.beta_slow,
                                       r.original_max_position)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.last_hidden: Optional[torch.Tensor] = None
        self.last_selection: Dict[int, torch.Tensor] = {}
        self.act_fp8 = False      # emulate FP8 (1x128 scaled) activations entering the linear layers
        # emulate MXFP8 (e4m3, one UE8M0 scale per 32 inputs) activations entering the routed
        # experts: the W4A8 form of the reference's expert GEMMs (moe.w4a8 kernels, MXFP8 K32
        # quantisation in kernels/moe_frontend.cuh)
        self.expert_act_mx8 = False

    def _aq_mx(self, x: torch.Tensor) -> torch.Tensor:
        if not self.expert_act_mx8 or x.shape[-1] % 32:
            return x
        q, s = codecs.mxfp8_quant(x.float().cpu(), 32)
        return codecs.mxfp8_dequant(q, s, 32).to(x.device, x.dtype)

    def _aq(self, x: torch.Tensor) -> torch.Tensor:
        """What an FP8 GEMM actually multiplies: the activation after e4m3 quantisation with one
        scale per (row, 128) — identity unless ``act_fp8`` is set."""
        if not self.act_fp8 or x.shape[-1] % 128:
            return x
        q, s = codecs.fp8_act_quant_1x128(x.cpu())
        return (q.float().reshape(*x.shape[:-1], -1, 128) * s.unsqueeze(-1)).reshape(x.shape).to(x.device, x.dtype)

    # -- pieces ----------------------------------------------------------
    def new_session(self, max_tokens: int) -> OracleSession:
        dev = self.W["norm.weight"].device
        return OracleSession(self.cfg, max_tokens, dev, self.dtype)

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        w = self.W["embed.weight"]
        vl = w.shape[0]
        local = tokens - self.rank * vl
        ok = (local >= 0) & (local < vl)
        x = torch.where(ok[:, None], w[torch.clamp(local, 0, vl - 1)].to(self.dtype),
                        torch.zeros((), dtype=self.dtype, device=w.device))
        return self.comm.all_reduce(x)

    def _boundary(self, x: torch.Tensor, p: str, br: str):
        cfg = self.cfg
        if cfg.hc_mult == 1:
            return rmsnorm(x, self.W[f"{p}.{br}_norm.weight"], cfg.rms_eps), None
        pre, post, comb = hc_coefficients(x, self.W[f"{p}.hc_{br}_fn"], self.W[f"{p}.hc_{br}_base"],
                                          self.W[f"{p}.hc_{br}_scale"], cfg.sinkhorn_iters,
                                          cfg.hc_eps, cfg.rms_eps)
        h = rmsnorm(hc_collapse(x, pre), self.W[f"{p}.{br}_norm.weight"], cfg.rms_eps)
        return h, (post, comb)

    def _residual(self, x, a, hc):
        if hc is None:
            return x + a
        return hc_post(x, a, hc[0], hc[1])

    def _attention(self, p: str, layer: int, h: torch.Tensor, pos: torch.Tensor, s: OracleSession,
                   src_prefix: Optional[str], idx_layer_is_source: bool, draft: bool) -> torch.Tensor:
        cfg, W = self.cfg, self.W
        T = h.shape[0]
        Dh = cfg.head_dim
        h = self._aq(h)
        if cfg.q_lora_rank:
            qa = rmsnorm(h @ W[f"{p}.attn.wq_a.weight"].t(), W[f"{p}.attn.q_norm.weight"], cfg.rms_eps)
            q = qa @ W[f"{p}.attn.wq_b.weight"].t()
        else:
            q = h @ W[f"{p}.attn.wq.weight"].t()
        Hl = q.shape[-1] // Dh
        q = apply_rope(q.reshape(T, Hl, Dh), pos, self.freqs)
        kv = rmsnorm(h @ W[f"{p}.attn.wkv.weight"].t(), W[f"{p}.attn.kv_norm.weight"], cfg.rms_eps)
        kv = apply_rope(kv, pos, self.freqs)
        win = s.buf(s.window, p, s.max_tokens, Dh)
        p0, p1 = int(pos[0]), int(pos[-1]) + 1
        if cfg.kv_quant == "v41":       # what the window cache actually stores
            kv = codecs.kv_v41_decode(codecs.kv_v41_encode(kv.cpu()), Dh).to(kv.device)
        win[p0:p1] = kv.to(win.dtype)

        # compressor at source layers --------------------------------------------------
        r = cfg.compress_ratio if draft else cfg.ratio_of(layer)     # of the stream this layer writes or reads
        if (not draft) and layer in cfg.kv_source_layers:
            C = Dh + cfg.index_dim
            cv = h @ W[f"{p}.attn.compressor.wkv.weight"].t()
            cg = h @ W[f"{p}.attn.compressor.wgate.weight"].t()
            car = s.buf(s.carry, p, s.max_tokens, 2, C)
            car[p0:p1, 0], car[p0:p1, 1] = cv.to(car.dtype), cg.to(car.dtype)
            maxC = s.max_tokens // r + 1
            comp = s.buf(s.comp, p, maxC, Dh)
            keys = s.buf(s.keys, p, maxC, cfg.index_dim)
            # group g completes at position (g+1)*r-1; take those completing inside [p0, p1)
            gs = list(range(-(-(p0 + 1) // r) - 1, p1 // r))
            if gs:
                gi = torch.tensor(gs, device=h.device)
                rows = (gi[:, None] * r + torch.arange(r, device=h.device)[None, :])      # [G, r]
                v, gt = car[rows, 0].to(torch.float32), car[rows, 1].to(torch.float32)   # [G,r,C]
                wgt = torch.softmax(gt, dim=1)
                pooled = (v * wgt).sum(1)                                                # [G, C]
                ck = rmsnorm(pooled[:, :Dh], W[f"{p}.attn.compressor.norm.weight"], cfg.rms_eps)
                ck = apply_rope(ck, gi, self.cfreqs)
                ik = pooled[:, Dh:]
                if cfg.kv_quant == "v41":
                    ck = codecs.kv_v41fp4_decode(codecs.kv_v41fp4_encode(ck.cpu()), Dh).to(ck.device)
                    ik = codecs.index_key_decode(codecs.index_key_encode(ik.cpu()), cfg.index_dim).to(ik.device)
                comp[gi] = ck.to(comp.dtype)
                keys[gi] = ik.to(keys.dtype)

        # indexer ----------------------------------------------------------------------
        sel = None
        if src_prefix is not None:
            comp = s.comp[src_prefix]
            nvalid = (pos + 1) // r                                                      # [T]
            if idx_layer_is_source:
                keys = s.keys[src_prefix]
                Hi, Di = cfg.index_heads, cfg.index_dim
                qi = (h @ W[f"{p}.attn.indexer.wq.weight"].t()).reshape(T, Hi, Di)
                if cfg.kv_quant == "v41":
                    qi = codecs.bf16_round(qi)
                wi = h @ W[f"{p}.attn.indexer.weights_proj.weight"].t()                  # [T, Hi]
                nmax = int(nvalid.max())
                if nmax > 0:
                    sc = torch.relu(torch.einsum("thd,cd->thc", qi.to(torch.float32),
                                                 keys[:nmax].to(torch.float32)))
                    score = (sc * wi.to(torch.float32)[:, :, None]).sum(1)               # [T, nmax]
                    cidx = torch.arange(nmax, device=h.device)[None, :]
                    score = torch.where(cidx < nvalid[:, None], score,
                                        torch.full_like(score, float("-inf")))
                    k = min(cfg.index_topk, nmax)
                    # exact top-k; ties at the cut by ascending position (stable sort)
                    order = torch.sort(score, dim=-1, descending=True, stable=True).indices[:, :k]
                    okm = torch.gather(score, 1, order) > float("-inf")
                    ids = torch.where(okm, order, torch.full_like(order, -1))
                    # ascending position, invalid (-1) last
                    skey = torch.where(ids >= 0, ids, torch.full_like(ids, 1 << 30))
                    sel = torch.sort(skey, -1).values
                    sel = torch.where(sel >= (1 << 30), torch.full_like(sel, -1), sel)
                else:
                    sel = torch.full((T, 0), -1, dtype=torch.long, device=h.device)
                self.last_selection[layer] = sel
            else:
                sel = self.last_selection[cfg.index_source_of(layer)]

        # attention --------------------------------------------------------------------
        scale = 1.0 / math.sqrt(Dh)
        w0 = max(0, p0 - cfg.window + 1)
        kwin = win[w0:p1].to(torch.float32)                                             # [Kw, Dh]
        kpos = torch.arange(w0, p1, device=h.device)
        logit = torch.einsum("thd,kd->thk", q.to(torch.float32), kwin) * scale
        vis = (kpos[None, :] <= pos[:, None]) & (kpos[None, :] > pos[:, None] - cfg.window)
        logit = torch.where(vis[:, None, :], logit, torch.full_like(logit, float("-inf")))
        vals = [kwin[None].expand(T, -1, -1)]
        logits = [logit]
        if sel is not None and sel.shape[1] > 0:
            ksel = comp[torch.clamp(sel, min=0)].to(torch.float32)                      # [T, k, Dh]
            ls = torch.einsum("thd,tkd->thk", q.to(torch.float32), ksel) * scale
            ls = torch.where((sel >= 0)[:, None, :], ls, torch.full_like(ls, float("-inf")))
            logits.append(ls)
            vals.append(ksel)
        if cfg.attn_sink:
            sink = W[f"{p}.attn.attn_sink"].to(torch.float32)
            logits.append(sink[None, :, None].expand(T, Hl, 1))
        L = torch.cat(logits, -1)
        P = torch.softmax(L, -1)
        o = torch.einsum("thk,kd->thd", P[..., : kwin.shape[0]], kwin)
        if len(vals) > 1:
            k0 = kwin.shape[0]
            o = o + torch.einsum("thk,tkd->thd", P[..., k0:k0 + vals[1].shape[1]], vals[1])
        o = apply_rope(o, pos, self.freqs, inverse=True).to(self.dtype)
        if cfg.o_groups:
            G = cfg.o_groups // self.world
            per = Hl * Dh // G
            wa = W[f"{p}.attn.wo_a.weight"].reshape(G, cfg.o_lora_rank, per)
            mid = torch.einsum("tgp,grp->tgr", o.reshape(T, G, per), wa).reshape(T, G * cfg.o_lora_rank)
            out = mid @ W[f"{p}.attn.wo_b.weight"].t()
        else:
            out = self._aq(o.reshape(T, Hl * Dh)) @ W[f"{p}.attn.wo.weight"].t()
        return self.comm.all_reduce(out)

    def _ffn(self, p: str, h: torch.Tensor, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg, W = self.cfg, self.W
        T = h.shape[0]
        image_rows = (tokens.to(h.device) == cfg.image_token) if (tokens is not None and cfg.router_bias_vl) else None
        ids, wts = route(h @ W[f"{p}.ffn.gate.weight"].t(), cfg, W.get(f"{p}.ffn.gate.bias"),
                         W.get(f"{p}.ffn.gate.bias_vl"), image_rows)
        w1, w3, w2 = (W[f"{p}.ffn.experts.{n}.weight"] for n in ("w1", "w3", "w2"))
        y = torch.zeros(T, cfg.hidden, dtype=torch.float32, device=h.device)
        El = w1.shape[0]
        e0 = self.rank * El if (self.moe_parallel == "ep" and self.world > 1) else 0
        h = self._aq(h)
        # fixed top-k order accumulation (kernels/ffn_sum_shared.cuh:7-33)
        for j in range(cfg.topk):
            for e in range(El):
                m = ids[:, j] == (e + e0)
                if m.any():
                    hh = self._aq_mx(h[m])
                    a = self._aq_mx(self._aq(swiglu(hh @ w1[e].t(), hh @ w3[e].t(), cfg.swiglu_limit)))
                    y[m] += (a @ w2[e].t()).to(torch.float32) * wts[m, j:j + 1]
        if cfg.n_shared:
            a = self._aq(swiglu(h @ W[f"{p}.ffn.shared_experts.w1.weight"].t(),
                                h @ W[f"{p}.ffn.shared_experts.w3.weight"].t(), cfg.swiglu_limit))
            y = y + (a @ W[f"{p}.ffn.shared_experts.w2.weight"].t()).to(torch.float32)
        return self.comm.all_reduce(y.to(self.dtype))

    def _engram(self, p: str, e: int, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Hashed n-gram memory in front of an Engram layer: gather the rows named by ``ids`` [T, n]
        from table e (row-sharded tables: every rank contributes the rows it owns, summed), project
        them to (copies + 1) x hidden and gate them into the residual copies
        (reference: src/engram_gpu.rs; kernels/core.cu:952 ca_engram_gate)."""
        from . import engram as EG
        cfg, W = self.cfg, self.W
        table = W[f"engram.{e}.table"]
        T = ids.shape[0]
        rows = table[ids.reshape(-1)].reshape(T, -1).to(torch.float32)
        if cfg.kv_quant == "v41":
            rows = codecs.bf16_round(rows)
        xm = x if cfg.hc_mult > 1 else x[:, None, :]
        out = EG.apply_reference(xm.to(torch.float32), rows, W[f"{p}.engram.wkv.weight"].to(torch.float32),
                                 W[f"{p}.engram.q_weight"].to(torch.float32),
                                 W[f"{p}.engram.k_weight"].to(torch.float32), cfg.rms_eps)
        return out if cfg.hc_mult > 1 else out[:, 0]

    def _layer(self, p, layer, x, pos, s, draft=False, engram_ids=None, tokens=None):
        cfg = self.cfg
        src = cfg.kv_source_of(layer) if not draft else -1
        src_prefix = f"layers.{src}" if src >= 0 else None
        if engram_ids is not None and not draft and layer in cfg.engram.layers:
            e = cfg.engram.layers.index(layer)
            x = self._engram(p, e, x, engram_ids[:, e])
        h, hc = self._boundary(x, p, "attn")
        a = self._attention(p, layer, h.to(self.dtype), pos, s, src_prefix,
                            (not draft) and layer in cfg.index_source_layers, draft)
        x = self._residual(x, a, hc)
        h, hc = self._boundary(x, p, "ffn")
        f = self._ffn(p, h.to(self.dtype), None if draft else tokens)
        return self._residual(x, f, hc)

    def head(self, x: torch.Tensor, subset: bool = False) -> torch.Tensor:
        """final (hc combine) -> RMSNorm -> vocabulary head -> gathered fp32 logits
        (reference: src/model_io.rs:21,704)."""
        cfg, W = self.cfg, self.W
        if cfg.hc_mult > 1:
            T = x.shape[0]
            flat = x.reshape(T, -1).to(torch.float32)
            inv = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
            m = (flat @ W["hc_head_fn"].t()) * inv
            pre = torch.sigmoid(m * W["hc_head_scale"][0] + W["hc_head_base"]) + cfg.hc_eps
            x = hc_collapse(x, pre)
        hn = rmsnorm(x, W["norm.weight"], cfg.rms_eps).to(self.dtype)
        if subset:
            # the drafter's subset head: logits only for the subset's tokens, -inf elsewhere
            # (single rank; "mtp.head_subset.weight" holds what a 4-bit copy of those rows decodes to)
            assert self.world == 1, "the subset head is built for one rank"
            ids = W["mtp.head_subset.ids"].to(hn.device)
            w = W["mtp.head_subset.weight"] if "mtp.head_subset.weight" in W else W["head.weight"][ids]
            logits = torch.full((hn.shape[0], cfg.vocab), float("-inf"), dtype=torch.float32, device=hn.device)
            # the 4-bit head multiplies MXFP8 activations (e4m3, one UE8M0 scale per 32 inputs)
            q8, s8 = codecs.mxfp8_quant(hn.float().cpu(), 32)
            hq = codecs.mxfp8_dequant(q8, s8, 32).to(hn.device, torch.float32)
            logits[:, ids] = hq @ w.to(torch.float32).t()
            return logits
        logits = (hn @ W["head.weight"].t()).to(torch.float32)
        return self.comm.all_gather(logits, dim=1)

    # -- public ----------------------------------------------------------
    def forward(self, tokens: torch.Tensor, s: OracleSession, start: Optional[int] = None,
                need_logits: bool = True, commit: bool = True,
                x_patch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Optional[torch.Tensor]:
        """Run ``tokens`` at positions ``start..start+T`` (default: append after the committed
        length).  Returns logits [T, vocab] (fp32).  ``commit=False`` leaves ``s.length`` alone so
        that a verification round can accept a prefix with ``s.length = ...`` afterwards."""
        cfg = self.cfg
        start = s.length if start is None else start
        T = tokens.numel()
        assert start + T <= s.max_tokens, "conversation exceeds its region"
        pos = torch.arange(start, start + T, device=tokens.device)
        x = self.embed(tokens)
        if x_patch is not None:
            # rows that stand for image tokens take the vision tower's features instead
            x = x.clone()
            x[x_patch[0].long()] = x_patch[1].to(x.dtype)
        if cfg.hc_mult > 1:
            x = x[:, None, :].expand(T, cfg.hc_mult, cfg.hidden).contiguous()      # core.cu:536
        eg_ids = None
        if cfg.engram is not None and cfg.engram.layers:
            # token ids are kept by position so that the n-gram hashes of speculative rows can be
            # recomputed after a rejection without any history rollback
            from . import engram as EG
            if s.token_at is None:
                s.token_at = torch.zeros(s.max_tokens, dtype=torch.long)
            s.token_at[start:start + T] = tokens.to("cpu", torch.long)
            md = EG.metadata_for(cfg)
            prev = s.token_at[max(0, start - (md.ngram - 1)):start].tolist()
            eg_ids = torch.from_numpy(EG.hash_positions(md, prev, tokens.tolist(), start).astype("int64")
                                      ).to(tokens.device)
        for l in range(cfg.n_layers):
            x = self._layer(f"layers.{l}", l, x, pos, s, engram_ids=eg_ids, tokens=tokens)
        self.last_hidden = x
        if commit:
            s.length = start + T
        return self.head(x) if need_logits else None

    def draft_forward(self, tokens: torch.Tensor, hidden: torch.Tensor, s: OracleSession,
                      start: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Draft head: combine the embedding of each token with the target's hidden state of the
        previous position, run the draft layer(s), return (logits, new hidden)
        (reference conditioning: src/dspark_conditioning.rs; main_proj [d,3d])."""
        cfg, W = self.cfg, self.W
        T = tokens.numel()
        pos = torch.arange(start, start + T, device=tokens.device)
        e = rmsnorm(self.embed(tokens), W["mtp.0.enorm.weight"], cfg.rms_eps)
        hsrc = hidden if cfg.hc_mult == 1 else hidden.mean(1)
        hh = rmsnorm(hsrc, W["mtp.0.hnorm.weight"], cfg.rms_eps)
        x = (torch.cat([e, hh], -1).to(self.dtype) @ W["mtp.0.main_proj.weight"].t())
        if cfg.hc_mult > 1:
            x = x[:, None, :].expand(T, cfg.hc_mult, cfg.hidden).contiguous()
        for j in range(cfg.draft.layers):
            x = self._layer(f"mtp.{j}", cfg.n_layers + j, x, pos, s, draft=True)
        logits = self.head(x, subset=bool(cfg.draft.subset_rows))
        if cfg.draft.markov_rank:
            # Markov correction: a rank-r bigram term from the token each row was fed
            # (reference: src/dspark_markov.rs:886-971, kernels/core.cu:1110-1122)
            mk = f"mtp.{cfg.draft.layers - 1}.markov_head"
            lat = W[f"{mk}.embed.weight"][tokens.long()].to(self.dtype)
            bias = (lat @ W[f"{mk}.head.weight"].t()).to(torch.float32)
            logits = logits + self.comm.all_gather(bias, dim=1)
        return logits, x


def _draft_confidence(self, tokens: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Confidence of the proposal each draft row is about to make, [T] in (0, 1): a sigmoid over
    [residual stream of the draft pass before the final norm ; Markov embedding of the token the row
    was fed] (reference: kernels/dspark_confidence_fused.cuh; weights widened to fp32)."""
    cfg, W = self.cfg, self.W
    if cfg.hc_mult > 1:
        T = x.shape[0]
        flat = x.reshape(T, -1).to(torch.float32)
        inv = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        pre = torch.sigmoid((flat @ W["hc_head_fn"].t()) * inv * W["hc_head_scale"][0] + W["hc_head_base"]) + cfg.hc_eps
        x = hc_collapse(x, pre)
    feat = x.to(torch.bfloat16).to(torch.float32)
    if cfg.draft.markov_rank:
        lat = W[f"mtp.{cfg.draft.layers - 1}.markov_head.embed.weight"][tokens.long()]
        feat = torch.cat([feat, lat.to(torch.bfloat16).to(torch.float32)], -1)
    w = W[f"mtp.{cfg.draft.layers - 1}.confidence_head.proj.weight"].to(torch.bfloat16).to(torch.float32)
    return torch.sigmoid(feat @ w.reshape(-1))


OracleModel.draft_confidence = _draft_confidence


def greedy_generate(model: OracleModel, prompts: Sequence[torch.Tensor], steps: int
                    ) -> Tuple[List[List[int]], List[torch.Tensor]]:
    """Prefill every prompt then decode greedily; returns tokens and the per-step logits
    (the plumbing-check workload: batch 2, 64 prompt tokens, 16 greedy steps)."""
    sessions = [model.new_session(int(p.numel()) + steps + 1) for p in prompts]
    outs: List[List[int]] = [[] for _ in prompts]
    all_logits: List[torch.Tensor] = []
    last = []
    for p, s in zip(prompts, sessions):
        lg = model.forward(p, s)
        all_logits.append(lg[-1:].clone())
        last.append(int(lg[-1].argmax()))
    for _ in range(steps):
        step_logits = []
        for i, s in enumerate(sessions):
            outs[i].append(last[i])
            lg = model.forward(torch.tensor([last[i]], device=prompts[i].device), s)
            step_logits.append(lg)
            last[i] = int(lg[-1].argmax())
        all_logits.append(torch.cat(step_logits, 0))
    return outs, all_logits
