"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped library imports this file: only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may use it, and only as the checker or the
timed CPU baseline.

PARITY UNPINNED for the attention arithmetic: the reference tree (drawthingsai/draw-things-community)
holds no attention kernel and no test that pins attention numerics.  The arithmetic lives in two
un-vendored dependencies, liuliu/s4nnc @ e96e31183d6ed5811c68eeb8dbe4f6215ef5fc95 and liuliu/ccv @
023a9a894445493d8475711c0160be0bac8e6620 (WORKSPACE.linux:100-116, Package.swift:15-19).  What this file
restates is the operator's *semantic specification* that the reference spells out itself, in its explicit
(non-flash) model graphs, plus the pieces around it that the tree does contain:

  * explicit attention graph  Libraries/SwiftDiffusion/Sources/Models/UNet.swift:217-265,
                              Flux1.swift:192-223
  * scale conventions         Flux1.swift:224-232 (.scale1 / .scaleMerged), Wan.swift:95-103
  * grouped KV heads          Llama.swift:74-96
  * causal over a KV cache    Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:183-196
  * additive mask             CLIPTextModel.swift:57-70, TextEncoder.swift:151-158
  * Flux RoPE table + cmul    Flux1.swift:5-72, 187-188
  * seeded N(0,1)             Random/TorchRandomSource.swift:25-138  (this part IS pinned: the reference
                              states it reproduces torch's CPU randn, and tests/test_oracle.py checks this
                              restatement bit-for-bit against torch.randn)
  * cost model                Models/InstructionCount/InstructionCount.swift:9-17
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

# --------------------------------------------------------------------------------------------------
# The operator
# --------------------------------------------------------------------------------------------------

MASK_FILL = -torch.finfo(torch.float32).max  # the reference fills with -greatestFiniteMagnitude (TextEncoder.swift:147)


def sdpa_explicit(q, k, v, scale, is_causal=False, mask=None, *, compute_dtype=torch.float32,
                  p_dtype=None, return_lse=False, sinks=None, sliding_window=0):
    """softmax(scale * Q K^T [+ mask]) V written the way the reference's explicit graphs write it.

    q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] (BSHD).  Steps, with the reference line each follows:
      1. transposed(1,2) to BHSD                                    UNet.swift:218-221
      2. queries pre-multiplied by the scale                        UNet.swift:219 (scale folded here)
      3. grouped heads: query heads [i*G,(i+1)*G) use KV head i     Llama.swift:74-86
      4. Matmul(transposeB) -> scores [B,H,Sq,Sk]                   UNet.swift:254
      5. + additive mask                                            CLIPTextModel.swift:62
      6. causal: key j visible to query i iff j <= i + (Sk - Sq)    Qwen3_5.swift:183-196 (a single new
         query over T cached rows sees all T rows)
      7. softmax over the last axis                                 UNet.swift:256
      8. optional cast of P to V's dtype (upcastAttention)          UNet.swift:257-259
      9. P * V, transposed back to BSHD                             UNet.swift:261-262
    compute_dtype float64 gives the high-precision variant used to bound the fp32 oracle's own error.
    Operator variants (DeepSeek4.swift:482-493 builds the node with hasAttentionSinks and slidingWindow; their
    arithmetic is in the absent back end, so the usual definitions are restated): `sinks` [Hq] is one extra
    unscaled score column per head that takes part in the softmax and has no value row; `sliding_window` W hides
    keys j <= i + (Sk - Sq) - W.
    """
    B, Sq, Hq, D = q.shape
    _, Sk, Hkv, _ = k.shape
    assert Hq % Hkv == 0
    G = Hq // Hkv
    qf = q.to(compute_dtype).permute(0, 2, 1, 3) * scale  # [B,Hq,Sq,D]
    kf = k.to(compute_dtype).permute(0, 2, 1, 3)          # [B,Hkv,Sk,D]
    vf = v.to(compute_dtype).permute(0, 2, 1, 3)
    if G > 1:
        kf = kf.repeat_interleave(G, dim=1)
        vf = vf.repeat_interleave(G, dim=1)
    s = qf @ kf.transpose(-1, -2)                          # [B,Hq,Sq,Sk]
    if mask is not None:
        s = s + mask.to(compute_dtype)
    if is_causal:
        i = torch.arange(Sq).view(Sq, 1)
        j = torch.arange(Sk).view(1, Sk)
        hidden = j > i + (Sk - Sq)
        s = s.masked_fill(hidden, float("-inf"))
    if sliding_window > 0:
        i = torch.arange(Sq).view(Sq, 1)
        j = torch.arange(Sk).view(1, Sk)
        s = s.masked_fill(j <= i + (Sk - Sq) - sliding_window, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    if sinks is not None:
        sk = sinks.to(compute_dtype).view(1, Hq, 1, 1)
        m = torch.maximum(m, sk.expand_as(m))
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(s - m)
    l = e.sum(dim=-1, keepdim=True)
    if sinks is not None:
        l = l + torch.exp(sk - m)
    p = e / torch.where(l > 0, l, torch.ones_like(l))      # a row with no visible key yields zeros
    if p_dtype is not None:
        p = p.to(p_dtype).to(compute_dtype)
    o = (p @ vf).permute(0, 2, 1, 3).contiguous()          # [B,Sq,Hq,D]
    if return_lse:
        lse = (m + torch.log(l)).squeeze(-1)               # [B,Hq,Sq]
        return o, lse
    return o


def sdpa_varlen_explicit(q, k, v, scale, offsets_q, offsets_k, is_causal=False, **kw):
    """Variable-length batch (Qwen3_5VL.swift:428-437: packed rows plus sequence offsets): sequence s attends its
    own rows only.  q [1,sum Sq,Hq,D], k/v [1,sum Sk,Hkv,D]; offsets are Python lists with n_seq + 1 entries."""
    out = torch.zeros(q.shape, dtype=kw.get("compute_dtype", torch.float32))
    for s in range(len(offsets_q) - 1):
        q0, q1, k0, k1 = offsets_q[s], offsets_q[s + 1], offsets_k[s], offsets_k[s + 1]
        if q1 > q0 and k1 > k0:  # queries of a sequence without keys see nothing: zeros, like a fully hidden row
            out[:, q0:q1] = sdpa_explicit(q[:, q0:q1], k[:, k0:k1], v[:, k0:k1], scale, is_causal, **kw)
    return out


def sparse_indexed_explicit(q, k_raw, v_raw, k_comp, v_comp, selected, scale, sinks=None, sliding_window=0,
                            is_causal=True, compute_dtype=torch.float32, return_lse=False):
    """SparseIndexedAttention (DeepSeek4.swift:521-545: queries, raw keys / values, compressed keys / values, selected
    rows [queryLength, selectedRowCount], sinks; isCausal, hasAttentionSinks, slidingWindow).  The operator's arithmetic
    is in the absent back end, so the definition is restated from its use (:1080-1133: the selected rows are what a
    top-k indexer picked, or every compressed row the query may see): query i attends, in ONE softmax, to the raw rows
    j with j <= i + (Sr - Sq) [causal] and j > i + (Sr - Sq) - W [window], and to compressed row c once for every time
    c appears in selected[i]; entries outside [0, Sc) name no row; the sink of the head joins the denominator.
    q [B,Sq,Hq,D], k_raw/v_raw [B,Sr,Hkv,D], k_comp/v_comp [B,Sc,Hkv,D] or None, selected int [B or 1,Sq,n]."""
    B, Sq, Hq, D = q.shape
    Sr, Hkv = k_raw.shape[1], k_raw.shape[2]
    G = Hq // Hkv
    qf = q.to(compute_dtype).permute(0, 2, 1, 3) * scale                                  # [B,Hq,Sq,D]
    kr = k_raw.to(compute_dtype).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)          # [B,Hq,Sr,D]
    vr = v_raw.to(compute_dtype).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s_raw = qf @ kr.transpose(-1, -2)                                                     # [B,Hq,Sq,Sr]
    i = torch.arange(Sq).view(Sq, 1)
    j = torch.arange(Sr).view(1, Sr)
    hidden = torch.zeros(Sq, Sr, dtype=torch.bool)
    if is_causal:
        hidden |= j > i + (Sr - Sq)
    if sliding_window > 0:
        hidden |= j <= i + (Sr - Sq) - sliding_window
    s_raw = s_raw.masked_fill(hidden, float("-inf"))
    parts, values = [s_raw], None
    Sc = 0 if k_comp is None else k_comp.shape[1]
    if Sc > 0 and selected is not None and selected.shape[-1] > 0:
        sel = selected.long().expand(B, Sq, selected.shape[-1])                            # [B,Sq,n]
        ok = (sel >= 0) & (sel < Sc)
        idx = sel.clamp(0, Sc - 1)
        kc = k_comp.to(compute_dtype).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)      # [B,Hq,Sc,D]
        vc = v_comp.to(compute_dtype).permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
        bi = torch.arange(B).view(B, 1, 1, 1)
        hi = torch.arange(Hq).view(1, Hq, 1, 1)
        ksel = kc[bi, hi, idx.unsqueeze(1)]                                                # [B,Hq,Sq,n,D]
        vsel = vc[bi, hi, idx.unsqueeze(1)]
        s_sel = torch.einsum("bhqd,bhqnd->bhqn", qf, ksel).masked_fill(~ok.unsqueeze(1), float("-inf"))
        parts.append(s_sel)
        values = vsel
    s = torch.cat(parts, dim=-1)
    m = s.amax(dim=-1, keepdim=True)
    if sinks is not None:
        sk = sinks.to(compute_dtype).view(1, Hq, 1, 1)
        m = torch.maximum(m, sk.expand_as(m))
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(s - m)
    l = e.sum(dim=-1, keepdim=True)
    if sinks is not None:
        l = l + torch.exp(sk - m)
    p = e / torch.where(l > 0, l, torch.ones_like(l))
    o = p[..., :Sr] @ vr
    if values is not None:
        o = o + torch.einsum("bhqn,bhqnd->bhqd", p[..., Sr:], values)
    o = o.permute(0, 2, 1, 3).contiguous()
    if return_lse:
        return o, (m + torch.log(l)).squeeze(-1)
    return o


def instruction_count(batch, heads, head_dim, seq_a, seq_b):
    """The reference's own cost model for the op, in FMA-instructions (InstructionCount.swift:9-17)."""
    return batch * heads * (2 * head_dim + 5) * seq_a * seq_b


def flops(B, Hq, Sq, Sk, D):
    """Algorithmic FLOPs of one forward call: QK^T and PV, multiply and add each."""
    return 4 * B * Hq * Sq * Sk * D


# --------------------------------------------------------------------------------------------------
# Flux rotary table and complex multiply
# --------------------------------------------------------------------------------------------------

def flux_rope_table(height, width, token_length, channels, heads=1):
    """[1, token_length + height*width, heads, channels] table of interleaved (cos, sin) pairs.

    Restates Flux1RotaryPositionEmbedding (Flux1.swift:5-72) without reference images: the head dim is
    split into three axes of channels/8, 7*channels/16 and 7*channels/16 entries; text tokens sit at
    position (0,0,0), image token (y,x) at (0,y,x); theta_k = pos / 10000^(2k/dim) in float64, stored as
    float32.
    """
    assert channels % 16 == 0
    dim0, dim1 = channels // 8, channels * 7 // 16
    dim2 = dim1
    n = token_length + height * width
    pos = np.zeros((n, 3), dtype=np.float64)
    ys, xs = np.meshgrid(np.arange(height), np.arange(width), indexing="ij")
    pos[token_length:, 1] = ys.reshape(-1)
    pos[token_length:, 2] = xs.reshape(-1)
    rot = np.zeros((n, channels), dtype=np.float32)
    off = 0
    for axis, dim in enumerate((dim0, dim1, dim2)):
        kk = np.arange(dim // 2, dtype=np.float64)
        inv = 1.0 / np.power(10000.0, kk * 2 / dim)
        theta = pos[:, axis:axis + 1] * inv[None, :]
        rot[:, off * 2:(off + dim // 2) * 2:2] = np.cos(theta).astype(np.float32)
        rot[:, off * 2 + 1:(off + dim // 2) * 2:2] = np.sin(theta).astype(np.float32)
        off += dim // 2
    t = torch.from_numpy(rot).view(1, n, 1, channels)
    return t.expand(1, n, heads, channels).contiguous() if heads > 1 else t


def cmul(x, rot):
    """Functional.cmul(left:right:) (Flux1.swift:187-188): adjacent pairs are complex numbers,
    (x0 + i x1) * (cos + i sin)."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = rot[..., 0::2], rot[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out


def qwen_rotary_table(sequence_length, cached_len, head_dim, rotary_dim=None, theta=10_000_000.0):
    """[1, sequence_length, head_dim] interleaved (cos, sin) table, restating Qwen3_5RotaryEmbedding
    (Qwen3_5.swift:85-108): token i sits at position cached_len + i; pair k < rotary_dim/2 holds
    (cos, sin) of position / theta^(2k/rotary_dim) computed in float64; the remaining pairs hold (1, 0), so
    the head dims beyond rotary_dim pass through cmul unchanged (the reference's configs rotate 64 of 256 dims,
    Qwen3_5.swift:59-82)."""
    rotary_dim = head_dim if rotary_dim is None else rotary_dim
    pos = (cached_len + np.arange(sequence_length, dtype=np.float64))[:, None]
    k = np.arange(rotary_dim // 2, dtype=np.float64)[None, :]
    ang = pos / theta ** (k * 2.0 / rotary_dim)
    tab = np.zeros((1, sequence_length, head_dim), dtype=np.float32)
    tab[0, :, 0:rotary_dim:2] = np.cos(ang)
    tab[0, :, 1:rotary_dim:2] = np.sin(ang)
    tab[0, :, rotary_dim::2] = 1.0
    return torch.from_numpy(tab)


def qk_prologue_explicit(x, weight, rotary, eps, dtype, norm_per_token=False, post_scale=1.0):
    """The nodes the reference runs on queries / keys before the attention node, each output rounded to `dtype`:
    RMSNorm over the head dim (Flux1.swift:164-181, Qwen3_5.swift:164-167) or over all h*k channels of a token
    (Wan.swift:86-91), y = x / sqrt(mean(x^2) + eps) * weight in fp32; Functional.cmul with the rotary table
    (Flux1.swift:187-188); multiplication by a constant (Wan.swift:94-97).  x [B,S,H,D] in `dtype` on the CPU;
    weight [D] or [H*D]; rotary broadcastable to x.  Returns a `dtype` tensor."""
    y = x
    if weight is not None:
        xf = x.float()
        if norm_per_token:
            B, S, H, D = x.shape
            flat = xf.reshape(B, S, H * D)
            inv = 1.0 / torch.sqrt(flat.pow(2).mean(dim=-1, keepdim=True) + eps)
            y = ((flat * inv) * weight.float().reshape(1, 1, H * D)).reshape(B, S, H, D).to(dtype)
        else:
            inv = 1.0 / torch.sqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
            y = ((xf * inv) * weight.float()).to(dtype)
    if rotary is not None:
        y = cmul(y.float(), rotary.float()).to(dtype)
    if post_scale != 1.0:
        y = (y.float() * torch.tensor(post_scale, dtype=torch.float32)).to(dtype)
    return y


def decode_step_explicit(q, k_cache, v_cache, k_new, v_new, rotary, scale, cached_len, dtype, q_norm_weight=None,
                         k_norm_weight=None, norm_eps=1e-6, sinks=None, sliding_window=0):
    """The reference's KV-cache step as separate nodes (Qwen3_5.swift:164-196), every node's output rounded to
    `dtype` as a graph of 16-bit tensors does: optional qNorm / kNorm (RMSNorm over the head dim, :164-167), cmul on
    the queries (rotary rows of the last Sq tokens) and on the new keys, new keys / values moved into the cache at row
    cached_len, causal attention over rows [0, cached_len + T_new).  Inputs are `dtype` tensors on the CPU; k_cache /
    v_cache ([B, capacity, Hkv, D]) are updated in place.  Returns fp32 attention output computed from the rounded
    operands."""
    Sq, Tn = q.shape[1], k_new.shape[1]
    rot = None if rotary is None else rotary[:, :, None, :]
    qr = qk_prologue_explicit(q, q_norm_weight, None if rot is None else rot[:, Tn - Sq:], norm_eps, dtype)
    kr = qk_prologue_explicit(k_new, k_norm_weight, rot, norm_eps, dtype)
    k_cache[:, cached_len:cached_len + Tn] = kr
    v_cache[:, cached_len:cached_len + Tn] = v_new
    total = cached_len + Tn
    return sdpa_explicit(qr.to(dtype), k_cache[:, :total], v_cache[:, :total], scale, True, sinks=sinks,
                         sliding_window=sliding_window)


# --------------------------------------------------------------------------------------------------
# Seeded N(0,1): restatement of TorchRandomSource (MT19937 + 16-wide Box-Muller)
# --------------------------------------------------------------------------------------------------

class TorchRandomSourceRestated:
    """MT19937 + Box-Muller generator that the reference says equals torch's CPU randn
    (Random/TorchRandomSource.swift:25-138).  Pure Python: small counts only."""

    def __init__(self, seed):
        key = [0] * 624
        s = seed & 0xFFFFFFFF
        for i in range(624):                       # :28-31
            key[i] = s
            s = (1812433253 * (s ^ (s >> 30)) + i + 1) & 0xFFFFFFFF
        self.key, self.pos, self.next_gauss = key, 624, None

    def _twist(self):                              # :45-57
        key = self.key
        for i in range(624):
            y = (key[i] & 0x80000000) | (key[(i + 1) % 624] & 0x7FFFFFFF)
            key[i] = key[(i + 397) % 624] ^ (y >> 1) ^ (0x9908B0DF if y & 1 else 0)
        self.pos = 0

    def next_u32(self):                            # :37-67
        if self.pos == 624:
            self._twist()
        y = self.key[self.pos]
        self.pos += 1
        y ^= y >> 11
        y ^= (y << 7) & 0x9D2C5680
        y ^= (y << 15) & 0xEFC60000
        y ^= y >> 18
        return y & 0xFFFFFFFF

    def next_float(self):                          # :82-85
        return np.float32(self.next_u32() & 16777215) * np.float32(1.0 / 16777216.0)

    def next_double(self):                         # :69-79
        a = (self.next_u32() << 32) | self.next_u32()
        return (a & 9007199254740991) * (1.0 / 9007199254740992.0)

    def _gauss(self):                              # :88-101
        if self.next_gauss is not None:
            g, self.next_gauss = self.next_gauss, None
            return g
        u1 = self.next_double()
        u2 = 1 - self.next_double()
        radius = math.sqrt(-2.0 * math.log(u2))
        theta = 2.0 * math.pi * u1
        self.next_gauss = radius * math.sin(theta)
        return radius * math.cos(theta)

    def normal_array(self, count):                 # :108-138
        if count < 16:
            return np.array([self._gauss() for _ in range(count)], dtype=np.float32)
        data = np.array([self.next_float() for _ in range(count)], dtype=np.float32)

        def box_muller(i):
            u1 = np.float32(1) - data[i:i + 8]
            u2 = data[i + 8:i + 16].copy()
            radius = np.sqrt(np.float32(-2.0) * np.log(u1))
            theta = np.float32(2.0 * math.pi) * u2
            data[i:i + 8] = radius * np.cos(theta)
            data[i + 8:i + 16] = radius * np.sin(theta)

        for i in range(0, count - 15, 16):
            box_muller(i)
        if count % 16 != 0:
            for i in range(count - 16, count):
                data[i] = self.next_float()
            box_muller(count - 16)
        return data


def seeded_normal(shape, seed, scale=1.0):
    """N(0,1)*scale in fp32 from torch's CPU generator, which TorchRandomSource reproduces."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32) * scale


# --------------------------------------------------------------------------------------------------
# The five benchmark configurations (synthetic inputs with the shapes and distributions asked for)
# --------------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class AttnConfig:
    name: str
    B: int
    Sq: int
    Sk: int
    Hq: int
    Hkv: int
    D: int
    dtype: str          # "f32" | "f16" | "bf16"
    seed: int
    is_causal: bool = False
    input_scale: float = 1.0
    rope_hw: tuple | None = None   # (height, width, text_tokens) -> Flux RoPE pre-applied to q, k

    @property
    def scale(self):
        return 1.0 / math.sqrt(self.D)

    def shrink(self, **kw):
        d = self.__dict__ | kw
        return AttnConfig(**d)


CONFIGS = {
    "sd15_self": AttnConfig("sd15_self", 2, 4096, 4096, 8, 8, 40, "f32", 0),
    "sdxl_cross": AttnConfig("sdxl_cross", 2, 4096, 77, 20, 20, 64, "f16", 1, input_scale=0.5),
    "flux_joint": AttnConfig("flux_joint", 1, 4608, 4608, 24, 24, 128, "bf16", 2, rope_hw=(64, 64, 512)),
    "wan_self": AttnConfig("wan_self", 1, 75600, 75600, 40, 40, 128, "bf16", 3),
    "decode_b1": AttnConfig("decode_b1", 1, 1, 8192, 32, 8, 128, "f16", 4, is_causal=True),
    "decode_b16": AttnConfig("decode_b16", 16, 1, 8192, 32, 8, 128, "f16", 4, is_causal=True),
}

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def make_inputs(cfg: AttnConfig, heads=None):
    """q, k, v in the config's I/O dtype.  Draw order q, k, v from one seeded generator; RoPE (when the
    config has it) is applied in fp32 before the cast, i.e. inputs arrive "RoPE pre-applied".
    `heads=(h0, h1)` draws only that query-head range (and the KV heads it reads) with per-head seeds
    seed*1000+h, so a rank of a head-sharded run generates just its slice."""
    dt = TORCH_DTYPE[cfg.dtype]
    if heads is None:
        g = torch.Generator(device="cpu").manual_seed(cfg.seed)
        q = torch.randn((cfg.B, cfg.Sq, cfg.Hq, cfg.D), generator=g) * cfg.input_scale
        k = torch.randn((cfg.B, cfg.Sk, cfg.Hkv, cfg.D), generator=g) * cfg.input_scale
        v = torch.randn((cfg.B, cfg.Sk, cfg.Hkv, cfg.D), generator=g) * cfg.input_scale
    else:
        h0, h1 = heads
        G = cfg.Hq // cfg.Hkv
        assert h0 % G == 0 and h1 % G == 0
        qs, ks, vs = [], [], []
        for h in range(h0, h1):
            g = torch.Generator(device="cpu").manual_seed(cfg.seed * 1000 + h)
            qs.append(torch.randn((cfg.B, cfg.Sq, 1, cfg.D), generator=g) * cfg.input_scale)
        for h in range(h0 // G, h1 // G):
            g = torch.Generator(device="cpu").manual_seed(cfg.seed * 1000 + 500 + h)
            ks.append(torch.randn((cfg.B, cfg.Sk, 1, cfg.D), generator=g) * cfg.input_scale)
            vs.append(torch.randn((cfg.B, cfg.Sk, 1, cfg.D), generator=g) * cfg.input_scale)
        q, k, v = torch.cat(qs, 2), torch.cat(ks, 2), torch.cat(vs, 2)
    if cfg.rope_hw is not None:
        hh, ww, tt = cfg.rope_hw
        assert tt + hh * ww == cfg.Sq == cfg.Sk
        rot = flux_rope_table(hh, ww, tt, cfg.D)
        q, k = cmul(q, rot), cmul(k, rot)
    return q.to(dt), k.to(dt), v.to(dt)


def error_stats(out, ref):
    """max-abs and mean-abs difference (the two figures the tolerance is stated in)."""
    d = (out.double() - ref.double()).abs()
    return float(d.max()), float(d.mean())


TOL_MAX_ABS = 2e-3    # fp16/bf16 output vs the fp32 oracle
TOL_MEAN_ABS = 2e-4
