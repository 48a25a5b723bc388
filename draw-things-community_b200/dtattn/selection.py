"""Host-side mirror of how the reference decides *which* attention a model is built with.

Reference: `UseFlashAttention` / `FlashAttentionLevel` (Libraries/SwiftDiffusion/Sources/Models/
UNetProtocol.swift:8-19), `valueOr` (UNetProtocol.swift:650-661) and the choice in
Libraries/LocalImageGenerator/Sources/LocalImageGenerator.swift:3882-3891.  With this library every level maps to
the same operator; the levels only differ in where the 1/sqrt(k) factor is applied.
"""
from __future__ import annotations

import enum
import math

from . import GEMMFlag, ScaledDotProductAttention


class UseFlashAttention(enum.Enum):
    none = 0       # --no-flash-attention: the explicit matmul/softmax graph
    sdpa = 1
    quantized = 2  # only when DeviceCapability.isMQASupported, i.e. on Metal


class FlashAttentionLevel(enum.Enum):
    none = 0
    scale1 = 1        # Q is multiplied by 1/sqrt(k) before the operator, which gets scale 1
    scaleMerged = 2   # the operator gets scale 1/sqrt(k)
    quantized = 3


def uses_flash_attention(mfa_enabled: int, is_mqa_supported: bool = False) -> UseFlashAttention:
    """LocalImageGenerator.swift:3882-3891.  Off Metal `isMFAEnabled` is 1 and `isMQASupported` is false
    (DeviceCapability.swift:117-134), so a CUDA host always lands on `.sdpa`."""
    if mfa_enabled == 0:
        return UseFlashAttention.none
    if mfa_enabled == 1:
        return UseFlashAttention.quantized if is_mqa_supported else UseFlashAttention.sdpa
    return UseFlashAttention.sdpa


def value_or(uses: UseFlashAttention, value: FlashAttentionLevel) -> FlashAttentionLevel:
    """UNetProtocol.swift:650-661: the model's own default level applies only under `.sdpa`."""
    if uses is UseFlashAttention.none:
        return FlashAttentionLevel.none
    if uses is UseFlashAttention.quantized:
        return FlashAttentionLevel.quantized
    return value


# per-model defaults (UNetProtocol.swift:773, 869, 1185, 1458)
MODEL_DEFAULT_LEVEL = {"sd15": FlashAttentionLevel.scaleMerged, "sdxl": FlashAttentionLevel.scaleMerged,
                       "flux1": FlashAttentionLevel.scaleMerged, "wan": FlashAttentionLevel.scale1}


def attention_for_level(level: FlashAttentionLevel, head_dim: int, upcast_attention: bool = False, **kw):
    """(operator, factor to multiply the queries with before the call) for a level, as the model builders do
    (UNet.swift:136-153, Flux1.swift:224-232).  `.none` and `.quantized` have no operator here: the first is the
    explicit graph (this repository keeps it only as the test oracle), the second is a Metal-only level."""
    flags = [] if upcast_attention else [GEMMFlag.Float16]
    if level is FlashAttentionLevel.scale1:
        return ScaledDotProductAttention(scale=1.0, flags=flags, **kw), 1.0 / math.sqrt(head_dim)
    if level is FlashAttentionLevel.scaleMerged:
        return ScaledDotProductAttention(scale=1.0 / math.sqrt(head_dim), flags=flags, **kw), 1.0
    raise NotImplementedError(f"FlashAttentionLevel.{level.name} has no operator in this library")


def instruction_count(batch: int, heads: int, head_dim: int, seq_a: int, seq_b: int) -> int:
    """ScaledDotProductAttentionInstructionCount (Models/InstructionCount/InstructionCount.swift:9-17): the
    reference's cost model for the operator, in FMA instructions."""
    assert min(batch, heads, head_dim, seq_a, seq_b) >= 0
    return batch * heads * (2 * head_dim + 5) * seq_a * seq_b
