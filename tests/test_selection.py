"""The flash-level selection logic of the reference (UNetProtocol.swift:8-19, 650-661; LocalImageGenerator.swift:
3882-3891) mirrored on the host, and the equivalence of its levels on the GPU."""
import pytest
import torch

from oracle import sdpa_oracle as so


def test_selection_rules(dtattn):
    from dtattn import selection as sel
    assert sel.uses_flash_attention(0) is sel.UseFlashAttention.none
    assert sel.uses_flash_attention(1, is_mqa_supported=False) is sel.UseFlashAttention.sdpa      # CUDA hosts
    assert sel.uses_flash_attention(1, is_mqa_supported=True) is sel.UseFlashAttention.quantized  # Metal only
    assert sel.uses_flash_attention(2, True) is sel.UseFlashAttention.sdpa
    L = sel.FlashAttentionLevel
    assert sel.value_or(sel.UseFlashAttention.none, L.scaleMerged) is L.none
    assert sel.value_or(sel.UseFlashAttention.quantized, L.scale1) is L.quantized
    assert sel.value_or(sel.UseFlashAttention.sdpa, L.scale1) is L.scale1
    assert sel.MODEL_DEFAULT_LEVEL["wan"] is L.scale1 and sel.MODEL_DEFAULT_LEVEL["flux1"] is L.scaleMerged
    op, qf = sel.attention_for_level(L.scale1, 64)
    assert op.scale == 1.0 and abs(qf - 0.125) < 1e-12
    op, qf = sel.attention_for_level(L.scaleMerged, 64, upcast_attention=True)
    assert abs(op.scale - 0.125) < 1e-12 and qf == 1.0 and op.flags == dtattn.GEMMFlag.NONE
    for lvl in (L.none, L.quantized):
        with pytest.raises(NotImplementedError):
            sel.attention_for_level(lvl, 64)
    assert sel.instruction_count(1, 24, 128, 4608, 4608) == so.instruction_count(1, 24, 128, 4608, 4608)


@pytest.mark.gpu
def test_levels_agree_on_gpu(dtattn):
    """.scale1 (Q pre-multiplied) and .scaleMerged give the same attention up to the rounding of the scaled Q."""
    from dtattn import selection as sel
    B, S, H, D = 1, 384, 4, 128
    q = so.seeded_normal((B, S, H, D), 5).to(torch.bfloat16).cuda()
    k = so.seeded_normal((B, S, H, D), 6).to(torch.bfloat16).cuda()
    v = so.seeded_normal((B, S, H, D), 7).to(torch.bfloat16).cuda()
    outs = []
    for lvl in (sel.FlashAttentionLevel.scale1, sel.FlashAttentionLevel.scaleMerged):
        op, qf = sel.attention_for_level(lvl, D)
        outs.append(op((q.float() * qf).to(torch.bfloat16), k, v).float().cpu())
    ref = so.sdpa_explicit(q.cpu(), k.cpu(), v.cpu(), D ** -0.5)
    for o in outs:
        mx, mean = so.error_stats(o, ref)
        assert mx <= 2e-3 + 2 ** -8 * float(ref.abs().max()) and mean <= 4e-4
