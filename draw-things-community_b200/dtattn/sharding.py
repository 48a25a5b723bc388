"""Host-side bookkeeping of the head-sharded mode: which heads a rank owns and how the gathered output is
laid out.  No compute lives here; the exchange and the permute run in libdtattn.so
(dt_sdpa_forward_headsharded, dt_permute_gathered)."""
from __future__ import annotations


def head_range(rank: int, world: int, Hq: int, Hkv: int):
    """(q_begin, q_end, kv_begin, kv_end): rank r owns query heads [r*Hq/world, (r+1)*Hq/world) and the KV
    heads they read.  Query heads [i*G, (i+1)*G) read KV head i (Llama.swift:74-86), so a rank's query range
    must cover whole groups."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if Hq % world:
        raise ValueError(f"{Hq} query heads do not divide over {world} ranks")
    G = Hq // Hkv
    per = Hq // world
    if per % G and G % per:
        raise ValueError("a rank's heads must be whole KV groups or share one KV head")
    q0, q1 = rank * per, (rank + 1) * per
    kv0 = q0 // G
    kv1 = max(kv0 + 1, -(-q1 // G))
    return q0, q1, kv0, kv1


def gathered_to_bshd(gathered, world: int):
    """The layout contract of dt_permute_gathered as a torch expression:
    [world, B, S, Hl, D] (rank-major all-gather order) -> [B, S, world*Hl, D]."""
    w, B, S, Hl, D = gathered.shape
    assert w == world
    return gathered.permute(1, 2, 0, 3, 4).reshape(B, S, world * Hl, D)


def chunk_rows(Sq: int, chunks: int, items_per_row_block: int = 1, sms: int = 148, tile: int = 256):
    """Row ranges dt_sdpa_forward_headsharded cuts the queries into.  The attention kernel is persistent (one
    CTA per SM; a work item is 256 query rows of one head), so a chunk holds a whole number of rounds over the
    SMs: rows per chunk are a multiple of tile * sms / gcd(sms, items_per_row_block), where items_per_row_block
    = batch * local heads."""
    if chunks <= 1:
        return [(0, Sq)]
    import math
    unit = tile * (sms // math.gcd(sms, items_per_row_block))
    per = -(-Sq // chunks)
    per = min(Sq, -(-per // unit) * unit)
    return [(r0, min(Sq, r0 + per)) for r0 in range(0, Sq, per)]


def projection_rows(M: int, world: int, tile: int = 128):
    """Row ownership of the head-sharded output projection (dt_sdpa_forward_projected_headsharded): the M = B*Sq
    flattened output rows are dealt out in blocks of rows_per_rank, a multiple of the GEMM's 128-row tile so that a
    tile has one owner.  Returns (rows_per_rank, [(row_begin, row_end) per rank]); trailing ranks may own nothing."""
    per = -(-M // world)
    rpr = -(-per // tile) * tile
    return rpr, [(min(M, r * rpr), min(M, (r + 1) * rpr)) for r in range(world)]


def weight_slice(weight, rank: int, world: int, Hq: int, D: int):
    """The K-slice of the unify-heads Dense weight [C, Hq*D] that multiplies rank r's heads."""
    per = Hq // world
    return weight[:, rank * per * D:(rank + 1) * per * D]
