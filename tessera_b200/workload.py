"""The projection set of one decoded token of the 27B-class hybrid model.

Shapes follow the synthetic configuration the benchmark is quoted on: hidden
5120, 64 layers, SwiGLU FFN 17408, vocabulary 151936; every 4th layer is GQA
attention (24 query heads, 4 KV heads, head_dim 256, fused query+gate
projection), the others are gated delta-rule linear-attention layers (48
value heads of 128, 16 key heads of 128).  Weight types are a Q4_K_M-style
mix: Q4_K everywhere except Q6_K for ffn_down and attn_v of every other layer
and for the output head.  Tensor names and the column/row split follow the
reference's tensor-parallel map (src/models/qwen3_5/weights.cpp:131-165 of the
reference); the linear-attention projections, which the reference leaves
replicated, are split here too (column: attn_qkv, attn_gate, ssm_beta,
ssm_alpha; row: ssm_out) so that every rank streams 1/world of the weights.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

HIDDEN = 5120
LAYERS = 64
FFN = 17408
VOCAB = 151936
FULL_ATTENTION_INTERVAL = 4
Q_HEADS, KV_HEADS, HEAD_DIM = 24, 4, 256
SSM_INNER = 6144            # 48 value heads x 128
SSM_QKV = 2 * 16 * 128 + SSM_INNER  # 16 key heads x 128 for q and k, plus v
SSM_HEADS = 48

COLUMN, ROW = "column", "row"


@dataclass(frozen=True)
class Projection:
    name: str
    layer: int
    dtype: str      # "q4k" | "q6k"
    n: int          # output features (rows of W)
    k: int          # input features
    kind: str       # COLUMN: split n across ranks; ROW: split k, then all-reduce
    act: str        # which activation buffer feeds it


def block_bytes(dtype: str) -> int:
    return {"q4k": 144, "q6k": 210}[dtype]


def weight_bytes(dtype: str, n: int, k: int) -> int:
    return n * (k // 256) * block_bytes(dtype)


def decode_projections() -> List[Projection]:
    out: List[Projection] = []
    for layer in range(LAYERS):
        mixed = "q6k" if layer % 2 == 1 else "q4k"
        if layer % FULL_ATTENTION_INTERVAL == FULL_ATTENTION_INTERVAL - 1:
            out += [
                Projection("attn_q", layer, "q4k", Q_HEADS * HEAD_DIM * 2, HIDDEN, COLUMN, "x"),
                Projection("attn_k", layer, "q4k", KV_HEADS * HEAD_DIM, HIDDEN, COLUMN, "x"),
                Projection("attn_v", layer, mixed, KV_HEADS * HEAD_DIM, HIDDEN, COLUMN, "x"),
                Projection("attn_output", layer, "q4k", HIDDEN, Q_HEADS * HEAD_DIM, ROW, "attn"),
            ]
        else:
            out += [
                Projection("attn_qkv", layer, "q4k", SSM_QKV, HIDDEN, COLUMN, "x"),
                Projection("attn_gate", layer, "q4k", SSM_INNER, HIDDEN, COLUMN, "x"),
                Projection("ssm_beta", layer, "q4k", SSM_HEADS, HIDDEN, COLUMN, "x"),
                Projection("ssm_alpha", layer, "q4k", SSM_HEADS, HIDDEN, COLUMN, "x"),
                Projection("ssm_out", layer, "q4k", HIDDEN, SSM_INNER, ROW, "attn"),
            ]
        out += [
            Projection("ffn_gate", layer, "q4k", FFN, HIDDEN, COLUMN, "x"),
            Projection("ffn_up", layer, "q4k", FFN, HIDDEN, COLUMN, "x"),
            Projection("ffn_down", layer, mixed, HIDDEN, FFN, ROW, "ffn"),
        ]
    out.append(Projection("output", LAYERS, "q6k", VOCAB, HIDDEN, COLUMN, "x"))
    return out


def row_blocks(dtype: str, blocks: int, rank: int, world: int):
    """Block range [b0, b1) of a row-parallel projection's k on this rank: blocks*rank/world
    rounded down, the rule of the library's slicer (tsr_slice_shape) -- counted in units of
    four blocks for Q6_K where the count allows it, because rows of 210-byte blocks are 8-byte
    aligned (what the staged Q6_K kernel needs) only when they hold a multiple of four."""
    unit = 4 if (dtype == "q6k" and blocks % 4 == 0 and blocks // 4 >= world) else 1
    units = blocks // unit
    return unit * (units * rank // world), unit * (units * (rank + 1) // world)


def shard(p: Projection, rank: int, world: int):
    """(n_local, k_local) of this rank.  Column: rows [n*rank/world, n*(rank+1)/world), except
    ffn_gate / ffn_up, whose rows are the k range of the layer's ffn_down on this rank (the
    rank's slice of the FFN activation is produced where it is consumed).  Row: whole
    256-element blocks, see row_blocks: 68 blocks on 8 ranks gives ranks of 8 and 9 blocks
    (Q4_K) or of 8 and 12 (Q6_K)."""
    if world == 1:
        return p.n, p.k
    if p.name in ("ffn_gate", "ffn_up"):
        down = "q6k" if p.layer % 2 == 1 else "q4k"
        b0, b1 = row_blocks(down, FFN // 256, rank, world)
        return (b1 - b0) * 256, p.k
    if p.kind == COLUMN:
        return p.n * (rank + 1) // world - p.n * rank // world, p.k
    b0, b1 = row_blocks(p.dtype, p.k // 256, rank, world)
    return p.n, (b1 - b0) * 256


def total_weight_bytes(rank: int = 0, world: int = 1) -> int:
    total = 0
    for p in decode_projections():
        n, k = shard(p, rank, world)
        total += weight_bytes(p.dtype, n, k)
    return total


def total_parameters() -> int:
    return sum(p.n * p.k for p in decode_projections())
