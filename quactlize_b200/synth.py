"""Seeded synthetic weights and activations with the shapes and value distributions of the benchmark configurations.

These stand in for real checkpoints: raw GGUF k-quant super-blocks are built byte by byte (fp16 d/dmin ~ |N(0,0.01)|,
sub-scales/sub-mins uniform over their code range, uniform codes), generic per-group weights are uniform codes with
|N(0,0.02)|/7 fp16 scales.  Everything is numpy on the host; callers move tensors to the device.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = {10: 84, 11: 110, 12: 144, 13: 176, 14: 210}
# (d offset, dmin offset or -1) inside a raw block; quactlize/include/gguf_unit_pack.hpp:15-34 in the reference
_HDR = {10: (80, 82), 11: (108, -1), 12: (0, 2), 13: (0, 2), 14: (208, -1)}


def kquant_blocks(qtype: int, nblocks: int, seed: int, d_std: float = 0.01) -> np.ndarray:
    """uint8 [nblocks, block_bytes] of well-formed raw k-quant blocks.

    Every non-header byte is uniform random, which makes codes, 6-bit sub-scales/sub-mins (Q4_K/Q5_K/Q3_K), 4-bit
    pairs (Q2_K) and int8 sub-scales (Q6_K) uniform over their full range; the fp16 headers are |N(0,d_std)|."""
    rng = np.random.default_rng(seed)
    bb = BLOCK_BYTES[qtype]
    b = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    d_off, m_off = _HDR[qtype]
    d = np.abs(rng.normal(0.0, d_std, size=nblocks)).astype(np.float16)
    b[:, d_off:d_off + 2] = d.view(np.uint8).reshape(nblocks, 2)
    if m_off >= 0:
        dm = np.abs(rng.normal(0.0, d_std, size=nblocks)).astype(np.float16)
        b[:, m_off:m_off + 2] = dm.view(np.uint8).reshape(nblocks, 2)
    return b


def activations(rows: int, k: int, seed: int, dtype=np.float16) -> np.ndarray:
    """[rows,k] ~ N(0,1) in fp16 (or float32 for callers that convert to bf16 themselves)."""
    rng = np.random.default_rng(seed)
    return rng.normal(0.0, 1.0, size=(rows, k)).astype(np.float32).astype(dtype)


def group_planes(experts: int, n: int, k: int, bits: int, group_size: int, seed: int, zero_point=None):
    """Generic per-group W{bits}A16 artifact: (low uint8 [E,n,k*bits/8], scale fp16 [E,k/gs,n], zero fp16 [E,k/gs,n]).

    Codes are uniform in [0, 2^bits); scale = |N(0,0.02)|/7; zero = -zp*scale with zp = 2^(bits-1) by default
    (the additive form W = q*scale + zero).  Element k of a row sits at bit k*bits, LSB first."""
    rng = np.random.default_rng(seed)
    nbytes = k * bits // 8
    low = rng.integers(0, 256, size=(experts, n, nbytes), dtype=np.uint8)
    scale = (np.abs(rng.normal(0.0, 0.02, size=(experts, k // group_size, n))) / 7.0).astype(np.float16)
    zp = float(1 << (bits - 1)) if zero_point is None else float(zero_point)
    zero = (-(np.float32(zp)) * scale.astype(np.float32)).astype(np.float16)
    return low, scale, zero


def zipf_rows_per_expert(tokens: int, experts: int, top_k: int, seed: int, alpha: float = 1.1) -> np.ndarray:
    """Per-expert row counts of a Zipf(alpha)-skewed router: each token picks top_k distinct experts with
    probability proportional to rank^-alpha (rank order shuffled by the seed).  Sums to tokens*top_k; ragged;
    an expert may receive no rows."""
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, experts + 1, dtype=np.float64) ** alpha
    w = w[rng.permutation(experts)]
    counts = np.zeros(experts, np.int64)
    g = -np.log(-np.log(rng.random((tokens, experts))))          # Gumbel top-k = sampling without replacement
    pick = np.argsort(-(np.log(w)[None, :] + g), axis=1)[:, :top_k]
    np.add.at(counts, pick.reshape(-1), 1)
    return counts


def uniform_routes(tokens: int, experts: int, top_k: int, seed: int) -> np.ndarray:
    """[tokens, top_k] expert ids, uniform without replacement per token."""
    rng = np.random.default_rng(seed)
    return np.argsort(rng.random((tokens, experts)), axis=1)[:, :top_k].astype(np.int64)
