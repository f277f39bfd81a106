"""Shared input builders and comparison helpers for the parity tests.

Inputs are seeded N(0,1) bf16 matrices (the benchmark contract's distribution); quantised
operands come from the CPU oracle so the GPU kernel and the checker consume identical bytes.
"""
import numpy as np

from oracle import oracle as O


def randn_bf16(rows, k, seed):
    return O.bf16_bits(np.random.default_rng(seed).standard_normal((rows, k)).astype(np.float32))


def fp8_operand_1d(rows, k, seed, gran=128, groups=1):
    """Per-row scales (activations): (bf16 bits, e4m3 bytes, packed words)."""
    bits = randn_bf16(rows, k, seed)
    q, sf = O.cast_bf16_to_fp8_sf(bits, k, gran, groups)
    return bits, q, sf


def fp8_operand_2d(rows, k, seed, groups=1):
    """One scale per 128x128 tile (weights), expanded per row into the packed layout.
    Returns (bf16 bits, e4m3 bytes, packed words, tile scales f32 (rows/128, k/128))."""
    bits = randn_bf16(rows, k, seed)
    q, exps = O.quantize_fp8_ue8m0_blocks(bits, k, 128)
    sf_f32 = O.exps_to_f32(exps)
    packed = O.transform_sf2d_packed(sf_f32, rows, k, groups)
    return bits, q, packed, sf_f32


def fp4_operand(rows, k, seed, groups=1, rule=O.SF_RULE_REFERENCE_CPU):
    bits = randn_bf16(rows, k, seed)
    q, sf = O.cast_bf16_to_fp4_packed_sf(bits, k, groups, rule)
    return bits, q, sf


def sample_indices(n, count, seed, edges=(0, 1, 31, 32, 63, 64, 127, 128, 129, 191, 192, 255, 256)):
    """Random rows plus the rows either side of every tile boundary that exists."""
    rng = np.random.default_rng(seed)
    picks = set(int(i) for i in rng.integers(0, n, size=min(count, n)))
    for e in edges:
        if e < n:
            picks.add(e)
    picks.add(n - 1)
    if n > 1:
        picks.add(n - 2)
    return np.array(sorted(picks), dtype=np.uint32)


def to_f32(t):
    """torch tensor (bf16 / f32) on any device -> numpy f32."""
    import torch
    return t.detach().to(torch.float32).cpu().numpy()


def dev(arr, dtype=None):
    """numpy array -> cuda tensor without value conversion (uint32/uint16 reinterpret as int32/int16)."""
    import torch
    a = np.ascontiguousarray(arr)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    elif a.dtype == np.uint16:
        a = a.view(np.int16)
    t = torch.from_numpy(a).cuda()
    if dtype is not None:
        t = t.view(dtype)
    return t


def peer_layout(all_counts, rank, alignment=128):
    """numpy restatement of the arena layout every rank derives from the all-gathered (world, experts) pair counts:
    groups sit on their owner in expert order, each starting at a multiple of the alignment, rows ordered by source
    rank.  Returns (pair_base (experts), group_ends (experts / world), [rows in use here, valid rows here, largest arena])."""
    all_counts = np.asarray(all_counts, dtype=np.int64)
    world, experts = all_counts.shape
    local = experts // world
    rows_of = all_counts.sum(0)
    before_me = all_counts[:rank].sum(0)
    padded = (rows_of + alignment - 1) // alignment * alignment
    start = np.zeros(experts, np.int64)
    arena = np.zeros(world, np.int64)
    for owner in range(world):
        sl = slice(owner * local, (owner + 1) * local)
        start[sl] = np.cumsum(padded[sl]) - padded[sl]
        arena[owner] = padded[sl].sum()
    mine = slice(rank * local, (rank + 1) * local)
    group_ends = start[mine] + rows_of[mine]
    return start + before_me, group_ends, [int(arena[rank]), int(rows_of[mine].sum()), int(arena.max())]
