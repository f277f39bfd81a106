"""GPU parity of the MoE row movers (bit-exact against numpy / the oracle) and of one whole
expert-parallel step on a single rank (dispatch -> grouped GEMMs -> combine)."""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from deepgemm_rust_b200.moe_ep import DeviceRowOps, ExpertParallel, PeerExpertParallel, PipelinedPeerMoe
from oracle import oracle as O
from tests.helpers import dev, fp8_operand_1d, fp8_operand_2d, peer_layout, to_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def test_row_movers_bit_exact(ctx):
    rng = np.random.default_rng(5)
    rows, k, gran = 100, 1152, 128
    cols, stride = dg.sf_packed_cols(k, gran), dg.sf_aligned_rows(rows)
    xq = rng.integers(0, 256, (rows, k), dtype=np.uint8)
    xsf = rng.integers(0, 2 ** 32, cols * stride, dtype=np.uint32)
    idx = rng.integers(0, rows, 333).astype(np.int32)
    pitch = (k + 4 * cols + 15) // 16 * 16
    sent = dg.moe_pack_rows_dev(ctx, dev(xq), dev(xsf), rows, k, gran, dev(idx), pitch).cpu().numpy()
    assert np.array_equal(sent[:, :k], xq[idx])
    words = sent[:, k:k + 4 * cols].copy().view(np.uint32)
    assert np.array_equal(words, xsf.reshape(cols, stride)[:, idx].T)
    assert np.all(sent[:, k + 4 * cols:] == 0)
    # unpack into an arena with padding rows
    n_dst = 400
    src = rng.integers(-1, 333, n_dst).astype(np.int32)
    data, sf = dg.moe_unpack_rows_dev(ctx, dev(sent), k, gran, dev(src), n_dst)
    data, sf = data.cpu().numpy(), sf.cpu().numpy().view(np.uint32).reshape(cols, dg.sf_aligned_rows(n_dst))
    valid = src >= 0
    assert np.array_equal(data[valid], sent[src[valid], :k]) and np.all(data[~valid] == 0)
    assert np.array_equal(sf[:, :n_dst][:, valid], words[src[valid]].T) and np.all(sf[:, :n_dst][:, ~valid] == 0)
    # generic gather of bf16 rows
    y = rng.integers(0, 65536, (n_dst, 256), dtype=np.uint16)
    got = dg.gather_rows_dev(ctx, dev(y, torch.bfloat16), dev(src), n_dst).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got[valid], y[src[valid]]) and np.all(got[~valid] == 0)
    # weighted combine against the oracle (same fused multiply-add chain)
    tokens, topk, n = 57, 8, 512
    rows_bits = O.bf16_bits(rng.standard_normal((300, n)).astype(np.float32))
    pos = rng.integers(-1, 300, (tokens, topk)).astype(np.int32)
    w = rng.random((tokens, topk)).astype(np.float32)
    got = dg.moe_combine_dev(ctx, dev(rows_bits, torch.bfloat16), dev(pos), dev(w)).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, O.moe_combine(rows_bits, pos, w))
    ctx.sync()


def test_expert_parallel_step_single_rank(ctx):
    experts, topk, tokens, hidden, n1, k2, n2 = 8, 2, 200, 512, 1024, 512, 384
    g = torch.Generator().manual_seed(9)
    logits = torch.randn((tokens, experts), generator=g)
    probs = torch.softmax(logits, -1)
    topw, topi = probs.topk(topk, dim=-1)
    topi[:, 1] = torch.where(topi[:, 1] == 3, topi[:, 0], topi[:, 1])      # expert 3 may end up empty for some seeds
    _, xq, xsf = fp8_operand_1d(tokens, hidden, 81)
    _, w1q, w1sf, _ = fp8_operand_2d(experts * n1, hidden, 82, experts)
    _, w2q, w2sf, _ = fp8_operand_2d(experts * n2, k2, 83, experts)
    ep = ExpertParallel(experts, topk, DeviceRowOps(ctx))
    plan = ep.plan(topi.cuda())
    a, a_sf = ep.dispatch(plan, dev(xq), dev(xsf), hidden)
    # arena rows hold exactly the routed tokens, grouped by expert, groups aligned to 128
    m_idx = plan.m_indices.cpu().numpy()
    flat = topi.reshape(-1).numpy()
    order = np.argsort(flat, kind="stable")
    arena = a.cpu().numpy()
    starts = np.concatenate([[0], np.cumsum((np.bincount(flat, minlength=experts) + 127) // 128 * 128)[:-1]])
    seen = np.zeros(experts, np.int64)
    for p in order:
        e, t = flat[p], p // topk
        r = starts[e] + seen[e]
        seen[e] += 1
        assert m_idx[r] == e and np.array_equal(arena[r], xq[t])
    assert int((m_idx >= 0).sum()) == tokens * topk and np.all(arena[m_idx < 0] == 0)
    # grouped GEMM 1 on the arena against the oracle, on the valid rows
    h = torch.zeros((plan.m_pad, n1), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(a, a_sf, plan.m_pad, hidden, hidden), plan.m_indices,
                                             dg.LpOperand(dev(w1q), dev(w1sf), experts * n1, hidden, hidden), dg.Sm100Out.Bf16(h, n1), experts)
    ctx.sync()
    valid = np.nonzero(m_idx >= 0)[0]
    a_sf_np = a_sf.cpu().numpy().view(np.uint32)
    hn = to_f32(h)
    for e in range(experts):
        rows = valid[m_idx[valid] == e].astype(np.uint32)
        if rows.size == 0:
            continue
        want = O.lp_gemm_rows(arena, a_sf_np, 8, 128, 1, plan.m_pad, rows, w1q, w1sf, 8, 128, experts, n1,
                              np.arange(e * n1, (e + 1) * n1, dtype=np.uint32), hidden)
        assert O.calc_diff(hn[rows.astype(np.int64)], want) <= 2e-5
    # silu(gate) * up of GEMM 1's output, quantised for GEMM 2: bit-exact with the two oracle steps on the same bf16 bits
    actq, actsf = dg.silu_mul_cast_fp8_sf_dev(ctx, h, n1, plan.m_pad, k2, 128)
    ctx.sync()
    h_bits = h.view(torch.int16).cpu().numpy().view(np.uint16)
    want_q, want_sf = O.cast_bf16_to_fp8_sf(O.silu_mul_bf16(h_bits), k2, 128)
    actq_np, actsf_np = actq.cpu().numpy(), actsf.cpu().numpy().view(np.uint32)
    assert np.array_equal(actq_np, want_q) and np.array_equal(actsf_np, want_sf)
    # grouped GEMM 2 consumes the activation
    y = torch.zeros((plan.m_pad, n2), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(actq, actsf, plan.m_pad, k2, k2), plan.m_indices,
                                             dg.LpOperand(dev(w2q), dev(w2sf), experts * n2, k2, k2), dg.Sm100Out.Bf16(y, n2), experts)
    ctx.sync()
    yn = to_f32(y)
    for e in range(experts):
        rows = valid[m_idx[valid] == e].astype(np.uint32)
        if rows.size == 0:
            continue
        want = O.lp_gemm_rows(actq_np, actsf_np, 8, 128, 1, plan.m_pad, rows, w2q, w2sf, 8, 128, experts, n2,
                              np.arange(e * n2, (e + 1) * n2, dtype=np.uint32), k2)
        assert O.calc_diff(yn[rows.astype(np.int64)], want) <= 2e-5
    out = ep.combine(plan, y, topw.cuda().contiguous())
    ctx.sync()
    # combine: token t gets sum_j w[t,j] * y[arena row of pair (t,j)], bit-exact with the oracle reduction
    y_bits = y.view(torch.int16).cpu().numpy().view(np.uint16)
    pos = np.zeros((tokens, topk), np.int32)
    seen[:] = 0
    for p in order:
        e = flat[p]
        pos[p // topk, p % topk] = starts[e] + seen[e]
        seen[e] += 1
    want = O.moe_combine(y_bits, pos, topw.numpy())
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)


def arena_layout(expert_of_pair, experts, alignment=128):
    """numpy restatement of the single-rank arena: groups in expert order, each starting at a multiple of the
    alignment, pairs of one expert in pair order.  Returns (row of each pair, group ends, rows in use)."""
    flat = np.asarray(expert_of_pair)
    ok = (flat >= 0) & (flat < experts)
    counts = np.bincount(flat[ok], minlength=experts)
    padded = (counts + alignment - 1) // alignment * alignment
    starts = np.cumsum(padded) - padded
    pos = np.full(flat.size, -1, np.int64)
    seen = np.zeros(experts, np.int64)
    for p, e in enumerate(flat):
        if ok[p]:
            pos[p] = starts[e] + seen[e]
            seen[e] += 1
    return pos, starts + counts, int(padded.sum())


def test_peer_exchange_single_rank(ctx):
    experts, topk, tokens, hidden, n = 8, 3, 700, 512, 256          # 2100 pairs: nine ranking chunks, the last one ragged
    g = torch.Generator().manual_seed(21)
    topw, topi = torch.softmax(torch.randn((tokens, experts), generator=g), -1).topk(topk, dim=-1)
    topi[topi == 5] = 6                                               # an expert nobody routes to
    topi[3, 1] = -1                                                   # a dropped pair
    topi[10, 0] = experts                                             # an id out of range is dropped as well
    _, xq, xsf = fp8_operand_1d(tokens, hidden, 31)
    _, wq, wsf, _ = fp8_operand_2d(experts * n, hidden, 32, experts)
    pe = PeerExpertParallel(ctx, experts, topk, tokens, hidden, n)
    try:
        for step in range(2):                                         # the second step reuses every buffer
            a_op, ends = pe.dispatch(topi.cuda(), dev(xq), dev(xsf))
            ctx.sync()
            pos, want_ends, rows_in_use = arena_layout(topi.reshape(-1).numpy(), experts)
            assert np.array_equal(pe.pos_of_pair.cpu().numpy()[:pos.size], pos)
            assert np.array_equal(ends.cpu().numpy().view(np.uint32), want_ends)
            totals = pe.totals.cpu().numpy()
            assert totals[0] == rows_in_use and totals[1] == (pos >= 0).sum() and totals[2] == 0 and totals[3] == rows_in_use
            arena = pe.arena.cpu().numpy()
            sf = pe.arena_sf.cpu().numpy().view(np.uint32).reshape(pe.sf_cols, pe.sf_stride)
            xsf2 = xsf.reshape(pe.sf_cols, -1)
            live = np.nonzero(pos >= 0)[0]
            assert np.array_equal(arena[pos[live]], xq[live // topk])
            assert np.array_equal(sf[:, pos[live]], xsf2[:, live // topk])
            untouched = np.ones(pe.capacity, bool)
            untouched[pos[live]] = False
            assert not arena[untouched].any() and not sf[:, untouched].any()
            # the grouped GEMM takes the group-end table as it is and writes the buffer the combine reads
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, dg.LpOperand(dev(wq), dev(wsf), experts * n, hidden, hidden),
                                                          dg.Sm100Out.Bf16(pe.result, n), experts)
            out = pe.combine(topw.cuda().contiguous())
            ctx.sync()
            y_bits = pe.result.view(torch.int16).cpu().numpy().view(np.uint16)
            flat = topi.reshape(-1).numpy()
            for e in range(experts):
                rows = pos[(flat == e)].astype(np.uint32)
                if rows.size:
                    want = O.lp_gemm_rows(arena, pe.arena_sf.cpu().numpy().view(np.uint32), 8, 128, 1, pe.capacity, rows, wq, wsf, 8, 128,
                                          experts, n, np.arange(e * n, (e + 1) * n, dtype=np.uint32), hidden)
                    assert O.calc_diff(to_f32(pe.result)[rows.astype(np.int64)], want) <= 2e-5
            want = O.moe_combine(y_bits, pos.reshape(tokens, topk).astype(np.int32), topw.numpy())
            assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
            assert not pe.overflowed()
    finally:
        pe.close()


def test_peer_exchange_reports_overflow(ctx):
    # an arena too small for the routing: rows that do not fit are dropped, flagged, and skipped by the combine
    experts, topk, tokens, hidden, n = 4, 2, 256, 512, 128
    topi = torch.zeros((tokens, topk), dtype=torch.int64)
    topi[:, 1] = 1
    _, xq, xsf = fp8_operand_1d(tokens, hidden, 41)
    pe = PeerExpertParallel(ctx, experts, topk, tokens, hidden, n, capacity=384)
    try:
        pe.dispatch(topi.cuda(), dev(xq), dev(xsf))
        ctx.sync()
        assert pe.overflowed()
        pos = pe.pos_of_pair.cpu().numpy().reshape(tokens, topk)
        assert np.array_equal(pos[:, 0], np.arange(tokens))           # expert 0 fits in rows [0, 256)
        assert np.array_equal(pos[:128, 1], 256 + np.arange(128)) and np.all(pos[128:, 1] == -1)
    finally:
        pe.close()


def test_pipelined_micro_batches_equal_the_single_batch(ctx):
    # exchange on a second stream, three token micro-batches (the last one shorter): every token's output must equal
    # the unchunked step bit for bit
    experts, topk, tokens, hidden, n = 8, 2, 500, 512, 256
    g = torch.Generator().manual_seed(33)
    topw, topi = torch.softmax(torch.randn((tokens, experts), generator=g), -1).topk(topk, dim=-1)
    _, xq, xsf = fp8_operand_1d(tokens, hidden, 51)
    _, wq, wsf, _ = fp8_operand_2d(experts * n, hidden, 52, experts)
    w_op = dg.LpOperand(dev(wq), dev(wsf), experts * n, hidden, hidden)
    topi_d, topw_d, xq_d, xsf_d = topi.cuda(), topw.cuda().contiguous(), dev(xq), dev(xsf)

    def compute(pe, a_op, ends):
        dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, w_op, dg.Sm100Out.Bf16(pe.result, n), experts)

    pe = PeerExpertParallel(ctx, experts, topk, tokens, hidden, n)
    a_op, ends = pe.dispatch(topi_d, xq_d, xsf_d)
    compute(pe, a_op, ends)
    want = pe.combine(topw_d).view(torch.int16).cpu().numpy()
    ctx.sync()
    pe.close()
    pipe = PipelinedPeerMoe(ctx, experts, topk, tokens, hidden, n, chunks=3)
    try:
        for _ in range(2):
            out = pipe.run(topi_d, xq_d, xsf_d, topw_d, compute)
            torch.cuda.synchronize()
            assert np.array_equal(out.view(torch.int16).cpu().numpy(), want)
            assert pipe.routed_rows() == tokens * topk
    finally:
        pipe.close()


def test_layout_kernel_for_every_rank_of_a_larger_job(ctx):
    # the layout kernel only sees the all-gathered count matrix, so one GPU can check what each rank of a 4-rank (and an
    # 8-rank) job would derive, against the numpy restatement; counts include empty experts and groups that need padding
    rng = np.random.default_rng(17)
    for world, experts in [(4, 32), (8, 256), (1, 8)]:
        counts = rng.integers(0, 700, (world, experts)).astype(np.uint32)
        counts[:, 3] = 0
        counts[world - 1, :] = rng.integers(0, 3, experts)
        local = experts // world
        for rank in range(world):
            pair_base = torch.zeros(experts, dtype=torch.int32, device="cuda")
            ends = torch.zeros(local, dtype=torch.int32, device="cuda")
            totals = torch.zeros(4, dtype=torch.int32, device="cuda")
            dg.ep_layout_dev(ctx, dev(counts), world, rank, experts, 128, 1 << 30, pair_base, ends, totals)
            ctx.sync()
            want_base, want_ends, want_totals = peer_layout(counts, rank)
            assert np.array_equal(pair_base.cpu().numpy().view(np.uint32), want_base)
            assert np.array_equal(ends.cpu().numpy().view(np.uint32), want_ends)
            got = totals.cpu().numpy()
            assert [int(got[0]), int(got[1]), int(got[3])] == want_totals and got[2] == 0
        # a capacity one row short of the largest arena raises the overflow flag on every rank
        dg.ep_layout_dev(ctx, dev(counts), world, 0, experts, 128, want_totals[2] - 1, pair_base, ends, totals)
        ctx.sync()
        assert totals.cpu().numpy()[2] == 1


def test_pair_ranking_is_a_stable_counting_sort(ctx):
    rng = np.random.default_rng(23)
    experts, pairs = 40, 5000                                  # twenty chunks of 256 pairs, the last one ragged
    ids = rng.integers(-1, experts + 1, pairs).astype(np.int32)     # -1 and `experts` are out of range: dropped
    local_rank = torch.zeros(pairs, dtype=torch.int32, device="cuda")
    hist = torch.zeros(dg.ep_block_hist_words(pairs, experts), dtype=torch.int32, device="cuda")
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    dg.ep_count_dev(ctx, dev(ids), pairs, experts, local_rank, hist, counts)
    ctx.sync()
    ok = (ids >= 0) & (ids < experts)
    assert np.array_equal(counts.cpu().numpy(), np.bincount(ids[ok], minlength=experts))
    # position of every kept pair among the pairs of its expert = chunk base + rank inside the chunk, in pair order
    base = hist.cpu().numpy().reshape(-1, experts)
    lr = local_rank.cpu().numpy()
    seen = np.zeros(experts, np.int64)
    for p in range(pairs):
        if ok[p]:
            assert base[p // 256, ids[p]] + lr[p] == seen[ids[p]]
            seen[ids[p]] += 1
        else:
            assert lr[p] == -1


def test_peer_exchange_masked_layout(ctx):
    # decode-style step: every local expert owns a fixed slot of rows, the exchange writes token rows and their scale words
    # straight into the (experts, slot_rows, k) operand of the masked grouped GEMM and hands it the per-expert row counts
    experts, topk, tokens, hidden, n, slot = 8, 2, 90, 512, 256, 64
    g = torch.Generator().manual_seed(44)
    topw, topi = torch.softmax(torch.randn((tokens, experts), generator=g), -1).topk(topk, dim=-1)
    topi[topi == 2] = 3                                               # an empty slot
    _, xq, xsf = fp8_operand_1d(tokens, hidden, 61)
    _, wq, wsf, _ = fp8_operand_2d(experts * n, hidden, 62, experts)
    pe = PeerExpertParallel(ctx, experts, topk, tokens, hidden, n, slot_rows=slot)
    try:
        a_op, masked_m = pe.dispatch(topi.cuda(), dev(xq), dev(xsf))
        ctx.sync()
        flat = topi.reshape(-1).numpy()
        counts = np.bincount(flat, minlength=experts)
        assert counts.max() <= slot and not pe.overflowed()
        assert np.array_equal(masked_m.cpu().numpy(), counts)
        pos = np.zeros(flat.size, np.int64)
        seen = np.zeros(experts, np.int64)
        for p, e in enumerate(flat):
            pos[p] = e * slot + seen[e]
            seen[e] += 1
        assert np.array_equal(pe.pos_of_pair.cpu().numpy()[:pos.size], pos)
        arena = pe.arena.cpu().numpy()
        assert np.array_equal(arena[pos], xq[np.arange(flat.size) // topk])
        cols = pe.sf_cols
        sf = pe.arena_sf.cpu().numpy().view(np.uint32).reshape(experts, cols, dg.sf_aligned_rows(slot))
        xsf2 = xsf.reshape(cols, -1)
        assert np.array_equal(sf[pos // slot, :, pos % slot], xsf2[:, np.arange(flat.size) // topk].T)
        dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a_op, masked_m, dg.LpOperand(dev(wq), dev(wsf), experts * n, hidden, hidden),
                                             dg.Sm100Out.Bf16(pe.result, n), experts, max(1, int(counts.mean())))
        out = pe.combine(topw.cuda().contiguous())
        ctx.sync()
        # every valid result row against the oracle, then the reduction bit for bit
        yn = to_f32(pe.result)
        for e in range(experts):
            rows = pos[flat == e].astype(np.uint32)
            if rows.size:
                want = O.lp_gemm_rows(arena, pe.arena_sf.cpu().numpy().view(np.uint32), 8, 128, experts, slot, rows, wq, wsf, 8, 128,
                                      experts, n, np.arange(e * n, (e + 1) * n, dtype=np.uint32), hidden)
                assert O.calc_diff(yn[rows.astype(np.int64)], want) <= 2e-5
        y_bits = pe.result.view(torch.int16).cpu().numpy().view(np.uint16)
        want = O.moe_combine(y_bits, pos.reshape(tokens, topk).astype(np.int32), topw.numpy())
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
    finally:
        pe.close()
    # a slot too small for its expert: the rows that do not fit are dropped and flagged
    pe = PeerExpertParallel(ctx, experts, topk, tokens, hidden, n, slot_rows=16)
    try:
        pe.dispatch(topi.cuda(), dev(xq), dev(xsf))
        ctx.sync()
        assert pe.overflowed()
        got = pe.pos_of_pair.cpu().numpy()[:flat.size]
        seen[:] = 0
        for p, e in enumerate(flat):
            assert got[p] == (e * 16 + seen[e] if seen[e] < 16 else -1)
            seen[e] += 1
    finally:
        pe.close()


def test_peer_exchange_refuses_a_context_on_another_stream():
    # the collectives that order the ranks run on torch's current stream; a context whose kernels run elsewhere would race
    own = dg.DgContext(0, own_stream=True)
    pe = PeerExpertParallel(own, 8, 2, 16, 512, 256)
    try:
        with pytest.raises(RuntimeError):
            pe._check_stream()
        with torch.cuda.stream(torch.cuda.ExternalStream(own.stream)):
            pe._check_stream()
    finally:
        pe.close()
        own.close()
