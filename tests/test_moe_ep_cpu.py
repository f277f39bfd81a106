"""Host logic of the expert-parallel driver on CPU ranks (gloo, world sizes 1 and 2): plan, count
exchange, dispatch and combine must route every (token, expert) pair to the owning rank's arena and
bring its result back to the right token.  Row movers are a torch stand-in defined here (the shipped
ones are CUDA kernels); the "GEMM" is a marker function of (expert, token) that is exact in bf16."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepgemm_rust_b200.moe_ep import ExpertParallel


class TorchRowOps:
    def pack(self, xq, xsf, rows, k, gran, idx, pitch):
        cols = (k + 4 * gran - 1) // (4 * gran)
        stride = (rows + 3) // 4 * 4
        out = torch.zeros((idx.numel(), pitch), dtype=torch.uint8)
        out[:, :k] = xq[idx.long()]
        words = xsf.view(cols, stride)[:, idx.long()].t().reshape(-1).clone().reshape(idx.numel(), cols)  # (n, cols) int32
        out[:, k:k + 4 * cols] = words.view(torch.uint8)
        return out

    def unpack(self, recv, k, gran, idx, n_dst):
        cols = (k + 4 * gran - 1) // (4 * gran)
        stride = (n_dst + 3) // 4 * 4
        data = torch.zeros((n_dst, k), dtype=torch.uint8)
        sf = torch.zeros((cols, stride), dtype=torch.int32)
        valid = idx >= 0
        rows = recv[idx[valid].long()]
        data[valid] = rows[:, :k]
        sf[:, :n_dst][:, valid] = rows[:, k:k + 4 * cols].reshape(-1).clone().view(torch.int32).reshape(-1, cols).t()
        return data, sf.reshape(-1)

    def gather(self, src, idx, n_dst):
        out = torch.zeros((n_dst, src.shape[1]), dtype=src.dtype)
        valid = idx >= 0
        out[valid] = src[idx[valid].long()]
        return out

    def combine(self, rows, pos, weights):
        acc = torch.zeros((pos.shape[0], rows.shape[1]), dtype=torch.float32)
        for j in range(pos.shape[1]):
            acc += weights[:, j:j + 1] * rows[pos[:, j].long()].float()
        return acc.to(torch.bfloat16)


def _run_rank(rank, world, port, results):
    if world > 1:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, topk, tokens, k, n = 8, 2, 24, 128, 8
        g = torch.Generator().manual_seed(100 + rank)
        topk_idx = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)])
        if rank == 0:
            topk_idx[:, 0] = torch.where(topk_idx[:, 0] == 5, torch.tensor(6), topk_idx[:, 0])   # expert 5 gets fewer rows
        weights = torch.tensor([[1.0, 0.5]]).repeat(tokens, 1)
        tag = torch.arange(tokens) + 1 + 32 * rank                 # unique per token across ranks, < 256
        xq = tag.to(torch.uint8).unsqueeze(1).repeat(1, k)
        xsf = (tag * 3 + 1).to(torch.int32)                        # one packed word per token (k = 128, gran 128)
        ep = ExpertParallel(experts, topk, TorchRowOps(), alignment=4)
        plan = ep.plan(topk_idx)
        a, a_sf = ep.dispatch(plan, xq, xsf, k)
        # arena invariants
        assert a.shape == (plan.m_pad, k) and plan.m_pad % 4 == 0
        valid = plan.m_indices >= 0
        assert int(valid.sum()) == plan.n_recv == int(plan.expert_rows.sum())
        assert torch.all(a[~valid] == 0)
        row_tag = a[:, 0].long()
        assert torch.equal(a_sf.view(-1, (plan.m_pad + 3) // 4 * 4)[0, :plan.m_pad][valid], (row_tag[valid] * 3 + 1).int())
        mi = plan.m_indices[valid]
        assert torch.all(mi[1:] >= mi[:-1])                        # groups in order
        for le in range(ep.local_experts):                         # every group starts on the alignment
            rows = torch.nonzero(plan.m_indices == le).flatten()
            if rows.numel():
                assert int(rows[0]) % 4 == 0 and int(rows[-1] - rows[0]) == rows.numel() - 1
        # marker "GEMM": column 0 = global expert + 1, column 1 = token tag (both exact in bf16), the rest zero
        g_expert = plan.m_indices.long() + rank * ep.local_experts + 1
        y = torch.zeros((plan.m_pad, n), dtype=torch.float32)
        y[valid, 0] = g_expert[valid].float()
        y[valid, 1] = row_tag[valid].float()
        out = ep.combine(plan, y.to(torch.bfloat16), weights).float()
        want0 = (topk_idx[:, 0] + 1).float() + 0.5 * (topk_idx[:, 1] + 1).float()
        ok = torch.equal(out[:, 0], want0) and torch.equal(out[:, 1], 1.5 * tag.float()) and torch.all(out[:, 2:] == 0)
        results[rank] = bool(ok)
    finally:
        if world > 1:
            dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_expert_parallel_single_rank():
    results = {}
    _run_rank(0, 1, 0, results)
    assert results == {0: True}


@pytest.mark.parametrize("world", [2])
def test_expert_parallel_gloo(world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_run_rank, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(results) == {r: True for r in range(world)}


def test_peer_layout_restatement_is_consistent():
    # the numpy restatement the GPU tests hold the layout kernel to: arenas are disjoint unions of contiguous
    # (expert, source rank) segments, groups start aligned, and on one rank it agrees with ExpertParallel.plan
    from tests.helpers import peer_layout
    rng = np.random.default_rng(3)
    for world, experts in [(2, 8), (4, 32)]:
        counts = rng.integers(0, 300, (world, experts))
        counts[:, 1] = 0
        local = experts // world
        bases = [peer_layout(counts, r)[0] for r in range(world)]
        for owner in range(world):
            _, ends, totals = peer_layout(counts, owner)
            taken = np.zeros(totals[0], bool)
            prev_end = 0
            for l in range(local):
                e = owner * local + l
                start = (prev_end + 127) // 128 * 128
                row = start
                for src in range(world):
                    assert bases[src][e] == row
                    assert not taken[row:row + counts[src, e]].any()
                    taken[row:row + counts[src, e]] = True
                    row += counts[src, e]
                assert row == ends[l]
                prev_end = ends[l]
            assert taken.sum() == totals[1]
    topk_idx = torch.stack([torch.randperm(8)[:2] for _ in range(50)])
    plan = ExpertParallel(8, 2, TorchRowOps()).plan(topk_idx)
    counts = np.bincount(topk_idx.reshape(-1).numpy(), minlength=8)[None, :]
    _, ends, totals = peer_layout(counts, 0)
    assert totals[0] == plan.m_pad and totals[1] == plan.n_recv
    m_idx = plan.m_indices.numpy()
    for e in range(8):
        assert (m_idx == e).sum() == counts[0, e] and (counts[0, e] == 0 or np.nonzero(m_idx == e)[0].max() + 1 == ends[e])
