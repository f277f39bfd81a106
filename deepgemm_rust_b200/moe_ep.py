"""Expert-parallel driver for the contiguous m-grouped GEMM: experts sharded over ranks, token rows
exchanged with NCCL all-to-all before (dispatch) and after (combine) the grouped GEMMs.

The reference is single-GPU (deepgemm/src/moe.rs:101, top-1, no collectives); this is the multi-GPU
form of the same steps: build the group-contiguous arena (moe.rs:176-252), run the grouped GEMMs
(ops_sm100.rs:759), bring every token's expert outputs home and reduce them (moe.rs:314-360).

Rank r owns experts [r*E/W, (r+1)*E/W); its weights never move.  A step:
  plan      sort (token, expert) pairs by expert, exchange per-expert counts (one small all-to-all and
            one host read of W*E/W integers for the split sizes), derive arena positions on the device
  dispatch  pack e4m3 rows + scale words into send rows, all_to_all_single, unpack into the arena
            (every group starts at a multiple of the mk alignment; padding rows are zero)
  compute   the caller's grouped GEMMs on the arena
  combine   gather result rows in arrival order, all_to_all_single back, weighted sum per token

The index arithmetic is plain torch and runs on any device (the CPU tests drive it with gloo); the row
movers come from the `ops` object: `DeviceRowOps` (CUDA kernels of this library, the only one shipped).
"""
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


def _align_up(x: torch.Tensor, a: int) -> torch.Tensor:
    return (x + (a - 1)) // a * a


@dataclass
class Plan:
    tokens: int
    topk: int
    pairs: int                    # tokens * topk rows this rank sends
    n_recv: int                   # rows this rank receives
    m_pad: int                    # arena rows (groups padded to the alignment)
    send_splits: List[int]
    recv_splits: List[int]
    tok_of_sorted: torch.Tensor   # (pairs) int32: token of the i-th send row
    pos_of_pair: torch.Tensor     # (tokens, topk) int32: send-order position of each (token, j)
    dst_pos: torch.Tensor         # (n_recv) int32: arena row of the j-th received row
    src_idx: torch.Tensor         # (m_pad) int32: received row feeding each arena row, -1 for padding
    m_indices: torch.Tensor       # (m_pad) int32: local expert of each arena row, -1 for padding
    expert_rows: torch.Tensor     # (local experts) int64: valid rows per local expert


class DeviceRowOps:
    """Row movers on the GPU through the C-ABI library."""

    def __init__(self, ctx):
        import deepgemm_rust_b200 as dg
        self.dg, self.ctx = dg, ctx

    def pack(self, xq, xsf, rows, k, gran, idx, pitch):
        return self.dg.moe_pack_rows_dev(self.ctx, xq, xsf, rows, k, gran, idx, pitch)

    def unpack(self, recv, k, gran, idx, n_dst):
        return self.dg.moe_unpack_rows_dev(self.ctx, recv, k, gran, idx, n_dst)

    def gather(self, src, idx, n_dst):
        return self.dg.gather_rows_dev(self.ctx, src, idx, n_dst)

    def combine(self, rows, pos, weights):
        return self.dg.moe_combine_dev(self.ctx, rows, pos, weights)


class ExpertParallel:
    def __init__(self, num_experts: int, topk: int, ops, group: Optional[dist.ProcessGroup] = None, alignment: int = 128):
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and (group is not None or dist.get_world_size() > 1)
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts, self.local_experts, self.topk = num_experts, num_experts // self.world, topk
        self.ops, self.alignment = ops, alignment

    # ------------------------------------------------------------------ plan
    def plan(self, topk_idx: torch.Tensor) -> Plan:
        tokens, topk = topk_idx.shape
        dev = topk_idx.device
        flat = topk_idx.reshape(-1).to(torch.int64)
        order = torch.argsort(flat, stable=True)
        pairs = flat.numel()
        inv = torch.empty_like(order)
        inv[order] = torch.arange(pairs, device=dev)
        counts = torch.bincount(flat, minlength=self.num_experts).reshape(self.world, self.local_experts)
        if self.distributed:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)
        else:
            recv_counts = counts
        # the one host read of a step: split sizes of the two row exchanges and the arena size
        expert_rows = recv_counts.sum(0)
        padded = _align_up(expert_rows, self.alignment)
        host = torch.cat([counts.sum(1), recv_counts.sum(1), padded.sum().reshape(1)]).cpu().tolist()
        send_splits, recv_splits, m_pad = host[:self.world], host[self.world:2 * self.world], int(host[-1])
        n_recv = int(sum(recv_splits))
        # received rows arrive ordered by (source rank, local expert, token); arena wants (local expert, source rank, token)
        starts = torch.cumsum(padded, 0) - padded
        base = starts.unsqueeze(0) + torch.cumsum(recv_counts, 0) - recv_counts            # (world, local experts)
        seg_counts = recv_counts.reshape(-1)
        seg_begin = torch.cumsum(seg_counts, 0) - seg_counts
        seg_of_row = torch.repeat_interleave(torch.arange(seg_counts.numel(), device=dev), seg_counts, output_size=n_recv)
        dst_pos = base.reshape(-1)[seg_of_row] + (torch.arange(n_recv, device=dev) - seg_begin[seg_of_row])
        src_idx = torch.full((m_pad,), -1, dtype=torch.int32, device=dev)
        src_idx[dst_pos] = torch.arange(n_recv, device=dev, dtype=torch.int32)
        m_indices = torch.full((m_pad,), -1, dtype=torch.int32, device=dev)
        m_indices[dst_pos] = (seg_of_row % self.local_experts).to(torch.int32)
        return Plan(tokens, topk, pairs, n_recv, m_pad, [int(x) for x in send_splits], [int(x) for x in recv_splits],
                    (order // topk).to(torch.int32), inv.reshape(tokens, topk).to(torch.int32), dst_pos.to(torch.int32), src_idx,
                    m_indices, expert_rows)

    # -------------------------------------------------------------- exchange
    def _exchange(self, send: torch.Tensor, n_out: int, out_splits, in_splits) -> torch.Tensor:
        if not self.distributed:
            return send
        recv = torch.empty((n_out, send.shape[1]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)
        return recv

    def dispatch(self, plan: Plan, xq: torch.Tensor, xsf: torch.Tensor, k: int, gran: int = 128):
        """e4m3 token rows + packed scales (this rank's tokens) -> arena (m_pad, k) + packed scales on the expert ranks."""
        cols = (k + 4 * gran - 1) // (4 * gran)
        pitch = (k + 4 * cols + 15) // 16 * 16
        send = self.ops.pack(xq, xsf, plan.tokens, k, gran, plan.tok_of_sorted, pitch)
        recv = self._exchange(send, plan.n_recv, plan.recv_splits, plan.send_splits)
        return self.ops.unpack(recv, k, gran, plan.src_idx, plan.m_pad)

    def combine(self, plan: Plan, y: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Arena result rows (m_pad, n) bf16 -> per-token weighted sums (tokens, n) on the token ranks."""
        if not self.distributed:
            # one rank: result rows never leave; reduce straight from the arena through the composed index
            arena_pos = plan.dst_pos[plan.pos_of_pair.reshape(-1).long()].reshape(plan.tokens, plan.topk).contiguous()
            return self.ops.combine(y, arena_pos, weights)
        back = self.ops.gather(y, plan.dst_pos, plan.n_recv)
        home = self._exchange(back, plan.pairs, plan.send_splits, plan.recv_splits)
        return self.ops.combine(home, plan.pos_of_pair, weights)
