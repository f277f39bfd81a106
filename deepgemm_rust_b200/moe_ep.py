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

`PeerExpertParallel` is the same step without the collectives' staging: every rank maps its peers' arenas and
result buffers, dispatch writes each row straight into its arena row on the owner and combine reads each
result row straight from the owner (kernels of this library, plain stores/loads over NVLink); the only
collectives left are an all-gather of the per-expert counts and two one-word all-reduces that order the ranks.

`ExpertParallel`'s index arithmetic is plain torch and runs on any device (the CPU tests drive it with gloo); the row
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


class PeerExpertParallel:
    """Expert-parallel dispatch / combine over peer memory.  One instance per rank and per layer shape.

    capacity: arena rows every rank provides.  The default is the worst case (all pairs of all ranks routed to
    one rank), so no routing can overflow; a smaller value saves memory, and a step that would overflow it drops
    the rows that do not fit and reports it through `overflowed()`.
    Alignment-padding rows of the arena are never written (they hold zeros until a longer group has used them, then
    stale rows); the grouped GEMM computes them inside its tiles and stores none of them.
    Nothing in a step reads back to the host: the arena's row count stays on the device (`totals`), the grouped
    GEMMs take `group_ends`, and operands are declared with `capacity` rows.
    The context's stream must be torch's current stream whenever dispatch() or combine() is called (checked): the
    collectives between the ranks are ordered against that stream only.
    """

    def __init__(self, ctx, num_experts: int, topk: int, max_tokens: int, hidden: int, out_n: int, gran: int = 128,
                 group: Optional[dist.ProcessGroup] = None, alignment: int = 128, capacity: Optional[int] = None,
                 slot_rows: int = 0):
        import deepgemm_rust_b200 as dg
        self.dg, self.ctx, self.group = dg, ctx, group
        self.distributed = dist.is_available() and dist.is_initialized() and (group is not None or dist.get_world_size() > 1)
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts, self.local_experts, self.topk = num_experts, num_experts // self.world, topk
        self.max_pairs, self.hidden, self.out_n, self.gran, self.alignment = max_tokens * topk, hidden, out_n, gran, alignment
        worst = self.world * self.max_pairs + alignment * self.local_experts
        cap = min(capacity, worst) if capacity else worst
        # slot_rows: the masked layout (decode-style steps): every local expert owns a fixed slot of that many arena rows and
        # `group_ends` holds the valid row count of each slot, i.e. the masked GEMM's masked_m with m_max = slot_rows
        self.slot_rows = slot_rows
        if slot_rows:
            cap = slot_rows * self.local_experts
        self.capacity = cap = (cap + 127) // 128 * 128
        self.sf_cols = dg.sf_packed_cols(hidden, gran)
        self.sf_stride = dg.sf_aligned_rows(slot_rows) if slot_rows else dg.sf_aligned_rows(cap)
        dev = self.device = torch.device(f"cuda:{ctx.ordinal}")

        def region(nbytes):
            return (nbytes + 255) // 256 * 256
        sf_words = self.sf_cols * self.sf_stride * (self.local_experts if slot_rows else 1)
        sizes = [region(cap * hidden), region(sf_words * 4), region(cap * out_n * 2)]
        offs = [0, sizes[0], sizes[0] + sizes[1]]
        self._base, handle = dg.peer_alloc(ctx, sum(sizes), export=self.distributed)
        self._opened = []
        bases = [self._base]
        if self.distributed:
            mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(dev)
            every = torch.empty((self.world, dg.PEER_HANDLE_BYTES), dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(every, mine, group=group)
            every = every.cpu().numpy()
            bases = []
            for r in range(self.world):
                if r == self.rank:
                    bases.append(self._base)
                else:
                    bases.append(dg.peer_open(ctx, every[r].tobytes()))
                    self._opened.append(bases[-1])
        self._peer_data = torch.tensor([b + offs[0] for b in bases], dtype=torch.int64, device=dev)
        self._peer_sf = torch.tensor([b + offs[1] for b in bases], dtype=torch.int64, device=dev)
        self._peer_rows = torch.tensor([b + offs[2] for b in bases], dtype=torch.int64, device=dev)
        self.arena = dg.tensor_from_ptr(self._base + offs[0], (cap, hidden), torch.uint8, ctx.ordinal)
        self.arena_sf = dg.tensor_from_ptr(self._base + offs[1], (sf_words,), torch.int32, ctx.ordinal)
        self.result = dg.tensor_from_ptr(self._base + offs[2], (cap, out_n), torch.bfloat16, ctx.ordinal)
        self.arena.zero_()
        self.arena_sf.zero_()
        i32 = dict(dtype=torch.int32, device=dev)
        self._local_rank = torch.empty(self.max_pairs, **i32)
        self._block_hist = torch.empty(dg.ep_block_hist_words(self.max_pairs, num_experts), **i32)
        self._counts = torch.empty(num_experts, **i32)
        self._all_counts = torch.empty((self.world, num_experts), **i32) if self.distributed else self._counts.view(1, -1)
        self._pair_base = torch.empty(num_experts, **i32)
        self.group_ends = torch.empty(self.local_experts, **i32)
        self.totals = torch.zeros(4, **i32)          # arena rows in use, valid rows, overflow flag, largest arena
        self.pos_of_pair = torch.empty(self.max_pairs, **i32)
        self._fence_word = torch.zeros(1, **i32)
        self._experts = None
        self._tokens = 0
        self.max_blocks = 0                           # grid bound of the dispatch / combine kernels (0: as many blocks as items)
        self._fence()                                 # every rank's buffers are mapped and cleared before the first step

    def _fence(self):
        """Orders the ranks on the stream: what each wrote before is visible to all after."""
        if self.distributed:
            self._check_stream()
            dist.all_reduce(self._fence_word, group=self.group)

    def _check_stream(self):
        """The collectives that order the ranks run on torch's current stream, the library's kernels on the context's
        stream: the two must be the same stream, or nothing orders a peer's stores against this rank's GEMM."""
        current = torch.cuda.current_stream(self.device).cuda_stream
        if (self.ctx.stream or 0) != (current or 0):
            raise RuntimeError("PeerExpertParallel: the context's stream is not torch's current stream on this device; create the "
                               "DgContext on the stream the step runs on, or wrap the step in torch.cuda.stream(...)")

    def operand(self):
        """The arena as the grouped GEMMs' A: `capacity` rows, of which the group table bounds the work (masked layout: one
        slot of `slot_rows` rows per local expert, as the masked GEMM wants it)."""
        if self.slot_rows:
            return self.dg.LpOperand(self.arena, self.arena_sf, self.slot_rows, self.hidden, self.hidden, 8, self.gran)
        return self.dg.LpOperand(self.arena, self.arena_sf, self.capacity, self.hidden, self.hidden, 8, self.gran)

    def dispatch(self, topk_idx: torch.Tensor, xq: torch.Tensor, xsf: torch.Tensor, sf_stride: Optional[int] = None):
        """This rank's e4m3 token rows + packed scales -> arena rows on the expert ranks.  Returns (operand, group_ends).
        sf_stride: words between two scale columns of xsf (default: the packed layout of exactly these tokens); a larger
        value lets xsf point into the scale words of a longer token batch."""
        dg, ctx = self.dg, self.ctx
        tokens, topk = topk_idx.shape
        pairs = tokens * topk
        if topk != self.topk or pairs > self.max_pairs:
            raise ValueError(f"routing of shape {tuple(topk_idx.shape)} exceeds what this exchange was built for")
        self._experts = topk_idx.reshape(-1).to(torch.int32)
        self._tokens = tokens
        dg.ep_count_dev(ctx, self._experts, pairs, self.num_experts, self._local_rank, self._block_hist, self._counts)
        if self.distributed:
            dist.all_gather_into_tensor(self._all_counts, self._counts, group=self.group)
        dg.ep_layout_dev(ctx, self._all_counts, self.world, self.rank, self.num_experts, self.alignment, self.capacity, self._pair_base,
                         self.group_ends, self.totals, self.slot_rows)
        dg.ep_dispatch_dev(ctx, self._experts, self._local_rank, self._block_hist, self._pair_base, pairs, topk, self.num_experts, self.world,
                           xq, self.hidden, xsf, sf_stride or dg.sf_aligned_rows(tokens), self.sf_cols, self._peer_data, self._peer_sf, self.sf_stride,
                           self.capacity, self.pos_of_pair, self.max_blocks, self.slot_rows)
        self._fence()
        return self.operand(), self.group_ends

    def combine(self, weights: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`result` rows of all ranks (the last grouped GEMM wrote them) -> per-token weighted sums on the token ranks
        (written to `out` (tokens, out_n) bf16 if given)."""
        self._fence()
        if out is None:
            out = torch.empty((self._tokens, self.out_n), dtype=torch.bfloat16, device=self.device)
        self.dg.ep_combine_dev(self.ctx, self._experts, self.pos_of_pair, weights, self._tokens, self.topk, self.num_experts, self.world,
                               self._peer_rows, self.out_n, self.out_n, out, self.out_n, self.max_blocks)
        return out

    def overflowed(self) -> bool:
        """Host read: did the last dispatch need more arena rows than `capacity` on some rank?"""
        return bool(self.totals[2].item())

    def close(self):
        if self._base is None:
            return
        torch.cuda.synchronize(self.device)
        self._fence()
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self.dg.peer_close(self.ctx, p)
        self._opened = []
        if self.distributed:
            dist.barrier(group=self.group)
        self.arena = self.arena_sf = self.result = None
        self.dg.peer_free(self.ctx, self._base)
        self._base = None


class PipelinedPeerMoe:
    """A MoE layer over `PeerExpertParallel` in `chunks` token micro-batches: the peer-memory dispatch and combine of one
    micro-batch run on a second stream while the grouped GEMMs of another run on the caller's stream.

    compute(exchange, a_op, group_ends) is the caller's expert computation for one micro-batch: it must enqueue, on the
    compute context's stream, work that reads the arena operand and leaves the result rows in `exchange.result`.
    Every micro-batch has its own exchange buffers, so nothing of one micro-batch is overwritten while another is in
    flight; all collectives are issued from the exchange stream in the same order on every rank.  A token's output does
    not depend on which micro-batch it travelled in (rows are independent in the GEMMs and the reduction order is the
    token's own top-k order), so the result equals the unchunked step bit for bit.
    """

    def __init__(self, compute_ctx, num_experts: int, topk: int, max_tokens: int, hidden: int, out_n: int, chunks: int = 2, gran: int = 128,
                 group: Optional[dist.ProcessGroup] = None, alignment: int = 128, blocks_per_sm: int = 2):
        import deepgemm_rust_b200 as dg
        self.dg, self.chunks = dg, chunks
        self.compute_ctx = compute_ctx
        self.device = torch.device(f"cuda:{compute_ctx.ordinal}")
        self.chunk_tokens = (max_tokens + chunks - 1) // chunks
        self.side = torch.cuda.Stream(device=self.device)
        self.exchange_ctx = dg.DgContext(compute_ctx.ordinal, stream=self.side.cuda_stream)
        with torch.cuda.stream(self.side):
            self.exchanges = [PeerExpertParallel(self.exchange_ctx, num_experts, topk, self.chunk_tokens, hidden, out_n, gran, group, alignment)
                              for _ in range(chunks)]
        self.side.synchronize()
        # the exchange kernels run beside a persistent GEMM that needs one block slot and most of the shared memory of
        # every SM: two 256-thread blocks per SM move rows fast enough for NVLink and leave that slot free
        for e in self.exchanges:
            e.max_blocks = blocks_per_sm * compute_ctx.num_sms()
        self.out_n = out_n

    def run(self, topk_idx: torch.Tensor, xq: torch.Tensor, xsf: torch.Tensor, weights: torch.Tensor, compute) -> torch.Tensor:
        dg = self.dg
        tokens = topk_idx.shape[0]
        main = torch.cuda.current_stream(self.device)
        out = torch.empty((tokens, self.out_n), dtype=torch.bfloat16, device=self.device)
        bounds = [(c * self.chunk_tokens, min(tokens, (c + 1) * self.chunk_tokens)) for c in range(self.chunks)]
        bounds = [b for b in bounds if b[0] < b[1]]
        sf_stride = dg.sf_aligned_rows(tokens)
        self.side.wait_stream(main)                      # the inputs were produced on the caller's stream
        landed, computed = [], []
        with torch.cuda.stream(self.side):
            for c, (t0, t1) in enumerate(bounds):
                # a micro-batch's scale words are columns [t0, t1) of the packed (sf_cols, align4(tokens)) matrix: same stride, offset base
                a_op, ends = self.exchanges[c].dispatch(topk_idx[t0:t1], xq[t0:t1], xsf.view(-1)[t0:], sf_stride)
                ev = torch.cuda.Event()
                ev.record(self.side)
                landed.append((a_op, ends, ev))
        for c in range(len(bounds)):
            a_op, ends, ev = landed[c]
            main.wait_event(ev)
            compute(self.exchanges[c], a_op, ends)
            done = torch.cuda.Event()
            done.record(main)
            computed.append(done)
        with torch.cuda.stream(self.side):
            for c, (t0, t1) in enumerate(bounds):
                self.side.wait_event(computed[c])
                self.exchanges[c].combine(weights[t0:t1], out[t0:t1])
        main.wait_stream(self.side)
        return out

    def routed_rows(self) -> int:
        return sum(int(e.totals[1].item()) for e in self.exchanges)

    def close(self):
        with torch.cuda.stream(self.side):          # the exchanges' context lives on the side stream, and so do their fences
            for e in self.exchanges:
                e.close()
        self.exchanges = []
        self.exchange_ctx.close()
