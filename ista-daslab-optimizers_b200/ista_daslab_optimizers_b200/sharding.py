"""ZeRO-1 style sharding of the MicroAdam step over the GPUs of one node.

The reference has no counterpart (its only multi-GPU provision is to size the state lazily so
that FSDP shards work, micro_adam.py:158-160).  Every top-k block of a tensor is an independent
unit of the step: its window rows, error-feedback codes and block statistics depend on nothing
outside the block.  So the flattened parameter list is cut into `world_size` contiguous runs of
top-k blocks, balanced by element count; a rank keeps optimizer state only for its run, updates
only those parameters, and the updated ranges are then exchanged so that every rank again holds
all parameters (one all-gather with unequal pieces).

Two ways to exchange (`exchange=`):

* 'params' (any alpha): the owner runs both kernels on its slices and the updated parameter ranges
  travel, (N-1)/N of all parameter bytes into every GPU per step;
* 'rows' (alpha = 0): only kernel A (error feedback, top-k) is sharded.  The window rows of all
  tensors sit side by side in one buffer per rank, every rank sends the columns of the row it
  just produced (4 bytes per selected value, 0.04 bytes per parameter at k = 1 %), and every rank
  then runs kernel B over all parameters.  The error-feedback state stays sharded, the window
  (0.4 bytes per parameter at m = 10, k = 1 %) is replicated, and no parameter crosses a link.

A cut inside a tensor is made only on a top-k block boundary that is also a quantisation block
boundary, so a rank's slice of a tensor behaves exactly like a smaller tensor of its own and the
sharded result is bit-identical to the unsharded one.  Tensors where that is impossible
(d_block_size not a multiple of quant_block_size, or a single block) are never cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import ctypes
import math

import torch
import torch.distributed as dist

from . import _native as N
from .micro_adam import MicroAdam
from .tools import block_split


@dataclass(frozen=True)
class Piece:
    """Flat element range [lo, hi) of parameter `index`, owned by `rank`."""
    rank: int
    index: int
    lo: int
    hi: int


def plan_shards(numels: Sequence[int], d_block_size: int, quant_block_size: int, world_size: int) -> List[Piece]:
    """Cuts the parameter list into world_size contiguous runs of top-k blocks.

    A block goes to rank floor(midpoint * world_size / total), where midpoint is the position of
    the block's middle in the concatenation of all tensors: ranks are non-decreasing along the
    list, every rank's share is within one block of total / world_size, and the plan depends only
    on the sizes, so every rank computes the same one.
    """
    total = sum(numels)
    pieces: List[Piece] = []
    if total == 0:
        return pieces
    start = 0
    for idx, d in enumerate(numels):
        if d == 0:
            continue
        splittable = d > d_block_size and d_block_size % quant_block_size == 0
        if not splittable:
            r = min(world_size - 1, (2 * start + d) * world_size // (2 * total))
            pieces.append(Piece(r, idx, 0, d))
        else:
            nblocks = -(-d // d_block_size)
            # first block of rank r: smallest b with (2*(start + b*dbs) + len_b) * W >= 2*total*r
            cuts = [0]
            for r in range(1, world_size):
                # with full-size blocks: 2*start + (2b+1)*dbs >= 2*total*r / W
                num = 2 * total * r - world_size * (2 * start + d_block_size)
                b = 0 if num <= 0 else -(-num // (2 * d_block_size * world_size))
                cuts.append(min(max(b, cuts[-1]), nblocks))
            cuts.append(nblocks)
            # the last block may be short: its midpoint is earlier than the formula assumes, which can
            # only move it to an earlier rank; recheck it explicitly
            last_lo = (nblocks - 1) * d_block_size
            last_rank = min(world_size - 1, (2 * (start + last_lo) + (d - last_lo)) * world_size // (2 * total))
            for r in range(world_size):
                b0, b1 = cuts[r], cuts[r + 1]
                if r > last_rank and b1 == nblocks and b0 < nblocks:
                    b0 = b1 = nblocks                      # handled by last_rank below
                if b0 < b1:
                    lo, hi = b0 * d_block_size, min(d, b1 * d_block_size)
                    if b1 == nblocks and r != last_rank:
                        hi = last_lo                        # the short block belongs to last_rank
                    if lo < hi:
                        pieces.append(Piece(r, idx, lo, hi))
            if not any(p.index == idx and p.hi == d for p in pieces):
                # the short block alone (or appended to last_rank's run)
                prev = [p for p in pieces if p.index == idx and p.rank == last_rank]
                if prev and prev[-1].hi == last_lo:
                    pieces[pieces.index(prev[-1])] = Piece(last_rank, idx, prev[-1].lo, d)
                else:
                    pieces.append(Piece(last_rank, idx, last_lo, d))
        start += d
    pieces.sort(key=lambda p: (p.index, p.lo))
    return pieces


def block_geometry(d: int, d_block_size: int, k_init: float) -> dict:
    """Block geometry of a flat range of d elements (micro_adam.py:70-84)."""
    dbs = d if d < d_block_size else d_block_size
    nfull, d_index = block_split(d, dbs)
    k_many = int(math.ceil(dbs * k_init))
    k_few = int(math.ceil((d - d_index) * k_init))
    return dict(d=d, d_block_size=dbs, nfull=nfull if d_index > 0 else 0, k_many=k_many, k_few=k_few,
                k=k_many * nfull + k_few)


def plan_row_columns(numels: Sequence[int], plan: Sequence[Piece], d_block_size: int, k_init: float, world_size: int):
    """Where the window rows of all tensors sit in one [m, sum k] buffer: (first column of every tensor and the
    total, first column of every piece of the plan, the contiguous column range of every rank)."""
    geos = [block_geometry(n, d_block_size, k_init) for n in numels]
    col = [0]
    for g in geos:
        col.append(col[-1] + g['k'])
    piece_col = {}
    per_rank = [[] for _ in range(world_size)]
    for pc in plan:
        if pc.hi > pc.lo:
            g = geos[pc.index]
            c0 = col[pc.index] + (pc.lo // g['d_block_size']) * g['k_many']
            piece_col[(pc.index, pc.lo)] = c0
            per_rank[pc.rank].append((c0, c0 + block_geometry(pc.hi - pc.lo, d_block_size, k_init)['k']))
    rank_cols = []
    for cols in per_rank:
        for (a0, a1), (b0, b1) in zip(cols, cols[1:]):
            if a1 != b0:
                raise AssertionError("a rank's window columns must be contiguous")
        rank_cols.append((cols[0][0], cols[-1][1]) if cols else (0, 0))
    return col, piece_col, rank_cols


class ShardedMicroAdam(MicroAdam):
    """MicroAdam whose state and update are sharded over the ranks of `process_group`.

    Every rank constructs it over the same full parameter list and, each step, provides the
    gradients of (at least) its own slices in `p.grad`.  After `step()` every rank holds all updated
    parameters.  `rank` / `world_size` may be given explicitly without a process group to run one
    shard on its own (no exchange), which is how the sharded arithmetic is tested on one GPU.
    """

    def __init__(self, params, m, lr, quant_block_size, k_init=0.01, alpha=0, betas=(0.9, 0.999), weight_decay=0,
                 eps=1e-8, *, process_group=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 gather: bool = True, overlap_chunks: int = 6, exchange: str = 'params', **kw):
        super().__init__(params, m, lr, quant_block_size, k_init, alpha, betas, weight_decay, eps, **kw)
        if exchange not in ('params', 'rows'):
            raise ValueError("exchange must be 'params' or 'rows'")
        if exchange == 'rows' and (self.alpha != 0 or not self.use_fused):
            raise ValueError("exchange='rows' needs alpha == 0 and the fused kernels (the alpha term reads the "
                             "error feedback of every element, which only its owner holds)")
        self.exchange = exchange
        self.process_group = process_group
        if rank is None or world_size is None:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError('ShardedMicroAdam needs torch.distributed initialised, or explicit rank and world_size')
            rank, world_size = dist.get_rank(process_group), dist.get_world_size(process_group)
        self.rank, self.world_size = int(rank), int(world_size)
        self.gather = gather and self.world_size > 1
        self._all_params = [p for g in self.param_groups for p in g['params']]
        self.plan = plan_shards([p.numel() for p in self._all_params], self.d_block_size, self.quant_block_size,
                                self.world_size)
        self._my_slice: Dict[int, Tuple[int, int]] = {}
        for pc in self.plan:
            if pc.rank == self.rank:
                assert id(self._all_params[pc.index]) not in self._my_slice
                self._my_slice[id(self._all_params[pc.index])] = (pc.lo, pc.hi)
        self._gather_views = None
        self.last_gather_bytes = 0
        # the step runs in this many groups of pieces; a group's parameters travel while the next group is computed
        self.overlap_chunks = max(1, int(overlap_chunks))
        self._chunks = None
        self._comm_stream = None

    def _slice_of(self, p):
        return self._my_slice.get(id(p))

    # ---------------------------------------------------------------------------- gradients
    @torch.no_grad()
    def reduce_gradients(self, average: bool = True) -> int:
        """The gradient side of the shard plan: sums (or averages) every range of `p.grad` over the ranks
        into the rank that owns it, in place, instead of all-reducing whole gradients; only the owner's
        copy of a range is meaningful afterwards, and it is the only one the step reads.  Moves
        (N-1)/N of the gradient bytes once (a reduce-scatter with unequal pieces) where an all-reduce
        moves them twice.  Returns the bytes this rank owns."""
        grads = [p.grad for p in self._all_params]
        if any(g is None for g in grads):
            raise RuntimeError('reduce_gradients needs a gradient on every parameter')
        return reduce_to_owners(self.plan, grads, self.rank, self.world_size, self.process_group, average)

    def _after_update(self):
        if not self.gather:
            return
        if self._gather_views is None:
            self._gather_views = build_gather_views(self.plan, self._all_params, self.world_size)
        self.last_gather_bytes = exchange_pieces(self._gather_views, self.rank, self.process_group)

    # ---------------------------------------------------------------------------- overlapped step
    def _chunk_plan(self):
        """Every rank's pieces cut into `overlap_chunks` consecutive groups of about equal size (the same
        cut on every rank, computed from the plan alone), with the exchange views of each group."""
        if self._chunks is None:
            per_rank = [[pc for pc in self.plan if pc.rank == r] for r in range(self.world_size)]
            groups = [[[] for _ in range(self.world_size)] for _ in range(self.overlap_chunks)]
            for r, pieces in enumerate(per_rank):
                total = sum(pc.hi - pc.lo for pc in pieces) or 1
                done = 0
                for pc in pieces:
                    mid = done + (pc.hi - pc.lo) / 2
                    groups[min(self.overlap_chunks - 1, int(mid * self.overlap_chunks / total))][r].append(pc)
                    done += pc.hi - pc.lo
            self._chunks = []
            for g in groups:
                flat = [pc for r in range(self.world_size) for pc in g[r]]
                views = build_gather_views(flat, self._all_params, self.world_size)
                mine = {id(self._all_params[pc.index]) for pc in g[self.rank]}
                self._chunks.append((mine, views))
        return self._chunks

    # ---------------------------------------------------------------------------- exchange of window rows
    def _geometry(self, d: int) -> dict:
        return block_geometry(d, self.d_block_size, self.k_init)

    def _rows_setup(self):
        """State of the 'rows' mode: one I and one V buffer [m, sum of k] for all tensors, error feedback for
        the owned slices only; per-parameter state keeps the reference's key names (I, V are views)."""
        params = self._all_params
        dev = params[0].device
        geos = [self._geometry(p.numel()) for p in params]
        self._col, piece_col, self._rank_cols = plan_row_columns([p.numel() for p in params], self.plan, self.d_block_size,
                                                                 self.k_init, self.world_size)
        self._pitch = self._col[-1] + 64                     # slack: staging reads whole 16-byte pieces
        if self._pitch >= 2 ** 31:
            raise ValueError('too many window columns for one buffer')
        self._I_flat = torch.zeros(self.m, self._pitch, dtype=torch.int16, device=dev)
        self._V_flat = torch.zeros(self.m, self._pitch, dtype=torch.bfloat16, device=dev)
        self._dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
        self._ring = 0
        mine = {pc.index: pc for pc in self.plan if pc.rank == self.rank}
        self._rows_items = []
        for i, (p, g) in enumerate(zip(params, geos)):
            st = self.state[p]
            c0 = self._col[i]
            st.update(d=g['d'], d_block_size=g['d_block_size'], topk_full_blocks_count=g['nfull'], k=g['k'],
                      k_block_size_many=g['k_many'], k_block_size_few=g['k_few'], index=0,
                      I=self._I_flat[:, c0:c0 + g['k']], V=self._V_flat[:, c0:c0 + g['k']])
            item = dict(p=p, full=g, col=c0, piece=None)
            pc = mine.get(i)
            if pc is not None and pc.hi > pc.lo:
                sg = self._geometry(pc.hi - pc.lo)
                nq, _ = block_split(sg['d'], self.quant_block_size)
                st['shard_lo'], st['shard_hi'] = pc.lo, pc.hi
                st['error'] = torch.zeros((sg['d'] + 1) // 2, dtype=torch.uint8, device=dev)
                st['min_vals'] = torch.zeros(nq + 1, dtype=torch.bfloat16, device=dev)
                st['max_vals'] = torch.zeros(nq + 1, dtype=torch.bfloat16, device=dev)
                item['piece'] = (pc.lo, pc.hi, sg, piece_col[(pc.index, pc.lo)])
            self._rows_items.append(item)
        self._rows_descs = None

    def _rows_fill(self):
        """Descriptor arrays of the two kernels: owned slices for kernel A, whole tensors for kernel B."""
        items = [it for it in self._rows_items if it['p'].grad is not None]
        key = tuple((id(it['p']), it['p'].grad.dtype) for it in items)
        if self._rows_descs is None or self._rows_descs[0] != key:
            a_items = [it for it in items if it['piece'] is not None]
            da, db = (N.MabTensor * max(1, len(a_items)))(), (N.MabTensor * max(1, len(items)))()
            for d, it in zip(da, a_items):
                lo, hi, sg, col = it['piece']
                st = self.state[it['p']]
                d.error, d.min_vals, d.max_vals = st['error'].data_ptr(), st['min_vals'].data_ptr(), st['max_vals'].data_ptr()
                d.I, d.V = self._I_flat.data_ptr() + 2 * col, self._V_flat.data_ptr() + 2 * col
                d.d, d.k, d.d_block_size = sg['d'], sg['k'], sg['d_block_size']
                d.topk_full_blocks_count, d.k_block_size_many, d.k_block_size_few = sg['nfull'], sg['k_many'], sg['k_few']
                d.row_pitch = self._pitch
            for d, it in zip(db, items):
                g = it['full']
                d.error = d.min_vals = d.max_vals = self._dummy.data_ptr()      # not read when alpha == 0
                d.I, d.V = self._I_flat.data_ptr() + 2 * it['col'], self._V_flat.data_ptr() + 2 * it['col']
                d.d, d.k, d.d_block_size = g['d'], g['k'], g['d_block_size']
                d.topk_full_blocks_count, d.k_block_size_many, d.k_block_size_few = g['nfull'], g['k_many'], g['k_few']
                d.row_pitch = self._pitch
            self._rows_descs = (key, a_items, da, items, db)
        _, a_items, da, items, db = self._rows_descs
        group_of = {id(p): g for g in self.param_groups for p in g['params']}
        for descs, its, sliced in ((da, a_items, True), (db, items, False)):
            for d, it in zip(descs, its):
                p, g = it['p'], it['p'].grad
                if not (p.is_contiguous() and g.is_contiguous()):
                    raise N.NativeError('parameters and gradients must be contiguous')
                if not p.is_cuda:
                    raise N.NativeError(f'parameter on {p.device}: MicroAdam for B200 has no CPU implementation')
                lo = it['piece'][0] if sliced else 0
                grp = group_of[id(p)]
                d.param, d.grad = p.data_ptr() + lo * p.element_size(), g.data_ptr() + lo * g.element_size()
                d.param_dtype, d.grad_dtype = N.dtype_code(p), N.dtype_code(g)
                d.ring_index = self._ring
                d.lr, d.weight_decay = float(grp['lr']), float(grp.get('weight_decay', self.weight_decay))
        return a_items, da, items, db

    def _rows_call(self, fn_name, descs, n):
        if n == 0:
            return
        lib = N.load()
        device = self._all_params[0].device
        need = lib.mab_fused_step_workspace_bytes(n)
        ws = self._rows_ws.get(fn_name)
        if ws is None or ws.numel() < need:
            ws = self._rows_ws[fn_name] = torch.empty(need, dtype=torch.uint8, device=device)
        args = self._step_args()
        with torch.cuda.device(device):
            N.check(getattr(lib, fn_name)(descs, n, ctypes.byref(args), ws.data_ptr(), ws.numel(), N.current_stream(device)), fn_name)

    def rows_phase_a(self):
        """Kernel A on the owned slices: writes this rank's columns of row `ring` of I and V."""
        a_items, da, _, _ = self._rows_fill()
        self._rows_call('mab_fused_ef_topk_quant', da, len(a_items))

    def row_views(self) -> List[List[torch.Tensor]]:
        """Per rank, the columns of the current row of I and of V it owns, as contiguous byte views
        (NCCL moves no int16)."""
        return [[self._I_flat[self._ring, c0:c1].view(torch.uint8), self._V_flat[self._ring, c0:c1].view(torch.uint8)]
                if c1 > c0 else [] for c0, c1 in self._rank_cols]

    def rows_phase_b(self):
        """Kernel B over all parameters, then the ring advances."""
        _, _, items, db = self._rows_fill()
        self._rows_call('mab_fused_window_adam_update', db, len(items))
        self._ring = (self._ring + 1) % self.m
        for it in items:
            self.state[it['p']]['index'] = self._ring

    def rows_prepare(self):
        """Allocates the state of the 'rows' mode (done by the first step otherwise)."""
        if not hasattr(self, '_rows_items'):
            self._rows_ws = {}
            self._rows_setup()

    def _rows_step(self):
        self.rows_prepare()
        ev = None
        if self.kernel_events is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
        self.rows_phase_a()
        if ev:
            ev[1].record()
        if self.gather:
            self.last_gather_bytes = exchange_pieces(self.row_views(), self.rank, self.process_group)
        if ev:
            ev[2].record()
        self.rows_phase_b()
        if ev:
            ev[3].record()
            self.kernel_events.append(('rows', ev))

    @torch.no_grad()
    def step(self, closure=None):
        if self.exchange == 'rows':
            self.steps += 1
            loss = None
            if closure is not None:
                with torch.enable_grad():
                    loss = closure()
            self._rows_step()
            return loss
        if not self.gather or self.overlap_chunks <= 1 or dist.get_backend(self.process_group) != 'nccl':
            return super().step(closure)
        self.steps += 1
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._refresh_entries()
        device = self._all_params[0].device
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        compute = torch.cuda.current_stream(device)
        self._comm_stream.wait_stream(compute)
        received = 0
        for ci, (mine, views) in enumerate(self._chunk_plan()):
            entries = [e for e in self._entries if id(e.p) in mine]
            fused = [e for e in entries if e.fused]
            if fused:
                self._fused_step(fused, group_key=ci)
            for e in entries:
                if not e.fused:
                    self._generic_update(e)
            ready = torch.cuda.Event()
            ready.record(compute)
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                received += exchange_pieces(views, self.rank, self.process_group)
        compute.wait_stream(self._comm_stream)
        self.last_gather_bytes = received
        if self.kernel_events:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.kernel_events.append(('step_end', ev))
        return loss


def build_gather_views(plan: Sequence[Piece], params: Sequence[torch.Tensor], world_size: int) -> List[List[torch.Tensor]]:
    """Per rank, flat views of the parameter ranges it owns.  Views adjacent in memory (parameters
    that are slices of one flat buffer) are merged, so that a flat model needs one view per rank."""
    per_rank: List[List[torch.Tensor]] = [[] for _ in range(world_size)]
    last: List[Optional[Tuple[int, int, int, torch.dtype]]] = [None] * world_size   # storage ptr, begin, end, dtype
    for pc in plan:
        p = params[pc.index]
        if not p.is_contiguous():
            raise RuntimeError('sharded parameters must be contiguous')
        es = p.element_size()
        storage = p.untyped_storage()
        sp = storage.data_ptr()
        begin = p.data_ptr() + pc.lo * es
        end = p.data_ptr() + pc.hi * es
        prev = last[pc.rank]
        if prev is not None and prev[0] == sp and prev[2] == begin and prev[3] == p.dtype:
            begin = prev[1]
            per_rank[pc.rank].pop()
        n = (end - begin) // es
        view = torch.empty(0, dtype=p.dtype, device=p.device).set_(storage, (begin - sp) // es, (n,))
        per_rank[pc.rank].append(view)
        last[pc.rank] = (sp, begin, end, p.dtype)
    return per_rank


def reduce_to_owners(plan: Sequence[Piece], tensors: Sequence[torch.Tensor], rank: int, world_size: int, group=None,
                     average: bool = True) -> int:
    """Sums (averages) every planned range of `tensors` over the ranks into its owner, in place (one reduce per
    owned view, all in flight together).  Returns the bytes this rank owns."""
    if world_size == 1:
        return 0
    views = build_gather_views(plan, tensors, world_size)
    works = []
    for r, vs in enumerate(views):
        dst = dist.get_global_rank(group, r) if group is not None else r
        for v in vs:
            works.append(dist.reduce(v, dst=dst, op=dist.ReduceOp.SUM, group=group, async_op=True))
    for w in works:
        w.wait()
    if average:
        for v in views[rank]:
            v.div_(world_size)
    return sum(v.numel() * v.element_size() for v in views[rank])


def exchange_pieces(views: List[List[torch.Tensor]], rank: int, group=None) -> int:
    """Every rank sends the ranges it owns (views[rank]) to all others, in place: an all-gather with
    unequal pieces.  NCCL: grouped point-to-point sends and receives; other backends: one broadcast
    per view.  Returns the bytes this rank received."""
    received = sum(v.numel() * v.element_size() for r, vs in enumerate(views) if r != rank for v in vs)
    backend = dist.get_backend(group)
    if backend == 'nccl':
        # every rank sends its views to every peer and receives theirs in place, as one NCCL group: all
        # NVLink ports of every GPU are busy in both directions, whatever the sizes of the pieces
        world = len(views)
        ops = []
        for peer in range(world):
            if peer == rank:
                continue
            dst = dist.get_global_rank(group, peer) if group is not None else peer
            ops += [dist.P2POp(dist.isend, v, dst, group) for v in views[rank]]
            ops += [dist.P2POp(dist.irecv, v, dst, group) for v in views[peer]]
        for w in dist.batch_isend_irecv(ops) if ops else []:
            w.wait()
        return received
    works = []
    for r, vs in enumerate(views):
        src = dist.get_global_rank(group, r) if group is not None else r
        for v in vs:
            works.append(dist.broadcast(v, src=src, group=group, async_op=True))
    for w in works:
        w.wait()
    return received


def flatten_parameters(params: Sequence[torch.nn.Parameter]) -> torch.Tensor:
    """Re-homes the parameters (same dtype and device) as consecutive views of one flat buffer, each
    starting on a 256-byte boundary, and returns the buffer.  With flat parameters the exchange after
    a sharded step is one collective instead of one per tensor."""
    params = list(params)
    dtype, device = params[0].dtype, params[0].device
    es = params[0].element_size()
    align = 256 // es
    offsets, total = [], 0
    for p in params:
        if p.dtype != dtype or p.device != device:
            raise ValueError('flatten_parameters needs one dtype and one device')
        offsets.append(total)
        total += -(-p.numel() // align) * align
    flat = torch.zeros(total, dtype=dtype, device=device)
    for p, off in zip(params, offsets):
        view = flat[off:off + p.numel()].view(p.shape)
        view.copy_(p.data)
        p.data = view
    return flat
