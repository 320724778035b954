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
* 'rows' (alpha = 0): only kernel A (error feedback, top-k) is sharded.  The window of all tensors
  sits in one buffer per rank with one equally wide region per rank in every row; every rank fills
  its region of the row a step produces (4 bytes per selected value, 0.04 bytes per parameter at
  k = 1 %), one in-place all-gather completes the row, and every rank then runs kernel B over all
  parameters.  The error-feedback state stays sharded, the window
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
        """State of the 'rows' mode.

        One int16 buffer holds the whole window, laid out [m rows][world regions][I | V][width] with one region per
        rank: a rank's pieces write their columns side by side into its region (indices in the I half, bf16 value
        bits in the V half).  Regions have one width (the widest rank's column count, padded to 128 bytes), so the
        row a step produces is exchanged by one in-place all-gather over that row.  Error feedback and block
        statistics exist for the owned pieces only; every rank describes every piece to kernel B."""
        params = self._all_params
        dev = params[0].device
        W = self.world_size
        pieces = [pc for pc in self.plan if pc.hi > pc.lo]
        cols = [0] * W
        self._rows_pieces = []                                 # (piece, geometry, first column inside the owner's region)
        for pc in pieces:
            g = self._geometry(pc.hi - pc.lo)
            self._rows_pieces.append((pc, g, cols[pc.rank]))
            cols[pc.rank] += g['k']
        self._rank_cols = cols
        self._width = -(-(max(cols) + 8) // 64) * 64           # elements per half region
        self._pitch = W * 2 * self._width                      # elements between consecutive rows
        if self._pitch >= 2 ** 31:
            raise ValueError('too many window columns for one buffer')
        # 64 elements of slack behind the last row: kernel B stages whole 16-byte pieces around a slice
        self._window = torch.zeros(self.m * self._pitch + 64, dtype=torch.int16, device=dev)
        self._dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
        self._ring = 0
        self._rows_state = {}                                  # (parameter index, lo) -> error feedback of an owned piece
        for pc, g, col in self._rows_pieces:
            p = params[pc.index]
            if pc.rank != self.rank:
                continue
            nq, _ = block_split(g['d'], self.quant_block_size)
            base = pc.rank * 2 * self._width + col
            rows = self._window[:self.m * self._pitch].view(self.m, self._pitch)
            st = self.state[p]
            st.update(d=g['d'], d_block_size=g['d_block_size'], topk_full_blocks_count=g['nfull'], k=g['k'],
                      k_block_size_many=g['k_many'], k_block_size_few=g['k_few'], index=0,
                      shard_lo=pc.lo, shard_hi=pc.hi,
                      I=rows[:, base:base + g['k']], V=rows[:, base + self._width:base + self._width + g['k']].view(torch.bfloat16),
                      error=torch.zeros((g['d'] + 1) // 2, dtype=torch.uint8, device=dev),
                      min_vals=torch.zeros(nq + 1, dtype=torch.bfloat16, device=dev),
                      max_vals=torch.zeros(nq + 1, dtype=torch.bfloat16, device=dev))
            self._rows_state[(pc.index, pc.lo)] = st
        self._rows_descs = None

    def _rows_fill(self):
        """Descriptor arrays of the two kernels: owned pieces for kernel A, every piece of every rank for kernel B."""
        params = self._all_params
        a_pieces = [x for x in self._rows_pieces if x[0].rank == self.rank]
        for pc, _, _ in a_pieces:
            if params[pc.index].grad is None:
                raise RuntimeError(f"exchange='rows': parameter {pc.index} has no gradient on rank {self.rank}, which owns "
                                   f"elements [{pc.lo}, {pc.hi}) of it; every rank must provide the gradients of its own slices "
                                   "on every step (the window advances for all tensors together)")
        gdt = tuple((params[pc.index].grad.dtype if params[pc.index].grad is not None else params[pc.index].dtype)
                    for pc, _, _ in self._rows_pieces)
        if self._rows_descs is None or self._rows_descs[0] != gdt:
            da, db = (N.MabTensor * max(1, len(a_pieces)))(), (N.MabTensor * max(1, len(self._rows_pieces)))()
            wptr = self._window.data_ptr()
            for descs, its in ((da, a_pieces), (db, self._rows_pieces)):
                for d, (pc, g, col) in zip(descs, its):
                    base = pc.rank * 2 * self._width + col
                    d.I, d.V = wptr + 2 * base, wptr + 2 * (base + self._width)
                    d.d, d.k, d.d_block_size = g['d'], g['k'], g['d_block_size']
                    d.topk_full_blocks_count, d.k_block_size_many, d.k_block_size_few = g['nfull'], g['k_many'], g['k_few']
                    d.row_pitch = self._pitch
            for d, (pc, g, col) in zip(da, a_pieces):
                st = self._rows_state[(pc.index, pc.lo)]
                d.error, d.min_vals, d.max_vals = st['error'].data_ptr(), st['min_vals'].data_ptr(), st['max_vals'].data_ptr()
            for d in db:
                d.error = d.min_vals = d.max_vals = self._dummy.data_ptr()      # not read when alpha == 0
            self._rows_descs = (gdt, a_pieces, da, db)
        _, a_pieces, da, db = self._rows_descs
        group_of = {id(p): g for g in self.param_groups for p in g['params']}
        for descs, its, with_grad in ((da, a_pieces, True), (db, self._rows_pieces, False)):
            for d, (pc, g, col), in zip(descs, its):
                p = params[pc.index]
                if not p.is_cuda:
                    raise N.NativeError(f'parameter on {p.device}: MicroAdam for B200 has no CPU implementation')
                if not p.is_contiguous() or (p.grad is not None and not p.grad.is_contiguous()):
                    raise N.NativeError('parameters and gradients must be contiguous')
                grp = group_of[id(p)]
                d.param = p.data_ptr() + pc.lo * p.element_size()
                d.param_dtype = N.dtype_code(p)
                if p.grad is not None:
                    d.grad = p.grad.data_ptr() + pc.lo * p.grad.element_size()
                    d.grad_dtype = N.dtype_code(p.grad)
                else:                                          # kernel B only needs the element type the update is rounded to
                    d.grad = d.param
                    d.grad_dtype = d.param_dtype
                d.ring_index = self._ring
                d.lr, d.weight_decay = float(grp['lr']), float(grp.get('weight_decay', self.weight_decay))
        return a_pieces, da, db

    def _rows_call(self, fn_name, descs, n, probe=None):
        if n == 0:
            return
        lib = N.load()
        device = self._all_params[0].device
        args = self._step_args()
        need = lib.mab_fused_step_workspace_bytes_for(descs, n, ctypes.byref(args))
        ws = self._rows_ws.get(fn_name)
        if ws is None or ws.numel() < need:
            ws = self._rows_ws[fn_name] = torch.empty(need, dtype=torch.uint8, device=device)
        if probe is not None:
            args.probe_out = probe['buf'].data_ptr()
        with torch.cuda.device(device):
            N.check(getattr(lib, fn_name)(descs, n, ctypes.byref(args), ws.data_ptr(), ws.numel(), N.current_stream(device)), fn_name)

    def rows_phase_a(self, probe=None):
        """Kernel A on the owned pieces: writes this rank's region of row `ring` of the window.  On a logging step it is
        followed by the probes of the owned gradients and error feedback."""
        a_pieces, da, _ = self._rows_fill()
        self._rows_call('mab_fused_ef_topk_quant', da, len(a_pieces), probe)

    def current_row(self) -> torch.Tensor:
        """The row of the window this step writes, [world, 2 * width] int16: region r is rank r's to fill."""
        return self._window[self._ring * self._pitch:(self._ring + 1) * self._pitch].view(self.world_size, 2 * self._width)

    def rows_exchange(self) -> int:
        """Every rank's region of the current row travels to all others: one in-place all-gather.  Returns the bytes
        this rank received."""
        return gather_row_regions(self.current_row(), self.rank, self.process_group)

    def rows_phase_b(self, probe=None):
        """Kernel B over all parameters, then the ring advances.  Every rank computes the same update, so on a logging
        step only rank 0 takes its probes (the log sums over the ranks)."""
        _, _, db = self._rows_fill()
        self._rows_call('mab_fused_window_adam_update', db, len(self._rows_pieces), probe if self.rank == 0 else None)
        self._ring = (self._ring + 1) % self.m
        for st in self._rows_state.values():
            st['index'] = self._ring

    def rows_prepare(self):
        """Allocates the state of the 'rows' mode (done by the first step otherwise)."""
        if not hasattr(self, '_rows_pieces'):
            self._rows_ws = {}
            self._rows_setup()

    def _rows_step(self):
        self.rows_prepare()
        probe = self._probe_begin()
        if probe is not None and probe['buf'] is None:
            probe['buf'] = torch.zeros(N.MAB_PROBE_SLOTS, dtype=torch.float64, device=self._all_params[0].device)
        ev = None
        if self.kernel_events is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
        self.rows_phase_a(probe)
        if ev:
            ev[1].record()
        if self.gather:
            self.last_gather_bytes = self.rows_exchange()
        if ev:
            ev[2].record()
        self.rows_phase_b(probe)
        if ev:
            ev[3].record()
            self.kernel_events.append(('rows', ev))
        self._probe_end(probe)

    # ---------------------------------------------------------------------------- checkpoint of the 'rows' mode
    def state_dict(self):
        """'rows' mode: the replicated window, the ring position, the step counter and the error feedback of the
        owned pieces, keyed by (parameter index, first element); a checkpoint belongs to one (rank, world size)."""
        if self.exchange != 'rows':
            return super().state_dict()
        self.rows_prepare()
        return {'exchange': 'rows', 'rank': self.rank, 'world_size': self.world_size, 'steps': self.steps, 'ring': self._ring,
                'm': self.m, 'width': self._width, 'window': self._window.clone(),
                'pieces': {key: {k: st[k].clone() for k in ('error', 'min_vals', 'max_vals')} for key, st in self._rows_state.items()},
                'param_groups': super().state_dict()['param_groups']}

    def load_state_dict(self, state_dict):
        if self.exchange != 'rows':
            return super().load_state_dict(state_dict)
        if state_dict.get('exchange') != 'rows':
            raise ValueError("this optimizer exchanges window rows; the checkpoint was not written in that mode")
        self.rows_prepare()
        if (state_dict['rank'], state_dict['world_size'], state_dict['m'], state_dict['width']) != (self.rank, self.world_size, self.m, self._width):
            raise ValueError('checkpoint of another rank, world size or window geometry')
        if set(state_dict['pieces']) != set(self._rows_state):
            raise ValueError('checkpoint holds other pieces than this rank owns')
        if not (0 <= int(state_dict['ring']) < self.m):
            raise ValueError(f"ring position {state_dict['ring']} outside [0, {self.m})")
        win = state_dict['window']
        if win.dtype != torch.int16 or win.shape != self._window.shape:
            raise TypeError('window of the checkpoint has another element type or shape')
        self._check_rows_window(win)
        for key, saved in state_dict['pieces'].items():
            st = self._rows_state[key]
            for k in ('error', 'min_vals', 'max_vals'):
                if saved[k].dtype != st[k].dtype or saved[k].shape != st[k].shape:
                    raise TypeError(f"'{k}' of piece {key} has another element type or shape")
        self._window.copy_(win)                                # in place: the descriptors and the state views stay valid
        for key, saved in state_dict['pieces'].items():
            for k in ('error', 'min_vals', 'max_vals'):
                self._rows_state[key][k].copy_(saved[k])
        self._ring = int(state_dict['ring'])
        for st in self._rows_state.values():
            st['index'] = self._ring
        self.steps = int(state_dict['steps'])
        for g, saved in zip(self.param_groups, state_dict['param_groups']):
            g.update({k: v for k, v in saved.items() if k != 'params'})

    def _check_rows_window(self, win: torch.Tensor):
        """Every index of every piece (all ranks: kernel B reads them all) must lie inside its block."""
        rows = win[:self.m * self._pitch].view(self.m, self._pitch)
        for pc, g, col in self._rows_pieces:
            base = pc.rank * 2 * self._width + col
            I = rows[:, base:base + g['k']]
            k_index = g['nfull'] * g['k_many']
            tail = g['d'] - g['nfull'] * g['d_block_size']
            bad = bool((I < 0).any())
            if k_index > 0:
                bad |= bool((I[:, :k_index] >= g['d_block_size']).any())
            if g['k'] > k_index:
                bad |= bool((I[:, k_index:] >= max(tail, 1)).any())
            if bad:
                raise ValueError(f'window of the checkpoint holds an index outside its top-k block (parameter {pc.index})')

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
        probe = self._probe_begin()
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
                self._fused_step(fused, group_key=ci, probe=probe)
            for e in entries:
                if not e.fused:
                    self._generic_update(e, probe)
            ready = torch.cuda.Event()
            ready.record(compute)
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                received += exchange_pieces(views, self.rank, self.process_group)
        compute.wait_stream(self._comm_stream)
        self._probe_end(probe)
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
    """Sums (averages) every planned range of `tensors` over the ranks into its owner, in place: a reduce-scatter
    with unequal pieces.  When every rank's ranges merge into one view (tensors that are slices of one flat
    buffer) and the backend is NCCL, that is one `reduce_scatter` call whose per-rank inputs are the views
    themselves (nothing is copied or padded); otherwise one reduce per owned view, all in flight together.
    Returns the bytes this rank owns."""
    if world_size == 1:
        return 0
    views = build_gather_views(plan, tensors, world_size)
    if dist.get_backend(group) == 'nccl' and all(len(vs) == 1 for vs in views):
        dist.reduce_scatter(views[rank][0], [vs[0] for vs in views], op=dist.ReduceOp.SUM, group=group)
    else:
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


def gather_row_regions(row: torch.Tensor, rank: int, group=None) -> int:
    """`row` is [world, n] and contiguous, region `rank` filled in: all-gathers the regions in place (NCCL's
    in-place convention: the send buffer is the rank's own slot of the receive buffer).  Returns the bytes received."""
    row = row.view(torch.uint8)                                # the collectives move no int16
    mine = row[rank]
    if dist.get_backend(group) != 'nccl':
        mine = mine.clone()
    dist.all_gather_into_tensor(row.view(-1), mine, group=group)
    return (row.shape[0] - 1) * mine.numel()


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
