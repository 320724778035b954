"""MicroAdam on B200: the reference's `torch.optim` interface over the sm_100a kernels.

Drop-in for `ista_daslab_optimizers.MicroAdam` (ista_daslab_optimizers/micro_adam/micro_adam.py:13-328):
same constructor, same per-parameter state keys, dtypes and shapes (micro_adam.py:61-94), same
order of sub-steps.  Differences a caller can observe:

* the step runs as two fused kernels over all tensors (plus the operator-level kernels for
  geometries the fused kernels do not cover), not ~25 launches per tensor;
* top-k ties go to the lower index and indices are stored in ascending order
  (torch.topk(sorted=False) at micro_adam.py:193-200 leaves both unspecified);
* on the fused path `p.grad` is left untouched (the reference uses it as scratch and leaves the
  update in it, micro_adam.py:276-313); on the operator-level path it is scratch as in the reference;
* a `quant_block_size` that is not a power of two in [8, 128] (the reference's README uses 100000) makes
  quantisation blocks ignore the borders of the top-k blocks (micro_adam.py:217-231).  With alpha == 0 and a
  multiple of 8 >= 64 the step is then three kernels (selection + residual, statistics + codes, update) and
  `p.grad` ends up holding the residual; other values take the operator-level kernels, with the update
  itself still fused when alpha == 0;
* alpha == -2 (micro_adam.py:238-273) keeps the residual in `quant_err` between the two fused kernels (gradient and
  parameter of one element type; other combinations take the operator-level path);
* the logging probes (micro_adam.py:155-156, 306-308, 320-324, 330-350) run only when a `log_fn` is given: every
  `log_interval` steps the fused kernels also sum the reference's quantities into a small device buffer (one more
  small kernel and one device-to-host read on such a step) and `log_fn` gets the dictionary the reference
  sends to wandb;
* `state_dict()` also carries the step counter (the reference loses it, micro_adam.py:35).

There is no CPU path: parameters must live on a CUDA device and the native library must be built.
"""
from __future__ import annotations

import ctypes
import math
import time
from typing import Dict, List, Optional, Tuple

import torch

from . import _native as N
from .tools import CopyDirection, block_split, get_first_device


class _Entry:
    """One flat slice of one parameter that this process updates."""
    __slots__ = ('p', 'st', 'lo', 'hi', 'fused', 'window_fused', 'group')

    def __init__(self, p, st, lo, hi, group):
        self.p, self.st, self.lo, self.hi, self.fused, self.group = p, st, lo, hi, False, group
        self.window_fused = False       # second half of the step (window -> update -> parameters) on the fused kernel


class MicroAdam(torch.optim.Optimizer):
    def __init__(self, params, m, lr, quant_block_size, k_init=0.01, alpha=0, betas=(0.9, 0.999), weight_decay=0,
                 eps=1e-8, *, d_block_size: Optional[int] = None, use_fused: bool = True, log_fn=None):
        defaults = dict(lr=lr, weight_decay=weight_decay, eps=eps, alpha=alpha)
        super().__init__(params, defaults)

        assert (0 <= alpha < 1) or alpha == -2, 'Alpha must be in the [0, 1) interval or -2'   # micro_adam.py:18
        if not (1 <= int(m) <= N.MAB_MAX_WINDOW):
            raise ValueError(f'm must be in [1, {N.MAB_MAX_WINDOW}]')

        self.m = int(m)
        self.lr = lr
        self.quant_block_size = int(quant_block_size)
        self.k_init = k_init
        self.alpha = alpha
        self.weight_decay = weight_decay
        self.beta1 = betas[0]
        self.beta2 = betas[1]
        self.eps = eps

        self.densify_update_using_ef = (self.alpha > 0)
        self.densify_update_using_quant_error = (self.alpha == -2)                                    # micro_adam.py:31

        self.model_size = sum(p.numel() for group in self.param_groups for p in group['params'])

        self.steps = 0
        self.log_interval = 100
        self.device = get_first_device()
        self.shared_memory_carveout = 100
        self.threads = 512
        self.use_fused = bool(use_fused)
        self.log_fn = log_fn      # callable(dict) or None; None (the default) switches the probes off

        N.load()   # fail here, loudly, if the native library is not built
        if d_block_size is None:
            self.blocks = N.get_sm_count() * int(100 / self.shared_memory_carveout)                  # micro_adam.py:40
            self.max_floats = N.get_max_floats_for_shared_memory_per_thread_block()                    # micro_adam.py:43
            self.d_block_size = self.max_floats // 2 // int(100 / self.shared_memory_carveout)       # micro_adam.py:44
        else:
            self.blocks = N.get_sm_count()
            self.d_block_size = int(d_block_size)
            self.max_floats = 2 * self.d_block_size

        self.dict_size_count: Dict[int, int] = {}                                                     # micro_adam.py:52-57
        for group in self.param_groups:
            for p in group['params']:
                self.dict_size_count[p.numel()] = 1 + self.dict_size_count.get(p.numel(), 0)

        self._entries: List[_Entry] = []
        self._entries_key: Optional[tuple] = None
        self._descs = {}          # descriptor arrays of the fused step, one per group of entries
        self._workspace: Optional[torch.Tensor] = None
        self._window_workspace: Optional[torch.Tensor] = None
        # set to a list to have every fused step append [start, between the two kernels, end] CUDA events
        self.kernel_events: Optional[list] = None

    # ------------------------------------------------------------------------------ state
    def _slice_of(self, p) -> Optional[Tuple[int, int]]:
        """Flat element range of `p` this process owns.  The whole tensor here; a sharded subclass
        returns a sub-range cut on top-k block boundaries, or None."""
        return 0, p.numel()

    def _initialize_parameter_state(self, p, lr, wd, lo: int = 0, hi: Optional[int] = None):
        """micro_adam.py:61-94, for the flat slice [lo, hi) of p (the whole tensor by default)."""
        hi = p.numel() if hi is None else hi
        layer_size = hi - lo
        st = self.state[p]
        dev = p.device

        st['blocks'] = max(1, int(math.floor(self.blocks * p.numel() * self.dict_size_count.get(p.numel(), 1) / self.model_size)))
        st['lr'] = lr
        st['weight_decay'] = wd
        st['d'] = layer_size

        st['d_block_size'] = layer_size if layer_size < self.d_block_size else self.d_block_size
        st['topk_full_blocks_count'], st['d_index_topk'] = block_split(st['d'], st['d_block_size'])
        st['k_block_size_many'] = int(math.ceil(st['d_block_size'] * self.k_init))
        st['k_block_size_few'] = int(math.ceil((st['d'] - st['d_index_topk']) * self.k_init))
        st['k_index'] = st['topk_full_blocks_count'] * st['k_block_size_many']
        st['k'] = st['k_block_size_many'] * st['topk_full_blocks_count'] + st['k_block_size_few']

        st['index'] = 0
        st['I'] = torch.zeros(self.m, st['k'], dtype=torch.int16, device=dev)
        st['V'] = torch.zeros(self.m, st['k'], dtype=torch.bfloat16, device=dev)

        st['quant_full_blocks_count'], st['d_index_quant'] = block_split(st['d'], self.quant_block_size)
        st['error'] = torch.zeros(int(math.ceil(st['d'] / 2)), dtype=torch.uint8, device=dev)
        st['min_vals'] = torch.zeros(st['quant_full_blocks_count'] + 1, dtype=torch.bfloat16, device=dev)
        st['max_vals'] = torch.zeros(st['quant_full_blocks_count'] + 1, dtype=torch.bfloat16, device=dev)
        if self.densify_update_using_quant_error:                                                      # micro_adam.py:67-68
            st['quant_err'] = torch.zeros(layer_size, dtype=p.dtype, device=dev)
        if (lo, hi) != (0, p.numel()):
            st['shard_lo'], st['shard_hi'] = lo, hi

    def state_dict(self):
        sd = super().state_dict()
        sd['steps'] = self.steps
        return sd

    # element type every tensor of the per-parameter state must keep (micro_adam.py:86-94)
    _STATE_DTYPES = {'I': torch.int16, 'V': torch.bfloat16, 'error': torch.uint8,
                     'min_vals': torch.bfloat16, 'max_vals': torch.bfloat16}

    def load_state_dict(self, state_dict):
        """Restores a state written by `state_dict()` of this class or of the reference class.

        `torch.optim.Optimizer.load_state_dict` casts every state tensor to the parameter's element type,
        which would turn the 4-bit codes, the int16 indices and the bf16 statistics into floats that the
        kernels then misread.  The tensors are therefore taken from the incoming dictionary again with the
        element types they were saved with (only the device changes), and checked: wrong element type or
        shape, or a window index outside its block, raises instead of reaching a kernel.  `I` saved in another
        element type (checkpoint pipelines that cast everything, micro_adam.py:175-178) is accepted if every
        value is an integer inside the block."""
        state_dict = dict(state_dict)
        steps = state_dict.pop('steps', None)
        super().load_state_dict(state_dict)
        saved_ids = [i for g in state_dict['param_groups'] for i in g['params']]
        params = [p for g in self.param_groups for p in g['params']]
        for sid, p in zip(saved_ids, params):
            saved = state_dict['state'].get(sid)
            if not saved or 'I' not in saved:
                continue
            st = self.state[p]
            for key, want in self._STATE_DTYPES.items():
                src = saved[key]
                if not torch.is_tensor(src):
                    raise TypeError(f"optimizer state '{key}' is not a tensor")
                if key == 'I' and src.dtype != want:
                    as_int = src.to(torch.int16)
                    if not torch.equal(as_int.to(src.dtype), src):
                        raise ValueError("optimizer state 'I' holds values that are not 16-bit integers")
                    src = as_int
                if src.dtype != want:
                    raise TypeError(f"optimizer state '{key}' has element type {src.dtype}, expected {want}")
                st[key] = src.detach().to(device=p.device, copy=True)
            d, k, nq = int(st['d']), int(st['k']), int(st['quant_full_blocks_count'])
            shapes = {'I': (self.m, k), 'V': (self.m, k), 'error': ((d + 1) // 2,), 'min_vals': (nq + 1,), 'max_vals': (nq + 1,)}
            for key, shape in shapes.items():
                if tuple(st[key].shape) != shape:
                    raise ValueError(f"optimizer state '{key}' has shape {tuple(st[key].shape)}, expected {shape}")
            self._check_window_indices(st)
            if 'quant_err' in saved and torch.is_tensor(saved['quant_err']):
                st['quant_err'] = saved['quant_err'].detach().to(device=p.device, dtype=p.dtype, copy=True)
            if not (0 <= int(st['index']) < self.m):
                raise ValueError(f"optimizer state 'index' = {st['index']} outside [0, {self.m})")
        if steps is not None:
            self.steps = int(steps)
        self._entries_key = None

    @staticmethod
    def _check_window_indices(st):
        """Every stored index must lie inside its top-k block (the update kernel uses it as an offset)."""
        I = st['I']
        if I.numel() == 0:
            return
        k_index, dbs = int(st['k_index']), int(st['d_block_size'])
        tail = int(st['d']) - int(st['d_index_topk']) if int(st['k_block_size_few']) > 0 else 0
        bad = bool((I < 0).any())
        if k_index > 0:
            bad |= bool((I[:, :k_index] >= dbs).any())
        if I.shape[1] > k_index:
            bad |= bool((I[:, k_index:] >= max(tail, 1)).any())
        if bad:
            raise ValueError("optimizer state 'I' holds an index outside its top-k block")

    # ------------------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        self.steps += 1                                                                                # micro_adam.py:98
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        self._refresh_entries()
        probe = self._probe_begin()
        fused = [e for e in self._entries if e.fused]
        if fused:
            self._fused_step(fused, probe=probe)
        for e in self._entries:
            if not e.fused:
                self._generic_update(e, probe)
        late = [e for e in self._entries if not e.fused and e.window_fused]
        if late:
            self._fused_window_update(late, probe)
        self._after_update()
        self._probe_end(probe)
        if self.kernel_events and len(self.kernel_events[-1]) == 3:
            ev = torch.cuda.Event(enable_timing=True)   # end of whatever _after_update enqueued
            ev.record()
            self.kernel_events[-1].append(ev)
        return loss

    # ------------------------------------------------------------------------------ logging probes
    def _probe_begin(self) -> Optional[dict]:
        """On a logging step (micro_adam.py:155,306,320: every `log_interval` steps, here only when a `log_fn` is given):
        the dictionary the step's probes are summed into.  The fused kernels add theirs to a small device buffer
        (`probe['buf']`, MAB_PROBE_SLOTS doubles) that is read back once, at the end of the step."""
        if self.log_fn is None or self.steps % self.log_interval != 0:
            return None
        probe = dict(norm_g=0.0, norm_u=0.0, norm_e=0.0, sp_u=0.0, t0=time.time(), buf=None)
        if self._entries:
            probe['buf'] = torch.zeros(N.MAB_PROBE_SLOTS, dtype=torch.float64, device=self._entries[0].p.device)
        return probe

    def _probe_end(self, probe: Optional[dict]):
        if probe is None:
            return
        if probe['buf'] is not None:
            b = probe['buf'].tolist()                     # the one device-to-host read of a logging step
            probe['norm_g'] += b[N.MAB_PROBE_NORM_G]
            probe['norm_u'] += b[N.MAB_PROBE_NORM_U]
            probe['norm_e'] += b[N.MAB_PROBE_NORM_E]
            probe['sp_u'] += b[N.MAB_PROBE_ZEROS_U]
            if self.densify_update_using_quant_error:
                probe['norm_qe'] = probe.get('norm_qe', 0.0) + b[N.MAB_PROBE_NORM_QE]
                probe['sp_qe'] = probe.get('sp_qe', 0.0) + b[N.MAB_PROBE_ZEROS_QE]
        self._log(probe)

    def _log(self, probe: dict):
        """micro_adam.py:330-350: sums the probes over the ranks and hands them to `log_fn` (the reference sends the
        same keys to wandb; the quantisation-error entries are those of alpha == -2, else 0)."""
        vals = [probe.get('norm_qe', 0.0), probe['norm_g'], probe['norm_u'], probe['norm_e'], probe['sp_u'],
                probe.get('sp_qe', 0.0), time.time() - probe['t0']]
        dist = torch.distributed
        if dist.is_available() and dist.is_initialized():
            dev = self.param_groups[0]['params'][0].device if dist.get_backend() == 'nccl' else 'cpu'
            sync = torch.tensor(vals, dtype=torch.float, device=dev)
            dist.all_reduce(sync, op=dist.ReduceOp.SUM)
            vals = sync.tolist()
            if dist.get_rank() != 0:
                return
        norm_qe, norm_g, norm_u, norm_e, sp_u, sp_qe, elapsed = vals
        self.log_fn({
            'step/optimizer_steps': self.steps,
            'step/gpu_mem_usage': torch.cuda.memory_allocated() / 2 ** 20 if torch.cuda.is_available() else 0.0,
            'step/norm_quant_err': math.sqrt(norm_qe),
            'step/sparsity_quant_err': sp_qe / self.model_size * 100.,
            'step/norm_g': math.sqrt(norm_g),
            'step/norm_u': math.sqrt(norm_u),
            'step/norm_error': math.sqrt(norm_e),
            'step/sparsity_u': sp_u / self.model_size * 100.,
            'step/elapsed_step': elapsed,
        })

    def _after_update(self):
        """Hook for subclasses (the sharded optimizer gathers the updated parameters here)."""

    def _refresh_entries(self):
        active = []
        for gi, group in enumerate(self.param_groups):
            for p in group['params']:
                if p.grad is None:                                                                     # micro_adam.py:125
                    continue
                sl = self._slice_of(p)
                if sl is None or sl[0] == sl[1]:
                    continue
                if not p.is_cuda:
                    raise N.NativeError(f'parameter on {p.device}: MicroAdam for B200 has no CPU implementation')
                if p.grad.is_sparse:
                    raise N.NativeError('sparse gradients are not supported')
                active.append((p, sl, gi))
        key = tuple((id(p), sl, p.dtype, p.grad.dtype) for p, sl, _ in active)
        if key == self._entries_key:
            return
        entries = []
        for p, (lo, hi), gi in active:
            st = self.state[p]
            if len(st) == 0 or 'I' not in st:                                                          # micro_adam.py:158-160
                group = self.param_groups[gi]
                self._initialize_parameter_state(p, group['lr'], group.get('weight_decay', self.weight_decay), lo, hi)
            if st['I'].dtype != torch.int16:                                                           # micro_adam.py:175-178
                st['I'] = st['I'].to(torch.int16)
            if st['d'] != hi - lo:
                raise RuntimeError(f'state of a parameter holds d={st["d"]} but the slice to update has {hi - lo} elements')
            entries.append(_Entry(p, st, lo, hi, gi))
        self._entries = entries
        self._entries_key = key
        self._descs = {}
        if self.use_fused and entries:
            args = self._step_args()
            for e in entries:
                d = N.MabTensor()
                self._fill_static(d, e)
                self._fill_dynamic(d, e)
                e.fused = bool(N.load().mab_fused_supported(ctypes.byref(d), ctypes.byref(args)))
                e.window_fused = (not e.fused and self.alpha == 0 and
                                  bool(N.load().mab_fused_window_supported(ctypes.byref(d), ctypes.byref(args))))

    def _step_args(self) -> N.MabStepArgs:
        a = N.MabStepArgs()
        a.steps, a.m, a.quant_block_size = self.steps, self.m, self.quant_block_size
        a.alpha = float(self.alpha)
        a.beta1, a.beta2, a.eps = float(self.beta1), float(self.beta2), float(self.eps)
        return a

    @staticmethod
    def _fill_static(d: N.MabTensor, e: _Entry):
        st = e.st
        d.error, d.min_vals, d.max_vals = st['error'].data_ptr(), st['min_vals'].data_ptr(), st['max_vals'].data_ptr()
        d.I, d.V = st['I'].data_ptr(), st['V'].data_ptr()
        d.d, d.k = st['d'], st['k']
        d.d_block_size = st['d_block_size']
        d.topk_full_blocks_count = st['topk_full_blocks_count'] if st['d_index_topk'] > 0 else 0
        d.k_block_size_many, d.k_block_size_few = st['k_block_size_many'], st['k_block_size_few']
        d.param_dtype, d.grad_dtype = N.dtype_code(e.p), N.dtype_code(e.p.grad)
        d.quant_err = st['quant_err'].data_ptr() if 'quant_err' in st else None

    def _fill_dynamic(self, d: N.MabTensor, e: _Entry):
        p, g = e.p, e.p.grad
        if not (p.is_contiguous() and g.is_contiguous()):
            raise N.NativeError('parameters and gradients must be contiguous (the reference requires p.grad.view(-1))')
        group = self.param_groups[e.group]
        d.param = p.data_ptr() + e.lo * p.element_size()
        d.grad = g.data_ptr() + e.lo * g.element_size()
        d.ring_index = e.st['index']
        d.lr = float(group['lr'])                                                                      # micro_adam.py:121
        d.weight_decay = float(group.get('weight_decay', self.weight_decay))                           # micro_adam.py:122

    def _fused_step(self, entries: List[_Entry], group_key=0, probe: Optional[dict] = None):
        """One fused step over `entries`; `group_key` names the group so that its descriptor array is reused.  On a
        logging step the kernels add their probes to `probe['buf']`."""
        lib = N.load()
        n = len(entries)
        descs = self._descs.get(group_key)
        if descs is None or len(descs) != n:
            descs = self._descs[group_key] = (N.MabTensor * n)()
            for d, e in zip(descs, entries):
                self._fill_static(d, e)
        for d, e in zip(descs, entries):
            self._fill_dynamic(d, e)
            e.st['index'] = (e.st['index'] + 1) % self.m                                               # micro_adam.py:211
        device = entries[0].p.device
        args = self._step_args()
        need = lib.mab_fused_step_workspace_bytes_for(descs, n, ctypes.byref(args))    # with scratch for loose quantisation blocks
        if self._workspace is None or self._workspace.numel() < need or self._workspace.device != device:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=device)
        if probe is not None:
            args.probe_out = probe['buf'].data_ptr()
        ws, ws_bytes = self._workspace.data_ptr(), self._workspace.numel()
        with torch.cuda.device(device):
            stream = N.current_stream(device)
            if self.kernel_events is None or probe is not None:
                N.check(lib.mab_fused_step(descs, n, ctypes.byref(args), ws, ws_bytes, stream), 'mab_fused_step')
            else:
                # the same two kernels through their own entry points, with CUDA events between them
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                ev[0].record()
                N.check(lib.mab_fused_ef_topk_quant(descs, n, ctypes.byref(args), ws, ws_bytes, stream),
                        'mab_fused_ef_topk_quant')
                ev[1].record()
                N.check(lib.mab_fused_window_adam_update(descs, n, ctypes.byref(args), ws, ws_bytes, stream),
                        'mab_fused_window_adam_update')
                ev[2].record()
                self.kernel_events.append(ev)

    def _fused_window_update(self, entries: List[_Entry], probe: Optional[dict] = None):
        """Second half of the step (micro_adam.py:234-235, 276-304 with alpha == 0) for entries whose first half ran
        on the operator-level calls: weight decay, window -> Adam update, parameter update in one kernel over all of
        them.  With alpha == 0 that kernel reads neither the gradient nor the error feedback, so quantisation blocks
        that straddle top-k blocks do not matter to it; the update is not written to `p.grad`."""
        lib = N.load()
        n = len(entries)
        descs = self._descs.get('window')
        if descs is None or len(descs) != n:
            descs = self._descs['window'] = (N.MabTensor * n)()
            for d, e in zip(descs, entries):
                self._fill_static(d, e)
        for d, e in zip(descs, entries):
            self._fill_dynamic(d, e)
        device = entries[0].p.device
        need = lib.mab_fused_step_workspace_bytes(n)
        if self._window_workspace is None or self._window_workspace.numel() < need or self._window_workspace.device != device:
            self._window_workspace = torch.empty(need, dtype=torch.uint8, device=device)
        args = self._step_args()
        if probe is not None:
            args.probe_out = probe['buf'].data_ptr()
        with torch.cuda.device(device):
            N.check(lib.mab_fused_window_adam_update(descs, n, ctypes.byref(args), self._window_workspace.data_ptr(),
                                                     self._window_workspace.numel(), N.current_stream(device)),
                    'mab_fused_window_adam_update')

    def _generic_update(self, e: _Entry, probe: Optional[dict] = None):
        """The reference's update_step (micro_adam.py:146-328) on the operator-level kernels; `probe` collects the
        squared norms and the zero count the reference logs.  For an entry marked `window_fused` it stops after the
        error feedback has been requantised (micro_adam.py:231); `_fused_window_update` does the rest."""
        p, st = e.p, e.st
        group = self.param_groups[e.group]
        lr, wd = group['lr'], group.get('weight_decay', self.weight_decay)
        pf = p.data.view(-1)[e.lo:e.hi]
        grad = p.grad.view(-1)[e.lo:e.hi]
        d, qbs = st['d'], self.quant_block_size
        dbs, k_many, k_few, k = st['d_block_size'], st['k_block_size_many'], st['k_block_size_few'], st['k']
        index, I, V = st['index'], st['I'], st['V']
        error, min_vals, max_vals = st['error'], st['min_vals'], st['max_vals']

        if probe is not None:
            probe['norm_g'] += float(grad.float().norm(p=2) ** 2)                                      # :155-156
        N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, 1.0)                          # :190
        N.block_topk(d, dbs, k_many, k_few, grad, I[index])                                            # :193-200
        N.copy_values(d, k, dbs, k_many, I[index], grad, V[index], CopyDirection.d2k.value)            # :202-209
        st['index'] = (index + 1) % self.m                                                             # :211
        N.zerorize_block_components(grad, I[index], d, k, dbs, k_many)                                 # :214
        N.quant_stats(d, qbs, min_vals, max_vals, grad)                                                # :217-228
        N.asymm_block_quant(d, qbs, error, min_vals, max_vals, grad)                                   # :231
        if e.window_fused:
            if probe is not None:                                                                      # :320-324
                grad.zero_()
                N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, 1.0)
                probe['norm_e'] += float(grad.float().norm(p=2) ** 2)
            return
        if wd > 0:
            pf.mul_(1 - lr * wd)                                                                       # :234-235
        if self.densify_update_using_quant_error:                                                      # :238-273, the form without lr
            quant_err = st['quant_err']                                                                # :67-68
            quant_err.zero_()
            quant_err.add_(grad)                                                                       # :259-260
            pf.add_(grad, alpha=-1)                                                                    # :263
            grad.zero_()                                                                               # :266
            N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, 1.0)                      # :267
            pf.add_(grad)                                                                              # :268
            quant_err.sub_(grad)                                                                       # :270
            if probe is not None:                                                                      # :272-273
                probe['norm_qe'] = probe.get('norm_qe', 0.0) + float(quant_err.float().norm(p=2) ** 2)
                probe['sp_qe'] = probe.get('sp_qe', 0.0) + float((quant_err == 0).sum())
        N.compute_microadam_update(st['blocks'], self.threads, self.shared_memory_carveout, self.steps, self.beta1,
                                   self.beta2, self.eps, dbs, k_many, d, self.m, k, I, V, grad)        # :276-291
        if self.densify_update_using_ef:
            N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, self.alpha)               # :298
        pf.add_(grad, alpha=-lr)                                                                       # :304
        if probe is not None:                                                                          # :306-308
            probe['norm_u'] += float(grad.float().norm(p=2) ** 2)
            probe['sp_u'] += float((grad == 0).sum())
        if self.densify_update_using_ef:                                                               # :311-316
            grad.zero_()
            N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, 1 - self.alpha)
            N.quant_stats(d, qbs, min_vals, max_vals, grad)
            N.asymm_block_quant(d, qbs, error, min_vals, max_vals, grad)
        if probe is not None:                                                                          # :320-324
            grad.zero_()
            N.asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, grad, 1.0)
            probe['norm_e'] += float(grad.float().norm(p=2) ** 2)
