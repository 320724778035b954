"""CPU oracle for the MicroAdam optimizer step.  TEST INFRASTRUCTURE ONLY.

This file restates, on torch CPU tensors, the arithmetic of the MicroAdam step of
IST-DASLab/ISTA-DASLab-Optimizers (ista_daslab_optimizers/micro_adam/micro_adam.py).  It is
the checker the CUDA kernels are compared against and the CPU baseline that the benchmark
times; the shipped optimizer never imports it.

What is pinned and what is not
------------------------------
* The control flow (state geometry, order of the sub-steps, ring-buffer handling, weight
  decay, the alpha > 0 error-feedback integration) follows micro_adam.py line by line and is
  checked bit for bit against the unmodified reference file executed on CPU (see
  oracle/reference_harness.py and tests/golden/).
* Seven functions that micro_adam.py calls live in a third-party package,
  `ista-daslab-optimizers-cuda` (no pinned version in pyproject.toml:19), whose sources are
  not part of the reference tree, and the reference ships no test vectors for them.  Their
  arithmetic below is restated from the call sites, from the comments next to them and from
  the in-tree 4-bit codec (ista_daslab_optimizers/utils/quantizers.py:18-27).  For those
  seven functions: PARITY UNPINNED.

Arithmetic rules (every CUDA kernel reproduces them operation for operation)
-----------------------------------------------------------------------------
Every named operation is one IEEE-754 binary32 operation rounded to nearest-even, never a
fused multiply-add.
 1. Element i belongs to quantisation block b = i // qbs (this covers d < qbs and the short
    last block, whose statistics sit at index d // qbs; micro_adam.py:217-226).
 2. Codes: byte i // 2; even i in the high nibble, odd i in the low nibble
    (quantizers.py:24-27); for odd d the last low nibble is 0.
 3. Qinv: mn = f32(min[b]); mx = f32(max[b]); u = (mx - mn) / 15; x = f32(code) * u; x = x + mn.
 4. Accumulate: t = alpha * x; y = f32(dst) + t; dst = round_to_dst_dtype(y).
 5. Top-k per block: key |a| (value in the gradient dtype); the k largest; ties go to the
    lower index; indices are emitted in ascending order as int16 (micro_adam.py:193-200;
    torch.topk(sorted=False) leaves order and ties unspecified, this fixes them).
 6. V[row, j] = bf16_rne(a[...]) then a[...] = 0 (micro_adam.py:202-214).
 7. Statistics: exact min / max over the block, then bf16_rne (micro_adam.py:217-226).
 8. Q: u as in 3; u == 0 -> code 0; else code = clamp(floor((r - mn) / u + 0.5), 0, 15).
 9. Window / Adam update (micro_adam.py:277-291): over the valid rows r < min(steps, m), with
    age = ((steps - 1) - r) mod m,  m_j += w1[age] * V[r, .],  v_j += w2[age] * V[r, .]^2 in
    row order, w1[age] = f32(beta1**age * (1 - beta1)), w2 likewise;
    u = (m_j / f32(1 - beta1**steps)) / (sqrt(v_j / f32(1 - beta2**steps)) + eps); 0 where
    no row touches.  Checked to a tolerance, not bit for bit.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

# d_block_size on a B200: 232448 bytes of opt-in shared memory / 4 / 2 (micro_adam.py:43-44)
B200_MAX_FLOATS = 58112
B200_D_BLOCK_SIZE = B200_MAX_FLOATS // 2

K2D, D2K = 0, 1  # tools.py:12-14 CopyDirection


# ----------------------------------------------------------------------------- geometry

def block_split(model_size: int, block_size: int):
    """tools.py:85-92."""
    if model_size < block_size:
        return 1, model_size
    blocks_count = int(model_size / block_size)
    start_index_last_block = model_size - model_size % block_size
    return blocks_count, start_index_last_block


@dataclass
class Geometry:
    """Integer geometry of one tensor (micro_adam.py:74-94)."""
    d: int
    d_block_size: int
    topk_full_blocks_count: int
    d_index_topk: int
    k_block_size_many: int
    k_block_size_few: int
    k_index: int
    k: int
    quant_full_blocks_count: int
    d_index_quant: int

    @staticmethod
    def make(d: int, global_d_block_size: int, k_init: float, qbs: int) -> "Geometry":
        dbs = d if d < global_d_block_size else global_d_block_size
        nb, d_index_topk = block_split(d, dbs)
        k_many = int(math.ceil(dbs * k_init))
        k_few = int(math.ceil((d - d_index_topk) * k_init))
        k_index = nb * k_many
        k = k_many * nb + k_few
        nq, d_index_quant = block_split(d, qbs)
        return Geometry(d, dbs, nb, d_index_topk, k_many, k_few, k_index, k, nq, d_index_quant)


# ----------------------------------------------------------------------------- 4-bit codec

def _expand_stats(vals_bf16: torch.Tensor, d: int, qbs: int) -> torch.Tensor:
    """f32 copy of the per-block statistic of every element (rule 1)."""
    v = vals_bf16.float()
    nfull = d // qbs
    parts = []
    if nfull > 0:
        parts.append(v[:nfull].repeat_interleave(qbs))
    rem = d - nfull * qbs
    if rem > 0:
        parts.append(v[nfull:nfull + 1].expand(rem))
    return torch.cat(parts) if len(parts) > 1 else parts[0].contiguous()


def unpack_codes(error: torch.Tensor, d: int) -> torch.Tensor:
    """uint8 codes of the d elements (rule 2)."""
    hi = (error >> 4) & 0xF
    lo = error & 0xF
    return torch.stack((hi, lo), dim=1).reshape(-1)[:d]


def pack_codes(codes: torch.Tensor, d: int) -> torch.Tensor:
    if d % 2:
        codes = torch.cat((codes, codes.new_zeros(1)))
    c = codes.view(-1, 2)
    return ((c[:, 0] << 4) | c[:, 1]).to(torch.uint8)


def asymm_block_quant_inv(d, qbs, error, min_vals, max_vals, x, alpha):
    """x += alpha * Qinv(error) (rules 3-4; call sites micro_adam.py:190,267,298,313,322)."""
    mn = _expand_stats(min_vals, d, qbs)
    mx = _expand_stats(max_vals, d, qbs)
    u = torch.div(torch.sub(mx, mn), 15.0)
    v = torch.mul(unpack_codes(error, d).float(), u)
    v = torch.add(v, mn)
    t = torch.mul(v, torch.tensor(float(alpha), dtype=torch.float32))
    y = torch.add(x.float(), t)
    x.copy_(y)  # float32 -> x.dtype conversion is round-to-nearest-even


def asymm_block_quant(d, qbs, error, min_vals, max_vals, x):
    """error = Q(x; min, max) (rule 8; call sites micro_adam.py:231,316)."""
    mn = _expand_stats(min_vals, d, qbs)
    mx = _expand_stats(max_vals, d, qbs)
    u = torch.div(torch.sub(mx, mn), 15.0)
    t = torch.sub(x.float(), mn)
    q = torch.div(t, u)
    s = torch.add(q, 0.5)
    c = torch.floor(s)
    c = torch.clamp(c, 0.0, 15.0)
    c = torch.where(u == 0, torch.zeros_like(c), c)
    c = torch.nan_to_num(c, nan=0.0)
    error.copy_(pack_codes(c.to(torch.uint8), d))


def quant_stats(d, qbs, min_vals, max_vals, x):
    """Per-block min / max, stored as bf16 (rule 7; micro_adam.py:217-226)."""
    nq, d_index_quant = block_split(d, qbs)
    if nq == 1:
        min_vals[:nq] = x[:d_index_quant].min()
        max_vals[:nq] = x[:d_index_quant].max()
    else:
        min_vals[:nq] = x[:d_index_quant].view(nq, qbs).min(dim=1).values
        max_vals[:nq] = x[:d_index_quant].view(nq, qbs).max(dim=1).values
    if d_index_quant < d:
        min_vals[nq] = x[d_index_quant:].min()
        max_vals[nq] = x[d_index_quant:].max()


# ----------------------------------------------------------------------------- block top-k

def canonical_topk_indices(keys: torch.Tensor, k: int) -> torch.Tensor:
    """Row-wise indices of the k largest keys, ties to the lower index, ascending (rule 5).

    keys: [rows, n] non-negative.  Returns int64 [rows, k].
    """
    rows, n = keys.shape
    if k == 0:
        return torch.empty(rows, 0, dtype=torch.int64)
    kth = torch.topk(keys, k, dim=1, sorted=True).values[:, k - 1:k]          # [rows, 1]
    gt = keys > kth
    need = k - gt.sum(dim=1, keepdim=True)                                     # ties to take
    tie = keys == kth
    tie_rank = torch.cumsum(tie.to(torch.int32), dim=1)
    sel = gt | (tie & (tie_rank <= need))
    idx = sel.nonzero(as_tuple=False)[:, 1]
    return idx.view(rows, k)


def canonical_topk_indices_by_sort(keys: torch.Tensor, k: int) -> torch.Tensor:
    """Same contract through a stable descending sort; used to cross-check the fast version."""
    order = torch.sort(keys, dim=1, descending=True, stable=True).indices[:, :k]
    return torch.sort(order, dim=1).values


def block_topk(a: torch.Tensor, geo: Geometry, out_row: torch.Tensor):
    """I[row, :] for one step (micro_adam.py:193-200)."""
    if geo.k_index > 0:
        keys = a[:geo.d_index_topk].abs().view(geo.topk_full_blocks_count, geo.d_block_size)
        out_row[:geo.k_index] = canonical_topk_indices(keys, geo.k_block_size_many).to(torch.int16).view(-1)
    if geo.k_block_size_few > 0:
        keys = a[geo.d_index_topk:].abs().view(1, -1)
        out_row[geo.k_index:] = canonical_topk_indices(keys, geo.k_block_size_few).to(torch.int16).view(-1)


def _global_index(indices: torch.Tensor, d_block_size: int, k_block_size: int) -> torch.Tensor:
    j = torch.arange(indices.numel(), dtype=torch.int64)
    return (j // k_block_size) * d_block_size + indices.to(torch.int64)


def copy_values(d, k, d_block_size, k_block_size, indices, inp, out, direction):
    """d2k: out[j] = inp[(j // k_block_size) * d_block_size + indices[j]]; k2d the other way
    (micro_adam.py:202-209; sparse_mfac/sparse_core_mfac_w_ef.py:105-124)."""
    g = _global_index(indices, d_block_size, k_block_size)
    if direction == D2K:
        out.copy_(inp[g])
    else:
        out[g] = inp.to(out.dtype)


def zerorize_block_components(x, indices, d, k, d_block_size, k_block_size):
    """x[(j // k_block_size) * d_block_size + indices[j]] = 0 (micro_adam.py:214)."""
    x[_global_index(indices, d_block_size, k_block_size)] = 0


# ----------------------------------------------------------------------------- other consumers of (I, V)

def sparse_rows_dot(d, rows, k, d_block_size, k_block_size, g, I, V, out):
    """out[r] = sum_j V[r, j] * g[(j // k_block_size) * d_block_size + I[r, j]]
    (native SP, sparse_mfac/sparse_core_mfac_w_ef.py:188-203).  Checked to a tolerance (the sum order is free)."""
    for r in range(rows):
        gi = _global_index(I[r], d_block_size, k_block_size)
        out[r] = torch.dot(V[r].double(), g[gi].double()).float()


def sparse_rows_combine(d, rows, k, d_block_size, k_block_size, M, I, V, out):
    """out[...] += sum_r M[r] * V[r, :] at the rows' positions, rows in order, fp32
    (native LCG, sparse_mfac/sparse_core_mfac_w_ef.py:205-221)."""
    acc = torch.zeros(d, dtype=torch.float32)
    for r in range(rows):
        gi = _global_index(I[r], d_block_size, k_block_size)
        acc[gi] = torch.add(acc[gi], torch.mul(V[r].float(), M[r]))
    out.copy_(torch.add(out.float(), acc))


# ----------------------------------------------------------------------------- window / Adam

def adam_tables(steps: int, m: int, beta1: float, beta2: float):
    """Host-side float64 -> float32 tables of rule 9, indexed by ring row."""
    rows = min(steps, m)
    w1 = [0.0] * m
    w2 = [0.0] * m
    for r in range(rows):
        age = ((steps - 1) - r) % m
        w1[r] = (beta1 ** age) * (1.0 - beta1)
        w2[r] = (beta2 ** age) * (1.0 - beta2)
    bc1 = 1.0 - beta1 ** steps
    bc2 = 1.0 - beta2 ** steps
    f32 = lambda v: torch.tensor(v, dtype=torch.float64).to(torch.float32)
    return rows, f32(w1), f32(w2), f32(bc1), f32(bc2)


def compute_microadam_update(blocks, threads, carveout, steps, beta1, beta2, eps,
                             d_block_size, k_block_size, d, m, k, I, V, out):
    """out = Adam-style update from the sparse window (rule 9; micro_adam.py:277-291)."""
    rows, w1, w2, bc1, bc2 = adam_tables(steps, m, beta1, beta2)
    m_acc = torch.zeros(d, dtype=torch.float32)
    v_acc = torch.zeros(d, dtype=torch.float32)
    for r in range(rows):
        g = _global_index(I[r], d_block_size, k_block_size)
        val = V[r].float()
        m_acc[g] = torch.add(m_acc[g], torch.mul(val, w1[r]))
        v_acc[g] = torch.add(v_acc[g], torch.mul(torch.mul(val, val), w2[r]))
    m_hat = torch.div(m_acc, bc1)
    v_hat = torch.div(v_acc, bc2)
    den = torch.add(torch.sqrt(v_hat), torch.tensor(eps, dtype=torch.float32))
    out.copy_(torch.div(m_hat, den))


# ----------------------------------------------------------------------------- full step

class MicroAdamOracle:
    """Standalone CPU MicroAdam: same constructor meaning, state keys and step order as the
    reference class (micro_adam.py:13-328), alpha == -2 (micro_adam.py:238-273) included."""

    def __init__(self, params: Sequence[torch.Tensor], m, lr, quant_block_size, k_init=0.01, alpha=0,
                 betas=(0.9, 0.999), weight_decay=0, eps=1e-8, d_block_size=B200_D_BLOCK_SIZE):
        assert 0 <= alpha < 1 or alpha == -2, 'alpha must be in [0, 1) or -2'                  # micro_adam.py:18
        self.params = list(params)
        self.m = m
        self.lr = lr
        self.quant_block_size = int(quant_block_size)
        self.k_init = k_init
        self.alpha = alpha
        self.weight_decay = weight_decay
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.d_block_size = d_block_size
        self.steps = 0
        self.state: Dict[int, dict] = {}

    def _init_state(self, p):
        geo = Geometry.make(p.numel(), self.d_block_size, self.k_init, self.quant_block_size)
        st = dict(geo=geo, index=0,
                  I=torch.zeros(self.m, geo.k, dtype=torch.int16),
                  V=torch.zeros(self.m, geo.k, dtype=torch.bfloat16),
                  error=torch.zeros(int(math.ceil(geo.d / 2)), dtype=torch.uint8),
                  min_vals=torch.zeros(geo.quant_full_blocks_count + 1, dtype=torch.bfloat16),
                  max_vals=torch.zeros(geo.quant_full_blocks_count + 1, dtype=torch.bfloat16))
        return st

    @torch.no_grad()
    def step(self, grads: Sequence[Optional[torch.Tensor]], lr=None, weight_decay=None):
        """One step.  grads[i] is used as scratch, as p.grad is in the reference."""
        self.steps += 1
        lr = self.lr if lr is None else lr
        wd = self.weight_decay if weight_decay is None else weight_decay
        for pi, (p, g) in enumerate(zip(self.params, grads)):
            if g is None:
                continue
            if pi not in self.state:
                self.state[pi] = self._init_state(p)
            self._update(p, g.view(-1), self.state[pi], lr, wd)

    def _update(self, p, grad, st, lr, wd):
        geo: Geometry = st['geo']
        d, qbs = geo.d, self.quant_block_size
        index, I, V = st['index'], st['I'], st['V']
        error, mn, mx = st['error'], st['min_vals'], st['max_vals']

        asymm_block_quant_inv(d, qbs, error, mn, mx, grad, 1.0)                       # :190
        block_topk(grad, geo, I[index])                                               # :193-200
        copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, I[index], grad, V[index], D2K)
        st['index'] = (index + 1) % self.m                                            # :211
        zerorize_block_components(grad, I[index], d, geo.k, geo.d_block_size, geo.k_block_size_many)
        quant_stats(d, qbs, mn, mx, grad)                                             # :217-228
        asymm_block_quant(d, qbs, error, mn, mx, grad)                                # :231
        if wd > 0:
            p.mul_(1 - lr * wd)                                                       # :234-235
        if self.alpha == -2:                                                          # :238-273, without lr
            if 'quant_err' not in st:
                st['quant_err'] = torch.zeros_like(p)                                 # :67-68
            quant_err = st['quant_err']
            quant_err.zero_()
            quant_err.add_(grad.view(p.shape))                                        # :259-260
            p.add_(grad.view(p.shape), alpha=-1)                                      # :263
            grad.zero_()                                                              # :266
            asymm_block_quant_inv(d, qbs, error, mn, mx, grad, 1)                     # :267
            p.add_(grad.view(p.shape))                                                # :268
            quant_err.sub_(grad.view(p.shape))                                        # :270
        grad.zero_()                                                                  # :276
        compute_microadam_update(0, 0, 0, self.steps, self.beta1, self.beta2, self.eps,
                                 geo.d_block_size, geo.k_block_size_many, d, self.m, geo.k, I, V, grad)
        if self.alpha > 0:
            asymm_block_quant_inv(d, qbs, error, mn, mx, grad, self.alpha)            # :298
        p.add_(grad.view(p.shape), alpha=-lr)                                         # :304
        if self.alpha > 0:                                                            # :311-316
            grad.zero_()
            asymm_block_quant_inv(d, qbs, error, mn, mx, grad, 1 - self.alpha)
            quant_stats(d, qbs, mn, mx, grad)
            asymm_block_quant(d, qbs, error, mn, mx, grad)
