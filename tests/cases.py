"""Seeded parity cases shared by the golden-vector generator and the tests.

A case fixes shapes, element type, hyper-parameters and the number of steps; parameters and
per-step gradients come from ista_daslab_optimizers_b200.synthetic, so every machine sees the
same bits.  `run_case` drives any implementation exposing the small adapter interface below and
returns, per step and tensor, a digest of the bit-exact state plus a sample of the parameters.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Sequence, Tuple

import torch

from ista_daslab_optimizers_b200 import synthetic as S


@dataclass
class Case:
    name: str
    shapes: Sequence[Tuple[int, ...]]
    dtype: torch.dtype
    steps: int
    m: int = 10
    lr: float = 1e-3
    k_init: float = 0.01
    qbs: int = 64
    alpha: float = 0.0
    weight_decay: float = 0.0
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    grad_sigma: float = 1e-3
    grad_kind: str = 'normal'          # 'normal' | 'student_t3_ties'
    zero_tensors: Sequence[int] = ()   # tensors that start at zero with an all-zero first gradient
    seed: int = 0
    d_block_size: int = 29056

    def params(self) -> List[torch.Tensor]:
        out = []
        for i, s in enumerate(self.shapes):
            n = int(torch.Size(s).numel())
            if i in self.zero_tensors:
                out.append(torch.zeros(s, dtype=self.dtype))
            else:
                out.append(S.normal_tensor(self.seed, 100 + i, n, 0.02, self.dtype).view(s))
        return out

    def grads(self, step: int) -> List[torch.Tensor]:
        """Gradients of 0-based `step`."""
        out = []
        for i, s in enumerate(self.shapes):
            n = int(torch.Size(s).numel())
            if i in self.zero_tensors and step == 0:
                out.append(torch.zeros(s, dtype=self.dtype))
                continue
            stream = 10_000 * (step + 1) + i
            if self.grad_kind == 'normal':
                g = S.normal_tensor(self.seed + 1, stream, n, self.grad_sigma)
            else:
                g = S.round_to_8_mantissa_bits(S.student_t3_tensor(self.seed + 1, stream, n, self.grad_sigma))
            out.append(g.to(self.dtype).view(s))
        return out


CASES: Dict[str, Case] = {c.name: c for c in [
    # the reference's own CPU-runnable configuration: one fp32 parameter [1048576], 12 steps so that the m=10 window wraps
    Case('c1_fp32_1m', [(1048576,)], torch.float32, 12),
    # small mixed shapes, heavy-tailed gradients with exact ties, a zero tensor, alpha and weight decay
    Case('mixed_fp32_alpha', [(7,), (65,), (64, 64), (333, 77), (100001,), (256, 256, 3, 3), (4096,)], torch.float32, 12,
         alpha=0.5, weight_decay=0.1, grad_kind='student_t3_ties', zero_tensors=(2, 6)),
    # bf16 parameters and gradients with weight decay (the Llama configuration's element type)
    Case('bf16_wd', [(4096,), (1024, 256), (100001,), (29056 * 2 + 640,)], torch.bfloat16, 12, weight_decay=0.1,
         grad_sigma=1e-4),
    Case('bf16_alpha', [(4096,), (70000,)], torch.bfloat16, 6, alpha=0.25, weight_decay=0.1, grad_kind='student_t3_ties'),
    # quantisation blocks that straddle top-k blocks: only the operator-level kernels apply
    Case('qbs_100000', [(100001,), (300, 200)], torch.float32, 3, qbs=100000, alpha=0.5),
    # the same without the alpha term: kernel A in two parts (residual + merged block extremes, then statistics + codes)
    Case('qbs_100000_a0', [(100001,), (300, 200), (29056 * 3 + 8,), (29056 * 7 + 4097,)], torch.float32, 4, qbs=100000, weight_decay=0.1),
    Case('qbs_100000_a0_bf16', [(100001,), (300, 200), (29056 * 4,)], torch.bfloat16, 4, qbs=100000, weight_decay=0.1, grad_sigma=1e-4),
    # many loose quantisation blocks per top-k block (1000 and 72 elements), blocks that end mid-tile
    Case('qbs_1000_a0', [(29056 * 2 + 1000,), (4096,), (70001,)], torch.float32, 4, qbs=1000, weight_decay=0.1),
    Case('qbs_72_a0_bf16', [(29056 * 2 + 72 * 5,), (4100,)], torch.bfloat16, 4, qbs=72, grad_sigma=1e-4),
    # not a multiple of 8: the operator-level first half, the update (window -> parameters) still fused
    Case('qbs_100_a0', [(100001,), (300, 200)], torch.float32, 4, qbs=100, weight_decay=0.1),
    Case('qbs_32_m5', [(65536,), (1000,)], torch.float32, 7, qbs=32, m=5, k_init=0.05),
    # alpha == -2: the quantisation error is added to the parameters
    Case('alpha_m2', [(70000,), (4096,)], torch.float32, 4, alpha=-2, weight_decay=0.1),
    # bf16 with a quantisation block other than 64: the general decode / statistics / encode code of the bf16 kernel
    Case('bf16_qbs32', [(70000,), (4096,), (29056 + 32 * 7,)], torch.bfloat16, 5, qbs=32, weight_decay=0.1, grad_sigma=1e-4),
    # windows too large for the compact per-tile arrays of the update kernel (m = 20 rows of 5 % of a block):
    # the wide variant of the fused step, with and without weight decay, with the alpha term, fp32 and bf16
    Case('wide_fp32', [(29056 * 2 + 640,), (4096,), (70000,)], torch.float32, 22, m=20, k_init=0.05),
    Case('wide_bf16_wd', [(29056 * 2 + 640,), (4096,)], torch.bfloat16, 14, m=20, k_init=0.05, weight_decay=0.1, grad_sigma=1e-4),
    Case('wide_fp32_alpha', [(29056 + 64 * 9,), (300, 200)], torch.float32, 14, m=20, k_init=0.05, alpha=0.5, weight_decay=0.1,
         grad_kind='student_t3_ties'),
    # k larger than the number of 8-element groups of a block: the selection cannot start from group maxima
    Case('dense_topk_fp32', [(4096,), (29056 + 64,)], torch.float32, 3, k_init=0.2, m=3),
    Case('dense_topk_bf16', [(4096,), (29056 + 64,)], torch.bfloat16, 3, k_init=0.2, m=3, grad_sigma=1e-4),
    # few rows of few entries (m = 5, 0.5 % of a block)
    Case('narrow_m5', [(29056 * 3 + 8,), (1000,)], torch.float32, 7, m=5, k_init=0.005, weight_decay=0.1),
    Case('narrow_m5_bf16', [(29056 * 3 + 8,), (1000,)], torch.bfloat16, 7, m=5, k_init=0.005, weight_decay=0.1, grad_sigma=1e-4),
    # alpha == -2 on bf16 (a tensor with a short last block, an odd-sized one) and with the window wrapping
    Case('alpha_m2_bf16', [(29056 * 2 + 640,), (4097,)], torch.bfloat16, 12, alpha=-2, weight_decay=0.1, grad_sigma=1e-4),
]}


# the case behind tests/golden/reference_state_3steps.pt (a reference-written checkpoint): a tensor with a short
# last block, a single-block tensor and a 2-D one, with weight decay
CKPT_CASE = Case('ckpt_fp32', [(29056 + 640,), (2048,), (100, 70)], torch.float32, 6, weight_decay=0.1)


def _h(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.detach().cpu().contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes())
    return h.hexdigest()


def state_digest(I_row, V_row, error, min_vals, max_vals, d: int, qbs: int) -> str:
    """Digest of everything that must match bit for bit after a step.  Statistics slot d // qbs is
    compared only when the tensor has a short last block (it is never written otherwise)."""
    used = (d + qbs - 1) // qbs
    return _h(I_row, V_row, error, min_vals[:used], max_vals[:used])


PARAM_SAMPLES = 32


def param_sample(p: torch.Tensor) -> List[float]:
    """Up to PARAM_SAMPLES evenly strided elements, as float32."""
    flat = p.detach().float().cpu().view(-1)
    return flat[::max(1, flat.numel() // PARAM_SAMPLES)][:PARAM_SAMPLES].tolist()


@dataclass
class Trace:
    digests: List[List[str]] = field(default_factory=list)       # [step][tensor]
    samples: List[List[List[float]]] = field(default_factory=list)  # [step][tensor][i]
    params: List[List[torch.Tensor]] = field(default_factory=list)  # [step][tensor]: every element, float32 on the CPU (keep_params)


class Adapter:
    """What run_case needs from an implementation."""

    def step(self, grads: List[torch.Tensor]) -> None: ...
    def state(self, i: int) -> dict: ...       # keys: I, V, error, min_vals, max_vals, index (after the step), d
    def param(self, i: int) -> torch.Tensor: ...


def run_case(case: Case, make: Callable[[Case, List[torch.Tensor]], Adapter], keep_params: bool = False) -> Trace:
    """Runs the case; with keep_params the trace also holds every parameter element after every step."""
    params = case.params()
    impl = make(case, params)
    tr = Trace()
    for t in range(case.steps):
        impl.step(case.grads(t))
        if keep_params:
            tr.params.append([impl.param(i).detach().float().cpu().clone() for i in range(len(case.shapes))])
        dg, sm = [], []
        for i in range(len(case.shapes)):
            st = impl.state(i)
            row = (st['index'] - 1) % case.m
            dg.append(state_digest(st['I'][row], st['V'][row], st['error'], st['min_vals'], st['max_vals'], st['d'], case.qbs))
            sm.append(param_sample(impl.param(i)))
        tr.digests.append(dg)
        tr.samples.append(sm)
    return tr


def param_tolerances(dtype: torch.dtype, lr: float):
    """(rtol, atol) for parameters: rel 1e-5 (fp32) / 1e-2 (bf16), the tolerance the path's specification states.
    A new parameter is p - lr * u, so where |p| is close to lr * |u| the result is what is left of a cancellation
    and its error is relative to the operands, not to the result: atol = rtol * lr * 4, 4 standing for the largest
    |u| (an Adam update is bounded by (1 - beta1) / sqrt(1 - beta2) = 3.2 for the default betas).  (It shows on a
    few elements per million: torch's CPU kernels round the scalar of add_(.., alpha=-lr) to bf16 for bf16 tensors,
    torch's CUDA kernels and this library keep it in fp32, and p = bf16(lr) then gives 0 against -5e-7.)"""
    rtol = 1e-5 if dtype == torch.float32 else 1e-2
    return rtol, rtol * lr * 4


def assert_params_close(case: Case, got: Trace, want: Trace):
    """Every parameter element after every step."""
    rtol, atol = param_tolerances(case.dtype, case.lr)
    assert len(got.params) == len(want.params) == case.steps
    for step, (mine, theirs) in enumerate(zip(got.params, want.params)):
        for i, (a, b) in enumerate(zip(mine, theirs)):
            torch.testing.assert_close(a, b, rtol=rtol, atol=atol, msg=lambda m: f'step {step}, tensor {i}: {m}')


class OracleAdapter(Adapter):
    def __init__(self, case: Case, params):
        from oracle.microadam_oracle import MicroAdamOracle
        self.params = params
        self.opt = MicroAdamOracle(params, m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init,
                                   alpha=case.alpha, betas=case.betas, weight_decay=case.weight_decay, eps=case.eps,
                                   d_block_size=case.d_block_size)

    def step(self, grads):
        self.opt.step([g.clone() for g in grads])

    def state(self, i):
        st = self.opt.state[i]
        return dict(I=st['I'], V=st['V'], error=st['error'], min_vals=st['min_vals'], max_vals=st['max_vals'],
                    index=st['index'], d=st['geo'].d)

    def param(self, i):
        return self.params[i]


class ReferenceAdapter(Adapter):
    """The unmodified reference class on CPU (needs a reference checkout)."""

    def __init__(self, case: Case, params):
        from oracle.reference_harness import load_reference_microadam
        Ref = load_reference_microadam(max_floats=2 * case.d_block_size)
        self.params = [torch.nn.Parameter(p) for p in params]
        self.opt = Ref(self.params, m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha,
                       betas=case.betas, weight_decay=case.weight_decay, eps=case.eps)

    def step(self, grads):
        for p, g in zip(self.params, grads):
            p.grad = g.clone()
        self.opt.step()

    def state(self, i):
        return self.opt.state[self.params[i]]

    def param(self, i):
        return self.params[i].data


class CudaAdapter(Adapter):
    """The shipped optimizer on cuda:0."""

    def __init__(self, case: Case, params, use_fused=True):
        from ista_daslab_optimizers_b200 import MicroAdam
        self.params = [torch.nn.Parameter(p.cuda()) for p in params]
        self.opt = MicroAdam(self.params, m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init,
                             alpha=case.alpha, betas=case.betas, weight_decay=case.weight_decay, eps=case.eps,
                             d_block_size=case.d_block_size, use_fused=use_fused)

    def step(self, grads):
        for p, g in zip(self.params, grads):
            p.grad = g.cuda()
        self.opt.step()

    def state(self, i):
        return self.opt.state[self.params[i]]

    def param(self, i):
        return self.params[i].data
