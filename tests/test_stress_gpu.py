"""A reduced form of BASELINE config 5: many mixed-shape fp32 tensors, heavy-tailed gradients with
exact ties, zero-initialised tensors with all-zero first gradients, alpha = 0.5 - against the CPU
oracle, bit-exact state and parameters to tolerance."""
import pytest
import torch

import cases
from ista_daslab_optimizers_b200 import synthetic as S

pytestmark = pytest.mark.gpu


def test_stress_mixed_shapes_ties_zeros_alpha():
    shapes = [s if len(s) == 4 else (min(s[0], 700), min(s[1], 900)) for s in S.stress_shapes(0, count=40)]
    case = cases.Case('stress', shapes, torch.float32, 12, alpha=0.5, grad_kind='student_t3_ties',
                      zero_tensors=tuple(range(0, 40, 10)))
    got = cases.run_case(case, cases.CudaAdapter)
    want = cases.run_case(case, cases.OracleAdapter)
    assert got.digests == want.digests
    for a, b in zip(got.samples, want.samples):
        for x, y in zip(a, b):
            torch.testing.assert_close(torch.tensor(x), torch.tensor(y), rtol=1e-5, atol=1e-9)
