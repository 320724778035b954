"""Writes tests/golden/reference_state_3steps.pt: a `state_dict()` of the UNMODIFIED reference MicroAdam.

    python tests/golden/make_reference_state.py [--reference /path/to/ISTA-DASLab-Optimizers]

The reference class (imported through oracle/reference_harness.py, CPU stand-ins for its native modules)
takes 3 steps on the seeded case below; the file holds its `state_dict()` as the reference writes it, the
parameters at that point, the case's name and the step count (the reference does not save its own).  The
checkpoint tests load it into the CUDA optimizer and into the oracle and continue both.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, 'ista-daslab-optimizers_b200'), os.path.join(ROOT, 'tests')]

CASE = 'ckpt_fp32'
STEPS = 3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', default=None)
    args = ap.parse_args()
    if args.reference:
        os.environ['MICROADAM_REFERENCE_DIR'] = args.reference
    import torch
    import cases
    case = cases.CKPT_CASE
    ad = cases.ReferenceAdapter(case, case.params())
    for t in range(STEPS):
        ad.step(case.grads(t))
    out = {'case': CASE, 'steps': STEPS, 'state_dict': ad.opt.state_dict(),
           'params': [p.detach().clone() for p in ad.params], 'torch': str(torch.__version__)}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'reference_state_3steps.pt')
    torch.save(out, path)
    print('wrote', path, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
