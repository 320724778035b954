"""Generates tests/golden/microadam_golden.json from the UNMODIFIED reference MicroAdam.

    python tests/golden/make_golden.py [--reference /path/to/ISTA-DASLab-Optimizers]

Needs a checkout of the reference (it is imported through oracle/reference_harness.py, which
supplies CPU stand-ins for the native modules the reference cannot import on its own).  The
cases and their seeded inputs are defined in tests/cases.py.  For every case, step and tensor the
file records a SHA-256 over the bit-exact state (window row written, error-feedback codes,
block statistics) and a strided sample of the parameters (float32 bit patterns, hex).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, 'ista-daslab-optimizers_b200'), os.path.join(ROOT, 'tests')]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', default=None)
    args = ap.parse_args()
    if args.reference:
        os.environ['MICROADAM_REFERENCE_DIR'] = args.reference
    import torch
    import cases
    import struct
    f32hex = lambda v: struct.pack('>f', v).hex()
    out = {'torch': torch.__version__, 'param_samples': cases.PARAM_SAMPLES, 'cases': {}}
    for name, case in cases.CASES.items():
        tr = cases.run_case(case, cases.ReferenceAdapter)
        out['cases'][name] = {'digests': tr.digests,
                              'samples': [[''.join(f32hex(v) for v in s) for s in step] for step in tr.samples]}
        print(name, 'ok', tr.digests[-1][0][:16])
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'microadam_golden.json')
    with open(path, 'w') as f:
        json.dump(out, f, indent=0, separators=(',', ':'))
    print('wrote', path, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
