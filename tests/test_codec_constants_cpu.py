"""The identities behind `div15_rn` and `rcp_rn_normal` (csrc/common.cuh), checked over every float of their range by
a small C program (about half a minute on one core)."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(shutil.which('gcc') is None, reason='needs gcc')
def test_division_by_15_and_reciprocal_identities_hold_for_every_float(tmp_path):
    exe = str(tmp_path / 'codec_constants_check')
    subprocess.run(['gcc', '-O2', '-march=native', '-o', exe, os.path.join(HERE, 'codec_constants_check.c'), '-lm'], check=True)
    out = subprocess.run([exe], check=False, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout + out.stderr
    assert 'div15 mismatches 0, reciprocal mismatches 0' in out.stdout
