"""The CPU oracle against the golden vectors (made from the unmodified reference) and against
itself: no GPU needed."""
import math
import struct

import pytest
import torch

import cases
from oracle import microadam_oracle as O
from oracle.reference_harness import reference_available


def decode_samples(hexstr):
    return [struct.unpack('>f', bytes.fromhex(hexstr[i:i + 8]))[0] for i in range(0, len(hexstr), 8)]


@pytest.mark.parametrize('name', list(cases.CASES))
def test_oracle_matches_golden(name, golden):
    case = cases.CASES[name]
    tr = cases.run_case(case, cases.OracleAdapter)
    g = golden['cases'][name]
    assert tr.digests == g['digests']
    for step, (mine, theirs) in enumerate(zip(tr.samples, g['samples'])):
        for i, (a, b) in enumerate(zip(mine, theirs)):
            # same machine arithmetic as the reference run: parameters agree to the last bit
            assert a == decode_samples(b), (name, step, i)


@pytest.mark.skipif(not reference_available(), reason='no reference checkout on this machine')
@pytest.mark.parametrize('name', ['mixed_fp32_alpha', 'bf16_alpha', 'qbs_100000'])
def test_oracle_matches_live_reference(name):
    case = cases.CASES[name]
    a = cases.run_case(case, cases.OracleAdapter)
    b = cases.run_case(case, cases.ReferenceAdapter)
    assert a.digests == b.digests
    assert a.samples == b.samples


def test_block_split_and_geometry():
    assert O.block_split(7, 64) == (1, 7)
    assert O.block_split(64, 64) == (1, 64)
    assert O.block_split(130, 64) == (2, 128)
    g = O.Geometry.make(1048576, 29056, 0.01, 64)
    assert (g.topk_full_blocks_count, g.d - g.d_index_topk, g.k_block_size_many, g.k_block_size_few, g.k) == (36, 2560, 291, 26, 10502)
    g = O.Geometry.make(124439808, 29056, 0.01, 64)
    assert (g.topk_full_blocks_count, g.k_block_size_few, g.k) == (4282, 221, 1246283)
    g = O.Geometry.make(4096, 29056, 0.01, 64)
    assert (g.d_block_size, g.topk_full_blocks_count, g.k_block_size_many, g.k_block_size_few, g.k) == (4096, 1, 41, 0, 41)
    g = O.Geometry.make(2 ** 31, 29056, 0.01, 64)
    assert (g.topk_full_blocks_count, g.d - g.d_index_topk, g.k) == (73908, 12800, 21507356)


def test_topk_tie_rule():
    keys = torch.tensor([[1., 3., 3., 2., 3., 0., 3.]])
    assert O.canonical_topk_indices(keys, 3).tolist() == [[1, 2, 4]]
    assert O.canonical_topk_indices(keys, 5).tolist() == [[1, 2, 3, 4, 6]]
    assert O.canonical_topk_indices(torch.zeros(2, 9), 4).tolist() == [[0, 1, 2, 3]] * 2
    k = torch.randn(37, 1500, generator=torch.Generator().manual_seed(3)).abs().to(torch.bfloat16).float()
    assert torch.equal(O.canonical_topk_indices(k, 17), O.canonical_topk_indices_by_sort(k, 17))


def test_codec_round_trip_and_edge_blocks():
    d, qbs = 1000, 64
    x = torch.linspace(-1, 1, d)
    mn = torch.zeros(d // qbs + 1, dtype=torch.bfloat16)
    mx = torch.zeros_like(mn)
    O.quant_stats(d, qbs, mn, mx, x)
    err = torch.zeros((d + 1) // 2, dtype=torch.uint8)
    O.asymm_block_quant(d, qbs, err, mn, mx, x)
    y = torch.zeros(d)
    O.asymm_block_quant_inv(d, qbs, err, mn, mx, y, 1.0)
    step = (mx.float() - mn.float()).max().item() / 15
    assert (x - y).abs().max().item() <= step * 0.5 + 2 ** -8   # half a code step plus the bf16 rounding of min
    # all-equal block: u == 0 -> code 0, decodes to min
    x = torch.full((64,), 0.375)
    mn, mx = torch.zeros(2, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.bfloat16)
    O.quant_stats(64, 64, mn, mx, x)
    err = torch.full((32,), 255, dtype=torch.uint8)
    O.asymm_block_quant(64, 64, err, mn, mx, x)
    assert err.eq(0).all()
    # odd d: the last low nibble is 0
    x = torch.tensor([0., 1., 2.])
    mn, mx = torch.zeros(1, dtype=torch.bfloat16), torch.zeros(1, dtype=torch.bfloat16)
    O.quant_stats(3, 64, mn, mx, x)
    err = torch.zeros(2, dtype=torch.uint8)
    O.asymm_block_quant(3, 64, err, mn, mx, x)
    # codes 0, 7, 15: u = fl(2/15) is rounded up, so 1/u = 7.4999996 and floor(7.9999996) = 7
    assert err.tolist() == [0x07, 0xF0]


def test_adam_tables_age():
    rows, w1, w2, bc1, bc2 = O.adam_tables(12, 10, 0.9, 0.999)
    assert rows == 10
    # step 12 wrote row 1 (age 0), step 11 row 0 (age 1), step 10 row 9 (age 2)
    assert math.isclose(w1[1].item(), 0.1, rel_tol=1e-6)
    assert math.isclose(w1[0].item(), 0.09, rel_tol=1e-6)
    assert math.isclose(w1[9].item(), 0.081, rel_tol=1e-6)
    rows, w1, *_ = O.adam_tables(3, 10, 0.9, 0.999)
    assert rows == 3 and w1[3:].eq(0).all()
