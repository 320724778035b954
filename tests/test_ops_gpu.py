"""Operator-level kernels against the CPU oracle, through the C ABI (bit-exact unless noted)."""
import pytest
import torch

from ista_daslab_optimizers_b200 import synthetic as S
from oracle import microadam_oracle as O

pytestmark = pytest.mark.gpu

DBS = O.B200_D_BLOCK_SIZE


@pytest.fixture(scope='module')
def N():
    from ista_daslab_optimizers_b200 import _native
    _native.load()
    return _native


def bits(t):
    return t.detach().cpu().contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.detach().cpu()


def make_state(d, qbs, seed, dtype):
    """A plausible (error, min, max) triple: quantise a random residual with the oracle."""
    x = S.normal_tensor(seed, 1, d, 1e-3).to(dtype)
    mn = torch.zeros(d // qbs + 1, dtype=torch.bfloat16)
    mx = torch.zeros_like(mn)
    O.quant_stats(d, qbs, mn, mx, x)
    err = torch.zeros((d + 1) // 2, dtype=torch.uint8)
    O.asymm_block_quant(d, qbs, err, mn, mx, x)
    return err, mn, mx


SIZES = [1, 2, 7, 63, 64, 65, 127, 129, 1000, DBS - 1, DBS, DBS + 1, 2 * DBS + 3, 100001]


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('qbs', [64, 32, 100, 100000])
def test_quant_inv_quant_stats(N, dtype, qbs):
    for d in SIZES:
        err, mn, mx = make_state(d, qbs, d, dtype)
        for alpha in (1.0, 0.3):
            x = S.normal_tensor(d, 2, d, 1e-3).to(dtype)
            xg = x.cuda()
            O.asymm_block_quant_inv(d, qbs, err, mn, mx, x, alpha)
            N.asymm_block_quant_inv(d, qbs, err.cuda(), mn.cuda(), mx.cuda(), xg, alpha)
            assert torch.equal(bits(x), bits(xg)), (d, alpha)
        # statistics and codes of the accumulated tensor
        mn2, mx2 = torch.zeros_like(mn), torch.zeros_like(mx)
        O.quant_stats(d, qbs, mn2, mx2, x)
        mng, mxg = torch.zeros_like(mn).cuda(), torch.zeros_like(mx).cuda()
        N.quant_stats(d, qbs, mng, mxg, xg)
        assert torch.equal(bits(mn2), bits(mng)) and torch.equal(bits(mx2), bits(mxg)), d
        e2 = torch.full_like(err, 0xAB)
        O.asymm_block_quant(d, qbs, e2, mn2, mx2, x)
        eg = torch.full_like(err, 0xAB).cuda()
        N.asymm_block_quant(d, qbs, eg, mng, mxg, xg)
        assert torch.equal(e2, eg.cpu()), d


def test_quant_degenerate_blocks(N):
    d, qbs = 256, 64
    x = torch.zeros(d)
    x[64:128] = 0.375          # all-equal block
    x[128:192] = torch.linspace(-1, 1, 64)
    x[192:] = 3e38             # max - min overflows nowhere, but values are huge
    x[200] = -3e38             # max - min = inf -> u = inf
    mn, mx = torch.zeros(5, dtype=torch.bfloat16), torch.zeros(5, dtype=torch.bfloat16)
    O.quant_stats(d, qbs, mn, mx, x)
    e = torch.zeros(d // 2, dtype=torch.uint8)
    O.asymm_block_quant(d, qbs, e, mn, mx, x)
    eg = torch.full((d // 2,), 0xFF, dtype=torch.uint8).cuda()
    N.asymm_block_quant(d, qbs, eg, mn.cuda(), mx.cuda(), x.cuda())
    assert torch.equal(e, eg.cpu())


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('k_init', [0.01, 0.05, 0.3])
def test_block_topk_copy_zerorize(N, dtype, k_init):
    for d in [5, 100, 4096, DBS - 1, DBS, DBS + 1, 3 * DBS + 12345]:
        for kind in ('normal', 'ties', 'zeros', 'few_nonzero'):
            if kind == 'normal':
                a = S.normal_tensor(7, d, d, 1e-3)
            elif kind == 'ties':
                a = S.round_to_8_mantissa_bits(S.student_t3_tensor(7, d, d, 1e-3))
                a = (a * 64).round() / 64 * 1e-2 if d > 100 else a       # very few distinct magnitudes
            elif kind == 'zeros':
                a = torch.zeros(d)
            else:
                a = torch.zeros(d)
                a[::max(1, d // 7)] = -1.5
            a = a.to(dtype)
            geo = O.Geometry.make(d, DBS, k_init, 64)
            row = torch.zeros(geo.k, dtype=torch.int16)
            O.block_topk(a, geo, row)
            ag = a.cuda()
            rowg = torch.full((geo.k,), -1, dtype=torch.int16).cuda()
            N.block_topk(d, geo.d_block_size, geo.k_block_size_many, geo.k_block_size_few, ag, rowg)
            assert torch.equal(row, rowg.cpu()), (d, kind)
            v = torch.zeros(geo.k, dtype=torch.bfloat16)
            O.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, row, a, v, O.D2K)
            vg = torch.zeros(geo.k, dtype=torch.bfloat16).cuda()
            N.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, rowg, ag, vg, O.D2K)
            assert torch.equal(bits(v), bits(vg)), (d, kind)
            O.zerorize_block_components(a, row, d, geo.k, geo.d_block_size, geo.k_block_size_many)
            N.zerorize_block_components(ag, rowg, d, geo.k, geo.d_block_size, geo.k_block_size_many)
            assert torch.equal(bits(a), bits(ag)), (d, kind)
            # k2d puts the values back
            back = torch.zeros(d, dtype=dtype).cuda()
            N.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, rowg, vg, back, O.K2D)
            ref = torch.zeros(d, dtype=dtype)
            O.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, row, v, ref, O.K2D)
            assert torch.equal(bits(ref), bits(back)), (d, kind)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('m,k_init', [(10, 0.01), (5, 0.05), (20, 0.05)])
def test_compute_microadam_update(N, dtype, m, k_init):
    for d in [100, 4096, DBS, 2 * DBS + 777]:
        geo = O.Geometry.make(d, DBS, k_init, 64)
        I = torch.zeros(m, geo.k, dtype=torch.int16)
        V = torch.zeros(m, geo.k, dtype=torch.bfloat16)
        for r in range(m):
            a = S.normal_tensor(11, 100 * d + r, d, 1e-3)
            O.block_topk(a, geo, I[r])
            O.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, I[r], a, V[r], O.D2K)
        for steps in (1, 3, m, m + 2, 57):
            out = torch.zeros(d, dtype=dtype)
            O.compute_microadam_update(0, 0, 0, steps, 0.9, 0.999, 1e-8, geo.d_block_size, geo.k_block_size_many, d, m, geo.k, I, V, out)
            outg = torch.full((d,), 7.0, dtype=dtype).cuda()
            N.compute_microadam_update(148, 512, 100, steps, 0.9, 0.999, 1e-8, geo.d_block_size, geo.k_block_size_many, d, m,
                                       geo.k, I.cuda(), V.cuda(), outg)
            # the update is tolerance-checked by contract (rel 1e-5 fp32, 1e-2 bf16)
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            torch.testing.assert_close(outg.cpu().float(), out.float(), rtol=tol, atol=1e-12)
            assert ((out == 0) == (outg.cpu() == 0)).all()


@pytest.mark.parametrize('vdtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('gdtype', [torch.float32, torch.bfloat16])
def test_sparse_rows_dot_and_combine(N, gdtype, vdtype):
    """The Sparse M-FAC consumers of the ring buffer (scalar products with every row, linear combination of the rows)."""
    m, k_init = 6, 0.02
    for d in [100, 4096, DBS, 2 * DBS + 777]:
        geo = O.Geometry.make(d, DBS, k_init, 64)
        I = torch.zeros(m, geo.k, dtype=torch.int16)
        V = torch.zeros(m, geo.k, dtype=vdtype)
        for r in range(m):
            a = S.normal_tensor(13, 100 * d + r, d, 1.0)
            O.block_topk(a, geo, I[r])
            O.copy_values(d, geo.k, geo.d_block_size, geo.k_block_size_many, I[r], a, V[r], O.D2K)
        g = S.normal_tensor(14, d, d, 1.0).to(gdtype)
        for rows in (1, m):
            sp = torch.zeros(rows)
            O.sparse_rows_dot(d, rows, geo.k, geo.d_block_size, geo.k_block_size_many, g, I, V, sp)
            spg = torch.full((rows,), 7.0, device='cuda')
            N.sparse_rows_dot(d, rows, geo.k, geo.d_block_size, geo.k_block_size_many, g.cuda(), I.cuda(), V.cuda(), spg)
            torch.testing.assert_close(spg.cpu(), sp, rtol=1e-4, atol=1e-4 * float(V.float().abs().max()))
            spg2 = torch.zeros(rows, device='cuda')
            N.sparse_rows_dot(d, rows, geo.k, geo.d_block_size, geo.k_block_size_many, g.cuda(), I.cuda(), V.cuda(), spg2)
            assert torch.equal(spg, spg2)                           # fixed summation order
            M = S.normal_tensor(15, rows, rows, 1.0)
            out = S.normal_tensor(16, d, d, 1.0).to(gdtype)
            outg = out.cuda()
            O.sparse_rows_combine(d, rows, geo.k, geo.d_block_size, geo.k_block_size_many, M, I, V, out)
            N.sparse_rows_combine(d, rows, geo.k, geo.d_block_size, geo.k_block_size_many, M.cuda(), I.cuda(), V.cuda(), outg)
            assert torch.equal(bits(out), bits(outg)), (d, rows)    # same operations in the same order: bit-exact


def test_device_queries(N):
    assert N.get_sm_count() == torch.cuda.get_device_properties(0).multi_processor_count
    floats = N.get_max_floats_for_shared_memory_per_thread_block()
    assert floats * 4 == torch.cuda.get_device_properties(0).shared_memory_per_block_optin


def test_bounded_wait_gives_up_and_reports(N):
    """The give-up path of the kernels' bounded waits, run without any fault: a one-block kernel waits on a barrier
    that expects bytes no copy delivers, gives up after a few probes and raises the device flag; the context stays
    usable and the flag can be cleared."""
    torch.cuda.synchronize()
    N.device_error_clear()
    assert N.device_error() == 0
    N.check(N.load().mab_wait_selftest(4, None), 'mab_wait_selftest')
    assert N.device_error() == 1
    N.device_error_clear()
    assert N.device_error() == 0
    x = torch.arange(10, device='cuda').sum().item()          # the context still works
    assert x == 45
    assert N.load().mab_wait_selftest(0, None) == -1             # limit outside [1, 4096]


@pytest.mark.parametrize('lr,wd', [(1e-3, 0.1), (1e-2, 0.09), (1e-2, 0.1), (0.05, 0.5)])
def test_weight_decay_on_every_bf16_value(N, lr, wd):
    """The fused step skips the decay pass over bf16 parameters when 0 <= lr * wd <= 2^-10, because
    bf16(p * (1 - lr * wd)) == p for every bf16 p then; with a larger product it multiplies.  Either way the
    untouched elements must hold exactly what `p.mul_(1 - lr * wd)` gives: checked on all finite bf16 values."""
    from ista_daslab_optimizers_b200 import MicroAdam
    patterns = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    finite = patterns[torch.isfinite(patterns.float())]
    vals = torch.cat([finite, finite[:29056 * 3 - finite.numel()]]).cuda()     # three full top-k blocks
    p = torch.nn.Parameter(vals.clone())
    opt = MicroAdam([p], m=10, lr=lr, quant_block_size=64, k_init=0.01, weight_decay=wd)
    p.grad = torch.empty_like(p).normal_(0, 1e-4, generator=torch.Generator(device='cuda').manual_seed(3))
    opt.step()
    assert all(e.fused for e in opt._entries)
    want = vals.clone().mul_(1 - lr * wd)
    st = opt.state[p]
    touched = torch.zeros(p.numel(), dtype=torch.bool, device='cuda')
    idx = st['I'][0].long() + (torch.arange(st['k'], device='cuda') // st['k_block_size_many']) * st['d_block_size']
    touched[idx] = True
    assert int(touched.sum()) == st['k']
    got = p.detach()
    assert torch.equal(got[~touched].view(torch.int16), want[~touched].view(torch.int16))
    assert not torch.equal(got[touched].view(torch.int16), want[touched].view(torch.int16))
