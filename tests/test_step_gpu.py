"""The whole optimizer step on the GPU against the CPU oracle and the golden vectors."""
import struct

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def decode_samples(hexstr):
    return [struct.unpack('>f', bytes.fromhex(hexstr[i:i + 8]))[0] for i in range(0, len(hexstr), 8)]


def check_trace(case, tr, ref_digests, ref_samples):
    assert tr.digests == ref_digests, [(s, i) for s, (a, b) in enumerate(zip(tr.digests, ref_digests))
                                       for i, (x, y) in enumerate(zip(a, b)) if x != y][:5]
    # parameters: rel 1e-5 (fp32) / 1e-2 (bf16), the tolerance the path's specification states, with the absolute
    # floor of cases.param_tolerances for elements that are what is left of a cancellation
    rtol, atol = cases.param_tolerances(case.dtype, case.lr)
    for mine, theirs in zip(tr.samples, ref_samples):
        for a, b in zip(mine, theirs):
            torch.testing.assert_close(torch.tensor(a), torch.tensor(b), rtol=rtol, atol=atol)


@pytest.mark.parametrize('use_fused', [True, False], ids=['fused', 'operators'])
@pytest.mark.parametrize('name', list(cases.CASES))
def test_step_matches_golden_and_oracle(name, use_fused, golden):
    case = cases.CASES[name]
    tr = cases.run_case(case, lambda c, p: cases.CudaAdapter(c, p, use_fused=use_fused), keep_params=True)
    g = golden['cases'][name]
    check_trace(case, tr, g['digests'], [[decode_samples(s) for s in step] for step in g['samples']])
    ref = cases.run_case(case, cases.OracleAdapter, keep_params=True)
    check_trace(case, tr, ref.digests, ref.samples)
    cases.assert_params_close(case, tr, ref)          # every element of every parameter, after every step


def test_wide_cases_take_the_wide_update_kernel():
    """The cases named wide_* must exceed what the per-tile arrays of the update kernel hold, or they test nothing new."""
    import math
    for name in ('wide_fp32', 'wide_bf16_wd', 'wide_fp32_alpha'):
        case = cases.CASES[name]
        k_many = max(math.ceil(min(int(torch.Size(s).numel()), case.d_block_size) * case.k_init) for s in case.shapes)
        assert min(case.steps, case.m) * k_many > 16384, name


def test_no_kernel_gave_up_a_wait():
    """Runs a multi-block case (tiles staged by the copy engine) and checks the device error flag."""
    from ista_daslab_optimizers_b200 import _native
    case = cases.CASES['c1_fp32_1m']
    ad = cases.CudaAdapter(case, case.params())
    for t in range(2):
        ad.step(case.grads(t))
    torch.cuda.synchronize()
    assert _native.device_error() == 0


def test_fused_path_is_taken_when_supported():
    case = cases.CASES['bf16_wd']
    ad = cases.CudaAdapter(case, case.params())
    ad.step(case.grads(0))
    assert all(e.fused for e in ad.opt._entries)
    case = cases.CASES['qbs_100000']
    ad = cases.CudaAdapter(case, case.params())
    ad.step(case.grads(0))
    assert not any(e.fused or e.window_fused for e in ad.opt._entries)
    # without the alpha term quantisation blocks of any multiple of 8 >= 64 take the three-kernel fused step
    case = cases.CASES['qbs_100000_a0']
    ad = cases.CudaAdapter(case, case.params())
    ad.step(case.grads(0))
    assert all(e.fused for e in ad.opt._entries)
    # and other sizes the operator-level first half with the fused update
    case = cases.CASES['qbs_100_a0']
    ad = cases.CudaAdapter(case, case.params())
    ad.step(case.grads(0))
    assert all(e.window_fused and not e.fused for e in ad.opt._entries)


def test_fused_step_leaves_grad_untouched_and_is_deterministic():
    case = cases.CASES['mixed_fp32_alpha']
    runs = []
    for _ in range(2):
        ad = cases.CudaAdapter(case, case.params())
        for t in range(3):
            grads = case.grads(t)
            ad.step(grads)
            for p, g in zip(ad.params, grads):
                assert torch.equal(p.grad.cpu(), g)
        runs.append([p.detach().cpu().clone() for p in ad.params])
    for a, b in zip(*runs):
        assert torch.equal(a, b)


def test_grad_none_and_param_groups():
    from ista_daslab_optimizers_b200 import MicroAdam
    p1 = torch.nn.Parameter(torch.randn(5000, device='cuda'))
    p2 = torch.nn.Parameter(torch.randn(300, 70, device='cuda'))
    p3 = torch.nn.Parameter(torch.randn(64, device='cuda'))
    opt = MicroAdam([{'params': [p1], 'lr': 1e-2}, {'params': [p2, p3], 'weight_decay': 0.5}], m=4, lr=1e-3, quant_block_size=64)
    before = [p.detach().clone() for p in (p1, p2, p3)]
    p1.grad = torch.randn_like(p1)
    p2.grad = torch.randn_like(p2)
    opt.step()
    assert not torch.equal(p1, before[0]) and not torch.equal(p2, before[1]) and torch.equal(p3, before[2])
    assert len(opt.state[p3]) == 0 and opt.state[p1]['index'] == 1
    # weight decay of the second group: untouched entries shrink by exactly 1 - lr * wd
    untouched = (p2.detach() - before[1] * (1 - 1e-3 * 0.5)).abs() < 1e-7
    assert untouched.float().mean() > 0.9
    sd = opt.state_dict()
    assert sd['steps'] == 1
    opt2 = MicroAdam([{'params': [p1], 'lr': 1e-2}, {'params': [p2, p3], 'weight_decay': 0.5}], m=4, lr=1e-3, quant_block_size=64)
    opt2.load_state_dict(sd)
    assert opt2.steps == 1 and torch.equal(opt2.state[p1]['I'], opt.state[p1]['I'])


def test_rejects_bad_alpha_and_cpu_params():
    from ista_daslab_optimizers_b200 import MicroAdam, _native
    with pytest.raises(AssertionError):
        MicroAdam([torch.nn.Parameter(torch.zeros(8, device='cuda'))], m=10, lr=1e-3, quant_block_size=64, alpha=-1)
    p = torch.nn.Parameter(torch.zeros(8))
    p.grad = torch.zeros(8)
    opt = MicroAdam([p], m=10, lr=1e-3, quant_block_size=64)
    with pytest.raises(_native.NativeError):
        opt.step()


@pytest.mark.parametrize('name', ['bf16_wd', 'c1_fp32_1m', 'mixed_fp32_alpha', 'alpha_m2', 'wide_fp32', 'qbs_100000_a0', 'qbs_100_a0'])
def test_logging_probes_report_the_reference_quantities(name):
    """log_fn switches the probes of micro_adam.py:155-156, 272-273, 306-308, 320-324 on: every log_interval steps the
    numbers of micro_adam.py:330-350 arrive, taken by the fused kernels (one more small kernel and one read on such a
    step); the state stays what the unprobed optimizer produces.  Expected values come from the oracle's state."""
    import math
    from ista_daslab_optimizers_b200 import _native
    from oracle import microadam_oracle as O
    case = cases.CASES[name]
    logged = []
    plain = cases.CudaAdapter(case, case.params())
    probed = cases.CudaAdapter(case, case.params())
    ref = cases.OracleAdapter(case, case.params())
    probed.opt.log_fn = logged.append
    probed.opt.log_interval = 2
    n_total = sum(int(torch.Size(s).numel()) for s in case.shapes)
    for t in range(4):
        grads = case.grads(t)
        plain.step(grads)
        before = _native.kernel_launch_count()
        probed.step(grads)
        launches = _native.kernel_launch_count() - before
        ref.step(grads)
        hybrid = name == 'qbs_100_a0'             # first half on the operator-level kernels, second half fused
        loose = name == 'qbs_100000_a0'           # kernel A in two parts; the probe of the gradient runs before them
        assert all((e.window_fused and not e.fused) if hybrid else e.fused for e in probed.opt._entries)
        if (t + 1) % 2:
            assert hybrid or launches == (3 if loose else 2)
            continue
        assert hybrid or launches == (5 if loose else 3)
        rec = logged[-1]
        assert rec['step/optimizer_steps'] == t + 1
        norm_g = math.sqrt(sum(float(g.double().norm() ** 2) for g in grads))
        assert rec['step/norm_g'] == pytest.approx(norm_g, rel=1e-4)
        norm_e = norm_u = zeros_u = norm_qe = zeros_qe = 0.0
        for i in range(len(case.shapes)):
            st = ref.opt.state[i]
            geo = st['geo']
            x = torch.zeros(geo.d, dtype=case.dtype)
            O.asymm_block_quant_inv(geo.d, case.qbs, st['error'], st['min_vals'], st['max_vals'], x, 1.0)
            norm_e += float(x.double().norm() ** 2)
            if case.alpha <= 0:                                  # u is the window's update alone: recomputed from the oracle's window
                u = torch.zeros(geo.d, dtype=case.dtype)
                O.compute_microadam_update(0, 0, 0, ref.opt.steps, *case.betas, case.eps, geo.d_block_size, geo.k_block_size_many,
                                           geo.d, case.m, geo.k, st['I'], st['V'], u)
                norm_u += float(u.double().norm() ** 2)
                zeros_u += float((u == 0).sum())
            if case.alpha == -2:
                norm_qe += float(st['quant_err'].double().norm() ** 2)
                zeros_qe += float((st['quant_err'] == 0).sum())
        tol = 1e-3 if case.dtype == torch.float32 else 1e-2
        assert rec['step/norm_error'] == pytest.approx(math.sqrt(norm_e), rel=tol)
        if case.alpha <= 0:
            assert rec['step/norm_u'] == pytest.approx(math.sqrt(norm_u), rel=tol)
            assert rec['step/sparsity_u'] == pytest.approx(zeros_u / n_total * 100, rel=1e-4)
        else:
            assert 0.0 <= rec['step/sparsity_u'] < 100.0 and rec['step/norm_u'] > 0.0
        if case.alpha == -2:
            assert rec['step/norm_quant_err'] == pytest.approx(math.sqrt(norm_qe), rel=tol, abs=1e-12)
            assert rec['step/sparsity_quant_err'] == pytest.approx(zeros_qe / n_total * 100, abs=0.5)
    assert len(logged) == 2
    for i in range(len(case.shapes)):
        a, b = plain.state(i), probed.state(i)
        assert torch.equal(a['I'], b['I']) and torch.equal(a['error'], b['error'])
        assert torch.equal(plain.param(i), probed.param(i))


@pytest.mark.parametrize('qbs', [64, 1000], ids=['qbs64', 'qbs1000'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_flat_shards_cut_at_arbitrary_elements(dtype, qbs):
    """FSDP-style use (micro_adam.py:158-160 sizes the state lazily so that it fits whatever shard a rank holds): the
    parameters handed to the optimizer are slices [lo, hi) of one flat buffer, cut at arbitrary elements, so their
    storage starts at odd offsets (2-byte alignment only for bf16) and top-k blocks are counted from the shard's
    start.  Every shard must behave exactly like a tensor of its own: compared with the oracle on the same slices."""
    from ista_daslab_optimizers_b200 import MicroAdam, _native
    from oracle.microadam_oracle import MicroAdamOracle
    total = 3 * 29056 + 12345
    cuts = [0, 1, 29056 + 3, 2 * 29056 + 1001, total]                 # shards of 1, 29058, 30054 and 40464 elements
    gen = torch.Generator().manual_seed(11)
    flat = (torch.randn(total, generator=gen) * 0.02).to(dtype)
    hyper = dict(m=10, lr=1e-3, quant_block_size=qbs, k_init=0.01, alpha=0, betas=(0.9, 0.999), weight_decay=0.1, eps=1e-8)
    flat_gpu = flat.cuda()
    grad_gpu = torch.zeros_like(flat_gpu)
    shards = [torch.nn.Parameter(flat_gpu[a:b]) for a, b in zip(cuts, cuts[1:])]
    for p, (a, b) in zip(shards, zip(cuts, cuts[1:])):
        p.grad = grad_gpu[a:b]
    opt = MicroAdam(shards, **hyper)
    cpu_shards = [flat[a:b].clone() for a, b in zip(cuts, cuts[1:])]
    ref = MicroAdamOracle(cpu_shards, d_block_size=opt.d_block_size, **hyper)
    rtol, atol = cases.param_tolerances(dtype, hyper['lr'])
    for t in range(12):
        g = (torch.randn(total, generator=gen) * 1e-3).to(dtype)
        grad_gpu.copy_(g)
        opt.step()
        ref.step([g[a:b].clone() for a, b in zip(cuts, cuts[1:])])
        for i, p in enumerate(shards):
            a, b = opt.state[p], ref.state[i]
            row = (a['index'] - 1) % hyper['m']
            assert torch.equal(a['I'][row].cpu(), b['I'][row]), (t, i)
            assert torch.equal(a['V'][row].cpu().view(torch.int16), b['V'][row].view(torch.int16)), (t, i)
            assert torch.equal(a['error'].cpu(), b['error']), (t, i)
            used = (p.numel() + qbs - 1) // qbs
            assert torch.equal(a['min_vals'][:used].cpu().view(torch.int16), b['min_vals'][:used].view(torch.int16)), (t, i)
            torch.testing.assert_close(p.detach().cpu().float(), cpu_shards[i].float(), rtol=rtol, atol=atol)
    assert all(e.fused for e in opt._entries)
    assert _native.device_error() == 0


@pytest.mark.parametrize('name', ['alpha_m2', 'alpha_m2_bf16'])
def test_alpha_m2_runs_fused_and_leaves_the_quantisation_error(name):
    """alpha == -2 (micro_adam.py:238-273) on the two fused kernels: every tensor takes the fused path, two launches per
    step, and `quant_err` holds a - Qinv(e) as the oracle computes it."""
    from ista_daslab_optimizers_b200 import _native
    case = cases.CASES[name]
    gpu = cases.CudaAdapter(case, case.params())
    ref = cases.OracleAdapter(case, case.params())
    rtol, atol = cases.param_tolerances(case.dtype, case.lr)
    for t in range(3):
        grads = case.grads(t)
        before = _native.kernel_launch_count()
        gpu.step(grads)
        assert _native.kernel_launch_count() - before == 2
        assert all(e.fused for e in gpu.opt._entries)
        ref.step(grads)
        for i in range(len(case.shapes)):
            got = gpu.state(i)['quant_err'].float().cpu()
            want = ref.opt.state[i]['quant_err'].float().view(-1)
            # the error is a difference of nearly equal numbers: compared relative to the step of the quantiser
            step_q = float((ref.opt.state[i]['max_vals'].float() - ref.opt.state[i]['min_vals'].float()).max()) / 15
            torch.testing.assert_close(got, want, rtol=rtol, atol=max(atol, step_q * (1e-5 if case.dtype == torch.float32 else 1e-2)))
