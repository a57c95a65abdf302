"""The short division / square-root sequences inside the Adam, replay and fused reduce kernels round exactly like the
IEEE operations of the reference's arithmetic (srm2/ops.py:50-56, srm2/csrc/srm2_cpu.cpp:27-32).

Checked on the GPU itself through the C ABI (srm2_verify_exact), because the sequences start from that GPU's own
reciprocal / reciprocal-square-root approximations:
  * square root: every float of the guarded range, exhaustively;
  * division: for every one of the 2^23 divisor significands, every dividend whose quotient lies within 64 units of a
    rounding midpoint (the only quotients a final error of 2^-19 ulp can misround), every dividend for the divisors that
    enumeration leaves out, and 2^32 random pairs over the guarded exponents; the bound |b*y - 1| <= 2^-22 on the refined
    reciprocal that the argument rests on is checked for every divisor;
  * the whole packed Adam step against the plain IEEE step on 2^28 random operand sets of each kind (training-like
    values; arbitrary bit patterns including NaN, infinities, zeros and subnormals, which must take the IEEE path).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SQRT, DIV_HARD, DIV_ALL, DIV_RANDOM, ADAM = range(5)


@pytest.fixture(scope='module')
def dev():
    if not torch.cuda.is_available():
        pytest.skip('needs a CUDA device')
    return torch.device('cuda:0')


def run(dev, what, lo, hi, variant, param):
    from elara_b200 import _lib
    out = torch.zeros(5, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().srm2_verify_exact(what, lo, hi, variant, param, out.data_ptr(), _lib.stream_of(dev)), 'verify_exact')
    tested, bad, a, b, aux = out.tolist()
    return tested, bad, (a, b), aux


def test_sqrt_every_float_of_the_guarded_range(dev):
    tested, bad, first, _ = run(dev, SQRT, 0, 1 << 32, 1, 0)
    assert tested > 1_000_000_000              # 128 binades of 2^23 significands
    assert bad == 0, f'first mismatch at bits {first[0]:08x}'


def test_division_near_midpoints_for_every_divisor(dev):
    tested, bad, first, loose = run(dev, DIV_HARD, 0, 1 << 23, 1, 32)
    assert tested > 1_500_000_000
    assert loose == 0, 'a refined reciprocal is off by more than 2^-22'
    assert bad == 0, f'first mismatch a={first[0]:08x} b={first[1]:08x}'


def test_division_every_dividend_for_the_remaining_divisors(dev):
    tested, bad, first, _ = run(dev, DIV_ALL, 0, 1 << 14, 1, 9)        # divisors with >= 9 trailing zero bits
    assert tested == (1 << 14) * (1 << 23)
    assert bad == 0, f'first mismatch a={first[0]:08x} b={first[1]:08x}'


def test_division_random_pairs_over_the_guarded_exponents(dev):
    tested, bad, first, _ = run(dev, DIV_RANDOM, 99, 99 + (1 << 32), 1, 0)
    assert tested > 4_000_000_000
    assert bad == 0, f'first mismatch a={first[0]:08x} b={first[1]:08x}'


def test_division_brute_force_sweep(dev):
    """Optional and long: every dividend significand against every divisor significand that ends in SRM2_DIV_SWEEP_SHIFT
    zero bits (shift 3: an eighth of all divisors, 8.8e12 quotients, a few minutes on a B200; shift 0 would be all of
    them).  Not needed for the argument — the midpoint enumeration above covers every divisor — but it is the same claim
    checked the blunt way.  Skipped unless the variable is set."""
    import os, time
    shift = os.environ.get('SRM2_DIV_SWEEP_SHIFT')
    if shift is None:
        pytest.skip('set SRM2_DIV_SWEEP_SHIFT (0..8) to run the brute-force sweep')
    shift = int(shift)
    assert 0 <= shift <= 8
    total = tested_all = 0
    t0 = time.time()
    step = 1 << 14                           # divisors per call: each call is a second or two of GPU time
    for lo in range(0, 1 << (23 - shift), step):
        tested, bad, first, _ = run(dev, DIV_ALL, lo, lo + step, 1, shift)
        torch.cuda.synchronize(dev)
        assert bad == 0, f'first mismatch a={first[0]:08x} b={first[1]:08x}'
        tested_all += tested
    print(f'division sweep: shift {shift}, {tested_all} quotients, 0 mismatches, {time.time() - t0:.0f} s')
    assert tested_all == (1 << (23 - shift)) * (1 << 23)


@pytest.mark.parametrize('mode', [0, 1])
def test_packed_adam_step_equals_ieee_step(dev, mode):
    tested, bad, first, _ = run(dev, ADAM, 5 + mode, 5 + mode + (1 << 28), 0, mode)
    assert tested == 1 << 28
    assert bad == 0, f'first mismatch g={first[0]:08x} m={first[1]:08x}'


def test_rejects_bad_arguments(dev):
    from elara_b200 import _lib
    out = torch.zeros(5, dtype=torch.int64, device=dev)
    L = _lib.lib()
    assert L.srm2_verify_exact(SQRT, 0, 16, 7, 0, out.data_ptr(), 0) == -1
    assert L.srm2_verify_exact(DIV_HARD, 0, (1 << 23) + 1, 1, 32, out.data_ptr(), 0) == -1
    assert L.srm2_verify_exact(9, 0, 1, 1, 0, out.data_ptr(), 0) == -1
    assert L.srm2_verify_exact(SQRT, 0, 16, 1, 0, 0, 0) == -1
