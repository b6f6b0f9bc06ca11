"""Finite-difference check of the op's gradient in double precision on a 10 x 10 x 3 input, by the method of
the reference's own (unfinished) test, Tests/TestNeedWork/gradient_test.py:11-42: the gradient the op
defines (the same filter on the upstream gradient with reverse=True, lattice_filter_op_loader.py:32-54)
against a numerical one, compared through

    measure1 = mean(computed - estimated) / mean(computed)     (reference threshold 1e-3)
    measure2 = max(computed - estimated) / max(computed)       (reference threshold 2e-2)

The op's gradient is a definition, not the exact adjoint: it divides by the homogeneous channel AFTER the
transposed filter where the adjoint divides BEFORE it, so the two agree only where that channel is constant
over the image (README.md:88-89 of the reference: "don't match ... for some values of theta").  The
reference's test setting (reference image in 0..255, theta 1, every point alone on its simplex) is such a
case and is asserted with the reference's thresholds; a bilateral setting with real smoothing is reported
and only bounded loosely."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _measures(ta, tb, ref_scale, seed):
    import torch
    import permutohedral_lattice_b200 as plb
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((1, 10, 10, 3))).cuda().requires_grad_(True)
    ref = torch.from_numpy(rng.integers(0, 256, (1, 10, 10, 3)).astype(np.float64) * ref_scale).cuda()
    upstream = torch.from_numpy(rng.standard_normal((1, 10, 10, 3))).cuda()
    y = plb.lattice_filter(x, ref, True, ta, tb)
    y.backward(upstream)
    computed = x.grad.cpu().numpy().ravel()
    # numerical gradient of L(x) = sum(upstream * filter(x)) by central differences, element by element
    eps = 1e-3
    base = x.detach()
    estimated = np.zeros_like(computed)
    for j in range(computed.size):
        e = torch.zeros(computed.size, dtype=torch.float64, device="cuda")
        e[j] = eps
        e = e.view_as(base)
        hi = plb.lattice_filter(base + e, ref, True, ta, tb)
        lo = plb.lattice_filter(base - e, ref, True, ta, tb)
        estimated[j] = float(((hi - lo) * upstream).sum()) / (2 * eps)
    mask = computed != 0
    computed, estimated = computed[mask], estimated[mask]
    diff = computed - estimated
    return (np.mean(diff) / np.mean(computed), np.max(diff) / np.max(computed),
            float(np.corrcoef(computed, estimated)[0, 1]))


def test_gradient_matches_finite_differences_in_the_reference_test_setting():
    m1, m2, corr = _measures(1.0, 1.0, 1.0, seed=3)
    print("gradient check (reference setting): measure1 = %.3g, measure2 = %.3g" % (m1, m2))
    assert abs(m1) < 1e-3 and abs(m2) < 2e-2 and corr > 0.999999


def test_gradient_definition_against_finite_differences_with_real_smoothing():
    m1, m2, corr = _measures(8.0, 0.125, 1.0 / 256.0, seed=3)
    print("gradient check (theta 8 / 0.125): measure1 = %.3g, measure2 = %.3g, correlation = %.4f" % (m1, m2, corr))
    # informational: the CPU reference gives measure1 = -0.047, measure2 = 0.20, correlation 0.988 on this input
    assert np.isfinite([m1, m2]).all() and corr > 0.95 and abs(m2) < 0.5
