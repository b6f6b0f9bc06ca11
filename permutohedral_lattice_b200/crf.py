"""Mean-field inference of a dense CRF around the lattice filter: the caller the reference library was
written for (README.md:15-16 of MiguelMonteiro/permutohedral_lattice names CRF-as-RNN; the library itself
ships no CRF code, so this module follows the published mean-field update, not a reference file).

One iteration, for label distributions Q[B, *S, L], unaries U[B, *S, L] (negative log-likelihoods) and a
guide image I[B, *S, R]:

    Qb = lattice_filter(Q, I, bilateral=True,  theta_alpha, theta_beta)      appearance kernel
    Qs = lattice_filter(Q, I, bilateral=False, theta_gamma)                  smoothness kernel
    message  = bilateral_weight * Qb + spatial_weight * Qs
    pairwise = message @ compatibility                                       [L, L], Potts by default
    Q        = softmax(-U - pairwise)

Both lattices depend on the image only: they are built once (`Lattice`) and applied in every iteration.
Everything after the two filters (weights, compatibility product, unaries, softmax) is one fused kernel,
pl_crf_update_f32: one read of Qb, Qs and U and one write of Q per iteration.
"""
import torch

from . import capi
from .lattice_filter import Lattice, _stream_handle


class DenseCRF:
    def __init__(self, image, n_labels, theta_alpha=80.0, theta_beta=0.0625, theta_gamma=3.0,
                 bilateral_weight=1.0, spatial_weight=1.0, compatibility=None):
        """image [B, *S, R] float32 on the GPU; compatibility [L, L] (default: Potts, 1 - identity)."""
        shape = tuple(image.shape[:-1])
        self.n_labels = int(n_labels)
        self.bilateral = Lattice(image, None, True, theta_alpha, theta_beta, 1.0, max_channels=n_labels)
        self.spatial = Lattice(None, shape, False, 1.0, 1.0, theta_gamma, max_channels=n_labels)
        self.bilateral_weight = float(bilateral_weight)
        self.spatial_weight = float(spatial_weight)
        # None: Potts model (1 - identity), which the kernel evaluates without the L x L product
        self.compatibility = None if compatibility is None else compatibility.to(
            device=image.device, dtype=torch.float32).contiguous()
        if self.compatibility is not None and tuple(self.compatibility.shape) != (self.n_labels, self.n_labels):
            raise ValueError("compatibility must be [n_labels, n_labels]")

    def step(self, q, unaries):
        if q.shape[-1] != self.n_labels or unaries.shape != q.shape:
            raise ValueError("q and unaries must be [B, *S, n_labels]")
        if unaries.dtype != torch.float32 or not unaries.is_cuda:
            raise TypeError("unaries must be a float32 CUDA tensor")
        unaries = unaries.contiguous()
        qb = self.bilateral.apply(q)
        qs = self.spatial.apply(q)
        out = torch.empty_like(qb)
        n_points = out.numel() // self.n_labels
        with torch.cuda.device(out.device):
            capi.check(capi.lib().pl_crf_update_f32(
                out.data_ptr(), unaries.data_ptr(), qb.data_ptr(), qs.data_ptr(),
                0 if self.compatibility is None else self.compatibility.data_ptr(), self.bilateral_weight,
                self.spatial_weight, n_points, self.n_labels, _stream_handle(out.device)), "pl_crf_update_f32")
        return out

    def infer(self, unaries, iterations=5):
        """Q after `iterations` mean-field updates, starting from softmax(-unaries)."""
        q = torch.softmax(-unaries, dim=-1)
        for _ in range(int(iterations)):
            q = self.step(q, unaries)
        return q


def _main():
    """python -m permutohedral_lattice_b200.crf [--batch B] [--size S] [--labels L] [--iterations K]
    Times mean-field iterations on the synthetic dense-CRF workload (seeded; no dataset belongs to this path)."""
    import argparse

    from . import workloads
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--size", type=int, default=512)
    ap.add_argument("--labels", type=int, default=21)
    ap.add_argument("--iterations", type=int, default=10)
    args = ap.parse_args()
    w = workloads.config2(batch=args.batch, size=args.size, channels=args.labels)
    image = torch.from_numpy(w.reference).cuda()
    q0 = torch.from_numpy(w.input).cuda()
    unaries = -torch.log(q0 + 1e-6)
    crf = DenseCRF(image, args.labels, w.theta_alpha, w.theta_beta, 3.0)
    q = q0
    for _ in range(3):
        q = crf.step(q, unaries)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.iterations):
        q = crf.step(q, unaries)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / args.iterations
    print("%d x %dx%d, %d labels: %.3f ms per mean-field iteration (two lattice applications + fused update), "
          "%.1f Mpixels/s" % (args.batch, args.size, args.size, args.labels, ms,
                             args.batch * args.size * args.size / ms / 1e3))


if __name__ == "__main__":
    _main()
