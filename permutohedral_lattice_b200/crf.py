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
The softmax and the small matrix product run as torch operations on the same stream.
"""
import torch

from .lattice_filter import Lattice


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
        if compatibility is None:
            compatibility = 1.0 - torch.eye(n_labels, dtype=torch.float32, device=image.device)
        self.compatibility = compatibility.to(device=image.device, dtype=torch.float32)

    def step(self, q, unaries):
        message = self.bilateral_weight * self.bilateral.apply(q) + self.spatial_weight * self.spatial.apply(q)
        return torch.softmax(-unaries - message @ self.compatibility, dim=-1)

    def infer(self, unaries, iterations=5):
        """Q after `iterations` mean-field updates, starting from softmax(-unaries)."""
        q = torch.softmax(-unaries, dim=-1)
        for _ in range(int(iterations)):
            q = self.step(q, unaries)
        return q
