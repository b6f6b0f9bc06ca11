"""Seeded synthetic inputs for the five benchmark / parity configurations.

No public dataset belongs to this path (the reference ships one demo photograph), so every
configuration is generated: numpy PCG64 (`default_rng(seed)`), seed = 100 * config + batch item.

  c0  512x512 RGB bilateral, input = reference, theta 8 / 0.125, pd 5, vd 4, forward
  c1  1024x1024 grey guided by RGB, theta 16 / 0.1, pd 5, vd 2, forward + backward
  c2  16 x 512x512 dense-CRF message passing, 21 channels, theta 80 / 0.0625, pd 5, vd 22, fwd + bwd
  c3  8 x 128^3 volume, 2 channels guided by the clean phantom, theta 5 / 0.1, pd 4, vd 3, fwd + bwd
  c4  8 x 1024x1024, 16-D patch features given as positions, pd 16, vd 4, forward
  c5  c2's input and gradient through the CRF's smoothness kernel: spatial-only (bilateral=False),
      theta_gamma 3, pd 2, vd 22, fwd + bwd (not one of the five benchmark configurations; it exercises the
      direct-indexing path)
"""
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class Workload:
    name: str
    input: np.ndarray                       # [B, *S, C] float32
    reference: Optional[np.ndarray] = None  # [B, *S, R] float32 (op path)
    positions: Optional[np.ndarray] = None  # [B, N, pd] float32 (positions-in path)
    grad: Optional[np.ndarray] = None       # upstream gradient for the backward call
    bilateral: bool = True
    theta_alpha: float = 1.0
    theta_beta: float = 1.0
    theta_gamma: float = 1.0
    backward: bool = False
    meta: dict = field(default_factory=dict)

    @property
    def batch(self):
        return self.input.shape[0]

    @property
    def pixels_per_item(self):
        return int(np.prod(self.input.shape[1:-1]))

    @property
    def pd(self):
        if self.positions is not None:
            return self.positions.shape[-1]
        nsd = self.input.ndim - 2
        return nsd + (self.reference.shape[-1] if self.bilateral else 0)

    @property
    def vd(self):
        return self.input.shape[-1] + 1


def voronoi_rgb(rng, h, w, cells=64):
    """Piecewise-constant Voronoi colour map + low-frequency sine field (amplitude 0.1) + Gaussian
    noise (sigma 0.05), clipped to [0, 1]; float32 [h, w, 3]."""
    sites = rng.random((cells, 2)) * np.array([h, w])
    colours = rng.random((cells, 3))
    yy, xx = np.meshgrid(np.arange(h, dtype=np.float64), np.arange(w, dtype=np.float64),
                         indexing="ij")
    label = np.zeros((h, w), np.int64)
    best = np.full((h, w), np.inf)
    for k in range(cells):
        d = (yy - sites[k, 0]) ** 2 + (xx - sites[k, 1]) ** 2
        m = d < best
        best[m] = d[m]
        label[m] = k
    img = colours[label]
    fy, fx = rng.uniform(1.0, 3.0, 2)
    phase = rng.uniform(0.0, 2 * np.pi, 3)
    field_ = np.sin(2 * np.pi * (fy * yy / h + fx * xx / w))
    img = img + 0.1 * field_[..., None] * np.cos(phase)[None, None, :]
    img = img + rng.normal(0.0, 0.05, img.shape)
    return np.clip(img, 0.0, 1.0).astype(np.float32)


def ellipsoid_phantom(rng, d, count=12):
    zz, yy, xx = np.meshgrid(*(np.arange(d, dtype=np.float32),) * 3, indexing="ij")
    vol = np.zeros((d, d, d), np.float32)
    for _ in range(count):
        c = rng.uniform(0.2 * d, 0.8 * d, 3)
        a = rng.uniform(0.08 * d, 0.3 * d, 3)
        inten = rng.uniform(0.0, 1.0)
        m = ((zz - c[0]) / a[0]) ** 2 + ((yy - c[1]) / a[1]) ** 2 + ((xx - c[2]) / a[2]) ** 2 <= 1.0
        vol[m] = inten
    return vol


def config0(size=512):
    rng = np.random.default_rng(0)
    img = voronoi_rgb(rng, size, size)[None]
    return Workload("c0_rgb_bilateral_%d" % size, input=img.copy(), reference=img, theta_alpha=8.0,
                    theta_beta=0.125)


def config1(size=1024):
    rng = np.random.default_rng(100)
    rgb = voronoi_rgb(rng, size, size)
    lum = 0.2989 * rgb[..., 0] + 0.587 * rgb[..., 1] + 0.114 * rgb[..., 2]
    grey = (lum + rng.normal(0.0, 0.1, lum.shape)).astype(np.float32)[None, ..., None]
    grad = rng.standard_normal(grey.shape).astype(np.float32)
    return Workload("c1_grey_by_rgb_%d" % size, input=grey, reference=rgb[None], grad=grad,
                    theta_alpha=16.0, theta_beta=0.1, backward=True)


def config2(batch=16, size=512, channels=21):
    inputs, refs, grads = [], [], []
    for b in range(batch):
        rng = np.random.default_rng(200 + b)
        refs.append(voronoi_rgb(rng, size, size))
        logits = 3.0 * rng.standard_normal((size, size, channels), dtype=np.float32)
        e = np.exp(logits - logits.max(-1, keepdims=True))
        inputs.append((e / e.sum(-1, keepdims=True)).astype(np.float32))
        grads.append(rng.standard_normal((size, size, channels), dtype=np.float32))
    return Workload("c2_dense_crf_%dx%d" % (batch, size), input=np.stack(inputs),
                    reference=np.stack(refs), grad=np.stack(grads), theta_alpha=80.0,
                    theta_beta=0.0625, backward=True)


def config3(batch=8, size=128):
    inputs, refs, grads = [], [], []
    for b in range(batch):
        rng = np.random.default_rng(300 + b)
        clean = ellipsoid_phantom(rng, size)
        noisy = np.stack([clean, clean], -1) + rng.normal(0.0, 0.2, clean.shape + (2,))
        inputs.append(noisy.astype(np.float32))
        refs.append(clean[..., None])
        grads.append(rng.standard_normal(clean.shape + (2,), dtype=np.float32))
    return Workload("c3_volume_%dx%d" % (batch, size), input=np.stack(inputs),
                    reference=np.stack(refs), grad=np.stack(grads), theta_alpha=5.0, theta_beta=0.1,
                    backward=True)


def config4(batch=8, size=1024, pd=16):
    inputs, positions = [], []
    for b in range(batch):
        rng = np.random.default_rng(400 + b)
        rgb = voronoi_rgb(rng, size, size)
        pad = np.pad(rgb, ((2, 2), (2, 2), (0, 0)), mode="edge")
        patches = np.concatenate([pad[dy:dy + size, dx:dx + size] for dy in range(5)
                                  for dx in range(5)], -1)            # [H, W, 75]
        q, _ = np.linalg.qr(rng.standard_normal((75, pd)))
        pos = (patches.reshape(-1, 75).astype(np.float64) @ q) / 0.2
        inputs.append(rgb)
        positions.append(pos.astype(np.float32))
    return Workload("c4_patch_pd%d_%dx%d" % (pd, batch, size), input=np.stack(inputs),
                    positions=np.stack(positions))


def config5(batch=16, size=512, channels=21):
    w = config2(batch, size, channels)
    return Workload("c5_crf_smoothness_%dx%d" % (batch, size), input=w.input, grad=w.grad, bilateral=False,
                    theta_gamma=3.0, backward=True)


CONFIGS = {0: config0, 1: config1, 2: config2, 3: config3, 4: config4, 5: config5}


def small(config):
    """Reduced-size variant of a configuration (same distributions, theta scaled with the image side
    so the vertex density stays comparable) for parity tests the CPU oracle finishes in seconds."""
    if config == 0:
        w = config0(96)
    elif config == 1:
        w = config1(128)
        w.theta_alpha = 4.0
    elif config == 2:
        w = config2(batch=3, size=64)
        w.theta_alpha = 10.0
    elif config == 3:
        w = config3(batch=2, size=24)
        w.theta_alpha = 2.0
    elif config == 4:
        w = config4(batch=2, size=48)
    elif config == 5:
        w = config5(batch=3, size=64)
    else:
        raise KeyError(config)
    w.name += "_small"
    return w
