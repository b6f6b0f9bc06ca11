"""Bilateral filtering of an image file on the GPU, with the command line of the reference's demo
program (Tests/test_bilateral_gpu.cpp:11-14,31-50):

    python -m permutohedral_lattice_b200.bilateral_demo <image file> <output file> \\
        <spatial standard deviation> <colour standard deviation>

The image is filtered by itself (input = reference, values scaled to [0, 1]) in float and, like the
reference program, once more in double; both times are printed and the float result is saved
(rounded to 8 bits as Tests/bilateral_filter.py:31 does).
"""
import sys
import time

import numpy as np
import torch

from . import lattice_filter


def filter_image(pixels_u8, theta_alpha, theta_beta, dtype=torch.float32):
    """pixels_u8 [H, W, C] uint8 -> (filtered uint8 image, seconds)."""
    x = torch.from_numpy(np.ascontiguousarray(pixels_u8)).cuda().to(dtype).div_(255.0)[None]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = lattice_filter(x, x, True, theta_alpha, theta_beta)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    return np.round(out[0].double().cpu().numpy() * 255.0).clip(0, 255).astype(np.uint8), secs


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) < 4:
        print("Usage: python -m permutohedral_lattice_b200.bilateral_demo <image file> <output file> "
              "<spatial standard deviation> <color standard deviation>")
        return 1
    from PIL import Image
    image = np.array(Image.open(argv[0]))
    if image.ndim == 2:
        image = image[:, :, None]
    theta_alpha, theta_beta = float(argv[2]), float(argv[3])
    result, secs = filter_image(image, theta_alpha, theta_beta)
    print("Measured from function call: %f seconds" % secs)
    print("Testing for double percision")
    _, secs = filter_image(image, theta_alpha, theta_beta, torch.float64)
    print("Measured from function call: %f seconds" % secs)
    Image.fromarray(result[:, :, 0] if result.shape[2] == 1 else result).save(argv[1])
    return 0


if __name__ == "__main__":
    sys.exit(main())
