"""Generates the golden fixtures of this folder from the UNMODIFIED reference CPU implementation
(oracle/_ref/libpl_ref.so, built by oracle/build.py from the reference tree, hash table pre-sized so
it never grows).  Needs the reference tree; run from the repository root:

    python tests/golden/make_golden.py          # the fp32 fixtures
    python tests/golden/make_golden.py f64      # the fp64 fixtures (*_f64.npz)
    python tests/golden/make_golden.py images   # the reference's demo photograph and the two results it ships

Each <case>.npz holds the inputs, the call arguments and what the reference produced: forward and
reverse outputs, the vertex count, the vertex keys (sorted rows) and each pixel's enclosing-simplex
keys and barycentric weights.  photo_crop.npz additionally carries a 96x96 crop of the reference's
demo photograph (Images/input.bmp) as uint8.

`images` re-encodes, pixel for pixel, the golden vectors the reference ships as image files, so that the
full-size checks against them also run where the reference tree is absent: shipped_input.png
(Images/input.bmp), shipped_bilateral_out_1.png (Images/bilateral_out_1.bmp, written by
Tests/bilateral_filter.py:22-31) and shipped_filtered_grey.png (Images/filtered_grey.bmp, written by
Tests/greyscale_test.py:17-36).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import cpu_oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def sorted_rows(keys):
    order = np.lexsort(keys.T[::-1])
    return keys[order]


def run_case(name, inp, ref=None, positions=None, bilateral=True, ta=1.0, tb=1.0, tg=1.0,
             dtype=np.float32):
    """inp [*S, C]; ref [*S, R] or None; positions [n, pd] or None (positions-in path)."""
    sdims = list(inp.shape[:-1])
    n = int(np.prod(sdims))
    c = inp.shape[-1]
    if positions is None:
        if bilateral:
            pos = O.compute_positions(ref.reshape(n, -1), sdims, ta, tb, impl="reference",
                                      dtype=dtype)
        else:
            pos = O.compute_positions(None, sdims, tg, -1.0, impl="reference", dtype=dtype)
    else:
        pos = positions
    fwd = O.filter(inp.reshape(n, c), pos, reverse=False, impl="reference", dtype=dtype)
    rev = O.filter(inp.reshape(n, c), pos, reverse=True, impl="reference", structure=False,
                   dtype=dtype)
    data = dict(
        input=inp.astype(dtype),
        bilateral=np.array(bilateral), theta_alpha=dtype(ta), theta_beta=dtype(tb),
        theta_gamma=dtype(tg),
        out_forward=fwd.out.reshape(inp.shape), out_reverse=rev.out.reshape(inp.shape),
        num_vertices=np.int64(fwd.num_vertices), keys_sorted=sorted_rows(fwd.keys),
        pixel_keys=fwd.pixel_keys(), pixel_weights=fwd.pix_weight,
    )
    if ref is not None:
        data["reference"] = ref.astype(dtype)
    if positions is not None:
        data["positions"] = positions.astype(dtype)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **data)
    print(name, "n", n, "pd", pos.shape[1], "vd", c + 1, "M", fwd.num_vertices)


def main():
    rng = np.random.default_rng(20181)
    # pd 5, vd 4: RGB filtered by itself (the reference's demo setting, theta 8 / 0.125)
    img = rng.random((40, 48, 3), dtype=np.float32)
    img = (0.5 * img + 0.5 * np.round(img * 3) / 3).astype(np.float32)
    run_case("rgb_pd5_vd4", img, ref=img, ta=8.0, tb=0.125)
    # pd 5, vd 2: grey guided by RGB, odd sizes
    run_case("grey_pd5_vd2", rng.random((33, 29, 1), dtype=np.float32),
             ref=rng.random((33, 29, 3), dtype=np.float32), ta=5.0, tb=0.1)
    # pd 5, vd 22: CRF-like, 21 channels
    logits = 3 * rng.standard_normal((32, 36, 21)).astype(np.float32)
    e = np.exp(logits - logits.max(-1, keepdims=True))
    ref = np.repeat(np.repeat(rng.random((4, 6, 3), dtype=np.float32), 8, 0), 6, 1)
    ref = np.clip(ref + rng.normal(0, 0.05, ref.shape), 0, 1).astype(np.float32)
    run_case("crf_pd5_vd22", (e / e.sum(-1, keepdims=True)).astype(np.float32), ref=ref, ta=10.0,
             tb=0.0625)
    # pd 4, vd 3: volume guided by one channel
    vol = rng.random((10, 12, 9, 1), dtype=np.float32)
    vol = np.round(vol * 4) / 4
    run_case("volume_pd4_vd3", rng.standard_normal((10, 12, 9, 2)).astype(np.float32),
             ref=vol.astype(np.float32), ta=5.0, tb=0.1)
    # pd 16, vd 4: positions given
    run_case("patch_pd16_vd4", rng.random((700, 3), dtype=np.float32),
             positions=(rng.standard_normal((700, 16)) * 1.5).astype(np.float32))
    # spatial-only kernels (bilateral = False): pd 2 and pd 3
    run_case("spatial_pd2_vd4", rng.random((21, 17, 3), dtype=np.float32), bilateral=False, tg=3.0)
    run_case("spatial_pd3_vd2", rng.random((7, 9, 8, 1), dtype=np.float32), bilateral=False, tg=2.0)
    # 1-D signal guided by itself: pd 2, vd 2
    sig = np.cumsum(rng.standard_normal((300, 1)), 0).astype(np.float32)
    run_case("signal_pd2_vd2", sig, ref=sig, ta=4.0, tb=0.5)
    # crop of the reference's demo photograph
    from PIL import Image
    from oracle import build as B
    photo = np.array(Image.open(os.path.join(B.reference_root(), "Images", "input.bmp")))
    crop = photo[500:596, 300:396]
    x = (crop / 255.0).astype(np.float32)
    run_case("photo_crop", x, ref=x, ta=8.0, tb=0.125)
    d = dict(np.load(os.path.join(HERE, "photo_crop.npz")))
    d["crop_u8"] = crop
    np.savez_compressed(os.path.join(HERE, "photo_crop.npz"), **d)


def main_f64():
    """T = double (the reference registers its op for double too, src/LatticeFilterKernel.cpp:193)."""
    rng = np.random.default_rng(64064)
    f64 = dict(dtype=np.float64)
    img = rng.random((28, 30, 3))
    img = 0.5 * img + 0.5 * np.round(img * 3) / 3
    run_case("rgb_pd5_vd4_f64", img, ref=img, ta=8.0, tb=0.125, **f64)
    logits = 3 * rng.standard_normal((20, 24, 21))
    e = np.exp(logits - logits.max(-1, keepdims=True))
    ref = np.repeat(np.repeat(rng.random((4, 4, 3)), 5, 0), 6, 1)
    ref = np.clip(ref + rng.normal(0, 0.05, ref.shape), 0, 1)
    run_case("crf_pd5_vd22_f64", e / e.sum(-1, keepdims=True), ref=ref, ta=10.0, tb=0.0625, **f64)
    run_case("spatial_pd2_vd4_f64", rng.random((21, 17, 3)), bilateral=False, tg=3.0, **f64)
    run_case("volume_pd4_vd3_f64", rng.standard_normal((8, 9, 7, 2)),
             ref=np.round(rng.random((8, 9, 7, 1)) * 4) / 4, ta=5.0, tb=0.1, **f64)
    run_case("patch_pd16_vd4_f64", rng.random((300, 3)),
             positions=rng.standard_normal((300, 16)) * 1.5, **f64)


def main_images():
    from PIL import Image
    from oracle import build as B
    src = os.path.join(B.reference_root(), "Images")
    for bmp, png in (("input.bmp", "shipped_input.png"), ("bilateral_out_1.bmp", "shipped_bilateral_out_1.png"),
                     ("filtered_grey.bmp", "shipped_filtered_grey.png")):
        a = np.array(Image.open(os.path.join(src, bmp)))
        Image.fromarray(a).save(os.path.join(HERE, png), optimize=True)
        assert np.array_equal(np.array(Image.open(os.path.join(HERE, png))), a)
        print(png, a.shape, os.path.getsize(os.path.join(HERE, png)), "bytes")


if __name__ == "__main__":
    if sys.argv[1:] == ["f64"]:
        main_f64()
    elif sys.argv[1:] == ["images"]:
        main_images()
    else:
        main()
