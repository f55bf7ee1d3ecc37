"""GPU parity of the image workloads (5x5 box blur over RGB bytes, AdjustBrightness over the flat
number layout) through the C ABI: bit-exact against the CPU restatement of the reference's own
CPU code, on the reference's image sizes, odd sizes, and a size larger than L2."""
import json
import os

import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import native as N
from strict_b200.kernel import DeviceVariable as DV, FlatNumbers

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "reference_known_answers.json")))
L = N.lib


def test_adjust_brightness_known_answers(ctx):
    g = GOLD["adjust_brightness"]
    for case in g["cases"]:
        v = FlatNumbers.of(ctx, g["test_color"], 4).adjust_brightness(case["brightness"])
        assert list(v[0]) == case["expected"]
    run = g["run"]
    n = run["width"] * run["height"]
    image = FlatNumbers.of(ctx, np.tile(np.array(run["default_color"], np.float32), n), 4)
    image.adjust_brightness(run["brightness"])
    centre = image[(run["height"] // 2) * run["width"] + run["width"] // 2]
    assert list(centre[:3]) == run["expected_centre"] and centre[3] == 1.0


@pytest.mark.parametrize("fw,channels,offset,count,total", [(4, 3, 0, 1000, 4000), (4, 3, 4, 999, 4000), (4, 3, 2, 500, 2100), (5, 2, 3, 77, 400),
                                                            (1, 1, 0, 4097, 4097), (3, 3, 1, 100000, 300001), (4, 4, 0, 1 << 20, 1 << 22)])
def test_adjust_brightness_flat_layout_bit_exact(ctx, oracle, rng, fw, channels, offset, count, total):
    """Element i, member m at offset + i*FlatWidth + m (ValueArrayInstance.cs:128,339): views that
    start inside the backing array, structs of other widths, members that are not touched."""
    flat = rng.random(total).astype(np.float32)
    for brightness, clamp in ((0.1, False), (-0.3, True), (0.25, False)):
        want = oracle.adjust_brightness(flat, offset, count, fw, channels, brightness, clamp)
        view = FlatNumbers.of(ctx, flat, fw, offset, count).adjust_brightness(brightness, channels, clamp)
        got = view.backing.to_host()
        assert np.array_equal(got, want)
        view.backing.free()


def test_flat_numbers_view_semantics(ctx):
    colors = np.arange(40, dtype=np.float32)
    v = FlatNumbers.of(ctx, colors, 4)
    assert v.Count == 10 and v.FlatWidth == 4 and v[3] == (12.0, 13.0, 14.0, 15.0) and v.GetFlat(5) == 5.0
    s = v.slice(2, 3)  # shares the backing, like the reference's slices
    assert s.offset == 8 and s.Count == 3 and s[0] == (8.0, 9.0, 10.0, 11.0)
    s.adjust_brightness(100.0)
    host = v.to_host()
    assert host[2].tolist() == [108.0, 109.0, 110.0, 11.0] and host[1].tolist() == [4.0, 5.0, 6.0, 7.0] and host[5].tolist() == [20.0, 21.0, 22.0, 23.0]
    with pytest.raises(IndexError):
        v.slice(8, 3)
    with pytest.raises(ValueError):
        FlatNumbers.of(ctx, colors, 4, offset=1, count=10)


@pytest.mark.parametrize("w,h", [tuple(s) for s in GOLD["blur"]["sizes"]] + [(1, 1), (2, 9), (5, 5), (16, 5), (16, 4), (32, 6), (48, 37), (100, 3),
                                                                             (512, 512), (2048, 1024), (1000, 777), (2064, 70)])
def test_blur_bit_exact(ctx, oracle, w, h):
    """Sizes of the reference's tests (10, 20, 80x60, 320; its timing runs use 512x512 and
    2048x1024), images narrower than the kernel's strips, widths that are not multiples of 16
    (generic kernel), heights around the five-row window and the 32-row blocks."""
    px = oracle.gen_tokens(42, 9, w * h * 3, 256).astype(np.uint8)
    want = oracle.blur5x5_rgb8(px, w, h)
    got = sb.blur5x5_rgb8(ctx, px, w, h)
    assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]


def test_blur_iterations_and_unaligned_buffers(ctx, oracle):
    w, h = 320, 200
    px = oracle.gen_tokens(7, 9, w * h * 3, 256).astype(np.uint8)
    assert np.array_equal(sb.blur5x5_rgb8(ctx, px, w, h, iterations=5), oracle.blur5x5_rgb8(px, w, h, iterations=5))
    # buffers that are not 16-byte aligned take the generic kernel
    import ctypes as C
    a, b = DV(ctx, px.size + 16, np.uint8), DV(ctx, px.size + 16, np.uint8)
    N.check(L().strictb200_upload(ctx.h, C.c_void_p(a.p.value + 3), N.ptr(px), px.size))
    N.check(L().strictb200_blur5x5_rgb8(ctx.h, C.c_void_p(a.p.value + 3), C.c_void_p(b.p.value + 5), w, h))
    got = b.to_host()[5:5 + px.size]
    assert np.array_equal(got, oracle.blur5x5_rgb8(px, w, h))
    with pytest.raises(ValueError):
        N.check(L().strictb200_blur5x5_rgb8(ctx.h, a.p, a.p, w, h))  # in place is not supported
    a.free(), b.free()


def test_blur_larger_than_l2_properties(ctx, oracle):
    """8192 x 8192 x 3 = 201 MB per buffer: a constant image stays constant, and a band of rows
    taken from the middle equals the oracle's blur of that band with its halo."""
    w, h = 8192, 8192
    n = w * h * 3
    a, b = DV(ctx, n, np.uint8), DV(ctx, n, np.uint8)
    N.check(L().strictb200_memset(ctx.h, a.p, 77, n))
    N.check(L().strictb200_blur5x5_rgb8(ctx.h, a.p, b.p, w, h))
    assert (b.to_host() == 77).all()
    tok = DV(ctx, n // 4, np.int32)  # seeded bytes: the four bytes of every generated id's low word
    N.check(L().strictb200_gen_tokens(ctx.h, 42, 11, n // 4, 1 << 31, tok.p))
    host = tok.to_host().view(np.uint8)[:n].copy()
    tok.free()
    a.upload(host)
    N.check(L().strictb200_blur5x5_rgb8(ctx.h, a.p, b.p, w, h))
    got = b.to_host().reshape(h, w * 3)
    r0, r1 = 4000, 4070
    band = oracle.blur5x5_rgb8(host.reshape(h, w * 3)[r0 - 2:r1 + 2].reshape(-1), w, r1 - r0 + 4).reshape(r1 - r0 + 4, w * 3)
    assert np.array_equal(got[r0:r1], band[2:-2])
    top = oracle.blur5x5_rgb8(host.reshape(h, w * 3)[:40].reshape(-1), w, 40).reshape(40, w * 3)
    assert np.array_equal(got[:38], top[:38])
    a.free(), b.free()


def test_blur_division_covers_every_sum(ctx, oracle):
    """The strip kernel divides by 25 with one floating-point multiply-add; its exactness argument
    holds for every window sum 0..6375, so an image is built whose interior windows take every one
    of those sums (a brightness ramp across the columns, with seeded noise), the coverage is
    checked on the host, and the result is compared with the oracle's integer division."""
    w, h = 2048, 96
    rng = np.random.default_rng(25)
    level = np.repeat(np.linspace(-20.0, 275.0, w), 3)[None, :]
    px = np.clip(np.rint(level + rng.normal(0.0, 12.0, (h, w * 3))), 0, 255).astype(np.uint8)
    img = px.reshape(h, w, 3).astype(np.int64)
    sums = sum(img[2 + dy:h - 2 + dy, 2 + dx:w - 2 + dx] for dy in range(-2, 3) for dx in range(-2, 3))
    assert np.array_equal(np.unique(sums), np.arange(6376)), np.setdiff1d(np.arange(6376), sums)[:10]
    want = oracle.blur5x5_rgb8(px.reshape(-1), w, h)
    assert np.array_equal(want.reshape(h, w, 3)[2:-2, 2:-2], sums // 25)  # the oracle divides as integers
    for rows in (0, 8, 64):
        with ctx.option("blur_rows", rows):
            got = sb.blur5x5_rgb8(ctx, px.reshape(-1), w, h)
        assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]
