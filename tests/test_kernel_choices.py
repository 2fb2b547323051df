"""What the many-row product picks for a shape: its tile width and whether it splits K.

The choice is host arithmetic in the CUDA library (a time model fitted to measurements on a B200), so
it is checked here without a GPU: the library is compiled (nvcc cross-compiles) and only asked.  The
expected widths are the ones that measured fastest on a B200 for these shapes (graphs of 24 products,
CUDA events); a change of the model that moves one of them has to be measured again.
"""

import pytest

from ayaka_py_b200 import ops
from ayaka_py_b200.csrc import build

try:                                   # the library is there already, or nvcc is there to make it
    if not build.library_path().is_file():
        build.find_nvcc()
except RuntimeError as problem:
    pytest.skip(f"the CUDA library cannot be built here: {problem}", allow_module_level=True)

XL = {"qkv": (4800, 1600), "proj": (1600, 1600), "fc": (6400, 1600), "proj2": (1600, 6400)}
SMALL = {"qkv": (2304, 768), "proj": (768, 768), "fc": (3072, 768), "proj2": (768, 3072)}
LARGE = {"qkv": (3840, 1280), "proj": (1280, 1280), "fc": (5120, 1280), "proj2": (1280, 5120)}


@pytest.mark.parametrize("shape,M,tile", [
    (XL["qkv"], 2048, 192), (XL["fc"], 2048, 256), (XL["proj"], 2048, 192), (XL["qkv"], 1024, 160), (XL["fc"], 768, 160),
    (XL["fc"], 256, 96), (XL["proj"], 1024, 96), (XL["qkv"], 512, 160),
    (SMALL["qkv"], 2048, 256), (SMALL["fc"], 2048, 192), (SMALL["proj"], 2048, 96),
])
def test_tile_width_is_the_measured_best(shape, M, tile):
    N, K = shape
    assert ops.prefill_plan(M, N, K) == (tile, 1)


@pytest.mark.parametrize("shape,M", [(XL["proj2"], 128), (XL["proj2"], 256), (XL["proj2"], 576), (XL["proj2"], 1024),
                                     (SMALL["proj2"], 128), (SMALL["proj2"], 512), (SMALL["proj2"], 2048), (XL["proj"], 128)])
def test_long_k_with_few_tiles_is_split(shape, M):
    N, K = shape
    tile, parts = ops.prefill_plan(M, N, K)
    assert parts > 1, (tile, parts)


@pytest.mark.parametrize("shape,M,plan", [
    (XL["proj"], 128, (64, 4)), (XL["proj"], 768, (160, 2)), (XL["proj2"], 128, (128, 8)), (XL["proj2"], 512, (256, 4)),
    (XL["proj2"], 1024, (192, 2)), (XL["qkv"], 128, (96, 2)), (SMALL["proj2"], 768, (192, 4)), (SMALL["proj"], 256, (32, 2)),
    # a shape the model was not fitted to (GPT-2 large), measured afterwards: the pick is the best of 8 widths x 4 splits
    (LARGE["qkv"], 576, (160, 1)), (LARGE["proj"], 576, (96, 2)), (LARGE["fc"], 576, (192, 1)), (LARGE["proj2"], 576, (256, 4)),
    (LARGE["proj2"], 192, (128, 4)), (LARGE["qkv"], 1088, (256, 1)), (LARGE["proj2"], 1088, (160, 2)),
])
def test_split_plan_is_the_measured_best(shape, M, plan):
    N, K = shape
    assert ops.prefill_plan(M, N, K) == plan


def test_a_split_fits_the_sms_and_the_tile():
    for M in (65, 100, 128, 300, 576, 1000, 2048):
        for N, K in list(XL.values()) + list(SMALL.values()) + [(264, 12800), (8, 64), (50257, 1600)]:
            for sms in (148, 132, 64):
                tile, parts = ops.prefill_plan(M, N, K, sms)
                assert 32 <= tile <= 256 and tile % 32 == 0 and parts in (1, 2, 4, 8)
                if parts > 1:
                    tiles = -(-M // 128) * -(-N // tile)
                    blocks = -(-K // 64)
                    assert tiles * parts <= sms and tile % (16 * parts) == 0 and N % 8 == 0
                    assert 128 * tile * 4 <= 196608                              # the sums meet in the stage ring
                    assert (parts - 1) * -(-blocks // parts) < blocks       # every part has a K block


def test_wide_rows_keep_to_the_staged_widths_when_it_pays():
    # 32-bit rows in and out: 192 columns go through the staged epilogue, 256 do not
    assert ops.prefill_plan(2048, 1600, 6400, wide_rows=True)[0] == 192
    assert ops.prefill_plan(2048, 1600, 1600, wide_rows=True)[0] == 192
