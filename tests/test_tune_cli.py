"""Argument handling of the kernel sweep (`python -m scanscam_b200.tune`): no device needed."""
import pytest

from scanscam_b200 import tune


def test_shapes_are_parsed():
    args = tune.parse_args(["cfg2,1024x262144,cl:8x4096x512,h16:16384x4096,shard:1024x131072", "--iters", "5"])
    assert args.iters == 5
    assert args.parsed == [("cfg2", "rows", (16384, 4096)), ("1024x262144", "rows", (1024, 262144)),
                           ("cl:8x4096x512", "cl", (8, 4096, 512)), ("h16:16384x4096", "h16", (16384, 4096)),
                           ("shard:1024x131072", "shard", (1024, 131072))]


@pytest.mark.parametrize("bad", ["cfg99", "12x", "cl:8x4096", "axb", "zz:4x4", "0x16", "fused:4x4x4"])
def test_bad_shapes_are_refused(bad):
    with pytest.raises(ValueError):
        tune.parse_shape(bad)


def test_unknown_family_is_refused():
    with pytest.raises(SystemExit):
        tune.parse_args(["cfg2", "--families", "warp,nosuch"])
