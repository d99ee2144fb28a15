"""Decisions that are made on the host before a kernel is launched: how the streaming product cuts its
blocks, which tile size the experts get.  No GPU and no compiled library is needed for these."""
import pytest


def test_streaming_blocks_stay_inside_a_block_of_sixteen_warps():
    from fieldrun_b200.csrc import ops
    for tiles in (1, 8, 57, 220, 4000):
        for features, inner in ((8192, 3072), (3072, 6144), (1536, 3072), (3072, 1536), (48, 64), (16, 32)):
            for tile_rows in (8, 16, 32):
                for paired in (False, True):
                    shape = ops.stream_shape(tiles, features, inner, tile_rows, paired)
                    assert shape["groups"] in (1, 2, 4) and shape["splits"] >= 1
                    assert shape["splits"] * shape["groups"] * (tile_rows // 8) <= 16
                    # a part of the inner size is a multiple of 128, so at most inner / 128 parts have work
                    assert shape["splits"] <= max(1, inner // 128)


def test_streaming_blocks_cut_the_inner_size_more_when_there_are_few_tiles():
    from fieldrun_b200.csrc import ops
    one_layer = ops.stream_shape(1, 3072, 6144, 8)["splits"]          # a dense layer: one "expert"
    many = ops.stream_shape(220, 3072, 1536, 8)["splits"]
    assert one_layer > many >= 2


@pytest.mark.parametrize("assignments,experts,expected", [(8, 256, 8), (64, 256, 8), (512, 256, 8), (1536, 256, 16), (3000, 256, 16)])
def test_streamed_experts_get_tiles_of_few_rows(assignments, experts, expected):
    import torch
    from fieldrun_b200.config import PartSpec
    from fieldrun_b200.parts import build_part
    spec = PartSpec("routed_experts", {"hidden_size": 128, "num_experts": experts, "top_k": 8, "expert_width": 128,
                                       "scoring": "sigmoid", "renormalize": True, "routed_scale": 1.0, "use_bias": True},
                    {"router": "r", "bias": "b", "w1": "e.{e}.w1", "w3": "e.{e}.w3", "w2": "e.{e}.w2"})
    part = build_part("feed_forward", spec, torch.bfloat16)
    assert not part.on_tensor_cores(assignments)
    assert part.tile_rows(assignments) == expected
