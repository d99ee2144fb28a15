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


@pytest.mark.parametrize("assignments,decode,tensor_cores,expected", [
    (8, True, False, 8), (64, True, False, 8), (512, True, False, 8), (1024, True, False, 8), (1536, True, True, 32),
    (64, False, False, 8), (256, False, False, 8), (512, False, True, 32), (3000, False, True, 32), (10000, False, True, 64),
    (131072, False, True, 256)])
def test_experts_get_tiles_by_the_rows_an_expert_sees(assignments, decode, tensor_cores, expected):
    """256 experts: decode steps stream with tiles of 8 rows up to 4 rows per expert on average, prompts up to 1
    (their tokens crowd on fewer experts); beyond, tcgen05 with tiles of 32 rows and more."""
    import torch
    from fieldrun_b200.config import PartSpec
    from fieldrun_b200.parts import build_part
    spec = PartSpec("routed_experts", {"hidden_size": 128, "num_experts": 256, "top_k": 8, "expert_width": 128,
                                       "scoring": "sigmoid", "renormalize": True, "routed_scale": 1.0, "use_bias": True},
                    {"router": "r", "bias": "b", "w1": "e.{e}.w1", "w3": "e.{e}.w3", "w2": "e.{e}.w2"})
    part = build_part("feed_forward", spec, torch.bfloat16)
    assert part.on_tensor_cores(assignments, decode) == tensor_cores
    assert part.tile_rows(assignments, decode) == expected
