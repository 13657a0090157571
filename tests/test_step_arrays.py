"""The work lists that the attention part derives from a step on the host: how the keys of a decode-only
step are cut into splits of equal length, and which grid that needs."""
import numpy as np
import pytest
import torch

from vllm_cpp_b200.config.model_spec import PartSpec
from vllm_cpp_b200.csrc import ops
from vllm_cpp_b200.engine.runner import HostStep
import vllm_cpp_b200.parts.model  # noqa: F401  (registers the parts)
from vllm_cpp_b200.parts.attention import PagedAttention


@pytest.fixture(autouse=True)
def b200_sm_count(monkeypatch):
    """These tests run without a device: the work lists are sized for a B200's 148 SMs."""
    monkeypatch.setattr(ops, "_sm_count", 148)


def part(nh, nkv, window=0):
    return PagedAttention(hidden_size=nh * 128, num_heads=nh, num_kv_heads=nkv, head_dim=128, qkv_bias=True,
                          out_bias=False, window=window, position=PartSpec("rope", {"theta": 1e6, "rotary_dim": 128, "pairing": "half"}),
                          dtype=torch.bfloat16, device="cpu")


def splits_of(att, ctx_lens):
    host = HostStep([1] * len(ctx_lens), list(ctx_lens), 16)
    per = int(att.step_arrays()[att._splits_key()](host)[0])
    return per, host.shapes[att._splits_key()]


@pytest.mark.parametrize("nh,nkv,batch,ctx,per,grid", [(28, 4, 8, 4095, 8, 8), (28, 4, 1, 4095, 4, 16), (28, 4, 64, 4095, 64, 1),
                                                       (28, 4, 32, 4095, 32, 2), (40, 8, 8, 100, 1, 2), (28, 4, 1, 0, 1, 1)])
def test_equal_contexts_fill_the_device_once(nh, nkv, batch, ctx, per, grid):
    assert splits_of(part(nh, nkv), [ctx] * batch) == (per, grid)


@pytest.mark.parametrize("seed", range(20))
def test_mixed_contexts(seed):
    rng = np.random.default_rng(seed)
    nkv = int(rng.choice([1, 2, 4, 8]))
    window = int(rng.choice([0, 0, 700]))
    att = part(nkv * int(rng.integers(1, 8)), nkv, window)
    ctx = rng.integers(0, int(rng.choice([200, 5000, 40000])), size=int(rng.integers(1, 200)))
    per, grid = splits_of(att, ctx)
    hi = ctx + 1
    lo = np.maximum(0, hi - window) if window else 0 * hi
    tiles = -(-hi // ops.DECODE_KEY_TILE) - lo // ops.DECODE_KEY_TILE
    need = -(-tiles // per)
    slots = att.decode_slots(len(ctx))
    # the grid holds every request's splits and is no larger than twice what the longest needs
    assert need.max() <= grid <= ops.DECODE_MAX_SPLITS and 3 * grid <= 4 * need.max() + 3 and grid in att.SPLIT_GRIDS
    longest = int(tiles.max())
    floor = max(-(-longest // ops.DECODE_MAX_SPLITS), min(4, -(-longest // 8)))     # the grid's limit; splits not too short
    # one wave, unless the floor decides
    assert need.sum() <= slots or per == floor
    # and no longer splits than that takes
    if per > floor:
        assert (-(-tiles // (per - 1))).sum() > slots


def test_steps_with_prompt_portions_have_no_splits():
    att = part(28, 4)
    host = HostStep([1, 5], [10, 0], 16)
    assert int(att.step_arrays()[att._splits_key()](host)[0]) == 0 and not host.shapes
