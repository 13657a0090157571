"""The counter-based generator of the random-weights mode: the same values on the host and on the device."""
import numpy as np
import pytest
import torch

from vllm_cpp_b200.weights import random_init as ri


def float64_box_muller(key, first, count):
    """The generator's formula restated in float64 with library functions (docstring of weights/random_init.py)."""
    mask = (1 << 64) - 1
    out = np.empty(count)
    for j in range(count):
        z = (key + (first + j + 1) * 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        u1 = ((z >> 40) + 1) / 2.0 ** 24
        angle = 2.0 * np.pi * (((z >> 16) & 0xFFFFFF) + 0.5) / 2.0 ** 24
        out[j] = np.sqrt(-2.0 * np.log(u1)) * np.cos(angle)
    return out


def test_values_follow_the_formula():
    key = ri.tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    got = ri.standard_normal(key, 1000, 4000).astype(np.float64)
    want = float64_box_muller(key, 1000, 4000)
    assert np.abs(got - want).max() < 2e-6


def test_a_value_depends_on_seed_name_and_index_only():
    key = ri.tensor_key(7, "a.weight")
    whole = ri.normal_values(key, 0, 3_000_000, 0.0, 0.02)          # crosses the generator's chunks
    assert np.array_equal(ri.normal_values(key, 1_048_000, 5000, 0.0, 0.02), whole[1_048_000: 1_053_000])
    assert not np.array_equal(ri.normal_values(ri.tensor_key(7, "b.weight"), 0, 100, 0.0, 0.02), whole[:100])
    assert not np.array_equal(ri.normal_values(ri.tensor_key(8, "a.weight"), 0, 100, 0.0, 0.02), whole[:100])
    rows = ri.random_rows("a.weight", (1000, 3000), [0, 17, 999], "matrix", 7, 0.02, 0.1)
    assert np.array_equal(rows, whole.reshape(1000, 3000)[[0, 17, 999]])
    t = ri.random_tensor("a.weight", (1000, 3000), "matrix", 7, 0.02, 0.1)
    assert np.array_equal(t.numpy().ravel(), whole)
    g = ri.random_tensor("g.weight", (4096,), "gain", 7, 0.02, 0.1).numpy()
    assert abs(g.mean() - 1.0) < 0.01 and abs(g.std() - 0.1) < 0.01


def test_moments():
    x = ri.standard_normal(ri.tensor_key(0, "moments"), 0, 2_000_000).astype(np.float64)
    assert abs(x.mean()) < 4e-3 and abs(x.std() - 1.0) < 4e-3
    assert abs((x ** 3).mean()) < 2e-2 and abs((x ** 4).mean() - 3.0) < 5e-2
    assert np.isfinite(x).all() and 4.5 < np.abs(x).max() < 6.0


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype,role", [((257, 1031), torch.float32, "matrix"), ((3584,), torch.float32, "gain"),
                                             ((301, 80), torch.bfloat16, "matrix"), ((5, 7, 11), torch.bfloat16, "bias")])
def test_device_values_equal_host_values_to_the_bit(shape, dtype, role):
    host = ri.random_tensor("model.layers.1.self_attn.q_proj.weight", shape, role, 11, 0.02, 0.05, dtype=dtype)
    dev = ri.random_tensor("model.layers.1.self_attn.q_proj.weight", shape, role, 11, 0.02, 0.05, dtype=dtype, device="cuda")
    assert dev.is_cuda and dev.dtype == dtype
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    assert torch.equal(dev.cpu().view(bits), host.view(bits))


@pytest.mark.gpu
def test_rows_of_a_large_device_tensor_can_be_rebuilt_on_the_host():
    """At the vocabulary and width of Qwen2.5-7B: far rows of a tensor filled on the device against the
    host's values for those rows alone (indices beyond 2^29 elements)."""
    shape = (152064, 3584)
    dev = ri.random_tensor("lm_head.weight", shape, "matrix", 0, 0.02, 0.02, dtype=torch.bfloat16, device="cuda")
    rows = [0, 1, 77777, 152063]
    host = torch.from_numpy(ri.random_rows("lm_head.weight", shape, rows, "matrix", 0, 0.02, 0.02)).to(torch.bfloat16)
    assert torch.equal(dev[rows].cpu().view(torch.int16), host.view(torch.int16))
    assert abs(float(dev[:4096].float().std()) - 0.02) < 5e-4


@pytest.mark.gpu
def test_device_init_equals_the_written_folder(tmp_path):
    """init_random_on_device fills a model with what write_random_model stores and the loader reads."""
    from helpers import TINY_B
    from vllm_cpp_b200.config.registry import resolve_architecture
    from vllm_cpp_b200.parts.model import DecoderModel
    from vllm_cpp_b200.weights.loader import load_checkpoint
    for dtype, name in ((torch.bfloat16, "bfloat16"), (torch.float32, "float32")):
        _, spec = resolve_architecture(TINY_B, "")
        a, b = DecoderModel(spec, dtype, "cuda"), DecoderModel(spec, dtype, "cuda")
        ri.init_random_on_device(a, 4)
        ri.write_random_model(str(tmp_path / name), TINY_B, seed=4, dtype=name)
        load_checkpoint(b, str(tmp_path / name))
        assert torch.equal(a.embed, b.embed) and torch.equal(a.lm_head, b.lm_head)
        for x, y in zip(a.blocks, b.blocks):
            assert torch.equal(x.mixer.w_qkv, y.mixer.w_qkv) and torch.equal(x.mixer.b_qkv, y.mixer.b_qkv)
            assert torch.equal(x.feed_forward.w_down, y.feed_forward.w_down)
            assert torch.equal(x.mixer_norm.weight, y.mixer_norm.weight)
