"""Weights: the safetensors container, loading by name with one clear error, random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TINY_A, TINY_B, make_weights
from vllm_cpp_b200 import resolve_architecture
from vllm_cpp_b200.parts.model import DecoderModel
from vllm_cpp_b200.weights.loader import WeightsError, load_checkpoint
from vllm_cpp_b200.weights.random_init import write_random_model
from vllm_cpp_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def cpu_model(cfg, dtype=torch.float32):
    _, spec = resolve_architecture(cfg)
    return DecoderModel(spec, dtype, "cpu")


def test_container_round_trip_and_types(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t)
    for k in t:
        assert f.tensor(k).dtype == t[k].dtype and torch.equal(f.tensor(k), t[k])
    # the plain reader sees the same bytes
    raw = open(p, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    assert json.loads(raw[8:8 + n])["a"]["shape"] == [3, 5]


def test_container_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="not found"):
        SafetensorsFile(str(tmp_path / "none"))
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 2]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))


def test_load_by_name_places_types(tmp_path):
    w = make_weights(TINY_B, 0, "float32")
    plain.write_model_folder(str(tmp_path), TINY_B, w, store="F32")
    m = cpu_model(TINY_B, torch.bfloat16)
    load_checkpoint(m, str(tmp_path))
    assert m.embed.dtype == torch.bfloat16 and m.lm_head is not m.embed and m.lm_head.dtype == torch.bfloat16
    att = m.blocks[1].mixer
    assert att.w_qkv.shape == (5 * 32, 96) and att.w_qkv.dtype == torch.bfloat16
    assert att.b_qkv.dtype == torch.float32          # stored in 32-bit, stays 32-bit
    assert m.blocks[0].mixer_norm.weight.dtype == torch.float32
    q = torch.from_numpy(w["model.layers.1.self_attn.q_proj.weight"]).to(torch.bfloat16)
    assert torch.equal(att.w_qkv[:96], q)
    m32 = cpu_model(TINY_B, torch.float32)
    load_checkpoint(m32, str(tmp_path))
    assert torch.equal(m32.blocks[2].feed_forward.w_gate_up[224:], torch.from_numpy(w["model.layers.2.mlp.up_proj.weight"]))


def test_tied_model_aliases_and_ignores_a_stored_copy(tmp_path):
    w = make_weights(TINY_A, 0, "float32")
    w["lm_head.weight"] = w["model.embed_tokens.weight"].copy()
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = np.ones(8, dtype=np.float32)
    plain.write_model_folder(str(tmp_path), TINY_A, w, store="F32")
    m = cpu_model(TINY_A)
    load_checkpoint(m, str(tmp_path))
    assert m.lm_head is m.embed


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = make_weights(TINY_B, 0, "float32")
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = np.zeros(7, dtype=np.float32)
    w["model.layers.2.mlp.down_proj.weight"] = np.zeros((224, 96), dtype=np.float32)
    w["model.layers.9.extra.weight"] = np.zeros(3, dtype=np.float32)
    plain.write_model_folder(str(tmp_path), TINY_B, w, store="F32")
    with pytest.raises(WeightsError) as e:
        load_checkpoint(cpu_model(TINY_B), str(tmp_path))
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.9.extra.weight" in msg
    assert "wrong shapes (2)" in msg and "q_proj.bias is [7], expected [96]" in msg
    assert "down_proj.weight is [224, 96], expected [96, 224]" in msg


def test_missing_files(tmp_path):
    with pytest.raises(WeightsError, match="no weights"):
        load_checkpoint(cpu_model(TINY_A), str(tmp_path))


def test_sharded_checkpoint(tmp_path):
    w = make_weights(TINY_A, 0, "float32")
    names = sorted(w)
    half = len(names) // 2
    for i, part in enumerate((names[:half], names[half:])):
        write_safetensors(str(tmp_path / f"s{i}.safetensors"), {n: torch.from_numpy(w[n]) for n in part})
    index = {"weight_map": {n: ("s0.safetensors" if n in names[:half] else "s1.safetensors") for n in names}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    m = cpu_model(TINY_A)
    load_checkpoint(m, str(tmp_path))
    assert torch.equal(m.embed, torch.from_numpy(w["model.embed_tokens.weight"]))


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=5, dtype="bfloat16")
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=5, dtype="bfloat16")
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=6, dtype="float32")
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["lm_head.weight"].float(), c["lm_head.weight"])
    cfg, w = plain.read_model_folder(str(tmp_path / "a"))
    assert cfg == TINY_B and set(w) == set(plain.parameter_shapes(TINY_B))
    assert all(w[k].shape == s for k, s in plain.parameter_shapes(TINY_B).items())
    assert abs(w["model.layers.0.mlp.gate_proj.weight"].std() - 0.02) < 0.002
    assert abs(w["model.norm.weight"].mean() - 1.0) < 0.02
    m = cpu_model(TINY_B, torch.bfloat16)
    load_checkpoint(m, str(tmp_path / "a"))
    assert torch.equal(m.embed, a["model.embed_tokens.weight"])
    # a plain forward runs on what was written
    assert np.isfinite(plain.forward(w, cfg, [1, 2, 3])).all()
