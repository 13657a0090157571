"""The plain implementation checked against itself and against hand-computed cases."""
import numpy as np

import plain_qwen2 as plain
from helpers import CONFIGS, make_weights, token_ids


def test_prefix_logits_do_not_depend_on_later_tokens():
    for name, (cfg, _) in CONFIGS.items():
        w = make_weights(cfg, 0, "float32")
        ids = token_ids(cfg, 40, 7)
        full = plain.forward(w, cfg, ids)
        part = plain.forward(w, cfg, ids[:23])
        assert np.abs(full[:23] - part).max() < 1e-9 * np.abs(full).max(), name


def test_window_changes_only_late_positions():
    cfg, _ = CONFIGS["C"]
    w = make_weights(cfg, 0, "float32")
    ids = token_ids(cfg, 60, 8)
    windowed = plain.forward(w, cfg, ids)
    full_cfg = dict(cfg, use_sliding_window=False)
    full = plain.forward(w, full_cfg, ids)
    win = cfg["sliding_window"]
    assert np.abs(windowed[:win] - full[:win]).max() == 0.0
    assert np.abs(windowed[win + 5:] - full[win + 5:]).max() > 1e-6 * np.abs(full).max()


def test_rope_rotates_pairs_by_position():
    x = np.zeros((3, 1, 8)); x[:, 0, 0] = 1.0            # pair (0, 4)
    y = plain.rope(x, [0, 1, 2], theta=10000.0)
    assert np.allclose(y[0, 0], x[0, 0])
    assert np.allclose(y[1, 0, [0, 4]], [np.cos(1.0), np.sin(1.0)], atol=1e-7)
    assert np.allclose(y[2, 0, [0, 4]], [np.cos(2.0), np.sin(2.0)], atol=1e-7)
    # pair (1, 5) turns by p / theta^(2/8)
    x = np.zeros((1, 1, 8)); x[0, 0, 5] = 1.0
    a = np.float32(3.0) / np.float32(10000.0) ** np.float32(0.25)
    y = plain.rope(x, [3], theta=10000.0)
    assert np.allclose(y[0, 0, [1, 5]], [-np.sin(a), np.cos(a)], atol=1e-6)


def test_attention_single_key_and_group_map():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((4, 6, 8)), rng.standard_normal((4, 2, 8)), rng.standard_normal((4, 2, 8))
    o = plain.attention(q, k, v, 6, 2)
    assert np.allclose(o[0, 0], v[0, 0]) and np.allclose(o[0, 5], v[0, 1])     # first token sees itself only
    s = (q[1, 4] @ k[:2, 1].T) / np.sqrt(8)
    p = np.exp(s - s.max()); p /= p.sum()
    assert np.allclose(o[1, 4], p @ v[:2, 1])
    ow = plain.attention(q, k, v, 6, 2, window=1)
    assert np.allclose(ow[3, 2], v[3, 0])


def test_rms_norm_and_swiglu_formulas():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms_norm(x, np.array([2.0, 1.0]), 0.0), [[2 * 3 / np.sqrt(12.5), 4 / np.sqrt(12.5)]])
    assert np.isclose(plain.silu(np.array(0.0)), 0.0) and np.isclose(plain.silu(np.array(2.0)), 2 / (1 + np.exp(-2)))


def test_sampler_follows_the_reference_cases():
    # tests/unit/test_sampler.cpp:6-41 of the reference
    assert plain.greedy(np.array([0.1, 2.0, 2.0, -1.0])) == 1
    probs = np.array([0.05, 0.85, 0.10], dtype=np.float32)
    assert plain.top_p_filter(probs, [0, 1, 2], 0.8) == [1]
    assert plain.top_k_filter(probs, [0, 1, 2], 3) == [1, 2, 0]
    logits = np.log(np.array([0.05, 0.85, 0.10], dtype=np.float32))
    assert plain.sample(logits, 1.0, 0.8, -1, 1.0, [], 0.5) == 1
    assert plain.sample(logits, 0.0, 1.0, -1, 1.0, [], 0.9) == 1
    # inverse CDF in id order without filters
    assert plain.sample(logits, 1.0, 1.0, -1, 1.0, [], 0.01) == 0
    assert plain.sample(logits, 1.0, 1.0, -1, 1.0, [], 0.95) == 2
    # penalty on a generated id flips the winner
    assert plain.sample(np.array([1.0, 0.9]), 0.0, 1.0, -1, 2.0, [0], 0.0) == 1


def test_folder_round_trip(tmp_path):
    cfg, _ = CONFIGS["A"]
    w = make_weights(cfg, 1, "bfloat16")
    plain.write_model_folder(str(tmp_path / "m"), cfg, w, store="BF16")
    cfg2, w2 = plain.read_model_folder(str(tmp_path / "m"))
    assert cfg2 == cfg and all(np.array_equal(w[k], w2[k]) for k in w)


def test_plain_sampler_equals_the_reference_sampler_code():
    """tests/golden/sampler_golden.json holds what the reference's own host sampler
    (src/sampler/sampler.cpp, src/sampler/topk_topp.cpp, compiled by tests/golden/make_sampler_golden.sh)
    returns for 48 seeded rows: greedy, temperature, top-k, top-p, ties."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "sampler_golden.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) == 48
    for c in cases:
        tok = plain.sample(np.array(c["logits"], dtype=np.float32), c["temperature"], c["top_p"], c["top_k"], 1.0, [], c["u"])
        assert tok == c["token"], c


def test_plain_logits_against_the_reference_itself():
    """tests/golden/reference_logits.npz holds what the unmodified reference computed on a B200 for two tiny
    tied models, token by token (made by tests/golden/make_reference_logits.py).  The reference rounds the
    operands of every product to half precision and is built with --use_fast_math (CMakeLists.txt:13), so
    the plain float64 result differs from it by that rounding; with the same operand rounding restated
    (operand=np.float16) the two agree several times closer.  A wrong formula (pairing of the rotation,
    eps, scale, order of norm and residual, head grouping) moves the logits by their own size."""
    import os
    from helpers import GOLDEN_CONFIGS, GOLDEN_PROMPTS
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_logits.npz"))
    for name, cfg in GOLDEN_CONFIGS.items():
        w = make_weights(cfg, 0, "float32")
        for n in GOLDEN_PROMPTS:
            ids = token_ids(cfg, n, seed=n)
            ref = golden[f"{name}_{n}"].astype(np.float64)
            assert ref.shape == (n, cfg["vocab_size"])
            scale = np.abs(ref).max()
            exact = plain.forward(w, cfg, ids)
            rounded = plain.forward(w, cfg, ids, operand=np.float16)
            assert np.abs(exact - ref).max() <= 2e-2 * scale, (name, n)
            assert np.abs(rounded - ref).max() <= 3e-3 * scale, (name, n)
            assert (exact.argmax(axis=1) == ref.argmax(axis=1)).all(), (name, n)
