#!/usr/bin/env python3
"""Makes reference_logits.npz: logits of the unmodified jiamumuzhao/vllm-cpp for two tiny models.

    python baseline/build_reference.py                       # libvllm.a + ref_driver (needs the checkout)
    python tests/golden/make_reference_logits.py [--out tests/golden/reference_logits.npz]    # needs a GPU

For each configuration of GOLDEN_CONFIGS the weights of helpers.make_weights(cfg, 0, "float32") are
written as a model folder, and for each prompt length the reference's QwenModel::forward
(src/model/qwen.cpp:291-328) is fed the prompt token by token from an empty cache through
baseline/ref_driver.cpp; the logits of every position are stored under "<config>_<length>".
Only models the reference computes rightly can be anchored this way: tied embeddings (it copies an
untied lm_head over the embedding table, qwen.cpp:279-281) and rms_norm_eps = 1e-6 (it passes that
literal, :303,312,322).  tests/test_plain.py compares the plain implementation with the stored file.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.dirname(HERE)]

import plain_qwen2 as plain                                             # noqa: E402
from helpers import GOLDEN_CONFIGS, GOLDEN_PROMPTS, make_weights, token_ids          # noqa: E402
from baseline.build_reference import driver_env, driver_path            # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "reference_logits.npz"))
    a = ap.parse_args()
    driver = driver_path()
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, cfg in GOLDEN_CONFIGS.items():
            folder = os.path.join(tmp, name)
            plain.write_model_folder(folder, cfg, make_weights(cfg, 0, "float32"), store="F32")
            for n in GOLDEN_PROMPTS:
                ids = token_ids(cfg, n, seed=n)
                raw = os.path.join(tmp, f"{name}_{n}.f32")
                subprocess.run([driver, "logits", "--model", folder, "--tokens", ",".join(map(str, ids)), "--out", raw,
                                "--block-size", "16", "--max-model-len", str(cfg["max_position_embeddings"])],
                               check=True, env=driver_env(), stdout=subprocess.DEVNULL)
                out[f"{name}_{n}"] = np.fromfile(raw, dtype=np.float32).reshape(n, cfg["vocab_size"])
    np.savez_compressed(a.out, **out)
    print(f"wrote {a.out}: " + ", ".join(f"{k}{v.shape}" for k, v in out.items()))


if __name__ == "__main__":
    main()
