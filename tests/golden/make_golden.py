"""One-off anchor of the plain implementation (tests/plain/qwen2_plain.py) to the
reference's own CPU code.

What it does: writes a very small random Qwen2 model (model.safetensors + config.json, in
this folder), runs walkinglabs/microLLM-rocm's `microllm_hf_infer` built for the CPU
(-DMICROLLM_ENABLE_HIP=OFF) on a few prompts with `--workload prefill --logits-output`, and
stores the last-position logits it wrote in `reference_logits.json`, together with the
logits after a cached decode step (`--workload both --new-tokens 3 --cache-logits-output`).
tests/test_plain.py then checks the plain implementation against these files; the reference
binary is not needed again.

Usage:  python tests/golden/make_golden.py /path/to/microllm_hf_infer
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from microllm_rocm_b200.config import Qwen2Config, get_architecture  # noqa: E402
from microllm_rocm_b200.weights import write_random_model  # noqa: E402

CONFIGS = {
    # tied head, one kv head, group of 4
    "a": dict(vocab_size=96, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
              intermediate_size=48, max_position_embeddings=64, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, torch_dtype="float32", bos_token_id=0, eos_token_id=1),
    # untied head, two kv heads, group of 3, other theta and eps, three layers
    "b": dict(vocab_size=80, hidden_size=48, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
              intermediate_size=40, max_position_embeddings=64, rope_theta=1e6, rms_norm_eps=1e-5,
              tie_word_embeddings=False, torch_dtype="float32", bos_token_id=0, eos_token_id=1),
}
PROMPTS = {"a": [[5, 17, 90, 3, 9], [1], [7, 7, 7, 7, 7, 7, 7, 7, 7, 7, 7, 2, 95, 0, 33, 41, 8]],
           "b": [[79, 0, 12, 45, 45, 3, 60, 21, 9], [33, 2]]}


def main():
    binary = sys.argv[1]
    arch = get_architecture("Qwen2ForCausalLM")
    golden = {}
    for key, raw in CONFIGS.items():
        folder = os.path.join(HERE, f"model_{key}")
        cfg = Qwen2Config.from_dict(raw)
        write_random_model(arch, cfg, seed=11 + len(key), folder=folder, storage_dtype="float32")
        entries = []
        for prompt in PROMPTS[key]:
            with tempfile.TemporaryDirectory() as tmp:
                out = os.path.join(tmp, "l.f32")
                cached = os.path.join(tmp, "c.f32")
                base = [binary, "--config", os.path.join(folder, "config.json"), "--weights",
                        os.path.join(folder, "model.safetensors"), "--tokens", ",".join(map(str, prompt)),
                        "--device", "cpu"]
                subprocess.run(base + ["--workload", "prefill", "--logits-output", out], check=True,
                               capture_output=True)
                last = np.fromfile(out, dtype="<f4")
                run = subprocess.run(base + ["--workload", "both", "--new-tokens", "3", "--cache-logits-output", cached],
                                     check=True, capture_output=True, text=True)
                info = json.loads(run.stdout.strip().splitlines()[-1])
                after = np.fromfile(cached, dtype="<f4")
            entries.append({"prompt": prompt, "last_logits": [float(x) for x in last],
                            "generated": info.get("generated_tokens") or info.get("tokens"),
                            "cached_logits": [float(x) for x in after]})
        golden[key] = entries
    with open(os.path.join(HERE, "reference_logits.json"), "w") as f:
        json.dump(golden, f)
    print("wrote", os.path.join(HERE, "reference_logits.json"))


if __name__ == "__main__":
    main()
