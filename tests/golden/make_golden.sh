#!/bin/sh
# Regenerates the files of tests/golden/ from MegEngine/InferLLM's own code, compiled on the CPU.
#
#   tests/golden/make_golden.sh REFERENCE_SOURCE_DIR [BUILD_DIR]
#
# 1. builds the reference's library with its naive kernels (cmake -DINFER_ARCH=naive);
# 2. writes a tiny random LLaMA (golden_model/: config.json + float32 model.safetensors) with
#    inferllm_b200's random-weights writer, and the same weights in the reference's .bin container;
# 3. runs ref_harness on golden_tokens.txt and stores its logits in golden_logits.f32.
# 4. runs ref_ops_harness, which calls the reference's grouped-head attention loops directly, and
#    stores their inputs and results in golden_gqa_ops.f32.
# tests/test_plain_and_golden.py then compares the plain implementation (tests/plain_llama.py) with those
# logits; it needs neither the reference nor a compiler.
set -e
REF=${1:?reference source directory}
HERE=$(cd "$(dirname "$0")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
BUILD=${2:-$ROOT/baseline/_ref/build}
mkdir -p "$BUILD"
(cd "$BUILD" && cmake "$REF" -DCMAKE_POLICY_VERSION_MINIMUM=3.5 -DINFER_ARCH=naive > cmake.log 2>&1 \
    && make -j8 InferLLM > make.log 2>&1)
g++ -std=c++11 -O2 -Wno-multichar -I "$REF/src" -I "$REF/include" "$HERE/ref_harness.cpp" \
    "$BUILD/libInferLLM.a" -lpthread -o "$BUILD/ref_harness"
g++ -std=c++11 -O2 -Wno-multichar -I "$REF/src" -I "$REF/include" "$HERE/ref_ops_harness.cpp" \
    "$BUILD/libInferLLM.a" -lpthread -o "$BUILD/ref_ops_harness"
"$BUILD/ref_ops_harness" "$HERE/golden_gqa_ops.f32"
cd "$ROOT"
python - <<PY
import json, torch, numpy as np
from inferllm_b200 import config_from_dict, write_random_model
# The reference fixes eps 1e-6 in the layers and 1e-5 in the head, theta 10000, one KV head per
# head, no tying (src/graph/llama_like.cpp:77-78, src/core/graph.h:160-163): the golden model
# keeps to that (and to an intermediate size that the reference's rounding rule leaves alone,
# src/core/graph.cpp:61); "final_norm_eps" is read by the test only.
cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
           num_key_value_heads=2, head_dim=16, intermediate_size=88, vocab_size=64, rope_theta=10000.0,
           rms_norm_eps=1e-6, max_position_embeddings=256, tie_word_embeddings=False)
write_random_model(config_from_dict(cfg), "$HERE/golden_model", seed=2024, dtype=torch.float32)
c = json.load(open("$HERE/golden_model/config.json")); c["final_norm_eps"] = 1e-5
json.dump(c, open("$HERE/golden_model/config.json", "w"), indent=1)
rng = np.random.default_rng(5)
with open("$HERE/golden_tokens.txt", "w") as f:
    for n in (9, 1, 40):
        f.write(" ".join(str(t) for t in rng.integers(0, 64, n)) + "\n")
PY
python "$HERE/write_ref_bin.py" "$HERE/golden_model" "$BUILD/golden_model.bin"
"$BUILD/ref_harness" "$BUILD/golden_model.bin" "$HERE/golden_tokens.txt" "$HERE/golden_logits.f32" 2> "$BUILD/harness.log"
ls -la "$HERE"
