#!/usr/bin/env python3
"""Write a model folder (config.json + model.safetensors, float32) in MegEngine/InferLLM's own
.bin container, so that the compiled reference can load it.

Layout as the reference's converter writes it and its loader reads it
(application/llama/convert.py:69-143, src/core/graph.cpp:270-333, src/graph/llama_like.cpp:26-52):
magic 0x123456; five int32 offsets/lengths; the parameters n_embd, n_head, n_layer, fc_hidden,
n_vocab; the vocabulary as n_vocab x {uint32 length, bytes} (empty strings here: the harness feeds
token ids); then per tensor {n_dims, name_len, ftype = 0 (float32); dims; name; raw data}.
Tensor names are the checkpoint's own; the reference maps them through its alias table
(src/graph/llama_like.cpp:9-22).
"""
import json
import struct
import sys

from safetensors.torch import load_file


def main(folder, out):
    cfg = json.load(open(f"{folder}/config.json"))
    tensors = load_file(f"{folder}/model.safetensors")
    params = struct.pack("<5i", cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_hidden_layers"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    vocab = b"".join(struct.pack("<I", 0) for _ in range(cfg["vocab_size"]))
    header_len = 4 + 5 * 4
    param_off = header_len
    vocab_off = param_off + len(params)
    tensor_off = vocab_off + len(vocab)
    with open(out, "wb") as f:
        f.write(struct.pack("<i", 0x123456))
        f.write(struct.pack("<5i", param_off, len(params), vocab_off, len(vocab), tensor_off))
        f.write(params)
        f.write(vocab)
        for name, t in tensors.items():
            t = t.float().contiguous()
            nb = name.encode()
            f.write(struct.pack("<3i", t.dim(), len(nb), 0))
            f.write(struct.pack(f"<{t.dim()}i", *t.shape))
            f.write(nb)
            f.write(t.numpy().tobytes())


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
