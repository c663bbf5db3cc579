#!/usr/bin/env python3
"""Regenerates the golden logits under tests/golden/ from the REFERENCE engine's own model code.

    python tests/golden/make_golden.py --reference /path/to/CocoRoF-iian [--build /tmp/iian-build]

For each tiny configuration it (1) writes a model folder with random weights (bfloat16 values, so that
every reader sees the same numbers), (2) writes the same weights as a float32 GGUF under the reference's
tensor names (src/iian/arch/qwen3.cpp:24-57) with `tokenizer.ggml.model = no_vocab`, (3) builds the
reference's libiian with CMake on the CPU and the small harness reference_logits.cpp against it, (4) runs
the reference's Qwen3 graph on one whole prompt with a float32 cache and stores the logits of every
position.  tests/test_plain.py compares tests/plain_qwen3.py with the stored logits.

Needs the `gguf` Python package (a file-format writer), cmake, ninja and a C++ compiler; no GPU, no network.
"""
import argparse
import json
import os
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CASES = {"tinyA": ("A", 33, 1), "tinyB": ("B", 61, 3)}       # name -> (configuration, prompt length, token seed)


def write_gguf(model_dir: str, path: str) -> None:
    import gguf
    import plain_qwen3 as plain
    cfg, w = plain.load_folder(model_dir)
    wr = gguf.GGUFWriter(path, "qwen3")
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    wr.add_uint32("qwen3.block_count", cfg["num_hidden_layers"])
    wr.add_uint32("qwen3.context_length", cfg["max_position_embeddings"])
    wr.add_uint32("qwen3.embedding_length", cfg["hidden_size"])
    wr.add_uint32("qwen3.feed_forward_length", cfg["intermediate_size"])
    wr.add_uint32("qwen3.attention.head_count", nh)
    wr.add_uint32("qwen3.attention.head_count_kv", cfg.get("num_key_value_heads", nh))
    wr.add_uint32("qwen3.attention.key_length", hd)
    wr.add_uint32("qwen3.attention.value_length", hd)
    wr.add_uint32("qwen3.rope.dimension_count", hd)
    wr.add_float32("qwen3.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"])
    wr.add_float32("qwen3.rope.freq_base", cfg["rope_theta"])
    wr.add_uint32("qwen3.vocab_size", cfg["vocab_size"])
    wr.add_string("tokenizer.ggml.model", "no_vocab")
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    per_layer = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
                 "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm",
                 "self_attn.k_norm": "attn_k_norm", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
                 "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    for i in range(cfg["num_hidden_layers"]):
        for ours, theirs in per_layer.items():
            names[f"model.layers.{i}.{ours}.weight"] = f"blk.{i}.{theirs}.weight"
    for ours, t in w.items():
        wr.add_tensor(names[ours], t.to(torch.float32).numpy().astype(np.float32))
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of CocoRoF/iian")
    ap.add_argument("--build", default="/tmp/iian-build")
    ap.add_argument("--work", default="/tmp/iian-golden")
    args = ap.parse_args()
    from helpers import random_tokens, tiny_config
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder

    if not os.path.isfile(os.path.join(args.build, "build.ninja")):
        subprocess.check_call(["cmake", "-S", args.reference, "-B", args.build, "-G", "Ninja", "-DIIAN_BUILD_TOOLS=OFF",
                               "-DCMAKE_BUILD_TYPE=Release"])
    subprocess.check_call(["cmake", "--build", args.build, "--target", "iian", "-j", "8"])
    os.makedirs(args.work, exist_ok=True)
    lib_dirs = sorted({os.path.dirname(os.path.join(dp, f)) for dp, _, fs in os.walk(args.build) for f in fs
                       if f.endswith(".so") and (f.startswith("libiian") or f.startswith("libggml"))})
    exe = os.path.join(args.work, "reference_logits")
    ggml = os.path.join(args.reference, "third_party", "ggml")
    cmd = ["g++", "-std=c++20", "-O2", os.path.join(HERE, "reference_logits.cpp"), "-o", exe,
           "-I", os.path.join(args.reference, "include"), "-I", os.path.join(ggml, "include"),
           "-I", os.path.join(args.reference, "third_party")]
    for d in lib_dirs:
        cmd += ["-L", d, f"-Wl,-rpath,{d}"]
    cmd += ["-liian", "-lggml", "-lggml-base", "-lggml-cpu"]
    subprocess.check_call(cmd)

    arch = get_architecture("Qwen3ForCausalLM")
    for name, (cfg_name, n_tok, tok_seed) in CASES.items():
        out_dir = os.path.join(HERE, name)
        cfg = tiny_config(cfg_name)
        write_model_folder(out_dir, arch, cfg, seed=100 + tok_seed, store_dtype=torch.bfloat16)
        toks = random_tokens(cfg.vocab_size, n_tok, tok_seed)
        with open(os.path.join(out_dir, "tokens.json"), "w") as f:
            json.dump(toks, f)
        gguf_path = os.path.join(args.work, f"{name}.gguf")
        tok_path = os.path.join(args.work, f"{name}.tokens")
        write_gguf(out_dir, gguf_path)
        with open(tok_path, "w") as f:
            f.write(" ".join(str(t) for t in toks))
        subprocess.check_call([exe, gguf_path, tok_path, os.path.join(out_dir, "logits.f32"), "paged"])
        for mode in ("flash", "softmax"):                      # the reference's other two attention paths, as a cross-check
            other = os.path.join(args.work, f"{name}.{mode}.f32")
            subprocess.check_call([exe, gguf_path, tok_path, other, mode])
            a = np.fromfile(os.path.join(out_dir, "logits.f32"), dtype="<f4")
            b = np.fromfile(other, dtype="<f4")
            print(f"{name}: reference paged vs {mode}: max |d| = {np.abs(a - b).max():.3g}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
