"""The reference arm of the benchmark: the unmodified CocoRoF/iian, built with CMake under ``baseline/_ref``,
run through its own command line (``iian bench``, src/iian/cli/cmd_bench.cpp:18-96) on the same shape with
random weights.  Nothing of ``iian_b200``'s engine is on that path: this module only writes the model file the
reference reads (a GGUF with bfloat16 tensors under the reference's tensor names, src/iian/arch/qwen3.cpp:24-57,
and a synthetic byte-pair vocabulary of the right length, because its engine detokenizes what it generates) and
parses the JSON the reference prints.

Build (once, on the machine that has nvcc; the binaries travel with the repository's working tree):

    cmake -S <reference> -B /tmp/refbuild -G Ninja -DGGML_CUDA=ON -DCMAKE_CUDA_ARCHITECTURES=100 \\
          -DGGML_NATIVE=OFF -DIIAN_BUILD_TESTS=OFF -DIIAN_CURL=OFF -DCMAKE_BUILD_TYPE=Release
    ninja -C /tmp/refbuild iian iian-cli
    cp /tmp/refbuild/tools/iian/iian baseline/_ref/bin/;  cp -L <the five lib*.so> baseline/_ref/lib/
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
EXE = os.path.join(REF, "bin", "iian")
LIB = os.path.join(REF, "lib")

PER_LAYER = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
             "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm",
             "self_attn.k_norm": "attn_k_norm", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
             "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}


def available() -> Optional[str]:
    """None if the reference's binaries are there, else why not."""
    if not os.path.isfile(EXE):
        return f"the reference's command line was not built ({os.path.relpath(EXE, os.path.dirname(HERE))} is missing)"
    for lib in ("libiian.so", "libggml.so.0", "libggml-base.so.0", "libggml-cpu.so.0"):
        if not os.path.isfile(os.path.join(LIB, lib)):
            return f"the reference's library {lib} is missing under baseline/_ref/lib"
    return None


def gguf_name(ours: str) -> str:
    fixed = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    if ours in fixed:
        return fixed[ours]
    parts = ours.split(".")            # model.layers.<i>.<what>.weight
    i = parts[2]
    what = ".".join(parts[3:-1])
    return f"blk.{i}.{PER_LAYER[what]}.weight"


def write_gguf(path: str, shape: dict, seed: int = 0, device: str = "cpu", std: float = 0.02) -> int:
    """The shape ``shape`` (config.json keys) with the same random weights the engine's own arm draws (the generator
    is keyed by seed and tensor name), as a GGUF the reference loads: matrices in bfloat16, norm weights in float32.
    Returns the file's size in bytes."""
    import gguf
    import numpy as np
    import torch
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    from iian_b200.config.registry import get_architecture
    from iian_b200.engine.model import declare_tensors
    from iian_b200.models.qwen3 import qwen3_config_from_dict
    from iian_b200.weights import random_init as ri

    cfg = qwen3_config_from_dict(shape)
    arch = get_architecture("Qwen3ForCausalLM")
    declared = declare_tensors(arch, arch.build_spec(cfg))
    wr = gguf.GGUFWriter(path, "qwen3")
    hd = cfg.head_dim
    wr.add_uint32("qwen3.block_count", cfg.num_hidden_layers)
    wr.add_uint32("qwen3.context_length", cfg.max_position_embeddings)
    wr.add_uint32("qwen3.embedding_length", cfg.hidden_size)
    wr.add_uint32("qwen3.feed_forward_length", cfg.intermediate_size)
    wr.add_uint32("qwen3.attention.head_count", cfg.num_attention_heads)
    wr.add_uint32("qwen3.attention.head_count_kv", cfg.num_key_value_heads)
    wr.add_uint32("qwen3.attention.key_length", hd)
    wr.add_uint32("qwen3.attention.value_length", hd)
    wr.add_uint32("qwen3.rope.dimension_count", hd)
    wr.add_float32("qwen3.attention.layer_norm_rms_epsilon", cfg.rms_norm_eps)
    wr.add_float32("qwen3.rope.freq_base", cfg.rope_theta)
    wr.add_uint32("qwen3.vocab_size", cfg.vocab_size)
    # a synthetic byte-pair vocabulary: one distinct printable word per id (the engine turns generated ids into text)
    wr.add_string("tokenizer.ggml.model", "gpt2")
    wr.add_string("tokenizer.ggml.pre", "qwen2")
    wr.add_array("tokenizer.ggml.tokens", [f"w{i:06d}" for i in range(cfg.vocab_size)])
    wr.add_array("tokenizer.ggml.token_type", [1] * cfg.vocab_size)
    wr.add_array("tokenizer.ggml.merges", ["w 0"])
    wr.add_uint32("tokenizer.ggml.eos_token_id", 1)
    wr.add_uint32("tokenizer.ggml.bos_token_id", 1)
    wr.add_bool("tokenizer.ggml.add_bos_token", False)
    dev = torch.device(device)
    for name, spec in declared.items():
        if spec.optional:
            continue
        if name == "lm_head.weight" and cfg.tie_word_embeddings:
            continue
        t = ri.draw(name, spec, seed, dev, std, 0.0)
        if spec.init == "ones_jitter":
            wr.add_tensor(gguf_name(name), t.cpu().numpy().astype(np.float32))
        else:
            raw = t.to(torch.bfloat16).cpu().contiguous().view(torch.uint8).numpy()      # [rows, 2 * cols] bytes
            wr.add_tensor(gguf_name(name), raw, raw_dtype=gguf.GGMLQuantizationType.BF16)
        del t
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return os.path.getsize(path)


def run_bench(gguf_path: str, concurrency: int, prompt_tokens: int, gen_tokens: int, extra=(), timeout: int = 1500) -> dict:
    """``iian bench <gguf> --concurrency C --prompt-tokens P --gen-tokens G --json`` of the reference; its JSON row."""
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = LIB + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    cmd = [EXE, "bench", gguf_path, "--concurrency", str(concurrency), "--prompt-tokens", str(prompt_tokens),
           "--gen-tokens", str(gen_tokens), "--json"] + list(extra)
    t0 = time.time()
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0:
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-3:]
        raise RuntimeError(f"the reference's bench exited with {proc.returncode}: {' | '.join(tail)}")
    text = proc.stdout
    rows = json.loads(text[text.index("["):])
    row = dict(rows[0])
    row["wall_total_s"] = time.time() - t0
    return row
