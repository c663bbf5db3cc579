"""The command line without a GPU: commands, option precedence (command line > IIAN_<FLAG> > --config
file > default, src/iian/cli/args.cpp:152-183), the random-weights command."""
import json
import os
import subprocess
import sys

import pytest

from helpers import TINY
from iian_b200.cli.args import Options
from iian_b200.cli.main import engine_config_from_args, main, sampling_from_args, _add_engine_flags, _add_sampling_flags

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def opts():
    o = Options("t", "t")
    _add_sampling_flags(o)
    _add_engine_flags(o)
    return o


def test_option_precedence(tmp_path, monkeypatch):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps({"max-num-seqs": 7, "block_size": 32, "temp": 0.1}))
    monkeypatch.setenv("IIAN_BLOCK_SIZE", "64")
    ns = opts().parse(["--config", str(cfg), "--temp", "0.9"])
    assert ns.max_num_seqs == 7              # from the file
    assert ns.block_size == 64               # the environment beats the file
    assert ns.temp == 0.9                    # the command line beats both
    assert ns.max_num_batched_tokens == 1024 and ns.top_p == 1.0      # defaults
    assert {"max_num_seqs", "block_size", "temp"} <= ns.given and "top_p" not in ns.given
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"no-such-flag": 1}))
    with pytest.raises(SystemExit):
        opts().parse(["--config", str(bad)])


def test_flags_map_to_the_configs():
    ns = opts().parse(["-c", "512", "--kv-cache-tokens", "2048", "--block-size", "8", "--no-prefix-caching", "--no-warmup",
                       "--max-num-seqs", "3", "--max-num-batched-tokens", "99", "--no-chunked-prefill",
                       "--long-prefill-token-threshold", "5", "--scheduling-policy", "priority", "--dtype", "float32",
                       "--seed", "11", "-n", "9", "--temp", "0", "--top-k", "4", "--top-p", "0.5", "--min-p", "0.1"])
    e = engine_config_from_args(ns)
    assert (e.max_model_len, e.kv_cache_tokens, e.block_size, e.enable_prefix_caching, e.warmup) == (512, 2048, 8, False, False)
    assert (e.sched.max_num_seqs, e.sched.max_num_batched_tokens, e.sched.enable_chunked_prefill) == (3, 99, False)
    assert e.sched.long_prefill_token_threshold == 5 and e.sched.policy == "priority" and e.dtype == "float32" and e.seed == 11
    s = sampling_from_args(ns)
    assert s.max_tokens == 9 and s.is_greedy and s.top_k == 4 and s.top_p == 0.5 and s.min_p == 0.1 and s.seed == 11
    assert sampling_from_args(opts().parse([])).seed is None and sampling_from_args(opts().parse([])).temperature == 0.7
    p = sampling_from_args(opts().parse(["--repeat-penalty", "1.2", "--presence-penalty", "0.5", "--frequency-penalty", "-1",
                                         "--stop", "7,9"]))
    assert (p.repetition_penalty, p.presence_penalty, p.frequency_penalty, p.stop_token_ids) == (1.2, 0.5, -1.0, [7, 9])
    assert p.has_processors and not sampling_from_args(opts().parse([])).has_processors


def test_commands(capsys):
    assert main(["version"]) == 0 and "iian_b200" in capsys.readouterr().out
    assert main(["complet"]) == 1 and "did you mean 'complete'" in capsys.readouterr().err
    assert main([]) == 0 and "random-weights" in capsys.readouterr().out


def test_random_weights_command(tmp_path):
    src = tmp_path / "config.json"
    src.write_text(json.dumps(dict(TINY["C"], architectures=["Qwen3ForCausalLM"])))
    out = tmp_path / "model"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "iian"), "random-weights", str(src), str(out), "--seed", "3",
                           "--store-dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    from iian_b200.config.registry import load_model_config
    arch, cfg = load_model_config(str(out))
    assert arch.name == "Qwen3ForCausalLM" and cfg.sliding_window == 20 and cfg.hidden_size == 80
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "iian"), "random-weights", str(tmp_path / "nothing.json"), str(out)],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 1
