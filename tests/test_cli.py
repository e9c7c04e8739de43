"""The command line: option names of the reference, checks, and a run on the GPU."""
import json
import os
import subprocess
import sys

import pytest

from tiny_configs import TINY_A
from tiny_transformer_inference_engine_b200.engine.cli import build_parser, main

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_option_names_of_the_reference():
    a = build_parser().parse_args(["--ckpt", "m", "--prompt-ids", "1,2", "--token", "5", "--top_k", "3", "--top_p", "0.5",
                                   "--temperature", "0.7", "--num-gpu-blocks", "9", "--block-size", "8", "--serving"])
    assert (a.model, a.tokens, a.top_k, a.top_p, a.temperature, a.num_gpu_blocks, a.block_size) == ("m", 5, 3, 0.5, 0.7, 9, 8)
    d = build_parser().parse_args(["--model", "m"])
    assert (d.tokens, d.temperature, d.top_k, d.top_p, d.device, d.num_gpu_blocks, d.block_size) == (100, 1.0, 0, 1.0, "auto", 256, 16)


@pytest.mark.parametrize("bad", [["--tokens", "-1"], ["--temperature", "0"], ["--top-k", "-2"], ["--top-p", "0"], ["--top-p", "1.5"]])
def test_bad_options_are_refused(bad, capsys):
    with pytest.raises(SystemExit):
        main(["--model", "m", "--prompt-ids", "1", *bad])
    assert "tokens/top-k must be nonnegative" in capsys.readouterr().err


@pytest.mark.gpu
def test_cli_generates(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    p = subprocess.run([sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--random-config", str(cfg), "--seed", "4",
                        "--prompt-ids", "1,2,3", "--prompt-ids", "9,8,7,6,5", "--tokens", "6", "--greedy", "--dtype", "float32",
                        "--num-gpu-blocks", "16", "--ignore-eos"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(l) for l in p.stdout.strip().split("\n")]
    assert [l["prompt_ids"] for l in lines] == [[1, 2, 3], [9, 8, 7, 6, 5]]
    assert all(len(l["generated_ids"]) == 6 for l in lines)


def test_text_prompts_need_the_tokenizer(monkeypatch, capsys):
    """``--prompt`` is the reference's text option; without tiktoken's vocabulary it is refused with a message that names
    the way out.  With a tokenizer the text is encoded before anything else is looked at."""
    import types
    broken = types.ModuleType("tiktoken")

    def no_vocabulary(name):
        raise OSError("no vocabulary file")

    broken.get_encoding = no_vocabulary
    monkeypatch.setitem(sys.modules, "tiktoken", broken)
    with pytest.raises(SystemExit):
        main(["--model", "m", "--prompt", "Once upon a time"])
    err = capsys.readouterr().err
    assert "--prompt needs tiktoken's gpt2 vocabulary" in err and "--prompt-ids" in err

    seen = []
    working = types.ModuleType("tiktoken")
    working.get_encoding = lambda name: types.SimpleNamespace(encode_ordinary=lambda t: seen.append(t) or [1, 2, 3], decode=lambda ids: "")
    monkeypatch.setitem(sys.modules, "tiktoken", working)
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(SystemExit):
            main(["--model", "m", "--prompt", "Once upon a time"])
        assert seen == ["Once upon a time"] and "CUDA is unavailable" in capsys.readouterr().err


@pytest.mark.gpu
def test_ranges_around_the_operations_change_nothing(tmp_path):
    """``TTIE_NVTX=1`` wraps every operation of the kernel library in a profiler range of its name; the tokens are the same."""
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    cmd = [sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--random-config", str(cfg), "--seed", "4",
           "--prompt-ids", "1,2,3", "--tokens", "6", "--temperature", "0.9", "--top-k", "20", "--dtype", "float32", "--num-gpu-blocks", "16", "--ignore-eos"]
    outs = []
    for flag in ("0", "1"):
        p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=dict(os.environ, TTIE_NVTX=flag))
        assert p.returncode == 0, p.stderr[-2000:]
        outs.append(json.loads(p.stdout.strip())["generated_ids"])
    assert outs[0] == outs[1] and len(outs[0]) == 6
