"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits on disk."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from plain_model import plain_forward
from tiny_configs import TINY_B, SEEDS
import trace_util as tu
from gpu_util import requests_for, TOL

from tiny_transformer_inference_engine_b200 import ModelConfig, write_random_model
from tiny_transformer_inference_engine_b200.weights import read_safetensors

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = TINY_B
    folder = write_random_model(ModelConfig.from_dict(cfg), SEEDS["B"], str(tmp_path / "model"), perturb_norms=True)
    w = read_safetensors(folder)
    reqs = requests_for(cfg, (40, 71, 128, 9, 100), 21)
    steps = tu.mixed(reqs, seed=3)
    lines = [json.dumps({"step": i, **st}) for i, st in enumerate(steps)]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(tu.max_live_tokens(steps))],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    exp = {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    fed, V, worst = {}, cfg["vocab_size"], 0.0
    for i, st in enumerate(steps):
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{i}.f32"
        assert path.exists() == (wanted > 0)
        arr = np.fromfile(path, dtype="<f4").reshape(wanted, V)
        k = 0
        for e in st["entries"]:
            start = fed.get(e["id"], 0)
            for wpos in e["want"]:
                ref = exp[e["id"]][start + wpos]
                worst = max(worst, float((torch.from_numpy(arr[k]).double() - ref.double()).abs().max() / ref.abs().max()))
                k += 1
            fed[e["id"]] = start + len(e["tokens"])
    assert worst < TOL[dtype], worst
