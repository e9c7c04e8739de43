"""Configuration, registry and weight loading (no GPU)."""
import json
import os

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from tiny_transformer_inference_engine_b200.config import ModelConfig, ConfigError, EngineConfig, CacheConfig, SchedulerConfig
from tiny_transformer_inference_engine_b200.models.model import Model
from tiny_transformer_inference_engine_b200.registry import model_spec, RegistryError, build_part, known_models
from tiny_transformer_inference_engine_b200.parts.base import PartSpec
from tiny_transformer_inference_engine_b200.weights import (WeightError, write_random_model, load_folder,
                                                            read_safetensors, random_tensors)


def test_config_roundtrip(tmp_path):
    c = ModelConfig.from_dict(TINY_B)
    assert c.head_dim == 32 and c.hidden_size == 256 and c.bias and c.rope_theta == 500000.0
    c.save(str(tmp_path))
    assert ModelConfig.from_json(str(tmp_path)) == c
    # the reference's own keys alone are enough: no architecture key, hidden_size defaults to d_model
    raw = dict(vocab_size=50, d_model=32, num_layers=1, num_heads=2, max_seq_len=16, causal=True, dropout=0.0,
               dtype="torch.float32", some_training_key=3)
    c2 = ModelConfig.from_dict(raw)
    assert c2.architecture == "mqa_gpt" and c2.hidden_size == 32 and c2.num_kv_heads == 1
    assert c2.extra == {"some_training_key": 3} and c2.dtype == "float32"


@pytest.mark.parametrize("change,word", [
    ({"d_model": 65}, "multiple of num_heads"), ({"num_kv_heads": 3}, "multiple of num_kv_heads"),
    ({"causal": False}, "causal"), ({"vocab_size": 0}, "positive"), ({"dtype": "int8"}, "dtype"),
    ({"rope_theta": -1.0}, "rope_theta")])
def test_config_refuses(change, word):
    with pytest.raises(ConfigError, match=word):
        ModelConfig.from_dict({**TINY_A, **change})


def test_config_missing_sizes():
    raw = dict(TINY_A)
    del raw["vocab_size"], raw["num_layers"]
    with pytest.raises(ConfigError, match=r"vocab_size.*num_layers"):
        ModelConfig.from_dict(raw)


def test_registry_unknown_names():
    with pytest.raises(RegistryError, match="unknown architecture 'gpt9'.*mqa_gpt"):
        model_spec(ModelConfig.from_dict({**TINY_A, "architecture": "gpt9"}))
    with pytest.raises(RegistryError, match="unknown mixer"):
        build_part("mixer", PartSpec("no_such_mixer"))
    assert "mqa_gpt" in known_models()


def test_tensor_names_are_the_references():
    m = Model(model_spec(ModelConfig.from_dict(TINY_B)))
    names = set(m.param_specs())
    assert "embedding.embedding.weight" in names and "lm_head.weight" in names and "final_norm.weight" in names
    for i in range(3):
        for n in ("attn_norm.weight", "attn.q_proj.weight", "attn.k_proj.bias", "attn.v_proj.weight", "attn.out.bias",
                  "mlp_norm.weight", "mlp.gate_proj.weight", "mlp.up_proj.bias", "mlp.down_proj.weight"):
            assert f"layers.{i}.{n}" in names
    assert len(names) == 3 + 3 * (2 + 8 + 6)
    assert m.param_specs()["layers.1.mlp.gate_proj.weight"][2].shape == (256, 96)
    no_bias = set(Model(model_spec(ModelConfig.from_dict(TINY_A))).param_specs())
    assert not any(n.endswith(".bias") for n in no_bias)


def test_random_model_folder_is_reproducible(tmp_path):
    c = ModelConfig.from_dict(TINY_A)
    a = write_random_model(c, 7, str(tmp_path / "a"))
    b = write_random_model(c, 7, str(tmp_path / "b"))
    d = write_random_model(c, 8, str(tmp_path / "d"))
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    ta, tb, td = read_safetensors(a), read_safetensors(b), read_safetensors(d)
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], td["lm_head.weight"])
    assert abs(ta["lm_head.weight"].std().item() - 0.02) < 2e-3
    assert torch.equal(ta["final_norm.weight"], torch.ones(64))


def test_storage_rules(tmp_path):
    c = ModelConfig.from_dict(TINY_A)
    folder = write_random_model(c, 1, str(tmp_path / "m"), store_dtype="bfloat16", perturb_norms=True)
    stored = read_safetensors(folder)
    assert stored["lm_head.weight"].dtype == torch.bfloat16 and stored["final_norm.weight"].dtype == torch.float32
    specs = Model(model_spec(c)).param_specs()
    bf = load_folder(folder, specs, torch.bfloat16, "cpu")
    assert bf["lm_head.weight"].dtype == torch.bfloat16
    assert bf["final_norm.weight"].dtype == torch.float32          # stored in 32-bit stays so
    f32 = load_folder(folder, specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["lm_head.weight"], stored["lm_head.weight"].float())


def test_one_error_lists_everything(tmp_path):
    from safetensors.torch import save_file
    c = ModelConfig.from_dict(TINY_A)
    t = random_tensors(c, 3)
    del t["layers.1.mlp.up_proj.weight"], t["final_norm.weight"]
    t["layers.0.attn.q_proj.weight"] = torch.zeros(64, 63)
    t["_orig_mod.extra.thing"] = torch.zeros(2)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    folder = tmp_path / "bad"
    folder.mkdir()
    c.save(str(folder))
    save_file(t, str(folder / "model.safetensors"))
    specs = Model(model_spec(c)).param_specs()
    with pytest.raises(WeightError) as ei:
        load_folder(str(folder), specs, torch.float32, "cpu")
    e = ei.value
    assert [n for n, _ in e.missing] == ["final_norm.weight", "layers.1.mlp.up_proj.weight"]
    assert [n for n, _ in e.unexpected] == ["extra.thing"]                      # _orig_mod. is stripped
    assert e.wrong_shape == [("layers.0.attn.q_proj.weight", (64, 63), (64, 64))]
    assert [n for n, _, _ in e.wrong_dtype] == ["lm_head.weight"]
    msg = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [64, 64]", "wrong dtype (1)"):
        assert word in msg


def test_orig_mod_prefix_is_stripped(tmp_path):
    from safetensors.torch import save_file
    c = ModelConfig.from_dict(TINY_A)
    t = {"_orig_mod." + k: v for k, v in random_tensors(c, 3).items()}
    folder = tmp_path / "m"
    folder.mkdir()
    save_file(t, str(folder / "model.safetensors"))
    loaded = load_folder(str(folder), Model(model_spec(c)).param_specs(), torch.float32, "cpu")
    assert "lm_head.weight" in loaded


def test_engine_config_checks():
    with pytest.raises(ValueError):
        SchedulerConfig(max_num_seqs=64, max_num_batched_tokens=32)
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        CacheConfig(num_gpu_blocks=1)
    with pytest.raises(ValueError):
        CacheConfig(enable_prefix_caching=True)


def test_missing_extension_fails_loudly():
    from tiny_transformer_inference_engine_b200.ops import get_ops, KernelError
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(KernelError, match="no CPU path"):
        get_ops("cuda:0")


def test_reference_checkpoint_is_converted_to_a_model_folder(tmp_path):
    """A file saved the way the reference saves its checkpoints (inference.py:16-29,87: ``model_config``, ``model`` with
    the compiled-model prefix on some keys) becomes config.json + model.safetensors; the engine loads the folder and its
    logits are the plain model's for the same tensors.  The feed-forward width comes from the tensors, the rotary base and
    the norms' eps are the values the reference fixes in code."""
    from plain_model import plain_forward
    from plain_ops import PlainOps
    from tiny_configs import TINY_B, SEEDS
    from tiny_transformer_inference_engine_b200 import Engine, EngineConfig, CacheConfig, SchedulerConfig
    from tiny_transformer_inference_engine_b200.weights import convert_checkpoint, CheckpointError
    from tiny_transformer_inference_engine_b200.weights.convert import main as convert_main
    cfg = dict(TINY_B, rope_theta=10000.0, rms_norm_eps=1e-5)
    w = random_tensors(ModelConfig.from_dict(cfg), SEEDS["B"], perturb_norms=True)
    saved_cfg = {k: cfg[k] for k in ("vocab_size", "d_model", "num_layers", "num_heads", "num_kv_heads", "max_seq_len", "bias")}
    saved_cfg.update(causal=True, dropout=0.0, eos_token_id=7, rope_theta=123.0, rms_norm_eps=0.5)   # declared, never used by its layers
    state = {("_orig_mod." + k if i % 2 else k): v for i, (k, v) in enumerate(w.items())}
    path = str(tmp_path / "ckpt_step1.pt")
    torch.save({"model_config": saved_cfg, "model": state, "train_config": {"attn_type": "mqa"}, "step": 1}, path)
    folder = str(tmp_path / "model")
    assert convert_main([path, folder]) == 0
    mc = ModelConfig.from_json(folder)
    assert (mc.hidden_size, mc.rope_theta, mc.rms_norm_eps, mc.eos_token_id, mc.architecture) == (cfg["hidden_size"], 10000.0, 1e-5, 7, "mqa_gpt")
    ec = EngineConfig(dtype="float32", device="cpu", use_cuda_graphs=False, cache=CacheConfig(block_size=8, num_gpu_blocks=20),
                      sched=SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64))
    eng = Engine.from_folder(folder, ec, ops=PlainOps())
    from tiny_transformer_inference_engine_b200 import StepEntry
    toks = [5, 900, 17, 3, 250, 1, 77]
    eng.manager.admit("a")
    eng.manager.extend("a", 0, len(toks))
    got = eng.stepper.step([StepEntry("a", 0, toks, list(range(len(toks))))])
    want = plain_forward(cfg, w, toks)
    assert (got.cpu() - want).abs().max() < 1e-5 * want.abs().max()
    # the file itself is accepted where a folder is
    eng2 = Engine.from_checkpoint(path, ec, ops=PlainOps())
    eng2.manager.admit("a")
    eng2.manager.extend("a", 0, len(toks))
    assert torch.equal(eng2.stepper.step([StepEntry("a", 0, toks, list(range(len(toks))))]), got)
    # what cannot be converted says why
    torch.save({"model": state}, path)
    with pytest.raises(CheckpointError, match="missing model_config"):
        convert_checkpoint(path, folder)
    torch.save({"model_config": saved_cfg, "model": state, "quant_metadata": {"lm_head.weight": {}}}, path)
    with pytest.raises(CheckpointError, match="quantized"):
        convert_checkpoint(path, folder)
    torch.save({"model_config": saved_cfg, "model": {k: v for k, v in state.items() if "gate_proj" not in k}}, path)
    with pytest.raises(CheckpointError, match="gate_proj"):
        convert_checkpoint(path, folder)
    assert convert_main([str(tmp_path / "nothing.pt"), folder]) == 1
