import json
import os

import pytest
import torch

from tiny_models import CONFIGS, TINY_A, TINY_B, make_weights, write_model_dir, write_safetensors


def test_typed_config_reads_its_keys(tmp_path):
    from mini_sglang_b200.config import load_config
    d = write_model_dir(str(tmp_path / "m"), TINY_B, make_weights(TINY_B, 1))
    cfg, spec = load_config(d)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (96, 3, 6, 2)
    assert cfg.head_dim == 32 and cfg.intermediate_size == 160 and cfg.vocab_size == 320
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and not cfg.tie_word_embeddings
    assert spec.architecture == "Qwen3ForCausalLM" and len(spec.layers) == 3
    m = spec.layers[0].mixer
    assert m.kind == "paged_attention" and m["num_heads"] == 6 and m["head_dim"] == 32 and m["qk_norm"]
    assert abs(m["scale"] - 32 ** -0.5) < 1e-12
    assert spec.layers[1].position["theta"] == 1e6
    assert [r.layer for r in spec.schedule] == [0, 1, 2] and [r.cache for r in spec.schedule] == [0, 1, 2]
    assert spec.eos_token_ids == [7]


def test_config_defaults_and_errors():
    from mini_sglang_b200.config import ConfigError, Qwen3Config, architecture_of
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert Qwen3Config.from_dict(raw).head_dim == 16
    raw = dict(TINY_A)
    del raw["rope_theta"]
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(raw).rope_theta == 12345.0
    for key, val, msg in [("num_key_value_heads", 3, "multiple"), ("hidden_act", "gelu", "silu"),
                          ("use_sliding_window", True, "sliding"), ("rope_scaling", {"rope_type": "yarn", "factor": 4}, "rope")]:
        bad = dict(TINY_A)
        bad[key] = val
        with pytest.raises(ConfigError, match=msg):
            Qwen3Config.from_dict(bad)
    with pytest.raises(ConfigError, match="missing key 'vocab_size'"):
        Qwen3Config.from_dict({k: v for k, v in TINY_A.items() if k != "vocab_size"})
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Qwen3ForCausalLM"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})


def test_registry_takes_a_new_architecture():
    from mini_sglang_b200.config import ARCHITECTURES, Qwen3Config, architecture_of, register_architecture
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec

    def twice(cfg):
        spec = build_qwen3_spec(cfg)
        spec.architecture = "ToyTwice"
        return spec

    register_architecture("ToyTwice", Qwen3Config, twice)
    try:
        assert architecture_of({"architectures": ["ToyTwice"]}).build_spec is twice
    finally:
        del ARCHITECTURES["ToyTwice"]


def test_expected_tensors_and_packing_names():
    from mini_sglang_b200.config import Qwen3Config
    from mini_sglang_b200.config.qwen3 import build_qwen3_spec
    from mini_sglang_b200.parts import expected_tensors
    from tiny_models import tensor_shapes
    for name, cfg in CONFIGS.items():
        exp = expected_tensors(build_qwen3_spec(Qwen3Config.from_dict(cfg)))
        want = tensor_shapes(cfg)
        got = {n: tuple(d.shape) for n, d in exp.items() if not d.optional}
        assert got == want, name
    tied = expected_tensors(build_qwen3_spec(Qwen3Config.from_dict(TINY_A)))
    assert tied["lm_head.weight"].optional


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from mini_sglang_b200.config import load_config
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import CheckpointSource, WeightsError
    w = make_weights(TINY_B, 1)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    w["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(31, dtype=torch.bfloat16)
    w["lm_head.weight"] = torch.zeros(320, 95, dtype=torch.bfloat16)
    d = write_model_dir(str(tmp_path / "bad"), TINY_B, w)
    _, spec = load_config(d)
    with pytest.raises(WeightsError) as ei:
        CheckpointSource(d, expected_tensors(spec), torch.bfloat16, "cpu")
    msg = str(ei.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected (1): model.layers.7.extra.weight" in msg
    assert "wrong shape (2)" in msg and "lm_head.weight is [320, 95], expected [320, 96]" in msg
    assert "model.layers.0.self_attn.k_norm.weight is [31], expected [32]" in msg


def test_kept_precision(tmp_path):
    from mini_sglang_b200.config import load_config
    from mini_sglang_b200.parts import expected_tensors
    from mini_sglang_b200.weights import CheckpointSource
    w = make_weights(TINY_A, 0)
    w["model.norm.weight"] = w["model.norm.weight"].float() + 1e-4          # stored in 32-bit: stays so
    w["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)         # tied model with a stray head: ignored
    d = write_model_dir(str(tmp_path / "m"), TINY_A, w)
    _, spec = load_config(d)
    exp = expected_tensors(spec)
    src = CheckpointSource(d, exp, torch.bfloat16, "cpu")
    assert src.fetch("model.norm.weight").dtype == torch.float32
    assert torch.equal(src.fetch("model.norm.weight"), w["model.norm.weight"])
    assert src.fetch("model.embed_tokens.weight").dtype == torch.bfloat16
    assert torch.equal(src.fetch("model.layers.0.mlp.down_proj.weight"), w["model.layers.0.mlp.down_proj.weight"])
    src32 = CheckpointSource(d, exp, torch.float32, "cpu")
    t = src32.fetch("model.embed_tokens.weight")
    assert t.dtype == torch.float32 and torch.equal(t, w["model.embed_tokens.weight"].float())


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    from mini_sglang_b200.config import load_config
    from mini_sglang_b200.weights import open_model_dir, write_random_model
    d1 = write_random_model(str(tmp_path / "r1"), TINY_B, seed=3)
    d2 = write_random_model(str(tmp_path / "r2"), TINY_B, seed=3)
    d3 = write_random_model(str(tmp_path / "r3"), TINY_B, seed=4)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    cfg, _ = load_config(d1)
    assert cfg.hidden_size == 96
    f1, i1 = open_model_dir(d1)
    f2, i2 = open_model_dir(d2)
    f3, i3 = open_model_dir(d3)
    assert set(i1) == set(i2)
    for n in i1:
        a, b, c = i1[n].file.read(n), i2[n].file.read(n), i3[n].file.read(n)
        assert a.dtype == torch.bfloat16 and torch.equal(a, b)
        assert not torch.equal(a, c)
    e = i1["model.embed_tokens.weight"].file.read("model.embed_tokens.weight").float()
    assert abs(e.std().item() - 0.02) < 2e-3
    nrm = i1["model.norm.weight"].file.read("model.norm.weight").float()
    assert abs(nrm.mean().item() - 1.0) < 0.05
    # what our writer wrote, the safetensors package reads the same way
    from safetensors import safe_open
    with safe_open(os.path.join(d1, "model.safetensors"), "pt", "cpu") as f:
        assert torch.equal(f.get_tensor("model.norm.weight"), i1["model.norm.weight"].file.read("model.norm.weight"))


def test_safetensors_reader_rejects_garbage(tmp_path):
    from mini_sglang_b200.weights import SafetensorsError, SafetensorsFile
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!!")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes(b"\x00\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))


def test_engine_options_keep_the_references_names_and_defaults(tmp_path):
    """Every option of the reference's command line that concerns one GPU without a server (mini_sglang/managers/
    server_args.py:62-183) parses here under the same name, and the defaults it has there are the defaults here, page_size
    apart (1 there, 16 here; 1 is accepted).  What the engine cannot do is refused in words."""
    import argparse

    from mini_sglang_b200.engine.args import EngineArgs, ServerArgs
    ap = argparse.ArgumentParser()
    EngineArgs.add_cli_args(ap)
    d = str(tmp_path)
    ns = ap.parse_args(["--model", d, "--page_size", "1", "--attention_backend", "fa3", "--tp_size", "1", "--device", "cuda",
                        "--gpu_memory_utilization", "0.8", "--max_num_reqs", "64", "--schedule_policy", "fcfs", "--log_level", "WARNING",
                        "--random_seed", "7", "--profile", "--disable_radix_cache", "--disable_cuda_graph", "--max_capture_bs", "32",
                        "--schedule-conservativeness", "0.5", "--max_prefill_tokens", "4096", "--dummy_load"])
    a = EngineArgs.from_cli_args(ns)
    assert (a.page_size, a.max_num_reqs, a.schedule_policy, a.random_seed, a.max_capture_bs) == (1, 64, "fcfs", 7, 32)
    assert a.profile and a.disable_radix_cache and a.disable_cuda_graph and a.dummy_load
    assert (a.gpu_memory_utilization, a.schedule_conservativeness, a.max_prefill_tokens) == (0.8, 0.5, 4096)
    b = EngineArgs.from_cli_args(ap.parse_args(["--model", d]))
    assert (b.max_num_reqs, b.max_capture_bs, b.schedule_policy, b.tp_size, b.device) == (1024, 128, "lpm", 1, "cuda")
    assert (b.gpu_memory_utilization, b.log_level, b.schedule_conservativeness, b.max_prefill_tokens) == (0.9, "INFO", 1.0, 16384)
    assert not (b.profile or b.disable_radix_cache or b.disable_cuda_graph or b.dummy_load) and isinstance(b.random_seed, int)
    assert ServerArgs is EngineArgs
    for bad, words in [(dict(tp_size=2), "one GPU"), (dict(device="cpu"), "CUDA"), (dict(schedule_policy="lifo"), "policy"),
                       (dict(schedule_policy="lpm", disable_radix_cache=True), "radix"), (dict(dtype="float16"), "dtype"),
                       (dict(page_size=0), "page_size")]:
        with pytest.raises(ValueError, match=words):
            EngineArgs(model=d, **bad)
    with pytest.raises(ValueError, match="not a folder"):
        EngineArgs(model=str(tmp_path / "nothing here"))
