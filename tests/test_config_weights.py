"""Configuration, registry and weight loading: what is read, what is refused, what errors say."""
import json
import os

import pytest
import torch

import tiny_configs
from helpers import read_tensors, write_model


def test_qwen2_config_reads_every_key():
    from velox_b200.config import Qwen2Config

    c = Qwen2Config.from_dict(tiny_configs.TINY_W)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (240, 4, 5, 5)
    assert c.head_dim == 48 and c.intermediate_size == 200 and c.vocab_size == 331
    assert c.rms_norm_eps == 3e-6 and c.rope_theta == 50000.0 and c.rope_scaling_factor == 2.0
    assert c.sliding_window == 24 and c.max_window_layers == 1
    assert [c.layer_window(i) for i in range(4)] == [None, 24, 24, 24]
    assert not c.tie_word_embeddings
    assert Qwen2Config.from_dict(c.to_json_dict()) == c


def test_qwen2_config_defaults_follow_the_reference():
    from velox_b200.config import Qwen2Config

    c = Qwen2Config.from_dict({"architectures": ["Qwen2ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 1,
                               "num_attention_heads": 4, "intermediate_size": 8, "vocab_size": 10})
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    assert c.tie_word_embeddings is False and c.sliding_window is None


@pytest.mark.parametrize("patch,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66, "head_dim": None}, "divisible"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"vocab_size": -1}, "vocab_size"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
])
def test_config_errors_name_the_key(patch, needle):
    from velox_b200.config import ConfigError, Qwen2Config

    cfg = dict(tiny_configs.TINY_A)
    cfg.update(patch)
    with pytest.raises(ConfigError, match=needle):
        Qwen2Config.from_dict(cfg)


def test_registry_picks_the_model_by_architecture(tmp_path):
    from velox_b200.config import ConfigError, architecture_of, load_model_config, supported_architectures

    write_model(str(tmp_path), tiny_configs.TINY_B, seed=1)
    config = load_model_config(str(tmp_path))
    assert config.architecture == "Qwen2ForCausalLM" and config.num_key_value_heads == 1
    assert "Qwen2ForCausalLM" in supported_architectures()
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({})


def test_named_model_sizes_are_configurations_of_the_architecture():
    """Every --model-size name parses as this architecture; 1.5b has the sizes the benchmark names."""
    from velox_b200.config import Qwen2Config, architecture_of
    from velox_b200.config.presets import MODEL_SIZES, model_size

    for name in MODEL_SIZES:
        cfg = model_size(name)
        assert architecture_of(cfg).name == "Qwen2ForCausalLM"
        c = Qwen2Config.from_dict(cfg)
        assert c.num_attention_heads % c.num_key_value_heads == 0
    c = Qwen2Config.from_dict(model_size("1.5b"))
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.tie_word_embeddings) == (28, 1536, 12, 2, 128, 8960, 151936, True)
    cfg = model_size("7b")
    cfg["hidden_size"] = 1  # a copy: the table is not touched
    assert model_size("7b")["hidden_size"] == 3584
    with pytest.raises(KeyError, match="known"):
        model_size("70b")


def test_benchmark_command_line_options():
    from velox_b200.cli.benchmark import build_prompts, parse_args

    args = parse_args(["--model-size", "tiny-a", "--prompt-len", "9", "--decode-len", "5", "--batch", "1,4"])
    assert args.max_tokens == 5 and args.prompt_len == 9 and args.batch == "1,4" and args.model is None
    prompts = build_prompts("mixed", 3, 50, 100, seed=0, fixed_len=args.prompt_len)
    assert [len(p) for p in prompts] == [9, 9, 9] and all(0 <= t < 50 for p in prompts for t in p)
    with pytest.raises(SystemExit):
        parse_args(["--model", "x", "--model-size", "tiny-a"])
    with pytest.raises(SystemExit):
        parse_args([])


def test_spec_names_every_checkpoint_tensor():
    from velox_b200.config import get_architecture

    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(arch.parse_config(tiny_configs.TINY_B))
    names = spec.checkpoint_tensors()
    assert names["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    assert names["model.layers.0.mlp.gate_proj.weight"].shape == (704, 256)
    assert names["lm_head.weight"].shape == (512, 256)
    assert len(names) == 3 * 12 + 3
    tied = arch.build_spec(arch.parse_config(tiny_configs.TINY_A))
    assert "lm_head.weight" not in tied.checkpoint_tensors()
    assert tied.lm_head.weights["weight"].sources[0].name == "model.embed_tokens.weight"
    # the fused weights keep the order q, k, v and gate, up
    qkv = spec.layers[1].mixer.weights["qkv.weight"]
    assert [s.name.split(".")[-2] for s in qkv.sources] == ["q_proj", "k_proj", "v_proj"]
    assert qkv.shape == ((8 + 2) * 32, 256)
    gate_up = spec.layers[1].feed_forward.weights["gate_up.weight"]
    assert [s.name.split(".")[-2] for s in gate_up.sources] == ["gate_proj", "up_proj"]


def test_random_weights_are_seeded_per_tensor(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_model(a, tiny_configs.TINY_A, seed=1)
    write_model(b, tiny_configs.TINY_A, seed=1)
    write_model(c, tiny_configs.TINY_A, seed=2)
    ta, tb, tc = read_tensors(a), read_tensors(b), read_tensors(c)
    assert set(ta) == set(tb)
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["model.norm.weight"], tc["model.norm.weight"])
    assert abs(ta["model.norm.weight"].mean().item() - 1.0) < 0.02
    assert abs(ta["model.embed_tokens.weight"].std().item() - 0.02) < 0.002
    with open(os.path.join(a, "config.json")) as handle:
        assert json.load(handle)["architectures"] == ["Qwen2ForCausalLM"]
    # a deeper model shares the tensors of its first layers: the seed is per name
    deeper = dict(tiny_configs.TINY_A, num_hidden_layers=3)
    d = str(tmp_path / "d")
    write_model(d, deeper, seed=1)
    td = read_tensors(d)
    assert torch.equal(td["model.layers.1.mlp.up_proj.weight"], ta["model.layers.1.mlp.up_proj.weight"])


def test_loader_lists_missing_unexpected_and_misshapen(tmp_path):
    from safetensors.torch import save_file

    from velox_b200.config import get_architecture
    from velox_b200.weights import Checkpoint, WeightError, check_checkpoint

    folder = str(tmp_path)
    write_model(folder, tiny_configs.TINY_B, seed=1)
    tensors = read_tensors(folder)
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(7, 3)
    tensors["model.layers.9.extra"] = torch.zeros(1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(arch.parse_config(tiny_configs.TINY_B))
    with pytest.raises(WeightError) as info:
        check_checkpoint(Checkpoint(folder), spec)
    err = info.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra"]
    assert err.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (7, 3), (256, 704))]
    text = str(err)
    for needle in ("missing", "unexpected", "model.layers.9.extra", "(7, 3)", "(256, 704)"):
        assert needle in text


def test_loader_storage_dtypes_and_tied_head(tmp_path):
    from velox_b200.config import get_architecture
    from velox_b200.weights import Checkpoint, WeightStore

    folder = str(tmp_path)
    write_model(folder, tiny_configs.TINY_A, seed=1, dtype="bfloat16")
    arch = get_architecture("Qwen2ForCausalLM")
    spec = arch.build_spec(arch.parse_config(tiny_configs.TINY_A))
    raw = read_tensors(folder)
    for dtype in (torch.bfloat16, torch.float32):
        store = WeightStore(Checkpoint(folder), spec, dtype, "cpu")
        embed = store.load(spec.embedding.weights["weight"])
        head = store.load(spec.lm_head.weights["weight"])
        assert embed.dtype == dtype and head.data_ptr() == embed.data_ptr()
        norm = store.load(spec.final_norm.weights["weight"])
        assert norm.dtype == torch.float32
        assert torch.equal(norm, raw["model.norm.weight"].float())
        qkv = store.load(spec.layers[0].mixer.weights["qkv.weight"])
        want = torch.cat([raw[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"]).to(dtype)
        assert torch.equal(qkv, want)
        bias = store.load(spec.layers[0].mixer.weights["qkv.bias"])
        assert bias.dtype == torch.float32 and bias.shape == (4 * 16 + 2 * 2 * 16,)


def test_missing_folder_and_missing_files(tmp_path):
    from velox_b200.config import load_model_config
    from velox_b200.weights import Checkpoint

    with pytest.raises(FileNotFoundError):
        load_model_config(str(tmp_path / "nope"))
    os.makedirs(tmp_path / "empty")
    with pytest.raises(FileNotFoundError):
        Checkpoint(str(tmp_path / "empty"))


def test_engine_config_validation():
    from velox_b200.config import EngineConfig, resolve_dtype

    EngineConfig(model="x").validate()
    for bad in (dict(max_num_seqs=0), dict(max_num_batched_tokens=100, max_prefill_chunk_size=200),
                dict(max_num_batched_tokens=16, max_prefill_chunk_size=8, max_num_seqs=32),
                dict(gpu_memory_utilization=0.0), dict(block_size=12), dict(num_gpu_blocks=1), dict(dtype="int8")):
        with pytest.raises(ValueError):
            EngineConfig(model="x", **bad).validate()
    assert resolve_dtype("auto") is torch.bfloat16 and resolve_dtype("fp32") is torch.float32


def test_no_cuda_means_a_loud_error():
    from velox_b200.ops import kernels

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(kernels.KernelError, match="CUDA"):
        kernels._require_cuda()
