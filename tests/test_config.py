"""YAML config: the reference's own files load, ours load, bad values are refused."""
import glob
import os

import pytest

from jittorinfer_b200.config import ServerConfig, load_yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shipped_configs_load():
    files = sorted(glob.glob(os.path.join(ROOT, "configs", "*.yaml")))
    assert len(files) == 6          # the four reference configs + EP with data-parallel attention + column-sharded experts
    for f in files:
        c = load_yaml(f)
        assert c.model.endswith(".gguf") and c.n_parallel >= 8
    assert load_yaml(os.path.join(ROOT, "configs", "config_deepseek_v2_ep.yaml")).world_size == 8
    tp = load_yaml(os.path.join(ROOT, "configs", "config_deepseek_v2_tp.yaml"))
    assert tp.world_size == 8 and tp.ep_size == 1 and tp.run_ahead


def test_reference_style_file_and_defaults(tmp_path):
    p = tmp_path / "ref.yaml"
    p.write_text("main_gpu: 1\nn_gpu_layers: 99\nsplit_mode: LLAMA_SPLIT_MODE_LAYER\ntensor_split: [0]\nuse_mmap: true\n"
                 "n_threads: 128\ndefrag_thold: 0.5\nenable_mla: false\nenable_fused_moe: true\noffload_input: true\n"
                 "enable_ge: true\npresample_count: -1\nenable_cann_flash_attention: true\nn_ctx: 65536\nn_batch: 16\n"
                 "n_parallel: 16\nmodel: \"/data/x-f16.gguf\"\nport: 8084\nn_threads_http: 16\nhostname: \"127.0.0.1\"\n"
                 "reasoning_format: COMMON_REASONING_FORMAT_DEEPSEEK\n")
    c = load_yaml(str(p))
    assert c.port == 8084 and c.n_ctx == 65536 and c.presample_count == -1 and c.cuda_graphs
    assert "n_threads" in c.ignored and "enable_cann_flash_attention" in c.ignored
    assert load_yaml(str(tmp_path / "missing.yaml")) == ServerConfig()


def test_bad_values_rejected(tmp_path):
    for body in ("tp_size: 3\n", "split_mode: SIDEWAYS\n", "kv_block_size: 32\n", "tp_size: 4\nep_size: 2\n"):
        p = tmp_path / "bad.yaml"
        p.write_text(body)
        with pytest.raises(ValueError):
            load_yaml(str(p))


def test_kv_cache_sizing_from_memory_budget():
    from jittorinfer_b200.runtime.factory import kv_tokens_for_budget
    GB = 1 << 30
    # DeepSeek-V2 on a 180 GB device with 60 GB of weights resident: 90 % occupancy leaves room for ~1.4 M tokens
    n = kv_tokens_for_budget(180 * GB, 120 * GB, 0.9, n_layer=60, kv_row=576, elem_bytes=2)
    assert n % 64 == 0 and 1_400_000 < n < 1_600_000
    assert (180 * 0.9 - 60 - 2) * GB - n * 60 * 576 * 2 < 64 * 60 * 576 * 2 + GB        # fills the budget to within a block
    assert kv_tokens_for_budget(180 * GB, 10 * GB, 0.9, 60, 576, 2) == 0                # weights already exceed the budget
    cfg = ServerConfig(kv_cache_auto=True, max_seq_len=4352, gpu_memory_utilization=0.9)
    cfg.validate()


def test_automatic_layer_split_by_weight_size():
    """split_mode LAYER with layer_split_gpus = 0 (default): as many GPUs as the weights need, one when they fit."""
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.server.launch import auto_layer_split
    gib = 1 << 30
    free8 = [178 * gib] * 8
    assert auto_layer_split(preset("lite").n_params() * 2, free8) == 1          # 31 GB
    n_v2 = auto_layer_split(preset("v2").n_params() * 2, free8)                  # ~470 GB of bf16 weights
    assert 3 <= n_v2 <= 4
    assert auto_layer_split(10 ** 15, free8) == 8 and auto_layer_split(1, []) == 1
    assert ServerConfig().layer_split_gpus == 0


def test_reference_yaml_under_n_ranks_means_tp_plus_ep():
    from jittorinfer_b200.server.launch import apply_world
    cfg = ServerConfig()
    apply_world(cfg, 1)
    assert (cfg.tp_size, cfg.ep_size) == (1, 1)
    apply_world(cfg, 8)
    assert (cfg.tp_size, cfg.ep_size) == (8, 8)
    dp = ServerConfig(ep_size=4, attention_dp=True)
    apply_world(dp, 4)
    assert (dp.tp_size, dp.ep_size) == (1, 4)
    with pytest.raises(SystemExit):
        apply_world(ServerConfig(tp_size=2), 4)
