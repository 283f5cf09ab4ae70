import torch

from sonar_b200.config import ModelConfig
from sonar_b200.loader.weights import load_model
from sonar_b200.utils.metrics import EngineMetrics
from sonar_b200.utils.perf_model import ModelCost


def _count(model, skip=("embed_tokens",)):
    return sum(p.numel() for n, p in model.named_parameters() if p.dim() >= 2 and not any(s in n for s in skip))


def test_cost_model_counts_the_real_parameters():
    for preset in ("tiny-llama", "tiny-qwen3-moe", "tiny-deepseek"):
        cfg = ModelConfig(model=preset, dtype=torch.float32, load_format="dummy", skip_tokenizer_init=True)
        model = load_model(cfg, "cpu")
        cost = ModelCost.from_config(cfg)
        total = cost.layer_params_total * cost.num_layers + cost.head_params
        real = _count(model)
        assert abs(total - real) / real < 0.06, (preset, total, real)      # small extras: indexer, first dense layers
        assert cost.layer_params_active <= cost.layer_params_total
    cfg = ModelConfig(model="llama-3-8b", load_format="dummy", skip_tokenizer_init=True)
    cost = ModelCost.from_config(cfg)
    assert 6.9e9 < cost.layer_params_total * 32 < 7.1e9                   # 8.03 B minus embeddings and LM head
    flops, nbytes = cost.step(new_tokens=256, sampled_rows=256, context_tokens=256 * 1152)
    assert 3.5e12 < flops < 4.6e12 and 1.5e10 < nbytes < 6e10


def test_mfu_gauge_and_flops_counter():
    from sonar_b200.request import SchedulerStats
    cfg = ModelConfig(model="tiny-llama", dtype=torch.float32, load_format="dummy", skip_tokenizer_init=True)
    m = EngineMetrics("tiny", ModelCost.from_config(cfg))
    for _ in range(3):
        m.update_from_scheduler(SchedulerStats(num_running=2, step_generation_tokens=2))
    text = m.render()
    assert "sonar:model_flops_total" in text and "sonar:model_flops_utilization" in text
    assert m.counters["model_flops_total"] > 0
