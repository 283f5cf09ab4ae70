"""One worker per GPU: device set-up, model load, KV sizing, step execution.

Parity: ``aphrodite/v1/worker/gpu_worker.py:128`` (``init_device`` :288,
``determine_available_memory`` :436, ``initialize_from_config`` :620,
``compile_or_warm_up_model`` :647, ``execute_model`` :939).
"""
from __future__ import annotations

import gc
import os

import torch

from sonar_b200.config import EngineConfig
from sonar_b200.core.kv_cache_manager import KVCacheConfig, KVCacheSpec, get_kv_cache_config
from sonar_b200.core.scheduler import ModelRunnerOutput, SchedulerOutput
from sonar_b200.logger import init_logger
from sonar_b200.parallel import state
from sonar_b200.worker.model_runner import ModelRunner

logger = init_logger(__name__)


class Worker:
    def __init__(self, cfg: EngineConfig, rank: int = 0, local_rank: int = 0, world_size: int = 1,
                 init_method: str | None = None) -> None:
        self.cfg = cfg
        self.rank, self.local_rank, self.world_size = rank, local_rank, world_size
        self.init_method = init_method
        self.device: torch.device | None = None
        self.runner: ModelRunner | None = None
        self._baseline_free = 0

    # ------------------------------------------------------------------
    def init_device(self) -> None:
        cfg = self.cfg
        if cfg.device == "cuda":
            self.device = torch.device("cuda", self.local_rank)
            torch.cuda.set_device(self.device)
            gc.collect()
            torch.cuda.empty_cache()
            self._baseline_free, _ = torch.cuda.mem_get_info()
        else:
            self.device = torch.device("cpu")
        p = cfg.parallel
        if self.world_size > 1 or os.environ.get("WORLD_SIZE"):
            state.init_distributed_environment(self.world_size, self.rank, self.local_rank, self.init_method,
                                               backend="nccl" if cfg.device == "cuda" else "gloo")
        if not state.model_parallel_is_initialized():
            import torch.distributed as dist
            if dist.is_initialized():
                dp_here = p.data_parallel_size if dist.get_world_size() == p.world_size_across_dp else 1
                state.initialize_model_parallel(p.tensor_parallel_size, p.pipeline_parallel_size, dp_here,
                                                p.prefill_context_parallel_size, p.decode_context_parallel_size)
        torch.manual_seed(cfg.model.seed)
        self._install_tp_context()
        self.runner = ModelRunner(cfg, self.device)

    def _install_tp_context(self) -> None:
        from sonar_b200 import envs
        from sonar_b200.parallel import tp_ops
        mode = envs.SONAR_TP_COMM
        ctx = None
        if (self.cfg.device == "cuda" and state.tp_world_size() > 1 and mode in ("fused", "custom")
                and not self.cfg.parallel.disable_custom_all_reduce):
            from sonar_b200.parallel import fused_tp
            ctx = fused_tp.make_context(self.cfg, self.device, mode)
        tp_ops.set_tp_context(ctx if ctx is not None else tp_ops.TPContext())

    def load_model(self) -> None:
        self.runner.load_model()

    def get_kv_cache_spec(self) -> tuple[KVCacheSpec, int]:
        return self.runner.kv_cache_spec(), self.runner.num_local_layers()

    def determine_available_memory(self) -> int:
        """Bytes this rank can give to the KV cache."""
        cfg = self.cfg
        if cfg.device != "cuda":
            return int(os.environ.get("SONAR_CPU_KVCACHE_BYTES", 1 << 30))
        torch.cuda.synchronize()
        free, total = torch.cuda.mem_get_info()
        budget = int(total * cfg.cache.gpu_memory_utilization)
        used_by_us = self._baseline_free - free
        reserve = self.runner.profile_activation_bytes()
        avail = budget - used_by_us - reserve - (total - self._baseline_free)
        logger.info("memory: total %.1f GiB, weights+state %.1f GiB, step reserve %.1f GiB → KV %.1f GiB",
                    total / 2**30, used_by_us / 2**30, reserve / 2**30, avail / 2**30)
        return max(avail, 0)

    def initialize_from_config(self, kv_cfg: KVCacheConfig) -> None:
        self.runner.initialize_kv_cache(kv_cfg)

    def compile_or_warm_up_model(self) -> None:
        warm = getattr(self.runner, "warm_up", None)
        if warm is not None:
            warm()

    def execute_model(self, so: SchedulerOutput) -> ModelRunnerOutput | None:
        return self.runner.execute_model(so)

    def get_stats(self) -> dict:
        return dict(self.runner.stats)

    def check_health(self) -> bool:
        return True

    def shutdown(self) -> None:
        self.runner = None
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def size_kv_cache(cfg: EngineConfig, specs: list[tuple[KVCacheSpec, int]], available: list[int]) -> KVCacheConfig:
    """One block count for all ranks: the smallest any of them can afford."""
    best = None
    for (spec, layers), avail in zip(specs, available):
        kc = get_kv_cache_config(spec, layers, avail, cfg.model.max_model_len, cfg.cache.num_gpu_blocks_override)
        if best is None or kc.num_blocks < best.num_blocks:
            best = kc
    assert best is not None
    return best
