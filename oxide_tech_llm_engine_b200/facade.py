"""Root façade: `Engine.builder()...build()`, the one-object entry point of the reference's root
crate (`OxideEngine::builder()`, src/lib.rs of the workspace root), mapped onto `EngineConfig`,
`LLMEngine` and `EngineHandle`."""
from __future__ import annotations

from typing import Optional

from .config import EngineConfig
from .sampling_params import SamplingParams


class EngineBuilder:
    def __init__(self):
        self._kw: dict = {}
        self._weights = None
        self._model_cfg = None
        self._random_init = False

    def model(self, path_or_preset: str) -> "EngineBuilder":
        self._kw["model"] = path_or_preset
        return self

    def backend(self, name: str) -> "EngineBuilder":
        if name not in ("cuda", "cpu"):
            raise ValueError(f"backend {name!r} is not available in this build (cuda | cpu)")
        self._kw["backend"] = name
        return self

    def context_size(self, n: int) -> "EngineBuilder":
        self._kw["ctx_size"] = int(n)
        return self

    def max_slots(self, n: int) -> "EngineBuilder":
        self._kw["max_num_seqs"] = int(n)
        return self

    def tensor_parallel(self, n: int) -> "EngineBuilder":
        self._kw["tp"] = int(n)
        return self

    def weights(self, mode: str) -> "EngineBuilder":
        self._kw["weight_mode"] = mode
        return self

    def speculative(self, mode: str, draft_tokens: int = 5) -> "EngineBuilder":
        self._kw.update(speculative=mode, draft_tokens=draft_tokens)
        return self

    def kv_tiers(self, host_blocks: int, storage_dir: Optional[str] = None, storage_blocks: int = 0,
                 quant: str = "none") -> "EngineBuilder":
        """Blocks the prefix cache evicts go to host memory (and files) and come back on a hit."""
        self._kw.update(kv_host_blocks=int(host_blocks), kv_storage_dir=storage_dir,
                        kv_storage_blocks=int(storage_blocks), kv_host_quant=quant)
        return self

    def decode_burst(self, steps: int, max_batch: int = 8) -> "EngineBuilder":
        """Small greedy batches decode `steps` tokens per host round trip (in-graph step advance)."""
        self._kw.update(decode_burst=int(steps), burst_max_batch=int(max_batch))
        return self

    def option(self, **kw) -> "EngineBuilder":
        self._kw.update(kw)
        return self

    def with_weights(self, source, model_cfg=None) -> "EngineBuilder":
        self._weights, self._model_cfg = source, model_cfg
        return self

    def random_init(self, model_cfg=None) -> "EngineBuilder":
        self._random_init, self._model_cfg = True, model_cfg
        return self

    def config(self) -> EngineConfig:
        return EngineConfig(**self._kw)

    def build(self, **dist_kw) -> "Engine":
        from .engine.engine import LLMEngine

        cfg = self.config()
        weights, mc = self._weights, self._model_cfg
        if weights is None and not self._random_init and (cfg.model.endswith(".gguf") or cfg.model.endswith(".safetensors")):
            from .models.weights import open_weights

            weights = open_weights(cfg.model)
        if weights is None and not self._random_init and mc is None:
            from .models.config import preset
            from .models.weights import SyntheticSource

            mc = preset(cfg.model)
            weights = SyntheticSource(mc, seed=cfg.seed)
        return Engine(LLMEngine(cfg, mc if mc is not None else (weights.cfg if weights is not None else None),
                                weights=weights, random_init=self._random_init, **dist_kw))


class Engine:
    """Thin wrapper: synchronous `generate`, or `serve()` to get the threaded handle the HTTP server uses."""

    def __init__(self, llm_engine):
        self.llm = llm_engine
        self._handle = None

    @staticmethod
    def builder() -> EngineBuilder:
        return EngineBuilder()

    def generate(self, prompts, params: Optional[SamplingParams] = None):
        return self.llm.generate(prompts, params)

    def serve(self):
        from .engine.handle import EngineHandle

        if self._handle is None:
            self._handle = EngineHandle(self.llm)
        return self._handle

    def close(self) -> None:
        if self._handle is not None:
            self._handle.shutdown() if hasattr(self._handle, "shutdown") else None
        self.llm.close()
