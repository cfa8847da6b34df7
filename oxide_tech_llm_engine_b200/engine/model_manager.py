"""Named models behind one server: load by name / alias / path, list, unload, default.

Resolution order of a model string: exact path -> <models_dir>/<name>[.gguf] -> ./models/<name>[.gguf]
-> current directory -> catalog preset (random-init weights of that shape, for tests and benches).
Reference parity: DynamicModelManager (oxide-engine/src/model_manager.rs:10-136) and the
`POST /v1/models/load` hot-swap of the server.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Callable, Optional

from ..errors import ModelLoadError
from ..models.config import PRESETS


@dataclass
class LoadedModel:
    name: str
    path: Optional[str]
    handle: object       # EngineHandle
    tokenizer: object
    model_cfg: object

    def embedding_rows(self, ids):
        """Token-embedding rows as float32 numpy [len(ids), d_model] (embeddings / rerank routes)."""
        import numpy as np
        import torch

        eng = self.handle.engine
        model = eng.model
        idx = torch.as_tensor(np.asarray(ids, dtype=np.int64))
        if eng.cpu:
            return model.embed[idx].numpy()
        if getattr(model, "embed", None) is not None:
            return model.embed[idx.to(model.embed.device)].float().cpu().numpy()
        from .. import ops

        out = torch.empty(len(idx), self.model_cfg.d_model, dtype=torch.bfloat16, device=model.device)
        ops.dequant_rows(model.embed_q.code, model.embed_q.w, out, n_src_rows=self.model_cfg.vocab_size,
                         k=self.model_cfg.d_model, row_ids=idx.to(device=model.device, dtype=torch.int32))
        return out.float().cpu().numpy()


class ModelManager:
    def __init__(self, loader: Callable[[str, Optional[str]], LoadedModel], models_dir: Optional[str] = None):
        self.loader = loader
        self.models_dir = models_dir
        self.models: dict[str, LoadedModel] = {}
        self.aliases: dict[str, str] = {}
        self.default: Optional[str] = None
        self._lock = threading.Lock()

    def resolve_path(self, name: str) -> Optional[str]:
        cands = [name]
        for d in (self.models_dir, "./models", "."):
            if d:
                cands += [os.path.join(d, name), os.path.join(d, name + ".gguf")]
        for c in cands:
            if os.path.exists(c):
                return c
        return None

    def register(self, m: LoadedModel, alias: Optional[str] = None, default: bool = False) -> None:
        with self._lock:
            self.models[m.name] = m
            if alias:
                self.aliases[alias] = m.name
            if default or self.default is None:
                self.default = m.name

    def load(self, name: str, alias: Optional[str] = None) -> LoadedModel:
        with self._lock:
            key = self.aliases.get(name, name)
            if key in self.models:
                return self.models[key]
        path = self.resolve_path(name)
        if path is None and name not in PRESETS:
            raise ModelLoadError(f"model {name!r} not found (searched {self.models_dir or '.'}, ./models, catalog)")
        m = self.loader(name, path)
        self.register(m, alias)
        return m

    def get(self, name: Optional[str]) -> LoadedModel:
        with self._lock:
            if name:
                key = self.aliases.get(name, name)
                if key in self.models:
                    return self.models[key]
            if self.default is None:
                raise ModelLoadError("no model loaded")
            return self.models[self.default]

    def list(self) -> list[str]:
        with self._lock:
            return list(self.models.keys()) + list(self.aliases.keys())

    def unload(self, name: str) -> bool:
        with self._lock:
            key = self.aliases.get(name, name)
            m = self.models.pop(key, None)
            self.aliases = {a: k for a, k in self.aliases.items() if k != key}
            if self.default == key:
                self.default = next(iter(self.models), None)
        if m is None:
            return False
        m.handle.shutdown()
        return True
