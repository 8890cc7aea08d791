"""The engine's own options as one typed, validated object.

The reference spreads them over the constructor arguments of its scheduler and module constants
(ampere_kv/scheduler.py:44-49: block count, batch limit, prefill chunk size, each checked there;
ampere_kv/runner.py:17-19: token limit and page size) and refuses a request that cannot fit at
submit time (scheduler.py:79-93).  Here they are fields of :class:`EngineConfig`, checked in one
place, and every entry point (the Python entry, the command line, trace replay, the benchmark)
builds the engine from one.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

_DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}
ADMISSION_RULES = ("budget", "optimistic")


class EngineConfigError(ValueError):
    """An engine option is of the wrong type, out of range, or contradicts another."""


def dtype_name(value) -> str:
    """``"bfloat16"`` or ``"float32"`` for a name, a short name or a torch dtype."""
    text = str(value).replace("torch.", "")
    if text not in _DTYPE_NAMES:
        raise EngineConfigError(f"dtype must be one of {sorted(set(_DTYPE_NAMES))}, got {value!r}")
    return _DTYPE_NAMES[text]


@dataclass(frozen=True)
class EngineConfig:
    #: compute dtype: ``bfloat16`` (serving) or ``float32`` (everything in true 32-bit)
    dtype: str = "bfloat16"
    #: dtype of the cache pages; None = the compute dtype.  The attention kernels read pages as they are stored,
    #: so a cache dtype other than the compute dtype is refused.
    kv_dtype: str | None = None
    #: tokens per cache page
    page_size: int = 16
    #: pages of every cache group's pool; None = derived from ``max_tokens``
    num_pages: int | None = None
    #: tokens the pool must hold when ``num_pages`` is not given; None = four contexts of at most 8,192 tokens
    max_tokens: int | None = None
    #: most requests alive at a time (state slots, rows of the block tables)
    max_seqs: int = 256
    #: token budget of one scheduler round (decoded tokens and prompt portions together)
    max_batch_tokens: int = 2048
    #: longest prompt + new tokens a request may ask for; None = the model's ``max_position_embeddings``
    max_context: int | None = None
    #: what admission reserves: ``budget`` (all pages a request can ever hold) or ``optimistic`` (its next portion)
    admission: str = "budget"
    #: replay decode-only steps as CUDA graphs
    cuda_graphs: bool = True
    #: queue each scheduler round before the previous round's tokens are read
    lookahead: bool = True
    #: wrap scheduler rounds and model steps in NVTX ranges (for a timeline profiler)
    nvtx: bool = False

    def __post_init__(self):
        object.__setattr__(self, "dtype", dtype_name(self.dtype))
        if self.kv_dtype is not None:
            object.__setattr__(self, "kv_dtype", dtype_name(self.kv_dtype))
        self.validate()

    def validate(self) -> None:
        def positive_int(name: str, optional: bool = False) -> None:
            value = getattr(self, name)
            if value is None and optional:
                return
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise EngineConfigError(f"engine option '{name}' must be a positive integer, got {value!r}")

        positive_int("page_size")
        positive_int("num_pages", optional=True)
        positive_int("max_tokens", optional=True)
        positive_int("max_seqs")
        positive_int("max_batch_tokens")
        positive_int("max_context", optional=True)
        if self.admission not in ADMISSION_RULES:
            raise EngineConfigError(f"engine option 'admission' must be one of {list(ADMISSION_RULES)}, "
                                    f"got {self.admission!r}")
        if self.kv_dtype is not None and self.kv_dtype != self.dtype:
            raise EngineConfigError(f"engine option 'kv_dtype' ({self.kv_dtype}) must equal 'dtype' ({self.dtype}): "
                                    f"cache pages are read by the attention kernels as they are stored")
        for name in ("cuda_graphs", "lookahead", "nvtx"):
            if not isinstance(getattr(self, name), bool):
                raise EngineConfigError(f"engine option '{name}' must be true or false, got {getattr(self, name)!r}")

    def replace(self, **changes) -> "EngineConfig":
        unknown = sorted(set(changes) - {f.name for f in dataclasses.fields(self)})
        if unknown:
            raise EngineConfigError(f"unknown engine option(s) {unknown}; known: "
                                    f"{[f.name for f in dataclasses.fields(self)]}")
        return dataclasses.replace(self, **changes)

    @classmethod
    def from_options(cls, config: "EngineConfig | None" = None, **options) -> "EngineConfig":
        """``config`` with ``options`` laid over it (or the defaults, when there is none)."""
        return (config or cls()).replace(**options) if options or config is None else config

    def resolved(self, max_position: int) -> "EngineConfig":
        """The same options with every derived value filled in for a model of ``max_position`` positions:
        ``max_context`` (at most what the model's positions allow), ``num_pages``."""
        max_context = self.max_context if self.max_context is not None else max_position
        if max_context > max_position:
            raise EngineConfigError(f"engine option 'max_context' ({max_context}) exceeds the model's "
                                    f"max_position_embeddings ({max_position})")
        num_pages = self.num_pages
        if num_pages is None:
            tokens = self.max_tokens if self.max_tokens is not None else min(max_position, 8192) * 4
            num_pages = (tokens + self.page_size - 1) // self.page_size + self.max_seqs
        return dataclasses.replace(self, max_context=max_context, num_pages=num_pages,
                                   kv_dtype=self.kv_dtype or self.dtype)
