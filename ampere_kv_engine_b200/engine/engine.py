"""The Python entry point: a model folder (or a configuration and a seed) to generated tokens.

``Engine.generate`` is the multi-request form of the reference's ``generate_tokens``
(ampere_kv/runner.py:301-406) driven through its scheduler loop
(``while any unfinished: scheduler.step()``, ampere_kv/bench_external.py:109-114): host token
ids in, host token ids out, greedy by default, stop at EOS unless ``ignore_eos``.
"""

from __future__ import annotations

import torch

from ..config.engine_config import EngineConfig, dtype_name
from ..models.decoder import DecoderModel
from ..models.registry import ARCHITECTURES, config_from_dict, load_config
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import load_weights
from ..weights.random_init import init_random
from .batch import SeqStep
from .scheduler import Request, Scheduler
from .step import ModelRunner

def parse_dtype(name) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype_name(name)]


def set_exact_matmul() -> None:
    """No reduced-precision matrix mode anywhere: float32 products stay float32 (no TF32), and
    bfloat16 products accumulate and reduce in float32."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # pragma: no cover
        pass


class Engine:
    """Model + cache + scheduler + sampler on one device."""

    def __init__(self, model: DecoderModel, config: EngineConfig | None = None, **options):
        """``config`` and/or single options of :class:`EngineConfig` by keyword (they override ``config``'s)."""
        set_exact_matmul()
        self.model = model
        self.device = model.device
        if config is None and "dtype" not in options:
            options["dtype"] = dtype_name(model.dtype)      # no word on the dtype: the model's
        config = EngineConfig.from_options(config, **options)
        if parse_dtype(config.dtype) != model.dtype:
            raise ValueError(f"engine option 'dtype' is {config.dtype} but the model was built in {model.dtype}")
        self.config = config = config.resolved(model.spec.max_position)
        self.runner = ModelRunner(model, page_size=config.page_size, num_pages=config.num_pages,
                                  max_seqs=config.max_seqs, kv_dtype=parse_dtype(config.kv_dtype),
                                  cuda_graphs=config.cuda_graphs)
        self.manager = self.runner.manager
        self.sampler = Sampler(self.device)
        self.vocab_size = model.spec.vocab_size
        self.max_batch_tokens = config.max_batch_tokens
        self.max_seqs = max_seqs = config.max_seqs
        self.admission = config.admission
        self.eos_token_ids = tuple(model.spec.eos_token_ids)
        self._stream_counter = 0
        # pinned landing places of the chosen tokens (+ the status word); three, since one step may be in flight
        # while the one before it is read, and a third is filled only after both of those
        self._readback = [torch.zeros(max_seqs + 2, dtype=torch.int32) for _ in range(3)]
        if self.device.type == "cuda":
            self._readback = [t.pin_memory() for t in self._readback]
        self._readback_turn = 0

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_pretrained(cls, model_dir: str, *, dtype=None, device="cuda", config: EngineConfig | None = None,
                        **engine_options) -> "Engine":
        """``dtype`` (or ``config.dtype``; default bfloat16) is the compute dtype the weights are loaded in."""
        options = EngineConfig.from_options(config, **engine_options, **({} if dtype is None else {"dtype": dtype}))
        arch, model_config = load_config(model_dir)
        model = DecoderModel(arch.build_spec(model_config), dtype=parse_dtype(options.dtype), device=device)
        load_weights(model, model_dir)
        return cls(model, options)

    @classmethod
    def from_random(cls, model_config, seed: int = 0, *, dtype=None, device="cuda",
                    config: EngineConfig | None = None, **engine_options) -> "Engine":
        """``model_config``: a typed configuration, or a dict of config.json keys (with ``architectures``)."""
        options = EngineConfig.from_options(config, **engine_options, **({} if dtype is None else {"dtype": dtype}))
        if isinstance(model_config, dict):
            arch, model_config = config_from_dict(model_config)
        else:
            arch = ARCHITECTURES[model_config.architectures[0]]
        model = DecoderModel(arch.build_spec(model_config), dtype=parse_dtype(options.dtype), device=device)
        init_random(model, seed)
        return cls(model, options)

    # ------------------------------------------------------------------ executor interface (for the scheduler)

    def execute(self, entries: list[SeqStep], wanted: list[Request]) -> list[int]:
        """Run the batch and return the chosen token of every wanted request (blocks until the device is done)."""
        return self.collect(self.launch(entries, wanted, [len(r.output_ids) for r in wanted]))

    def launch(self, entries: list[SeqStep], wanted: list[Request], steps: list[int]):
        """Enqueue the batch and the choice of its tokens without waiting for either.  ``steps``: the index of the
        token being chosen within each wanted request (the sampler's draw depends on it).  The chosen tokens stay
        on the device (``runner.sampled``, row i for ``wanted[i]``), where the next step's entries with a
        ``source`` find them, and travel to a pinned host buffer that :meth:`collect` reads."""
        if self.config.nvtx:
            decode = sum(1 for e in entries if len(e.tokens) == 1)
            torch.cuda.nvtx.range_push(f"step: decode_tokens={decode} prompt_tokens="
                                       f"{sum(len(e.tokens) for e in entries) - decode} seqs={len(entries)}")
            try:
                logits = self.runner.step(entries)
            finally:
                torch.cuda.nvtx.range_pop()
        else:
            logits = self.runner.step(entries)
        if logits is None:
            return None
        # the choice lands where the next step's entries with a ``source`` look for it, right behind the kernels'
        # status word: one read-back brings both
        count = self.sampler.sample(logits, [r.sampling for r in wanted], steps, out=self.runner.sampled).shape[0]
        slot = self._readback[self._readback_turn]
        self._readback_turn = (self._readback_turn + 1) % len(self._readback)
        if self.device.type == "cuda":
            slot[:count + 1].copy_(self.runner.outcome[:count + 1], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        else:
            slot[:count + 1].copy_(self.runner.outcome[:count + 1])
            done = None
        return slot, count, done

    def collect(self, handle) -> list[int]:
        """The tokens of a launched batch, once the device has them."""
        if handle is None:
            self.runner.raise_on_status()
            return []
        slot, count, done = handle
        if done is not None:
            done.synchronize()
        host = slot[:count + 1].tolist()      # the status word, then the tokens
        if host[0]:
            self.runner.raise_on_status()
        return host[1:]

    def new_scheduler(self, **overrides) -> Scheduler:
        options = dict(max_batch_tokens=self.max_batch_tokens, max_seqs=self.max_seqs,
                       eos_token_ids=self.eos_token_ids, admission=self.admission,
                       max_context=self.config.max_context, lookahead=self.config.lookahead,
                       nvtx=self.config.nvtx)
        options.update(overrides)
        return Scheduler(self, **options)

    # ------------------------------------------------------------------ generation

    def generate(self, prompts: list[list[int]], max_new_tokens: int = 32, *, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False) -> list[list[int]]:
        """New token ids for every prompt (host lists in, host lists out)."""
        if prompts and isinstance(prompts[0], int):
            raise TypeError("generate() takes a list of prompts, each a list of token ids")
        scheduler = self.new_scheduler()
        requests = []
        for index, prompt in enumerate(prompts):
            sampling = SamplingParams(temperature=temperature, seed=seed, stream=index)
            requests.append(scheduler.submit(f"g{self._stream_counter}-{index}", prompt, max_new_tokens,
                                             sampling=sampling, ignore_eos=ignore_eos))
        self._stream_counter += 1
        while scheduler.has_work():
            scheduler.step()
        return [list(r.output_ids) for r in requests]
