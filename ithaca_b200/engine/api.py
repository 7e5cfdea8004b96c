"""The Python entry point: a model folder (or a configuration and a seed) in, tokens out.

The reference has no Python surface; its programmatic entry is ``Model::load`` +
``Chat::generate`` (src/model.cpp:45, src/chat.cpp:292) behind the command line
(src/main.cpp:1033-1144).  ``Engine`` is that pair: it loads the model the
folder's ``config.json`` names, owns the cache, and offers ``step`` (the step
function) and ``generate`` (the loop with sampling).  Option names are the
reference's where it has them: ``ctx`` (``--ctx``), ``max_tokens``/``temp``/
``top_k``/``top_p``/``rep_pen`` (``GenOpts``).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch

from ..cache.cache import PAGE_SIZE, SequenceCache
from ..config import config_from_dict
from ..parts import Runtime
from ..sampling.sampler import Sampler, SamplingOptions
from ..weights.random_init import random_tensors
from .generate import GenerationOptions, GenStats, generate_loop
from .model import build_model, load_model, weight_manifest
from .graph import GraphDecoder
from .step import Stepper


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_tokens: Optional[int] = None, max_slots: Optional[int] = None, ctx: Optional[int] = None, graphs: bool = True,
                 max_step_tokens: Optional[int] = 16384, _model=None, _config=None, _source=None):
        """``max_tokens``: the most positions live sequences hold at any time, each rounded up
        to a multiple of 64; it sizes the cache (default: 8 sequences of ``ctx``).
        ``ctx``: the most positions one sequence may hold (default: the model's
        ``max_position_embeddings``, as the reference caps ``--ctx`` at the trained
        context, src/model.cpp:259).  ``graphs``: replay decode steps of the generation
        loop from CUDA graphs.  ``max_step_tokens``: the most tokens one pass over the model
        takes (it bounds the activations' memory); a step that brings more, such as a batch of
        long prompts, is run as several passes with the same result (None: no limit)."""
        if not torch.cuda.is_available():
            raise RuntimeError("ithaca_b200 runs on a CUDA device only; none is available")
        torch.cuda.set_device(device)
        self.runtime = Runtime(dtype=dtype, device=device)
        if _model is None:
            if model_dir is None:
                raise ValueError("a model folder is needed")
            _model, _config = load_model(model_dir, self.runtime)
            _source = ("folder", model_dir)
        self.model, self.config = _model, _config
        self._source = _source
        spec = self.model.spec
        self.context_length = min(ctx, spec.max_position) if ctx else spec.max_position
        if max_tokens is None:
            max_tokens = 8 * _round_up(min(self.context_length, 4096), PAGE_SIZE)
        self.cache = SequenceCache(self.model.cache_requests(), max_tokens=max_tokens, max_slots=max_slots,
                                   kv_dtype=self.runtime.kv_dtype, device=device)
        self.stepper = Stepper(self.model, self.cache, max_position=self.context_length, max_step_tokens=max_step_tokens)
        self._status_host: Optional[torch.Tensor] = None
        self._status_event: Optional[torch.cuda.Event] = None
        self._status_pending = False
        self.last_stats: Optional[GenStats] = None
        self._sampler: Optional[Sampler] = None
        self._decoder = GraphDecoder(self.stepper) if graphs and getattr(self.model, "graph_safe", False) else None

    @classmethod
    def from_random(cls, config: Dict[str, Any], seed: int = 0, *, dtype: str = "bfloat16",
                    weights_dtype: Optional[str] = None, device: str = "cuda:0", **kw) -> "Engine":
        """A model with random weights made on the device (nothing is written to disk).  The weights are
        the ones ``write_random_model`` writes for the same configuration, seed and storage type."""
        if not torch.cuda.is_available():
            raise RuntimeError("ithaca_b200 runs on a CUDA device only; none is available")
        torch.cuda.set_device(device)
        arch, cfg = config_from_dict(config)
        runtime = Runtime(dtype=dtype, device=device)
        manifest = weight_manifest(cfg.model_spec())
        storage = weights_dtype or config.get("torch_dtype", "bfloat16")
        tensors = random_tensors(manifest, seed, storage, device=device)
        model = build_model(arch, cfg, tensors, runtime)
        return cls(None, dtype=dtype, device=device, _model=model, _config=cfg,
                   _source=("random", manifest, seed, storage), **kw)

    def dump_tensor(self, name: str) -> torch.Tensor:
        """The tensor of that name as the model was given it (host memory, storage type), before any part
        stacked, reordered or converted it: from the folder the model was loaded from, or made again from
        the seed.  For whoever wants to compute with the model's exact weights elsewhere."""
        if self._source is None:
            raise ValueError("this engine was built from a model object; it has no record of the tensors' origin")
        if self._source[0] == "folder":
            from ..weights.loader import read_model_tensors
            found = read_model_tensors(self._source[1])
            if name not in found:
                raise KeyError(f"the model folder has no tensor '{name}'")
            return found[name]
        _, manifest, seed, storage = self._source
        if name not in manifest:
            raise KeyError(f"the model has no tensor '{name}'")
        from ..weights.random_init import random_tensor
        return random_tensor(name, manifest[name], seed, storage, "cpu")

    def tensor_names(self) -> List[str]:
        return sorted(weight_manifest(self.model.spec))

    # -- the step function ---------------------------------------------------------------------
    def _settle(self) -> None:
        """Anything that touches the cache first drops the decode step that may have been launched ahead."""
        if self._decoder is not None:
            self._decoder.flush()

    def alloc_slot(self) -> int:
        self._settle()
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self._settle()
        self.cache.free_slot(slot)

    def truncate(self, slot: int, n: int) -> None:
        """Keeps the first ``n`` positions of the slot's sequence; the next step's tokens follow them
        (the reference's ``rewind``, src/model.cpp:1047-1058, which its chat loop uses to keep the
        cache of a prefix that the next prompt shares, src/chat.cpp:311-318).  What lay behind is
        overwritten by the tokens fed next and is never read before that.  A sequence whose layers
        keep a fixed-size state can only go back to 0; a windowed group refuses to go back behind
        pages it has released.  On refusal nothing has changed."""
        self._settle()
        self.cache.truncate(slot, n)

    def length(self, slot: int) -> int:
        """Positions the slot's sequence holds."""
        self._settle()
        return self.cache.length(slot)

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Union[str, None, Sequence[Sequence[int]]] = "last") -> Optional[torch.Tensor]:
        """Runs each slot's next tokens as one batch and returns float32 logits [wanted, vocab] on the
        device.  The kernels' status word travels to the host behind the step without a wait; it is looked
        at when the next call arrives (and by ``check_status``), so a refused access surfaces one call
        later at the latest."""
        self._settle()
        self._poll_status()
        logits = self.stepper.step(slots, tokens, want)
        self._note_status()
        return logits

    def _note_status(self) -> None:
        st = self.runtime.status
        if st is None:
            return
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(st, non_blocking=True)
        self._status_event.record()
        self._status_pending = True

    def _poll_status(self, wait: bool = False) -> None:
        if not self._status_pending:
            return
        if wait:
            self._status_event.synchronize()
        elif not self._status_event.query():
            return
        self._status_pending = False
        word = int(self._status_host[0])
        if word:
            self.runtime.status.zero_()
            from .step import describe_status, wait_detail
            from ..cache.pages import CacheError
            raise CacheError("a kernel reported " + describe_status(word) + wait_detail(word)
                             + "; the results since the last check are not to be used")

    def profile_step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], want="last"):
        """One step with CUDA events around every kernel call: returns (logits, rows); see ``engine.profile``."""
        from .profile import profile_step
        return profile_step(self, slots, tokens, want)

    def check_status(self) -> None:
        """Waits for the device and raises if a kernel has recorded something it refused to do."""
        self._poll_status(wait=True)
        self.stepper.check_status()

    # -- Backend of the generation loop --------------------------------------------------------
    def free_slots(self) -> int:
        return self.cache.max_slots - self.cache.table.n_slots_in_use()

    def room_for(self, lengths: Sequence[int], slots: Optional[Sequence[Optional[int]]] = None) -> bool:
        page = self.cache.page_size
        need = 0
        for i, n in enumerate(lengths):
            have = 0
            if slots is not None and slots[i] is not None:
                have = -(-int(self.cache.table._reserved[slots[i]]) // page)      # pages the slot holds already
            need += max(0, -(-n // page) - have)
        return all(need <= pool.n_free for pool in self.cache.table.pools) if self.cache.table.pools else True

    def step_and_sample(self, slots, tokens, streams, counters, recent) -> List[int]:
        if self._decoder is not None and all(len(t) == 1 for t in tokens):
            return self._decoder.step_and_sample(slots, tokens, streams, counters, recent, self._sampler)
        self._settle()
        logits = self.stepper.step(slots, tokens, "last")
        host = self._sampler.sample(logits, streams, counters, recent).cpu()      # waits for the step
        self.stepper.check_status()
        return host.tolist()

    # -- generation ----------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], options: Optional[GenerationOptions] = None,
                 on_token: Optional[Callable[[int, int], bool]] = None, resume=None, **kw) -> List[List[int]]:
        """Generates for every prompt (lists of token ids); returns the new ids per prompt.
        Keyword arguments are ``GenerationOptions`` fields.  Counters of the run are in
        ``last_stats``.  ``resume``: see ``generate_loop`` (``Session`` uses it)."""
        if options is None:
            options = GenerationOptions(**kw)
        elif kw:
            raise ValueError("give either options or keyword arguments")
        self._sampler = Sampler(options.sampling(), self.runtime.device)
        try:
            out, stats = generate_loop(prompts, options, self, stop_token_ids=self.model.spec.stop_token_ids,
                                       on_token=on_token, resume=resume)
        finally:
            self._settle()
        self.last_stats = stats
        return out

    def session(self) -> "Session":
        """A sequence that lives on between calls to ``generate`` and keeps its cache: see ``Session``."""
        from .session import Session
        return Session(self)
