"""The engine: a model, its cache and the step function, behind one object.

    engine = Engine.load("model_dir", dtype="bfloat16", max_tokens=65536)
    a = engine.open_sequence()
    logits = engine.step([(a, [5, 17, 3])], want=[[2]])     # the prompt, in one step
    logits = engine.step([(a, [42])], want=[[0]])           # then one token
    engine.close_sequence(a)

``step`` runs exactly the tokens it is given, as one batch, on top of what the
cache holds for each slot, and returns 32-bit logits at the wanted places.  It
is the only way tokens reach the model: generation, the command line and trace
replay all go through it.  (The reference's counterpart is ``step_seq_await``
for one sequence, src/model.rs:2272-2308.)
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import architectures  # noqa: F401  (registers the known architectures)
from ..cache import SequenceCache
from ..config import GenerationConfig, load_config, resolve_architecture
from ..kernels import build as kernel_build
from ..parts.base import BuildContext, ProductChoice
from ..weights import DictSource, FolderSource, load_params, random_tensor
from ..sampling import DeviceSampler, HostSampler, SamplingParams
from .batch import make_context
from .generate import GenerationLoop, GenerationOutput, Request
from .graphs import StepGraphs
from .model import Model
from .profile import StepProfile

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', not {d!r}")
    return _DTYPES[d]


def _device(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"device {dev} asked for: this engine runs on a CUDA GPU only "
                           f"(there is no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA GPU is visible: this engine has no CPU path")
    return dev


class Engine:
    DEFAULT_CONTEXT = 4096     # the reference's default context, src/model.rs:1331

    def __init__(self, config, plan, model: Model, dtype: torch.dtype, device: torch.device, *,
                 max_tokens: Optional[int], max_batch: int, max_seq_len: Optional[int],
                 use_graphs: Optional[bool], generation_config: Optional[GenerationConfig] = None):
        self.config, self.plan, self.model = config, plan, model
        self.dtype, self.device = dtype, device
        self.generation_config = generation_config
        # S = min(asked or 4096, max_position_embeddings), src/model.rs:1331
        self.max_seq_len = min(max_seq_len or self.DEFAULT_CONTEXT, plan.max_position)
        if max_tokens is None:
            max_tokens = max_batch * self.max_seq_len
        self.cache = SequenceCache(model.cache_layout(), max_tokens=max_tokens,
                                   max_slots=max_batch, max_seq_len=self.max_seq_len,
                                   dtype=dtype, device=device)
        self.use_graphs = (dtype == torch.bfloat16) if use_graphs is None else bool(use_graphs)
        self.graphs = StepGraphs(model, self.cache, device)
        self.vocab_size = plan.vocab_size
        self.max_batch = self.cache.max_slots
        self.profile: Optional[StepProfile] = None
        self.sampler = DeviceSampler(device)      # its kernels are compiled when first used

    # -- construction --------------------------------------------------------
    @classmethod
    def _build(cls, arch, config, source, dtype, device, products=None, **kw) -> "Engine":
        dtype, device = _dtype(dtype), _device(device)
        torch.cuda.set_device(device)
        plan = arch.plan(config)
        model = Model(plan, BuildContext(dtype, device, products or ProductChoice()))
        get = load_params(model.expected(), source, dtype, device)
        with torch.cuda.device(device):
            model.load(get)
        kernel_build.compile_modules(model.kernel_modules())
        for m in model.kernel_modules():
            kernel_build.module(m)
        return cls(config, plan, model, dtype, device, **kw)

    @classmethod
    def load(cls, model_dir: str, dtype="bfloat16", device="cuda:0", *, max_tokens=None,
             max_batch: int = 64, max_seq_len=None, use_graphs=None,
             products: Optional[ProductChoice] = None) -> "Engine":
        """A model folder: config.json chooses the architecture, the safetensors
        file(s) give the weights.  ``products`` names the kernels of the linear
        layers (``parts.ProductChoice``; None: the defaults)."""
        arch, config = load_config(model_dir)
        return cls._build(arch, config, FolderSource(model_dir), dtype, device, products=products,
                          max_tokens=max_tokens, max_batch=max_batch, max_seq_len=max_seq_len,
                          use_graphs=use_graphs,
                          generation_config=GenerationConfig.from_model_dir(model_dir))

    @classmethod
    def from_tensors(cls, config: dict, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                     device="cuda:0", **kw) -> "Engine":
        arch = resolve_architecture(config)
        cfg = arch.config_cls.from_dict(config)
        kw.setdefault("max_tokens", None), kw.setdefault("max_batch", 64)
        kw.setdefault("max_seq_len", None), kw.setdefault("use_graphs", None)
        return cls._build(arch, cfg, DictSource(tensors), dtype, device, **kw)

    @classmethod
    def random(cls, config: dict, seed: int, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        """Random weights made on the device, tensor by tensor, without a folder
        (for sizes that are not worth writing to disk)."""
        arch = resolve_architecture(config)
        cfg = arch.config_cls.from_dict(config)
        kw.setdefault("max_tokens", None), kw.setdefault("max_batch", 64)
        kw.setdefault("max_seq_len", None), kw.setdefault("use_graphs", None)
        dev = _device(device)

        class _Made(DictSource):
            def __init__(self, expected):
                self.expected, self.where = expected, f"random weights (seed {seed})"

            def shapes(self):
                return {n: s.shape for n, s in self.expected.items()}

            def tensor(self, name):
                return random_tensor(name, self.expected[name], seed, torch.bfloat16, dev)

        plan = arch.plan(cfg)
        probe = Model(plan, BuildContext(torch.bfloat16, torch.device("cpu")))
        return cls._build(arch, cfg, _Made(probe.expected()), dtype, device, **kw)

    def check(self) -> None:
        """Waits for the device and raises ``KernelError`` if a kernel gave up on one of
        its bounded waits since the last check (its results are then void).  Generation
        checks after every batch; a caller that steps by itself calls this where it
        reads results."""
        from ..kernels import ops
        torch.cuda.synchronize(self.device)
        ops.check_kernel_errors()

    # -- sequences -------------------------------------------------------------
    def open_sequence(self) -> int:
        return self.cache.open()

    def close_sequence(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # -- the step --------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """entries: (slot, next tokens) per sequence; want: per entry, the places
        among its tokens whose logits are returned ([n_wanted, vocab], float32, in
        the order of the entries and of ``want``).  None when nothing is wanted.
        The tensor returned is the caller's: later steps do not change it."""
        if not entries:
            raise ValueError("a step needs at least one sequence")
        want = [list(w) for w in want] if want is not None else [[] for _ in entries]
        if len(want) != len(entries):
            raise ValueError("one list of wanted places per entry is needed")
        seen = set()
        for slot, toks in entries:
            if slot in seen:
                raise ValueError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if len(toks) == 0:
                raise ValueError(f"slot {slot} brings no tokens")   # src/model.rs:2286
            bad = [t for t in toks if not 0 <= int(t) < self.vocab_size]
            if bad:
                raise ValueError(f"token {bad[0]} is outside the vocabulary of {self.vocab_size}")
        for i, ((_slot, toks), w) in enumerate(zip(entries, want)):
            for p in w:
                if not 0 <= int(p) < len(toks):
                    raise ValueError(f"wanted place {p} is outside the {len(toks)} tokens of entry {i}")
        for slot, toks in entries:
            self.cache.reserve(slot, len(toks))
        self.cache.flush()
        packed = [(slot, self.cache.length[slot], list(toks)) for slot, toks in entries]
        decode = all(len(t) == 1 for _s, t in entries)
        graph = None
        if self.use_graphs and decode:
            graph = self.graphs.decode(len(entries), max(s + 1 for _slot, s, _t in packed))
        elif self.use_graphs:
            graph = self.graphs.prompt(sum(len(t) for _s, t in entries), len(entries),
                                       sum(len(w) for w in want))
        started = self.profile.begin() if self.profile else None
        with torch.cuda.device(self.device):
            if graph is not None and decode:
                all_rows = graph.run(packed)      # the graph's own buffer: the next replay rewrites it
                idx = [i for i, w in enumerate(want) for _p in w]
                if not idx:
                    logits = None
                elif idx == list(range(len(idx))):
                    logits = all_rows[:len(idx)].clone()
                else:
                    logits = all_rows[torch.tensor(idx, device=self.device)]
            elif graph is not None:
                logits = graph.run(packed, want)
                logits = logits.clone() if logits is not None else None
            else:
                ctx = make_context(packed, want, self.device)
                logits = self.model.forward(ctx, self.cache)
        for slot, toks in entries:
            self.cache.advance(slot, len(toks))
        if self.profile:
            self.profile.end("decode" if decode else "prompt", len(entries),
                             sum(len(t) for _s, t in entries), started)
        return logits

    # -- stepping ahead --------------------------------------------------------
    class Chosen:
        """Tokens chosen on the device, on their way to the host: ``dev`` is the
        int32 device tensor; the copy to pinned memory was queued right behind the
        kernel that chose them, so ``tolist()`` waits for that copy only and not
        for work queued since (the step that already runs on these tokens)."""

        def __init__(self, dev: torch.Tensor, host: torch.Tensor):
            self.dev, self.host = dev, host
            host[:dev.shape[0]].copy_(dev, non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()

        def tolist(self) -> List[int]:
            self.event.synchronize()
            return self.host[:self.dev.shape[0]].tolist()

    def choose_ahead(self, logits: torch.Tensor, params, draws) -> "Engine.Chosen":
        """The device sampler's choice for every row, readable later."""
        if not hasattr(self, "_chosen_ring"):
            self._chosen_ring = [torch.zeros(max(self.max_batch, 1), dtype=torch.int32).pin_memory()
                                 for _ in range(4)]
            self._chosen_turn = 0
        host = self._chosen_ring[self._chosen_turn]
        self._chosen_turn = (self._chosen_turn + 1) % len(self._chosen_ring)
        with torch.cuda.device(self.device):
            return Engine.Chosen(self.sampler.choose(logits, params, draws), host)

    def can_step_ahead(self, n: int) -> bool:
        """Whether decode steps of up to ``n`` sequences can take their tokens on
        the device (they run as captured graphs)."""
        return bool(self.use_graphs) and 0 < n <= self.graphs.largest

    def step_ahead(self, entries: Sequence[Tuple[int, int]], chosen: torch.Tensor) -> torch.Tensor:
        """One decode step whose input tokens are still on the device: entry
        (slot, r) continues the sequence in ``slot`` with ``chosen[r]``, an int32
        device tensor (or the handle of ``choose_ahead``) that earlier work on this
        stream writes.  Nothing waits for the host.  Returns the step's logits, one row per entry in their order
        (rows beyond them, if any, are padding)."""
        if not entries:
            raise ValueError("a step needs at least one sequence")
        slots = [s for s, _r in entries]
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        if not self.can_step_ahead(len(entries)):
            raise ValueError("this many sequences cannot step ahead: ask can_step_ahead first")
        for slot in slots:
            self.cache.reserve(slot, 1)
        self.cache.flush()
        graph = self.graphs.decode(len(entries), max(self.cache.length[s] for s in slots) + 1)
        packed = [(slot, self.cache.length[slot], [0]) for slot in slots]
        with torch.cuda.device(self.device):
            logits = graph.run(packed, tokens_from=(getattr(chosen, "dev", chosen),
                                                    [r for _s, r in entries]))
        for slot in slots:
            self.cache.advance(slot, 1)
        return logits[:len(entries)]

    def rows(self, logits: torch.Tensor, keep: Sequence[int]) -> torch.Tensor:
        """The given rows of a step's logits, in that order, without waiting."""
        keep = list(keep)
        if keep == list(range(keep[0], keep[0] + len(keep))):
            return logits[keep[0]:keep[0] + len(keep)]
        return logits[torch.tensor(keep, device=logits.device)]

    # -- generation ------------------------------------------------------------
    def default_stop_ids(self) -> Tuple[int, ...]:
        """generation_config.json's eos list replaces config.json's eos
        (src/model.rs:1340-1348)."""
        if self.generation_config is not None and self.generation_config.eos_token_ids() is not None:
            return self.generation_config.eos_token_ids()
        return tuple(self.plan.stop_tokens)

    def default_sampling(self, do_sample: bool = False, seed: Optional[int] = None) -> SamplingParams:
        return SamplingParams.from_generation_config(self.generation_config, do_sample, seed)

    def generate(self, prompts, max_new_tokens: int = 128, *,
                 sampling: Optional[SamplingParams] = None, stop_ids=None, ignore_eos: bool = False,
                 device_argmax: bool = True, include_stop: bool = False,
                 look_ahead: bool = True) -> List[GenerationOutput]:
        """prompts: lists of token ids (or ready ``Request`` objects).  Requests
        are served in batches of unequal prompts; tokens come back as host ints.
        ``look_ahead`` (with ``device_argmax``): queue each decode step before the
        tokens of the one before have been read, its input taken on the device; the
        tokens returned are the same in the 32-bit path and, in bfloat16, the same
        up to the rounding of a step that ran in another bucket of rows
        (``engine.generate`` says when)."""
        sampling = (sampling or SamplingParams()).normalised()
        if ignore_eos:
            stops: Tuple[int, ...] = ()               # src/model.rs:1517-1521
        elif stop_ids is None:
            stops = self.default_stop_ids()
        else:
            stops = tuple(int(t) for t in stop_ids)
        requests = [p if isinstance(p, Request) else
                    Request(list(p), max_new_tokens, sampling, stops, include_stop) for p in prompts]
        sampler = self.sampler if device_argmax else HostSampler()

        def choose(logits, params, draws):
            out = sampler.choose(logits, params, draws)
            return out.tolist() if isinstance(out, torch.Tensor) else out

        ahead = self.choose_ahead if (look_ahead and device_argmax) else None
        loop = GenerationLoop(self, choose, max_batch=self.max_batch,
                              max_tokens=self.cache.max_tokens, max_seq_len=self.max_seq_len,
                              vocab_size=self.vocab_size, sync=self.check,
                              choose_ahead=ahead)
        return loop.run(requests)
