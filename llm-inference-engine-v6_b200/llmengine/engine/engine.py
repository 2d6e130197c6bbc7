"""The engine: one model on one GPU, its cache, and the step function.

Python entry point in the manner of the reference's binding (src/bindings.cpp:150-335):
`Engine(model_dir, dtype)`, `.generate(prompt_ids, max_new_tokens)`, `.forward_logits(ids)`,
`.forward_logits_paged(ids, block_manager)`, `.cfg`, `.max_pos`, `.dtype`, `.weight_names()`,
`.has_weight(name)`; dtype is "fp32" (everything in true 32-bit) or "bf16". Added: `temperature`
and `seed` for generate, `Engine.random(config, seed, dtype)`, and `step(...)`.

There is ONE step function. A step takes a batch of (request, its next tokens, wanted places):
portions of prompts beside single decoded tokens, cut anywhere; it runs only those tokens, from
the cache earlier steps left, and returns the logits of the wanted places. generate(), the
scheduler and trace replay all go through it; the reference has three copies of its layer loop
(forward_step, forward_step_paged, forward_decode_batch; src/engine.cpp:105-682) instead.
"""
from __future__ import annotations

import tempfile
import threading
import warnings
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from ..cache.host import host_module
from ..config.registry import config_from_dir
from ..ops import get_ops
from ..parts.base import BuildEnv
from ..sampling.sampler import Sampler
from ..weights.random_init import write_random_model
from .context import StepBuffers, StepContext, Workspace
from .model import Model

_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}
_DTYPE_NAMES = {torch.float32: "fp32", torch.bfloat16: "bf16"}


class CapacityError(RuntimeError):
    """The page pool cannot hold the tokens a step brings."""


class BlockManager:
    """Size of the page pool, in the reference's terms (src/bindings.cpp:268-285):
    BlockManager(num_blocks, block_size, num_layers, num_kv_heads, head_dim). The pages live on the
    device inside the engine that the manager is given to; the last three arguments are accepted
    for compatibility and checked against the model when the manager is bound."""

    def __init__(self, num_blocks: int, block_size: int, num_layers: Optional[int] = None,
                 num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None):
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("BlockManager: num_blocks and block_size must be >= 1")
        self.num_blocks, self.block_size = int(num_blocks), int(block_size)
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self._engine: Optional["Engine"] = None

    @property
    def free_blocks(self) -> int:
        e = self._engine
        if e is None or e.block_manager is not self:
            return self.num_blocks
        return e.cm.free_pages(0)


class Engine:
    def __init__(self, model_dir: str, dtype: str = "fp32", *, device: str = "cuda:0", block_size: int = 16,
                 num_blocks: Optional[int] = None, max_concurrent: int = 64, ops=None, cuda_graphs: Optional[bool] = None):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be 'fp32' | 'bf16', got: {dtype}")
        self.model_dir = model_dir
        self.device = torch.device(device)
        self.torch_dtype = _DTYPES[dtype]
        self.arch, self.cfg = config_from_dir(model_dir)
        self.spec = self.arch.describe(self.cfg)
        self.ops = ops if ops is not None else get_ops()
        if ops is None and self.device.type != "cuda":
            raise RuntimeError("Engine runs on a CUDA device only (its kernels have no CPU path)")
        self._default_block_size, self._default_num_blocks = block_size, num_blocks
        self._default_slots = max_concurrent
        self._lock = threading.RLock()  # one step at a time (the reference's forward_mu_)
        self.model: Optional[Model] = None
        self.cm = None
        self.block_manager: Optional[BlockManager] = None
        self.ws = Workspace(self.device)
        self.buffers: Optional[StepBuffers] = None
        self.sampler = Sampler(self.ops, self.device)
        self._next_private_id = -1
        # decode-only steps replay CUDA graphs (bfloat16 serving path; the 32-bit path stays eager)
        self.cuda_graphs = (self.torch_dtype == torch.bfloat16 and self.device.type == "cuda") if cuda_graphs is None else cuda_graphs
        self.graphs = None
        self._id_bases = 0
        self._ckpt_names: Optional[List[str]] = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bf16", *, model_dir: Optional[str] = None,
               weights_dtype: Optional[str] = None, **kw) -> "Engine":
        """Writes a model folder with random weights (see weights/random_init.py) and loads it.
        config: typed configuration or config.json dict. The folder is temporary unless given."""
        keep = None
        if model_dir is None:
            keep = tempfile.TemporaryDirectory(prefix="llmengine_random_")
            model_dir = keep.name
        wdt = _DTYPES[weights_dtype or dtype]
        write_random_model(model_dir, config, seed, wdt)
        eng = cls(model_dir, dtype, **kw)
        eng._ensure_model()
        eng._tmp = keep
        return eng

    @property
    def dtype(self) -> str:
        return _DTYPE_NAMES[self.torch_dtype]

    @property
    def max_pos(self) -> int:
        return self.spec.max_positions

    def config(self):
        return self.cfg

    def weight_names(self) -> List[str]:
        if self._ckpt_names is None:
            from ..weights.loader import Checkpoint
            ck = Checkpoint(self.model_dir)
            names = set(ck.names())
            names.update(n for n, twin in self.spec.duplicates.items() if twin in names)
            self._ckpt_names = sorted(names)
        return list(self._ckpt_names)

    def has_weight(self, name: str) -> bool:
        return name in self.weight_names()

    # ------------------------------------------------------------------ lazy parts
    def _ensure_model(self) -> Model:
        """Weights are read at the first forward, so that input errors come before weight errors
        (src/engine.cpp:81-85,720-728)."""
        if self.model is None:
            page = self.block_manager.block_size if self.block_manager else self._default_block_size
            env = BuildEnv(device=self.device, dtype=self.torch_dtype, ops=self.ops, page_size=page)
            model = Model(self.spec, env)
            model.load(self.model_dir)
            self.model = model
            if self.cuda_graphs and not model.capturable:
                self.cuda_graphs = False  # a part waits for the device inside its forward: steps stay eager
            for line in model.kernel_notes():
                warnings.warn(line, stacklevel=2)
        return self.model

    def _default_blocks(self, model: Model, block_size: int) -> int:
        if self._default_num_blocks is not None:
            return self._default_num_blocks
        want_tokens = min(self._default_slots, 8) * self.max_pos
        bpt = max(model.kv_bytes_per_token(), 1)
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            want_tokens = min(want_tokens, int(free * 0.3) // bpt)
        return max(want_tokens // block_size, 1)

    def configure_cache(self, num_blocks: Optional[int] = None, block_size: Optional[int] = None,
                        num_slots: Optional[int] = None, manager: Optional[BlockManager] = None) -> None:
        """(Re)creates the page pool. Every cache group gets `num_blocks` pages."""
        with self._lock:
            if self.cm is not None and self.cm.num_requests:
                raise RuntimeError("configure_cache: requests are still live")
            block_size = block_size or self._default_block_size
            if self.model is not None and self.model.env.page_size != block_size:
                self.model.env.page_size = block_size
            model = self._ensure_model()
            model.env.page_size = block_size
            num_blocks = num_blocks or self._default_blocks(model, block_size)
            num_slots = num_slots or self._default_slots
            H = host_module()
            self.cm = H.CacheManager(block_size, [H.GroupSpec(num_blocks, w) for w in model.windows], num_slots)
            for c in model.caches:  # drop the old pool before the new one is made
                c.k = c.v = None
                c.states = {}
            model.allocate_cache([num_blocks] * len(model.windows), num_slots)
            self.buffers = StepBuffers(self.device, len(model.windows), block_size, self.ws)
            self.graphs = None  # graphs point into the old pool
            self.block_manager = manager
            if manager is not None:
                manager._engine = self

    def bind_block_manager(self, bm: BlockManager, num_slots: Optional[int] = None) -> None:
        slots = num_slots or self._default_slots
        if (self.block_manager is bm and self.cm is not None and self.cm.num_slots >= slots):
            return
        self.configure_cache(bm.num_blocks, bm.block_size, slots, manager=bm)

    def _ensure_cache(self) -> None:
        if self.cm is None:
            self.configure_cache()

    # ------------------------------------------------------------------ the step function
    def step(self, entries, pad_to: Optional[Tuple[int, int, int, int]] = None) -> Tuple[StepContext, torch.Tensor]:
        """Device half of a step. `entries` (host StepEntries) name live requests whose pages for
        these tokens are already reserved. Returns (context, float32 logits [wanted rows, vocab]);
        the logits tensor is scratch that the next step overwrites. The caller advances the
        requests (cache manager) afterwards."""
        with self._lock:
            self._ensure_cache()
            ctx = self.buffers.prepare(self.cm, entries, self.spec.vocab_size, self.max_pos, pad_to)
            logits = self.model.forward(ctx)
            self.queue_error_check()
            return ctx, logits

    # ------------------------------------------------------------------ kernels that gave up
    def queue_error_check(self) -> None:
        """The tensor-core kernels bound every wait; one that gives up leaves a code in a device word
        and returns, and what the step computed is void. A copy of that word travels behind every
        step (4 bytes into pinned memory, also inside the decode graphs) and is looked at wherever
        the host has waited for the step anyway."""
        q = getattr(self.ops, "queue_error_check", None)
        if q is not None:
            q()

    def raise_if_kernel_error(self) -> None:
        """Call after the stream has been synchronized. On a code: the counters that the kernels
        leave at zero between launches are cleared (an aborted launch may not have), the device
        word is reset, and KernelError is raised; the caller decides what becomes of the requests."""
        take = getattr(self.ops, "take_step_error", None)
        code = take() if take is not None else 0
        if not code:
            return
        spaces = [self.ws] + ([c.buffers.ws for c in self.graphs.captured.values()] if self.graphs is not None else [])
        for ws in spaces:
            ws.zero("attention.split_counters")
            ws.zero("gemm.meet_counters")
            ws.zero("attention.work_counters")
        from ..ops import KernelError
        what = getattr(self.ops, "ERROR_CODES", {}).get(code, "unknown code")
        raise KernelError(f"a tensor-core kernel gave up a bounded wait (code {code}: {what}); the step's results are void")

    def step_and_sample(self, entries) -> List[int]:
        """A step followed by the choice of one token for every wanted row (greedy or by the rows'
        temperature, seed and draw index); the tokens come back to the host. Steps in which every
        request brings one token replay a CUDA graph when `cuda_graphs` is on."""
        with self._lock:
            self._ensure_cache()
            n = len(entries)
            if self.cuda_graphs and n and entries.max_tokens() == 1 and entries.num_rows() == n:
                if self.graphs is None:
                    from .graphs import DecodeGraphs
                    self.graphs = DecodeGraphs(self)
                return self.graphs.run(entries)
            ctx, logits = self.step(entries)
            tokens = self.sampler.sample(logits, ctx, ctx.n_rows)  # (waits for the stream)
            self.raise_if_kernel_error()
            return tokens

    def run_step(self, batch: Sequence[Tuple[int, Sequence[int], Sequence[int]]], end: Iterable[int] = ()) -> torch.Tensor:
        """The whole step function for callers that bring their own schedule (trace replay, tests):
        batch = [(request id, its next tokens, wanted places among them), ...]; requests are created
        at first sight, pages reserved (CapacityError if the pool cannot hold them), the tokens run
        as one batch, and requests in `end` give back what they hold afterwards."""
        with self._lock:
            self._ensure_cache()
            H = host_module()
            entries = H.StepEntries()
            fresh = []
            try:
                for rid, tokens, want in batch:
                    rid = int(rid)
                    if not self.cm.has_request(rid):
                        slot = self.cm.add_request(rid)
                        if slot < 0:
                            raise CapacityError(f"no state slot free for request {rid}")
                        fresh.append(rid)
                        self.model.reset_slot(slot)
                    if not self.cm.reserve(rid, len(tokens)):
                        raise CapacityError(f"KV pool exhausted at position {self.cm.length(rid)} of request {rid}")
                    entries.add(rid, [int(t) for t in tokens], [int(w) for w in want])
                ctx, logits = self.step(entries) if len(entries) else (None, torch.empty(0, self.spec.vocab_size))
                if len(entries):
                    if self.device.type == "cuda":
                        torch.cuda.current_stream().synchronize()
                    self.raise_if_kernel_error()
            except Exception:
                for rid in fresh:
                    self.cm.release(rid)
                raise
            for rid, tokens, _ in batch:
                self.cm.advance(int(rid), len(tokens))
            for rid in end:
                if self.cm.has_request(int(rid)):
                    self.cm.release(int(rid))
            return logits

    # ------------------------------------------------------------------ reference-style entry points
    def _validate_ids(self, ids: Sequence[int], where: str) -> None:
        V = self.spec.vocab_size
        for t in ids:
            if t < 0 or t >= V:
                raise ValueError(f"{where}: token id {t} out of range [0, {V})")

    def forward_logits(self, ids: Sequence[int]) -> np.ndarray:
        """Logits [T, V] (float32) at every position of one sequence, fresh cache
        (src/engine.cpp:694-716)."""
        ids = [int(t) for t in ids]
        if not ids:
            raise ValueError("forward_logits: ids is empty")
        self._validate_ids(ids, "forward_logits")
        if len(ids) > self.max_pos:
            raise RuntimeError("forward_logits: sequence length exceeds the position limit")
        with self._lock:
            self._ensure_cache()
            rid = self._private_id()
            logits = self.run_step([(rid, ids, list(range(len(ids))))], end=[rid])
            return logits.float().cpu().numpy().copy()

    def forward_logits_paged(self, ids: Sequence[int], block_manager: BlockManager) -> np.ndarray:
        """As forward_logits, through the given pool (src/engine.cpp:437-467); raises
        "KV pool exhausted ..." when the pool is too small, and gives every page back either way."""
        with self._lock:
            self.bind_block_manager(block_manager)
            return self.forward_logits(ids)

    def _next_id_base(self) -> int:
        """Schedulers that share this engine's cache get disjoint ranges of request ids."""
        self._id_bases += 1
        return self._id_bases << 32

    def _private_id(self) -> int:
        self._next_private_id -= 1
        return self._next_private_id

    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int, temperature: float = 0.0, seed: int = 0):
        """-> (prompt + generated ids, "stop" | "length" | "capacity"). Greedy unless temperature > 0.
        Validation order and errors as the reference (src/engine.cpp:718-774): empty prompt, negative
        max_new_tokens, id out of range -> ValueError; prompt + max_new_tokens beyond the position
        limit -> RuntimeError; all before the weights are read."""
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("generate: prompt_ids is empty")
        if max_new_tokens < 0:
            raise ValueError("generate: max_new_tokens negative")
        self._validate_ids(prompt, "generate")
        if len(prompt) + int(max_new_tokens) > self.max_pos:
            raise RuntimeError("generate: prompt + max_new_tokens exceeds the position limit")
        from .scheduler import ContinuousBatchScheduler
        with self._lock:
            self._ensure_cache()
            sched = ContinuousBatchScheduler(self, None, max_concurrent=1,
                                             max_prefill_tokens_per_step=max(len(prompt), 1))
            sched.enqueue(prompt, int(max_new_tokens), temperature=temperature, seed=seed)
            try:
                sched.run_until_idle()
            except Exception:
                if not sched.core.plan_open:
                    sched.core.finalize()  # the request ended with "error": its pages and slot go back now
                raise
            r = sched.results[0]
            return list(r.token_ids), r.finish_reason
