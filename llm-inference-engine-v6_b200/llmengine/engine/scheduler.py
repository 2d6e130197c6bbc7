"""Continuous batching above the step function.

The decisions (admission, portions under the token budget, page reservation, finishing) are made by
the C++ core (csrc/host/scheduler.cpp); this class runs each planned batch through Engine.step,
samples on the device and hands the tokens back. Names follow the reference's binding
(src/bindings.cpp:287-335): ContinuousBatchScheduler(engine, block_manager, max_concurrent=64,
max_prefill_tokens_per_step=256), enqueue, step, run_until_idle, idle, results, clear_results,
budget.
"""
from __future__ import annotations

from typing import List, Sequence

from ..cache.host import host_module
from ..ops import KernelError


class ContinuousBatchScheduler:
    def __init__(self, engine, block_manager=None, max_concurrent: int = 64, max_prefill_tokens_per_step: int = 256):
        if max_concurrent <= 0:
            raise ValueError("ContinuousBatchScheduler: max_concurrent must be >= 1")
        if max_prefill_tokens_per_step <= 0:
            raise ValueError("ContinuousBatchScheduler: max_prefill_tokens_per_step must be >= 1")
        self.engine = engine
        if block_manager is not None:
            engine.bind_block_manager(block_manager, max_concurrent)
        else:
            engine._ensure_cache()
        H = host_module()
        self.core = H.SchedulerCore(engine.cm, engine.spec.vocab_size, engine.max_pos,
                                    set(int(t) for t in engine.spec.eos_token_ids), max_concurrent,
                                    max_prefill_tokens_per_step, engine._next_id_base(),
                                    engine.model.portion_multiple)
        self._cm = engine.cm
        self.steps = 0

    def enqueue(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0, seed: int = 0) -> int:
        try:
            return self.core.enqueue([int(t) for t in prompt], int(max_new_tokens), float(temperature), int(seed))
        except OverflowError:
            raise ValueError("enqueue: token id or count out of the 32-bit range") from None

    def step(self) -> bool:
        """One iteration: plan, run the batch as one step, sample, commit. False when idle."""
        eng = self.engine
        if eng.cm is not self._cm:
            raise RuntimeError("the engine's cache was reconfigured while this scheduler was in use")
        with eng._lock:
            entries = self.core.plan()
            for rid in self.core.last_admitted:
                eng.model.reset_slot(self._cm.slot(rid))
            if len(entries):
                try:
                    tokens = eng.step_and_sample(entries)
                except KernelError:
                    # what the step computed is void: its requests end with "error" (their pages come
                    # back at the next plan); requests that were not in the step go on
                    self.core.fail_step("error")
                    raise
                self.core.commit(tokens)
                self.steps += 1
        return not self.core.idle

    def run_until_idle(self) -> None:
        while self.step():
            pass
        self.core.finalize()

    @property
    def idle(self) -> bool:
        return self.core.idle

    @property
    def results(self) -> List:
        return self.core.results

    def clear_results(self) -> None:
        self.core.clear_results()

    @property
    def budget(self) -> int:
        return self.core.budget

    @budget.setter
    def budget(self, b: int) -> None:
        self.core.budget = int(b)
