"""The engine: scheduler above, step function below, one loop.

One ``step()`` = schedule -> run the mixed batch -> sample -> apply tokens -> free what
finished (the reference's loop: v10_triton_paged_gqa/engine.py:101-135, 204-217).  The
loop is synchronous; a failure inside a step ends every live request with that error
and gives all pages and slots back, as the reference's ``fail_all`` does
(engine.py:215-217).
"""
from __future__ import annotations

from typing import Optional

from .. import ops
from ..config.engine import EngineConfig
from ..logger import logger
from ..parts.model import LayeredModel
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduler


class Engine:
    def __init__(self, model: LayeredModel, config: Optional[EngineConfig] = None):
        self.config = config or EngineConfig()
        self.runner = ModelRunner(model, self.config)
        self.scheduler = Scheduler(self.runner, self.config.max_num_batched_tokens, self.config.max_seq_len)

    def add_requests(self, requests: list) -> None:
        for request in requests:
            self.scheduler.validate(request)
        for request in requests:
            self.scheduler.add_request(request)

    def step(self) -> list:
        """One engine step; returns the requests that finished (or failed) in it."""
        scheduler = self.scheduler
        plan = scheduler.schedule()
        done = list(plan.failed)
        if plan.portions:
            entries = []
            for portion in plan.portions:
                request = portion.request
                prompt_len = len(request.prompt_tokens)
                if portion.start >= prompt_len:  # decoding (or recomputing produced tokens)
                    first = portion.start - prompt_len
                    tokens = request.output_tokens[first:first + portion.length]
                elif portion.start + portion.length <= prompt_len:
                    tokens = request.prompt_tokens[portion.start:portion.start + portion.length]
                else:
                    tokens = request.all_tokens[portion.start:portion.start + portion.length]
                entries.append(StepEntry(request.request_id, tokens,
                                         sample=scheduler.sample_spec(request) if portion.samples else None))
            result = self.runner.run(entries)
            sampled = result.tokens.tolist() if result.tokens is not None else []
            done += scheduler.update(plan, sampled)
            if done:  # nothing is handed back before the kernels' own error words have been read
                ops.raise_on_wait_errors()
        scheduler.drain_finished()
        return done

    def run(self) -> list:
        """Step until no request is waiting or running; returns all that ended."""
        ended = []
        try:
            while self.scheduler.has_work():
                ended += self.step()
        except Exception as exc:  # a failed step fails every live request
            logger.error("engine step failed: %s", exc)
            ended += self.scheduler.fail_all(exc)
            self.scheduler.drain_finished()
            raise
        return ended

    def generate(self, requests: list) -> list:
        self.add_requests(requests)
        self.run()
        return requests
