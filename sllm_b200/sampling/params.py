"""What a request asks of the sampler."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    """Names and meanings after the reference's generate() (serving/executor.py:334-345)
    and its dev command line (serving/cli.py:18-23): ``max_new`` tokens at most;
    ``temperature`` <= 0 is greedy (the engine facade's default, serving/executor.py:539);
    ``top_k``/``top_p`` filter as runtime/sampler.py:60-79 does; ``seed`` seeds the
    request's own generator; ``repetition_penalty`` as runtime/sampler.py:12-33;
    a token in ``stop_ids`` ends the request and is not part of its output."""
    max_new: int = 16
    temperature: float = 0.0
    top_k: int | None = None
    top_p: float | None = None
    seed: int | None = None
    repetition_penalty: float | None = None
    stop_ids: tuple = ()

    def __post_init__(self):
        if self.max_new < 1:
            raise ValueError("max_new must be >= 1")
        if self.top_k is not None and int(self.top_k) <= 0:
            raise ValueError("top_k must be >= 1")          # runtime/sampler.py:62-63
        self.stop_ids = tuple(int(s) for s in self.stop_ids)

    @property
    def penalised(self) -> bool:
        """Whether a repetition penalty applies (runtime/sampler.py:24: none, <= 0 and 1 change nothing)."""
        p = self.repetition_penalty
        return p is not None and p > 0 and p != 1.0
