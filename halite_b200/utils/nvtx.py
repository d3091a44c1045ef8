"""NVTX phase ranges and a step-window profiler for the training and rollout loops.

`phase("forward")` marks a range that `ncu --nvtx`, Nsight Systems and `torch.profiler` show on
the timeline; on a CPU-only run it does nothing. `StepWindowProfiler` implements the
`--profile-steps a:b` switch of the entry-point scripts: steps a..b-1 run between
`cudaProfilerStart` / `cudaProfilerStop` (so an external profiler started with
`--capture-range cudaProfilerApi` records exactly that window) and under `torch.profiler`, whose
kernel table is logged and whose Chrome trace is written next to the checkpoints.
"""

from __future__ import annotations

import contextlib
import os

import torch


def _on() -> bool:
    return torch.cuda.is_available()


@contextlib.contextmanager
def phase(name: str):
    if not _on():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def mark(name: str):
    if _on():
        torch.cuda.nvtx.mark(name)


def parse_step_window(text):
    """'a:b' -> (a, b) with b exclusive; None / '' -> None."""
    if not text:
        return None
    a, _, b = str(text).partition(":")
    a = int(a)
    b = int(b) if b else a + 1
    if b <= a:
        raise ValueError(f"--profile-steps {text!r}: the window is empty")
    return a, b


class StepWindowProfiler:
    def __init__(self, window, output_dir=None, log=None, rank=0):
        self.window = window
        self.output_dir = output_dir
        self.log = log
        self.rank = rank
        self._prof = None
        self.table = None

    def step_begin(self, step):
        if self.window is None or step != self.window[0]:
            return
        acts = [torch.profiler.ProfilerActivity.CPU]
        if _on():
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts)
        self._prof.__enter__()

    def step_end(self, step):
        if self._prof is None or step != self.window[1] - 1:
            return
        if _on():
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        self._prof.__exit__(None, None, None)
        prof, self._prof = self._prof, None
        key = "self_cuda_time_total" if _on() else "self_cpu_time_total"
        self.table = prof.key_averages().table(sort_by=key, row_limit=25)
        if self.log is not None:
            self.log.info(f"profile of steps {self.window[0]}..{self.window[1] - 1}\n{self.table}")
        if self.output_dir is not None:
            os.makedirs(self.output_dir, exist_ok=True)
            prof.export_chrome_trace(os.path.join(
                self.output_dir, f"profile_steps_{self.window[0]}_{self.window[1]}_rank{self.rank}.json"))
