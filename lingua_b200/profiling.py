"""Step-scheduled profiling: allocator memory snapshots first, then a torch.profiler trace.

Same schedule and config as lingua/profiling.py (ProfilerArgs :24, maybe_run_profiler :104): steps
``[mem_warmup, mem_warmup + mem_steps)`` record the CUDA caching-allocator history and dump a
snapshot (``memory_trace_plot/``), steps ``[profile_warmup, profile_warmup + profile_steps)`` run
``torch.profiler`` (CPU + CUDA, shapes, memory, FLOPs) and export a Chrome / Perfetto trace under
``profile_CPU_CUDA_<step>/``. The reference delegates the stepping to ``xformers.profiler``; here
it is a small state machine over ``torch.profiler``. ``perfetto_to_html`` wraps a trace into a
self-contained HTML page when ``viztracer``'s viewer templates are installed.
"""
from __future__ import annotations

import contextlib
import logging
import os
import pickle
import socket
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

from .distributed import get_global_rank, get_is_master

logger = logging.getLogger()


@dataclass
class ProfilerArgs:
    run: bool = False
    trace_folder: str = "profiling"
    mem_warmup: int = 100
    mem_steps: int = 2
    profile_warmup: int = 102
    profile_steps: int = 2


def perfetto_to_html(json_file, html_file) -> bool:
    """Embed a (possibly gzipped) trace into viztracer's viewer page. False if viztracer is absent."""
    import gzip
    import string

    try:
        import viztracer
    except ImportError:
        return False
    root = os.path.dirname(viztracer.__file__)
    sub = {}
    fh = gzip.open(json_file) if ".gz" in str(json_file) else open(json_file)
    with open(os.path.join(root, "html/trace_viewer_embedder.html"), encoding="utf-8") as f:
        tmpl = f.read()
    with open(os.path.join(root, "html/trace_viewer_full.html"), encoding="utf-8") as f:
        sub["trace_viewer_full"] = f.read()
    with fh as j:
        content = j.read()
        if isinstance(content, bytes):
            content = content.decode("utf-8")
        sub["json_data"] = content.replace("</script>", "<\\/script>")
    with open(html_file, "w+", encoding="utf-8") as out:
        out.write(string.Template(tmpl).substitute(sub))
    return True


class StepProfiler:
    """Call ``step()`` once per training iteration."""

    def __init__(self, output_dir: str, config: ProfilerArgs):
        self.output_dir, self.cfg = Path(output_dir), config
        self.step_idx = 0
        self.torch_prof: Optional[torch.profiler.profile] = None
        self.mem_on = False
        self.cuda = torch.cuda.is_available()

    # -- memory snapshots
    def _mem_start(self):
        if self.cuda:
            torch.cuda.memory._record_memory_history(max_entries=100000)
            self.mem_on = True

    def _mem_stop(self):
        if not self.mem_on:
            return
        out = self.output_dir / "memory_trace_plot"
        out.mkdir(parents=True, exist_ok=True)
        name = f"{socket.gethostname()}_{get_global_rank()}"
        try:
            snap = torch.cuda.memory._snapshot()
            with open(out / f"{name}.pickle", "wb") as f:
                pickle.dump(snap, f)
            try:
                from torch.cuda._memory_viz import trace_plot

                (out / f"{name}.html").write_text(trace_plot(snap))
            except Exception as e:  # the plot is a convenience; the pickle is the data
                logger.warning(f"memory trace plot not written: {e}")
        finally:
            torch.cuda.memory._record_memory_history(enabled=None)
            self.mem_on = False

    # -- torch profiler
    def _prof_start(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.cuda:
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.torch_prof = torch.profiler.profile(activities=acts, profile_memory=True, record_shapes=True,
                                                 with_stack=False, with_flops=True)
        self.torch_prof.__enter__()

    def _prof_stop(self):
        if self.torch_prof is None:
            return
        self.torch_prof.__exit__(None, None, None)
        out = self.output_dir / f"profile_CPU_CUDA_{self.step_idx:06d}"
        out.mkdir(parents=True, exist_ok=True)
        trace = out / f"{socket.gethostname()}_{get_global_rank()}.pt.trace.json"
        self.torch_prof.export_chrome_trace(str(trace))
        if get_is_master():
            perfetto_to_html(trace, str(trace).replace(".json", ".html"))
        self.torch_prof = None

    def step(self):
        c = self.cfg
        self.step_idx += 1
        s = self.step_idx
        if s == c.mem_warmup:
            self._mem_start()
        if s == c.mem_warmup + c.mem_steps:
            self._mem_stop()
        if s == c.profile_warmup:
            self._prof_start()
        if s == c.profile_warmup + c.profile_steps:
            self._prof_stop()

    def close(self):
        self._mem_stop()
        self._prof_stop()


@contextlib.contextmanager
def maybe_run_profiler(dump_dir, module, config: ProfilerArgs):
    if not config.run:
        yield None
        return
    trace_dir = os.path.join(dump_dir, config.trace_folder)
    logger.info(f"Profiling active.  Traces will be saved at {trace_dir}")
    if get_is_master():
        os.makedirs(trace_dir, exist_ok=True)
    if torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
        torch.distributed.barrier()
    prof = StepProfiler(trace_dir, config)
    if config.mem_warmup <= 0:
        prof._mem_start()
    try:
        yield prof
    finally:
        prof.close()


class nvtx_range:
    """``with nvtx_range("forward"):`` marks a phase of the step for timeline tools (Nsight Systems, the PyTorch
    profiler's NVTX view). A no-op without CUDA; costs about a microsecond per use with it."""

    __slots__ = ("name", "on")

    def __init__(self, name: str):
        import torch

        self.name, self.on = name, torch.cuda.is_available()

    def __enter__(self):
        if self.on:
            import torch

            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on:
            import torch

            torch.cuda.nvtx.range_pop()
        return False
