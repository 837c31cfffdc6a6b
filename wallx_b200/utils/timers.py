"""Named timers for the training loop.

Same role and surface as the reference's Megatron-style ``Timers`` (wall_x/utils/timers.py:81-502:
``timers(name, log_level).start()/.stop()``, ``log(names, ...)`` with min/max across ranks, optional
TensorBoard ``write``), with one design change: on CUDA a timer brackets its region with events on
the current stream and only resolves them when it is read, instead of calling
``torch.cuda.synchronize()`` at every ``start`` (:156-157), so timing does not serialise host and
device inside the hot loop. Cross-rank statistics use one all-gather of a ``[n_timers]`` vector.
"""
from __future__ import annotations

import time
from typing import Dict, Iterable, List, Optional

import torch


class TimerBase:
    """Interface of a named timer: ``start`` / ``stop`` / ``reset`` / ``elapsed`` (timers.py:42-78 of the reference)."""

    def __init__(self, name: str = ""):
        self.name = name

    def start(self, barrier: bool = False):
        raise NotImplementedError

    def stop(self, barrier: bool = False):
        raise NotImplementedError

    def reset(self):
        raise NotImplementedError

    def elapsed(self, reset: bool = True, barrier: bool = False) -> float:
        raise NotImplementedError


class DummyTimer(TimerBase):
    def __init__(self):
        super().__init__("dummy")

    def start(self, barrier: bool = False):
        return None

    def stop(self, barrier: bool = False):
        return None

    def reset(self):
        return None

    def elapsed(self, reset: bool = True, barrier: bool = False) -> float:
        raise RuntimeError("dummy timer has no elapsed time")

    def active_time(self) -> float:
        raise RuntimeError("dummy timer has no active time: the timer's log level is above the registry's")


class Timer(TimerBase):
    def __init__(self, name: str, use_cuda_events: Optional[bool] = None, nvtx: bool = False):
        super().__init__(name)
        self._elapsed = 0.0
        self._active = 0.0  # total over the timer's life; `reset` does not clear it
        self._started = False
        self._t0 = 0.0
        self._use_events = torch.cuda.is_available() if use_cuda_events is None else use_cuda_events
        self._pending: List = []
        self._ev0 = None
        self._nvtx = nvtx
        self._barrier_group = None

    def set_barrier_group(self, group):
        self._barrier_group = group

    def start(self, barrier: bool = False):
        assert not self._started, f"timer {self.name} has already been started"
        if barrier and torch.distributed.is_initialized():
            torch.distributed.barrier(group=self._barrier_group)
        if self._nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        if self._use_events:
            self._ev0 = torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        else:
            self._t0 = time.time()
        self._started = True

    def stop(self, barrier: bool = False):
        assert self._started, f"timer {self.name} is not started"
        if barrier and torch.distributed.is_initialized():
            torch.distributed.barrier(group=self._barrier_group)
        if self._use_events:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._pending.append((self._ev0, ev1))
        else:
            dt = time.time() - self._t0
            self._elapsed += dt
            self._active += dt
        if self._nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        self._started = False

    def _resolve(self):
        for e0, e1 in self._pending:
            e1.synchronize()
            dt = e0.elapsed_time(e1) / 1e3
            self._elapsed += dt
            self._active += dt
        self._pending = []

    def reset(self):
        self._resolve()  # keep the life-time total exact
        self._elapsed = 0.0
        self._started = False

    def active_time(self) -> float:
        """Seconds this timer has been running since it was created, resets included."""
        self._resolve()
        return self._active

    def elapsed(self, reset: bool = True, barrier: bool = False) -> float:
        """Seconds accumulated so far (resolves outstanding CUDA events)."""
        was = self._started
        if was:
            self.stop(barrier=barrier)
        self._resolve()
        out = self._elapsed
        if reset:
            self.reset()
        if was:
            self.start(barrier=barrier)
        return out


class Timers:
    def __init__(self, log_level: int = 0, log_option: str = "minmax", nvtx: bool = False):
        assert log_option in ("max", "minmax", "all")
        self._log_level = log_level
        self._log_option = log_option
        self._timers: Dict[str, Timer] = {}
        self._levels: Dict[str, int] = {}
        self._dummy = DummyTimer()
        self._max_log_level = 2
        self._nvtx = nvtx
        self._comm = None

    def set_comm(self, comm) -> None:
        """Gather the per-rank times with this transport's small all-reduce (an object with ``rank``, ``world``,
        ``device`` and ``all_reduce_vector``, e.g. :class:`wallx_b200.parallel.symm.SymmComm`) instead of a
        ``torch.distributed`` all-gather: with the NVLink transport the logging path then makes no NCCL call."""
        self._comm = comm

    def __call__(self, name: str, log_level: Optional[int] = None):
        if name in self._timers:
            if log_level is not None:
                assert log_level == self._levels[name], f"timer {name} was created with another log level"
            return self._timers[name]
        level = self._max_log_level if log_level is None else log_level
        assert level <= self._max_log_level
        if level > self._log_level:
            return self._dummy
        self._timers[name] = Timer(name, nvtx=self._nvtx)
        self._levels[name] = level
        return self._timers[name]

    def _gather(self, names: List[str], reset: bool, barrier: bool):
        local = torch.tensor([self._timers[n].elapsed(reset=reset, barrier=barrier) if n in self._timers else 0.0
                              for n in names], dtype=torch.float32)
        comm = self._comm
        if comm is not None and comm.world > 1 and comm.world * len(names) <= 4096:
            table = torch.zeros((comm.world, len(names)), dtype=torch.float32)
            table[comm.rank] = local  # every rank fills its own row: the sum over ranks is the gathered table
            return comm.all_reduce_vector(table.to(comm.device)).cpu()
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            world = torch.distributed.get_world_size()
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.distributed.get_backend() == "nccl" else "cpu"
            buf = torch.zeros((world, len(names)), dtype=torch.float32, device=dev)
            torch.distributed.all_gather_into_tensor(buf.view(-1), local.to(dev)) if dev != "cpu" else \
                torch.distributed.all_gather(list(buf.unbind(0)), local)
            return buf.cpu()
        return local.unsqueeze(0)

    # the reference's helper names (timers.py:302-436), for code that calls them directly
    def _get_elapsed_time_all_ranks(self, names, reset: bool = True, barrier: bool = False) -> torch.Tensor:
        """Seconds per rank and timer, ``[world, len(names)]`` (zero where a rank has no such timer)."""
        return self._gather(list(names), reset, barrier)

    def _get_global_min_max_time(self, names, reset: bool = True, barrier: bool = False, normalizer: float = 1.0):
        """``{name: (min, max)}`` over ranks, divided by ``normalizer``; timers that never ran are left out."""
        names = list(names)
        table = self._gather(names, reset, barrier) / normalizer
        return {n: (float(table[:, i].min()), float(table[:, i].max())) for i, n in enumerate(names) if float(table[:, i].max()) > 0.0}

    def _get_global_min_max_time_string(self, names, reset: bool = True, barrier: bool = False, normalizer: float = 1.0,
                                        max_only: bool = False) -> Optional[str]:
        mm = self._get_global_min_max_time(names, reset, barrier, normalizer)
        if not mm:
            return None
        lines = ["max time across ranks (ms):" if max_only else "(min, max) time across ranks (ms):"]
        for n, (lo, hi) in mm.items():
            lines.append(f"    {n:.<48s}: {hi * 1e3:.2f}" if max_only else f"    {n:.<48s}: ({lo * 1e3:.2f}, {hi * 1e3:.2f})")
        return "\n".join(lines)

    def _get_all_ranks_time_string(self, names, reset: bool = True, barrier: bool = False, normalizer: float = 1.0) -> Optional[str]:
        names = list(names)
        table = self._gather(names, reset, barrier) * 1e3 / normalizer
        lines = ["times across ranks (ms):"]
        for i, n in enumerate(names):
            if float(table[:, i].max()) == 0.0:
                continue
            lines.append(f"  {n}:")
            lines += [f"     rank {r:2d}: {float(table[r, i]):.2f}" for r in range(table.shape[0])]
        return "\n".join(lines) if len(lines) > 1 else None

    def get_all_timers_string(self, names: Optional[Iterable[str]] = None, normalizer: float = 1.0, reset: bool = True,
                              barrier: bool = False) -> Optional[str]:
        names = list(names) if names is not None else list(self._timers.keys())
        assert normalizer > 0.0
        if not names:
            return None
        table = self._gather(names, reset, barrier) * 1000.0 / normalizer
        lines = []
        if self._log_option in ("max", "minmax"):
            head = "(min, max) time across ranks (ms):" if self._log_option == "minmax" else "max time across ranks (ms):"
            lines.append(head)
            for i, n in enumerate(names):
                col = table[:, i]
                if float(col.max()) == 0.0:
                    continue
                if self._log_option == "minmax":
                    lines.append(f"    {n:.<48s}: ({float(col.min()):.2f}, {float(col.max()):.2f})")
                else:
                    lines.append(f"    {n:.<48s}: {float(col.max()):.2f}")
        else:
            lines.append("times across ranks (ms):")
            for i, n in enumerate(names):
                lines.append(f"  {n}:")
                for r in range(table.shape[0]):
                    lines.append(f"     rank {r:2d}: {float(table[r, i]):.2f}")
        return "\n".join(lines) if len(lines) > 1 else None

    def log(self, names: Optional[Iterable[str]] = None, rank: Optional[int] = None, normalizer: float = 1.0,
            reset: bool = True, barrier: bool = False) -> None:
        s = self.get_all_timers_string(names, normalizer, reset, barrier)
        if s is None:
            return
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            rank = torch.distributed.get_world_size() - 1 if rank is None else rank
            if torch.distributed.get_rank() != rank:
                return
        print(s, flush=True)

    def write(self, names: Iterable[str], writer, iteration: int, normalizer: float = 1.0, reset: bool = True,
              barrier: bool = False) -> None:
        names = list(names)
        table = self._gather(names, reset, barrier) / normalizer
        if writer is not None:
            for i, n in enumerate(names):
                writer.add_scalar(n + "-time", float(table[:, i].max()), iteration)
