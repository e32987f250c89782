# -*- coding: utf-8 -*-
"""Optional timeline of the communication side stream.

``CommTrace(optimizer)`` wraps the fused communicator's ``launch_group`` so that every group launch
records a start and a stop CUDA event on the side stream plus the host time of the launch;
``summary()`` (after a device synchronisation) yields per-group device time, the total
communication time and the **exposed communication time** of the traced iteration: the time between
the end of the last backward kernel on the compute stream and the end of the last communication
kernel, clamped at zero.  The reference has only wall-clock timers that are never switched on
(``distributed_optimizer.py:58-60,407-425``).  NVTX ranges are emitted when available so that the
launches also show up in external timeline tools.
"""
from __future__ import annotations

import json
import time
from typing import Dict, List, Optional

import torch


class CommTrace:
    def __init__(self, optimizer):
        self.opt = optimizer
        self.comm = optimizer.communicator
        if not getattr(self.comm, 'fused', False):
            raise ValueError('CommTrace needs the fused NVLink communicator')
        self.records: List[dict] = []
        self._orig = self.comm.launch_group
        self._backward_end: Optional[torch.cuda.Event] = None
        self.enabled = False

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
        return False

    def start(self) -> None:
        if self.enabled:
            return
        trace = self

        def traced(opt, gi):
            if opt is not trace.opt:
                return trace._orig(opt, gi)
            s = trace.comm.stream
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push('mgwfbp.group%d' % gi)
            t_host = time.perf_counter()
            ready = torch.cuda.Event(enable_timing=True)
            ready.record(torch.cuda.current_stream())
            s.wait_event(ready)
            start.record(s)
            trace._orig(opt, gi)
            stop.record(s)
            torch.cuda.nvtx.range_pop()
            n_el = opt.merge_schedule.group_sizes[gi]
            trace.records.append({'group': gi, 'bytes': 4 * n_el, 'host_ts': t_host, 'ready': ready, 'start': start, 'stop': stop})
        self.comm.launch_group = traced
        self.enabled = True

    def mark_backward_end(self) -> None:
        """Call right after ``loss.backward()`` returns (before ``step()``)."""
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream())
        self._backward_end = ev

    def stop(self) -> None:
        if self.enabled:
            self.comm.launch_group = self._orig
            self.enabled = False

    def summary(self) -> Dict[str, object]:
        torch.cuda.synchronize()
        groups = []
        for r in self.records:
            groups.append({'group': r['group'], 'bytes': r['bytes'], 'host_ts': r['host_ts'],
                           'wait_ms': r['ready'].elapsed_time(r['start']), 'device_ms': r['start'].elapsed_time(r['stop'])})
        exposed = None
        if self._backward_end is not None and self.records:
            exposed = max(self._backward_end.elapsed_time(self.records[-1]['stop']), 0.0)
        return {'groups': groups, 'comm_ms': sum(g['device_ms'] for g in groups), 'exposed_comm_ms': exposed}

    def dump(self, path: str) -> None:
        with open(path, 'w') as f:
            json.dump(self.summary(), f, indent=1)
