# -*- coding: utf-8 -*-
"""Read-only sampling of a GPU's SM clock, power draw and throttle reasons while a measurement runs.

A timing without its clock record says little on a part whose SM clock moves between 1.3 and 1.97 GHz with the
power draw, so the benchmark tools of this package (``ops/microbench.py``, ``parallel/comm/bench.py``) sample
``nvidia-smi`` in the background for the length of the timed interval and print the median SM clock of the samples
taken under load next to their figures.  Nothing is ever set: clocks, power limits and every other device setting
are left exactly as found.
"""
from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile
from typing import Dict, Optional

_QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
          'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
          'clocks_event_reasons.sw_power_cap')
_REASONS = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')


def parse_samples(lines) -> Dict[str, object]:
    """Summary of ``nvidia-smi --format=csv,noheader,nounits`` lines of the query above (also used by the tests)."""
    sm, smax, power, reasons = [], [], [], set()
    for line in lines:
        parts = [p.strip() for p in line.split(',')]
        if len(parts) < 9:
            continue
        try:
            sm.append(float(parts[1]))
            smax.append(float(parts[2]))
            power.append(float(parts[3]))
        except ValueError:
            continue
        for name, val in zip(_REASONS, parts[5:9]):
            if val.lower().startswith('active'):
                reasons.add(name)
    busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] if power else sm
    return {'sm_mhz': statistics.median(busy) if busy else None, 'sm_max_mhz': max(smax) if smax else None,
            'reasons': sorted(reasons), 'samples': len(sm), 'power_w_max': max(power) if power else None}


class ClockSampler:
    """``with ClockSampler(gpu_index) as s: ...; s.summary`` -- or ``start()`` / ``stop()``."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = int(gpu_index), int(period_ms)
        self._proc: Optional[subprocess.Popen] = None
        self._path: Optional[str] = None
        self.summary: Dict[str, object] = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}

    def start(self) -> 'ClockSampler':
        exe = shutil.which('nvidia-smi')
        if exe is None:
            return self
        fd, self._path = tempfile.mkstemp(suffix='.csv')
        self._out = os.fdopen(fd, 'w')
        self._proc = subprocess.Popen([exe, '-i', str(self.gpu_index), '--query-gpu=' + _QUERY, '--format=csv,noheader,nounits',
                                       '-lms', str(self.period_ms)], stdout=self._out, stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> Dict[str, object]:
        if self._proc is None:
            return self.summary
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except Exception:
            self._proc.kill()
        self._out.close()
        with open(self._path) as f:
            self.summary = parse_samples(f)
        os.unlink(self._path)
        self._proc = None
        return self.summary

    __enter__ = start

    def __exit__(self, *exc) -> bool:
        self.stop()
        return False
