"""Profiler helpers for the blackwell device.

``torch.profiler`` already records this backend's kernels (they are CUDA kernels to CUPTI) and its operators;
this module adds what the reference layers on top of a trace:

* ``BasicEvaluation(prof)`` -- per-operator self time, device-queue depth when each operator launched and the
  idle gaps of the device, used to rank operators by how much faster the step would get if their host
  overhead vanished;
* anti-pattern matchers over the operator list: fp32 matmuls that could run on the bf16 tensor cores, matmul
  dimensions that are not multiples of 8 (the tensor-map alignment the GEMM needs, otherwise it falls back),
  host tensors copied to the device right after creation, and small kernels dominated by launch overhead.

    with torch.profiler.profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
        step()
    print(report(prof))

Parity: reference torch_musa/profiler/__init__.py:15-31, _utils.py:20-251, _pattern_matcher.py:21-241.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class OpStat:
    name: str
    calls: int = 0
    self_cpu_us: float = 0.0
    device_us: float = 0.0
    queue_depth_sum: int = 0

    @property
    def mean_queue_depth(self) -> float:
        return self.queue_depth_sum / self.calls if self.calls else 0.0


class BasicEvaluation:
    """Self time, device time and launch-queue depth per operator; idle time of the device."""

    def __init__(self, prof):
        self.events = list(prof.events()) if hasattr(prof, "events") else list(prof)
        self.ops: Dict[str, OpStat] = {}
        self.kernels = []           # (start_us, end_us, name)
        self._collect()

    @staticmethod
    def _is_device(evt) -> bool:
        dt = getattr(evt, "device_type", None)
        return dt is not None and "CPU" not in str(dt)

    def _collect(self) -> None:
        for e in self.events:
            tr = getattr(e, "time_range", None)
            if tr is None:
                continue
            if self._is_device(e):
                self.kernels.append((tr.start, tr.end, e.name))
            else:
                st = self.ops.setdefault(e.name, OpStat(e.name))
                st.calls += 1
                st.self_cpu_us += float(getattr(e, "self_cpu_time_total", 0.0))
                st.device_us += float(getattr(e, "device_time_total", 0.0) or 0.0)
        self.kernels.sort()
        # queue depth: kernels launched but not finished when an operator starts on the host
        ends = sorted(k[1] for k in self.kernels)
        starts = [k[0] for k in self.kernels]
        import bisect

        for e in self.events:
            tr = getattr(e, "time_range", None)
            if tr is None or self._is_device(e):
                continue
            launched = bisect.bisect_right(starts, tr.start)
            finished = bisect.bisect_right(ends, tr.start)
            self.ops[e.name].queue_depth_sum += max(0, launched - finished)

    def device_busy_us(self) -> float:
        busy, cur_s, cur_e = 0.0, None, None
        for s, e, _ in self.kernels:
            if cur_e is None or s > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                cur_s, cur_e = s, e
            else:
                cur_e = max(cur_e, e)
        if cur_e is not None:
            busy += cur_e - cur_s
        return busy

    def device_span_us(self) -> float:
        return (max(k[1] for k in self.kernels) - min(k[0] for k in self.kernels)) if self.kernels else 0.0

    def idle_us(self) -> float:
        return max(0.0, self.device_span_us() - self.device_busy_us())

    def rank_by_host_overhead(self, top: int = 10) -> List[OpStat]:
        """Operators that start with an empty device queue cost their full host time: rank by self time / (1 + depth)."""
        return sorted(self.ops.values(), key=lambda s: -s.self_cpu_us / (1.0 + s.mean_queue_depth))[:top]


@dataclass
class Finding:
    pattern: str
    op: str
    detail: str
    count: int = 1


class Pattern:
    name = "pattern"

    def match(self, evt) -> Optional[str]:
        raise NotImplementedError

    def scan(self, events) -> List[Finding]:
        found: Dict[str, Finding] = {}
        for e in events:
            if BasicEvaluation._is_device(e):
                continue
            d = self.match(e)
            if d:
                key = e.name + "|" + d
                if key in found:
                    found[key].count += 1
                else:
                    found[key] = Finding(self.name, e.name, d)
        return list(found.values())


_MATMULS = ("aten::mm", "aten::addmm", "aten::bmm", "aten::baddbmm", "aten::linear", "aten::matmul")


def _shapes(evt):
    return [s for s in (getattr(evt, "input_shapes", None) or []) if s]


class FP32MatMulPattern(Pattern):
    """fp32 matrix products: the tensor cores take bf16/fp16 (use autocast or allow a lower-precision matmul)."""
    name = "fp32 matmul"

    def match(self, evt):
        if evt.name not in _MATMULS:
            return None
        dts = getattr(evt, "input_dtypes", None) or getattr(evt, "input_type", None) or []
        if any(str(d) in ("float", "torch.float32", "float32") for d in dts):
            return "float32 operands: runs on the library path, not on the bf16 tcgen05 GEMM"
        return None


class MatMulDimPattern(Pattern):
    """Matrix dimensions that are not multiples of 8: the TMA tensor map needs 16-byte rows."""
    name = "matmul dimension alignment"

    def match(self, evt):
        if evt.name not in _MATMULS:
            return None
        for shp in _shapes(evt):
            if len(shp) >= 2 and any(int(d) % 8 for d in shp[-2:]):
                return f"operand shape {list(shp)} has a dimension that is not a multiple of 8"
        return None


class ExtraDeviceCopyPattern(Pattern):
    """Tensors created on the host and copied to the device right away: create them on the device."""
    name = "extra host-to-device copy"
    _creators = ("aten::zeros", "aten::ones", "aten::full", "aten::arange", "aten::rand", "aten::randn", "aten::eye")

    def scan(self, events):
        out: Dict[str, Finding] = {}
        prev = None
        for e in events:
            if BasicEvaluation._is_device(e):
                continue
            if prev is not None and prev.name in self._creators and e.name in ("aten::to", "aten::_to_copy", "aten::copy_"):
                key = prev.name
                if key in out:
                    out[key].count += 1
                else:
                    out[key] = Finding(self.name, prev.name, f"{prev.name} followed by {e.name}: pass device= to the factory")
            if e.name.startswith("aten::") and e.name not in ("aten::empty", "aten::empty_strided", "aten::fill_", "aten::zero_"):
                prev = e
        return list(out.values())


class SmallKernelPattern(Pattern):
    """Operators whose device time is below their host time: launch-bound; capture the loop in a device graph."""
    name = "launch-bound operator"

    def match(self, evt):
        dev = float(getattr(evt, "device_time_total", 0.0) or 0.0)
        cpu = float(getattr(evt, "self_cpu_time_total", 0.0))
        if evt.name.startswith("aten::") and 0.0 < dev < 5.0 and cpu > 2 * dev:
            return "device time under 5 us and below half of the host time"
        return None


ALL_PATTERNS = (FP32MatMulPattern, MatMulDimPattern, ExtraDeviceCopyPattern, SmallKernelPattern)


def find_antipatterns(prof, patterns=ALL_PATTERNS) -> List[Finding]:
    events = list(prof.events()) if hasattr(prof, "events") else list(prof)
    out: List[Finding] = []
    for p in patterns:
        out += p().scan(events)
    return out


def report(prof, top: int = 10) -> str:
    ev = BasicEvaluation(prof)
    lines = [f"device busy {ev.device_busy_us() / 1e3:.2f} ms of {ev.device_span_us() / 1e3:.2f} ms "
             f"(idle {ev.idle_us() / 1e3:.2f} ms), {len(ev.kernels)} kernels",
             "operators ranked by exposed host overhead:"]
    for s in ev.rank_by_host_overhead(top):
        lines.append(f"  {s.name:40s} calls {s.calls:5d}  self cpu {s.self_cpu_us / 1e3:8.3f} ms  "
                     f"queue depth {s.mean_queue_depth:5.1f}")
    finds = find_antipatterns(prof)
    lines.append(f"{len(finds)} anti-pattern finding(s):")
    for f in finds:
        lines.append(f"  [{f.pattern}] {f.op} x{f.count}: {f.detail}")
    return "\n".join(lines)
