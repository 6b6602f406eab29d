"""Text renderings of an allocator snapshot (``torch.blackwell.memory._snapshot()`` or a pickled ``_dump_snapshot``):
the segment map, the event trace, and folded stacks for flame graphs of the live allocations.

    snap = torch.blackwell.memory._snapshot()                 # after _record_memory_history(stacks="cpp")
    print(memory_viz.segments_text(snap))
    memory_viz.write_flamegraph(snap, "live.folded")          # flamegraph.pl live.folded > live.svg, or speedscope

    python -m torch_musa_b200.core.memory_viz snapshot.pickle [--trace | --flamegraph out.folded]

The snapshot keeps torch.cuda's layout (``segments`` with ``blocks``, ``device_traces`` per device), so tools written
for that layout read it too; an event's ``frames`` is the symbolised C++ backtrace of the allocation site, one frame
per line.

Parity: reference torch_musa/core/memory.py:377-497 (summary, segments / trace text, flame graph input).
"""
from __future__ import annotations

import pickle
import sys
from collections import defaultdict
from typing import Any, Dict, Iterable, List, Tuple


def _size(n: int) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024 or unit == "TiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{n} B"
        n /= 1024.0
    return str(n)


def segments_text(snapshot: Dict[str, Any]) -> str:
    """One line per segment, one indented line per block; totals at the end."""
    out, reserved, allocated = [], 0, 0
    for seg in sorted(snapshot.get("segments", []), key=lambda s: (s.get("device", 0), s["address"])):
        kind = seg.get("segment_type", "?") + (", expandable" if seg.get("is_expandable") else "")
        pool = tuple(seg.get("segment_pool_id", (0, 0)))
        out.append(f"segment 0x{seg['address']:x} dev {seg.get('device', 0)} {_size(seg['total_size'])} ({kind}"
                   + (f", pool {pool}" if pool != (0, 0) else "") + f") allocated {_size(seg.get('allocated_size', 0))}")
        reserved += seg["total_size"]
        allocated += seg.get("allocated_size", 0)
        for b in seg.get("blocks", []):
            out.append(f"    0x{b.get('address', 0):x} {_size(b['size']):>12} {b.get('state', '?')}"
                       + (f" (requested {_size(b['requested_size'])})" if b.get("requested_size") else ""))
    out.append(f"total: reserved {_size(reserved)}, allocated {_size(allocated)}, "
               f"cached {_size(reserved - allocated)} in {len(snapshot.get('segments', []))} segments")
    return "\n".join(out)


def trace_text(snapshot: Dict[str, Any], device: int = 0, last: int = 0) -> str:
    """The recorded allocator events of one device in order (``last`` > 0: only the newest ones)."""
    traces = snapshot.get("device_traces", [])
    events = list(traces[device]) if device < len(traces) else []
    if last > 0:
        events = events[-last:]
    t0 = events[0].get("time_us", 0) if events else 0
    lines = [f"{e.get('time_us', 0) - t0:>10} us  {e['action']:<16} 0x{e.get('addr', 0):x} {_size(e.get('size', 0)):>12}"
             f"  stream 0x{e.get('stream', 0):x}" for e in events]
    return "\n".join(lines) if lines else "(no events recorded: call _record_memory_history() first)"


def _stack_of(event: Dict[str, Any]) -> Tuple[str, ...]:
    frames = event.get("frames")
    if not frames:
        return ("<no stack recorded>",)
    if isinstance(frames, str):
        lines = [ln.strip() for ln in frames.splitlines() if ln.strip()]
    else:   # torch.cuda layout: a list of {"filename", "line", "name"}
        lines = [f"{f.get('name', '?')} ({f.get('filename', '?')}:{f.get('line', 0)})" for f in frames]
    # the backtrace lists the innermost frame first; flame graphs want the outermost first
    cleaned = [ln.replace(";", ":") for ln in lines]
    return tuple(reversed(cleaned))


def live_allocations(snapshot: Dict[str, Any], device: int = 0) -> List[Dict[str, Any]]:
    """Allocation events of the trace that no later free event matches."""
    traces = snapshot.get("device_traces", [])
    live: Dict[int, Dict[str, Any]] = {}
    for e in (traces[device] if device < len(traces) else []):
        if e["action"] == "alloc":
            live[e["addr"]] = e
        elif e["action"] in ("free_requested", "free_completed", "free"):
            live.pop(e.get("addr"), None)
    return list(live.values())


def flamegraph_lines(snapshot: Dict[str, Any], device: int = 0, live_only: bool = True) -> List[str]:
    """Folded stacks (``frame;frame;frame bytes``) of the allocation sites, weighted by bytes."""
    traces = snapshot.get("device_traces", [])
    events: Iterable[Dict[str, Any]] = live_allocations(snapshot, device) if live_only else \
        [e for e in (traces[device] if device < len(traces) else []) if e["action"] == "alloc"]
    weight: Dict[Tuple[str, ...], int] = defaultdict(int)
    for e in events:
        weight[_stack_of(e)] += int(e.get("size", 0))
    return [";".join(stack) + f" {n}" for stack, n in sorted(weight.items(), key=lambda kv: -kv[1])]


def write_flamegraph(snapshot: Dict[str, Any], path: str, device: int = 0, live_only: bool = True) -> int:
    lines = flamegraph_lines(snapshot, device, live_only)
    with open(path, "w") as f:
        f.write("\n".join(lines) + ("\n" if lines else ""))
    return len(lines)


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Render a pickled allocator snapshot as text")
    ap.add_argument("snapshot")
    ap.add_argument("--trace", action="store_true", help="print the event trace instead of the segment map")
    ap.add_argument("--flamegraph", metavar="OUT", help="write folded stacks of the live allocations")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)
    with open(a.snapshot, "rb") as f:
        snap = pickle.load(f)
    if a.flamegraph:
        print(f"{write_flamegraph(snap, a.flamegraph, a.device)} stacks written to {a.flamegraph}")
    elif a.trace:
        print(trace_text(snap, a.device))
    else:
        print(segments_text(snap))
    return 0


if __name__ == "__main__":
    sys.exit(main())
