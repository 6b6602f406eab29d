"""Operator coverage of the backend, read from the dispatcher.

    python -m torch_musa_b200.utils.op_coverage                 # summary
    python -m torch_musa_b200.utils.op_coverage --markdown      # one table row per operator
    python -m torch_musa_b200.utils.op_coverage --missing 40    # CUDA operators without a native kernel here

Every operator with an explicit registration under the device's dispatch key runs code of this repository (a
hand-written kernel or a composition of them); everything else reaches the boxed fallback, which runs PyTorch's CUDA
kernel over the same memory and is counted at run time by ``torch.blackwell.fallback_counts()``.  The listing needs no
GPU.  ``observed(fn)`` runs a callable and reports which operators actually fell back.

Parity: reference tools/ops_scanner (coverage spreadsheets from a source scan) and tools/ops_filter; here the
dispatcher is the source of truth, so the report cannot drift from the build.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from typing import Callable, Dict, List

import torch


def _registrations(key: str) -> List[str]:
    return sorted(torch._C._dispatch_get_registrations_for_dispatch_key(key))


def _base(name: str) -> str:
    return name.split("::", 1)[1].split(".", 1)[0]


def report() -> Dict[str, object]:
    import torch_musa_b200  # noqa: F401  (registers the kernels)

    native = _registrations("PrivateUse1")
    autocast = _registrations("AutocastPrivateUse1")
    autograd = _registrations("AutogradPrivateUse1")
    cuda = [n for n in _registrations("CUDA") if n.startswith("aten::")]
    native_aten = [n for n in native if n.startswith("aten::")]
    custom = [n for n in native if not n.startswith("aten::")]
    native_bases = {_base(n) for n in native_aten}
    cuda_bases = {_base(n) for n in cuda}
    by_base = defaultdict(list)
    for n in native_aten:
        by_base[_base(n)].append(n.split("::", 1)[1])
    return {
        "native_overloads": len(native_aten),
        "native_base_operators": len(native_bases),
        "custom_operators": custom,
        "autocast_rules": len(autocast),
        "autograd_overrides": len(autograd),
        "cuda_base_operators": len(cuda_bases),
        "covered_of_cuda": len(native_bases & cuda_bases),
        "fallback_base_operators": sorted(cuda_bases - native_bases),
        "native_by_base": dict(sorted(by_base.items())),
    }


def observed(fn: Callable[[], object]) -> Dict[str, int]:
    """Runs ``fn`` and returns the operators that reached the fallback while it ran, with their call counts."""
    import torch_musa_b200 as bw

    bw.reset_fallback_counts()
    fn()
    return dict(sorted(bw.fallback_counts().items(), key=lambda kv: -kv[1]))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n", 1)[0])
    ap.add_argument("--markdown", action="store_true", help="table of natively served operators and their overloads")
    ap.add_argument("--missing", type=int, default=0, metavar="N", help="list up to N CUDA operators served by the fallback")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    r = report()
    if a.json:
        print(json.dumps(r, indent=1))
        return 0
    print(f"native aten operators: {r['native_base_operators']} ({r['native_overloads']} overloads); "
          f"custom operators: {len(r['custom_operators'])}; autocast rules: {r['autocast_rules']}")
    print(f"of the {r['cuda_base_operators']} aten operators with a CUDA kernel, {r['covered_of_cuda']} have a native "
          f"kernel here; the others run through the fallback on the library kernel")
    if a.markdown:
        print("\n| operator | overloads |\n|---|---|")
        for base, overloads in r["native_by_base"].items():
            print(f"| `{base}` | {', '.join(sorted(overloads))} |")
        for name in r["custom_operators"]:
            print(f"| `{name}` | (custom) |")
    if a.missing:
        print("\nserved by the fallback:", ", ".join(r["fallback_base_operators"][: a.missing]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
