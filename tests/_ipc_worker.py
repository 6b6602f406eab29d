"""Parent/child exchange of device tensors over torch.multiprocessing; run as a script so that the
allocator configuration of the environment applies to both processes.  Prints OK on success."""
import os
import sys

import torch
import torch.multiprocessing as mp


def child(q_in, q_out):
    import torch_musa_b200 as bw  # noqa: F401

    t, p = q_in.get()
    ok = bool((t.cpu() == torch.arange(t.numel(), dtype=torch.float32).view_as(t.cpu())).all())
    ok = ok and isinstance(p, torch.nn.Parameter) and p.requires_grad and float(p.sum().cpu()) == 12.0
    t.add_(1)                      # visible to the parent: same memory
    torch.blackwell.synchronize()
    view = q_in.get()              # a strided view of a second storage
    ok = ok and view.shape == (4, 3) and float(view.cpu()[1, 2]) == 18.0
    q_out.put(ok)
    del t, p, view
    q_in.get()                     # stay alive until the parent has looked


def main():
    import torch_musa_b200 as bw

    expandable = bool(bw._C._allocator_config()["expandable_segments"]) if hasattr(bw._C, "_allocator_config") else None
    ctx = mp.get_context("spawn")
    q_in, q_out = ctx.Queue(), ctx.Queue()
    proc = ctx.Process(target=child, args=(q_in, q_out))
    proc.start()
    t = torch.arange(6 * 1024, dtype=torch.float32).view(6, 1024).to("blackwell")
    p = torch.nn.Parameter(torch.full((3, 4), 1.0, device="blackwell"))
    q_in.put((t, p))
    base = torch.arange(24, dtype=torch.float32).to("blackwell").view(3, 8)
    q_in.put(base[:, 1:5].t())     # element [1, 2] is base[2, 2] = 18
    ok = q_out.get(timeout=120)
    torch.blackwell.synchronize()
    same_memory = bool((t.cpu() == torch.arange(6 * 1024, dtype=torch.float32).view(6, 1024) + 1).all())
    held_before = bw.ipc_collect()
    q_in.put(None)
    proc.join(60)
    held_after = bw.ipc_collect()
    snap = bw.memory_snapshot()
    kinds = {bool(s["is_expandable"]) for s in snap}
    print("child_ok", ok, "same_memory", same_memory, "held", held_before, held_after, "expandable_segments", kinds,
          "exit", proc.exitcode)
    if ok and same_memory and held_after == 0 and proc.exitcode == 0:
        print("OK")


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    main()
