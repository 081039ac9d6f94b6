"""Cost of one `tcgen05.mma` when a single thread issues a run of them (csrc/bench/mma_probe.cu):
`python -m zero_to_hero_b200.utils.mma_probe` prints, per operand form and output width, the SM cycles
per MMA until the run is issued and until it has completed, idle and with the CTA's other warps busy in
several ways. The figures size the MMA budget of the attention kernels."""
from __future__ import annotations

import argparse
import ctypes
import json

from ..ops import _lib

VARIANTS = ["SS N64", "SS N128", "SS N256", "SS N64, B MN-major", "SS N64, A and B MN-major",
            "TS N64 (A in tensor memory)", "SS N64, two accumulators", "SS N32", "SS N16"]
BUSY = ["idle", "dependent FMA chains", "shared-memory stores", "tensor-memory loads",
        "issue-saturating FMA", "exponentials"]


def probe(variant: int, nmma: int, busy: int) -> dict:
    fn = _lib.cuda_lib().z2h_mma_probe
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    out = (ctypes.c_longlong * 3)()
    rc = fn(variant, nmma, busy, out)
    if rc != 0:
        raise RuntimeError(f"z2h_mma_probe failed with code {rc}")
    if out[2] != 0:
        raise RuntimeError("the probe's bounded wait gave up")
    return {"form": VARIANTS[variant], "other_warps": BUSY[busy], "mmas": nmma,
            "issue_cycles_per_mma": round(out[0] / nmma, 1), "done_cycles_per_mma": round(out[1] / nmma, 1)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--mmas", type=int, default=128)
    ap.add_argument("--busy", type=int, nargs="*", default=[0, 2, 3, 5, 4])
    a = ap.parse_args()
    for b in a.busy:
        for v in range(len(VARIANTS)):
            print(json.dumps(probe(v, a.mmas, b)), flush=True)


if __name__ == "__main__":
    main()
