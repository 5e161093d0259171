"""Wait accounting of the tensor-core kernels: where each warp of one CTA spends its cycles.

    python -m simplicial_attention_b200.waitprof --build-only [--cta 20]          (no GPU needed)
    python -m simplicial_attention_b200.waitprof --kernel fwd|dk1_dv1|dq_dk2_dv2 --d 64|128 [--n 8192 --heads 2 --w1 512 --w2 32]

The kernels are compiled a second time with ``-DSA2_PROF=<CTA index>`` into ``libsa2_prof.so`` beside the
normal library (csrc/sa2_sm100.cuh: every bounded wait of that CTA, with blockIdx.y = blockIdx.z = 0, adds the
cycles it spent to a slot of its warp; a few code segments are booked the same way).  This module loads that
build through ``SA2_LIBRARY``, runs one kernel on random inputs and prints the table: one row per warp, column 0
the cycles from the start to the end of the warp's role, the other columns the slots named below.  A diagnostic
for kernel work - the accounting costs a few per cent, so no timing from this build is a benchmark.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
PROF_LIB = os.path.join(PKG, "libsa2_prof.so")

# what the slots 1..7 of a warp mean, per kernel and warp role (head dim 64 / 128 where they differ)
SLOTS = {
    "fwd": "d=64: issuers (warps 0-1) 1 A_e ready, 2 P ready, 3 W read by the output group; output group (4-7) 1 A_e stage "
           "free, 2 reference ready, 3 W complete; softmax groups (8-15) 1 S ready.  d=128: issuers of S (0-1) 1 A_e ready, "
           "2 K1 unit landed, 3 P V1 product of the buffer done; issuers of P V1 (2-3) 4 V1 unit landed, 5 P ready, 6 W read; "
           "output group (4-11) 1 A_e stage free, 2 reference ready, 3 W complete; softmax groups (12-19) 1 S ready, 2 W read; "
           "producers (20-21) 1 ring slot free",
    "dk1_dv1": "issuer of dV1 / dK1 (0) 1 P^T/G^T ready; issuers of S^T / dP^T (1 and 14; d=128: 1 and 2) 1 A_e/B_e stage full, "
               "2 the P^T/G^T pass of the half (d=128: its second products) done; compute groups 1 S^T/dP^T ready, 2 (d=64) second "
               "products of the half done; builders (last four or eight warps) 1 k2/v2 window landed, 2 stage free",
    "dq_dk2_dv2": "issuers of U / W (0, and 3 at d=64) 1 P/G ready, 2 U/W read by the fold group; issuers of S / dP (1, 2) "
                  "1 A_e/B_e ready, 2 buffer free, 3 K1/V1 unit landed (d=128), 4 cycles issuing products, 5 cycles in the commit; "
                  "producer (3 at d=128) 1 ring slot free; compute groups (4-11) 1 S/dP ready, 4 TMEM loads, 5 arithmetic, "
                  "6 TMEM stores and hand-over; operand / fold group (12-15) 1 U/W complete, 2 the other fold threads, "
                  "3 A_e/B_e stage free, 4 stores of A_e/B_e (d=64), 5 fold after its waits",
}


def build_prof(cta: int = 20, verbose: bool = False) -> str:
    from . import build
    return build.build(force=True, verbose=verbose, out=PROF_LIB, defines=(f"SA2_PROF={cta}",))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--build-only", action="store_true")
    ap.add_argument("--cta", type=int, default=20, help="blockIdx.x of the CTA that is accounted")
    ap.add_argument("--kernel", default="dq_dk2_dv2", choices=sorted(SLOTS))
    ap.add_argument("--d", type=int, default=64, choices=(64, 128))
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--w1", type=int, default=512)
    ap.add_argument("--w2", type=int, default=32)
    args = ap.parse_args()
    if args.build_only:
        print(build_prof(args.cta))
        return
    if not os.path.exists(PROF_LIB):
        build_prof(args.cta)
    os.environ["SA2_LIBRARY"] = PROF_LIB
    import torch
    import simplicial_attention_b200 as sa
    from simplicial_attention_b200 import _lib

    if not torch.cuda.is_available():
        sys.exit("waitprof runs the kernels: it needs a GPU (use --build-only to compile here)")
    lib = _lib.lib()
    lib.sa2_prof_read.argtypes = [C.POINTER(C.c_ulonglong), C.c_int]
    lib.sa2_prof_read.restype = C.c_int
    table = (C.c_ulonglong * 512)()
    g = torch.Generator(device="cuda").manual_seed(1)
    shape = (1, args.n, args.heads, args.d)
    q, k1, k2, v1, v2, do = (torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16) for _ in range(6))
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, args.w1, args.w2, kernel="tcgen05")
    call = sa.BackwardCall(q, k1, k2, v1, v2, out, lse, do, args.w1, args.w2, kernel="tcgen05")
    call.launch(_lib.BWD_ROWSUM)
    torch.cuda.synchronize()
    lib.sa2_prof_read(table, 512)          # clear what the set-up launches booked
    if args.kernel == "fwd":
        sa.sa2_forward(q, k1, k2, v1, v2, args.w1, args.w2, kernel="tcgen05")
    else:
        call.launch(_lib.BWD_K1 if args.kernel == "dk1_dv1" else _lib.BWD_Q)
    torch.cuda.synchronize()
    sa.check_device()
    lib.sa2_prof_read(table, 512)
    print(f"{args.kernel} d={args.d} n={args.n} heads={args.heads} w1={args.w1} w2={args.w2}; cycles of one CTA")
    print("slots:", SLOTS[args.kernel])
    print("warp    total " + " ".join(f"{'slot ' + str(k):>9}" for k in range(1, 8)))
    for w in range(24):
        row = [table[w * 8 + k] for k in range(8)]
        if any(row):
            print(f"{w:4d} " + " ".join(f"{v:9d}" for v in row))


if __name__ == "__main__":
    main()
