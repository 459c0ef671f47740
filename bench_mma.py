"""Cost of one ``tcgen05.mma`` (M = 128, K = 16, bf16, one CTA per SM) when instructions are issued back to
back: by N, by the source of A (shared or tensor memory) and with other warps loading / storing tensor memory
beside them. The numbers behind the tile shapes of the attention kernels (why every product of the dK/dV kernel
is N = 128). Prints one JSON line per case: clocks per instruction against the arithmetic's N / 2.

    python bench_mma.py
"""
from __future__ import annotations

import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from create_llm_by_cupy_b200.ops import native  # noqa: E402


def main():
    lib = native.lib()
    reps, depth = 50, 32
    out = (ctypes.c_longlong * 3)()
    for traffic in (0, 1, 2):
        for n, tmem in ((64, 0), (128, 0), (256, 0), (64, 1), (128, 1)):
            native.check(lib.b200_bench_mma(n, tmem, traffic, reps, depth, out), "b200_bench_mma")
            print(json.dumps({"N": n, "A": "tensor memory" if tmem else "shared memory",
                              "tmem_traffic": ["none", "loads", "loads+stores"][traffic],
                              "clocks_per_mma": round(out[0] / (reps * depth), 1), "arithmetic_clocks": n // 2,
                              "clocks_per_load_round": int(out[1])}))
    print(json.dumps({"status": native.read_status()}))


if __name__ == "__main__":
    main()
