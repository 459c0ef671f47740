"""Child of the bounds-check test: runs with B200_BOUNDS_CHECK=1, i.e. on the debug library in which kernels report
device-side lengths and indices that fall outside their range (every build clamps them)."""
import json
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

import torch  # noqa: E402

from create_llm_by_cupy_b200.ops import build, native  # noqa: E402
from create_llm_by_cupy_b200.ops import functional as F  # noqa: E402


def main():
    out = {"lib": os.path.basename(str(build.lib_path())), "bounds_check": build.BOUNDS_CHECK}
    g = torch.Generator().manual_seed(0)
    B, T, QH, KVH, D = 2, 256, 4, 2, 128
    q = torch.randn(B, T, QH, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, T, KVH, D, generator=g).to(torch.bfloat16).cuda()
    ok_len = torch.tensor([T, 100], dtype=torch.int32, device="cuda")
    o1, _ = F.flash_attn_fwd(q, k, v, valid_len=ok_len)
    torch.cuda.synchronize()
    out["in_range"] = list(native.read_status())
    bad_len = torch.tensor([T + 5, 100], dtype=torch.int32, device="cuda")
    o2, _ = F.flash_attn_fwd(q, k, v, valid_len=bad_len)
    torch.cuda.synchronize()
    st = native.status_tensor().tolist()
    out["too_long"] = st[:3]
    native.read_status()
    out["clamped_equal"] = bool(torch.equal(o1, o2))
    # a target id beyond the vocabulary in the fused loss
    M, V, K = 256, 512, 64
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(V, K, generator=g).to(torch.bfloat16).cuda()
    t = torch.randint(0, V, (M,), generator=g, dtype=torch.int32).cuda()
    tl = torch.zeros(M, device="cuda")
    F.gemm_ce_stats(x, w, t, tl, vocab=V)
    torch.cuda.synchronize()
    out["targets_in_range"] = list(native.read_status())
    t[7] = V + 3
    F.gemm_ce_stats(x, w, t, tl, vocab=V)
    torch.cuda.synchronize()
    out["target_beyond_vocab"] = native.status_tensor().tolist()[:3]
    native.read_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
