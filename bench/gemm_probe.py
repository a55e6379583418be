"""One matmul of a given shape, this library's tcgen05 kernel or cuBLAS, inside an NVTX range named "target" - the
command to put under ``ncu --nvtx --nvtx-include "target/"`` when the two kernels' counters are compared.

    python bench/gemm_probe.py ours 4096 57344 8192        # M N K; weight [N, K]
    python bench/gemm_probe.py cublas 4096 57344 8192
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

from hccl_b200.ops import mc2  # noqa: E402


def main():
    impl = sys.argv[1]
    m, n, k = (int(v) for v in sys.argv[2:5]) if len(sys.argv) >= 5 else (4096, 57344, 8192)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    f = (lambda: mc2.matmul(x, w, out=out)) if impl == "ours" else (lambda: torch.matmul(x, w.t(), out=out))
    for _ in range(3):
        f()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("target")
    f()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    print("done", impl, m, n, k)


if __name__ == "__main__":
    main()
