"""Runs the launch that norms, turns and caches the query and key heads of a stacked projection (and, with --add-norm, the norm
after a sum) of given sizes three times, for ncu to capture one launch of a case that ends by itself:

    python -m research_2_b200.profiling.norm_rotate_case --heads 12 --kv-heads 3 --dim 64 --rows 32768 &&
    ncu --set full --clock-control none -k regex:norm_rotate -s 1 -c 1 -o norm_rotate \
        python -m research_2_b200.profiling.norm_rotate_case --heads 12 --kv-heads 3 --dim 64 --rows 32768

With --time the case is timed inside a CUDA graph of 20 launches and microseconds per launch are printed.
"""
import argparse

import torch

from ..kernels import ops
from .kernel_cases import time_in_graph


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=3)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--width", type=int, default=768, help="with --add-norm: the stream's width")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--add-norm", action="store_true")
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    dev, h, g, hd, t, page = "cuda:0", args.heads, args.kv_heads, args.dim, args.rows, args.page_size
    if args.add_norm:
        x, y, gain = torch.randn(t, args.width, device=dev), torch.randn(t, args.width, device=dev), torch.ones(args.width, device=dev)

        def fn():
            ops.add_norm(x, y, 2.0, gain, 1e-5, torch.bfloat16)
    else:
        qkv = torch.randn(t, (h + 2 * g) * hd, device=dev).bfloat16()
        n_pages = -(-t // page) + 1
        pool = torch.zeros(n_pages * 2 * g * page * hd, device=dev, dtype=torch.bfloat16)
        slots = torch.arange(page, page + t, dtype=torch.int32, device=dev)
        positions = (torch.arange(t, dtype=torch.int32, device=dev) % 1024).contiguous()
        freq = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], device=dev)
        gains = torch.ones(hd, device=dev)
        scatter = ops.kv_scatter(slots, pool, pool[g * page * hd:], 2 * g * page * hd, page, n_pages, (h + g) * hd, g * hd, hd)

        def fn():
            ops.rotate_half(qkv, h + g, hd, hd, freq, positions, kv=scatter, n_kv_heads=g, k_col=h * hd, q_norm=gains, k_norm=gains,
                            n_q_heads=h, norm_eps=1e-5, magnitude=1.1)
    if args.time:
        print(f"{time_in_graph(fn):.1f} us a launch")
        return 0
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
